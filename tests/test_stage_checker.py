"""The C++ stage checker (tests/checker/rf_moe_stage_check.cu), the counterpart of the reference's
tests/moe/moe_topk_test.cpp plug-in: it must build, list its cases without a GPU, and pass on one."""
import os
import subprocess

import pytest

from tests import checker

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_checker_builds_and_lists_cases():
    exe = checker.build()
    out = subprocess.run([exe, "-l"], capture_output=True, text=True, cwd=ROOT, timeout=60)
    assert out.returncode == 0
    lines = out.stdout.strip().splitlines()
    assert len(lines) == 6 and lines[0].startswith("0: tokens 512")
    full = subprocess.run([exe, "-l", "--full"], capture_output=True, text=True, cwd=ROOT, timeout=60)
    assert "d_hidden 7168 d_expert 2048 experts 32" in full.stdout      # the reference's own parameter sets


def test_checker_reports_a_missing_library():
    exe = checker.build()
    out = subprocess.run([exe, "--lib", "/nonexistent/librf.so"], capture_output=True, text=True, cwd=ROOT, timeout=60)
    assert out.returncode == 100 and "cannot open" in out.stderr


@pytest.mark.gpu
def test_all_stage_tensors_match_the_cpp_restatement(rf_lib):
    exe = checker.build()
    out = subprocess.run([exe], capture_output=True, text=True, cwd=ROOT, timeout=900)
    print(out.stdout[-4000:])
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert out.stdout.count("  ok   ") == 6 * 13 and "FAIL" not in out.stdout
    assert "6 case(s), 0 failing stage tensor(s)" in out.stdout
