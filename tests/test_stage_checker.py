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


@pytest.mark.parametrize("case,t,d,f,e,k,n_shared", [(0, 512, 1024, 512, 4, 4, 1), (4, 333, 512, 256, 64, 6, 1)])
def test_cpp_restatement_agrees_with_the_numpy_oracle(tmp_path, case, t, d, f, e, k, n_shared):
    """The checker's C++ stage restatement and oracle/moe.py are independent statements of the same stages
    (the numpy one is pinned by the reference's own outputs): on the checker's seeded inputs integer stages
    agree exactly, fp16 stages within the reference tolerance."""
    import numpy as np
    from oracle import moe as om
    exe = checker.build()
    out = subprocess.run([exe, "-c", str(case), "--dump", str(tmp_path)], capture_output=True, text=True, cwd=ROOT,
                         timeout=600)
    assert out.returncode == 0, out.stderr

    def load(name, dtype, shape):
        return np.fromfile(tmp_path / f"{name}.bin", dtype=dtype).reshape(shape)

    fs = f * n_shared
    w = {"shared_experts.0.weight": load("shared_gate", np.float16, (d, fs)),
         "shared_experts.1.weight": load("shared_up", np.float16, (d, fs)),
         "shared_experts.2.weight": load("shared_down", np.float16, (fs, d))}
    for j in range(e):
        w[f"experts.{j}.0.weight"] = load(f"gate{j}", np.float16, (d, f))
        w[f"experts.{j}.1.weight"] = load(f"up{j}", np.float16, (d, f))
        w[f"experts.{j}.2.weight"] = load(f"down{j}", np.float16, (f, d))
    x = load("x", np.float16, (t, d))
    logits = load("logits", np.float16, (t, e))
    ref = om.moe_stages(x, w, e, k, logits16=logits)
    for name, shape in (("seq_experts_index", (t, k)), ("source_rows", (t * k,)), ("permuted_experts", (t * k,)),
                        ("permuted_rows", (t * k,)), ("first_token_offset", (e + 1,)), ("rev_permuted_rows", (t * k,))):
        assert np.array_equal(load(name, np.int32, shape), ref[name]), name
    assert np.array_equal(load("seq_experts_softmax", np.float16, (t, k)).view(np.uint16),
                          ref["seq_experts_softmax"].view(np.uint16))          # same deterministic softmax
    assert np.array_equal(load("expanded_seq_softmax", np.float16, (t * k,)).view(np.uint16),
                          ref["expanded_seq_softmax"].view(np.uint16))
    for name, shape in (("expanded_fc1_output", (t * k, f)), ("expanded_fc2_output", (t * k, d)),
                        ("shared_fc2_output", (t, d)), ("final_output", (t, d))):
        ok, nbad, mx = om.check(load(name, np.float16, shape), ref[name])
        assert ok, (name, nbad, mx)
