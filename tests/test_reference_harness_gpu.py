"""The reference's own harness, unmodified, against this library.

oracle/_ref (written by oracle/make_ref.py from a checkout of the reference; ignored by git) holds the
reference's scripts/eval.py, scripts/utils.py and scripts/problems/{gemm,moe}/ exactly as they are upstream,
plus a two-line submission.py per problem that imports this package's `custom_kernel`.  `python eval.py test`
then generates the reference's own inputs on the GPU (its seeds and shapes, scripts/problems/*/task.yml; for the
GEMM that is float8_e4m3fnuz data in the reference's [k][m] layout), calls `custom_kernel` and checks the result
with the reference's `check_implementation` (scripts/eval.py:148-185, scripts/utils.py:31-91).  Skipped where
oracle/_ref is absent.
"""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = os.path.join(ROOT, "oracle", "_ref", "scripts")

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.exists(os.path.join(SCRIPTS, "eval.py")),
                                 reason="oracle/_ref not made (python oracle/make_ref.py <reference checkout>)")]


def run_eval(mode, prob, timeout):
    env = dict(os.environ)
    env.pop("POPCORN_SEED", None)
    res = subprocess.run([sys.executable, "eval.py", mode, "--prob", prob], cwd=SCRIPTS, env=env, capture_output=True,
                         text=True, timeout=timeout)
    return res.returncode, res.stdout, res.stderr


@pytest.mark.parametrize("prob,n_cases", [("gemm", 11), ("moe", 3)])
def test_reference_eval_test_mode_passes(prob, n_cases):
    rc, out, err = run_eval("test", prob, 900)
    tail = (out + err)[-3000:]
    assert f"test-count: {n_cases}" in out, tail
    assert out.count(".status: pass") == n_cases and "check: pass" in out, tail
    assert rc == 0, tail
