"""bench.py host-side contract (no GPU): work formulas, the reference arm's JSON line, rank handling."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench_module():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_work_formulas():
    b = _bench_module()
    assert len(b.SWEEP) == 18 and b.SWEEP[0] == (1024, 1536, 7168) and b.SWEEP[-1] == (6144, 4096, 512)
    assert len(b.NCU_DRAM_BYTES) == len(b.SWEEP)
    # flops 2*M*N*K; bytes = fp8 operands + fp32 scales read once + bf16 C written once
    assert b.gemm_flops(1024, 1536, 7168) == 2.0 * 1024 * 1536 * 7168
    assert b.gemm_bytes(1024, 1536, 7168) == 1024 * 7168 + 1536 * 7168 + 4 * 1024 * 56 + 4 * 12 * 56 + 2 * 1024 * 1536
    assert b.gemm_bytes(1024, 576, 7168) == 1024 * 7168 + 576 * 7168 + 4 * 1024 * 56 + 4 * 5 * 56 + 2 * 1024 * 576
    # no shape moves more DRAM bytes than its operands and result once (no re-read waste)
    for shape, traffic in zip(b.SWEEP, b.NCU_DRAM_BYTES):
        assert traffic <= b.gemm_bytes(*shape)
    p = b.measured_peaks()
    assert p["hbm_gbs"] > 1000 and p["bf16_tflops"] >= p["bf16_tflops_sustained"] > 100


def test_reference_arm_prints_one_json_line_and_only_on_rank_0():
    env = dict(os.environ, OMP_NUM_THREADS="4")
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
           "--shapes", "1024x512x7168,1024x4096x512"]
    quiet = subprocess.run(cmd, env=dict(env, RANK="1", WORLD_SIZE="2"), capture_output=True, text=True, timeout=300)
    assert quiet.returncode == 0 and quiet.stdout.strip() == ""
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "fp8_blockscaled_gemm_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["steps"] == 1
    # the reference's own ref_kernel where oracle/_ref exists (made by oracle/make_ref.py), else the numpy restatement
    have_ref = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "scripts", "problems", "gemm", "reference.py"))
    assert d["cpu_baseline"]["kind"] == ("reference" if have_ref else "port")
    assert d["cpu_baseline"]["value"] == d["value"]
    # the arm sets its own thread count: torchrun's OMP_NUM_THREADS=1 (4 in this test) must not shrink it
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    b = _bench_module()
    assert d["config"] == b.sweep_config(1, "1024x512x7168,1024x4096x512")
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0
