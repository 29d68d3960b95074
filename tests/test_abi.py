"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
and rejects bad arguments before touching the GPU."""
import ctypes
import os
import re

from radeonflow_kernels_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        src = open(os.path.join(ROOT, "include", fn)).read()
        src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
        for m in re.finditer(r"^[A-Za-z_][\w \*]*?[\s\*]([A-Za-z_]\w*)\s*\(", src, flags=re.M):
            name = m.group(1)
            if name not in ("defined",):
                names.append(name)
    return names


def test_header_declares_the_reference_entry_points():
    names = declared_functions()
    assert "run" in names and "rf_fp8_gemm" in names


def test_every_declared_symbol_is_exported(rf_lib):
    missing = [n for n in declared_functions() if not hasattr(rf_lib, n)]
    assert not missing, missing


def test_version_string(rf_lib):
    assert b"sm_100a" in rf_lib.rf_version()


def test_perfmetrics_layout_matches_reference():
    # tests/checker/metrics.h:4-13: char[20] + 2 floats = 28 bytes; int count + 20 entries
    assert ctypes.sizeof(_lib.PerfMetricEntry) == 28
    assert ctypes.sizeof(_lib.PerfMetrics) == 4 + 20 * 28


def test_bad_arguments_are_rejected_on_the_host(rf_lib):
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    args = lambda m, n, k: (p16, p16, p16, p16, p16, m, n, k, 0, None, 0, None)
    assert rf_lib.rf_fp8_gemm(*args(128, 100, 128)) == 1      # n % 64 != 0
    assert rf_lib.rf_fp8_gemm(*args(128, 128, 100)) == 1      # k % 128 != 0
    assert rf_lib.rf_fp8_gemm(*args(0, 128, 128)) == 1
    assert rf_lib.rf_fp8_gemm(None, p16, p16, p16, p16, 128, 128, 128, 0, None, 0, None) == 2
    assert rf_lib.rf_fp8_gemm(p16 + 1, p16, p16, p16, p16, 128, 128, 128, 0, None, 0, None) == 3
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 128, 1024, 4) == 4 * 128 * 128 * 4
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 128, 1024, 1) == 0
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 100, 1024, 4) == 0
    # at most 64 K slices, and at most one per K block
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 128, 128 * 100, 100) == 64 * 128 * 128 * 4
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 128, 1024, 100) == 8 * 128 * 128 * 4
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128, 128, 1024, -2) == 0      # below RF_SPLIT_STREAMK: invalid


def test_public_header_compiles_as_c_and_cpp(tmp_path):
    """include/rf_b200.h is what a C or C++ caller of the reference binds against: plain C99, no CUDA headers."""
    import shutil
    import subprocess
    hdr = os.path.join(ROOT, "include", "rf_b200.h")
    for compiler, std, ext in (("gcc", "-std=c99", "c"), ("g++", "-std=c++17", "cpp")):
        if not shutil.which(compiler):
            continue
        src = tmp_path / f"t.{ext}"
        src.write_text(f'#include "{hdr}"\nint main(void) {{ PerfMetrics m; m.count = 0; return RF_OK + m.count; }}\n')
        res = subprocess.run([compiler, std, "-Wall", "-Wextra", "-pedantic", "-Werror", "-c", str(src), "-o",
                              str(tmp_path / f"t_{ext}.o")], capture_output=True, text=True)
        assert res.returncode == 0, res.stderr


def test_expert_parallel_entries_validate_on_the_host(rf_lib):
    """The multi-GPU entry points reject bad arguments before any device work (no GPU needed)."""
    buf = (ctypes.c_char * 4096)()
    p16 = (ctypes.addressof(buf) + 15) & ~15
    ptrs = (ctypes.c_void_p * 8)(*([p16] * 8))
    # scatter GEMM: null tables, bad world, n_dim % 64
    assert rf_lib.rf_moe_grouped_gemm_scatter(p16, 128, ptrs, p16, 1, 128, 128, None, ptrs, 2, None) == 2
    assert rf_lib.rf_moe_grouped_gemm_scatter(p16, 128, ptrs, p16, 1, 128, 128, p16, None, 2, None) == 2
    assert rf_lib.rf_moe_grouped_gemm_scatter(p16, 128, ptrs, p16, 1, 128, 128, p16, ptrs, 9, None) == 1
    assert rf_lib.rf_moe_grouped_gemm_scatter(p16, 128, ptrs, p16, 1, 100, 128, p16, ptrs, 2, None) == 1
    # dispatch: experts not divisible by the ranks, rank out of range, missing pointer
    d = lambda **kw: rf_lib.rf_moe_ep_dispatch(
        kw.get("x", p16), p16, p16, p16, p16, 64, 256, 128, kw.get("e", 8), kw.get("rank", 0), kw.get("world", 2),
        kw.get("cap", 512), ptrs, kw.get("meta", ptrs), p16, p16, None, None)
    assert d(e=7) == 1 and d(rank=2) == 1 and d(world=9) == 1
    assert d(cap=0) == 1                                                   # a receive buffer holds at least one row
    assert d(x=None) == 2
    assert rf_lib.rf_moe_ep_layout(p16, 0, 3, 8, 64, p16, p16, None) == 1      # 8 experts over 3 ranks
    assert rf_lib.rf_moe_ep_layout(p16, 0, 2, 8, 0, p16, p16, None) == 1       # capacity < 1


def test_expert_parallel_object_validates_its_configuration(rf_lib):
    """rf_moe_ep_create refuses bad configurations before it touches a device."""
    mk = lambda **kw: _lib.RfMoeEpConfig(*[kw.get(n, v) for n, v in (
        ("n_tokens", 64), ("d_hidden", 128), ("d_expert", 64), ("n_routed_experts", 8), ("n_experts_per_token", 2),
        ("n_shared_experts", 1), ("rank", 0), ("world", 2), ("capacity", 0), ("push_results", 1))])
    out = ctypes.c_void_p()
    create = lambda cfg: rf_lib.rf_moe_ep_create(ctypes.byref(cfg), ctypes.byref(out))
    assert create(mk(world=9)) == 1 and create(mk(rank=2)) == 1
    assert create(mk(n_tokens=0)) == 1 and create(mk(d_hidden=100)) == 1
    assert create(mk(n_routed_experts=6)) == 7            # power of two, divisible by the ranks
    assert create(mk(n_experts_per_token=9)) == 7
    assert create(mk(capacity=-1)) == 1
    assert rf_lib.rf_moe_ep_create(None, ctypes.byref(out)) == 2
    assert rf_lib.rf_moe_ep_forward(None, None, None, None) == 2


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.lib()
