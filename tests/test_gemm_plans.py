"""Tuned-plan table of the FP8 GEMM (the replacement of the reference's dispatch table and tuner,
src/gemm/gemm_launcher.cpp:229-247, tuner/gemm_tuner.py): host logic on CPU, effect on the GPU."""
import ctypes

import numpy as np
import pytest

from radeonflow_kernels_b200 import tune


def _get(L, m, n, k):
    bn, s = ctypes.c_int(0), ctypes.c_int(0)
    assert L.rf_fp8_gemm_get_plan(m, n, k, ctypes.byref(bn), ctypes.byref(s)) == 0
    return bn.value, s.value


def test_set_get_remove(rf_lib):
    shape = (1088, 1536, 7168)              # not one of the built-in entries
    model = _get(rf_lib, *shape)
    assert model[0] in (128, 256) and model[1] >= 1
    assert rf_lib.rf_fp8_gemm_set_plan(*shape, 128, 2) == 0
    assert _get(rf_lib, *shape) == (128, 2)
    assert rf_lib.rf_fp8_gemm_set_plan(*shape, 0, 0) == 0          # block_n 0 removes the entry
    assert _get(rf_lib, *shape) == model


def test_invalid_entries_are_rejected(rf_lib):
    assert rf_lib.rf_fp8_gemm_set_plan(1024, 1536, 7168, 100, 1) == 1      # tile width
    assert rf_lib.rf_fp8_gemm_set_plan(1024, 1536, 256, 128, 3) == 1       # more slices than K blocks
    assert rf_lib.rf_fp8_gemm_set_plan(1024, 100, 256, 128, 1) == 1        # n % 64
    assert rf_lib.rf_fp8_gemm_get_plan(1024, 100, 256, None, None) == 1


def test_builtin_table_covers_the_benchmark_shapes(rf_lib):
    for (m, n, k) in tune.BENCHMARK_SHAPES:
        bn, s = _get(rf_lib, m, n, k)
        assert bn in (128, 256, 512) and (1 <= s <= k // 128 or s == tune.STREAM_K)


def test_load_plans_file(rf_lib, tmp_path):
    path = tmp_path / "plans.txt"
    path.write_text("# comment\n2112 640 1024 128 2\n\n2112 704 1024 256 1   # trailing\nnot a line\n2112 768 1024 999 1\n")
    assert rf_lib.rf_fp8_gemm_load_plans(str(path).encode()) == -2         # malformed lines reported ...
    assert _get(rf_lib, 2112, 640, 1024) == (128, 2)                       # ... valid ones loaded
    assert _get(rf_lib, 2112, 704, 1024) == (256, 1)
    assert rf_lib.rf_fp8_gemm_load_plans(str(tmp_path / "missing.txt").encode()) == -1
    good = tmp_path / "good.txt"
    tune.write_plans([(2112, 640, 1024, 256, 1, 9.9)], str(good))
    assert rf_lib.rf_fp8_gemm_load_plans(str(good).encode()) == 1
    assert _get(rf_lib, 2112, 640, 1024) == (256, 1)
    for n in (640, 704):
        rf_lib.rf_fp8_gemm_set_plan(2112, n, 1024, 0, 0)


def test_tuner_candidates():
    c = tune.candidates(1024, 512, 7168)
    assert (128, 1) in c and (256, 1) in c and (128, 4) in c
    # tiles already fill the SMs: no split-K, but the ragged last wave (1344 tiles = 9.08 x 148) makes stream-K a candidate
    assert sorted(set(s for (_, s) in tune.candidates(6144, 7168, 2048))) == [tune.STREAM_K, 1]
    assert all(s == 1 for (_, s) in tune.candidates(128 * 148, 256, 1024))   # whole waves: nothing to share out
    assert all(s == tune.STREAM_K or 7168 // 128 // s >= 2 for (_, s) in c)
    assert (512, 1) in tune.candidates(6144, 4608, 7168, pair=True)
    assert tune.parse_shapes("64x128x256,1024X576x7168") == [(64, 128, 256), (1024, 576, 7168)]


@pytest.mark.gpu
@pytest.mark.parametrize("bn,split", [(128, 1), (128, 3), (256, 1), (256, 2)])
def test_registered_plan_is_used_and_correct(rf_lib, bn, split):
    import torch
    from oracle import fp8_gemm as o
    from radeonflow_kernels_b200 import gemm as G
    from tests.helpers import gemm_device_inputs
    m, n, k = 384, 576, 1024
    a, b, a_s, b_s = o.generate_input(m, n, k, 77, "randn")
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, bn, split) == 0
    try:
        assert rf_lib.rf_fp8_gemm_choose_split(m, n, k) == split
        assert rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, 0) == (split * m * n * 4 if split > 1 else 0)
        da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda:0")
        G.fp8_mm(da, db, das, dbs, c)
        torch.cuda.synchronize()
        assert G.device_status() == 0
        ok, n_bad, max_err = o.check(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
        assert ok, (n_bad, max_err)
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)


def test_stream_k_plan_entry(rf_lib):
    """A stream-K table entry is honoured where there is a ragged wave worth sharing out, and degrades to the plain
    pass where there is not (whole waves, or shares shorter than two K blocks)."""
    m, n, k = 1088, 3072, 1536                       # 9 x 12 = 108 tiles of 12 K blocks on 148 SMs
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, 256, tune.STREAM_K) == 0
    try:
        assert _get(rf_lib, m, n, k) == (256, tune.STREAM_K)
        assert rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, 0) == 148 * (128 * 256 * 4 + 8)
        assert rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, 2) == 2 * m * n * 4       # an explicit split still wins
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)
    m, n, k = 384, 576, 1024                         # 15 tiles x 8 K blocks: less than two K blocks per SM
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, 128, tune.STREAM_K) == 0
    try:
        assert _get(rf_lib, m, n, k) == (128, 1)
        assert rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, 0) == 0
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(300, 576, 512), (1024, 320, 256), (129, 64, 128), (2048, 1088, 384)])
def test_short_k_two_slab_configuration_with_ragged_tiles(rf_lib, m, n, k):
    """K <= 512 with the 256-wide tile runs the configuration with two store slabs per warp; N values that leave
    the last tile with one 64-column chunk (or a ragged one) exercise the slab alternation across tiles."""
    import torch
    from oracle import fp8_gemm as o
    from radeonflow_kernels_b200 import gemm as G
    from tests.helpers import canary_intact, canary_output, gemm_device_inputs
    a, b, a_s, b_s = o.generate_input(m, n, k, 5 + m, "randn")
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, 256, 1) == 0
    try:
        da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
        full, c = canary_output(m, n)
        for _ in range(2):
            G.fp8_mm(da, db, das, dbs, c)
        torch.cuda.synchronize()
        assert G.device_status() == 0
        assert canary_intact(full, m, n)
        ok, n_bad, max_err = o.check(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
        assert ok, (n_bad, max_err)
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)
