"""The allocation-free GEMM entry point (`rf_fp8_gemm_static_scratch`).

It serves callers that cannot allocate device memory where the GEMM runs (inside a graph
capture/replay loop, on a latency-critical thread that must stay out of the CUDA allocator, or when
all GPU memory belongs to another allocator): its split-K scratch is a fixed array inside the library.
The test calls it through the C ABI twice in a row, on different shapes that both use the shared
array, and requires bit-identical output to the ordinary entry point `rf_fp8_gemm` (same kernel,
same slice count, caller-provided scratch).  This file is named so that pytest collects it last.
"""
import numpy as np
import pytest
import torch

from oracle import fp8_gemm as o
from tests.helpers import canary_intact, canary_output, gemm_device_inputs

pytestmark = pytest.mark.gpu

STATIC_BYTES = 16 << 20


def run_both(rf_lib, m, n, k, split, seed):
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    full_new, c_new = canary_output(m, n)
    full_old, c_old = canary_output(m, n)
    st = rf_lib.rf_fp8_gemm_static_scratch(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                           c_new.data_ptr(), m, n, k, split, None)
    assert st == 0
    ws = torch.empty(max(16, rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, split)), dtype=torch.uint8, device="cuda:0")
    st = rf_lib.rf_fp8_gemm(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c_old.data_ptr(), m, n, k,
                            split, ws.data_ptr(), ws.numel(), None)
    assert st == 0
    torch.cuda.synchronize()
    assert canary_intact(full_new, m, n) and canary_intact(full_old, m, n)
    got = c_new.view(torch.uint16).cpu().numpy()
    ref = c_old.view(torch.uint16).cpu().numpy()
    assert np.array_equal(got, ref), "static-scratch variant differs from rf_fp8_gemm"
    ok, nbad, mx = o.check(got, o.fp8_gemm(a, b, a_s, b_s))
    assert ok, (nbad, mx)
    # the path's own status area: nothing expired, and reading it allocates nothing and leaves it clear
    import ctypes
    detail = ctypes.c_int(-1)
    assert rf_lib.rf_fp8_gemm_static_status(ctypes.byref(detail)) == 0 and detail.value == 0


def test_two_calls_in_a_row_match_the_ordinary_entry_point(rf_lib):
    # first call fills most of the shared array, the second reuses it with another geometry
    run_both(rf_lib, 1024, 512, 7168, 7, seed=1)       # 7 slices x 2 MiB = 14 MiB of the 16 MiB
    run_both(rf_lib, 320, 576, 2304, 3, seed=2)
    run_both(rf_lib, 256, 192, 1024, 1, seed=3)        # no scratch needed
    # stream-K through the built-in array: 128-wide tiles, 148 slots of 64 KiB and their flags
    assert 0 < rf_lib.rf_fp8_gemm_workspace_bytes(1024, 576, 7168, -1) <= STATIC_BYTES
    run_both(rf_lib, 1024, 576, 7168, -1, seed=4)


def test_automatic_split_never_exceeds_the_built_in_array(rf_lib):
    """1024 x 1536 x 7168: the tuned plan is 3 K slices (18.9 MB of scratch); with split_k = 0 the
    allocation-free entry must run it unsplit instead of refusing."""
    m, n, k = 1024, 1536, 7168
    assert rf_lib.rf_fp8_gemm_choose_split(m, n, k) * m * n * 4 > STATIC_BYTES
    a, b, a_s, b_s = o.generate_input(m, n, k, 9)
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda:0")
    st = rf_lib.rf_fp8_gemm_static_scratch(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                           c.data_ptr(), m, n, k, 0, None)
    assert st == 0
    torch.cuda.synchronize()
    ok, n_bad, max_err = o.check(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
    assert ok, (n_bad, max_err)


def test_sizes_beyond_the_built_in_array_are_rejected(rf_lib):
    m, n, k = 2048, 1024, 1024
    assert 8 * m * n * 4 > STATIC_BYTES
    a, b, a_s, b_s = o.generate_input(m, n, k, 4)
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda:0")
    st = rf_lib.rf_fp8_gemm_static_scratch(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                           c.data_ptr(), m, n, k, 8, None)
    assert st == 4          # RF_ERR_WORKSPACE
    st = rf_lib.rf_fp8_gemm_static_scratch(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                           c.data_ptr(), m, 100, k, 1, None)
    assert st == 1          # RF_ERR_BAD_SHAPE
