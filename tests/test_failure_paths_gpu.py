"""Failure detection on the GPU without faulting or hanging it: a bounded device-side wait is made to run
out (a flag that nothing sets, with the wait limit lowered to milliseconds), the kernel returns, the host
reads the status, and the device stays usable.  The reference has no counterpart: it aborts the process
(include/gpu_libs.h:31-37)."""
import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import fp8_gemm as o
from radeonflow_kernels_b200 import gemm as G
from tests.helpers import canary_intact, canary_output, gemm_device_inputs

pytestmark = pytest.mark.gpu


def _lonely_rendezvous(rf_lib, epoch):
    """World of two on ONE GPU: rank 0 is launched, rank 1 never is.  Both sync areas are local buffers."""
    mine = torch.zeros(16, dtype=torch.int32, device="cuda:0")
    theirs = torch.zeros(16, dtype=torch.int32, device="cuda:0")
    ptrs = (ctypes.c_void_p * 8)(mine.data_ptr(), theirs.data_ptr(), *([None] * 6))
    t0 = time.perf_counter()
    assert rf_lib.rf_moe_ep_rendezvous(ptrs, None, 0, 0, 2, epoch, None) == 0
    torch.cuda.synchronize()
    return mine.cpu().numpy(), theirs.cpu().numpy(), time.perf_counter() - t0


def _gemm_is_correct(m=192, n=320, k=512, seed=7):
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
    full, c = canary_output(m, n)
    G.fp8_mm(*gemm_device_inputs(a, b, a_s, b_s), c)
    torch.cuda.synchronize()
    assert canary_intact(full, m, n)
    ok, nbad, mx = o.check(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
    assert ok, (nbad, mx)


def test_a_wait_that_runs_out_returns_a_status_and_leaves_the_device_usable(rf_lib):
    assert G.device_status() == 0
    assert rf_lib.rf_set_wait_limit_ns(2_000_000) == 0          # 2 ms instead of 2 s
    try:
        mine, theirs, secs = _lonely_rendezvous(rf_lib, epoch=1)
        assert secs < 1.0, f"the wait should have given up after 2 ms, took {secs:.3f} s"
        assert theirs[0] == 1 and mine[0] == 1 and mine[1] == 0   # my flag went out, the peer's never came
        detail = ctypes.c_int(0)
        assert rf_lib.rf_device_status(ctypes.byref(detail)) == 6 and detail.value == 5   # RF_ERR_DEVICE_TIMEOUT, kErrSchedWait
        assert rf_lib.rf_device_status(ctypes.byref(detail)) == 0 and detail.value == 0   # reading cleared it
        _gemm_is_correct()
        assert G.device_status() == 0
    finally:
        assert rf_lib.rf_set_wait_limit_ns(0) == 0


def test_an_unread_status_from_an_earlier_launch_does_not_stop_later_kernels(rf_lib):
    """The recorded code carries the tag of the launch that lost its wait: kernels launched afterwards keep
    waiting normally and compute complete results even if nobody has read the status yet."""
    assert rf_lib.rf_set_wait_limit_ns(2_000_000) == 0
    try:
        _lonely_rendezvous(rf_lib, epoch=1)
    finally:
        assert rf_lib.rf_set_wait_limit_ns(0) == 0
    _gemm_is_correct(m=1024, n=576, k=7168, seed=11)             # split-K plan: two kernels, many waits each
    _gemm_is_correct(m=300, n=256, k=1024, seed=12)
    detail = ctypes.c_int(0)
    assert rf_lib.rf_device_status(ctypes.byref(detail)) == 6 and detail.value == 5     # still there, now cleared
    assert G.device_status() == 0
