"""Python boundary of the FP8 block-scaled GEMM.

Mirrors the reference's torch extension `fp8_mm` and `custom_kernel`
(scripts/gen_submission.py:247-262, :327-330): same argument order, the output
tensor is caller-allocated and returned.  Operand layout is K-major:
a [m,k] e4m3fn, b [n,k] e4m3fn, a_scale [m,k/128] fp32, b_scale
[ceil(n/128),k/128] fp32, c [m,n] bf16, all contiguous CUDA tensors.
"""
import ctypes

import torch

from . import _lib


def _check_inputs(a, b, a_scale, b_scale, c):
    if not (a.is_cuda and b.is_cuda and a_scale.is_cuda and b_scale.is_cuda and c.is_cuda):
        raise ValueError("fp8_mm: all tensors must be CUDA tensors (there is no CPU path)")
    for name, t in (("a", a), ("b", b), ("a_scale", a_scale), ("b_scale", b_scale), ("c", c)):
        if not t.is_contiguous():
            raise ValueError(f"fp8_mm: {name} must be contiguous (K-major layout)")
    if a.element_size() != 1 or b.element_size() != 1:
        raise ValueError("fp8_mm: a and b must be 1-byte e4m3 tensors")
    if a_scale.dtype != torch.float32 or b_scale.dtype != torch.float32:
        raise ValueError("fp8_mm: scales must be float32")
    if c.dtype != torch.bfloat16:
        raise ValueError("fp8_mm: c must be bfloat16")
    m, k = a.shape
    n, k2 = b.shape
    if k != k2 or tuple(c.shape) != (m, n):
        raise ValueError("fp8_mm: shape mismatch")
    kb = k // 128
    nb = (n + 127) // 128
    if tuple(a_scale.shape) != (m, kb) or tuple(b_scale.shape) != (nb, kb):
        raise ValueError("fp8_mm: scale shape mismatch")
    return m, n, k


def fp8_mm(a, b, a_scale, b_scale, c, split_k: int = 0, workspace=None):
    """c[m,n] = bf16(sum_kb a_scale*b_scale * A_kb.B_kb^T) on the current stream.

    With ``workspace=None`` the library's `run` entry is used (library-owned
    split-K scratch); otherwise the status-returning `rf_fp8_gemm` with the
    caller's scratch tensor.
    """
    m, n, k = _check_inputs(a, b, a_scale, b_scale, c)
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if workspace is None and split_k == 0:
        L.run(a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(), m, n, k, None, stream)
        return c
    need = L.rf_fp8_gemm_workspace_bytes(m, n, k, split_k)
    if workspace is None and need:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    st = L.rf_fp8_gemm(a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(), m, n, k,
                       split_k, ws_ptr, ws_bytes, stream)
    _lib.check(st, "rf_fp8_gemm")
    return c


def fp8_mm_reference_layout(a, b, a_scale, b_scale, c, fnuz=None):
    """The same product on the tensors the reference's generator hands out
    (scripts/problems/gemm/reference.py:28-37): `a` is the transposed view of a contiguous [k, m] tensor,
    `b` of [k, n], `a_scale` of [k/128, m], `b_scale` of [k/128, ceil(n/128)]; c is contiguous [m, n] bf16.
    No transposed copy is made: the library reads the operands in place as MN-major tiles.

    ``fnuz``: whether the bytes are e4m3fnuz (the reference's dtype); None = decide from the dtype, with
    uint8 read as e4m3fn.  An e4m3fnuz operand that holds +-240 (0x7F / 0xFF, as amax-scaled data does) or
    NaN (0x80) is computed from a converted copy; `device_status()` then reports the note 16 once.
    """
    if not all(t.is_cuda for t in (a, b, a_scale, b_scale, c)):
        raise ValueError("fp8_mm_reference_layout: all tensors must be CUDA tensors (there is no CPU path)")
    for name, t in (("a", a), ("b", b), ("a_scale", a_scale), ("b_scale", b_scale)):
        if t.dim() != 2 or not t.t().is_contiguous():
            raise ValueError(f"fp8_mm_reference_layout: {name} must be the transpose of a contiguous tensor")
    if not c.is_contiguous() or c.dtype != torch.bfloat16:
        raise ValueError("fp8_mm_reference_layout: c must be contiguous bfloat16")
    if a.element_size() != 1 or b.element_size() != 1:
        raise ValueError("fp8_mm_reference_layout: a and b must be 1-byte e4m3 tensors")
    if a_scale.dtype != torch.float32 or b_scale.dtype != torch.float32:
        raise ValueError("fp8_mm_reference_layout: scales must be float32")
    m, k = a.shape
    n, k2 = b.shape
    if k != k2 or tuple(c.shape) != (m, n):
        raise ValueError("fp8_mm_reference_layout: shape mismatch")
    if tuple(a_scale.shape) != (m, k // 128) or tuple(b_scale.shape) != ((n + 127) // 128, k // 128):
        raise ValueError("fp8_mm_reference_layout: scale shape mismatch")
    if fnuz is None:
        fnuz = a.dtype == torch.float8_e4m3fnuz
        if (b.dtype == torch.float8_e4m3fnuz) != fnuz:
            raise ValueError("fp8_mm_reference_layout: a and b must use the same FP8 format")
    L = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    entry = L.rf_fp8_gemm_colmajor_fnuz if fnuz else L.rf_fp8_gemm_colmajor
    st = entry(a.data_ptr(), b.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), c.data_ptr(), m, n, k, None, 0,
               stream)
    _lib.check(st, entry.__name__)
    return c


def custom_kernel(data):
    """scripts/gen_submission.py:327-330.  Accepts both the K-major contiguous operands of `fp8_mm` and the
    reference generator's own tuple (transposed views, e4m3fnuz), told apart by the strides of `a`."""
    a, b, a_scale, b_scale, c = data
    if a.dim() == 2 and not a.is_contiguous() and a.t().is_contiguous():
        return fp8_mm_reference_layout(a, b, a_scale, b_scale, c)
    fp8_mm(a, b, a_scale, b_scale, c)
    return c


def device_status() -> int:
    """Synchronises, returns and clears the device status: the code (1-6) of a bounded device-side wait that
    expired, else a note that stopped nothing (16: e4m3fnuz operand read from converted bytes; 32:
    expert-parallel receive buffer overflow), else 0."""
    detail = ctypes.c_int(0)
    _lib.lib().rf_device_status(ctypes.byref(detail))
    return detail.value
