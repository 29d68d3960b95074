"""B200 (sm_100a) kernels for RadeonFlow's two hot paths: the FP8 block-scaled
GEMM and the MoE layer.  The compute lives in librf_b200.so (hand-written CUDA
behind a C ABI, see include/rf_b200.h); this package is the thin Python mirror
of the reference's Python-level boundary (scripts/gen_submission.py:247-262,
:327-330, :376-404).  PyTorch is used for device memory and streams only.
"""
from . import _lib  # noqa: F401
from .gemm import custom_kernel as gemm_custom_kernel, fp8_mm, fp8_mm_reference_layout  # noqa: F401
from .moe import custom_kernel as moe_custom_kernel, moe_forward  # noqa: F401

__all__ = ["fp8_mm", "fp8_mm_reference_layout", "gemm_custom_kernel", "moe_custom_kernel", "moe_forward"]
