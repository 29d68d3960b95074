"""Shared helpers of the GPU parity tests: numpy <-> device tensors, canaries."""
import numpy as np
import torch

CANARY = 0x7FC1  # a bf16 NaN payload no kernel produces


def to_dev(x: np.ndarray, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).to("cuda:0")
    return t.view(dtype) if dtype is not None else t


def gemm_device_inputs(a, b, a_s, b_s):
    return (to_dev(a, torch.float8_e4m3fn), to_dev(b, torch.float8_e4m3fn), to_dev(a_s), to_dev(b_s))


def canary_output(m: int, n: int, pad_rows: int = 8):
    """bf16 [m+pad, n] filled with a canary; returns (full buffer, view of the first m rows)."""
    full = torch.full(((m + pad_rows) * n,), CANARY, dtype=torch.uint16, device="cuda:0")
    out = full[: m * n].view(torch.bfloat16).view(m, n)
    return full, out


def canary_intact(full, m: int, n: int) -> bool:
    tail = full[m * n:]
    return bool((tail == CANARY).all().item())
