"""numpy restatement of the FP8 block-scaled GEMM reference (TEST INFRASTRUCTURE).

Follows scripts/problems/gemm/reference.py:40-85 of the reference project:
both operands are dequantised to fp32 by broadcasting their block scales
(reference.py:63-68 for A, :71-81 for B), multiplied as one fp32 matmul and the
result rounded to bf16 (:84).  The kernel-side formulation (scale product
applied to each 128-deep partial sum, src/gemm/gemm_kernel.cpp:173-207, :480)
is provided as ``fp8_gemm_blockwise`` for small shapes; both agree to fp32
rounding.

Layouts are the K-major ones: A [M,K] bytes, B [N,K] bytes, a_scale [M,K/128],
b_scale [ceil(N/128),K/128], all row-major; C [M,N] bf16 returned as uint16 bits.
FP8 bytes are OCP e4m3fn; the ``*_fnuz`` functions restate the same arithmetic for e4m3fnuz bytes.
"""
import numpy as np

BLOCK = 128


def _e4m3fn_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if e == 0xF and m == 0x7:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-6)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = v
    return t


E4M3FN_TO_F32 = _e4m3fn_table()


def decode_e4m3fn(u8: np.ndarray) -> np.ndarray:
    """Bytes (OCP e4m3fn) -> fp32 values."""
    return E4M3FN_TO_F32[np.asarray(u8, dtype=np.uint8)]


def encode_e4m3fn(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest e4m3fn byte (ties to even mantissa), saturating at +-448.

    Only used by the input generators; values are clipped by the caller.
    """
    x = np.asarray(x, dtype=np.float32)
    pos = E4M3FN_TO_F32[:0x7F].astype(np.float64)          # 0 .. 448, ascending
    ax = np.minimum(np.abs(x).astype(np.float64), 448.0)
    hi = np.searchsorted(pos, ax, side="left").clip(0, len(pos) - 1)
    lo = (hi - 1).clip(0, len(pos) - 1)
    dlo = np.abs(ax - pos[lo])
    dhi = np.abs(pos[hi] - ax)
    pick_lo = (dlo < dhi) | ((dlo == dhi) & ((lo & 1) == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    return (code | sign).astype(np.uint8)


def _e4m3fnuz_table() -> np.ndarray:
    """e4m3fnuz (bias 8, no infinities, no negative zero; 0x80 is the one NaN): the format the
    reference's kernels compute in (__hip_fp8_e4m3_fnuz, src/gemm/gemm_kernel.cpp:30-34) and its
    checker casts to (torch.float8_e4m3fnuz, tests/checker/checker.cpp)."""
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        s = -1.0 if b & 0x80 else 1.0
        e = (b >> 3) & 0xF
        m = b & 0x7
        if b == 0x80:
            v = np.nan
        elif e == 0:
            v = s * (m / 8.0) * 2.0 ** (-7)
        else:
            v = s * (1.0 + m / 8.0) * 2.0 ** (e - 8)
        t[b] = v
    return t


E4M3FNUZ_TO_F32 = _e4m3fnuz_table()


def decode_e4m3fnuz(u8: np.ndarray) -> np.ndarray:
    """Bytes (e4m3fnuz) -> fp32 values."""
    return E4M3FNUZ_TO_F32[np.asarray(u8, dtype=np.uint8)]


def encode_e4m3fnuz(x: np.ndarray) -> np.ndarray:
    """fp32 -> nearest e4m3fnuz byte (ties to even mantissa), saturating at +-240; zero is always 0x00."""
    x = np.asarray(x, dtype=np.float32)
    pos = E4M3FNUZ_TO_F32[:0x80].astype(np.float64)         # 0 .. 240, ascending
    ax = np.minimum(np.abs(x).astype(np.float64), 240.0)
    hi = np.searchsorted(pos, ax, side="left").clip(0, len(pos) - 1)
    lo = (hi - 1).clip(0, len(pos) - 1)
    dlo = np.abs(ax - pos[lo])
    dhi = np.abs(pos[hi] - ax)
    pick_lo = (dlo < dhi) | ((dlo == dhi) & ((lo & 1) == 0))
    code = np.where(pick_lo, lo, hi).astype(np.uint8)
    sign = np.where(code == 0, 0, np.signbit(x).astype(np.uint8) << 7).astype(np.uint8)
    return (code | sign).astype(np.uint8)


def fp8_gemm_fnuz(a_u8, b_u8, a_scale, b_scale) -> np.ndarray:
    """reference.py:40-85 on e4m3fnuz bytes - bf16 bits [M,N]."""
    m, k = a_u8.shape
    n = b_u8.shape[0]
    a = decode_e4m3fnuz(a_u8) * np.repeat(a_scale.astype(np.float32), BLOCK, axis=1)[:, :k]
    bs = np.repeat(np.repeat(b_scale.astype(np.float32), BLOCK, axis=0), BLOCK, axis=1)[:n, :k]
    b = decode_e4m3fnuz(b_u8) * bs
    return f32_to_bf16_bits(a @ b.T)


def generate_input_fnuz(m: int, n: int, k: int, seed: int, amax: float = 224.0):
    """Seeded e4m3fnuz operands: N(0,1) values (as the reference draws them, reference.py:28-31) stretched
    so that part of them reaches the top binade, clipped to +-amax, rounded to e4m3fnuz; signed N(0,1)
    scales.  amax < 232 keeps every byte inside the subset that reads as a finite e4m3fn value."""
    rng = np.random.default_rng(seed)
    a = encode_e4m3fnuz(np.clip(60.0 * rng.standard_normal((m, k), dtype=np.float32), -amax, amax))
    b = encode_e4m3fnuz(np.clip(60.0 * rng.standard_normal((n, k), dtype=np.float32), -amax, amax))
    kb = (k + BLOCK - 1) // BLOCK
    nb = (n + BLOCK - 1) // BLOCK
    a_s = (rng.standard_normal((m, kb), dtype=np.float32) / np.float32(60.0)).astype(np.float32)
    b_s = (rng.standard_normal((nb, kb), dtype=np.float32) / np.float32(60.0)).astype(np.float32)
    return a, b, a_s, b_s


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16, returned as uint16 bit patterns.

    Same integer trick as src/gemm/gemm_kernel.cpp:210-218 (finite inputs).
    """
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def dequantize(a_u8, a_scale, b_u8, b_scale):
    """reference.py:63-81 - returns fp32 A[M,K], B[N,K] with scales applied."""
    m, k = a_u8.shape
    n = b_u8.shape[0]
    a = decode_e4m3fn(a_u8) * np.repeat(a_scale.astype(np.float32), BLOCK, axis=1)[:, :k]
    bs = np.repeat(np.repeat(b_scale.astype(np.float32), BLOCK, axis=0), BLOCK, axis=1)[:n, :k]
    b = decode_e4m3fn(b_u8) * bs
    return a, b


def fp8_gemm_f32(a_u8, b_u8, a_scale, b_scale) -> np.ndarray:
    a, b = dequantize(a_u8, a_scale, b_u8, b_scale)
    return a @ b.T


def fp8_gemm(a_u8, b_u8, a_scale, b_scale) -> np.ndarray:
    """reference.py:40-85 - bf16 bits [M,N]."""
    return f32_to_bf16_bits(fp8_gemm_f32(a_u8, b_u8, a_scale, b_scale))


def fp8_gemm_blockwise(a_u8, b_u8, a_scale, b_scale) -> np.ndarray:
    """Kernel-order statement: sum_kb (a_s*b_s) * (A_kb . B_kb^T), fp32.

    src/gemm/gemm_kernel.cpp:173-207 and :473-482.  O(K/128) matmuls; small
    shapes only.
    """
    m, k = a_u8.shape
    n = b_u8.shape[0]
    a = decode_e4m3fn(a_u8)
    b = decode_e4m3fn(b_u8)
    acc = np.zeros((m, n), dtype=np.float32)
    nb_of_col = np.arange(n) // BLOCK
    for kb in range(k // BLOCK):
        part = a[:, kb * BLOCK:(kb + 1) * BLOCK] @ b[:, kb * BLOCK:(kb + 1) * BLOCK].T
        s = a_scale[:, kb][:, None].astype(np.float32) * b_scale[nb_of_col, kb][None, :].astype(np.float32)
        acc += s * part
    return f32_to_bf16_bits(acc)


def generate_input(m: int, n: int, k: int, seed: int, scale_dist: str = "baseline"):
    """Seeded inputs with the benchmark's value distributions.

    A, B ~ N(0,1) clipped to +-240 and rounded to e4m3fn; draw order A, B,
    a_scale, b_scale.  ``scale_dist``: "baseline" = U[0.5,2]*2^-7 (positive),
    "randn" = N(0,1) signed scales as in reference.py:32-33.
    """
    rng = np.random.default_rng(seed)
    a = encode_e4m3fn(np.clip(rng.standard_normal((m, k), dtype=np.float32), -240, 240))
    b = encode_e4m3fn(np.clip(rng.standard_normal((n, k), dtype=np.float32), -240, 240))
    kb = (k + BLOCK - 1) // BLOCK
    nb = (n + BLOCK - 1) // BLOCK
    if scale_dist == "baseline":
        a_s = ((0.5 + 1.5 * rng.random((m, kb), dtype=np.float32)) * np.float32(2.0 ** -7)).astype(np.float32)
        b_s = ((0.5 + 1.5 * rng.random((nb, kb), dtype=np.float32)) * np.float32(2.0 ** -7)).astype(np.float32)
    elif scale_dist == "randn":
        a_s = rng.standard_normal((m, kb), dtype=np.float32)
        b_s = rng.standard_normal((nb, kb), dtype=np.float32)
    else:
        raise ValueError(scale_dist)
    return a, b, a_s, b_s


def check(received_bits, expected_bits, rtol=2e-2, atol=1e-3):
    """|r-e| <= atol + rtol*|e| plus NaN/Inf agreement (scripts/utils.py:53-73).

    Returns (ok, n_bad, max_abs_err).
    """
    r = bf16_bits_to_f32(received_bits).astype(np.float64)
    e = bf16_bits_to_f32(expected_bits).astype(np.float64)
    with np.errstate(invalid="ignore"):
        bad = np.abs(r - e) > atol + rtol * np.abs(e)
    bad |= np.isnan(r) ^ np.isnan(e)
    bad |= np.isposinf(r) ^ np.isposinf(e)
    bad |= np.isneginf(r) ^ np.isneginf(e)
    with np.errstate(invalid="ignore"):
        mx = float(np.nanmax(np.abs(r - e))) if r.size else 0.0
    return (not bad.any()), int(bad.sum()), mx
