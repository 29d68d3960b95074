"""CPU tests: the numpy GEMM oracle against fixtures made by the reference's own ref_kernel."""
import glob
import os

import numpy as np
import pytest

from oracle import fp8_gemm as o

_ALL = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "gemm_*.npz")))
GOLDEN = [p for p in _ALL if "fnuz" not in os.path.basename(p)]          # e4m3fn bytes, K-major
GOLDEN_FNUZ = [p for p in _ALL if "fnuz" in os.path.basename(p)]         # the reference's own e4m3fnuz data path


def test_golden_files_present():
    assert len(GOLDEN) >= 4


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_output(path):
    z = np.load(path)
    got = o.fp8_gemm(z["a"], z["b"], z["a_scale"], z["b_scale"])
    ok, nbad, _ = o.check(got, z["c_bits"], rtol=2e-2, atol=1e-3)
    assert ok, f"{nbad} elements outside the reference tolerance"
    # tighter than the tolerance: one bf16 ulp plus the fp32 summation-order noise of two different
    # BLAS calls (visible only on sums that nearly cancel), and rare
    g = o.bf16_bits_to_f32(got).astype(np.float64)
    e = o.bf16_bits_to_f32(z["c_bits"]).astype(np.float64)
    assert np.all(np.abs(g - e) <= np.abs(e) * 2.0 ** -7 + 1e-6 * np.abs(e).max())
    assert (got != z["c_bits"]).mean() < 1e-3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_blockwise_form_matches_reference_output(path):
    z = np.load(path)
    got = o.fp8_gemm_blockwise(z["a"], z["b"], z["a_scale"], z["b_scale"])
    ok, nbad, _ = o.check(got, z["c_bits"], rtol=2e-2, atol=1e-3)
    assert ok, nbad
    assert (got != z["c_bits"]).mean() < 1e-2


def test_e4m3fn_table_and_encoder():
    t = o.E4M3FN_TO_F32
    assert t[0x00] == 0.0 and t[0x7E] == 448.0 and np.isnan(t[0x7F]) and np.isnan(t[0xFF])
    assert t[0x38] == 1.0 and t[0xB8] == -1.0 and t[0x01] == 2.0 ** -9
    finite = np.array([b for b in range(256) if (b & 0x7F) != 0x7F and b != 0x80], dtype=np.uint8)
    assert np.array_equal(o.encode_e4m3fn(t[finite]), finite)
    # values with |x| <= 240 exist in e4m3fnuz too (bias 8: same set scaled by 1/2, max 240)
    vals = t[finite]
    vals = vals[np.abs(vals) <= 240]
    fnuz = set()
    for b in range(256):
        if b == 0x80:
            continue
        e, m = (b >> 3) & 0xF, b & 7
        v = (m / 8.0) * 2.0 ** -7 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 8)
        fnuz.add(-v if b & 0x80 else v)
    assert all(float(v) in fnuz for v in vals)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e-40], dtype=np.float32)
    bits = o.f32_to_bf16_bits(x)
    assert bits[0] == 0x3F80
    assert bits[1] == 0x3F80          # 1 + 2^-8: tie -> even
    assert bits[2] == 0x3F82          # 1 + 3*2^-8: tie -> even (up)
    assert o.bf16_bits_to_f32(bits)[3] == -2.5


def test_generator_is_seeded_and_clipped():
    a, b, a_s, b_s = o.generate_input(64, 128, 256, 7)
    a2, _, _, _ = o.generate_input(64, 128, 256, 7)
    assert np.array_equal(a, a2)
    assert np.nanmax(np.abs(o.decode_e4m3fn(a))) <= 240
    assert a_s.shape == (64, 2) and b_s.shape == (1, 2)
    assert a_s.min() >= 0.5 * 2 ** -7 and a_s.max() <= 2.0 * 2 ** -7


def test_e4m3fnuz_table_matches_torch():
    """The oracle's e4m3fnuz decode is torch's float8_e4m3fnuz (the dtype the reference generator casts to,
    scripts/problems/gemm/reference.py:28-29) for all 256 bytes, and its encoder rounds like torch's cast."""
    import torch
    t = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fnuz).float().numpy()
    assert np.array_equal(np.isnan(t), np.isnan(o.E4M3FNUZ_TO_F32))
    ok = ~np.isnan(t)
    assert np.array_equal(t[ok], o.E4M3FNUZ_TO_F32[ok])
    x = (np.random.default_rng(5).standard_normal(200000) * 70).astype(np.float32).clip(-240, 240)
    x[:16] = [0.0, -0.0, 2.0 ** -10, -2.0 ** -10, 2.0 ** -11, 240, -240, 232, 1.0625, 1.1875, 3e-4, -3e-4, 0.5, 1, 2, 4]
    mine = o.encode_e4m3fnuz(x)
    theirs = torch.from_numpy(x).to(torch.float8_e4m3fnuz).view(torch.uint8).numpy()
    assert np.array_equal(mine, theirs)


def test_e4m3fnuz_byte_is_half_its_e4m3fn_reading():
    """The identity the fnuz entry rests on: every e4m3fnuz byte except 0x80, 0x7F and 0xFF, read as
    e4m3fn, is exactly twice its value (subnormals included)."""
    for b in range(256):
        if b in (0x80, 0x7F, 0xFF):
            assert not np.isfinite(o.E4M3FN_TO_F32[b]) or b == 0x80
            continue
        assert o.E4M3FN_TO_F32[b] == 2.0 * o.E4M3FNUZ_TO_F32[b]


def test_fnuz_oracle_is_quarter_of_fn_oracle_on_shared_bytes():
    a, b, a_s, b_s = o.generate_input_fnuz(48, 128, 256, 11)
    assert not np.isin(a, [0x80, 0x7F, 0xFF]).any() and not np.isin(b, [0x80, 0x7F, 0xFF]).any()
    fz = o.bf16_bits_to_f32(o.fp8_gemm_fnuz(a, b, a_s, b_s))
    fn = o.bf16_bits_to_f32(o.f32_to_bf16_bits(np.float32(0.25) * o.fp8_gemm_f32(a, b, a_s, b_s)))
    assert np.allclose(fz, fn, rtol=2 ** -7, atol=1e-6 * np.abs(fz).max())


def test_fp8_codecs_round_trip_and_round_to_nearest():
    """encode(decode(b)) == b for every finite byte of both formats, and encode picks a nearest value
    (ties allowed either way at exact midpoints) for arbitrary inputs inside the format's range."""
    for dec, enc, table, top in ((o.decode_e4m3fn, o.encode_e4m3fn, o.E4M3FN_TO_F32, 448.0),
                                 (o.decode_e4m3fnuz, o.encode_e4m3fnuz, o.E4M3FNUZ_TO_F32, 240.0)):
        bytes_ = np.arange(256, dtype=np.uint8)
        vals = dec(bytes_)
        finite = np.isfinite(vals)
        back = enc(vals[finite])
        # -0 has no byte of its own in fnuz (0x80 is NaN) and may come back as +0 in fn
        assert np.array_equal(dec(back), vals[finite])
        rng = np.random.default_rng(0)
        x = np.concatenate([rng.uniform(-top, top, 20000), rng.standard_normal(20000),
                            rng.uniform(-2.0 ** -6, 2.0 ** -6, 5000)]).astype(np.float32)
        got = dec(enc(x)).astype(np.float64)
        grid = np.unique(table[np.isfinite(table)].astype(np.float64))
        nearest = np.abs(grid[None, :] - x.astype(np.float64)[:, None]).min(axis=1)
        assert np.allclose(np.abs(got - x), nearest, rtol=0, atol=1e-12)


@pytest.mark.parametrize("path", GOLDEN_FNUZ, ids=[os.path.basename(p) for p in GOLDEN_FNUZ])
def test_fnuz_oracle_matches_reference_output(path):
    """Fixtures made by the reference's own recipe (randn cast to float8_e4m3fnuz, transposed views) and its
    unmodified ref_kernel pin the e4m3fnuz reading of the numpy oracle."""
    z = np.load(path)
    assert len(GOLDEN_FNUZ) >= 2
    got = o.fp8_gemm_fnuz(z["a"], z["b"], z["a_scale"], z["b_scale"])
    ok, nbad, _ = o.check(got, z["c_bits"], rtol=2e-2, atol=1e-3)
    assert ok, f"{nbad} elements outside the reference tolerance"
    g = o.bf16_bits_to_f32(got).astype(np.float64)
    e = o.bf16_bits_to_f32(z["c_bits"]).astype(np.float64)
    assert np.all(np.abs(g - e) <= np.abs(e) * 2.0 ** -7 + 1e-6 * np.abs(e).max())
    assert (got != z["c_bits"]).mean() < 1e-3
