"""GPU parity tests of the FP8 block-scaled GEMM: CUDA path (through the C ABI) vs the numpy oracle.

Tolerance: rtol 2e-2 / atol 1e-3 on the bf16 output, the reference's own
(scripts/problems/gemm/reference.py:87, tests/gemm/gemm_test.cpp:202-205).
"""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import fp8_gemm as o
from radeonflow_kernels_b200 import gemm as G
from tests.helpers import canary_intact, canary_output, gemm_device_inputs

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 1e-3

# scripts/problems/gemm/task.yml:53-64 (tests) - shapes and seeds
REF_TEST_SHAPES = [
    (64, 64, 128, 6635), (64, 1536, 7168, 6635), (64, 3072, 1536, 1236), (64, 576, 7168, 542),
    (96, 7168, 256, 1234), (96, 7168, 2048, 4153), (96, 4608, 7168, 412), (128, 7168, 2304, 624),
    (128, 512, 7168, 2514), (512, 4096, 512, 543), (512, 1536, 7168, 12341),
]
# scripts/problems/gemm/task.yml:66-84 (benchmarks)
REF_BENCH_SHAPES = [
    (1024, 1536, 7168, 8135), (1024, 3072, 1536, 6251), (1024, 576, 7168, 12346), (1024, 7168, 256, 5364),
    (1024, 7168, 2048, 6132), (1024, 4608, 7168, 7531), (1024, 7168, 2304, 12345), (1024, 512, 7168, 6563),
    (1024, 4096, 512, 17512), (6144, 1536, 7168, 6543), (6144, 3072, 1536, 234), (6144, 576, 7168, 9863),
    (6144, 7168, 256, 764243), (6144, 7168, 2048, 76547), (6144, 4608, 7168, 65436), (6144, 7168, 2304, 452345),
    (6144, 512, 7168, 12341), (6144, 4096, 512, 45245),
]


def run_gemm(a, b, a_s, b_s, split_k=0, use_run_entry=True):
    m, n = a.shape[0], b.shape[0]
    full, c = canary_output(m, n)
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    if use_run_entry and split_k == 0:
        G.fp8_mm(da, db, das, dbs, c)
    else:
        G.fp8_mm(da, db, das, dbs, c, split_k=split_k, workspace=torch.empty(
            max(16, (split_k if split_k else 8) * m * n * 4), dtype=torch.uint8, device="cuda:0"))
    torch.cuda.synchronize()
    assert G.device_status() == 0, "a bounded device-side wait expired"
    assert canary_intact(full, m, n), "kernel wrote past the end of C"
    return c.view(torch.uint16).cpu().numpy()


def assert_close(got_bits, exp_bits):
    ok, nbad, mx = o.check(got_bits, exp_bits, RTOL, ATOL)
    assert ok, f"{nbad} of {got_bits.size} elements outside rtol={RTOL}/atol={ATOL}; max abs err {mx}"


_ALL_GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "gemm_*.npz")))
GOLDEN = [p for p in _ALL_GOLDEN if "fnuz" not in os.path.basename(p)]
GOLDEN_FNUZ = [p for p in _ALL_GOLDEN if "fnuz" in os.path.basename(p)]


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_against_reference_fixtures(path):
    z = np.load(path)
    got = run_gemm(z["a"], z["b"], z["a_scale"], z["b_scale"])
    assert_close(got, z["c_bits"])


@pytest.mark.parametrize("m,n,k,seed", REF_TEST_SHAPES)
@pytest.mark.parametrize("dist", ["baseline", "randn"])
def test_reference_test_shapes(m, n, k, seed, dist):
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, dist)
    assert_close(run_gemm(a, b, a_s, b_s), o.fp8_gemm(a, b, a_s, b_s))


@pytest.mark.parametrize("m,n,k,seed", REF_BENCH_SHAPES)
def test_reference_benchmark_shapes(m, n, k, seed):
    # signed N(0,1) scales (the reference generator's distribution) make atol=1e-3 bite
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
    assert_close(run_gemm(a, b, a_s, b_s), o.fp8_gemm(a, b, a_s, b_s))


def test_config0_baseline_distribution():
    a, b, a_s, b_s = o.generate_input(1024, 1536, 7168, 0, "baseline")
    assert_close(run_gemm(a, b, a_s, b_s), o.fp8_gemm(a, b, a_s, b_s))


@pytest.mark.parametrize("split", [1, 2, 3, 4, 7, 8])
def test_split_k_agrees_with_oracle(split):
    a, b, a_s, b_s = o.generate_input(320, 576, 2304, 99, "randn")
    assert_close(run_gemm(a, b, a_s, b_s, split_k=split), o.fp8_gemm(a, b, a_s, b_s))


# stream-K (split_k = -1): ragged last waves of the benchmark shapes, ragged M and N, a region smaller than one wave
# whose tiles are each shared by several CTAs, and one tile shared by all 148 CTAs (147 partial sums added in order)
STREAMK_SHAPES = [(1024, 7168, 2048, 5), (1024, 3072, 1536, 6), (6144, 512, 7168, 7), (6144, 7168, 2048, 8),
                  (1000, 1600, 1024, 9), (300, 4160, 896, 10), (1024, 1536, 7168, 11), (128, 64, 128 * 300, 12),
                  (4000, 4032, 384, 13)]


@pytest.mark.parametrize("m,n,k,seed", STREAMK_SHAPES)
def test_stream_k_agrees_with_oracle_and_is_deterministic(rf_lib, m, n, k, seed):
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    need = rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, -1)
    assert need > 0, "these shapes leave a ragged wave: the plan must be a stream-K pass"
    runs = []
    for rep in range(2):
        full, c = canary_output(m, n)
        # scratch with arbitrary old content: stale flags and slots must not matter
        ws = torch.randint(0, 255, (need,), dtype=torch.uint8, device="cuda:0")
        G.fp8_mm(da, db, das, dbs, c, split_k=-1, workspace=ws)
        torch.cuda.synchronize()
        assert G.device_status() == 0, "a bounded device-side wait expired"
        assert canary_intact(full, m, n)
        runs.append(c.view(torch.uint16).cpu().numpy())
    assert np.array_equal(runs[0], runs[1]), "partial sums are added in a fixed order: same bits every run"
    assert_close(runs[0], o.fp8_gemm(a, b, a_s, b_s))
    # too little scratch is refused on the host
    small = torch.empty(need - 256, dtype=torch.uint8, device="cuda:0")
    st = rf_lib.rf_fp8_gemm(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c.data_ptr(), m, n, k, -1,
                            small.data_ptr(), small.numel(), None)
    assert st == 4          # RF_ERR_WORKSPACE


def test_stream_k_back_to_back_launches_share_one_scratch(rf_lib):
    """Consecutive launches reuse slots and flags without clearing: each launch's flags carry its own number."""
    shapes = [(1024, 7168, 2048), (1024, 3072, 1536), (1024, 7168, 2048)]
    need = max(rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, -1) for (m, n, k) in shapes)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda:0")
    cases = []
    for i, (m, n, k) in enumerate(shapes):
        a, b, a_s, b_s = o.generate_input(m, n, k, 30 + i, "randn")
        cases.append((a, b, a_s, b_s, gemm_device_inputs(a, b, a_s, b_s), torch.empty((m, n), dtype=torch.bfloat16,
                                                                                     device="cuda:0")))
    for _ in range(3):
        for (a, b, a_s, b_s, dev, c) in cases:
            G.fp8_mm(*dev, c, split_k=-1, workspace=ws)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    for (a, b, a_s, b_s, dev, c) in cases:
        assert_close(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))


def test_stream_k_in_a_replayed_graph(rf_lib):
    """A captured launch carries the same flag number at every replay, so the flags must come back cleared: the
    owner clears what it consumed.  Operands change between replays; a stale flag would let an owner read the
    previous replay's partial sums (or half-written ones)."""
    m, n, k = 1024, 3072, 1536
    need = rf_lib.rf_fp8_gemm_workspace_bytes(m, n, k, -1)
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda:0")
    a, b, a_s, b_s = o.generate_input(m, n, k, 50, "randn")
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda:0")
    side = torch.cuda.Stream()
    G.fp8_mm(da, db, das, dbs, c, split_k=-1, workspace=ws)          # first use outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            G.fp8_mm(da, db, das, dbs, c, split_k=-1, workspace=ws)
            G.fp8_mm(da, db, das, dbs, c, split_k=-1, workspace=ws)
    for seed in (51, 52, 53):
        a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
        for dst, src in zip((da, db, das, dbs), gemm_device_inputs(a, b, a_s, b_s)):
            dst.copy_(src)
        c.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert G.device_status() == 0
        assert_close(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
    # nothing is left raised
    flags = ws[148 * 128 * 256 * 4:].view(torch.int64)
    assert int(flags.abs().sum().item()) == 0


@pytest.mark.parametrize("m", [1, 7, 33, 127, 129, 200, 255, 257])
def test_ragged_m(m):
    a, b, a_s, b_s = o.generate_input(m, 192, 384, 5 + m, "randn")
    assert_close(run_gemm(a, b, a_s, b_s), o.fp8_gemm(a, b, a_s, b_s))


def test_bitwise_against_blockwise_oracle_when_exact():
    # small-integer operands and power-of-two scales: every partial sum is exact in fp32, so the
    # result must be bit-identical whatever the summation order
    rng = np.random.default_rng(3)
    m, n, k = 256, 320, 1024
    a = o.encode_e4m3fn(rng.integers(-4, 5, (m, k)).astype(np.float32))
    b = o.encode_e4m3fn(rng.integers(-4, 5, (n, k)).astype(np.float32))
    a_s = (2.0 ** rng.integers(-3, 4, (m, k // 128))).astype(np.float32)
    b_s = (2.0 ** rng.integers(-3, 4, ((n + 127) // 128, k // 128))).astype(np.float32)
    got = run_gemm(a, b, a_s, b_s)
    exp = o.fp8_gemm_blockwise(a, b, a_s, b_s)
    assert np.array_equal(got, exp)
    assert np.array_equal(run_gemm(a, b, a_s, b_s, split_k=4), exp)


def test_scale_linearity_and_zero_scale_full_size():
    # size-independent properties at a benchmark size: doubling a_scale doubles C exactly (power of
    # two), zero b_scale rows zero the matching 128-column blocks
    m, n, k = 6144, 4608, 7168
    a, b, a_s, b_s = o.generate_input(m, n, k, 11, "baseline")
    base = run_gemm(a, b, a_s, b_s)
    dbl = run_gemm(a, b, (a_s * 2).astype(np.float32), b_s)
    assert np.array_equal(o.bf16_bits_to_f32(dbl), 2 * o.bf16_bits_to_f32(base))
    b_s0 = b_s.copy()
    b_s0[3, :] = 0
    z = o.bf16_bits_to_f32(run_gemm(a, b, a_s, b_s0))
    assert np.all(z[:, 384:512] == 0)
    assert np.array_equal(z[:, :384], o.bf16_bits_to_f32(base)[:, :384])
    # spot-check rows against the oracle
    rows = np.array([0, 1, 127, 128, 3000, 6143])
    exp = o.fp8_gemm(a[rows], b, a_s[rows], b_s)
    assert_close(base[rows], exp)


def test_largest_configuration_properties_and_spot_rows():
    """M = 16384, N = 28672, K = 7168 (the multi-GPU configuration, here on one GPU): operands drawn on the
    device, exact linearity in a power-of-two scale, and six full rows against the oracle."""
    m, n, k = 16384, 28672, 7168
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev)
    g.manual_seed(2024)
    a = torch.randn((m, k), device=dev, generator=g).clamp_(-240, 240).to(torch.float8_e4m3fn)
    b = torch.randn((n, k), device=dev, generator=g).clamp_(-240, 240).to(torch.float8_e4m3fn)
    a_s = ((0.5 + 1.5 * torch.rand((m, k // 128), device=dev, generator=g)) * 2.0 ** -7).float()
    b_s = ((0.5 + 1.5 * torch.rand((n // 128, k // 128), device=dev, generator=g)) * 2.0 ** -7).float()
    c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    c2 = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    G.fp8_mm(a, b, a_s, b_s, c)
    G.fp8_mm(a, b, a_s * 2, b_s, c2)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    assert torch.equal(c2.float(), 2 * c.float())
    del c2
    rows = torch.tensor([0, 127, 128, 8191, 12345, 16383], device=dev)
    exp = o.fp8_gemm(a[rows].view(torch.uint8).cpu().numpy(), b.view(torch.uint8).cpu().numpy(),
                     a_s[rows].cpu().numpy(), b_s.cpu().numpy())
    assert_close(c[rows].view(torch.uint16).cpu().numpy(), exp)


def test_extreme_fp8_values():
    m, n, k = 128, 128, 256
    rng = np.random.default_rng(8)
    vals = np.array([240.0, -240.0, 2.0 ** -9, -2.0 ** -9, 0.0, 1.0], dtype=np.float32)
    a = o.encode_e4m3fn(rng.choice(vals, (m, k)))
    b = o.encode_e4m3fn(rng.choice(vals, (n, k)))
    a_s = np.ones((m, 2), np.float32)
    b_s = np.ones((1, 2), np.float32)
    got = o.bf16_bits_to_f32(run_gemm(a, b, a_s, b_s)).astype(np.float64)
    af, bf = o.decode_e4m3fn(a).astype(np.float64), o.decode_e4m3fn(b).astype(np.float64)
    exact = af @ bf.T
    # products reach 57600 and sums cancel, so the reference tolerance is widened by the fp32
    # accumulation bound 2^-18 * sum|a||b| (any summation order of fp32 partial sums obeys it)
    bound = 1e-3 + 2e-2 * np.abs(exact) + 2.0 ** -18 * (np.abs(af) @ np.abs(bf).T)
    assert np.all(np.abs(got - exact) <= bound)


def test_perf_metrics_are_filled(rf_lib):
    import ctypes
    from radeonflow_kernels_b200 import _lib
    a, b, a_s, b_s = o.generate_input(1024, 1536, 7168, 0)
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    c = torch.empty((1024, 1536), dtype=torch.bfloat16, device="cuda:0")
    pm = _lib.PerfMetrics()
    rf_lib.run(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c.data_ptr(), 1024, 1536, 7168,
               ctypes.byref(pm), None)
    assert pm.count >= 1 and pm.entries[0].time > 0 and pm.entries[0].gflops > 0


@pytest.mark.parametrize("m,n,k,split", [(1024, 1536, 7168, 3), (1024, 576, 7168, 3), (1024, 512, 7168, 4),
                                         (300, 320, 2048, 8), (130, 64, 1024, 2), (6144, 512, 7168, 2)])
def test_library_scratch_and_caller_scratch_give_the_same_bits(rf_lib, m, n, k, split):
    """`run` (library-owned split-K scratch, plan from the table) against `rf_fp8_gemm` (caller's scratch, explicit
    split): same kernels, same slice order in the fix-up (src/gemm/gemm_kernel.cpp:288-303), so the same bits;
    twice in a row, because the library's scratch is reused."""
    a, b, a_s, b_s = o.generate_input(m, n, k, 77 + split, "randn")
    da, db, das, dbs = gemm_device_inputs(a, b, a_s, b_s)
    ws = torch.empty(split * m * n * 4, dtype=torch.uint8, device="cuda:0")
    full2, c2 = canary_output(m, n)
    assert rf_lib.rf_fp8_gemm(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c2.data_ptr(), m, n, k,
                              split, ws.data_ptr(), ws.numel(), None) == 0
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, 256 if n >= 256 else 128, split) == 0
    try:
        for _ in range(2):
            full1, c1 = canary_output(m, n)
            rf_lib.run(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c1.data_ptr(), m, n, k, None, None)
            torch.cuda.synchronize()
            assert canary_intact(full1, m, n) and canary_intact(full2, m, n)
            assert torch.equal(c1.view(torch.uint16), c2.view(torch.uint16))
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)
        rf_lib.rf_fp8_gemm_set_plan(1024, 1536, 7168, 256, 3)      # the built-in entries this test overwrote
        rf_lib.rf_fp8_gemm_set_plan(1024, 576, 7168, 128, 3)
        rf_lib.rf_fp8_gemm_set_plan(1024, 512, 7168, 128, 4)
    assert G.device_status() == 0
    assert_close(c1.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))


@pytest.mark.parametrize("block_n", ["512", "384"])
def test_cta_pair_configuration_matches_oracle(block_n):
    """The cta_group::2 configurations (256 x 256 and 256 x 128 tiles per 2-CTA cluster) are selected per
    process by an environment variable, so they run in a child process."""
    import subprocess
    import sys
    code = r'''
import os, sys
import numpy as np, torch
sys.path.insert(0, os.environ["RF_ROOT"])
from oracle import fp8_gemm as o
from radeonflow_kernels_b200 import gemm as G
for (m, n, k, split, dist) in [(300, 576, 1024, 1, "randn"), (1024, 1536, 7168, 1, "randn"), (512, 512, 2048, 2, "baseline")]:
    a, b, a_s, b_s = o.generate_input(m, n, k, 5, dist)
    d = lambda x, t=None: (torch.from_numpy(x).cuda().view(t) if t else torch.from_numpy(x).cuda())
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    G.fp8_mm(d(a, torch.float8_e4m3fn), d(b, torch.float8_e4m3fn), d(a_s), d(b_s), c, split_k=split)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    ok, nbad, mx = o.check(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))
    assert ok, (m, n, k, nbad, mx)
print("PAIR OK")
'''
    env = dict(os.environ, RF_FP8_GEMM_BN=block_n, RF_ROOT=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    res = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "PAIR OK" in res.stdout, (res.stdout + res.stderr)[-3000:]


@pytest.mark.parametrize("m,n,k,seed", [(64, 64, 128, 6635), (64, 576, 7168, 542), (96, 7168, 256, 1234),
                                         (128, 512, 7168, 2514), (512, 4096, 512, 543), (1024, 1536, 7168, 8135),
                                         (6144, 576, 7168, 9863), (1040, 320, 1024, 3)])
def test_reference_physical_layout_entry(rf_lib, m, n, k, seed):
    """`rf_fp8_gemm_colmajor`: operands as the reference stores them ([k][m], [k][n], scales [k/128][m] and
    [k/128][n/128]); same result as the oracle on the logical matrices."""
    a, b, a_s, b_s = o.generate_input(m, n, k, seed, "randn")
    from tests.helpers import to_dev
    da = to_dev(np.ascontiguousarray(a.T))
    db = to_dev(np.ascontiguousarray(b.T))
    das = to_dev(np.ascontiguousarray(a_s.T))
    dbs = to_dev(np.ascontiguousarray(b_s.T))
    full, c = canary_output(m, n)
    st = rf_lib.rf_fp8_gemm_colmajor(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c.data_ptr(),
                                     m, n, k, None, 0, None)
    assert st == 0
    torch.cuda.synchronize()
    assert G.device_status() == 0
    assert canary_intact(full, m, n)
    assert_close(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a, b, a_s, b_s))


def test_stream_k_plan_entry_is_a_plain_pass_where_stream_k_does_not_apply(rf_lib):
    """A shape whose table entry says stream-K still runs through the reference-layout entry (MN-major operands
    have no stream-K instantiation): the plan degrades to the plain pass, results unchanged."""
    m, n, k = 1040, 3072, 1536
    a, b, a_s, b_s = o.generate_input(m, n, k, 61, "randn")
    from tests.helpers import to_dev
    assert rf_lib.rf_fp8_gemm_set_plan(m, n, k, 256, -1) == 0
    try:
        assert rf_lib.rf_fp8_gemm_choose_split(m, n, k) == -1
        exp = o.fp8_gemm(a, b, a_s, b_s)
        # row-major entry: stream-K
        assert_close(run_gemm(a, b, a_s, b_s), exp)
        # reference layout: plain pass
        da, db = to_dev(np.ascontiguousarray(a.T)), to_dev(np.ascontiguousarray(b.T))
        das, dbs = to_dev(np.ascontiguousarray(a_s.T)), to_dev(np.ascontiguousarray(b_s.T))
        full, c = canary_output(m, n)
        st = rf_lib.rf_fp8_gemm_colmajor(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c.data_ptr(),
                                         m, n, k, None, 0, None)
        assert st == 0
        torch.cuda.synchronize()
        assert G.device_status() == 0 and canary_intact(full, m, n)
        assert_close(c.view(torch.uint16).cpu().numpy(), exp)
    finally:
        rf_lib.rf_fp8_gemm_set_plan(m, n, k, 0, 0)


def test_reference_physical_layout_rejects_unaligned_m(rf_lib):
    a, b, a_s, b_s = o.generate_input(72, 64, 128, 1)
    from tests.helpers import to_dev
    c = torch.empty((72, 64), dtype=torch.bfloat16, device="cuda:0")
    st = rf_lib.rf_fp8_gemm_colmajor(to_dev(np.ascontiguousarray(a.T)).data_ptr(), to_dev(b.T.copy()).data_ptr(),
                                     to_dev(a_s.T.copy()).data_ptr(), to_dev(b_s.T.copy()).data_ptr(), c.data_ptr(),
                                     72, 64, 128, None, 0, None)
    assert st == 1


@pytest.mark.parametrize("m,n,k,seed", [(64, 64, 128, 21), (96, 576, 512, 22), (1024, 1536, 7168, 23),
                                         (6144, 512, 1024, 24), (1040, 320, 1024, 25)])
def test_fnuz_entry_matches_fnuz_oracle(rf_lib, m, n, k, seed):
    """`rf_fp8_gemm_colmajor_fnuz`: reference layout and the reference's FP8 format (e4m3fnuz bytes)."""
    a, b, a_s, b_s = o.generate_input_fnuz(m, n, k, seed)
    from tests.helpers import to_dev
    da, db = to_dev(np.ascontiguousarray(a.T)), to_dev(np.ascontiguousarray(b.T))
    das, dbs = to_dev(np.ascontiguousarray(a_s.T)), to_dev(np.ascontiguousarray(b_s.T))
    full, c = canary_output(m, n)
    st = rf_lib.rf_fp8_gemm_colmajor_fnuz(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                          c.data_ptr(), m, n, k, None, 0, None)
    assert st == 0
    torch.cuda.synchronize()
    assert G.device_status() == 0
    assert canary_intact(full, m, n)
    assert_close(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm_fnuz(a, b, a_s, b_s))


def test_custom_kernel_takes_the_reference_generators_tuple():
    """Tensors built the way scripts/problems/gemm/reference.py:28-37 builds them (randn cast to
    float8_e4m3fnuz in [k, m] / [k, n], scales [k/128, m] / [k/128, n/128], all handed over as .T views)
    go through `custom_kernel` unchanged."""
    m, n, k = 1024, 576, 1024
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    a = torch.randn((k, m), dtype=torch.bfloat16, device="cuda", generator=gen).to(torch.float8_e4m3fnuz)
    b = torch.randn((k, n), dtype=torch.bfloat16, device="cuda", generator=gen).to(torch.float8_e4m3fnuz)
    a_s = torch.randn((k // 128, m), dtype=torch.float32, device="cuda", generator=gen)
    b_s = torch.randn((k // 128, (n + 127) // 128), dtype=torch.float32, device="cuda", generator=gen)
    c = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    out = G.custom_kernel((a.T, b.T, a_s.T, b_s.T, c))
    torch.cuda.synchronize()
    assert out is c and G.device_status() == 0
    exp = o.fp8_gemm_fnuz(a.T.contiguous().view(torch.uint8).cpu().numpy(), b.T.contiguous().view(torch.uint8).cpu().numpy(),
                          a_s.T.contiguous().cpu().numpy(), b_s.T.contiguous().cpu().numpy())
    assert_close(c.view(torch.uint16).cpu().numpy(), exp)


def _fnuz_call(rf_lib, a, b, a_s, b_s):
    from tests.helpers import to_dev
    m, n, k = a.shape[0], b.shape[0], a.shape[1]
    da, db = to_dev(np.ascontiguousarray(a.T)), to_dev(np.ascontiguousarray(b.T))
    das, dbs = to_dev(np.ascontiguousarray(a_s.T)), to_dev(np.ascontiguousarray(b_s.T))
    full, c = canary_output(m, n)
    st = rf_lib.rf_fp8_gemm_colmajor_fnuz(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(),
                                          c.data_ptr(), m, n, k, None, 0, None)
    assert st == 0
    torch.cuda.synchronize()
    assert canary_intact(full, m, n)
    return c.view(torch.uint16).cpu().numpy()


@pytest.mark.parametrize("bad,where", [(0x7F, "b"), (0xFF, "a"), (0x7F, "a")])
def test_fnuz_entry_computes_the_largest_magnitudes(rf_lib, bad, where):
    """+-240 (0x7F / 0xFF) has no e4m3fn reading at twice its value: the flagged operand is computed from its
    converted copy, the result still matches the fnuz oracle, the note (16) is reported once, and the GEMM
    that follows is unaffected."""
    m, n, k = 64, 128, 256
    a, b, a_s, b_s = o.generate_input_fnuz(m, n, k, 31)
    (a if where == "a" else b)[5, 77] = bad
    got = _fnuz_call(rf_lib, a, b, a_s, b_s)
    assert_close(got, o.fp8_gemm_fnuz(a, b, a_s, b_s))
    assert G.device_status() == 16          # a note, reported once and cleared by the read
    assert G.device_status() == 0
    a2, b2, a_s2, b_s2 = o.generate_input(96, 192, 384, 5, "randn")
    full, c = canary_output(96, 192)
    G.fp8_mm(*gemm_device_inputs(a2, b2, a_s2, b_s2), c)
    torch.cuda.synchronize()
    assert G.device_status() == 0 and canary_intact(full, 96, 192)
    assert_close(c.view(torch.uint16).cpu().numpy(), o.fp8_gemm(a2, b2, a_s2, b_s2))


@pytest.mark.parametrize("m,n,k,seed", [(64, 128, 256, 41), (96, 320, 512, 42), (1040, 576, 1024, 43)])
def test_fnuz_entry_on_amax_scaled_blocks(rf_lib, m, n, k, seed):
    """Block-quantised data (scale = amax / 240) puts +-240 into practically every 128-block of BOTH operands and
    many values below 2^-6 beside it; the result must still match the fnuz oracle."""
    rng = np.random.default_rng(seed)
    kb, nb = k // 128, (n + 127) // 128

    def quantise(x, blocks_r):
        """scale[r, kb] = amax of the block / 240; bytes = e4m3fnuz(x / scale): the block's largest element is +-240"""
        q = np.empty(x.shape, dtype=np.uint8)
        sc = np.empty((-(-x.shape[0] // blocks_r), kb), dtype=np.float32)
        for r in range(sc.shape[0]):
            for c in range(kb):
                blk = x[r * blocks_r:(r + 1) * blocks_r, c * 128:(c + 1) * 128]
                sc[r, c] = np.abs(blk).max() / np.float32(240.0)
                q[r * blocks_r:(r + 1) * blocks_r, c * 128:(c + 1) * 128] = o.encode_e4m3fnuz(blk / sc[r, c])
        return q, sc
    a, a_s = quantise(rng.standard_normal((m, k), dtype=np.float32), 1)
    b, b_s = quantise(rng.standard_normal((n, k), dtype=np.float32), 128)
    b_s = b_s[:nb]
    assert ((a & 0x7F) == 0x7F).sum() >= m * kb and ((b & 0x7F) == 0x7F).sum() >= nb * kb
    # every magnitude below 2^-6 (bytes 0x01-0x0F, the ones the conversion has to round) in both operands
    small = (rng.integers(1, 16, size=a[::3, 1::5].shape) | (rng.integers(0, 2, size=a[::3, 1::5].shape) << 7))
    a[::3, 1::5] = small.astype(np.uint8)
    b[1::2, 2::7] = (rng.integers(1, 16, size=b[1::2, 2::7].shape)).astype(np.uint8)
    assert not (a == 0x80).any() and not (b == 0x80).any()
    got = _fnuz_call(rf_lib, a, b, a_s, b_s)
    assert_close(got, o.fp8_gemm_fnuz(a, b, a_s, b_s))
    assert G.device_status() == 16 and G.device_status() == 0


def test_fnuz_nan_byte_stays_nan(rf_lib):
    """0x80 is NaN in e4m3fnuz (the reference's output would be NaN in that row); read as e4m3fn it would be
    -0.  The converted copy keeps it NaN: row 5 of C is NaN, every other row matches the oracle."""
    m, n, k = 64, 128, 256
    a, b, a_s, b_s = o.generate_input_fnuz(m, n, k, 31)
    a[5, 77] = 0x80
    got = _fnuz_call(rf_lib, a, b, a_s, b_s).view(np.uint16)
    is_nan = (got & 0x7FFF) > 0x7F80
    assert is_nan[5].all() and not np.delete(is_nan, 5, axis=0).any()
    a_ok = a.copy()
    a_ok[5, 77] = 0
    exp = o.fp8_gemm_fnuz(a_ok, b, a_s, b_s)
    assert_close(np.delete(got, 5, axis=0), np.delete(exp, 5, axis=0))
    assert G.device_status() == 16 and G.device_status() == 0


@pytest.mark.parametrize("path", GOLDEN_FNUZ, ids=[os.path.basename(p) for p in GOLDEN_FNUZ])
def test_fnuz_entry_against_reference_fixtures(rf_lib, path):
    """The reference's own data path (e4m3fnuz bytes, [k][m] / [k][n] storage) through `rf_fp8_gemm_colmajor_fnuz`
    against the output of the reference's unmodified ref_kernel."""
    z = np.load(path)
    a, b, a_s, b_s = z["a"], z["b"], z["a_scale"], z["b_scale"]
    m, k = a.shape
    n = b.shape[0]
    from tests.helpers import to_dev
    da, db = to_dev(np.ascontiguousarray(a.T)), to_dev(np.ascontiguousarray(b.T))
    das, dbs = to_dev(np.ascontiguousarray(a_s.T)), to_dev(np.ascontiguousarray(b_s.T))
    full, c = canary_output(m, n)
    assert rf_lib.rf_fp8_gemm_colmajor_fnuz(da.data_ptr(), db.data_ptr(), das.data_ptr(), dbs.data_ptr(), c.data_ptr(),
                                            m, n, k, None, 0, None) == 0
    torch.cuda.synchronize()
    assert G.device_status() == 0 and canary_intact(full, m, n)
    assert_close(c.view(torch.uint16).cpu().numpy(), z["c_bits"])
