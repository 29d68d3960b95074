"""Stream-K work sharing of the FP8 GEMM, checked on the host: `rf_fp8_gemm_work_pieces` runs the very walker the
kernel's three roles run.  Every K block of every tile must be done exactly once; a CTA leaves at most one partial
tile behind (it has one scratch slot); and a tile's owner, the CTA that holds the tile's last K block, only ever
depends on CTAs of lower block index that took their share of the tile as the FIRST thing they did."""
import ctypes

import pytest

SMS = 148
# benchmark shapes of scripts/problems/gemm/task.yml:66-84 with ragged last waves, plus small and odd ones
SHAPES = [(6144, 7168, 2048, 256), (6144, 7168, 2304, 256), (6144, 4608, 7168, 256), (6144, 512, 7168, 256),
          (1024, 7168, 2048, 256), (1024, 3072, 1536, 256), (1024, 1536, 7168, 256), (1024, 576, 7168, 128),
          (1024, 512, 7168, 128), (320, 576, 2304, 128), (128, 64, 128 * 300, 128), (6144, 1536, 7168, 256)]


def pieces_of(lib, m, n, k, bn, split, sms, cta):
    buf = (ctypes.c_int * (4 * 64))()
    cnt = lib.rf_fp8_gemm_work_pieces(m, n, k, bn, split, sms, cta, buf, 64)
    assert 0 <= cnt <= 64
    return [tuple(buf[4 * i:4 * i + 4]) for i in range(cnt)]


@pytest.mark.parametrize("m,n,k,bn", SHAPES)
def test_stream_k_covers_every_k_block_once(rf_lib, m, n, k, bn):
    kb = k // 128
    tiles = -(-m // 128) * -(-n // bn)
    seen = {}
    per_cta = []
    for cta in range(SMS):
        ps = pieces_of(rf_lib, m, n, k, bn, -1, SMS, cta)
        per_cta.append(ps)
        for (tile, split, k0, k1) in ps:
            assert 0 <= tile < tiles and split == 0 and 0 <= k0 < k1 <= kb
            for q in range(k0, k1):
                assert (tile, q) not in seen, f"K block {q} of tile {tile} done twice"
                seen[(tile, q)] = cta
    assert len(seen) == tiles * kb
    # load balance: no CTA has more than one tile's worth of K blocks above the mean
    loads = [sum(k1 - k0 for (_, _, k0, k1) in ps) for ps in per_cta]
    assert max(loads) - min(loads) <= kb
    region = tiles % SMS and (tiles if tiles < SMS else tiles % SMS + SMS)
    if region:
        # the shared region is balanced to one K block
        shared = [sum(k1 - k0 for (t, _, k0, k1) in ps if t >= tiles - region) for ps in per_cta]
        assert max(shared) - min(shared) <= 1
    for cta, ps in enumerate(per_cta):
        partial = [p for p in ps if p[3] - p[2] != kb]
        contrib = [p for p in partial if p[3] < kb]          # stops short of the tile's end: leaves partial sums
        assert len(contrib) <= 1, "one scratch slot per CTA"
        if contrib:
            assert ps[0] == contrib[0], "a contributor's partial tile is the first thing it does"
        for (tile, _, k0, k1) in partial:
            if k1 == kb and k0 > 0:                          # owner: everything below k0 comes from lower CTAs
                helpers = {seen[(tile, q)] for q in range(k0)}
                assert helpers and max(helpers) < cta


def test_plain_and_split_k_launches_walk_as_before(rf_lib):
    m, n, k, bn = 1024, 1536, 7168, 256
    tiles, kb = 8 * 6, 56
    for split in (1, 3):
        done = set()
        for cta in range(SMS):
            for (tile, s, k0, k1) in pieces_of(rf_lib, m, n, k, bn, split, SMS, cta):
                assert (k0, k1) == (kb * s // split, kb * (s + 1) // split)
                assert (tile, s) not in done
                done.add((tile, s))
        assert len(done) == tiles * split
    # fewer work items than SMs: the grid shrinks, CTAs beyond it have nothing
    assert pieces_of(rf_lib, m, n, k, bn, 1, SMS, 48) == []
    assert rf_lib.rf_fp8_gemm_work_pieces(m, n, k, 192, 1, SMS, 0, (ctypes.c_int * 4)(), 1) == -1


def test_stream_k_scratch_size(rf_lib):
    # one 128 x block_n fp32 slot and one 64-bit flag per SM
    assert rf_lib.rf_fp8_gemm_workspace_bytes(6144, 7168, 2048, -1) == SMS * (128 * 256 * 4 + 8)
    # tiles that fill whole waves: a plain pass, no scratch
    assert rf_lib.rf_fp8_gemm_workspace_bytes(128 * 148, 256, 1024, -1) == 0
