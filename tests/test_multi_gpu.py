"""Multi-GPU paths.  CPU part: two gloo ranks exercise the expert-parallel exchange protocol (count
all-gather, host-side layout planner, row exchange, and both ways back: owners pull the expert rows, or the
experts push them to the return address that travelled with each row) against the single-process oracle.  GPU part:
torch.distributed.run launches tests/mgpu_worker.py with one rank per visible GPU (one is enough to
run the peer-memory code path; more exercise NVLink)."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


GLOO_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["RF_ROOT"])
from oracle import moe as om
from radeonflow_kernels_b200.multi_gpu import ep_layout_reference

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
d, f, E, K, T_loc = 64, 64, 8, 2, 40
T = T_loc * world
x, w, cfg = om.generate_input(d, f, E, 1, K, T, 99)
bias = om.zipf_router_bias(E, 1.1, 3)
e_loc = E // world
x_loc = x[0, rank * T_loc:(rank + 1) * T_loc]
# local routing and local stable sort by GLOBAL expert id
logits = om.router_logits(x_loc, w["router.weight"], bias)
idx, gw, src = om.route(logits, K)
pe, pr, first, rev = om.permute(idx, src, E)
counts = torch.from_numpy(np.diff(first).astype(np.int32))
gathered = [torch.zeros_like(counts) for _ in range(world)]
dist.all_gather(gathered, counts)
counts_all = np.stack([g.numpy() for g in gathered])
send_base, recv_off = ep_layout_reference(counts_all, rank)
# dispatch: rows for owner q form a contiguous run of the local sorted order
rows = torch.from_numpy(x_loc[pr % T_loc].astype(np.float32))
dest_row = send_base[pe] + (np.arange(len(pe)) - first[pe])
owner = pe // e_loc
cap = int(counts_all.sum())
recv = torch.zeros((cap, d))
recv_meta = np.full(cap, -1, dtype=np.int64)
for q in range(world):            # emulate the peer stores with point-to-point sends
    sel = np.nonzero(owner == q)[0]
    # beside every row travels its destination row and its return address (rank << 28) | sorted position
    meta_sel = ((rank << 28) | sel).astype(np.float64)
    payload = torch.cat([torch.from_numpy(dest_row[sel].astype(np.float32))[:, None], rows[sel],
                         torch.from_numpy(meta_sel)[:, None].float() * 0], dim=1)
    payload = payload.double()
    payload[:, -1] = torch.from_numpy(meta_sel)
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([len(sel)], dtype=torch.int64))
    if q == rank:
        for s in range(world):
            n = int(sizes[s])
            buf = payload if s == rank else torch.zeros((n, d + 2), dtype=torch.float64)
            if s != rank and n:
                dist.recv(buf, src=s)
            if n:
                recv[buf[:, 0].long()] = buf[:, 1:d + 1].float()
                recv_meta[buf[:, 0].long().numpy()] = buf[:, -1].long().numpy()
    elif len(sel):
        dist.send(payload, dst=q)
# experts on the received rows
recv16 = recv.numpy().astype(np.float16)
y = np.zeros((cap, d), dtype=np.float16)
for j in range(e_loc):
    a, b = int(recv_off[j]), int(recv_off[j + 1])
    e = rank * e_loc + j
    if b > a:
        h = om.swiglu_fc1(recv16[a:b], w[f"experts.{e}.0.weight"], w[f"experts.{e}.1.weight"])
        y[a:b] = om.linear_fp16(h, w[f"experts.{e}.2.weight"])
assert int(recv_off[-1]) == int(counts_all[:, rank * e_loc:(rank + 1) * e_loc].sum())
# combine: pull rows back (emulated by gathering every rank's y)
ys = [torch.zeros((int(counts_all[:, q * e_loc:(q + 1) * e_loc].sum()), d)) for q in range(world)]
for q in range(world):
    t = torch.from_numpy(y[: ys[q].shape[0]].astype(np.float32)) if q == rank else ys[q]
    dist.broadcast(t, src=q)
    ys[q] = t
sh = om.linear_fp16(om.swiglu_fc1(x_loc, w["shared_experts.0.weight"], w["shared_experts.1.weight"]),
                    w["shared_experts.2.weight"]).astype(np.float32)
wts = gw[pr % T_loc, pr // T_loc].astype(np.float32)
out = sh.copy()
for i in range(K):
    p = rev[i * T_loc + np.arange(T_loc)]
    yrow = np.stack([ys[owner[pp]][dest_row[pp]].numpy() for pp in p])
    out += wts[p][:, None] * yrow
ref = om.moe_stages(x[0], w, E, K, router_bias=bias)["final_output"][rank * T_loc:(rank + 1) * T_loc]
ok, nbad, mx = om.check(out.astype(np.float16), ref)
assert ok, (nbad, mx)
# push variant: every owner returns row i of its y to row (meta & mask) of rank (meta >> 28)'s buffer,
# which is laid out in that rank's expert-sorted order; the combine is then local (rev only)
n_rows = int(recv_off[-1])
assert (recv_meta[:n_rows] >= 0).all()
home = torch.zeros((len(pe), d))
for q in range(world):                      # q = the owner whose results are being returned
    if q == rank:
        dst_rank = recv_meta[:n_rows] >> 28
        slot = recv_meta[:n_rows] & ((1 << 28) - 1)
        for s in range(world):
            sel = np.nonzero(dst_rank == s)[0]
            msg = torch.cat([torch.from_numpy(slot[sel].astype(np.float64))[:, None],
                             torch.from_numpy(y[sel].astype(np.float64))], dim=1)
            if s == rank:
                home[msg[:, 0].long()] = msg[:, 1:].float()
            else:
                dist.send(torch.tensor([len(sel)], dtype=torch.int64), dst=s)
                if len(sel):
                    dist.send(msg, dst=s)
    else:
        n = torch.zeros(1, dtype=torch.int64)
        dist.recv(n, src=q)
        if int(n):
            msg = torch.zeros((int(n), d + 1), dtype=torch.float64)
            dist.recv(msg, src=q)
            home[msg[:, 0].long()] = msg[:, 1:].float()
out2 = sh.copy()
for i in range(K):
    p = rev[i * T_loc + np.arange(T_loc)]
    out2 += wts[p][:, None] * home[p].numpy()
assert np.array_equal(out2.astype(np.float16), out.astype(np.float16)), "push and pull protocols must agree"
print("GLOO OK", rank)
'''


def test_expert_parallel_protocol_two_gloo_ranks(tmp_path):
    script = tmp_path / "gloo_worker.py"
    script.write_text(GLOO_WORKER)
    env = dict(os.environ, RF_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2",
               OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"GLOO OK {r}" in o, o[-2000:]


def test_layout_planner_small_case():
    from radeonflow_kernels_b200.multi_gpu import ep_layout_reference
    counts = np.array([[1, 2, 0, 3], [4, 0, 5, 6]])        # 2 ranks, 4 experts (2 per rank)
    sb0, ro0 = ep_layout_reference(counts, 0)
    sb1, ro1 = ep_layout_reference(counts, 1)
    # owner 0 holds experts 0,1, sources in the order 0,1: rows [e0: r0(1) r1(4)] [e1: r0(2) r1(0)]
    # owner 1 holds experts 2,3, sources in the order 1,0: rows [e2: r1(5) r0(0)] [e3: r1(6) r0(3)]
    assert sb0.tolist() == [0, 5, 5, 11] and sb1.tolist() == [1, 7, 0, 5]
    assert ro0.tolist() == [0, 5, 7] and ro1.tolist() == [0, 5, 14]


def test_layout_planner_clips_to_the_receive_capacity():
    """Rows beyond the capacity are never addressed: every owner's row ranges stop at it, and the pairs a sender
    must drop are exactly those whose destination row reaches it."""
    from radeonflow_kernels_b200.multi_gpu import ep_layout_reference
    rng = np.random.default_rng(5)
    world, e = 4, 16
    per = e // world
    counts = rng.integers(0, 9, size=(world, e))
    for q in range(world):
        total = int(counts[:, q * per:(q + 1) * per].sum())
        cap = max(1, total // 2)
        _, ro_full = ep_layout_reference(counts, q)
        _, ro = ep_layout_reference(counts, q, capacity=cap)
        assert ro.tolist() == np.minimum(ro_full, cap).tolist() and ro[-1] == min(total, cap)
        # senders: rows kept + rows dropped = rows produced, and every kept row is below the capacity
        kept = 0
        for s in range(world):
            sb, _ = ep_layout_reference(counts, s, capacity=cap)
            for ex in range(q * per, (q + 1) * per):
                rows = sb[ex] + np.arange(counts[s, ex])
                kept += int((rows < cap).sum())
        assert kept == min(total, cap)


@pytest.mark.gpu
def test_multi_gpu_worker_all_visible_gpus():
    import torch
    n = min(torch.cuda.device_count(), 8)
    assert n >= 1
    while n & (n - 1):
        n -= 1
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "mgpu_worker.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    for r in range(n):
        assert f"MGPU OK rank={r}" in out, out[-4000:]


def test_balanced_expert_placement_is_a_permutation_and_balances_skewed_load():
    from radeonflow_kernels_b200.multi_gpu import balanced_expert_placement
    rng = np.random.default_rng(3)
    e, world = 256, 8
    # skewed popularity with a random rank per expert; the hottest expert stays below one rank's fair share
    # (top-k routing without replacement caps an expert at one pair per token), so a balanced placement exists
    loads = 1.0 / (1.0 + rng.permutation(e)) ** 0.5
    order = balanced_expert_placement(loads, world)
    assert sorted(order.tolist()) == list(range(e))                    # every expert placed exactly once
    per_rank = loads[order].reshape(world, e // world).sum(axis=1)
    contiguous = loads.reshape(world, e // world).sum(axis=1)
    assert per_rank.max() / per_rank.mean() < 1.05                     # near-perfect balance ...
    assert contiguous.max() / contiguous.mean() > per_rank.max() / per_rank.mean()     # ... better than id order
    # ties and equal loads: deterministic, still E/world experts per rank
    order2 = balanced_expert_placement(np.ones(16), 4)
    assert sorted(order2.tolist()) == list(range(16))
    assert order2.tolist() == balanced_expert_placement(np.ones(16), 4).tolist()


def test_layout_planner_matches_a_brute_force_statement():
    """send_base / recv_offsets against a direct construction of every owner's receive buffer: rows ordered
    by expert, then by source rank starting at the owner, then by the source's own order."""
    from radeonflow_kernels_b200.multi_gpu import ep_layout_reference
    rng = np.random.default_rng(11)
    world, e = 4, 16
    per = e // world
    counts = rng.integers(0, 7, size=(world, e))
    for q in range(world):                                             # build owner q's buffer explicitly
        rows, offsets = [], [0]
        for ex in range(q * per, (q + 1) * per):
            for j in range(world):
                s = (q + j) % world
                rows += [(ex, s, i) for i in range(counts[s, ex])]
            offsets.append(len(rows))
        for s in range(world):
            sb, ro = ep_layout_reference(counts, s)
            for ex in range(q * per, (q + 1) * per):
                if counts[s, ex]:
                    assert rows[sb[ex]] == (ex, s, 0) and rows[sb[ex] + counts[s, ex] - 1] == (ex, s, counts[s, ex] - 1)
            if s == q:
                assert ro.tolist() == offsets
