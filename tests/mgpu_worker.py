"""Worker of the multi-GPU parity tests; launched by torch.distributed.run, one rank per GPU
(also valid with a single rank).  Checks, against the CPU oracle computed on the full problem:

  1. N-split FP8 GEMM: every rank ends up with the complete, correct C.
  2. Expert-parallel MoE: every rank's output rows equal the single-process oracle's rows, the
     top-k indices match the oracle's rule exactly, and the device-computed exchange layout equals
     the host-side planner.
Prints "MGPU OK rank=<r>" per rank on success.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import fp8_gemm as og  # noqa: E402
from oracle import moe as om  # noqa: E402
from radeonflow_kernels_b200 import gemm as G  # noqa: E402
from radeonflow_kernels_b200 import multi_gpu as mg  # noqa: E402


def main():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    flag = torch.zeros(1, device=dev)

    # ---- 1. N-split GEMM (small relative of M=16384, N=28672, K=7168)
    m, n, k = 384, 128 * world * 3, 1024
    a, b, a_s, b_s = og.generate_input(m, n, k, 77, "randn")
    n_loc = n // world
    sl = slice(rank * n_loc, (rank + 1) * n_loc)
    da = torch.from_numpy(a).to(dev).view(torch.float8_e4m3fn)
    db = torch.from_numpy(b[sl]).to(dev).view(torch.float8_e4m3fn)
    das = torch.from_numpy(a_s).to(dev)
    dbs = torch.from_numpy(b_s[rank * n_loc // 128:(rank + 1) * n_loc // 128]).to(dev)
    cbuf = mg.PeerBuffer(m * n * 2, dev)
    c = cbuf.tensor(torch.bfloat16, (m, n))
    c.fill_(float("nan"))
    mg.stream_barrier(flag)                      # nobody writes into a C that is still being cleared
    mg.fp8_gemm_nsplit(da, db, das, dbs, cbuf, m, n, k)
    mg.stream_barrier(flag)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    ok, nbad, mx = og.check(c.view(torch.uint16).cpu().numpy(), og.fp8_gemm(a, b, a_s, b_s))
    assert ok, f"rank {rank}: n-split GEMM {nbad} elements out of tolerance (max {mx})"
    cbuf.close()

    # ---- 2. expert-parallel MoE
    d, f, E, K, T_loc = 256, 128, 8 * world, 2, 96 + 16 * rank * 0
    T = T_loc * world
    x, w, cfg = om.generate_input(d, f, E, 1, K, T, 4242)
    bias = om.zipf_router_bias(E, 1.1, 5)
    e_loc = E // world
    wl = {"router.weight": w["router.weight"]}
    for j in range(e_loc):
        for q in range(3):
            wl[f"experts.{j}.{q}.weight"] = w[f"experts.{rank * e_loc + j}.{q}.weight"]
    for q in range(3):
        wl[f"shared_experts.{q}.weight"] = w[f"shared_experts.{q}.weight"]
    dw = {name: torch.from_numpy(v).to(dev) for name, v in wl.items()}
    x_loc = torch.from_numpy(x[0, rank * T_loc:(rank + 1) * T_loc]).to(dev)
    # first the variant whose combine pulls the expert outputs over NVLink, then (kept for the checks below)
    # the default one, whose second expert GEMM pushes its rows home from the epilogue
    pulled = mg.ExpertParallelMoE(cfg, dw, T_loc, dev, router_bias=torch.from_numpy(bias).to(dev), push_results=False)
    out_pull = pulled.forward(x_loc).clone()
    torch.cuda.synchronize()
    pulled.close()
    layer = mg.ExpertParallelMoE(cfg, dw, T_loc, dev, router_bias=torch.from_numpy(bias).to(dev))
    for _ in range(2):                           # twice: buffers are reused across steps
        out = layer.forward(x_loc)
    torch.cuda.synchronize()
    assert G.device_status() == 0
    assert torch.equal(out, out_pull), "push and pull variants must agree bit for bit (same fp32 combine order)"
    # oracle on the full problem, downstream of the logits this rank produced for its tokens
    logits_loc = layer.scores.cpu().numpy()
    ref_logits = om.router_logits(x[0], w["router.weight"], bias)
    okl, nb, mxl = om.check(logits_loc, ref_logits[rank * T_loc:(rank + 1) * T_loc])
    assert okl, f"rank {rank}: router logits {nb} out of tolerance"
    full_logits = ref_logits.copy()
    full_logits[rank * T_loc:(rank + 1) * T_loc] = logits_loc
    ref = om.moe_stages(x[0], w, E, K, logits16=full_logits)
    assert np.array_equal(layer.idx.cpu().numpy(), ref["seq_experts_index"][rank * T_loc:(rank + 1) * T_loc])
    ok, nbad, mx = om.check(out.cpu().numpy(), ref["final_output"][rank * T_loc:(rank + 1) * T_loc])
    assert ok, f"rank {rank}: EP MoE {nbad} elements out of tolerance (max {mx})"
    # exchange layout: device kernel == host planner
    counts_all = layer.counts_all.cpu().numpy().reshape(world, E)
    sb, ro = mg.ep_layout_reference(counts_all, rank)
    assert np.array_equal(layer.send_base.cpu().numpy(), sb)
    assert np.array_equal(layer.recv_offsets.cpu().numpy(), ro)
    assert layer.received_rows() == int(counts_all[:, rank * e_loc:(rank + 1) * e_loc].sum())
    # SM partition (the default on 2 to 4 GPUs): the dispatch as a few blocks that own an SM each and move the
    # rows with bulk copies, the shared expert's GEMMs beside them on the remaining SMs; and the dispatch spread
    # over every SM (the default on one GPU) - same result, bit for bit
    for blocks in (8, 0):
        layer.set_dispatch_blocks(blocks)
        out_part = layer.forward(x_loc).clone()
        torch.cuda.synchronize()
        assert G.device_status() == 0
        assert torch.equal(out_part, out_pull), f"dispatch with {blocks} blocks of its own changed the result"
    layer.set_dispatch_blocks(32 if 1 < world <= 4 else 0)
    layer.close()

    # ---- 3. receive buffers smaller than the traffic: rows beyond the capacity are dropped and reported,
    # never written; tokens that lost no pair still get the oracle's result
    need = int(counts_all[:, rank * e_loc:(rank + 1) * e_loc].sum())
    cap = max(8, min(int(counts_all[:, q * e_loc:(q + 1) * e_loc].sum()) for q in range(world)) // 2)
    small = mg.ExpertParallelMoE(cfg, dw, T_loc, dev, router_bias=torch.from_numpy(bias).to(dev), capacity=cap)
    out_small = small.forward(x_loc).clone()
    torch.cuda.synchronize()
    kept = (small.pair_rank.cpu().numpy() >= 0)
    assert small.received_rows() == min(need, cap)
    assert G.device_status() == 32, "the overflow must be reported"
    assert torch.isfinite(out_small.float()).all()
    # pair p (expert-sorted order) belongs to token perm_rows[p] % T_loc; recover it from the oracle's permutation
    ref_loc = om.moe_stages(x[0, rank * T_loc:(rank + 1) * T_loc], w, E, K, logits16=logits_loc)
    tok_of_pair = ref_loc["permuted_rows"] % T_loc
    whole = np.ones(T_loc, dtype=bool)
    whole[tok_of_pair[~kept]] = False
    if whole.any():
        okw, nbw, mxw = om.check(out_small.cpu().numpy()[whole], ref["final_output"][rank * T_loc:(rank + 1) * T_loc][whole])
        assert okw, f"rank {rank}: tokens that lost no pair differ ({nbw} elements, max {mxw})"
    small.close()
    print(f"MGPU OK rank={rank} world={world} gemm_maxerr={mx:.3g}", flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
