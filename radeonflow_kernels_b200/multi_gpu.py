"""Single-node multi-GPU forms of the two hot paths, one process per GPU.

* ``fp8_gemm_nsplit`` - the large FP8 GEMM split along N; every rank's epilogue TMA-stores its
  column slab of C into every rank's full C over NVLink (the all-gather is part of the kernel).
* ``ExpertParallelMoE`` - the MoE layer with experts sharded ``E / world`` per rank; tokens are
  dispatched by peer stores into the owner's receive buffer and expert outputs are combined by
  peer loads.  The per-step control traffic (a [world, E] count all-gather and two barriers) also
  goes through peer memory (``rf_moe_ep_rendezvous``); ``torch.distributed`` (NCCL) is used at set-up
  to exchange the IPC handles, and by the N-split GEMM for its completion barrier.

The reference is single-GPU (no collective call anywhere in it); these are additions on top of
its operator boundary, built from the same C-ABI stage entry points.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib


# --------------------------------------------------------------------------- host-side planner --
def ep_layout_reference(counts_all: np.ndarray, rank: int):
    """numpy statement of what ``rf_moe_ep_layout`` computes on the device.

    counts_all [world, E]: row s = number of (token, expert) pairs per global expert on source rank s.
    Expert e is owned by rank q = e // (E // world).  In the owner's receive buffer rows are ordered by
    (expert, source rank in the rotated order q, q+1, ..., q+world-1 mod world, source-local order): every
    owner walks its experts' rows starting with its own tokens, so at any moment the owners return results
    to different GPUs.  Returns (send_base [E], recv_offsets [E/world + 1]).
    """
    counts_all = np.asarray(counts_all, dtype=np.int64)
    world, n_experts = counts_all.shape
    per = n_experts // world
    tot = counts_all.sum(axis=0)
    send_base = np.zeros(n_experts, dtype=np.int64)
    for e in range(n_experts):
        q = e // per
        first = q * per
        before_me = sum(int(counts_all[(q + j) % world, e]) for j in range((rank - q) % world))
        send_base[e] = tot[first:e].sum() + before_me
    recv = np.concatenate([[0], np.cumsum(tot[rank * per:(rank + 1) * per])])
    return send_base.astype(np.int32), recv.astype(np.int32)


def balanced_expert_placement(loads: np.ndarray, world: int) -> np.ndarray:
    """Static load-aware expert placement (greedy longest-processing-time): experts, heaviest first,
    go to the rank with the least load that still has a free slot (E/world slots per rank).

    `loads` [E]: pairs per expert observed on a calibration batch (or any popularity estimate).
    Returns `order` with order[r * E/world + j] = original id of rank r's j-th expert.  Renumbering
    the experts in this order (router rows, bias entries, weight list) leaves the layer unchanged
    while the owner of new id e' stays e' // (E/world), which is what the exchange kernels assume.
    """
    loads = np.asarray(loads, dtype=np.float64)
    n = loads.size
    per = n // world
    tot = np.zeros(world)
    slots = [[] for _ in range(world)]
    for e in np.argsort(-loads, kind="stable"):
        r = min((r for r in range(world) if len(slots[r]) < per), key=lambda r: (tot[r], r))
        slots[r].append(int(e))
        tot[r] += loads[e]
    return np.array([e for r in range(world) for e in slots[r]], dtype=np.int64)


# ------------------------------------------------------------------------------- peer buffers --
class _RawCuda:
    """Adapter so torch can view a raw device allocation without copying."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerBuffer:
    """Same-sized device buffer on every rank, each mapped into every process (CUDA IPC).

    ``ptrs[r]`` is rank r's buffer as addressable from this process; ``ptrs[rank]`` is local.
    """

    def __init__(self, nbytes: int, device, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.nbytes = int(nbytes)
        self.device = torch.device(device)
        L = _lib.lib()
        ptr = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _lib.check(L.rf_peer_alloc(self.nbytes, ctypes.byref(ptr), handle), "rf_peer_alloc")
            self.local_ptr = ptr.value
            self.ptrs = [None] * self.world
            self.ptrs[self.rank] = self.local_ptr
            self._opened = []
            if self.world > 1:
                mine = torch.tensor(list(handle), dtype=torch.uint8, device=self.device)
                allh = torch.empty(self.world * 64, dtype=torch.uint8, device=self.device)
                dist.all_gather_into_tensor(allh, mine, group=group)
                allh = allh.cpu().numpy().reshape(self.world, 64)
                for r in range(self.world):
                    if r == self.rank:
                        continue
                    h = (ctypes.c_ubyte * 64)(*allh[r].tolist())
                    p = ctypes.c_void_p()
                    _lib.check(L.rf_peer_open(h, ctypes.byref(p)), "rf_peer_open")
                    self.ptrs[r] = p.value
                    self._opened.append(p.value)
        self._raw = _RawCuda(self.local_ptr, self.nbytes)
        self.ptr_array = (ctypes.c_void_p * self.world)(*self.ptrs)

    def tensor(self, dtype, shape):
        """Local buffer viewed as a torch tensor (no copy)."""
        flat = torch.as_tensor(self._raw, device=self.device)
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return flat[:n].view(dtype).view(*shape)

    def close(self):
        L = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)
            for p in self._opened:
                L.rf_peer_close(ctypes.c_void_p(p))
            self._opened = []
            if self.world > 1:
                dist.barrier(group=self.group)
            if self.local_ptr:
                L.rf_peer_free(ctypes.c_void_p(self.local_ptr))
                self.local_ptr = None


def stream_barrier(flag: torch.Tensor, group=None):
    """Stream-ordered barrier across ranks: a one-element all-reduce on the current stream.  Work
    queued before it on every rank (peer stores included) is complete before work queued after it."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flag, group=group)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# --------------------------------------------------------------------------------- N-split GEMM --
def fp8_gemm_nsplit(a, b_shard, a_scale, b_scale_shard, c_buf: PeerBuffer, m: int, n_total: int, k: int):
    """C[:, rank*n/world : (rank+1)*n/world] = A . B_shard^T, written into every rank's C.

    a [m,k] e4m3 and a_scale [m,k/128] are replicated; b_shard [n_total/world, k] and
    b_scale_shard [n_total/world/128, k/128] are this rank's rows.  ``c_buf`` holds the bf16
    [m, n_total] result on every rank.  The caller places a ``stream_barrier`` after the call.
    """
    L = _lib.lib()
    st = L.rf_fp8_gemm_nsplit(a.data_ptr(), b_shard.data_ptr(), a_scale.data_ptr(), b_scale_shard.data_ptr(),
                              c_buf.ptr_array, m, n_total, k, c_buf.rank, c_buf.world, _stream())
    _lib.check(st, "rf_fp8_gemm_nsplit")


# ------------------------------------------------------------------------ expert-parallel layer --
class ExpertParallelMoE:
    """MoE layer with experts sharded over the ranks of ``group`` (expert e on rank e // (E/world)).

    weights: 'router.weight' [E, d] and 'shared_experts.{0,1,2}.weight' replicated on every rank;
    'experts.{j}.{0,1,2}.weight' for the LOCAL experts j = 0..E/world-1 (global id rank*E/world + j).
    Every rank feeds its own ``n_tokens`` tokens.  ``capacity`` = rows the receive buffers hold
    (default: worst case, every pair of every rank lands here).

    ``push_results`` (default): the experts' second GEMM stores every output row from its epilogue straight
    into the GPU that owns the token (`rf_moe_grouped_gemm_scatter`), so the transfer back overlaps the GEMM
    tile by tile and the final combine is local.  False: the outputs stay on the expert's GPU and the
    combine kernel pulls them over NVLink (`rf_moe_ep_combine`).
    """

    def __init__(self, config, weights, n_tokens: int, device, group=None, capacity=None, router_bias=None,
                 push_results: bool = True):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = torch.device(device)
        self.E = int(config["n_routed_experts"])
        self.K = int(config["n_experts_per_token"])
        self.d = int(config["d_hidden"])
        self.f = int(config["d_expert"])
        self.fs = self.f * int(config["n_shared_experts"])
        if self.E % self.world:
            raise ValueError("n_routed_experts must be divisible by the number of ranks")
        self.E_loc = self.E // self.world
        self.T = int(n_tokens)
        self.n_pairs = self.T * self.K
        self.capacity = int(capacity) if capacity else self.n_pairs * self.world
        self.weights = weights
        self.router_bias = router_bias
        # on one GPU nothing travels: the plain second GEMM (TMA stores) plus the gathering combine is faster
        self.push_results = bool(push_results) and self.world > 1
        self.trace = None           # set to [] to time the stages of the next forward
        dev, T, K, E, d, f = self.device, self.T, self.K, self.E, self.d, self.f
        i32, f16 = torch.int32, torch.float16
        e = lambda shape, dt: torch.empty(shape, dtype=dt, device=dev)
        self.scores = e((T, E), f16)
        self.idx = e((T, K), i32)
        self.gate_w = e((T, K), f16)
        self.source_rows = e((T * K,), i32)
        self.perm_experts = e((T * K,), i32)
        self.perm_rows = e((T * K,), i32)
        self.first = e((E + 1,), i32)
        self.rev = e((T * K,), i32)
        self.exp_w = e((T * K,), f16)
        self.pair_rank = e((T * K,), i32)
        self.pair_row = e((T * K,), i32)
        self.counts = e((E,), i32)
        self.send_base = e((E,), i32)
        self.recv_offsets = e((self.E_loc + 1,), i32)
        self.single_offsets = torch.tensor([0, T], dtype=i32, device=dev)
        self.sh1 = e((T, self.fs), f16)
        self.sh2 = e((T, d), f16)
        self.h = e((self.capacity, f), f16)
        self.out = e((T, d), f16)
        self.flag = torch.zeros(1, dtype=torch.float32, device=dev)
        L = _lib.lib()
        self.sort_scratch = e((max(16, L.rf_moe_permute_scratch_bytes(T * K, E)),), torch.uint8)
        self.side_stream = torch.cuda.Stream(device=dev)
        self.ev_ready = torch.cuda.Event()
        self.ev_sent = torch.cuda.Event()
        # sync area: 8 arrival flags + the [world, E] count matrix, zeroed before the first epoch
        self.sync = PeerBuffer(4 * (8 + self.world * E), dev, group)
        self.sync.tensor(torch.int32, (8 + self.world * E,)).zero_()
        self.counts_all = self.sync.tensor(torch.int32, (8 + self.world * E,))[8:]
        self.epoch = 0
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=group)           # every rank's sync area is zero before anyone raises a flag
        self.recv_x = PeerBuffer(self.capacity * d * 2, dev, group)
        if self.push_results:
            # results come home by peer stores: one row per local (token, expert) pair, expert-sorted order
            self.y = PeerBuffer(max(16, self.n_pairs * d * 2), dev, group)
            self.recv_meta = PeerBuffer(4 * self.capacity, dev, group)
        else:
            self.y = PeerBuffer(self.capacity * d * 2, dev, group)
            self.recv_meta = None

        def ptr_array(tensors):
            arr = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
            return arr
        self._w_gate = ptr_array([weights[f"experts.{j}.0.weight"] for j in range(self.E_loc)])
        self._w_up = ptr_array([weights[f"experts.{j}.1.weight"] for j in range(self.E_loc)])
        self._w_down = ptr_array([weights[f"experts.{j}.2.weight"] for j in range(self.E_loc)])
        self._s_gate = ptr_array([weights["shared_experts.0.weight"]])
        self._s_up = ptr_array([weights["shared_experts.1.weight"]])
        self._s_down = ptr_array([weights["shared_experts.2.weight"]])

    def forward(self, x):
        """x: fp16 [T, d] local tokens -> fp16 [T, d]."""
        L = _lib.lib()
        T, K, E, d, f = self.T, self.K, self.E, self.d, self.f
        s = _stream()
        chk = _lib.check
        self._mark("start")
        bias = self.router_bias.data_ptr() if self.router_bias is not None else None
        chk(L.rf_moe_router_gemm(x.data_ptr(), self.weights["router.weight"].data_ptr(), bias, T, E, d,
                                 self.scores.data_ptr(), s), "rf_moe_router_gemm")
        chk(L.rf_moe_topk(self.scores.data_ptr(), T, E, K, self.idx.data_ptr(), self.gate_w.data_ptr(),
                          self.source_rows.data_ptr(), s), "rf_moe_topk")
        chk(L.rf_moe_permute(self.idx.data_ptr(), self.source_rows.data_ptr(), self.gate_w.data_ptr(), T, E, K,
                             self.perm_experts.data_ptr(), self.perm_rows.data_ptr(), self.first.data_ptr(),
                             self.rev.data_ptr(), self.exp_w.data_ptr(), self.sort_scratch.data_ptr(), s),
            "rf_moe_permute")
        # pair counts per global expert, all-gathered through peer memory; the rendezvous also orders this
        # step after every rank's previous combine (its reads of our y buffer)
        torch.sub(self.first[1:], self.first[:-1], out=self.counts)
        self._rendezvous(self.counts.data_ptr(), E)
        self._mark("route+counts")
        chk(L.rf_moe_ep_layout(self.counts_all.data_ptr(), self.rank, self.world, E, self.send_base.data_ptr(),
                               self.recv_offsets.data_ptr(), s), "rf_moe_ep_layout")
        # Dispatch runs on a side stream; the shared expert, which needs no exchange, runs on the main
        # stream at the same time (the copy kernel's blocks need no shared memory and co-reside with
        # the GEMM's CTAs), hiding the NVLink transfer.
        main = torch.cuda.current_stream()
        self.ev_ready.record(main)
        self.side_stream.wait_event(self.ev_ready)
        side = ctypes.c_void_p(self.side_stream.cuda_stream)
        chk(L.rf_moe_ep_dispatch(x.data_ptr(), self.perm_experts.data_ptr(), self.perm_rows.data_ptr(),
                                 self.first.data_ptr(), self.send_base.data_ptr(), T, T * K, d, E, self.rank, self.world,
                                 self.recv_x.ptr_array, self.recv_meta.ptr_array if self.push_results else None,
                                 self.pair_rank.data_ptr(), self.pair_row.data_ptr(), side),
            "rf_moe_ep_dispatch")
        self.ev_sent.record(self.side_stream)
        chk(L.rf_moe_grouped_gemm(x.data_ptr(), T, self._s_gate, self._s_up, self.single_offsets.data_ptr(), 1,
                                  self.fs, d, self.sh1.data_ptr(), s), "shared fc1")
        chk(L.rf_moe_grouped_gemm(self.sh1.data_ptr(), T, self._s_down, None, self.single_offsets.data_ptr(), 1, d,
                                  self.fs, self.sh2.data_ptr(), s), "shared fc2")
        main.wait_event(self.ev_sent)
        self._mark("dispatch+shared")
        self._rendezvous(None, 0)                       # every rank's dispatch has landed
        self._mark("barrier1")
        chk(L.rf_moe_grouped_gemm(self.recv_x.local_ptr, self.capacity, self._w_gate, self._w_up,
                                  self.recv_offsets.data_ptr(), self.E_loc, f, d, self.h.data_ptr(), s), "routed fc1")
        self._mark("routed fc1")
        if self.push_results:
            chk(L.rf_moe_grouped_gemm_scatter(self.h.data_ptr(), self.capacity, self._w_down,
                                              self.recv_offsets.data_ptr(), self.E_loc, d, f,
                                              self.recv_meta.local_ptr, self.y.ptr_array, self.world, s),
                "routed fc2 + return")
        else:
            chk(L.rf_moe_grouped_gemm(self.h.data_ptr(), self.capacity, self._w_down, None,
                                      self.recv_offsets.data_ptr(), self.E_loc, d, f, self.y.local_ptr, s),
                "routed fc2")
        self._mark("routed fc2")
        self._rendezvous(None, 0)                       # every rank's expert outputs are complete (and home)
        self._mark("barrier2")
        if self.push_results:
            chk(L.rf_moe_combine(self.y.local_ptr, self.sh2.data_ptr(), self.rev.data_ptr(), self.exp_w.data_ptr(),
                                 T, K, d, self.out.data_ptr(), s), "rf_moe_combine")
            self._mark("combine")
            return self.out
        # (Running the shared expert's second GEMM concurrently with this combine and adding its rows
        # afterwards with rf_moe_add_rows was measured: no gain on 8 GPUs, and one more fp16 rounding.)
        chk(L.rf_moe_ep_combine(self.y.ptr_array, self.sh2.data_ptr(), self.rev.data_ptr(), self.exp_w.data_ptr(),
                                self.pair_rank.data_ptr(), self.pair_row.data_ptr(), T, K, d, self.world,
                                self.out.data_ptr(), s), "rf_moe_ep_combine")
        self._mark("combine")
        return self.out

    def _mark(self, name):
        """Stage timing aid: when `self.trace` is a list, records (name, CUDA event) pairs on the main stream."""
        if self.trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream())
            self.trace.append((name, ev))

    def stage_times_ms(self):
        """Milliseconds between consecutive marks of the last traced forward (synchronises)."""
        torch.cuda.synchronize()
        t = self.trace or []
        return [(t[i][0], t[i - 1][1].elapsed_time(t[i][1])) for i in range(1, len(t))]

    def _rendezvous(self, counts_ptr, n_counts):
        self.epoch += 1
        _lib.check(_lib.lib().rf_moe_ep_rendezvous(self.sync.ptr_array, counts_ptr, n_counts, self.rank, self.world,
                                                   self.epoch, _stream()), "rf_moe_ep_rendezvous")

    def received_rows(self) -> int:
        """Rows this rank's experts processed in the last forward (synchronises)."""
        return int(self.recv_offsets[-1].item())

    def close(self):
        self.recv_x.close()
        self.y.close()
        if self.recv_meta is not None:
            self.recv_meta.close()
        self.sync.close()
