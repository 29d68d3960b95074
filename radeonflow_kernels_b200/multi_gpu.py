"""Single-node multi-GPU forms of the two hot paths, one process per GPU.

* ``fp8_gemm_nsplit`` - the large FP8 GEMM split along N; every rank's epilogue TMA-stores its
  column slab of C into every rank's full C over NVLink (the all-gather is part of the kernel).
* ``ExpertParallelMoE`` - the MoE layer with experts sharded ``E / world`` per rank; tokens are
  dispatched by peer stores into the owner's receive buffer and expert outputs come home by peer
  stores from the second expert GEMM's epilogue (or are pulled by the combine).  The per-step control
  traffic (a [world, E] count all-gather and two barriers) also goes through peer memory; the step is
  sequenced by the library's C++ ``RfMoeEp`` object.  ``torch.distributed`` (NCCL) is used at set-up to
  exchange the IPC handles, and by the N-split GEMM for its completion barrier.

The reference is single-GPU (no collective call anywhere in it); these are additions on top of
its operator boundary, built from the same C-ABI stage entry points.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from . import _lib


# --------------------------------------------------------------------------- host-side planner --
def ep_layout_reference(counts_all: np.ndarray, rank: int, capacity=None):
    """numpy statement of what ``rf_moe_ep_layout`` computes on the device.

    counts_all [world, E]: row s = number of (token, expert) pairs per global expert on source rank s.
    Expert e is owned by rank q = e // (E // world).  In the owner's receive buffer rows are ordered by
    (expert, source rank in the rotated order q, q+1, ..., q+world-1 mod world, source-local order): every
    owner walks its experts' rows starting with its own tokens, so at any moment the owners return results
    to different GPUs.  Returns (send_base [E], recv_offsets [E/world + 1]).  With ``capacity`` (rows of the
    receive buffers) the row ranges are clipped to it, as the device kernel does: a pair whose destination row
    ``send_base[e] + i`` is >= capacity is not sent.
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
    if capacity is not None:
        recv = np.minimum(recv, int(capacity))
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

    A thin owner of the library's ``RfMoeEp`` object: the per-step sequence (router GEMM, top-k, sort,
    count exchange, dispatch beside the shared expert, routed experts, results home, combine), its
    buffers, streams, events and epochs all live in C++ (``csrc/moe_ep_api.cu``); ``forward`` is one
    call.  ``torch.distributed`` is used here only to exchange the IPC handles at set-up and for the
    barriers around set-up and tear-down.

    weights: 'router.weight' [E, d] and 'shared_experts.{0,1,2}.weight' replicated on every rank;
    'experts.{j}.{0,1,2}.weight' for the LOCAL experts j = 0..E/world-1 (global id rank*E/world + j).
    Every rank feeds its own ``n_tokens`` tokens.  ``capacity`` = rows the receive buffers hold
    (default: worst case, every pair of every rank lands here); rows beyond it are dropped and reported
    (``_lib`` status detail 32), never written.

    ``push_results`` (default): the experts' second GEMM stores every output row from its epilogue straight
    into the GPU that owns the token, so the transfer back overlaps the GEMM tile by tile and the final
    combine is local.  False: the outputs stay on the expert's GPU and the combine pulls them over NVLink.
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
        if self.E % self.world:
            raise ValueError("n_routed_experts must be divisible by the number of ranks")
        if capacity is not None and int(capacity) < 1:
            raise ValueError("capacity must be at least one row")
        self.E_loc = self.E // self.world
        self.T = int(n_tokens)
        self.weights = weights              # keeps the tensors alive: the library holds their addresses
        self.router_bias = router_bias
        self.out = torch.empty((self.T, self.d), dtype=torch.float16, device=self.device)
        L = _lib.lib()
        cfg = _lib.RfMoeEpConfig(self.T, self.d, self.f, self.E, self.K, int(config["n_shared_experts"]), self.rank,
                                 self.world, int(capacity) if capacity else 0, 1 if push_results else 0)
        ep = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(L.rf_moe_ep_create(ctypes.byref(cfg), ctypes.byref(ep)), "rf_moe_ep_create")
            self._ep = ep
            if self.world > 1:
                mine = (ctypes.c_ubyte * _lib.RF_MOE_EP_HANDLE_BYTES)()
                _lib.check(L.rf_moe_ep_handles(ep, mine), "rf_moe_ep_handles")
                t = torch.tensor(list(mine), dtype=torch.uint8, device=self.device)
                allh = torch.empty(self.world * _lib.RF_MOE_EP_HANDLE_BYTES, dtype=torch.uint8, device=self.device)
                dist.all_gather_into_tensor(allh, t, group=group)
                blob = (ctypes.c_ubyte * (self.world * _lib.RF_MOE_EP_HANDLE_BYTES))(*allh.cpu().tolist())
                _lib.check(L.rf_moe_ep_connect(ep, blob), "rf_moe_ep_connect")

            def ptr_array(names):
                return (ctypes.c_void_p * len(names))(*[weights[n].data_ptr() for n in names])
            self._w = [ptr_array([f"experts.{j}.{q}.weight" for j in range(self.E_loc)]) for q in range(3)]
            _lib.check(L.rf_moe_ep_set_weights(
                ep, weights["router.weight"].data_ptr(), router_bias.data_ptr() if router_bias is not None else None,
                self._w[0], self._w[1], self._w[2], weights["shared_experts.0.weight"].data_ptr(),
                weights["shared_experts.1.weight"].data_ptr(), weights["shared_experts.2.weight"].data_ptr()),
                "rf_moe_ep_set_weights")
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=group)       # every rank's sync area is zero and mapped before anyone raises a flag

    def forward(self, x):
        """x: fp16 [T, d] local tokens -> fp16 [T, d]."""
        _lib.check(_lib.lib().rf_moe_ep_forward(self._ep, x.data_ptr(), self.out.data_ptr(), _stream()),
                   "rf_moe_ep_forward")
        return self.out

    def set_trace(self, on: bool):
        _lib.check(_lib.lib().rf_moe_ep_set_option(self._ep, _lib.RF_MOE_EP_OPT_TRACE, 1 if on else 0), "trace")

    def set_dispatch_blocks(self, blocks: int):
        _lib.check(_lib.lib().rf_moe_ep_set_option(self._ep, _lib.RF_MOE_EP_OPT_DISPATCH_BLOCKS, int(blocks)),
                   "dispatch blocks")

    def stage_times_ms(self):
        """(name, milliseconds) of the stages of the last traced forward (synchronises)."""
        ms = (ctypes.c_float * 16)()
        names = (ctypes.c_char_p * 16)()
        n = _lib.lib().rf_moe_ep_stage_times(self._ep, ms, names, 16)
        return [(names[i].decode(), float(ms[i])) for i in range(n)]

    def _buffer(self, which, dtype, shape):
        p, nb = ctypes.c_void_p(), ctypes.c_size_t()
        _lib.check(_lib.lib().rf_moe_ep_buffer(self._ep, which, ctypes.byref(p), ctypes.byref(nb)), "rf_moe_ep_buffer")
        flat = torch.as_tensor(_RawCuda(p.value, nb.value), device=self.device)
        return flat.view(dtype).view(*shape)

    @property
    def scores(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_SCORES, torch.float16, (self.T, self.E))

    @property
    def idx(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_INDEX, torch.int32, (self.T, self.K))

    @property
    def counts_all(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_COUNTS_ALL, torch.int32, (self.world * self.E,))

    @property
    def send_base(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_SEND_BASE, torch.int32, (self.E,))

    @property
    def recv_offsets(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_RECV_OFFSETS, torch.int32, (self.E_loc + 1,))

    @property
    def pair_rank(self):
        return self._buffer(_lib.RF_MOE_EP_BUF_PAIR_RANK, torch.int32, (self.T * self.K,))

    def received_rows(self) -> int:
        """Rows this rank's experts processed in the last forward (synchronises)."""
        return int(self.recv_offsets[-1].item())

    def close(self):
        if self._ep is None:
            return
        L = _lib.lib()
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)      # nobody still reads or writes a peer's buffers
            L.rf_moe_ep_disconnect(self._ep)
            if self.world > 1:
                dist.barrier(group=self.group)      # every mapping of my buffers is closed before I free them
            L.rf_moe_ep_destroy(self._ep)
            self._ep = None
