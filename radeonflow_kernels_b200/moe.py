"""Python boundary of the MoE layer.

Mirrors the reference's generated `custom_kernel(data)` for the MoE problem
(scripts/gen_submission.py:376-404): `data` = (input [bs, seq, d_hidden] fp16, weights dict with
the keys 'router.weight', 'experts.{i}.{0,1,2}.weight', 'shared_experts.{0,1,2}.weight', config
dict).  Unlike the reference wrapper, the router matmul also runs in the library (on the device),
not in PyTorch.  All tensors must be contiguous CUDA fp16 tensors; there is no CPU path.
"""
import ctypes

import torch

from . import _lib

_STAGE_FIELDS = {
    # name: (dtype, shape builder)
    "expert_scores": (torch.float16, lambda T, K, E, d, f, fs: (T, E)),
    "seq_experts_index": (torch.int32, lambda T, K, E, d, f, fs: (T, K)),
    "seq_experts_softmax": (torch.float16, lambda T, K, E, d, f, fs: (T, K)),
    "source_rows": (torch.int32, lambda T, K, E, d, f, fs: (T * K,)),
    "permuted_experts": (torch.int32, lambda T, K, E, d, f, fs: (T * K,)),
    "permuted_rows": (torch.int32, lambda T, K, E, d, f, fs: (T * K,)),
    "first_token_offset": (torch.int32, lambda T, K, E, d, f, fs: (E + 1,)),
    "expanded_seq_input": (torch.float16, lambda T, K, E, d, f, fs: (T * K, d)),
    "expanded_seq_softmax": (torch.float16, lambda T, K, E, d, f, fs: (T * K,)),
    "rev_permuted_rows": (torch.int32, lambda T, K, E, d, f, fs: (T * K,)),
    "expanded_fc1_output": (torch.float16, lambda T, K, E, d, f, fs: (T * K, f)),
    "expanded_fc2_output": (torch.float16, lambda T, K, E, d, f, fs: (T * K, d)),
    "shared_fc1_output": (torch.float16, lambda T, K, E, d, f, fs: (T, fs)),
    "shared_fc2_output": (torch.float16, lambda T, K, E, d, f, fs: (T, d)),
    "final_output": (torch.float16, lambda T, K, E, d, f, fs: (T, d)),
}


def _check_fp16_cuda(name, t):
    if not (t.is_cuda and t.dtype == torch.float16 and t.is_contiguous()):
        raise ValueError(f"moe: {name} must be a contiguous CUDA fp16 tensor (there is no CPU path)")


class MoEBuffers:
    """A filled MoEInputRaw (src/moe/moe.h:14-65) plus the torch tensors that own its buffers."""

    def __init__(self, x, weights, config, expert_scores=None):
        E = int(config["n_routed_experts"])
        K = int(config["n_experts_per_token"])
        d = int(config["d_hidden"])
        f = int(config["d_expert"])
        ns = int(config["n_shared_experts"])
        _check_fp16_cuda("input", x)
        T = x.numel() // d
        self.T, self.K, self.E, self.d, self.f, self.fs = T, K, E, d, f, f * ns
        raw = _lib.MoEInputRaw()
        raw.params = _lib.InputParams(int(config.get("batch_size", 1)), T // int(config.get("batch_size", 1)), d, f,
                                      E, K, ns, 0)
        self._keep = [x, weights]
        arrs = []
        for j in range(3):
            arr = (ctypes.c_void_p * E)()
            for i in range(E):
                w = weights[f"experts.{i}.{j}.weight"]
                _check_fp16_cuda(f"experts.{i}.{j}.weight", w)
                arr[i] = w.data_ptr()
            arrs.append(arr)
        self._keep.append(arrs)
        raw.expert_weight_gate = ctypes.cast(arrs[0], ctypes.POINTER(ctypes.c_void_p))
        raw.expert_weight_up = ctypes.cast(arrs[1], ctypes.POINTER(ctypes.c_void_p))
        raw.expert_weight_down = ctypes.cast(arrs[2], ctypes.POINTER(ctypes.c_void_p))
        for j, field in enumerate(("shared_expert_weight_gate", "shared_expert_weight_up", "shared_expert_weight_down")):
            w = weights[f"shared_experts.{j}.weight"]
            _check_fp16_cuda(f"shared_experts.{j}.weight", w)
            setattr(raw, field, w.data_ptr())
        _check_fp16_cuda("router.weight", weights["router.weight"])
        raw.router_weight = weights["router.weight"].data_ptr()
        raw.input_seq = x.data_ptr()
        self.stages = {}
        for name, (dtype, shape) in _STAGE_FIELDS.items():
            if name == "expert_scores" and expert_scores is not None:
                _check_fp16_cuda("expert_scores", expert_scores)
                t = expert_scores
            else:
                t = torch.empty(shape(T, K, E, d, f, self.fs), dtype=dtype, device=x.device)
            self.stages[name] = t
            setattr(raw, name, t.data_ptr())
        self.raw = raw


def moe_forward(x, weights, config, expert_scores=None, router_bias=None, metrics=None, fill_stages=True):
    """Runs the layer; returns (output [same shape as x], MoEBuffers with the stage tensors).

    `expert_scores` given  -> `run_topk` (the reference entry: logits are an input; every stage tensor is written);
    `expert_scores` None   -> the router GEMM runs on the device (optional fp32 bias).  With `fill_stages` it is
    followed by `run_topk`, so that every stage tensor of the reference's checker is written; without, the
    one-call entry `rf_moe_forward` runs (which, with `rf_moe_set_fused_gather(1)`, lets its first expert GEMM
    gather the token rows itself and leaves `expanded_seq_input` unwritten).
    """
    L = _lib.lib()
    buf = MoEBuffers(x, weights, config, expert_scores)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    pm = ctypes.byref(metrics) if metrics is not None else None
    if expert_scores is not None:
        st = L.run_topk(ctypes.byref(buf.raw), stream, pm)
        _lib.check(st, "run_topk")
    else:
        bias_ptr = None
        if router_bias is not None:
            if not (router_bias.is_cuda and router_bias.dtype == torch.float32 and router_bias.is_contiguous()):
                raise ValueError("moe: router_bias must be a contiguous CUDA float32 tensor")
            bias_ptr = router_bias.data_ptr()
            buf._keep.append(router_bias)
        if fill_stages:
            st = L.rf_moe_router_gemm(x.data_ptr(), weights["router.weight"].data_ptr(), bias_ptr, buf.T, buf.E, buf.d,
                                      buf.stages["expert_scores"].data_ptr(), stream)
            _lib.check(st, "rf_moe_router_gemm")
            st = L.run_topk(ctypes.byref(buf.raw), stream, pm)
            _lib.check(st, "run_topk")
        else:
            st = L.rf_moe_forward(ctypes.byref(buf.raw), bias_ptr, stream, pm)
            _lib.check(st, "rf_moe_forward")
    return buf.stages["final_output"].view(x.shape), buf


def custom_kernel(data):
    """scripts/gen_submission.py:376-404 - (input, weights, config) -> output tensor.

    Uses the library-owned workspace (`rf_run_from_python`, the counterpart of
    src/moe/moe.cpp:481-586) instead of per-call torch allocations.
    """
    x, weights, config = data
    _check_fp16_cuda("input", x)
    L = _lib.lib()
    E = int(config["n_routed_experts"])
    out = torch.empty_like(x)
    ull = ctypes.c_ulonglong
    ptrs = []
    for j in range(3):
        arr = (ull * E)()
        for i in range(E):
            w = weights[f"experts.{i}.{j}.weight"]
            _check_fp16_cuda(f"experts.{i}.{j}.weight", w)
            arr[i] = w.data_ptr()
        ptrs.append(arr)
    sh = [weights[f"shared_experts.{j}.weight"] for j in range(3)]
    for j, w in enumerate(sh):
        _check_fp16_cuda(f"shared_experts.{j}.weight", w)
    _check_fp16_cuda("router.weight", weights["router.weight"])
    bs = int(x.shape[0])
    seq = x.numel() // (bs * int(config["d_hidden"]))
    st = L.rf_run_from_python(
        seq, bs, int(config["d_hidden"]), int(config["d_expert"]), E, int(config["n_experts_per_token"]),
        int(config["n_shared_experts"]), x.data_ptr(), 0, ptrs[0], ptrs[1], ptrs[2], sh[0].data_ptr(),
        sh[1].data_ptr(), sh[2].data_ptr(), weights["router.weight"].data_ptr(), out.data_ptr(),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    _lib.check(st, "rf_run_from_python")
    return out
