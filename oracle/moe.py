"""numpy restatement of the MoE layer reference, stage by stage (TEST INFRASTRUCTURE).

End-to-end semantics: scripts/problems/moe/reference.py:10-142 (PyTorch oracle).
Stage semantics and tensor names: src/moe/moe_topk_kernel.cpp:15-251 and the
stage-level checker tests/moe/moe_topk_test.cpp:198-351.

Rounding points kept from the reference (all fp16 tensors): router logits,
softmax probabilities, the two fc1 products G and U, SiLU(G), H = SiLU(G)*U,
the fc2 product Y, the shared-expert output S, and the final sum.

Two things are defined more tightly than the reference does, so that expert
indices can be compared bit for bit on any machine:

* exp() inside the softmax is a fixed sequence of fp32 multiplies and adds
  (``det_exp``), and the row sum uses a fixed association order
  (``det_row_sum``); the CUDA kernel executes the same sequence.
* top-k ties: lowest expert index wins, the rule of
  src/moe/moe_topk_kernel.cpp:123 (torch.topk leaves ties unspecified).
"""
import numpy as np

F32 = np.float32
LOG2E = F32(1.4426950408889634)
# 2^f on [-0.5, 0.5]: Taylor coefficients ln2^i / i!, i = 0..7, rounded to fp32
EXP2_COEF = [F32(c) for c in (
    1.0, 0.6931471805599453, 0.2402265069591007, 0.05550410866482158, 0.009618129107628477,
    0.0013333558146428443, 0.0001540353039338161, 1.5252733804059840e-05)]
EXP_CLAMP = F32(-80.0)


def det_exp(x: np.ndarray) -> np.ndarray:
    """exp(x) for x <= 0 as a fixed fp32 operation sequence (no fused multiply-add).

    t = max(x, -80) * log2(e); n = rint(t); f = t - n; Horner in f; scale by 2^n.
    """
    x = np.maximum(np.asarray(x, dtype=F32), EXP_CLAMP)
    t = (x * LOG2E).astype(F32)
    n = np.rint(t).astype(F32)
    f = (t - n).astype(F32)
    p = np.full_like(f, EXP2_COEF[7])
    for c in EXP2_COEF[6::-1]:
        p = ((p * f).astype(F32) + c).astype(F32)
    return np.ldexp(p, n.astype(np.int32)).astype(F32)


def det_row_sum(e: np.ndarray) -> np.ndarray:
    """Row sums of fp32 [T, E] in the kernel's order.

    32 lanes per row; lane l owns the contiguous slice [l*V, (l+1)*V), V = max(E/32, 1)
    (lanes >= E contribute 0 when E < 32); each lane adds its slice left to right,
    then lanes are combined by a butterfly with strides 16, 8, 4, 2, 1.
    """
    t, n_e = e.shape
    v = max(n_e // 32, 1)
    lanes = np.zeros((t, 32), dtype=F32)
    part = e.reshape(t, -1, v)
    acc = part[:, :, 0].astype(F32)
    for j in range(1, v):
        acc = (acc + part[:, :, j]).astype(F32)
    lanes[:, : acc.shape[1]] = acc
    idx = np.arange(32)
    for stride in (16, 8, 4, 2, 1):
        lanes = (lanes + lanes[:, idx ^ stride]).astype(F32)
    return lanes[:, 0]


def softmax_fp16(logits16: np.ndarray) -> np.ndarray:
    """src/moe/moe_topk_kernel.cpp:65-97: fp16 row max, fp32 exp and sum, prob = fp16(e * (1/sum))."""
    lg = np.asarray(logits16, dtype=np.float16)
    mx = lg.max(axis=1, keepdims=True).astype(F32)
    e = det_exp((lg.astype(F32) - mx).astype(F32))
    s = det_row_sum(e)
    r = (F32(1.0) / s).astype(F32)
    return (e * r[:, None]).astype(F32).astype(np.float16)


def topk_lowest_index(probs16: np.ndarray, k: int):
    """k rounds of arg-max, ties to the lowest index, winners cleared (moe_topk_kernel.cpp:101-148).

    Returns (index int32 [T,k], weight fp16 [T,k]) in descending-score order.
    """
    p = probs16.astype(np.float32).copy()
    t = p.shape[0]
    idx = np.zeros((t, k), dtype=np.int32)
    w = np.zeros((t, k), dtype=np.float16)
    rows = np.arange(t)
    for i in range(k):
        j = np.argmax(p, axis=1)          # first maximum = lowest index
        idx[:, i] = j
        w[:, i] = probs16[rows, j]
        p[rows, j] = -np.inf
    return idx, w


def route(logits16: np.ndarray, k: int):
    """topk_kernel outputs: (seq_experts_index [T,k], seq_experts_softmax [T,k], source_rows [T*k])."""
    probs = softmax_fp16(logits16)
    idx, w = topk_lowest_index(probs, k)
    t = logits16.shape[0]
    source_rows = (np.arange(k, dtype=np.int32)[None, :] * t + np.arange(t, dtype=np.int32)[:, None]).reshape(-1)
    return idx, w, source_rows


def permute(seq_experts_index: np.ndarray, source_rows: np.ndarray, n_experts: int):
    """Stable sort of (expert, source_row) by expert (src/moe/moe.cpp:119-126), the offsets of
    compute_first_token_offset (moe_topk_kernel.cpp:152-172) and the inverse map of expand_input
    (:199-201).  Returns (permuted_experts, permuted_rows, first_token_offset [E+1], rev_permuted_rows).
    """
    flat = seq_experts_index.reshape(-1).astype(np.int32)
    order = np.argsort(flat, kind="stable")
    permuted_experts = flat[order].astype(np.int32)
    permuted_rows = source_rows[order].astype(np.int32)
    first = np.searchsorted(permuted_experts, np.arange(n_experts + 1), side="left").astype(np.int32)
    rev = np.zeros_like(permuted_rows)
    rev[permuted_rows] = np.arange(permuted_rows.size, dtype=np.int32)
    return permuted_experts, permuted_rows, first, rev


def linear_fp16(x16: np.ndarray, w16_in_out: np.ndarray) -> np.ndarray:
    """fp16 x fp16 -> fp32 accumulate -> fp16, weights given as [in, out]."""
    return (x16.astype(F32) @ w16_in_out.astype(F32)).astype(np.float16)


def silu_fp16(g16: np.ndarray) -> np.ndarray:
    g = g16.astype(F32)
    return (g / (F32(1.0) + np.exp(-g, dtype=F32))).astype(np.float16)


def swiglu_fc1(x16, w_gate, w_up):
    """fp16(SiLU(fp16(x.Wg)) * fp16(x.Wu)) - scripts/problems/moe/reference.py:23-24."""
    g = silu_fp16(linear_fp16(x16, w_gate))
    u = linear_fp16(x16, w_up)
    return (g.astype(F32) * u.astype(F32)).astype(np.float16)


def router_logits(x16, router_w16, bias=None):
    """fp16 logits [T,E] = x . router_w^T (+ fp32 bias before the fp16 rounding)."""
    acc = x16.astype(F32) @ router_w16.astype(F32).T
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=F32)[None, :]
    return acc.astype(np.float16)


def moe_stages(x16, weights, n_experts, top_k, logits16=None, router_bias=None):
    """All stage tensors of the layer (names of src/moe/moe.h:14-65).

    x16: fp16 [T, d]; weights: dict with 'router.weight' [E,d], 'experts.{e}.{0,1,2}.weight',
    'shared_experts.{0,1,2}.weight' ([in,out] layout) - the reference's keys
    (scripts/problems/moe/reference.py:124-138).
    """
    t, d = x16.shape
    if logits16 is None:
        logits16 = router_logits(x16, weights["router.weight"], router_bias)
    idx, w, source_rows = route(logits16, top_k)
    pe, pr, first, rev = permute(idx, source_rows, n_experts)
    tok = pr % t
    krank = pr // t
    expanded_in = x16[tok]
    expanded_sm = w[tok, krank]
    f = weights["experts.0.0.weight"].shape[1]
    fc1 = np.zeros((t * top_k, f), dtype=np.float16)
    fc2 = np.zeros((t * top_k, d), dtype=np.float16)
    for e in range(n_experts):
        a, b = int(first[e]), int(first[e + 1])
        if b > a:
            fc1[a:b] = swiglu_fc1(expanded_in[a:b], weights[f"experts.{e}.0.weight"], weights[f"experts.{e}.1.weight"])
            fc2[a:b] = linear_fp16(fc1[a:b], weights[f"experts.{e}.2.weight"])
    sh1 = swiglu_fc1(x16, weights["shared_experts.0.weight"], weights["shared_experts.1.weight"])
    sh2 = linear_fp16(sh1, weights["shared_experts.2.weight"])
    # combine: out[t] = sum_i w[t,i] * Y[rev[i*T+t]] + S[t]  (moe_topk_kernel.cpp:240-250), fp32 sum
    acc = sh2.astype(F32).copy()
    rows = np.arange(t)
    routed = np.zeros((t, d), dtype=F32)
    for i in range(top_k):
        pos = rev[i * t + rows]
        routed += expanded_sm[pos].astype(F32)[:, None] * fc2[pos].astype(F32)
    out = (routed + acc).astype(np.float16)
    return {
        "expert_scores": logits16, "seq_experts_index": idx, "seq_experts_softmax": w, "source_rows": source_rows,
        "permuted_experts": pe, "permuted_rows": pr, "first_token_offset": first, "rev_permuted_rows": rev,
        "expanded_seq_input": expanded_in, "expanded_seq_softmax": expanded_sm, "expanded_fc1_output": fc1,
        "expanded_fc2_output": fc2, "shared_fc1_output": sh1, "shared_fc2_output": sh2, "final_output": out,
    }


def generate_input(d_hidden, d_expert, n_experts, n_shared, top_k, n_tokens, seed):
    """Same tensors, scales and draw order as scripts/problems/moe/reference.py:184-238, on the CPU.

    Returns (x fp16 [1, T, d], weights dict (fp16), config dict).
    """
    rng = np.random.default_rng(seed)

    def randn(*shape):
        return rng.standard_normal(shape, dtype=np.float32)

    x = randn(1, n_tokens, d_hidden).astype(np.float16)
    w = {"router.weight": (randn(n_experts, d_hidden) / np.sqrt(d_hidden)).astype(np.float16)}
    for e in range(n_experts):
        w[f"experts.{e}.0.weight"] = (randn(d_hidden, d_expert) / np.sqrt(d_expert)).astype(np.float16)
        w[f"experts.{e}.1.weight"] = (randn(d_hidden, d_expert) / np.sqrt(d_expert)).astype(np.float16)
        w[f"experts.{e}.2.weight"] = (randn(d_expert, d_hidden) / np.sqrt(d_hidden)).astype(np.float16)
    fs = d_expert * n_shared
    w["shared_experts.0.weight"] = (randn(d_hidden, fs) / np.sqrt(fs)).astype(np.float16)
    w["shared_experts.1.weight"] = (randn(d_hidden, fs) / np.sqrt(fs)).astype(np.float16)
    w["shared_experts.2.weight"] = (randn(fs, d_hidden) / np.sqrt(d_hidden)).astype(np.float16)
    cfg = {"d_hidden": d_hidden, "d_expert": d_expert, "n_routed_experts": n_experts, "n_shared_experts": n_shared,
           "n_experts_per_token": top_k, "batch_size": 1, "seq_len": n_tokens}
    return x, w, cfg


def zipf_router_bias(n_experts: int, s: float, seed: int) -> np.ndarray:
    """Per-expert logit bias -s*ln(1+rank_e) with a seeded random rank assignment (load skew)."""
    rank = np.random.default_rng(seed).permutation(n_experts)
    return (-s * np.log1p(rank.astype(np.float64))).astype(np.float32)


def check(received16, expected16, rtol=1e-2, atol=1e-2):
    """|r-e| <= atol + rtol*|e| with NaN/Inf agreement (scripts/utils.py:53-73). (ok, n_bad, max_err)."""
    r = np.asarray(received16).astype(np.float64)
    e = np.asarray(expected16).astype(np.float64)
    with np.errstate(invalid="ignore"):
        bad = np.abs(r - e) > atol + rtol * np.abs(e)
    bad |= np.isnan(r) ^ np.isnan(e)
    bad |= np.isinf(r) ^ np.isinf(e)
    with np.errstate(invalid="ignore"):
        mx = float(np.nanmax(np.abs(r - e))) if r.size else 0.0
    return (not bad.any()), int(bad.sum()), mx
