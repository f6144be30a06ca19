"""NumPy restatement of the reference's MoE decode arithmetic (TEST ORACLE).

Conventions
-----------
* "T" is the expert dtype (bfloat16).  Tensors of dtype T are passed around as
  float32 arrays whose values are exactly representable in bfloat16; ``bf16()``
  rounds (nearest-even) to that set.
* Packed 4-bit tensors are ``uint32`` with 8 codes per word along the
  contraction axis: code ``i`` of a row sits in word ``i // 8`` at bit
  ``4 * (i % 8)`` (reference: src/zmlx/kernels/quant.py:109-120, 736-745).
* Canonical slot order of every router here: score descending, ties broken by
  ascending expert id (reference: src/zmlx/kernels/moe.py:42-43, 1769-1770).

Parity unpinned at the MLX boundary (see the package docstring).
"""

from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------
# bfloat16 emulation
# ---------------------------------------------------------------------------


def bf16(a):
    """Round float32 values to bfloat16 (nearest even); result stays float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    nan = np.isnan(a)
    r = (u + (((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF))) & np.uint32(0xFFFF0000)
    out = r.view(np.float32).copy()
    if nan.any():
        out[nan] = np.nan
    return out


def bf16_bits(a) -> np.ndarray:
    """bfloat16 bit patterns (uint16) of bf16-representable float32 values."""
    return (np.ascontiguousarray(bf16(a)).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


# ---------------------------------------------------------------------------
# Packed layouts and dequantisation
# ---------------------------------------------------------------------------

_E2M1 = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0,
     -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)


def unpack_u4(w: np.ndarray) -> np.ndarray:
    """(..., K/8) uint32 -> (..., K) uint8 codes.  quant.py:109-113."""
    w = np.asarray(w, dtype=np.uint32)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    q = (w[..., None] >> shifts) & np.uint32(0xF)
    return q.reshape(*w.shape[:-1], w.shape[-1] * 8).astype(np.uint8)


def pack_u4(q: np.ndarray) -> np.ndarray:
    """(..., K) codes in [0, 15] -> (..., K/8) uint32."""
    q = np.asarray(q).astype(np.uint32)
    assert q.shape[-1] % 8 == 0
    q = q.reshape(*q.shape[:-1], q.shape[-1] // 8, 8)
    shifts = (np.arange(8, dtype=np.uint32) * np.uint32(4))
    return (q << shifts).sum(axis=-1, dtype=np.uint32)


def dequant_affine(w, scales, biases, group_size: int = 64) -> np.ndarray:
    """w = q * scale[i // gs] + bias[i // gs] in float32.  quant.py:115-118, 738-745."""
    q = unpack_u4(w).astype(np.float32)
    s = np.repeat(np.asarray(scales, dtype=np.float32), group_size, axis=-1)
    b = np.repeat(np.asarray(biases, dtype=np.float32), group_size, axis=-1)
    return q * s + b


def dequant_mxfp4(w, scales_e8m0) -> np.ndarray:
    """mxfp4: e2m1 code times 2**(e8m0 - 127), one scale per 32 along K.

    The reference contains no mxfp4 arithmetic (its fused op rejects the mode,
    gather_qmm_swiglu.patch:714-718); this follows the OCP Microscaling
    format definition.  Parity unpinned.
    """
    v = _E2M1[unpack_u4(w)]
    e = np.asarray(scales_e8m0, dtype=np.uint8).astype(np.int32) - 127
    s = np.repeat(np.ldexp(np.float32(1.0), e).astype(np.float32), 32, axis=-1)
    return v * s


def dequant(w, scales, biases, *, mode: str = "affine", group_size: int = 64) -> np.ndarray:
    if mode == "affine":
        return dequant_affine(w, scales, biases, group_size)
    if mode == "mxfp4":
        return dequant_mxfp4(w, scales)
    raise ValueError(f"unknown quantisation mode {mode!r}")


# ---------------------------------------------------------------------------
# Quantised gather matmul family
# ---------------------------------------------------------------------------


def _broadcast_indices(x, w, lhs_indices, rhs_indices):
    """Index defaults and broadcasting of the gather ops.

    gather_qmm_swiglu.patch:754-758 (defaults + broadcast) and :778-781
    (output shape = indices.shape + (M, N)).
    """
    xb = x.shape[:-2]
    wb = w.shape[:-2]
    if lhs_indices is None:
        lhs_indices = np.arange(int(np.prod(xb, dtype=np.int64))).reshape(xb)
    if rhs_indices is None:
        rhs_indices = np.arange(int(np.prod(wb, dtype=np.int64))).reshape(wb)
    lhs, rhs = np.broadcast_arrays(np.asarray(lhs_indices), np.asarray(rhs_indices))
    return lhs.astype(np.int64), rhs.astype(np.int64)


def gather_qmm(x, w, scales, biases, *, lhs_indices=None, rhs_indices=None,
               group_size: int = 64, mode: str = "affine", out_bf16: bool = True,
               acc=np.float64) -> np.ndarray:
    """y[i] = x[lhs[i]] @ dequant(w[rhs[i]]).T  (transpose=True only).

    Call sites: src/zmlx/kernels/moe.py:1219-1229, 2147-2157;
    src/zmlx/patch/patterns/moe_mlp.py:571-574.  Result is materialised in T.
    """
    x = np.asarray(x, dtype=np.float32)
    lhs, rhs = _broadcast_indices(x, w, lhs_indices, rhs_indices)
    M, K = x.shape[-2:]
    N = w.shape[-2]
    xf = x.reshape(-1, M, K)
    wf = np.asarray(w).reshape(-1, N, w.shape[-1])
    sf = np.asarray(scales).reshape(-1, N, scales.shape[-1])
    bf_ = None if biases is None else np.asarray(biases).reshape(-1, N, biases.shape[-1])
    out = np.empty(lhs.shape + (M, N), dtype=np.float32)
    of = out.reshape(-1, M, N)
    cache: dict[int, np.ndarray] = {}
    for i, (l, r) in enumerate(zip(lhs.reshape(-1), rhs.reshape(-1))):
        r = int(r)
        if r not in cache:
            cache[r] = dequant(wf[r], sf[r], None if bf_ is None else bf_[r],
                               mode=mode, group_size=group_size).astype(acc)
        of[i] = (xf[int(l)].astype(acc) @ cache[r].T).astype(np.float32)
    return bf16(out) if out_bf16 else out


def sigmoid_plain(g):
    """1 / (1 + exp(-g)) in float32.  gather_qmm_swiglu.patch:47-55."""
    g = np.asarray(g, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32)


def sigmoid_stable(x):
    """y = 1/(1+exp(|x|)); x < 0 ? y : 1 - y.  src/zmlx/msl.py:20-24."""
    x = np.asarray(x, dtype=np.float32)
    with np.errstate(over="ignore"):
        y = (np.float32(1.0) / (np.float32(1.0) + np.exp(np.abs(x), dtype=np.float32))).astype(np.float32)
    return np.where(x < 0, y, np.float32(1.0) - y).astype(np.float32)


def swiglu_cpu_contract(g_t, u_t):
    """out = T(g * sigmoid(g) * u), g and u already rounded to T and widened.

    gather_qmm_swiglu.patch:47-55 (swiglu_cpu) after :142-163 materialised the
    two projections in T.
    """
    g = np.asarray(g_t, dtype=np.float32)
    u = np.asarray(u_t, dtype=np.float32)
    return bf16((g * sigmoid_plain(g)) * u)


def swiglu_per_op(g_t, u_t):
    """SwiGLU evaluated in T, one rounding per elementwise op.

    This is what unfused MLX ops on bf16 arrays do (silu(g) * u) and what the
    reference's elementwise kernel does in T (src/zmlx/kernels/transformer.py:882-897,
    a * kk_sigmoid(a) * b with kk_sigmoid in T, src/zmlx/msl.py:20-24).
    """
    g = np.asarray(g_t, dtype=np.float32)
    u = np.asarray(u_t, dtype=np.float32)
    with np.errstate(over="ignore"):
        e = bf16(np.exp(bf16(np.abs(g)), dtype=np.float32))
    y = bf16(np.float32(1.0) / bf16(np.float32(1.0) + e))
    sig = np.where(g < 0, y, bf16(np.float32(1.0) - y))
    return bf16(bf16(g * sig) * u)


def gather_qmm_swiglu(x, gate_w, gate_scales, gate_biases, up_w, up_scales, up_biases, *,
                      lhs_indices=None, rhs_indices=None, group_size: int = 64,
                      mode: str = "affine", swiglu: str = "cpu") -> np.ndarray:
    """silu(x @ Wg[e].T) * (x @ Wu[e].T) with the reference's CPU rounding contract.

    gather_qmm_swiglu.patch:64-192: two quantised matmuls written to T buffers,
    then swiglu_cpu over them.  Output shape: broadcast(lhs, rhs).shape + (M, N).
    """
    g = gather_qmm(x, gate_w, gate_scales, gate_biases, lhs_indices=lhs_indices,
                   rhs_indices=rhs_indices, group_size=group_size, mode=mode)
    u = gather_qmm(x, up_w, up_scales, up_biases, lhs_indices=lhs_indices,
                   rhs_indices=rhs_indices, group_size=group_size, mode=mode)
    if swiglu == "cpu":
        return swiglu_cpu_contract(g, u)
    if swiglu == "per_op":
        return swiglu_per_op(g, u)
    raise ValueError(swiglu)


def fused_quantized_swiglu_gemv(x, gate_w, gate_scales, gate_biases, up_w, up_scales, up_biases, *,
                                group_size: int = 64) -> np.ndarray:
    """Dense fused GEMV + SwiGLU: out[m, n] = T(silu(x_m . deq(Wg[n])) * (x_m . deq(Wu[n]))).

    src/zmlx/kernels/quant.py:103-124 (called from the dense MLP pattern, src/zmlx/patch/patterns/swiglu_mlp.py:
    281-317): both dot products are accumulated in float and stay in float through `acc_gate *
    kk_sigmoid(acc_gate) * acc_up` (sigmoid in the |x| form, src/zmlx/msl.py:20-24); one rounding at the store.
    x (M, K); weights (N, K/8) uint32; scales, biases (N, K/group_size).
    """
    wg = dequant_affine(np.asarray(gate_w)[None], np.asarray(gate_scales)[None], np.asarray(gate_biases)[None],
                        group_size)[0]
    wu = dequant_affine(np.asarray(up_w)[None], np.asarray(up_scales)[None], np.asarray(up_biases)[None],
                        group_size)[0]
    xf = np.asarray(x, dtype=np.float32)
    g = (xf.astype(np.float64) @ wg.astype(np.float64).T).astype(np.float32)
    u = (xf.astype(np.float64) @ wu.astype(np.float64).T).astype(np.float32)
    return bf16((g * sigmoid_stable(g)) * u)


# ---------------------------------------------------------------------------
# Routers
# ---------------------------------------------------------------------------


def _topk_desc_stable(scores: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest per row: score descending, then index ascending."""
    order = np.argsort(-scores.astype(np.float64), axis=-1, kind="stable")
    return order[..., :k]


def _softmax_f32(v: np.ndarray) -> np.ndarray:
    v = np.asarray(v, dtype=np.float32)
    m = v.max(axis=-1, keepdims=True)
    e = np.exp(v - m, dtype=np.float32)
    return (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)


def topk_gating_softmax(logits, k: int = 2, *, expert_bias=None, norm_topk_prob=None):
    """src/zmlx/kernels/moe.py:1239-1396 in float32; returns (weights, indices uint32).

    * norm and no bias: top-k of the logits, softmax over the k (:1287-1315, :1380-1386).
    * otherwise: full softmax [+ bias] -> top-k -> optional / (sum + 1e-20)
      (:1319-1323, :1388-1396).  On the bias path the returned weights include
      the bias (:249, :717).
    """
    x = np.asarray(logits, dtype=np.float32)
    K = int(k)
    if K <= 0:
        raise ValueError("topk_gating_softmax: k must be > 0")
    D = x.shape[-1]
    if K > D:
        raise ValueError(f"topk_gating_softmax: k={K} exceeds last dimension D={D}")
    norm = True if norm_topk_prob is None else bool(norm_topk_prob)
    if expert_bias is None and norm:
        idx = _topk_desc_stable(x, K)
        vals = np.take_along_axis(x, idx, axis=-1)
        return _softmax_f32(vals), idx.astype(np.uint32)
    gates = _softmax_f32(x)
    if expert_bias is not None:
        gates = (gates + np.asarray(expert_bias, dtype=np.float32).reshape(D)).astype(np.float32)
    idx = _topk_desc_stable(gates, K)
    scores = np.take_along_axis(gates, idx, axis=-1)
    if norm:
        scores = (scores / (scores.sum(axis=-1, keepdims=True, dtype=np.float32)
                            + np.float32(1e-20))).astype(np.float32)
    return scores, idx.astype(np.uint32)


def qwen3_gating(logits, k: int, *, norm_topk_prob: bool = True):
    """softmax(precise) -> top-k of the probabilities -> optional renormalise.

    src/zmlx/patch/patterns/moe_mlp.py:260-266.  Returns (indices, scores).
    argpartition order is unspecified in the reference; the canonical order is
    used here.
    """
    x = np.asarray(logits, dtype=np.float32)
    gates = _softmax_f32(x)
    idx = _topk_desc_stable(gates, int(k))
    scores = np.take_along_axis(gates, idx, axis=-1)
    if norm_topk_prob:
        scores = (scores / scores.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)
    return idx.astype(np.uint32), scores


def gpt_oss_gating(logits, k: int):
    """top-k of raw logits, softmax over the k.  moe_mlp.py:268-274."""
    x = np.asarray(logits, dtype=np.float32)
    idx = _topk_desc_stable(x, int(k))
    return idx.astype(np.uint32), _softmax_f32(np.take_along_axis(x, idx, axis=-1))


def deepseek_router_topk_sigmoid(logits, bias, *, k: int = 8, n_group: int = 1, topk_group: int = 1):
    """Sigmoid affinity + selection-only bias, group-limited selection, stable top-k.

    Fused-kernel semantics, src/zmlx/kernels/moe.py:1502-1679: score =
    sigmoid(l) + bias; group score = sum of the group's two largest scores
    (:1557-1569); keep ``topk_group`` groups, ties to the lower group (:1587);
    dropped groups get score 0.0, not -inf (:1617-1621); top-k with ties to the
    lower index; weights = sigmoid(l)[sel] / sum, no epsilon (:1653-1668).
    Validation as in :1690-1711.
    """
    x = np.asarray(logits, dtype=np.float32)
    K = int(k)
    if K <= 0:
        raise ValueError("deepseek_router_topk_sigmoid: k must be > 0")
    if x.ndim < 1:
        raise ValueError("deepseek_router_topk_sigmoid: logits must have rank >= 1")
    D = x.shape[-1]
    if K > D:
        raise ValueError(f"deepseek_router_topk_sigmoid: k={K} exceeds D={D}")
    b = np.asarray(bias, dtype=np.float32)
    if b.size != D:
        raise ValueError(f"deepseek_router_topk_sigmoid: bias must have shape ({D},)")
    b = b.reshape(D)
    G, TG = int(n_group), int(topk_group)
    if G <= 0:
        raise ValueError("deepseek_router_topk_sigmoid: n_group must be > 0")
    if TG <= 0 or TG > G:
        raise ValueError("deepseek_router_topk_sigmoid: invalid topk_group")
    if D % G != 0:
        raise ValueError("deepseek_router_topk_sigmoid: n_group must divide D")
    aff = sigmoid_stable(x)
    scores = (aff + b).astype(np.float32)
    if G > 1:
        per = D // G
        grouped = scores.reshape(*scores.shape[:-1], G, per)
        top2 = -np.sort(-grouped, axis=-1)[..., :2]
        gscore = (top2[..., 0] + top2[..., 1]).astype(np.float32) if per >= 2 else \
            (top2[..., 0] + np.float32(-np.inf))
        keep_idx = _topk_desc_stable(gscore, TG)
        keep = np.zeros(gscore.shape, dtype=bool)
        np.put_along_axis(keep, keep_idx, True, axis=-1)
        scores = np.where(keep[..., None], grouped, np.float32(0.0)).reshape(scores.shape)
    idx = _topk_desc_stable(scores, K)
    w = np.take_along_axis(aff, idx, axis=-1)
    w = (w * (np.float32(1.0) / w.sum(axis=-1, keepdims=True, dtype=np.float32))).astype(np.float32)
    return w, idx.astype(np.uint32)


# ---------------------------------------------------------------------------
# Combine contracts: out[t, d] = sum_i w[t, i] * y[t, i, d], slots in order 0..K-1
# ---------------------------------------------------------------------------


def moe_combine(y, w, *, mode: str):
    """The reference's combine kernels, src/zmlx/kernels/moe.py:831-1127, 1821-1921.

    mode:
      "fp32"         float32 accumulate, float32 out (:1020-1026); the GPU may
                     contract w*v+acc, so callers compare with a tolerance.
      "fp32_no_fma"  product rounded to float32, then added (:1075-1095); float32 out.
      "t"            as "fp32" but cast to T at the end (:840-846).
      "no_fma"       as "fp32_no_fma" but cast to T at the end (:899-912); equals
                     MLX's (y * w[..., None]).sum(-2).astype(T) (tests/test_fused_ops.py:349-362).
      "exact"        weights in T, product rounded to T, running sum rounded to T (:963-970);
                     same contract as kernels/discovered/glm_moe_combine.py:21-42.
      "stream_t"     streaming accumulate: acc = T(float(acc) + w*v) per slot (:1821-1860).
    """
    y = np.asarray(y, dtype=np.float32)
    w = np.asarray(w, dtype=np.float32)
    K = w.shape[-1]
    acc = np.zeros(y.shape[:-2] + y.shape[-1:], dtype=np.float32)
    if mode in ("fp32", "fp32_no_fma", "t", "no_fma"):
        for i in range(K):
            prod = (w[..., i, None] * y[..., i, :]).astype(np.float32)
            acc = (acc + prod).astype(np.float32)
        return bf16(acc) if mode in ("t", "no_fma") else acc
    if mode == "exact":
        wt = bf16(w)
        for i in range(K):
            prod = bf16(wt[..., i, None] * y[..., i, :])
            acc = bf16(acc + prod)
        return acc
    if mode == "stream_t":
        for i in range(K):
            prod = (w[..., i, None] * y[..., i, :]).astype(np.float32)
            acc = bf16(acc + prod)
        return acc
    raise ValueError(f"unknown combine mode {mode!r}")


def gather_qmm_combine_quantized(act, w, scales, biases, gate, indices, *, group_size: int = 64,
                                 mode: str = "affine", combine: str = "t"):
    """out[t] = sum_k gate[t,k] * T(act[t,k] @ dequant(w[idx[t,k]]).T).

    src/zmlx/kernels/moe.py:2043-2174 (and :1198-1236 for the single-gather
    form): every projection is materialised in T before the combine.
    """
    act = np.asarray(act, dtype=np.float32)
    if act.ndim != 3:
        raise ValueError("gather_qmm_combine_quantized: act must have shape (B, K, D_in)")
    B, K, D_in = act.shape
    lhs = np.arange(B * K).reshape(B, K)
    proj = gather_qmm(act.reshape(B * K, 1, D_in), w, scales, biases, lhs_indices=lhs,
                      rhs_indices=np.asarray(indices), group_size=group_size, mode=mode)
    return moe_combine(proj[..., 0, :], gate, mode=combine)


# ---------------------------------------------------------------------------
# Dense (shared-expert) MLP and whole-layer recipes
# ---------------------------------------------------------------------------


def shared_expert_mlp(x, p, *, group_size: int, mode: str):
    """down(silu(gate(x)) * up(x)) with every op materialised in T.

    The reference adds ``shared_experts(x)`` unchanged (moe_mlp.py:1059-1061);
    the module itself is mlx_lm's quantised dense MLP, i.e. three quantised
    matmuls and an elementwise SwiGLU on T arrays.
    """
    x = np.asarray(x, dtype=np.float32)
    x3 = x.reshape(1, -1, x.shape[-1])
    z = np.zeros((1,), dtype=np.int64)
    g = gather_qmm(x3, p["gate_w"][None], p["gate_s"][None], None if p.get("gate_b") is None else p["gate_b"][None],
                   lhs_indices=z, rhs_indices=z, group_size=group_size, mode=mode)[0]
    u = gather_qmm(x3, p["up_w"][None], p["up_s"][None], None if p.get("up_b") is None else p["up_b"][None],
                   lhs_indices=z, rhs_indices=z, group_size=group_size, mode=mode)[0]
    h = swiglu_per_op(g, u)
    y = gather_qmm(h[None], p["down_w"][None], p["down_s"][None],
                   None if p.get("down_b") is None else p["down_b"][None],
                   lhs_indices=z, rhs_indices=z, group_size=group_size, mode=mode)[0]
    return y.reshape(x.shape[:-1] + (y.shape[-1],))


def moe_layer(x, logits, p, *, family: str, top_k: int, group_size: int = 64, mode: str = "affine",
              expert_bias=None, n_group: int = 1, topk_group: int = 1,
              routed_scaling_factor: float = 1.0, norm_topk_prob: bool = True,
              combine: str | None = None, swiglu: str | None = None, shared=None):
    """One MoE block forward, in the order of moe_mlp.py:883-1063.

    ``x`` is (T, d) in T; ``logits`` is (T, E), the router linear's output
    (already rounded to the gate's dtype).  ``family`` selects the branch:

      "generic"  raw-logits branch (moe_mlp.py:276-289): topk_gating_softmax in
                 float32, weights cast to T, moe_combine (float32 accumulate, cast T).
      "qwen3"    moe_mlp.py:226-266 gating; native (y * w[..., None]).sum(-2)
                 combine with float32 weights == "no_fma" contract.
      "glm"      gate returns (indices, scores): deepseek_router_topk_sigmoid *
                 routed_scaling_factor (deepseek_router.py:108-120); combine
                 fp32_no_fma then cast to T (moe_mlp.py:995-1002).
      "deepseek" same gate; generic combine (moe_mlp.py:1055-1057).

    Returns (out (T, d) in T, indices (T, K) uint32, weights (T, K) float32).
    """
    x = np.asarray(x, dtype=np.float32)
    if family == "generic":
        w, idx = topk_gating_softmax(logits, top_k, expert_bias=expert_bias, norm_topk_prob=norm_topk_prob)
        w = bf16(w)
        cmode = combine or "t"
    elif family == "qwen3":
        idx, w = qwen3_gating(logits, top_k, norm_topk_prob=norm_topk_prob)
        cmode = combine or "no_fma"
    elif family in ("glm", "deepseek"):
        w, idx = deepseek_router_topk_sigmoid(logits, expert_bias, k=top_k, n_group=n_group,
                                              topk_group=topk_group)
        if routed_scaling_factor != 1.0:
            w = (w * np.float32(routed_scaling_factor)).astype(np.float32)
        cmode = combine or ("fp32_no_fma" if family == "glm" else "t")
    else:
        raise ValueError(family)
    T_, d = x.shape
    x5 = x.reshape(T_, 1, 1, d)
    sw = swiglu or ("cpu" if mode == "affine" else "per_op")
    h = gather_qmm_swiglu(x5, p["gate_w"], p["gate_s"], p.get("gate_b"), p["up_w"], p["up_s"], p.get("up_b"),
                          rhs_indices=idx.astype(np.int64), group_size=group_size, mode=mode, swiglu=sw)
    # h: (T, K, 1, f); down projection (moe_mlp.py:571-574) then squeeze(-2).
    K = idx.shape[-1]
    lhs = np.arange(T_ * K).reshape(T_, K)
    y = gather_qmm(h.reshape(T_ * K, 1, -1), p["down_w"], p["down_s"], p.get("down_b"), lhs_indices=lhs,
                   rhs_indices=idx.astype(np.int64), group_size=group_size, mode=mode)[..., 0, :]
    out = moe_combine(y, w, mode=cmode)
    if cmode in ("fp32", "fp32_no_fma"):
        out = bf16(out)  # .astype(expert dtype), moe_mlp.py:1002
    if shared is not None:
        out = bf16(out + shared_expert_mlp(x, shared, group_size=group_size, mode=mode))
    return out, idx, w
