"""MoE routing and combine ops (the reference's ``zmlx.kernels.moe`` surface).

Names, argument meaning, defaults and error behaviour follow
src/zmlx/kernels/moe.py (``__all__`` at :2177-2192); tensors are torch CUDA
tensors and the arithmetic runs in hand-written sm_100a kernels.  Slot order of
every router here is canonical: score descending, ties to the lower expert id
(the reference's own order for the sigmoid router, moe.py:1769-1770; for the
softmax family the reference leaves ``argpartition`` order unspecified).
"""

from __future__ import annotations

from typing import Any

import torch

from .. import _lib, ops

_MAX_FUSED_TOPK = 8  # kept for parity with moe.py:12; this build fuses up to k = 16
_DEEPSEEK_ROUTER_K = 8


def _cd(compute_dtype) -> torch.dtype:
    return torch.float32 if compute_dtype is None else compute_dtype


def _cast(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    return t if t.dtype == dtype else t.to(dtype)


def _logits_in(x: torch.Tensor, cd: torch.dtype) -> torch.Tensor:
    """Logits as the kernel reads them: bf16 stays bf16 (widened on load), else float32."""
    if x.dtype == torch.bfloat16 or x.dtype == torch.float32:
        return x
    return x.to(torch.float32)


# ---------------------------------------------------------------------------
# Softmax-family routers
# ---------------------------------------------------------------------------


def top2_gating_softmax(x: Any, *, threadgroup: int = 256, compute_dtype: Any | None = None) -> tuple[Any, Any]:
    """Top-2 of the logits and a 2-way softmax (moe.py:398-431)."""
    return topk_gating_softmax(x, 2, threadgroup=threadgroup, compute_dtype=compute_dtype)


def topk_gating_softmax(
    x: Any,
    k: int = 2,
    *,
    threadgroup: int = 256,
    compute_dtype: Any | None = None,
    expert_bias: Any | None = None,
    norm_topk_prob: bool | None = None,
) -> tuple[Any, Any]:
    """Top-k gating with softmax (moe.py:1239-1396).

    Without a bias and with ``norm_topk_prob`` unset or True: top-k of the
    logits, then softmax over the k.  Otherwise: full softmax [+ bias] -> top-k
    -> optional ``/ (sum + 1e-20)``; on the bias path the returned weights
    include the bias, as in the reference.

    Returns ``(weights (..., k) in compute_dtype, indices (..., k) uint32)``.
    ``threadgroup`` is accepted for signature parity and ignored.
    """
    cd = _cd(compute_dtype)
    K = int(k)
    if K <= 0:
        raise ValueError("topk_gating_softmax: k must be > 0")
    D = int(x.shape[-1])
    if K > D:
        raise ValueError(f"topk_gating_softmax: k={K} exceeds last dimension D={D}")
    norm = True if norm_topk_prob is None else bool(norm_topk_prob)
    bias = expert_bias
    if bias is not None:
        if bias.ndim > 2 or int(bias.shape[-1]) != D or bias.numel() != D:
            raise ValueError(f"topk_gating_softmax: expert_bias must have {D} elements")
        bias = bias.reshape(D)
    xin = _logits_in(x, cd)
    if bias is None and norm:
        w, idx = ops.router_softmax_topk(xin, K, flavour=_lib.ROUTER_TOPK_THEN_SOFTMAX)
    else:
        w, idx = ops.router_softmax_topk(xin, K, flavour=_lib.ROUTER_SOFTMAX_THEN_TOPK, bias=bias,
                                         renorm=1 if norm else 0)
    return _cast(w, cd), idx


def router_argpartition_logits_topk(logits: Any, *, k: int, compute_dtype: Any | None = None) -> tuple[Any, Any]:
    """Top-k of the logits + softmax over the selected logits (moe.py:1448-1490).

    Returns ``(scores, indices)`` like the reference (note the order).
    """
    if logits.ndim < 1:
        raise ValueError("router_argpartition_logits_topk: logits must have rank >= 1")
    cd = _cd(compute_dtype)
    D = int(logits.shape[-1])
    K = int(k)
    if K <= 0:
        raise ValueError("router_argpartition_logits_topk: k must be > 0")
    if K > D:
        raise ValueError(f"router_argpartition_logits_topk: k={K} exceeds D={D}")
    w, idx = ops.router_softmax_topk(_logits_in(logits, cd), K, flavour=_lib.ROUTER_TOPK_THEN_SOFTMAX)
    return _cast(w, cd), idx


def qwen3_gating(logits: Any, k: int, *, norm_topk_prob: bool = True) -> tuple[Any, Any]:
    """softmax -> top-k of the probabilities -> optional ``/ sum``; returns (indices, scores).

    The Qwen3 branch of the patched block, src/zmlx/patch/patterns/moe_mlp.py:260-266.
    """
    w, idx = ops.router_softmax_topk(_logits_in(logits, torch.float32), int(k),
                                     flavour=_lib.ROUTER_SOFTMAX_THEN_TOPK, renorm=2 if norm_topk_prob else 0)
    return idx, w


# ---------------------------------------------------------------------------
# DeepSeek / Kimi / GLM router: sigmoid affinity + selection-only bias
# ---------------------------------------------------------------------------


def deepseek_router_topk_sigmoid(
    logits: Any,
    bias: Any,
    *,
    k: int = _DEEPSEEK_ROUTER_K,
    n_group: int = 1,
    topk_group: int = 1,
    threadgroup: int = 256,
    compute_dtype: Any | None = None,
    routed_scaling_factor: float = 1.0,
) -> tuple[Any, Any]:
    """DeepSeek router top-k (moe.py:1745-1817).

    Selection scores are ``sigmoid(logits) + bias``; the returned weights are the
    normalised sigmoid values of the selected experts.  Group-limited selection
    follows the reference's fused kernel (moe.py:1552-1621).  Any expert count up
    to 1024 and any k up to 16 take the kernel; the reference fuses only
    256/384 experts with k = 8 and otherwise runs the same arithmetic in MLX ops.
    ``routed_scaling_factor`` (an extension, default 1) folds in the multiply of
    src/zmlx/patch/patterns/deepseek_router.py:118-119.
    """
    cd = _cd(compute_dtype)
    K = int(k)
    if K <= 0:
        raise ValueError("deepseek_router_topk_sigmoid: k must be > 0")
    if logits.ndim < 1:
        raise ValueError("deepseek_router_topk_sigmoid: logits must have rank >= 1")
    D = int(logits.shape[-1])
    if K > D:
        raise ValueError(f"deepseek_router_topk_sigmoid: k={K} exceeds D={D}")
    if bias.ndim != 1:
        if bias.numel() == D:
            bias = bias.reshape(D)
        else:
            raise ValueError(f"deepseek_router_topk_sigmoid: bias must have shape ({D},)")
    if int(bias.shape[0]) != D:
        raise ValueError(f"deepseek_router_topk_sigmoid: bias must have shape ({D},)")
    G, TG = int(n_group), int(topk_group)
    if G <= 0:
        raise ValueError("deepseek_router_topk_sigmoid: n_group must be > 0")
    if TG <= 0 or TG > G:
        raise ValueError("deepseek_router_topk_sigmoid: invalid topk_group")
    if D % G != 0:
        raise ValueError("deepseek_router_topk_sigmoid: n_group must divide D")
    w, idx = ops.router_sigmoid_topk(_logits_in(logits, cd), bias, K, n_group=G, topk_group=TG,
                                     scale=float(routed_scaling_factor))
    return _cast(w, cd), idx


# ---------------------------------------------------------------------------
# Dispatch and combine
# ---------------------------------------------------------------------------


def moe_dispatch(x: Any, indices: Any) -> Any:
    """(..., D) -> (..., K, D): one copy of the token per selected expert (moe.py:803-827)."""
    K = int(indices.shape[-1])
    return x.unsqueeze(-2).expand(*x.shape[:-1], K, x.shape[-1]).contiguous()


def _combine(expert_outputs: torch.Tensor, weights: torch.Tensor, mode: int) -> torch.Tensor:
    lead = tuple(weights.shape[:-1])
    K = int(weights.shape[-1])
    D = int(expert_outputs.shape[-1])
    if expert_outputs.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"moe_combine: expert outputs must be bfloat16 or float32, got {expert_outputs.dtype}")
    y = expert_outputs.reshape(-1, K, D)
    w = weights.reshape(-1, K)
    if w.dtype not in (torch.bfloat16, torch.float32):
        w = w.to(torch.float32)
    out = ops.combine(y, w, mode)
    return out.reshape(lead + (D,))


def moe_combine(expert_outputs: Any, weights: Any) -> Any:
    """float32 accumulate over the K slots, result in the expert dtype (moe.py:859-882)."""
    out = _combine(expert_outputs, weights, _lib.COMBINE_T if expert_outputs.dtype == torch.bfloat16
                   else _lib.COMBINE_FP32)
    return out


def moe_combine_no_fma(expert_outputs: Any, weights: Any) -> Any:
    """Product rounded to float32 before the add; equals ``(y * w[..., None]).sum(-2).astype(T)`` (moe.py:915-939)."""
    return _combine(expert_outputs, weights, _lib.COMBINE_NO_FMA if expert_outputs.dtype == torch.bfloat16
                    else _lib.COMBINE_FP32_NO_FMA)


def moe_combine_exact(expert_outputs: Any, weights: Any) -> Any:
    """Product and running sum rounded to the expert dtype (moe.py:973-992)."""
    if expert_outputs.dtype == torch.float32:
        return _combine(expert_outputs, weights, _lib.COMBINE_FP32_NO_FMA)
    return _combine(expert_outputs, weights, _lib.COMBINE_EXACT)


def moe_combine_fp32(expert_outputs: Any, weights: Any) -> Any:
    """float32 weights, float32 accumulate and output (moe.py:1029-1060)."""
    return _combine(expert_outputs, _cast(weights, torch.float32), _lib.COMBINE_FP32)


def moe_combine_fp32_no_fma(expert_outputs: Any, weights: Any) -> Any:
    """Like :func:`moe_combine_fp32` with FMA contraction disabled (moe.py:1098-1127)."""
    return _combine(expert_outputs, _cast(weights, torch.float32), _lib.COMBINE_FP32_NO_FMA)


def _combine_projected_experts(projected: Any, gate: Any, *, no_fma: bool, output_dtype: Any | None) -> Any:
    """moe.py:1130-1152."""
    out_dtype = projected.dtype if output_dtype is None else output_dtype
    if out_dtype == torch.float32:
        gate_fp32 = _cast(gate, torch.float32)
        return moe_combine_fp32_no_fma(projected, gate_fp32) if no_fma else moe_combine_fp32(projected, gate_fp32)
    gate_cast = _cast(gate, projected.dtype)
    out = moe_combine_no_fma(projected, gate_cast) if no_fma else moe_combine(projected, gate_cast)
    return _cast(out, out_dtype)


# ---------------------------------------------------------------------------
# Down projection + combine
# ---------------------------------------------------------------------------


def _should_use_streaming(batch_size: int, streaming: bool | None) -> bool:
    """moe.py:1924-1932."""
    if streaming is not None:
        return streaming
    return batch_size <= 16


def gather_mmk_combine(act: Any, weights: Any, gate: Any, indices: Any, *, no_fma: bool = False,
                       output_dtype: Any | None = None) -> Any:
    """Dense-weight gather-matmul-combine (moe.py:1155-1195).

    Dense expert weights are not on the quantised hot path; the projection is a
    plain batched library GEMM, the combine is the kernel above.
    """
    if act.ndim != 3:
        raise ValueError("gather_mmk_combine: act must have shape (B, K, D_in)")
    if weights.ndim != 3:
        raise ValueError("gather_mmk_combine: weights must have shape (E, D_in, D_out)")
    B, K, D_in = act.shape
    if weights.shape[1] != D_in:
        raise ValueError("gather_mmk_combine: weights second dimension must match act last dimension")
    idx = indices.reshape(-1).to(torch.int64)
    proj = torch.bmm(act.reshape(B * K, 1, D_in), weights[idx]).reshape(B, K, -1)
    return _combine_projected_experts(proj, gate, no_fma=no_fma, output_dtype=output_dtype)


def gather_qmm_combine(act: Any, weights: Any, gate: Any, indices: Any, *, streaming: bool | None = None,
                       no_fma: bool = False, output_dtype: Any | None = None, vectorized_k: bool = False) -> Any:
    """Dense-weight down-projection + combine (moe.py:1935-2040).

    ``streaming`` selects the reference's per-slot accumulate contract (the running
    sum is rounded to the output dtype after every slot, moe.py:1821-1841) for
    B <= 16 unless overridden; otherwise all projections are combined at once.
    """
    if act.ndim != 3:
        raise ValueError("gather_qmm_combine: act must have shape (B, K, D_in)")
    B, K, D_in = act.shape
    if weights.ndim != 3:
        raise ValueError("gather_qmm_combine: weights must have shape (E, D_in, D_out)")
    out_dtype = act.dtype if output_dtype is None else output_dtype
    if vectorized_k:
        return gather_mmk_combine(act, weights, gate, indices, no_fma=no_fma, output_dtype=out_dtype)
    idx = indices.reshape(-1).to(torch.int64)
    proj = torch.bmm(act.reshape(B * K, 1, D_in), weights[idx]).reshape(B, K, -1)
    return _finish_combine(proj, gate, B, streaming, no_fma, out_dtype)


def _finish_combine(proj: torch.Tensor, gate: torch.Tensor, B: int, streaming: bool | None, no_fma: bool,
                    out_dtype: torch.dtype) -> torch.Tensor:
    if _should_use_streaming(B, streaming):
        if out_dtype == torch.float32:
            g32 = _cast(gate, torch.float32)
            return moe_combine_fp32_no_fma(proj, g32) if no_fma else moe_combine_fp32(proj, g32)
        out = _combine(proj, gate, _lib.COMBINE_STREAM_T)
        return _cast(out, out_dtype)
    # non-streaming: sum(proj * gate[..., None]) in the promoted dtype (moe.py:2120-2125)
    if gate.dtype == torch.float32 or proj.dtype == torch.float32:
        out = _combine(proj, _cast(gate, torch.float32), _lib.COMBINE_FP32_NO_FMA)
    else:
        out = _combine(proj, gate, _lib.COMBINE_EXACT)
    return _cast(out, out_dtype)


def gather_qmmk_combine_quantized(act: Any, weights: Any, scales: Any, biases: Any, gate: Any, indices: Any, *,
                                  group_size: int = 64, bits: int = 4, no_fma: bool = False,
                                  output_dtype: Any | None = None, mode: str = "affine") -> Any:
    """One gather over all K slots, then a combine kernel (moe.py:1198-1236)."""
    if act.ndim != 3:
        raise ValueError("gather_qmmk_combine_quantized: act must have shape (B, K, D_in)")
    proj = _project_quantized(act, weights, scales, biases, indices, group_size, bits, mode)
    return _combine_projected_experts(proj, gate, no_fma=no_fma, output_dtype=output_dtype)


def _project_quantized(act, weights, scales, biases, indices, group_size, bits, mode) -> torch.Tensor:
    if bits != 4:
        raise ValueError(f"gather_qmm_combine_quantized: bits={bits} is not supported by this build (4 only)")
    B, K, D_in = act.shape
    if weights.ndim != 3:
        raise ValueError("gather_qmm_combine_quantized: weights must have shape (E, D_out, D_in/8)")
    E, D_out = int(weights.shape[0]), int(weights.shape[1])
    if act.dtype != torch.bfloat16:
        raise TypeError(f"gather_qmm_combine_quantized: activations must be bfloat16, got {act.dtype}")
    if B * K == 0:
        return torch.empty((B, K, D_out), dtype=torch.bfloat16, device=act.device)
    a2 = act.reshape(B * K, D_in)
    if a2.stride(-1) != 1 or a2.stride(0) % 8 != 0 or a2.data_ptr() % 16 != 0:
        a2 = a2.contiguous()
    plan = ops.build_plan(indices.reshape(-1), E)
    proj = ops.gather_qmm_rows(a2, weights.contiguous(), scales.contiguous(),
                               None if biases is None else biases.contiguous(), plan, B * K, rows_hint=B,
                               group_size=32 if mode == "mxfp4" else group_size, mode=mode)
    return proj.reshape(B, K, D_out)


def gather_qmm_combine_quantized(act: Any, weights: Any, scales: Any, biases: Any, gate: Any, indices: Any, *,
                                 group_size: int = 64, bits: int = 4, streaming: bool | None = None,
                                 no_fma: bool = False, output_dtype: Any | None = None, vectorized_k: bool = False,
                                 mode: str = "affine") -> Any:
    """Quantised down-projection + combine: ``sum_k gate[:, k] * (act[:, k] @ W[idx[:, k]].T)``.

    Reference: moe.py:2043-2174.  Each projection is materialised in the activation
    dtype, as ``mx.gather_qmm`` does, then combined in slot order under the contract
    the reference's flags select (``streaming``, ``no_fma``, ``output_dtype``).
    One kernel launch projects all B*K rows with every expert's weights streamed
    once; the reference loops over K from Python.
    """
    if act.ndim != 3:
        raise ValueError("gather_qmm_combine_quantized: act must have shape (B, K, D_in)")
    B = int(act.shape[0])
    out_dtype = act.dtype if output_dtype is None else output_dtype
    proj = _project_quantized(act, weights, scales, biases, indices, group_size, bits, mode)
    if vectorized_k:
        return _combine_projected_experts(proj, gate, no_fma=no_fma, output_dtype=out_dtype)
    return _finish_combine(proj, gate, B, streaming, no_fma, out_dtype)


__all__ = [
    "top2_gating_softmax",
    "topk_gating_softmax",
    "router_argpartition_logits_topk",
    "deepseek_router_topk_sigmoid",
    "moe_dispatch",
    "moe_combine",
    "moe_combine_no_fma",
    "moe_combine_exact",
    "moe_combine_fp32",
    "moe_combine_fp32_no_fma",
    "gather_mmk_combine",
    "gather_qmmk_combine_quantized",
    "gather_qmm_combine",
    "gather_qmm_combine_quantized",
]
