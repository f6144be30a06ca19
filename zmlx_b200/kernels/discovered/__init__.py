"""``zmlx.kernels.discovered`` -- the GLM-4.7-Flash shape specialisations the patched block tries first
(src/zmlx/patch/patterns/moe_mlp.py:712-716, 1011-1017).  Each returns ``None`` when the shape is not the one it
was specialised for, so that the caller falls back to the generic function -- the reference's contract.  Here they
are thin fronts of the generic kernels: a B200 kernel has no reason to be compiled per shape.
"""

from __future__ import annotations

from typing import Any

import torch

from .. import moe as _moe
from ..transformer import swiglu2 as _swiglu2
from ... import _lib

_COMBINE_D, _COMBINE_K = 2048, 4
_GATING_D, _GATING_K = 64, 4
_SWIGLU_D = 1536


def glm_moe_combine(expert_outputs: Any, weights: Any) -> Any | None:
    """Drop-in for ``moe.moe_combine`` when D=2048, K=4 (src/zmlx/kernels/discovered/glm_moe_combine.py:67-110).

    Same dtype: products and the running sum are rounded to that dtype, left to right (the kernel body,
    glm_moe_combine.py:28-42).  Different dtypes (bfloat16 experts, float32 weights): both are promoted, the
    arithmetic runs in float32 with the product rounded before the add, and the result is cast back to the
    expert dtype."""
    K, D = int(weights.shape[-1]), int(expert_outputs.shape[-1])
    if D != _COMBINE_D or K != _COMBINE_K:
        return None
    if expert_outputs.dtype == weights.dtype:
        return _moe.moe_combine_exact(expert_outputs, weights)
    out = _moe._combine(expert_outputs, weights.to(torch.float32), _lib.COMBINE_FP32_NO_FMA)
    return out.to(expert_outputs.dtype)


def glm_topk_gating(logits: Any, k: int = 4) -> tuple[Any, Any] | None:
    """Top-k of the logits, softmax over the k, for D=64, K=4
    (src/zmlx/kernels/discovered/glm_topk_gating.py:83-110).  Returns ``(indices, weights)`` -- indices first,
    weights in the logits' dtype -- or ``None`` for other shapes."""
    if int(logits.shape[-1]) != _GATING_D or int(k) != _GATING_K:
        return None
    w, idx = _moe.topk_gating_softmax(logits, int(k))
    return idx, w.to(logits.dtype)


def glm_fused_swiglu(gate: Any, up: Any) -> Any | None:
    """Drop-in for ``transformer.swiglu2`` when D=1536
    (src/zmlx/kernels/discovered/glm_fused_swiglu.py:65-90); ``None`` for other widths."""
    if int(gate.shape[-1]) != _SWIGLU_D:
        return None
    return _swiglu2(gate, up)


__all__ = ["glm_fused_swiglu", "glm_moe_combine", "glm_topk_gating"]
