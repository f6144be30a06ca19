"""Dense SwiGLU MLP pattern: quantised gate/up projection + SwiGLU in one kernel, then the quantised down projection.

Mirrors src/zmlx/patch/patterns/swiglu_mlp.py:217-330 (`_SwiGLUMLPPattern`): structural match on
``gate_proj/up_proj/down_proj`` (or ``w1/w3/w2``), the same exclusions (switch / dispatch modules; children of a MoE
block other than ``shared_experts``), the same fall-back to the module's own call when the projections are not 4-bit
affine.  Where the reference calls `fused_quantized_swiglu_gemv` (src/zmlx/kernels/quant.py:146-192, one thread per
output element, decode only: `ZMLX_FUSED_QSWIGLU_MAX_TOKENS` defaults to 1) this calls the grouped matmul of the MoE
path with a bank of one expert, which has no token limit; the down projection goes through the same library instead
of the stock module.  A dense MLP is the MoE block's expert arithmetic with E = 1 and no router.
"""

from __future__ import annotations

import os
from typing import Any

import torch
import torch.nn as nn

from ... import _lib, ops
from .._registry import register
from .._types import PatchConfig

_QSWIGLU_MODE_ENV = "ZMLX_FUSED_QSWIGLU_MODE"  # "off" keeps the module's own call (swiglu_mlp.py:150-159)


def _get_swiglu_projections(module: Any):
    if all(hasattr(module, a) for a in ("gate_proj", "up_proj", "down_proj")):
        return module.gate_proj, module.up_proj, module.down_proj
    if all(hasattr(module, a) for a in ("w1", "w3", "w2")):
        return module.w1, module.w3, module.w2
    return None


def _is_silu_activation(module: Any) -> bool:
    if hasattr(module, "hidden_act"):
        return module.hidden_act in ("silu", "swish")
    return True  # the default assumption for a gate + up layout (swiglu_mlp.py:22-36)


def _bank(proj: Any):
    """(weight (1, N, K/8), scales, biases) of a quantised projection the kernels take, or None."""
    w, s, b = getattr(proj, "weight", None), getattr(proj, "scales", None), getattr(proj, "biases", None)
    if w is None or s is None or b is None:
        return None
    if getattr(proj, "mode", "affine") != "affine" or int(getattr(proj, "bits", 4)) != 4 \
            or int(getattr(proj, "group_size", 64)) != 64:
        return None
    if w.dtype not in (torch.uint32, torch.int32) or not w.is_cuda:
        return None
    if w.ndim == 2:
        w, s, b = w[None], s[None], b[None]
    if w.ndim != 3 or w.shape[0] != 1 or not (w.is_contiguous() and s.is_contiguous() and b.is_contiguous()):
        return None
    return w, s, b


class _SwiGLUMLPPattern:
    @property
    def name(self) -> str:
        return "swiglu_mlp"

    def matches(self, module: Any, name: str, parent: Any | None = None) -> bool:
        if not isinstance(module, nn.Module):
            return False
        if "switch" in name.lower() or "dispatch" in name.lower():
            return False
        if parent is not None and (hasattr(parent, "router") or hasattr(parent, "gate")):
            if name.lower() != "shared_experts":
                return False
        return _get_swiglu_projections(module) is not None and _is_silu_activation(module)

    def apply(self, module: Any, config: PatchConfig) -> Any:
        original_call = module.__call__
        plans: dict = {}

        def patched_call(self_mod: Any, x: Any, *args: Any, **kw: Any) -> Any:
            projections = _get_swiglu_projections(self_mod)
            if (projections is None or args or kw or os.environ.get(_QSWIGLU_MODE_ENV, "").lower() == "off"
                    or not isinstance(x, torch.Tensor) or x.dtype != torch.bfloat16 or not x.is_cuda):
                return original_call(x, *args, **kw)
            banks = [_bank(p) for p in projections]
            if any(b is None for b in banks):
                return original_call(x, *args, **kw)
            (gw, gs, gb), (uw, us, ub), (dw, ds, db) = banks
            K = gw.shape[2] * 8
            if x.shape[-1] != K or gw.shape != uw.shape or dw.shape[2] * 8 != gw.shape[1]:
                return original_call(x, *args, **kw)
            x2 = x.reshape(-1, K)
            if x2.stride(1) != 1 or x2.stride(0) % 8 != 0 or x2.data_ptr() % 16 != 0:
                x2 = x2.contiguous()
            T = x2.shape[0]
            if T == 0:
                return original_call(x, *args, **kw)
            key = (T, x.device)
            plan = plans.get(key)
            if plan is None:  # every row belongs to the bank's only expert
                plan = ops.build_plan(torch.zeros(T, dtype=torch.int32, device=x.device), 1)
                if not torch.cuda.is_current_stream_capturing():
                    plans[key] = plan
            h = ops.gather_qmm_swiglu_rows(x2, gw, gs, gb, uw, us, ub, plan, T, rows_hint=T, swiglu=_lib.SWIGLU_FP32)
            y = ops.gather_qmm_rows(h, dw, ds, db, plan, T, rows_hint=T, x_by_output_row=True)
            return y.reshape(*x.shape[:-1], y.shape[-1])

        module._zmlx_original_call = original_call
        module._zmlx_original_class = module.__class__
        module.__class__ = type(module.__class__.__name__, (module.__class__,), {"__call__": patched_call})
        return module


register(_SwiGLUMLPPattern())
