"""DeepSeek / Kimi router pattern: ``x @ W.T`` -> fused sigmoid top-k -> ``* routed_scaling_factor``.

Mirrors src/zmlx/patch/patterns/deepseek_router.py:29-131.  Opt-in, like the reference's.  The kernel takes any
expert count up to 1024 and any k up to 16; the reference fuses 256/384 experts with k = 8 only and keeps that
restriction here so that the set of modules it rewrites is the same.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.nn as nn

from ...kernels.moe import deepseek_router_topk_sigmoid
from .._registry import register
from .._types import PatchConfig

_SUPPORTED_NR = {256, 384}
_SUPPORTED_K = 8


def _is_deepseek_gate_module(module: Any) -> bool:
    cls = module.__class__
    if (getattr(cls, "__name__", "") or "") != "MoEGate":
        return False
    mod_path = (getattr(cls, "__module__", "") or "").lower()
    return any(s in mod_path for s in ("deepseek_v3", "deepseek_v32", "kimi_k25", "zmlx_b200.nn"))


class _DeepSeekRouterPattern:
    @property
    def name(self) -> str:
        return "deepseek_router"

    def matches(self, module: Any, name: str, parent: Any | None = None) -> bool:
        if not isinstance(module, nn.Module) or not _is_deepseek_gate_module(module):
            return False
        return all(hasattr(module, a) for a in ("weight", "e_score_correction_bias", "top_k", "norm_topk_prob",
                                                 "n_group", "topk_group", "routed_scaling_factor"))

    def apply(self, module: Any, config: PatchConfig) -> Any:
        original_call = module.__call__

        def patched_call(self_mod: Any, x: Any) -> Any:
            try:
                top_k, n_group, topk_group = int(self_mod.top_k), int(self_mod.n_group), int(self_mod.topk_group)
                norm_topk_prob = bool(self_mod.norm_topk_prob)
                scaling = float(self_mod.routed_scaling_factor)
            except Exception:
                return original_call(x)
            weight, bias = getattr(self_mod, "weight", None), getattr(self_mod, "e_score_correction_bias", None)
            if (top_k != _SUPPORTED_K or not norm_topk_prob or n_group <= 0 or topk_group <= 0
                    or topk_group > n_group or weight is None or bias is None or weight.ndim != 2
                    or int(weight.shape[0]) not in _SUPPORTED_NR):
                return original_call(x)
            logits = x @ weight.T
            w, idx = deepseek_router_topk_sigmoid(logits, bias, k=top_k, n_group=n_group, topk_group=topk_group,
                                                  compute_dtype=torch.float32)
            if scaling != 1.0:
                w = w * scaling
            return idx.view(torch.int32), w

        module._zmlx_original_call = original_call
        module._zmlx_original_class = module.__class__
        module.__class__ = type(module.__class__.__name__, (module.__class__,), {"__call__": patched_call})
        return module


register(_DeepSeekRouterPattern())
