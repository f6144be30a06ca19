"""``patch(model)``: swap MoE blocks of a torch model for the fused-kernel path.

Mirrors src/zmlx/patch/__init__.py:129-305 (``patch``) and :308-384 (``unpatch``): same keyword arguments, preset
names, family safety excludes and the ``_zmlx_patch_result`` attribute.  Only the patterns of the MoE decode path
exist here (``moe_mlp``, ``deepseek_router``); names of the reference's other patterns are accepted in
``exclude`` and ignored in presets.
"""

from __future__ import annotations

import os
from typing import Any

import torch.nn as nn

from ._registry import _ensure_loaded, get_all_patterns, get_pattern, list_patterns, register  # noqa: F401
from ._traversal import apply_patterns
from ._types import PatchConfig, PatchPattern, PatchResult  # noqa: F401

#: Fused-activation preset of the reference; only ``moe_mlp`` is on this path.
FUSED_ACTIVATIONS: list[str] = ["swiglu_mlp", "geglu_mlp", "moe_mlp"]
ALL_PATTERNS: list[str] = ["swiglu_mlp", "geglu_mlp", "moe_mlp", "rmsnorm", "layernorm", "softmax", "residual_norm"]

_FIDELITY_EXCLUDES: dict[str, set[str]] = {
    "qwen": {"swiglu_mlp", "residual_norm"},
    "gpt_oss": {"residual_norm"},
    "mixtral": {"moe_mlp"},
    "glm": {"rmsnorm"},
}


def _model_family(model: Any) -> str:
    """Best-effort family detection from class / module names (src/zmlx/patch/__init__.py:46-72)."""
    candidates: list[str] = []
    for obj in (model, getattr(model, "model", None)):
        if obj is None:
            continue
        candidates.append(type(obj).__module__ or "")
        candidates.append(type(obj).__name__)
    combined = " ".join(candidates).lower()
    for key, fam in (("lfm", "lfm"), ("qwen", "qwen"), ("gpt_oss", "gpt_oss"), ("gptoss", "gpt_oss"),
                     ("nemotron", "nemotron"), ("llama", "llama"), ("mixtral", "mixtral"), ("deepseek", "deepseek"),
                     ("glm", "glm")):
        if key in combined:
            return fam
    return "unknown"


def _available(names: list[str]) -> list[PatchPattern]:
    known = set(list_patterns())
    return [get_pattern(n) for n in names if n in known]


def patch(
    model: nn.Module,
    *,
    mode: str | None = None,
    profile: str | None = None,
    patterns: list[str] | None = None,
    exclude: list[str] | None = None,
    compute_dtype: str = "float32",
    threadgroup: int | str = 256,
    moe_fused_swiglu_max_tokens: int | None = None,
    verbose: bool = False,
) -> nn.Module:
    """Patch a model in place to use the fused MoE kernels; returns the same model.

    Pattern selection: explicit ``patterns`` > ``profile`` > ``mode`` > the inference default.  Families with known
    fidelity issues are excluded from the default selection as in the reference; the reference's *performance*
    excludes (Qwen / GLM ``moe_mlp`` on stock MLX) do not apply because the fused op always exists here.
    Sets ``model._zmlx_patch_result`` (a :class:`PatchResult`).
    """
    _ensure_loaded()
    modes = {"inference": FUSED_ACTIVATIONS}
    profiles = {"qwen3": ["moe_mlp"], "qwen3-minimal": ["moe_mlp"]}
    config = PatchConfig(compute_dtype=compute_dtype, threadgroup=threadgroup,
                         moe_fused_swiglu_max_tokens=moe_fused_swiglu_max_tokens, verbose=verbose)
    explicit = patterns is not None
    if explicit:
        selected = [get_pattern(name) for name in patterns]
    elif profile is not None:
        if profile not in profiles:
            raise ValueError(f"Unknown profile {profile!r}. Expected one of: {', '.join(sorted(profiles))}")
        selected = _available(profiles[profile])
    elif mode is not None:
        if mode not in modes:
            raise ValueError(f"Unknown mode {mode!r}. Expected one of: {', '.join(modes)}")
        selected = _available(modes[mode])
    else:
        selected = _available(FUSED_ACTIVATIONS)
    if exclude:
        selected = [p for p in selected if p.name not in set(exclude)]
    family = _model_family(model)
    fidelity_risks = set(_FIDELITY_EXCLUDES.get(family, set()))
    if not explicit and profile is None and fidelity_risks:
        removed = {p.name for p in selected} & fidelity_risks
        selected = [p for p in selected if p.name not in fidelity_risks]
        if removed:
            print(f"[zmlx.patch] {family} model detected — excluded {sorted(removed)} (known fidelity issues). "
                  "Override with patterns=[...].")
    elif (explicit or profile is not None) and fidelity_risks & {p.name for p in selected}:
        print(f"[zmlx.patch] WARNING: {sorted(fidelity_risks & {p.name for p in selected})} may break token "
              f"fidelity on {family} models.")
    if verbose:
        print(f"[zmlx.patch] Applying {len(selected)} patterns: {[p.name for p in selected]}")
    result = apply_patterns(model, selected, config)
    if verbose:
        print(result.summary())
    model._zmlx_patch_result = result
    return model


def unpatch(model: nn.Module) -> nn.Module:
    """Undo :func:`patch`: restore the original class of every patched module."""
    for m in model.modules():
        orig = m.__dict__.pop("_zmlx_original_class", None)
        if orig is not None:
            m.__class__ = orig
            m.__dict__.pop("_zmlx_original_call", None)
        m.__dict__.pop("_zmlx_original_switch_call", None)
        m.__dict__.pop("_zmlx_fast_layer", None)
    if hasattr(model, "_zmlx_patch_result"):
        del model._zmlx_patch_result
    return model


__all__ = ["patch", "unpatch", "PatchConfig", "PatchResult", "PatchPattern", "register", "get_pattern",
           "list_patterns", "FUSED_ACTIVATIONS", "ALL_PATTERNS"]

_ = os  # environment flags are read by the patterns at patch time
