"""MoE block pattern: reproduce each family's gating, run the experts through the fused kernels, combine.

Mirrors src/zmlx/patch/patterns/moe_mlp.py (matching :773-785, apply :787-881, patched call :883-1063) for torch
modules.  What is captured at patch time (:787-881: the gate attribute, the expert bank, k, the family, the
combine mode) is turned into one ``MoELayer`` over the module's own tensors, so that a patched block is ONE
launch (``zmoe_layer_decode``: router linear, top-k, gate/up + SwiGLU, down, combine, shared expert) for up to
eight tokens and the plan-once separate kernels beyond that; the call order of :883-1063 (gate -> experts ->
combine -> + shared_experts(x)) is what those kernels implement.  Blocks the kernels do not cover (an unknown
gate, 8-bit banks, a custom activation) keep the op-by-op path below, which calls the same operator surface as
the reference.  Differences from the reference, all of them about Metal performance guards rather than
semantics: the fused SwiGLU path is on for every family by default (the reference keeps Qwen opt-in, :835-841)
and has no token-count cap unless ``moe_fused_swiglu_max_tokens`` is given (the reference caps at 1 because its
Metal kernel re-reads an expert per row, :296-298).  The environment variables that select *semantics* keep
their names; ``ZMLX_MOE_FAST_LAYER=0`` forces the op-by-op path.
"""

from __future__ import annotations

import os
from typing import Any

import torch
import torch.nn as nn

from ...kernels import moe
from ...kernels.fused_moe import gather_qmm_swiglu, has_gather_qmm_swiglu
from .._registry import register
from .._types import PatchConfig

_GLM_COMBINE_MODE_ENV = "ZMLX_GLM_COMBINE_MODE"
_QWEN_COMBINE_MODE_ENV = "ZMLX_QWEN_COMBINE_MODE"
_GLM_FUSED_SWIGLU_ENV = "ZMLX_GLM_FUSED_SWIGLU"
_QWEN_FUSED_SWIGLU_ENV = "ZMLX_QWEN_FUSED_SWIGLU"
_GLM_FUSED_DOWNPROJ_COMBINE_ENV = "ZMLX_GLM_FUSED_DOWNPROJ_COMBINE"
_QWEN_FUSED_DOWNPROJ_COMBINE_ENV = "ZMLX_QWEN_FUSED_DOWNPROJ_COMBINE"
_QWEN_FUSED_ROUTER_TOPK_ENV = "ZMLX_QWEN_FUSED_ROUTER_TOPK"
_FAST_LAYER_ENV = "ZMLX_MOE_FAST_LAYER"


def _combined_name(mod: Any) -> str:
    cls = mod.__class__
    return f"{getattr(cls, '__module__', '') or ''} {cls.__name__}".lower()


def _is_qwen3_moe_block(mod: Any) -> bool:
    return "qwen3" in _combined_name(mod)


def _is_gpt_oss_block(mod: Any) -> bool:
    return "gpt_oss" in _combined_name(mod)


def _is_lfm2_moe_block(mod: Any) -> bool:
    return "lfm" in _combined_name(mod)


def _is_glm_moe_block(mod: Any) -> bool:
    return "glm" in _combined_name(mod)


def _env_flag(name: str, default: bool) -> bool:
    raw = os.environ.get(name)
    if raw is None:
        return default
    try:
        return int(raw) != 0
    except ValueError:
        return raw.strip().lower() in {"1", "true", "yes", "on"}


def _glm_allow_fused_swiglu() -> bool:
    """Default on; ``ZMLX_GLM_FUSED_SWIGLU=0`` disables (moe_mlp.py:81-93)."""
    return _env_flag(_GLM_FUSED_SWIGLU_ENV, True)


def _qwen_allow_fused_swiglu() -> bool:
    """Default on here (the reference's default-off is a Metal performance guard, moe_mlp.py:96-107)."""
    return _env_flag(_QWEN_FUSED_SWIGLU_ENV, True)


def _glm_combine_mode() -> str:
    """``fp32_no_fma`` (default), ``fp32`` or ``exact`` (moe_mlp.py:312-329)."""
    raw = os.environ.get(_GLM_COMBINE_MODE_ENV, "fp32_no_fma").strip().lower()
    return raw if raw in {"fp32", "fp32_no_fma", "exact"} else "fp32_no_fma"


def _qwen_combine_mode() -> str:
    """``off`` (default: multiply then sum), ``fp32``, ``fp32_no_fma`` or ``exact`` (moe_mlp.py:183-199)."""
    raw = os.environ.get(_QWEN_COMBINE_MODE_ENV, "off").strip().lower()
    return raw if raw in {"fp32", "fp32_no_fma", "exact"} else "off"


def _is_quantized_switch_linear(mod: Any) -> bool:
    return all(hasattr(mod, a) for a in ("weight", "scales", "group_size", "bits"))


def _is_switch_glu_module(mod: Any) -> bool:
    return mod is not None and all(hasattr(mod, a) for a in ("gate_proj", "up_proj", "down_proj"))


def _is_standard_swiglu_activation(switch_mlp: Any) -> bool:
    act = getattr(switch_mlp, "activation", None)
    return act is None or act.__class__.__name__ == "SwiGLU"


def _can_fuse_switch_mlp(switch_mlp: Any) -> bool:
    """moe_mlp.py:482-520, with mxfp4 accepted as well (the kernels implement it)."""
    if not has_gather_qmm_swiglu():
        return False
    gate_proj = getattr(switch_mlp, "gate_proj", None)
    up_proj = getattr(switch_mlp, "up_proj", None)
    if gate_proj is None or up_proj is None:
        return False
    if not _is_quantized_switch_linear(gate_proj) or not _is_quantized_switch_linear(up_proj):
        return False
    if getattr(gate_proj, "mode", "affine") not in ("affine", "mxfp4"):
        return False
    if getattr(gate_proj, "mode", "affine") != getattr(up_proj, "mode", "affine"):
        return False
    if gate_proj.group_size != up_proj.group_size or gate_proj.bits != up_proj.bits:
        return False
    return _is_standard_swiglu_activation(switch_mlp)


def _should_fuse_swiglu_tokens(total_tokens: int, max_tokens: int | None) -> bool:
    return max_tokens is None or total_tokens <= max_tokens


def _gating(self_mod: Any, x: Any, gate_attr: str, k: int, *, is_qwen3: bool = False, is_gpt_oss: bool = False):
    """Run the model's gating faithfully; returns (indices, weights).  moe_mlp.py:202-289."""
    gate_out = getattr(self_mod, gate_attr)(x)
    if isinstance(gate_out, tuple):
        return gate_out
    if is_qwen3:
        norm_topk_prob = bool(getattr(self_mod, "norm_topk_prob", False))
        if _env_flag(_QWEN_FUSED_ROUTER_TOPK_ENV, False) and norm_topk_prob:
            w, idx = moe.topk_gating_softmax(gate_out, k=k, expert_bias=None, norm_topk_prob=True,
                                             compute_dtype=torch.float32)
            return idx, w
        return moe.qwen3_gating(gate_out, k, norm_topk_prob=norm_topk_prob)
    if is_gpt_oss:
        scores, inds = moe.router_argpartition_logits_topk(gate_out, k=k, compute_dtype=torch.float32)
        return inds, scores
    weights, indices = moe.topk_gating_softmax(gate_out, k=k, expert_bias=getattr(self_mod, "expert_bias", None),
                                               norm_topk_prob=getattr(self_mod, "norm_topk_prob", False),
                                               compute_dtype=torch.float32)
    return indices, weights.to(x.dtype)


def _fused_switch_mlp_call(switch_mlp: Any, x: torch.Tensor, indices: torch.Tensor, *, max_tokens: int | None):
    """gate_proj + up_proj + SwiGLU in one ``gather_qmm_swiglu``, then the down projection (moe_mlp.py:528-574)."""
    k = int(indices.shape[-1]) if indices.ndim else 1
    total_tokens = int(indices.numel()) // max(1, k)
    if not _should_fuse_swiglu_tokens(total_tokens, max_tokens):
        return switch_mlp._zmlx_original_switch_call(x, indices)
    gp, up, dp = switch_mlp.gate_proj, switch_mlp.up_proj, switch_mlp.down_proj
    mode = getattr(gp, "mode", "affine")
    x_expanded = x.unsqueeze(-2).unsqueeze(-3)
    activated = gather_qmm_swiglu(x_expanded, gp.weight, gp.scales, gp.get("biases"), up.weight, up.scales,
                                  up.get("biases"), rhs_indices=indices, transpose=True, group_size=gp.group_size,
                                  bits=gp.bits, mode=mode, swiglu_contract="cpu" if mode == "affine" else "per_op")
    lead = tuple(indices.shape[:-1])
    f = activated.shape[-1]
    act = activated.reshape(-1, k, f)
    proj = moe._project_quantized(act, dp.weight, dp.scales, dp.get("biases"), indices.reshape(-1, k),
                                  dp.group_size, dp.bits, getattr(dp, "mode", "affine"))
    return proj.reshape(lead + (k, proj.shape[-1]))


def _bank_params(bank: Any, prefix: str = "") -> dict | None:
    """The packed tensors of a SwitchGLU-style bank in ``MoELayer``'s naming; None when it is not a 4-bit bank."""
    out = {}
    for name in ("gate", "up", "down"):
        proj = getattr(bank, f"{name}_proj", None)
        if proj is None or not _is_quantized_switch_linear(proj) or int(proj.bits) != 4:
            return None
        if getattr(proj, "bias", None) is not None:
            return None
        out[f"{name}_w"], out[f"{name}_s"], out[f"{name}_b"] = proj.weight, proj.scales, proj.get("biases")
    return out


def _build_fast_layer(module: Any, switch_mlp: Any, gate_attr: str, k: int, *, is_qwen3: bool, is_glm: bool,
                      is_gpt_oss: bool, glm_combine_mode: str, qwen_combine_mode: str):
    """One ``MoELayer`` over the module's tensors (what moe_mlp.py:787-881 captures at patch time), or None when
    the block is outside what the kernels cover.  Nothing is copied: the layer points at the module's buffers."""
    from ...layer import MoELayer
    from ...synthetic import MoEConfig

    if not _env_flag(_FAST_LAYER_ENV, True) or is_gpt_oss or not _is_standard_swiglu_activation(switch_mlp):
        return None
    routed = _bank_params(switch_mlp)
    if routed is None:
        return None
    gp = switch_mlp.gate_proj
    mode = getattr(gp, "mode", "affine")
    gs = int(gp.group_size)
    if (mode, gs) not in (("affine", 64), ("mxfp4", 32)):
        return None
    if any(getattr(getattr(switch_mlp, f"{n}_proj"), "mode", "affine") != mode
           or int(getattr(switch_mlp, f"{n}_proj").group_size) != gs for n in ("up", "down")):
        return None
    gate = getattr(module, gate_attr)
    gw = getattr(gate, "weight", None)
    if gw is None or gw.ndim != 2 or gw.dtype != torch.bfloat16 or not gw.is_cuda:
        return None
    if getattr(gate, "bias", None) is not None:
        return None
    E, f, d = int(gp.weight.shape[0]), int(gp.weight.shape[1]), int(gp.weight.shape[2]) * 8
    if tuple(gw.shape) != (E, d):
        return None
    sigmoid_gate = all(hasattr(gate, a) for a in ("e_score_correction_bias", "n_group", "topk_group",
                                                   "routed_scaling_factor"))
    params = dict(routed)
    params["router_w"] = gw
    n_group = topk_group = 1
    scaling = 1.0
    norm = bool(getattr(module, "norm_topk_prob", False))
    combine = None
    if sigmoid_gate:
        if not bool(getattr(gate, "norm_topk_prob", True)):
            return None  # the kernels normalise the selected affinities, as the reference's fused router does
        family = "glm" if is_glm else "deepseek"
        params["expert_bias"] = gate.e_score_correction_bias.to(torch.float32)
        n_group, topk_group = int(gate.n_group), int(gate.topk_group)
        scaling = float(gate.routed_scaling_factor)
        if is_glm:
            combine = {"fp32": "fp32", "exact": "exact"}.get(glm_combine_mode, "fp32_no_fma")
    elif isinstance(gate, nn.Linear):
        if is_qwen3:
            family = "qwen3"
            # "off" = (y * scores[..., None]).sum(-2): multiply, then sum == the no-FMA contract
            combine = {"fp32": "fp32", "fp32_no_fma": "fp32_no_fma", "exact": "exact"}.get(qwen_combine_mode, "no_fma")
            if qwen_combine_mode in ("fp32", "fp32_no_fma"):
                return None  # those return float32 rows (moe_mlp.py:1029-1040): left to the op-by-op path
        else:
            family = "generic"
            bias = getattr(module, "expert_bias", None)
            params["expert_bias"] = None if bias is None else bias.to(torch.float32)
    else:
        return None
    params.setdefault("expert_bias", None)
    shared_mod = getattr(module, "shared_experts", None)
    n_shared = 0
    params["shared"] = None
    if shared_mod is not None:
        sh = _bank_params(shared_mod)
        if sh is None or tuple(sh["gate_w"].shape) != (1, f, d // 8):
            return None
        params["shared"] = sh
        n_shared = 1
    cfg = MoEConfig(name=f"patched-{module.__class__.__name__}", config_id=0, d_model=d, n_experts=E, top_k=int(k),
                    d_ff=f, family=family, mode=mode, group_size=gs, n_shared=n_shared, n_group=n_group,
                    topk_group=topk_group, routed_scaling_factor=scaling, norm_topk_prob=norm)
    try:
        return MoELayer(cfg, params, max_tokens=8, combine=combine)
    except Exception:
        return None


class _MoEMLPPattern:
    @property
    def name(self) -> str:
        return "moe_mlp"

    def matches(self, module: Any, name: str, parent: Any | None = None) -> bool:
        if not isinstance(module, nn.Module):
            return False
        has_gate = hasattr(module, "gate") or hasattr(module, "router")
        has_experts = hasattr(module, "experts") or hasattr(module, "switch_mlp")
        return bool(has_gate and has_experts)

    def apply(self, module: Any, config: PatchConfig) -> Any:
        original_call = module.__call__
        num_experts_per_tok = (getattr(module, "num_experts_per_tok", None) or getattr(module, "top_k", None)
                               or getattr(module, "num_selected_experts", None) or 2)
        gate_attr = "gate" if hasattr(module, "gate") else "router"
        switch_mlp = None
        if hasattr(module, "switch_mlp") and _is_switch_glu_module(module.switch_mlp):
            switch_mlp = module.switch_mlp
        elif hasattr(module, "experts") and _is_switch_glu_module(module.experts):
            switch_mlp = module.experts
        if switch_mlp is None:
            raise ValueError("no SwitchGLU-style expert bank (gate_proj/up_proj/down_proj) on this block")

        is_qwen3 = _is_qwen3_moe_block(module)
        is_gpt_oss = _is_gpt_oss_block(module)
        is_glm = _is_glm_moe_block(module)
        use_fused_swiglu = _can_fuse_switch_mlp(switch_mlp)
        if use_fused_swiglu:
            switch_mlp._zmlx_original_switch_call = switch_mlp.__call__
        if is_qwen3 and not _qwen_allow_fused_swiglu():
            use_fused_swiglu = False
        if is_glm and not _glm_allow_fused_swiglu():
            use_fused_swiglu = False
        max_tokens = config.moe_fused_swiglu_max_tokens
        glm_combine_mode = _glm_combine_mode()
        qwen_combine_mode = _qwen_combine_mode()
        fast = None
        if use_fused_swiglu:
            fast = _build_fast_layer(module, switch_mlp, gate_attr, num_experts_per_tok, is_qwen3=is_qwen3,
                                     is_glm=is_glm, is_gpt_oss=is_gpt_oss, glm_combine_mode=glm_combine_mode,
                                     qwen_combine_mode=qwen_combine_mode)
        module._zmlx_fast_layer = fast
        if config.verbose:
            gp = switch_mlp.gate_proj
            print(f"  [moe_mlp] fused SwiGLU={'on' if use_fused_swiglu else 'off'} "
                  f"(bits={getattr(gp, 'bits', '?')}, gs={getattr(gp, 'group_size', '?')}), "
                  f"one-launch block={'on' if fast is not None else 'off'}")

        def patched_call(self_mod: Any, x: Any) -> Any:
            if fast is not None and x.dtype == torch.bfloat16 and x.is_cuda:
                tokens = x.numel() // x.shape[-1]
                if _should_fuse_swiglu_tokens(tokens, max_tokens):
                    x2 = x.reshape(tokens, x.shape[-1])
                    out = torch.empty_like(x2)  # a fresh result, as every operator of the reference returns
                    fast.forward(x2, out=out)
                    return out.reshape(x.shape)
            shared = getattr(self_mod, "shared_experts", None)
            indices, gate_weights = _gating(self_mod, x, gate_attr, num_experts_per_tok, is_qwen3=is_qwen3,
                                            is_gpt_oss=is_gpt_oss)
            if use_fused_swiglu:
                expert_outputs = _fused_switch_mlp_call(switch_mlp, x, indices, max_tokens=max_tokens)
            else:
                expert_outputs = switch_mlp(x, indices)
            f32 = torch.float32
            if is_glm:
                if glm_combine_mode == "fp32":
                    y = moe.moe_combine_fp32(expert_outputs, gate_weights.to(f32)).to(expert_outputs.dtype)
                elif glm_combine_mode == "exact":
                    y = moe.moe_combine_exact(expert_outputs, gate_weights.to(expert_outputs.dtype))
                else:
                    y = moe.moe_combine_fp32_no_fma(expert_outputs, gate_weights.to(f32)).to(expert_outputs.dtype)
            elif is_qwen3:
                if qwen_combine_mode == "fp32":
                    y = moe.moe_combine_fp32(expert_outputs, gate_weights.to(f32))
                elif qwen_combine_mode == "fp32_no_fma":
                    y = moe.moe_combine_fp32_no_fma(expert_outputs, gate_weights.to(f32))
                elif qwen_combine_mode == "exact":
                    y = moe.moe_combine_exact(expert_outputs, gate_weights.to(expert_outputs.dtype))
                else:
                    # (y * scores[..., None]).sum(-2): multiply then sum == the no-FMA contract
                    y = moe.moe_combine_no_fma(expert_outputs, gate_weights)
            elif is_gpt_oss:
                if gate_weights.dtype == f32:
                    y = moe.moe_combine_fp32(expert_outputs, gate_weights)
                else:
                    y = moe.moe_combine_exact(expert_outputs, gate_weights)
            else:
                y = moe.moe_combine(expert_outputs, gate_weights)
            if shared is not None:
                y = y + shared(x)
            return y

        module._zmlx_original_call = original_call
        module._zmlx_original_class = module.__class__
        module.__class__ = type(module.__class__.__name__, (module.__class__,), {"__call__": patched_call})
        return module


register(_MoEMLPPattern())
