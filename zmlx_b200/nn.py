"""torch modules with the attribute surface of the mlx_lm MoE blocks that ZMLX patches.

The reference patches third-party ``mlx_lm`` modules (``QuantizedSwitchLinear``, ``SwitchGLU``, the Qwen3 /
GLM / DeepSeek MoE blocks and ``MoEGate``; referenced by name in src/zmlx/patch/patterns/moe_mlp.py:392-426 and
deepseek_router.py:38-69).  These are their torch stand-ins: same attribute names, MLX-layout packed
parameters, and an *unfused* forward written with plain torch ops (dequantise, matmul), which plays the role of
stock mlx_lm and is what ``zmlx_b200.patch.patch`` replaces.
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import quant


class QuantizedSwitchLinear(nn.Module):
    """Bank of E quantised linear layers, ``y = x @ dequant(W[e]).T`` (mlx_lm's QuantizedSwitchLinear)."""

    def __init__(self, weight, scales, biases=None, *, group_size: int = 64, bits: int = 4, mode: str = "affine"):
        super().__init__()
        self.register_buffer("weight", weight)
        self.register_buffer("scales", scales)
        self.register_buffer("biases", biases)
        self.group_size, self.bits, self.mode = group_size, bits, mode
        self.bias = None

    def get(self, name, default=None):  # mlx modules are dict-like: `proj.get("biases")`
        return getattr(self, name, default)

    def dequantized(self, idx: torch.Tensor) -> torch.Tensor:
        w = self.weight.view(torch.int32)[idx].view(torch.uint32)
        if self.mode == "affine":
            return quant.dequantize_affine(w, self.scales[idx], self.biases[idx], self.group_size)
        return quant.dequantize_mxfp4(w, self.scales[idx])

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        """x (..., 1, 1, K) or (..., K_slots, 1, K); indices (..., K_slots) -> (..., K_slots, 1, N) in x.dtype."""
        idx = indices.to(torch.int64)
        w = self.dequantized(idx)  # (..., K_slots, N, K) float32
        y = torch.matmul(x.to(torch.float32), w.transpose(-1, -2))
        return y.to(x.dtype)


class SwiGLU(nn.Module):
    def forward(self, x_up, x_gate):
        return torch.nn.functional.silu(x_gate) * x_up


class SwitchGLU(nn.Module):
    """gate/up/down expert banks with a SwiGLU in between (mlx_lm.models.switch_layers.SwitchGLU)."""

    def __init__(self, gate_proj, up_proj, down_proj):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.activation = None  # standard SwiGLU

    def forward(self, x: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
        x = x.unsqueeze(-2).unsqueeze(-3)  # (B, L, D) -> (B, L, 1, 1, D)
        x_up = self.up_proj(x, indices)
        x_gate = self.gate_proj(x, indices)
        h = torch.nn.functional.silu(x_gate) * x_up
        return self.down_proj(h, indices).squeeze(-2)


class QuantizedMLP(nn.Module):
    """Dense quantised SwiGLU MLP (the shared expert): the same banks with E = 1."""

    def __init__(self, gate_proj, up_proj, down_proj):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z = torch.zeros(x.shape[:-1] + (1,), dtype=torch.int64, device=x.device)
        xx = x.unsqueeze(-2).unsqueeze(-3)
        h = torch.nn.functional.silu(self.gate_proj(xx, z)) * self.up_proj(xx, z)
        return self.down_proj(h, z).squeeze(-2).squeeze(-2)


class QuantizedLinear(nn.Module):
    """One quantised linear layer, ``y = x @ dequant(W).T`` (mlx.nn.QuantizedLinear): weight (N, K/8) uint32,
    scales and biases (N, K/group_size)."""

    def __init__(self, weight, scales, biases=None, *, group_size: int = 64, bits: int = 4, mode: str = "affine"):
        super().__init__()
        self.register_buffer("weight", weight)
        self.register_buffer("scales", scales)
        self.register_buffer("biases", biases)
        self.group_size, self.bits, self.mode = group_size, bits, mode

    def get(self, name, default=None):
        return getattr(self, name, default)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = quant.dequantize_affine(self.weight.view(torch.uint32)[None], self.scales[None], self.biases[None],
                                    self.group_size)[0]
        return torch.matmul(x.to(torch.float32), w.T).to(x.dtype)


class MLP(nn.Module):
    """Dense SwiGLU MLP with quantised projections (the Llama / Qwen ``mlp`` module)."""

    def __init__(self, gate_proj, up_proj, down_proj):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.hidden_act = "silu"

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


def mlp_from_params(p: dict, *, group_size: int = 64) -> MLP:
    """Builds a dense MLP from a one-expert bank dict (``gate_w`` (1, N, K/8) ...), e.g. ``make_layer(...)["shared"]``."""
    def lin(name):
        return QuantizedLinear(p[f"{name}_w"][0].contiguous(), p[f"{name}_s"][0].contiguous(),
                               p[f"{name}_b"][0].contiguous(), group_size=group_size)
    return MLP(lin("gate"), lin("up"), lin("down"))


class Qwen3MoeSparseMoeBlock(nn.Module):
    """Softmax router over raw logits, top-k, optional renormalisation (mlx_lm qwen3_moe)."""

    def __init__(self, gate_weight, switch_mlp, *, top_k: int, norm_topk_prob: bool = True):
        super().__init__()
        self.gate = nn.Linear(gate_weight.shape[1], gate_weight.shape[0], bias=False, dtype=gate_weight.dtype,
                              device=gate_weight.device)
        self.gate.weight.data.copy_(gate_weight)
        self.switch_mlp = switch_mlp
        self.top_k = top_k
        self.num_experts_per_tok = top_k
        self.norm_topk_prob = norm_topk_prob

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        gates = torch.softmax(self.gate(x).to(torch.float32), dim=-1)
        scores, inds = torch.topk(gates, self.top_k, dim=-1)
        if self.norm_topk_prob:
            scores = scores / scores.sum(dim=-1, keepdim=True)
        y = self.switch_mlp(x, inds)
        return (y.to(torch.float32) * scores[..., None]).sum(dim=-2).to(x.dtype)


class MoEGate(nn.Module):
    """Sigmoid router with a selection-only bias and group-limited top-k; returns (indices, scores)."""

    def __init__(self, weight, e_score_correction_bias, *, top_k: int, n_group: int = 1, topk_group: int = 1,
                 routed_scaling_factor: float = 1.0, norm_topk_prob: bool = True):
        super().__init__()
        self.register_buffer("weight", weight)
        self.register_buffer("e_score_correction_bias", e_score_correction_bias)
        self.top_k, self.n_group, self.topk_group = top_k, n_group, topk_group
        self.routed_scaling_factor, self.norm_topk_prob = routed_scaling_factor, norm_topk_prob

    def forward(self, x: torch.Tensor):
        logits = (x @ self.weight.T).to(torch.float32)
        aff = torch.sigmoid(logits)
        scores = aff + self.e_score_correction_bias
        E = scores.shape[-1]
        if self.n_group > 1:
            g = scores.reshape(*scores.shape[:-1], self.n_group, E // self.n_group)
            gs = g.topk(2, dim=-1).values.sum(-1)
            keep = torch.zeros_like(gs).scatter_(-1, gs.topk(self.topk_group, dim=-1).indices, 1.0)
            scores = (g * keep[..., None]).reshape(scores.shape)
        inds = scores.topk(self.top_k, dim=-1).indices
        w = torch.gather(aff, -1, inds)
        if self.norm_topk_prob:
            w = w / w.sum(-1, keepdim=True)
        return inds, w * self.routed_scaling_factor


class GlmMoeBlock(nn.Module):
    """GLM-4 / DeepSeek-V3 style block: MoEGate, SwitchGLU experts, additive shared experts."""

    def __init__(self, gate: MoEGate, switch_mlp: SwitchGLU, shared_experts=None):
        super().__init__()
        self.gate, self.switch_mlp, self.shared_experts = gate, switch_mlp, shared_experts
        self.num_experts_per_tok = gate.top_k

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        inds, scores = self.gate(x)
        y = self.switch_mlp(x, inds)
        y = (y.to(torch.float32) * scores[..., None]).sum(dim=-2).to(x.dtype)
        if self.shared_experts is not None:
            y = y + self.shared_experts(x)
        return y


class DeepseekV3MoE(GlmMoeBlock):
    """Same structure; the class name selects the generic combine in the patch (moe_mlp.py:1055-1057)."""


def block_from_params(cfg, p: dict) -> nn.Module:
    """Builds the family's block from a ``synthetic.make_layer`` dict."""
    gs = 32 if cfg.mode == "mxfp4" else cfg.group_size

    def bank(d, name):
        return QuantizedSwitchLinear(d[f"{name}_w"], d[f"{name}_s"], d[f"{name}_b"], group_size=gs, bits=4, mode=cfg.mode)

    switch = SwitchGLU(bank(p, "gate"), bank(p, "up"), bank(p, "down"))
    shared = None
    if p.get("shared") is not None:
        s = p["shared"]
        shared = QuantizedMLP(bank(s, "gate"), bank(s, "up"), bank(s, "down"))
    if cfg.family in ("glm", "deepseek"):
        gate = MoEGate(p["router_w"], p["expert_bias"], top_k=cfg.top_k, n_group=cfg.n_group,
                       topk_group=cfg.topk_group, routed_scaling_factor=cfg.routed_scaling_factor)
        cls = GlmMoeBlock if cfg.family == "glm" else DeepseekV3MoE
        return cls(gate, switch, shared)
    return Qwen3MoeSparseMoeBlock(p["router_w"], switch, top_k=cfg.top_k, norm_topk_prob=cfg.norm_topk_prob)
