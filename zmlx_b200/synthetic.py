"""Seeded synthetic MoE layers in the shapes the benchmark configurations name.

No checkpoint or dataset is involved: weights are N(0, 0.02) quantised to the MLX
layouts, activations are bfloat16 N(0, 1), router weights bfloat16 N(0, 0.02) and
selection biases float32 N(0, 0.01), all from seeded generators
(value distributions as in the reference's tests,
tests/test_gather_qmm_swiglu.py:41, 91 and tests/test_kernels_catalog.py:176).
"""

from __future__ import annotations

from dataclasses import dataclass, replace

import torch

from . import quant


@dataclass(frozen=True)
class MoEConfig:
    name: str
    config_id: int
    d_model: int
    n_experts: int
    top_k: int
    d_ff: int
    family: str  # "generic" | "qwen3" | "glm" | "deepseek"
    mode: str = "affine"  # "affine" | "mxfp4"
    group_size: int = 64
    n_shared: int = 0
    n_group: int = 1
    topk_group: int = 1
    routed_scaling_factor: float = 1.0
    norm_topk_prob: bool = True

    @property
    def bytes_per_weight(self) -> float:
        return 0.5 + (4.0 / self.group_size if self.mode == "affine" else 1.0 / 32.0)

    @property
    def expert_bytes(self) -> int:
        """Packed bytes of one expert: gate + up + down codes, scales and biases."""
        return int(3 * self.d_model * self.d_ff * self.bytes_per_weight)

    @property
    def router_bytes(self) -> int:
        return self.n_experts * self.d_model * 2

    def algorithmic_bytes(self, distinct_experts: int, tokens: int) -> int:
        """Bytes one layer pass must move: every touched expert once, the shared
        experts, the router weight and the token rows in and out."""
        return ((distinct_experts + self.n_shared) * self.expert_bytes + self.router_bytes
                + tokens * self.d_model * 2 * 2)

    def scaled(self, **kw) -> "MoEConfig":
        return replace(self, **kw)


CONFIGS: dict[str, MoEConfig] = {
    # 1: single layer runnable on the reference's CPU path
    "c1": MoEConfig("c1-d1024-e32-top4", 1, 1024, 32, 4, 768, "generic"),
    # 2: Qwen3-30B-A3B-shaped layer
    "c2": MoEConfig("c2-qwen3-30b-a3b", 2, 2048, 128, 8, 768, "qwen3"),
    # 3: GLM-4.7-Flash-shaped layer, mxfp4, one shared expert
    "c3": MoEConfig("c3-glm-4.7-flash", 3, 2048, 64, 4, 1536, "glm", mode="mxfp4", group_size=32, n_shared=1,
                    routed_scaling_factor=1.8),
    # 5: DeepSeek-V3-shaped layer, group-limited routing, one shared expert
    "c5": MoEConfig("c5-deepseek-v3", 5, 7168, 256, 8, 2048, "deepseek", n_shared=1, n_group=8, topk_group=4,
                    routed_scaling_factor=2.5),
}


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _quantize_bank(cfg: MoEConfig, n_out: int, n_in: int, E: int, seed: int, device, chunk: int = 16):
    """(E, n_out, n_in) N(0, 0.02) weights, quantised chunk by chunk to bound memory."""
    g = _gen(seed, device)
    packed, scales, biases = [], [], []
    for e0 in range(0, E, chunk):
        n = min(chunk, E - e0)
        w = torch.randn((n, n_out, n_in), generator=g, device=device, dtype=torch.float32) * 0.02
        if cfg.mode == "affine":
            p, s, b = quant.quantize_affine(w, cfg.group_size)
            biases.append(b)
        else:
            p, s = quant.quantize_mxfp4(w)
        packed.append(p.view(torch.int32))
        scales.append(s)
        del w
    pw = torch.cat(packed).view(torch.uint32)
    return pw, torch.cat(scales), (torch.cat(biases) if biases else None)


def make_layer(cfg: MoEConfig, *, layer: int = 0, device="cpu") -> dict:
    """All tensors of one MoE layer.  Keys: router_w, expert_bias, gate_w/gate_s/gate_b,
    up_*, down_*, and ``shared`` (a dict of the same gate/up/down keys with E == 1) or None."""
    base = 1000 * cfg.config_id + 100003 * layer
    p: dict = {}
    g = _gen(base + 1, device)
    p["router_w"] = (torch.randn((cfg.n_experts, cfg.d_model), generator=g, device=device) * 0.02).to(torch.bfloat16)
    if cfg.family in ("glm", "deepseek"):
        p["expert_bias"] = torch.randn((cfg.n_experts,), generator=g, device=device) * 0.01
    else:
        p["expert_bias"] = None
    for i, (name, n_out, n_in) in enumerate((("gate", cfg.d_ff, cfg.d_model), ("up", cfg.d_ff, cfg.d_model),
                                             ("down", cfg.d_model, cfg.d_ff))):
        w, s, b = _quantize_bank(cfg, n_out, n_in, cfg.n_experts, base + 10 + i, device)
        p[f"{name}_w"], p[f"{name}_s"], p[f"{name}_b"] = w, s, b
    if cfg.n_shared:
        sh: dict = {}
        for i, (name, n_out, n_in) in enumerate((("gate", cfg.d_ff * cfg.n_shared, cfg.d_model),
                                                 ("up", cfg.d_ff * cfg.n_shared, cfg.d_model),
                                                 ("down", cfg.d_model, cfg.d_ff * cfg.n_shared))):
            w, s, b = _quantize_bank(cfg, n_out, n_in, 1, base + 20 + i, device)
            sh[f"{name}_w"], sh[f"{name}_s"], sh[f"{name}_b"] = w, s, b
        p["shared"] = sh
    else:
        p["shared"] = None
    return p


def make_tokens(cfg: MoEConfig, tokens: int, *, step: int = 0, device="cpu") -> torch.Tensor:
    """(tokens, d_model) bfloat16 N(0, 1) activations."""
    g = _gen(7 * cfg.config_id + tokens + 7919 * step, device)
    return torch.randn((tokens, cfg.d_model), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
