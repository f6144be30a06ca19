"""MLX-format checkpoint ingestion for the MoE block (safetensors files as published by mlx-community).

The reference loads models through ``mlx_lm.utils.load`` (src/zmlx/api.py:363-423) and patches the modules it finds;
the packed tensors of a quantised switch bank are stored exactly as the kernels of this package read them
(src/zmlx/kernels/fused_moe.py:64-69: weight ``(E, N, K/8)`` uint32, scales and biases ``(E, N, K/group_size)``), so
ingestion is a matter of names:

    {prefix}.gate.weight                                  (E, d)       router (``{prefix}.router.weight`` also taken;
                                                                        quantised routers -- .scales/.biases present,
                                                                        4 or 8 bits -- are dequantised to bfloat16)
    {prefix}.gate.e_score_correction_bias                 (E,)         selection bias of the sigmoid routers
    {prefix}.switch_mlp.{gate,up,down}_proj.weight        (E, N, K/8)  uint32
    {prefix}.switch_mlp.{gate,up,down}_proj.{scales,biases}
    {prefix}.shared_experts.{gate,up,down}_proj.{weight,scales,biases}   dense, (N, K/8) ...

``load_moe_params`` returns the parameter dict ``MoELayer`` and ``nn.block_from_params`` take.  Real checkpoints are
not available where this was written; ``save_moe_params`` writes the same names from a parameter dict and the tests
round-trip through it.
"""

from __future__ import annotations

import os
from typing import Iterable

import torch

_PROJ = ("gate", "up", "down")


def _open_all(paths: Iterable[str]):
    from safetensors import safe_open  # library code for the file format only

    handles = []
    for path in paths:
        handles.append(safe_open(path, framework="pt", device="cpu"))
    return handles


class _Index:
    """Name -> tensor over one or several safetensors shards (lazy: a tensor is read when asked for)."""

    def __init__(self, paths: Iterable[str]):
        self._handles = _open_all(paths)
        self._where = {}
        for h in self._handles:
            for k in h.keys():
                self._where[k] = h

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def get(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise KeyError(f"tensor {name!r} is not in the checkpoint")
        return self._where[name].get_tensor(name)

    def keys(self):
        return self._where.keys()


def shard_paths(path: str) -> list[str]:
    """A file, or every ``*.safetensors`` of a directory (sorted)."""
    if os.path.isdir(path):
        return sorted(os.path.join(path, f) for f in os.listdir(path) if f.endswith(".safetensors"))
    return [path]


def _as_u32(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.uint32:
        return t
    if t.dtype == torch.int32:
        return t.view(torch.uint32)
    raise TypeError(f"packed weights must be uint32, got {t.dtype}")


def _dequant_router(w: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, d_model: int) -> torch.Tensor:
    """Quantised router weight (E, d*bits/32) -> bfloat16 (E, d); bits follow from the shapes (4 or 8)."""
    w = _as_u32(w)
    bits = w.shape[-1] * 32 // d_model
    if bits not in (4, 8) or w.shape[-1] * 32 != d_model * bits:
        raise ValueError(f"router weight {tuple(w.shape)} does not pack {d_model} values at 4 or 8 bits")
    per = 32 // bits
    shifts = torch.arange(per, dtype=torch.int64) * bits
    q = ((w.to(torch.int64)[..., None] >> shifts) & ((1 << bits) - 1)).reshape(w.shape[0], d_model).to(torch.float32)
    gs = d_model // scales.shape[-1]
    s = scales.to(torch.float32).repeat_interleave(gs, dim=-1)
    b = biases.to(torch.float32).repeat_interleave(gs, dim=-1)
    return (q * s + b).to(torch.bfloat16)


def load_moe_params(path: str, prefix: str, *, device="cpu") -> dict:
    """The block under ``prefix`` (e.g. ``model.layers.3.mlp``) as a ``make_layer``-style dict on ``device``."""
    idx = _Index(shard_paths(path))
    sw = f"{prefix}.switch_mlp" if f"{prefix}.switch_mlp.gate_proj.weight" in idx else f"{prefix}.experts"
    if f"{sw}.gate_proj.weight" not in idx:
        raise KeyError(f"no switch bank under {prefix!r} (looked for {prefix}.switch_mlp / {prefix}.experts)")
    p: dict = {}
    for name in _PROJ:
        p[f"{name}_w"] = _as_u32(idx.get(f"{sw}.{name}_proj.weight")).contiguous().to(device)
        p[f"{name}_s"] = idx.get(f"{sw}.{name}_proj.scales").to(torch.bfloat16).contiguous().to(device)
        bname = f"{sw}.{name}_proj.biases"
        p[f"{name}_b"] = idx.get(bname).to(torch.bfloat16).contiguous().to(device) if bname in idx else None
    d_model = p["gate_w"].shape[-1] * 8
    gate = f"{prefix}.gate" if f"{prefix}.gate.weight" in idx else f"{prefix}.router"
    rw = idx.get(f"{gate}.weight")
    if f"{gate}.scales" in idx:
        rw = _dequant_router(rw, idx.get(f"{gate}.scales"), idx.get(f"{gate}.biases"), d_model)
    p["router_w"] = rw.to(torch.bfloat16).contiguous().to(device)
    bias = f"{gate}.e_score_correction_bias"
    p["expert_bias"] = idx.get(bias).to(torch.float32).contiguous().to(device) if bias in idx else None
    sh = f"{prefix}.shared_experts"
    if f"{sh}.gate_proj.weight" in idx:
        s: dict = {}
        for name in _PROJ:
            s[f"{name}_w"] = _as_u32(idx.get(f"{sh}.{name}_proj.weight"))[None].contiguous().to(device)
            s[f"{name}_s"] = idx.get(f"{sh}.{name}_proj.scales").to(torch.bfloat16)[None].contiguous().to(device)
            s[f"{name}_b"] = idx.get(f"{sh}.{name}_proj.biases").to(torch.bfloat16)[None].contiguous().to(device)
        p["shared"] = s
    else:
        p["shared"] = None
    return p


def moe_block_prefixes(path: str) -> list[str]:
    """Prefixes of every MoE block in the checkpoint, in layer order."""
    idx = _Index(shard_paths(path))
    found = set()
    for k in idx.keys():
        for tail in (".switch_mlp.gate_proj.weight", ".experts.gate_proj.weight"):
            if k.endswith(tail):
                found.add(k[: -len(tail)])

    def order(pfx: str):
        return [int(t) if t.isdigit() else t for t in pfx.split(".")]

    return sorted(found, key=order)


def save_moe_params(p: dict, path: str, prefix: str) -> None:
    """Writes a ``make_layer``-style dict under the MLX names (test and conversion helper)."""
    from safetensors.torch import save_file

    out = {f"{prefix}.gate.weight": p["router_w"].cpu().contiguous()}
    if p.get("expert_bias") is not None:
        out[f"{prefix}.gate.e_score_correction_bias"] = p["expert_bias"].cpu().contiguous()
    for name in _PROJ:
        out[f"{prefix}.switch_mlp.{name}_proj.weight"] = p[f"{name}_w"].cpu().contiguous()
        out[f"{prefix}.switch_mlp.{name}_proj.scales"] = p[f"{name}_s"].cpu().contiguous()
        if p.get(f"{name}_b") is not None:
            out[f"{prefix}.switch_mlp.{name}_proj.biases"] = p[f"{name}_b"].cpu().contiguous()
    if p.get("shared") is not None:
        for name in _PROJ:
            for suffix, key in (("weight", "w"), ("scales", "s"), ("biases", "b")):
                out[f"{prefix}.shared_experts.{name}_proj.{suffix}"] = p["shared"][f"{name}_{key}"][0].cpu().contiguous()
    save_file(out, path)
