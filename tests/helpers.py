"""Shared helpers of the test suite (golden-case expansion, tensor conversion, tolerances)."""

import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "known_answers.json")


def golden_cases():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


def expand_logits(case) -> np.ndarray:
    E, rows, spec = case["E"], case["rows"], case["logits"]
    if spec["kind"] == "zeros":
        return np.zeros((rows, E), dtype=np.float32)
    if spec["kind"] == "linspace_rows":
        row = np.linspace(spec["lo"], spec["hi"], E, dtype=np.float32)
        return np.stack([row + np.float32(spec["row_step"] * i) for i in range(rows)]).astype(np.float32)
    if spec["kind"] == "explicit":
        return np.asarray(spec["values"], dtype=np.float32)
    raise ValueError(spec["kind"])


def expand_bias(case) -> np.ndarray:
    E, spec = case["E"], case["bias"]
    b = np.zeros((E,), dtype=np.float32)
    if spec["kind"] == "sparse":
        b[np.asarray(spec["index"])] = np.asarray(spec["value"], dtype=np.float32)
    return b


def t2n(t) -> np.ndarray:
    """torch tensor -> numpy; bfloat16 widens to float32, uint32 keeps its bits."""
    import torch

    t = t.detach().cpu()
    if t.dtype == torch.bfloat16:
        return t.to(torch.float32).numpy()
    if t.dtype == torch.uint32:
        return t.view(torch.int32).numpy().view(np.uint32)
    return t.numpy()


def params_to_numpy(p: dict) -> dict:
    out = {}
    for k, v in p.items():
        if v is None:
            out[k] = None
        elif isinstance(v, dict):
            out[k] = params_to_numpy(v)
        else:
            out[k] = t2n(v)
    return out


def assert_close_rel(actual, expected, rel: float, what: str = "") -> float:
    """|a - e| <= rel * max(|e|, rms(e)) elementwise; returns the worst ratio.

    Pure relative error is meaningless for entries near zero; the rms floor ties
    the bound to the scale of the tensor.
    """
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    assert a.shape == e.shape, f"{what}: shape {a.shape} vs {e.shape}"
    assert np.isfinite(a).all(), f"{what}: non-finite values"
    rms = float(np.sqrt(np.mean(e * e))) if e.size else 0.0
    denom = np.maximum(np.abs(e), max(rms, 1e-30))
    ratio = np.abs(a - e) / denom
    worst = float(ratio.max()) if ratio.size else 0.0
    assert worst <= rel, f"{what}: max relative error {worst:.4g} exceeds {rel}"
    return worst


def subset_experts(params, experts, device):
    """Copy only the selected experts to the host (the oracle touches nothing else)."""
    import torch

    sel = torch.as_tensor(experts, device=device, dtype=torch.int64)
    out = {}
    for k in ("gate", "up", "down"):
        out[f"{k}_w"] = t2n(params[f"{k}_w"].view(torch.int32)[sel]).view(np.uint32)
        out[f"{k}_s"] = t2n(params[f"{k}_s"][sel])
        out[f"{k}_b"] = None if params[f"{k}_b"] is None else t2n(params[f"{k}_b"][sel])
    return out


def oracle_layer(cfg, params, x, logits, idx_gpu):
    """The oracle's recipe with the compiled matmuls; routing is recomputed by the oracle from the
    kernel's own bf16 logits and must match the kernel's indices exactly."""
    import torch

    from oracle import fast as F
    from oracle import semantics as S

    xn, ln = t2n(x), t2n(logits)
    bias = None if params["expert_bias"] is None else t2n(params["expert_bias"])
    if cfg.family == "generic":
        w, idx = S.topk_gating_softmax(ln, cfg.top_k, norm_topk_prob=cfg.norm_topk_prob)
        w = S.bf16(w)
        cmode = "t"
    elif cfg.family == "qwen3":
        idx, w = S.qwen3_gating(ln, cfg.top_k, norm_topk_prob=cfg.norm_topk_prob)
        cmode = "no_fma"
    else:
        w, idx = S.deepseek_router_topk_sigmoid(ln, bias, k=cfg.top_k, n_group=cfg.n_group,
                                                topk_group=cfg.topk_group)
        w = (w * np.float32(cfg.routed_scaling_factor)).astype(np.float32)
        cmode = "fp32_no_fma" if cfg.family == "glm" else "t"
    np.testing.assert_array_equal(t2n(idx_gpu).view(np.uint32), idx)  # expert indices bit-exact
    experts = np.unique(idx)
    remap = np.searchsorted(experts, idx).astype(np.int32)
    sub = subset_experts(params, experts, x.device)
    gs = 32 if cfg.mode == "mxfp4" else cfg.group_size
    y, _ = F.experts_forward(xn, remap, sub, group_size=gs, mode=cfg.mode,
                             swiglu="cpu" if cfg.mode == "affine" else "per_op")
    out = S.moe_combine(y, w, mode=cmode)
    if cmode == "fp32_no_fma":
        out = S.bf16(out)
    if cfg.n_shared:
        sh = {}
        for k, v in params["shared"].items():
            if v is None:
                sh[k] = None
            elif k.endswith("_w"):
                sh[k] = t2n(v.view(torch.int32)).view(np.uint32)[0]
            else:
                sh[k] = t2n(v)[0]
        out = S.bf16(out + S.shared_expert_mlp(xn, sh, group_size=gs, mode=cfg.mode))
    return out, w
