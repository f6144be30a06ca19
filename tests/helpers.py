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
