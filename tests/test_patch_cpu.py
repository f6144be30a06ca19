"""CPU: patch framework and MoE pattern logic with stand-in kernels (the style of the reference's
tests/test_moe_fused_swiglu_gate.py and tests/test_patch.py: fakes and monkeypatching, no device work)."""

import pytest
import torch

from zmlx_b200 import nn as znn
from zmlx_b200 import synthetic
from zmlx_b200.kernels import moe
from zmlx_b200.patch import PatchConfig, PatchResult, get_pattern, list_patterns, patch, unpatch
from zmlx_b200.patch.patterns import moe_mlp as mm


def _tiny(family="qwen3", **kw):
    base = {"qwen3": "c2", "glm": "c3", "deepseek": "c5"}[family]
    cfg = synthetic.CONFIGS[base].scaled(n_experts=8, d_model=128, d_ff=64, top_k=2, n_group=1, topk_group=1,
                                         mode="affine", group_size=64, **kw)
    return cfg, synthetic.make_layer(cfg)


class _Model(torch.nn.Module):
    def __init__(self, blocks):
        super().__init__()
        self.layers = torch.nn.ModuleList(blocks)


def test_registry_and_types():
    assert list_patterns() == ["deepseek_router", "moe_mlp", "swiglu_mlp"]
    assert get_pattern("moe_mlp").name == "moe_mlp"
    with pytest.raises(KeyError):
        get_pattern("nope")
    r = PatchResult(patched_count=2, pattern_counts={"moe_mlp": 2}, skipped=["x: boom"])
    assert r.summary().splitlines() == ["Patched 2 modules:", "  moe_mlp: 2", "  Skipped: 1"]
    assert PatchConfig().moe_fused_swiglu_max_tokens is None


def test_patch_swaps_call_and_unpatch_restores():
    cfg, p = _tiny()
    blk = znn.block_from_params(cfg, p)
    m = _Model([blk, torch.nn.Linear(4, 4)])
    x = torch.randn(1, 2, 128).bfloat16()
    y0 = blk(x)
    out = patch(m)
    assert out is m and m._zmlx_patch_result.patched_count == 1
    assert m._zmlx_patch_result.pattern_counts == {"moe_mlp": 1}
    assert type(blk).__name__ == "Qwen3MoeSparseMoeBlock" and type(blk) is not znn.Qwen3MoeSparseMoeBlock
    assert hasattr(blk, "_zmlx_original_call") and hasattr(blk.switch_mlp, "_zmlx_original_switch_call")
    unpatch(m)
    assert type(blk) is znn.Qwen3MoeSparseMoeBlock and not hasattr(m, "_zmlx_patch_result")
    assert torch.equal(blk(x), y0)


def test_selection_rules():
    cfg, p = _tiny()
    m = _Model([znn.block_from_params(cfg, p)])
    with pytest.raises(ValueError, match="Unknown mode"):
        patch(m, mode="training")
    with pytest.raises(ValueError, match="Unknown profile"):
        patch(m, profile="llama")
    patch(m, exclude=["moe_mlp"])
    assert m._zmlx_patch_result.patched_count == 0
    patch(m, profile="qwen3")
    assert m._zmlx_patch_result.patched_count == 1
    unpatch(m)
    patch(m, patterns=["deepseek_router"])  # no MoEGate in a Qwen block
    assert m._zmlx_patch_result.patched_count == 0


def test_env_flags(monkeypatch):
    monkeypatch.delenv("ZMLX_GLM_COMBINE_MODE", raising=False)
    assert mm._glm_combine_mode() == "fp32_no_fma"
    for raw, want in (("fp32", "fp32"), ("exact", "exact"), ("off", "fp32_no_fma"), ("garbage", "fp32_no_fma")):
        monkeypatch.setenv("ZMLX_GLM_COMBINE_MODE", raw)
        assert mm._glm_combine_mode() == want
    monkeypatch.delenv("ZMLX_QWEN_COMBINE_MODE", raising=False)
    assert mm._qwen_combine_mode() == "off"
    monkeypatch.setenv("ZMLX_QWEN_COMBINE_MODE", "FP32_NO_FMA")
    assert mm._qwen_combine_mode() == "fp32_no_fma"
    monkeypatch.setenv("ZMLX_GLM_FUSED_SWIGLU", "0")
    assert mm._glm_allow_fused_swiglu() is False
    monkeypatch.setenv("ZMLX_GLM_FUSED_SWIGLU", "x")
    assert mm._glm_allow_fused_swiglu() is False
    monkeypatch.setenv("ZMLX_QWEN_FUSED_SWIGLU", "true")
    assert mm._qwen_allow_fused_swiglu() is True


@pytest.mark.parametrize("family,combine_env,expect", [
    ("qwen3", None, "moe_combine_no_fma"), ("qwen3", ("ZMLX_QWEN_COMBINE_MODE", "fp32"), "moe_combine_fp32"),
    ("glm", None, "moe_combine_fp32_no_fma"), ("glm", ("ZMLX_GLM_COMBINE_MODE", "exact"), "moe_combine_exact"),
    ("deepseek", None, "moe_combine"),
])
def test_patched_call_routes_to_the_family_combine(monkeypatch, family, combine_env, expect):
    """Stand-in kernels record which ops the patched block calls and with what (cf. the reference's
    monkeypatched kwargs-routing tests, tests/test_moe_fused_swiglu_gate.py:189-326)."""
    if combine_env:
        monkeypatch.setenv(*combine_env)
    else:
        monkeypatch.delenv("ZMLX_QWEN_COMBINE_MODE", raising=False)
        monkeypatch.delenv("ZMLX_GLM_COMBINE_MODE", raising=False)
    cfg, p = _tiny(family, n_shared=(1 if family != "qwen3" else 0))
    blk = znn.block_from_params(cfg, p)
    calls = []

    def fake_fused(switch_mlp, x, indices, *, max_tokens):
        calls.append(("fused", tuple(indices.shape), max_tokens))
        return torch.ones(tuple(indices.shape) + (cfg.d_model,), dtype=x.dtype)

    def fake_combine(name):
        def f(y, w):
            calls.append((name, w.dtype))
            return y.float().mul(w[..., None].float()).sum(-2).to(y.dtype)
        return f

    monkeypatch.setattr(mm, "_fused_switch_mlp_call", fake_fused)
    for n in ("moe_combine", "moe_combine_no_fma", "moe_combine_exact", "moe_combine_fp32", "moe_combine_fp32_no_fma"):
        monkeypatch.setattr(moe, n, fake_combine(n))
    monkeypatch.setattr(moe, "qwen3_gating", lambda logits, k, norm_topk_prob=True: (
        torch.zeros(logits.shape[:-1] + (k,), dtype=torch.int32), torch.full(logits.shape[:-1] + (k,), 0.5)))
    m = _Model([blk])
    patch(m, moe_fused_swiglu_max_tokens=7)
    x = torch.randn(1, 3, 128).bfloat16()
    y = blk(x)
    assert y.shape == x.shape
    assert calls[0] == ("fused", (1, 3, 2), 7)
    assert calls[1][0] == expect
    if family != "qwen3":  # gate returned (indices, scores) itself and the shared expert was added
        shared = blk.shared_experts(x)
        assert torch.allclose(y.float(), (torch.ones_like(y).float() * blk.gate(x)[1].sum(-1, keepdim=True)).to(
            y.dtype).float() + shared.float(), atol=2e-2)


def test_fused_path_respects_token_cap(monkeypatch):
    cfg, p = _tiny()
    blk = znn.block_from_params(cfg, p)
    sw = blk.switch_mlp
    sw._zmlx_original_switch_call = lambda x, idx: "original"
    idx = torch.zeros((1, 5, 2), dtype=torch.int32)
    assert mm._fused_switch_mlp_call(sw, torch.zeros(1, 5, 128), idx, max_tokens=4) == "original"
    assert mm._should_fuse_swiglu_tokens(5, None) and not mm._should_fuse_swiglu_tokens(5, 4)


def test_can_fuse_rules():
    cfg, p = _tiny()
    sw = znn.block_from_params(cfg, p).switch_mlp
    assert mm._can_fuse_switch_mlp(sw)
    sw.up_proj.group_size = 32
    assert not mm._can_fuse_switch_mlp(sw)
    sw.up_proj.group_size = 64
    sw.activation = torch.nn.GELU()
    assert not mm._can_fuse_switch_mlp(sw)
    assert not mm._MoEMLPPattern().matches(torch.nn.Linear(2, 2), "x")


def test_swiglu_mlp_pattern_matches_dense_mlps_only():
    """src/zmlx/patch/patterns/swiglu_mlp.py:222-236: gate/up/down layout; not the switch bank, not a child of a
    MoE block unless it is `shared_experts`.  On CPU tensors the patched call is the module's own."""
    pat = get_pattern("swiglu_mlp")
    cfg, p = _tiny("glm", n_shared=1)
    blk = znn.block_from_params(cfg, p)
    dense = znn.mlp_from_params(p["shared"])
    assert pat.matches(dense, "mlp", None)
    assert not pat.matches(blk.switch_mlp, "switch_mlp", blk)
    assert pat.matches(blk.shared_experts, "shared_experts", blk)
    assert not pat.matches(dense, "mlp", blk)  # some other child of a block with a gate
    assert not pat.matches(torch.nn.Linear(4, 4), "proj", None)

    m = _Model([dense])
    x = torch.randn(2, 3, 128).bfloat16()
    y0 = dense(x)
    patch(m, patterns=["swiglu_mlp"])
    assert m._zmlx_patch_result.pattern_counts == {"swiglu_mlp": 1}
    assert type(dense) is not znn.MLP and torch.equal(dense(x), y0)
    unpatch(m)
    assert type(dense) is znn.MLP
