"""GPU parity: whole MoE block (router -> gate/up + SwiGLU -> down -> combine [+ shared expert])
at the benchmark configurations' shapes, against the oracle's per-family recipe."""

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import assert_close_rel, oracle_layer as _oracle_layer, t2n
from zmlx_b200 import synthetic
from zmlx_b200.layer import MoELayer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_LAYERS: dict = {}


def _layer(name):
    if name not in _LAYERS:
        cfg = synthetic.CONFIGS[name]
        _LAYERS[name] = (cfg, synthetic.make_layer(cfg, device=DEV))
    return _LAYERS[name]


# fused: the one-launch path (zmoe_layer_decode) takes the block; otherwise the separate kernels do
@pytest.mark.parametrize("name,T,fused", [("c1", 1, False), ("c1", 5, False), ("c2", 1, False), ("c2", 4, False),
                                          ("c2", 16, False), ("c2", 64, False), ("c2", 200, False), ("c3", 1, False), ("c3", 3, False),
                                          ("c3", 16, False), ("c5", 1, False), ("c5", 9, False), ("c5", 64, False), ("c5", 512, False),
                                          ("c1", 1, True), ("c1", 2, True), ("c1", 5, True), ("c1", 8, True),
                                          ("c2", 1, True), ("c2", 2, True), ("c2", 3, True), ("c2", 4, True),
                                          ("c2", 7, True), ("c2", 8, True), ("c5", 1, True), ("c5", 2, True),
                                          ("c5", 4, True), ("c5", 8, True),
                                          # more rows than one launch takes: consecutive passes of eight
                                          ("c2", 16, True), ("c2", 29, True), ("c5", 20, True), ("c5", 24, True), ("c5", 64, True)])
def test_layer_matches_oracle(name, T, fused):
    cfg, params = _layer(name)
    layer = MoELayer(cfg, params, max_tokens=max(64, T), fused=fused)
    assert (layer.fused_workspace_bytes(T) > 0) or layer._chunked_ok(T) or not fused
    x = synthetic.make_tokens(cfg, T, device="cpu").to(DEV)
    out = layer(x).clone()
    assert layer.fused_status(T) == 0
    ref, w_ref = _oracle_layer(cfg, params, x, layer.router_logits(T), layer.indices[:T])
    w_gpu = t2n(layer.weights[:T])
    if cfg.family == "generic":  # the block casts the weights to T before combining (moe_mlp.py:288)
        w_gpu = S.bf16(w_gpu)
    np.testing.assert_allclose(w_gpu, w_ref, rtol=5e-6, atol=1e-7)
    assert_close_rel(t2n(out), ref, 2e-2, f"{name} T={T}")
    # a second pass over the same tokens is bit-identical
    assert torch.equal(layer(x), out)


@pytest.mark.parametrize("name,T", [("c1", 1), ("c1", 6), ("c2", 1), ("c2", 2), ("c2", 4), ("c2", 8), ("c5", 1),
                                    ("c5", 2), ("c5", 8)])
def test_one_launch_block_agrees_with_the_separate_kernels(name, T):
    """Same routing bit for bit; outputs differ by the summation order of the K split only."""
    cfg, params = _layer(name)
    one = MoELayer(cfg, params, max_tokens=8, fused=True)
    sep = MoELayer(cfg, params, max_tokens=8, fused=False)
    x = synthetic.make_tokens(cfg, T, device="cpu").to(DEV)
    a = one(x).clone()
    b = sep(x).clone()
    assert one.fused_status(T) == 0
    assert torch.equal(one.router_logits(T), sep.router_logits(T))
    assert torch.equal(one.indices[:T], sep.indices[:T])
    assert torch.equal(one.weights[:T], sep.weights[:T])
    assert_close_rel(t2n(a), t2n(b), 2e-2, f"{name} T={T} one-launch vs separate")
    # repeated launches reuse the self-resetting barrier words
    for _ in range(3):
        assert torch.equal(one(x), a)
    assert one.fused_status(T) == 0


@pytest.mark.parametrize("name,T", [("c2", 1), ("c2", 4), ("c5", 1)])
def test_programmatic_dependent_launch_mode_gives_the_same_bits(name, T):
    """A chain of blocks launched as regular kernels that are set up while their predecessor still runs must equal
    the same chain launched cooperatively (also across repeated passes: the hand-over tags advance per launch)."""
    cfg, params = _layer(name)
    chains = {}
    for launch in ("cooperative", "pdl"):
        layers = [MoELayer(cfg, params, max_tokens=8, launch=launch) for _ in range(3)]
        x = synthetic.make_tokens(cfg, T, device="cpu").to(DEV)
        outs = []
        for _ in range(3):
            h = x
            for ly in layers:
                h = ly(h)
            outs.append(h.clone())
        torch.cuda.synchronize()
        assert all(ly.fused_status(T) == 0 for ly in layers)
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
        chains[launch] = outs[0]
    assert torch.equal(chains["cooperative"], chains["pdl"])


@pytest.mark.parametrize("norm,with_bias,T", [(False, False, 1), (True, True, 1), (False, True, 3), (True, True, 8)])
def test_one_launch_block_covers_the_softmax_then_top_k_family_with_bias(norm, with_bias, T):
    """The generic block with `norm_topk_prob` off and/or an `expert_bias` takes the full-softmax [+ bias] -> top-k
    [-> renormalise] router (moe.py:1326-1377); routing must be bit-identical to the stand-alone router kernels."""
    cfg = synthetic.CONFIGS["c1"].scaled(norm_topk_prob=norm)
    params = dict(synthetic.make_layer(cfg, device=DEV))
    if with_bias:
        g = torch.Generator(device="cpu").manual_seed(99)
        params["expert_bias"] = (torch.randn(cfg.n_experts, generator=g) * 0.01).to(DEV)
    one = MoELayer(cfg, params, max_tokens=8, fused=True)
    sep = MoELayer(cfg, params, max_tokens=8, fused=False)
    assert one._route_args()[0] == 1  # softmax-then-top-k family
    x = synthetic.make_tokens(cfg, T, device="cpu").to(DEV)
    a, b = one(x).clone(), sep(x).clone()
    assert one.fused_status(T) == 0
    assert torch.equal(one.indices[:T], sep.indices[:T])
    assert torch.equal(one.weights[:T], sep.weights[:T])
    assert_close_rel(t2n(a), t2n(b), 2e-2, f"c1 norm={norm} bias={with_bias} T={T}")


def test_one_launch_block_rejects_what_it_does_not_cover():
    cfg, params = _layer("c3")  # mxfp4
    layer = MoELayer(cfg, params, max_tokens=8)
    assert layer.fused_workspace_bytes(1) == 0
    cfg2, params2 = _layer("c2")
    layer2 = MoELayer(cfg2, params2, max_tokens=16)
    assert layer2.fused_workspace_bytes(9) == 0 and layer2.fused_workspace_bytes(8) > 0
    cfg5, params5 = _layer("c5")  # the widest shape: eight token rows leave one stage per team
    layer5 = MoELayer(cfg5, params5, max_tokens=16)
    assert layer5.fused_workspace_bytes(8) > 0 and layer5.fused_workspace_bytes(9) == 0
    assert torch.isfinite(layer5(synthetic.make_tokens(cfg5, 9, device="cpu").to(DEV)).float()).all()


def test_router_logits_match_a_float64_matmul():
    cfg, params = _layer("c2")
    layer = MoELayer(cfg, params, max_tokens=16)
    x = synthetic.make_tokens(cfg, 16, device="cpu").to(DEV)
    layer(x)
    ref = (x.double() @ params["router_w"].double().T).cpu().numpy()
    got = t2n(layer.router_logits(16))
    assert np.abs(got - ref).max() <= 2 ** -8 * np.abs(ref).max() + 1e-6


@pytest.mark.parametrize("name,T", [("c2", 1), ("c2", 4), ("c1", 8), ("c5", 1)])
def test_inbox_data_path_gives_the_same_bits(name, T):
    """The expert-parallel data path on one GPU: token rows pushed into and read from the inbox as tagged words,
    projected rows delivered through it, both launch parities -- same arithmetic, so the same bits."""
    cfg, params = _layer(name)
    plain = MoELayer(cfg, params, max_tokens=8)
    boxed = MoELayer(cfg, params, max_tokens=8, debug_force_inbox=True)
    for step in range(4):
        x = synthetic.make_tokens(cfg, T, step=step, device="cpu").to(DEV)
        a, b = plain(x).clone(), boxed(x).clone()
        assert torch.equal(a, b), f"step {step}"
        assert torch.equal(plain.indices[:T], boxed.indices[:T]) and torch.equal(plain.weights[:T], boxed.weights[:T])
    boxed.check_status()


def test_block_loaded_from_an_mlx_format_checkpoint_gives_the_same_bits(tmp_path):
    """safetensors under the mlx-community names -> `checkpoint.load_moe_params` -> `MoELayer`: same output as the
    layer built from the tensors that were written."""
    from zmlx_b200 import checkpoint

    cfg = synthetic.CONFIGS["c5"].scaled(n_experts=32, d_model=512, d_ff=256, top_k=4, n_group=4, topk_group=2)
    params = synthetic.make_layer(cfg, device=DEV)
    checkpoint.save_moe_params(params, str(tmp_path / "model.safetensors"), "model.layers.7.mlp")
    loaded = checkpoint.load_moe_params(str(tmp_path), checkpoint.moe_block_prefixes(str(tmp_path))[0], device=DEV)
    x = synthetic.make_tokens(cfg, 3, device="cpu").to(DEV)
    a = MoELayer(cfg, params, max_tokens=8)(x).clone()
    b = MoELayer(cfg, loaded, max_tokens=8)(x).clone()
    assert torch.equal(a, b)
