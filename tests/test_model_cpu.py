"""CPU checks of the stacked decode model's host side and of its restatement."""

import numpy as np
import pytest
import torch

from oracle import model as OM
from tests.helpers import t2n
from zmlx_b200 import synthetic
from zmlx_b200.model import (DECODER_CONFIGS, DecoderConfig, StackedDecoder, apply_rope, attention,
                             make_decoder_params, rms_norm, rope_tables)


def _tonp(tree):
    if isinstance(tree, dict):
        return {k: _tonp(v) for k, v in tree.items()}
    if isinstance(tree, list):
        return [_tonp(v) for v in tree]
    return None if tree is None else t2n(tree)


def _tiny():
    moe = synthetic.CONFIGS["c2"].scaled(d_model=128, n_experts=8, top_k=2, d_ff=128)
    return DecoderConfig("tiny", 2, 128, 4, 2, 32, 256, moe=moe)


def test_benchmark_configuration_shapes():
    c = DECODER_CONFIGS["c4"]
    assert (c.n_layers, c.d_model, c.n_heads, c.n_kv_heads, c.head_dim, c.rope_theta) == (48, 2048, 32, 4, 128, 1e6)
    assert (c.moe.n_experts, c.moe.top_k, c.moe.d_ff, c.moe.family) == (128, 8, 768, "qwen3")


def test_restatement_is_causal_and_deterministic():
    cfg = _tiny()
    p = _tonp(make_decoder_params(cfg, device="cpu"))
    ids = np.array([[3, 7, 11, 200, 5]])
    a = OM.forward_logits(cfg, p, ids)
    b = OM.forward_logits(cfg, p, ids)
    assert np.array_equal(a, b)
    # the logits after 3 tokens do not depend on what follows
    c = OM.forward_logits(cfg, p, ids[:, :3])
    ids2 = ids.copy()
    ids2[0, 3:] = [9, 9]
    toks, _ = OM.greedy(cfg, p, ids[:, :3], 2)
    assert toks.shape == (1, 2) and toks[0, 0] == c.argmax(-1)[0]


def test_torch_attention_pieces_match_the_restatement():
    cfg = _tiny()
    g = torch.Generator().manual_seed(1)
    x = torch.randn((2, 4, 6, 32), generator=g).to(torch.bfloat16)
    w = torch.ones(32, dtype=torch.bfloat16)
    np.testing.assert_allclose(t2n(rms_norm(x, w, 1e-6)), OM._rms(t2n(x), t2n(w), 1e-6), rtol=0, atol=2 ** -7)
    cos, sin = rope_tables(32, 16, 1e6, "cpu")
    got = t2n(apply_rope(x, cos[2:8], sin[2:8]))
    want = OM._rope(t2n(x), np.arange(2, 8), 1e6)
    np.testing.assert_allclose(got, want, rtol=0, atol=2 ** -6)
    # grouped-query attention against an explicit per-head loop
    q = torch.randn((1, 4, 3, 32), generator=g).to(torch.bfloat16)
    k = torch.randn((1, 2, 5, 32), generator=g).to(torch.bfloat16)
    v = torch.randn((1, 2, 5, 32), generator=g).to(torch.bfloat16)
    out = attention(q, k, v, 2).float()
    for h in range(4):
        for s in range(3):
            sc = (q[0, h, s].float() @ k[0, h // 2].float().T) / np.sqrt(32)
            sc[(2 + s + 1):] = float("-inf")
            ref = torch.softmax(sc, -1) @ v[0, h // 2].float()
            assert torch.allclose(out[0, h, s], ref, atol=2e-2)


def test_the_model_refuses_cpu_tensors():
    cfg = _tiny()
    with pytest.raises(RuntimeError):
        StackedDecoder(cfg, make_decoder_params(cfg, device="cpu"), max_batch=1, max_seq=8)
