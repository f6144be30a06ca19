"""GPU parity: patch(model) on torch blocks -- patched output vs the oracle's recipe and vs the unpatched block."""

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import assert_close_rel, params_to_numpy, t2n
from zmlx_b200 import nn as znn
from zmlx_b200 import synthetic
from zmlx_b200.patch import patch, unpatch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _Model(torch.nn.Module):
    def __init__(self, blk):
        super().__init__()
        self.layers = torch.nn.ModuleList([blk])


@pytest.mark.parametrize("base,family", [("c2", "qwen3"), ("c5", "deepseek"), ("c5", "glm")])
def test_patched_block_matches_oracle_and_unpatched(base, family):
    cfg = synthetic.CONFIGS[base].scaled(n_experts=16, d_model=256, d_ff=128, top_k=4, n_group=4 if family != "qwen3" else 1,
                                         topk_group=2 if family != "qwen3" else 1, family=family)
    p = synthetic.make_layer(cfg, device=DEV)
    blk = znn.block_from_params(cfg, p)
    m = _Model(blk)
    x = synthetic.make_tokens(cfg, 6, device="cpu").reshape(2, 3, cfg.d_model).to(DEV)
    y_ref_torch = blk(x)
    patch(m)
    assert m._zmlx_patch_result.patched_count == 1
    y = blk(x)
    assert y.shape == x.shape and y.dtype == torch.bfloat16
    pn = params_to_numpy(p)
    xn = t2n(x).reshape(6, cfg.d_model)
    logits = S.bf16(t2n((x.reshape(6, -1) @ p["router_w"].T)))
    ref, _, _ = S.moe_layer(xn, logits, pn, family=family, top_k=cfg.top_k, expert_bias=pn["expert_bias"],
                            n_group=cfg.n_group, topk_group=cfg.topk_group,
                            routed_scaling_factor=cfg.routed_scaling_factor, shared=pn["shared"])
    assert_close_rel(t2n(y).reshape(6, -1), ref, 2e-2, f"patched {family} block vs oracle")
    assert_close_rel(t2n(y), t2n(y_ref_torch), 3e-2, "patched vs unpatched torch block")
    unpatch(m)
    assert torch.equal(blk(x), y_ref_torch)
