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
    # the block itself, and -- as in the reference's default selection -- its dense shared expert (swiglu_mlp)
    want = {"moe_mlp": 1, "swiglu_mlp": 1} if cfg.n_shared else {"moe_mlp": 1}
    assert m._zmlx_patch_result.pattern_counts == want
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


@pytest.mark.parametrize("name,T", [("c2", 1), ("c2", 4), ("c5", 1)])
def test_patched_block_is_one_launch_and_matches_the_oracle(name, T):
    """patch(model) must reach the one-launch kernel: the workspace's launch counter advances by exactly one per
    call of the patched block, and the result follows the oracle's recipe for the block's family."""
    from tests.helpers import oracle_layer

    cfg = synthetic.CONFIGS[name]
    p = synthetic.make_layer(cfg, device=DEV)
    blk = znn.block_from_params(cfg, p)
    m = _Model(blk)
    patch(m)
    fast = blk._zmlx_fast_layer
    assert fast is not None, "the moe_mlp pattern did not build the fused layer for a supported block"
    x = synthetic.make_tokens(cfg, T, device="cpu").reshape(1, T, cfg.d_model).to(DEV)
    y0 = blk(x)  # the first call creates the workspace
    before = fast.launch_count(T)
    y = blk(x)
    torch.cuda.synchronize()
    assert fast.launch_count(T) == before + 1, "a patched call must be exactly one zmoe_layer_decode launch"
    fast.check_status()
    assert y.data_ptr() != y0.data_ptr() and torch.equal(y, y0)  # fresh result tensors, same bits
    ref, _ = oracle_layer(cfg, p, x.reshape(T, -1), fast.router_logits(T), fast.indices[:T])
    assert_close_rel(t2n(y).reshape(T, -1), ref, 2e-2, f"patched {name} block T={T} vs oracle")
    unpatch(m)
    assert not hasattr(blk, "_zmlx_fast_layer")


def test_deepseek_router_pattern_fires_on_a_256_expert_gate():
    """The opt-in deepseek_router pattern (reference: src/zmlx/patch/patterns/deepseek_router.py:76-120) rewrites
    MoEGate for 256 experts with k = 8: indices int32 in canonical order, weights = normalised affinities * scale."""
    cfg = synthetic.CONFIGS["c5"]
    g = torch.Generator(device="cpu").manual_seed(5)
    wr = (torch.randn((cfg.n_experts, 512), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    bias = (torch.randn((cfg.n_experts,), generator=g) * 0.01).to(DEV)
    gate = znn.MoEGate(wr, bias, top_k=8, n_group=8, topk_group=4, routed_scaling_factor=2.5)
    m = _Model(gate)
    x = torch.randn((3, 5, 512), generator=g).to(torch.bfloat16).to(DEV)
    idx_ref, w_ref = gate(x)
    patch(m, patterns=["deepseek_router"])
    assert m._zmlx_patch_result.patched_count == 1
    idx, w = gate(x)
    assert idx.dtype == torch.int32 and w.dtype == torch.float32, "the fused router did not run"
    logits = t2n(x.reshape(15, -1) @ wr.T)
    w_o, idx_o = S.deepseek_router_topk_sigmoid(logits, t2n(bias), k=8, n_group=8, topk_group=4)
    np.testing.assert_array_equal(t2n(idx).reshape(15, 8).view(np.uint32), idx_o)
    np.testing.assert_allclose(t2n(w).reshape(15, 8), w_o * np.float32(2.5), rtol=5e-6, atol=1e-7)
    # the unpatched gate picks the same experts (as sets: torch.topk orders ties differently)
    assert np.array_equal(np.sort(t2n(idx_ref).reshape(15, 8), -1), np.sort(t2n(idx).reshape(15, 8), -1))
    unpatch(m)


@pytest.mark.parametrize("T", [1, 5, 64])
def test_dense_swiglu_mlp_pattern_matches_the_fused_gemv_restatement(T):
    """The `swiglu_mlp` pattern on a dense quantised MLP (a one-expert bank): gate/up + SwiGLU in one kernel with
    gate and up kept in float (the contract of src/zmlx/kernels/quant.py:103-124), then the quantised down
    projection; T = 64 takes the tensor-memory matmul."""
    cfg = synthetic.CONFIGS["c3"].scaled(mode="affine", group_size=64)  # d 2048, f 1536, one shared expert
    p = synthetic.make_layer(cfg, device=DEV)["shared"]
    mlp = znn.mlp_from_params(p).to(DEV)

    class _M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.mlp = mlp

    m = _M()
    patch(m, patterns=["swiglu_mlp"])
    assert m._zmlx_patch_result.pattern_counts == {"swiglu_mlp": 1}
    x = synthetic.make_tokens(cfg, T, device="cpu").to(DEV)
    got = m.mlp(x.reshape(1, T, -1)).reshape(T, -1)
    pn = params_to_numpy(p)
    h = S.fused_quantized_swiglu_gemv(t2n(x), pn["gate_w"][0], pn["gate_s"][0], pn["gate_b"][0], pn["up_w"][0],
                                      pn["up_s"][0], pn["up_b"][0])
    ref = S.gather_qmm(h[:, None, :], pn["down_w"], pn["down_s"], pn["down_b"],
                       rhs_indices=np.zeros(T, dtype=np.uint32))[:, 0, :]
    assert_close_rel(t2n(got), ref, 2e-2, f"dense MLP T={T}")
    unpatch(m)
    assert type(m.mlp) is znn.MLP
    assert_close_rel(t2n(m.mlp(x)), ref, 3e-2, f"stock dense MLP T={T}")  # torch ops round op by op in bfloat16
