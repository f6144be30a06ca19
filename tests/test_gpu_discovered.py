"""GPU parity of the elementwise SwiGLU and of the GLM shape specialisations
(src/zmlx/kernels/transformer.py:925-1005, src/zmlx/kernels/discovered/*.py) against the oracle."""

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import t2n
from zmlx_b200.kernels import discovered, moe, transformer

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _bf(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


@pytest.mark.parametrize("shape", [(1, 1536), (3, 4, 1536), (5, 768), (1, 7), (0, 1536)])
def test_swiglu2_is_bit_exact_against_the_per_op_contract(shape):
    gate, up = _bf(shape, 1, 2.0), _bf(shape, 2)
    got = transformer.swiglu2(gate, up)
    assert got.shape == gate.shape and got.dtype == torch.bfloat16
    want = S.swiglu_per_op(t2n(gate), t2n(up))
    np.testing.assert_array_equal(t2n(got), want)
    if shape[-1] == 1536:
        assert torch.equal(discovered.glm_fused_swiglu(gate, up), got)
    else:
        assert discovered.glm_fused_swiglu(gate, up) is None


def test_swiglu2_rejects_mismatched_shapes_and_warns_on_compute_dtype():
    with pytest.raises(ValueError):
        transformer.swiglu2(_bf((2, 8), 1), _bf((2, 16), 2))
    with pytest.warns(DeprecationWarning):
        transformer.swiglu2(_bf((2, 8), 1), _bf((2, 8), 2), compute_dtype=torch.float32)


@pytest.mark.parametrize("same_dtype", [True, False])
def test_glm_moe_combine_contracts(same_dtype):
    y = _bf((6, 4, 2048), 3)
    g = torch.Generator().manual_seed(4)
    w = torch.rand((6, 4), generator=g).to(DEV)
    if same_dtype:
        w = w.to(torch.bfloat16)
        want = S.moe_combine(t2n(y), t2n(w), mode="exact")
    else:
        want = S.bf16(S.moe_combine(t2n(y), t2n(w), mode="fp32_no_fma"))
    got = discovered.glm_moe_combine(y, w)
    assert got.dtype == torch.bfloat16 and got.shape == (6, 2048)
    np.testing.assert_array_equal(t2n(got), want)
    assert discovered.glm_moe_combine(_bf((2, 4, 1024), 5), w[:2]) is None
    assert discovered.glm_moe_combine(_bf((2, 2, 2048), 5), w[:2, :2]) is None


def test_glm_topk_gating_returns_indices_then_weights():
    logits = _bf((9, 64), 6, 3.0)
    out = discovered.glm_topk_gating(logits, 4)
    idx, w = out
    w_ref, idx_ref = S.topk_gating_softmax(t2n(logits), 4)
    np.testing.assert_array_equal(t2n(idx).view(np.uint32), idx_ref)
    assert w.dtype == torch.bfloat16
    np.testing.assert_allclose(t2n(w), w_ref, rtol=2 ** -7, atol=0)  # weights are cast to the logits' dtype
    assert discovered.glm_topk_gating(_bf((9, 128), 6), 4) is None
    assert discovered.glm_topk_gating(logits, 2) is None
    w2, i2 = moe.topk_gating_softmax(logits, 4)
    assert torch.equal(i2, idx)
