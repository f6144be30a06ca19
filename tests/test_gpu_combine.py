"""GPU parity: combine kernels, bit-exact against the oracle's rounding contracts."""

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import t2n
from zmlx_b200.kernels import moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(B, K, D, seed):
    g = torch.Generator().manual_seed(seed)
    y = torch.randn((B, K, D), generator=g).to(torch.bfloat16)
    w = torch.randn((B, K), generator=g)
    return y, w


@pytest.mark.parametrize("B,K,D", [(3, 4, 64), (1, 8, 2048), (16, 4, 2048), (5, 2, 1023), (64, 8, 7168), (2, 1, 16)])
def test_contracts_bit_exact(B, K, D):
    y, w = _case(B, K, D, B * 100 + K)
    yn, wn = t2n(y), t2n(w)
    yg, wg = y.to(DEV), w.to(DEV)
    # product rounded before the add: bit-exact in every dtype combination
    np.testing.assert_array_equal(t2n(moe.moe_combine_fp32_no_fma(yg, wg)), S.moe_combine(yn, wn, mode="fp32_no_fma"))
    np.testing.assert_array_equal(t2n(moe.moe_combine_no_fma(yg, wg)), S.moe_combine(yn, wn, mode="no_fma"))
    wb = wg.to(torch.bfloat16)
    np.testing.assert_array_equal(t2n(moe.moe_combine_exact(yg, wb)), S.moe_combine(yn, t2n(wb), mode="exact"))
    # contraction allowed: within float32 rounding of the ordered sum
    np.testing.assert_allclose(t2n(moe.moe_combine_fp32(yg, wg)), S.moe_combine(yn, wn, mode="fp32"), rtol=1e-3,
                               atol=1e-5)
    out_t = t2n(moe.moe_combine(yg, wg))
    ref_t = S.moe_combine(yn, wn, mode="t")
    assert (out_t != ref_t).mean() < 0.01 and np.abs(out_t - ref_t).max() <= 2 ** -7 * np.abs(ref_t).max()


def test_no_fma_equals_multiply_then_sum_in_torch():
    # the reference pins moe_combine_no_fma bit-exactly to (y * w[..., None]).sum(-2).astype(T)
    # (tests/test_fused_ops.py:349-362); restate that with an ordered float32 loop
    y, w = _case(3, 4, 64, 0)
    acc = torch.zeros((3, 64))
    for i in range(4):
        acc = acc + y[:, i].float() * w[:, i, None]
    got = moe.moe_combine_no_fma(y.to(DEV), w.to(DEV)).cpu()
    assert torch.equal(got, acc.to(torch.bfloat16))
    y32 = y.float()
    got32 = moe.moe_combine_no_fma(y32.to(DEV), w.to(DEV)).cpu()
    assert got32.dtype == torch.float32 and torch.equal(got32, acc)


def test_identities_and_shapes():
    y, w = _case(6, 4, 128, 3)
    onehot = torch.zeros((6, 4))
    pick = torch.tensor([0, 3, 1, 2, 2, 0])
    onehot[torch.arange(6), pick] = 1.0
    for fn in (moe.moe_combine, moe.moe_combine_no_fma, moe.moe_combine_exact):
        out = fn(y.to(DEV), onehot.to(DEV)).cpu()
        assert torch.equal(out, y[torch.arange(6), pick])
    out = moe.moe_combine_fp32(y.reshape(2, 3, 4, 128).to(DEV), w.reshape(2, 3, 4).to(DEV))
    assert out.shape == (2, 3, 128) and out.dtype == torch.float32
    assert moe.moe_dispatch(y[:, 0].to(DEV), torch.zeros((6, 4), device=DEV)).shape == (6, 4, 128)
    empty = moe.moe_combine(torch.zeros((0, 4, 128), dtype=torch.bfloat16, device=DEV), torch.zeros((0, 4), device=DEV))
    assert empty.shape == (0, 128)


def test_determinism():
    y, w = _case(16, 8, 2048, 5)
    a = moe.moe_combine_fp32_no_fma(y.to(DEV), w.to(DEV))
    b = moe.moe_combine_fp32_no_fma(y.to(DEV), w.to(DEV))
    assert torch.equal(a, b)
