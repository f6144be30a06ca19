"""CPU: the compiled oracle (C) against the NumPy restatement."""

import numpy as np
import pytest
import torch

from oracle import fast as F
from oracle import semantics as S
from tests.helpers import assert_close_rel, t2n
from zmlx_b200 import quant


def _bank(E, N, K, mode, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((E, N, K), generator=g) * 0.02
    if mode == "affine":
        p, s, b = quant.quantize_affine(w, 64)
        return t2n(p), t2n(s), t2n(b)
    p, s = quant.quantize_mxfp4(w)
    return t2n(p), t2n(s), None


@pytest.mark.parametrize("mode", ["affine", "mxfp4"])
def test_gather_qmm_matches_numpy(mode):
    E, N, K, R = 6, 40, 256, 5
    w, s, b = _bank(E, N, K, mode, 11)
    rng = np.random.default_rng(5)
    x = S.bf16(rng.standard_normal((R, K)).astype(np.float32))
    lhs = np.array([0, 1, 1, 4, 3, 2, 0], dtype=np.int32)
    rhs = np.array([5, 0, 0, 2, 2, 1, 3], dtype=np.int32)
    got = F.gather_qmm_rows(x, w, s, b, lhs, rhs, mode=mode, group_size=64)
    ref = S.gather_qmm(x[:, None, :], w, s, b, lhs_indices=lhs, rhs_indices=rhs, mode=mode, group_size=64)[:, 0, :]
    # both round to bfloat16; float32 vs float64 accumulation may flip a last bit
    assert_close_rel(got, ref, 2 ** -7, "compiled vs numpy gather_qmm")
    assert (got != ref).mean() < 0.05


def test_swiglu_contract_matches_numpy():
    rng = np.random.default_rng(6)
    g = S.bf16(rng.standard_normal(5000).astype(np.float32) * 3)
    u = S.bf16(rng.standard_normal(5000).astype(np.float32))
    a = F.swiglu_cpu_contract(g, u)
    b = S.swiglu_cpu_contract(g, u)
    assert (a != b).mean() < 0.01  # expf vs np.exp may differ in the last float32 bit before rounding
    assert_close_rel(a, b, 2 ** -7, "swiglu")


def test_bad_index_is_rejected():
    w, s, b = _bank(2, 8, 64, "affine", 1)
    x = np.zeros((1, 64), dtype=np.float32)
    with pytest.raises(IndexError):
        F.gather_qmm_rows(x, w, s, b, np.array([0]), np.array([2]))


def test_quantiser_round_trip():
    g = torch.Generator().manual_seed(3)
    w = torch.randn((3, 16, 128), generator=g) * 0.02
    p, s, b = quant.quantize_affine(w, 64)
    assert p.dtype == torch.uint32 and p.shape == (3, 16, 16) and s.shape == (3, 16, 2) and s.dtype == torch.bfloat16
    deq = quant.dequantize_affine(p, s, b, 64)
    np.testing.assert_array_equal(t2n(deq), S.dequant_affine(t2n(p), t2n(s), t2n(b), 64))
    step = s.to(torch.float32).repeat_interleave(64, -1)
    assert ((deq - w).abs() <= 0.51 * step + 1e-4).all()
    p4, e8 = quant.quantize_mxfp4(w)
    assert e8.dtype == torch.uint8 and e8.shape == (3, 16, 4)
    deq4 = quant.dequantize_mxfp4(p4, e8)
    np.testing.assert_array_equal(t2n(deq4), S.dequant_mxfp4(t2n(p4), t2n(e8)))
    assert (deq4 - w).abs().max() <= 0.02 * 6  # coarse: within the fp4 grid of the group
    np.testing.assert_array_equal(t2n(quant.unpack_u4(p)), S.unpack_u4(t2n(p)))
