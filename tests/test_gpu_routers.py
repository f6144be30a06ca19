"""GPU parity: router kernels against the oracle and the reference's known answers."""

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import expand_bias, expand_logits, golden_cases, t2n
from zmlx_b200.kernels import moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sorted_pairs(idx, w):
    order = np.argsort(idx.astype(np.int64), axis=-1, kind="stable")
    return np.take_along_axis(idx, order, -1), np.take_along_axis(w, order, -1)


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_known_answers(case):
    logits = torch.from_numpy(expand_logits(case)).to(DEV)
    if case["router"] == "sigmoid":
        w, idx = moe.deepseek_router_topk_sigmoid(logits, torch.from_numpy(expand_bias(case)).to(DEV), k=case["k"],
                                                  n_group=case["n_group"], topk_group=case["topk_group"])
    else:
        w, idx = moe.topk_gating_softmax(logits, case["k"])
    assert idx.dtype == torch.uint32 and w.dtype == torch.float32
    np.testing.assert_array_equal(t2n(idx), np.asarray(case["indices"], dtype=np.uint32))
    if case.get("weights") is not None:
        np.testing.assert_array_equal(t2n(w), np.asarray(case["weights"], dtype=np.float32))
    if case.get("weights_sum_to_one"):
        np.testing.assert_allclose(t2n(w).sum(-1), 1.0, rtol=1e-6)


@pytest.mark.parametrize("E,k", [(32, 4), (128, 8), (64, 4), (256, 8), (384, 8), (1000, 16), (8, 8)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_family_matches_oracle(E, k, dtype):
    g = torch.Generator().manual_seed(E * 31 + k)
    logits = (torch.randn((37, E), generator=g) * 2).to(dtype)
    ln = t2n(logits)
    lg = logits.to(DEV)
    bias = torch.randn((E,), generator=g) * 0.01
    # top-k of logits then softmax (exact selection: compares logits only)
    w, idx = moe.topk_gating_softmax(lg, k)
    wr, ir = S.topk_gating_softmax(ln, k)
    np.testing.assert_array_equal(t2n(idx), ir)
    np.testing.assert_allclose(t2n(w), wr, rtol=2e-6, atol=1e-7)
    s, i2 = moe.router_argpartition_logits_topk(lg, k=k)
    np.testing.assert_array_equal(t2n(i2), ir)
    # full softmax -> top-k (selection on probabilities), with and without renormalisation / bias
    for kw in ({"norm_topk_prob": False}, {"expert_bias": bias, "norm_topk_prob": True},
               {"expert_bias": bias, "norm_topk_prob": False}):
        w, idx = moe.topk_gating_softmax(lg, k, **{kk: (v.to(DEV) if torch.is_tensor(v) else v) for kk, v in kw.items()})
        kwn = {kk: (t2n(v) if torch.is_tensor(v) else v) for kk, v in kw.items()}
        wr, ir = S.topk_gating_softmax(ln, k, **kwn)
        a_i, a_w = _sorted_pairs(t2n(idx), t2n(w))
        r_i, r_w = _sorted_pairs(ir, wr)
        np.testing.assert_array_equal(a_i, r_i)
        np.testing.assert_allclose(a_w, r_w, rtol=5e-6, atol=1e-7)
    ii, ss = moe.qwen3_gating(lg, k)
    ir, sr = S.qwen3_gating(ln, k)
    np.testing.assert_array_equal(t2n(ii), ir)
    np.testing.assert_allclose(t2n(ss), sr, rtol=5e-6, atol=1e-7)


def test_bf16_logit_ties_break_to_the_lower_id():
    # bf16 logits from a linear layer collide often; the canonical order must hold on exact ties
    g = torch.Generator().manual_seed(9)
    logits = (torch.randn((256, 128), generator=g) * 0.25).to(torch.bfloat16)
    ln = t2n(logits)
    ties = 0
    for row in ln:
        srt = np.sort(row)[::-1]
        ties += int(srt[7] == srt[8])
    assert ties > 0, "the generator should produce boundary ties"
    w, idx = moe.topk_gating_softmax(logits.to(DEV), 8)
    _, ir = S.topk_gating_softmax(ln, 8)
    np.testing.assert_array_equal(t2n(idx), ir)


@pytest.mark.parametrize("E,k,n_group,topk_group", [(64, 4, 1, 1), (256, 8, 8, 4), (384, 8, 8, 4), (256, 8, 1, 1),
                                                    (160, 6, 8, 3), (256, 8, 8, 8)])
def test_sigmoid_router_matches_oracle(E, k, n_group, topk_group):
    g = torch.Generator().manual_seed(E + k)
    logits = (torch.randn((29, E), generator=g) * 1.5).to(torch.bfloat16)
    bias = torch.randn((E,), generator=g) * 0.01
    w, idx = moe.deepseek_router_topk_sigmoid(logits.to(DEV), bias.to(DEV), k=k, n_group=n_group,
                                              topk_group=topk_group)
    wr, ir = S.deepseek_router_topk_sigmoid(t2n(logits), t2n(bias), k=k, n_group=n_group, topk_group=topk_group)
    # Slot order is part of the contract (score descending, expert id ascending): compared slot by slot.
    # expf on the device and np.exp may differ in the last bit of a score, so rows in which two of the oracle's
    # k+1 best scores lie within 2 ulp of each other are compared as sets instead (and counted).
    scores = S.sigmoid_stable(t2n(logits)) + t2n(bias)
    gi, ri = t2n(idx).astype(np.int64), ir.astype(np.int64)
    near = 0
    for r in range(gi.shape[0]):
        top = np.sort(scores[r].astype(np.float32))[::-1][:k + 1]
        gaps = np.abs(np.diff(top)) <= 2 * np.spacing(np.abs(top[:-1]).astype(np.float32))
        if gaps.any() or n_group > 1:
            # group-limited rows zero the scores of dropped groups; near-ties there show up as set differences only
            near += int(gaps.any())
            np.testing.assert_array_equal(np.sort(gi[r]), np.sort(ri[r]))
            if not gaps.any():
                np.testing.assert_array_equal(gi[r], ri[r])
        else:
            np.testing.assert_array_equal(gi[r], ri[r])
    assert near <= gi.shape[0] // 2, f"{near} of {gi.shape[0]} rows are near-ties: the generator is degenerate"
    a_i, a_w = _sorted_pairs(t2n(idx), t2n(w))
    r_i, r_w = _sorted_pairs(ir, wr)
    np.testing.assert_allclose(a_w, r_w, rtol=2e-6, atol=1e-7)
    w2, _ = moe.deepseek_router_topk_sigmoid(logits.to(DEV), bias.to(DEV), k=k, n_group=n_group,
                                             topk_group=topk_group, routed_scaling_factor=2.5)
    np.testing.assert_array_equal(t2n(w2), (t2n(w) * np.float32(2.5)).astype(np.float32))


def test_nan_rows_rank_last_and_never_index_out_of_range():
    """A row of NaN logits (NaN activations upstream) must not make the router read or write out of range: NaN
    scores rank below every number, among themselves by ascending id, like the oracle's stable argsort."""
    E, k = 64, 4
    logits = torch.randn((3, E))
    logits[1] = float("nan")      # whole row NaN -> ids 0..k-1
    logits[2, 5:60] = float("nan")  # most of a row NaN -> the finite ones win
    for fn, args in ((moe.topk_gating_softmax, {}),):
        w, idx = fn(logits.to(DEV), k, **args)
        ii = t2n(idx).astype(np.int64)
        assert ii.min() >= 0 and ii.max() < E
        np.testing.assert_array_equal(ii[1], np.arange(k))
        assert set(ii[2]).issubset(set(range(5)) | set(range(60, 64)))
    bias = torch.zeros(E)
    w, idx = moe.deepseek_router_topk_sigmoid(logits.to(DEV), bias.to(DEV), k=k)
    ii = t2n(idx).astype(np.int64)
    assert ii.min() >= 0 and ii.max() < E
    np.testing.assert_array_equal(ii[1], np.arange(k))
    _, ir = S.topk_gating_softmax(t2n(logits), k)
    np.testing.assert_array_equal(t2n(moe.topk_gating_softmax(logits.to(DEV), k)[1]), ir)


def test_leading_dims_and_empty_batch():
    logits = torch.randn((2, 3, 32), device=DEV)
    w, idx = moe.topk_gating_softmax(logits, 4)
    assert w.shape == (2, 3, 4) and idx.shape == (2, 3, 4)
    w, idx = moe.topk_gating_softmax(torch.zeros((0, 32), device=DEV), 4)
    assert w.shape == (0, 4) and idx.shape == (0, 4)
