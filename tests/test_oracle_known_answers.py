"""CPU: the oracle against the reference's known-answer cases and identities."""

import numpy as np
import pytest

from oracle import semantics as S
from tests.helpers import expand_bias, expand_logits, golden_cases


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c["name"])
def test_router_known_answers(case):
    logits = expand_logits(case)
    if case["router"] == "sigmoid":
        w, idx = S.deepseek_router_topk_sigmoid(logits, expand_bias(case), k=case["k"], n_group=case["n_group"],
                                                topk_group=case["topk_group"])
    else:
        w, idx = S.topk_gating_softmax(logits, case["k"])
    assert idx.dtype == np.uint32
    np.testing.assert_array_equal(idx, np.asarray(case["indices"], dtype=np.uint32))
    if case.get("weights") is not None:
        if case.get("weights_exact"):
            np.testing.assert_array_equal(w, np.asarray(case["weights"], dtype=np.float32))
        else:
            np.testing.assert_allclose(w, np.asarray(case["weights"], dtype=np.float32), rtol=1e-6, atol=1e-7)
    if case.get("weights_sum_to_one"):
        np.testing.assert_allclose(w.sum(-1), 1.0, rtol=1e-6)


def test_router_validation_messages():
    z = np.zeros((1, 8), dtype=np.float32)
    with pytest.raises(ValueError, match="k must be > 0"):
        S.topk_gating_softmax(z, 0)
    with pytest.raises(ValueError, match="exceeds last dimension"):
        S.topk_gating_softmax(z, 9)
    with pytest.raises(ValueError, match="invalid topk_group"):
        S.deepseek_router_topk_sigmoid(z, np.zeros(8, np.float32), k=2, n_group=2, topk_group=3)
    with pytest.raises(ValueError, match="n_group must divide D"):
        S.deepseek_router_topk_sigmoid(z, np.zeros(8, np.float32), k=2, n_group=3, topk_group=1)


def test_softmax_router_flavours_agree_on_the_set():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((16, 64)).astype(np.float32)
    w1, i1 = S.topk_gating_softmax(x, 4)  # top-k logits then softmax
    w2, i2 = S.topk_gating_softmax(x, 4, norm_topk_prob=True, expert_bias=np.zeros(64, np.float32))
    np.testing.assert_array_equal(i1, i2)
    np.testing.assert_allclose(w1, w2, rtol=2e-6)  # softmax over k == renormalised full softmax
    i3, w3 = S.qwen3_gating(x, 4)
    np.testing.assert_array_equal(i1, i3)
    np.testing.assert_allclose(w1, w3, rtol=2e-6)
    w4, _ = S.topk_gating_softmax(x, 4, norm_topk_prob=False)
    assert (w4.sum(-1) < 1.0).all()


def test_packed_layout_statement():
    # code i of a row is (word[i/8] >> 4*(i%8)) & 0xF  (src/zmlx/kernels/quant.py:109-113)
    w = np.array([[0x76543210, 0xFEDCBA98]], dtype=np.uint32)
    np.testing.assert_array_equal(S.unpack_u4(w)[0], np.arange(16))
    np.testing.assert_array_equal(S.pack_u4(np.arange(16)[None]), w)
    s = np.array([[0.5]], dtype=np.float32)
    b = np.array([[-1.0]], dtype=np.float32)
    np.testing.assert_array_equal(S.dequant_affine(w, s, b, 16)[0], np.arange(16) * 0.5 - 1.0)


def test_mxfp4_codes():
    codes = np.arange(16)[None]
    w = S.pack_u4(np.concatenate([codes, codes], axis=-1))  # 32 codes
    v = S.dequant_mxfp4(w, np.array([[128]], dtype=np.uint8))  # scale 2
    expect = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32) * 2
    np.testing.assert_array_equal(v[0, :16], expect)
    np.testing.assert_array_equal(v[0, 16:], expect)


def test_combine_identities():
    rng = np.random.default_rng(1)
    y = S.bf16(rng.standard_normal((5, 4, 32)).astype(np.float32))
    onehot = np.zeros((5, 4), dtype=np.float32)
    onehot[np.arange(5), [0, 1, 2, 3, 1]] = 1.0
    for mode in ("fp32", "fp32_no_fma", "t", "no_fma", "exact", "stream_t"):
        out = S.moe_combine(y, onehot, mode=mode)
        np.testing.assert_array_equal(out, y[np.arange(5), [0, 1, 2, 3, 1]])  # one-hot gate picks a slot exactly
    w = rng.standard_normal((5, 1)).astype(np.float32)
    np.testing.assert_array_equal(S.moe_combine(y[:, :1], w, mode="fp32_no_fma"), w * y[:, 0])  # K = 1
    # no_fma == (y * w[..., None]).sum(-2).astype(T) with float32 weights (tests/test_fused_ops.py:349-362)
    w4 = rng.standard_normal((5, 4)).astype(np.float32)
    ref = np.zeros((5, 32), dtype=np.float32)
    for i in range(4):
        ref = (ref + (y[:, i] * w4[:, i, None]).astype(np.float32)).astype(np.float32)
    np.testing.assert_array_equal(S.moe_combine(y, w4, mode="no_fma"), S.bf16(ref))


def test_bf16_rounding_is_nearest_even():
    import ml_dtypes

    rng = np.random.default_rng(2)
    x = (rng.standard_normal(10000) * np.exp(rng.uniform(-20, 20, 10000))).astype(np.float32)
    np.testing.assert_array_equal(S.bf16(x), x.astype(ml_dtypes.bfloat16).astype(np.float32))
    np.testing.assert_array_equal(S.from_bf16_bits(S.bf16_bits(x)), S.bf16(x))


def test_swiglu_contracts_differ_only_in_rounding():
    rng = np.random.default_rng(3)
    g = S.bf16(rng.standard_normal(4096).astype(np.float32) * 2)
    u = S.bf16(rng.standard_normal(4096).astype(np.float32))
    a = S.swiglu_cpu_contract(g, u)
    b = S.swiglu_per_op(g, u)
    exact = g / (1 + np.exp(-g.astype(np.float64))) * u
    assert np.abs(a - exact).max() <= 2 ** -8 * np.abs(exact).max()
    assert np.abs(b - exact).max() <= 4 * 2 ** -8 * np.abs(exact).max()


def test_nan_scores_rank_below_every_number():
    """Pinned tie/NaN rule of the canonical order: NaN scores come last, among themselves by ascending id
    (what a stable descending argsort gives); the GPU routers use the same total order."""
    import numpy as np

    from oracle import semantics as S

    row = np.array([[0.5, np.nan, -np.inf, 2.0, np.nan, 0.5]], dtype=np.float32)
    np.testing.assert_array_equal(S._topk_desc_stable(row, 6), [[3, 0, 5, 2, 1, 4]])
    _, idx = S.topk_gating_softmax(np.full((1, 8), np.nan, dtype=np.float32), 3)
    np.testing.assert_array_equal(idx, [[0, 1, 2]])


def test_dense_fused_gemv_restatement_against_a_scalar_loop():
    """`fused_quantized_swiglu_gemv` (src/zmlx/kernels/quant.py:103-124) as the kernel source spells it: one scalar
    loop per output element, dequantising code by code, float accumulators, `acc_gate * sigmoid(acc_gate) * acc_up`,
    one rounding at the store."""
    from zmlx_b200 import quant
    import torch

    g = torch.Generator().manual_seed(3)
    M, N, K = 2, 5, 128
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    gw, gs, gb = quant.quantize_affine(torch.randn(N, K, generator=g) * 0.05)
    uw, us, ub = quant.quantize_affine(torch.randn(N, K, generator=g) * 0.05)
    npy = lambda t: t.view(torch.int32).numpy().view(np.uint32) if t.dtype == torch.uint32 else t.float().numpy()
    got = S.fused_quantized_swiglu_gemv(npy(x), npy(gw), npy(gs), npy(gb), npy(uw), npy(us), npy(ub))
    want = np.zeros((M, N), dtype=np.float32)
    for m in range(M):
        for n in range(N):
            ag = au = 0.0
            for i in range(K):
                qg = (int(npy(gw)[n, i // 8]) >> (4 * (i % 8))) & 15
                qu = (int(npy(uw)[n, i // 8]) >> (4 * (i % 8))) & 15
                wg = qg * float(npy(gs)[n, i // 64]) + float(npy(gb)[n, i // 64])
                wu = qu * float(npy(us)[n, i // 64]) + float(npy(ub)[n, i // 64])
                ag += wg * float(npy(x)[m, i])
                au += wu * float(npy(x)[m, i])
            y = 1.0 / (1.0 + np.exp(abs(ag)))
            want[m, n] = ag * (y if ag < 0 else 1.0 - y) * au
    assert np.abs(got - S.bf16(want)).max() <= np.abs(want).max() * 2.0 ** -7  # at most one bfloat16 ulp apart
