"""GPU parity: gather_qmm_swiglu / gather_qmm / gather_qmm_combine against the oracle.

Tolerance: activations within 2e-2 relative (bf16), the bound the acceptance bar
states; measured errors are about one bfloat16 ulp.
"""

import numpy as np
import pytest
import torch

from oracle import fast as F
from oracle import semantics as S
from tests.helpers import assert_close_rel, t2n
from zmlx_b200 import ops, quant
from zmlx_b200.kernels import fused_moe, moe

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = 2e-2


def _bank(E, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn((E, N, K), generator=g) * 0.02
    return quant.quantize_affine(w, 64)


def _to(dev, *ts):
    return [t.to(dev) for t in ts]


def _oracle_swiglu(x2, gate, up, lhs, rhs, contract="cpu"):
    g = F.gather_qmm_rows(x2, *[t2n(t) for t in gate], lhs, rhs)
    u = F.gather_qmm_rows(x2, *[t2n(t) for t in up], lhs, rhs)
    return F.swiglu_cpu_contract(g, u) if contract == "cpu" else S.swiglu_per_op(g, u)


@pytest.mark.parametrize("E,M,K,N", [(8, 1, 512, 512), (8, 4, 1024, 768), (16, 16, 2048, 1024), (64, 1, 4096, 512),
                                     (8, 1, 2048, 2048), (4, 3, 192, 24), (8, 1, 768, 1000)])
def test_gather_qmm_swiglu_reference_shapes(E, M, K, N):
    """The sweep of the reference's own test (tests/test_gather_qmm_swiglu.py:121-305): x (1, M, K) * 0.1,
    two experts picked with lhs = 0."""
    gate, up = _bank(E, N, K, 1), _bank(E, N, K, 2)
    g = torch.Generator().manual_seed(3)
    x = (torch.randn((1, M, K), generator=g) * 0.1).to(torch.bfloat16)
    lhs = torch.zeros((2,), dtype=torch.int32)
    rhs = torch.arange(2, dtype=torch.int32)
    out = fused_moe.gather_qmm_swiglu(x.to(DEV), *_to(DEV, *gate), *_to(DEV, *up), lhs_indices=lhs.to(DEV),
                                      rhs_indices=rhs.to(DEV))
    assert out.shape == (2, M, N) and out.dtype == torch.bfloat16
    x2 = t2n(x).reshape(M, K)
    rows_l = np.tile(np.arange(M, dtype=np.int32), 2)
    rows_r = np.repeat(np.arange(2, dtype=np.int32), M)
    ref = _oracle_swiglu(x2, gate, up, rows_l, rows_r).reshape(2, M, N)
    assert_close_rel(t2n(out), ref, REL, "gather_qmm_swiglu")


def test_moe_call_shape_and_default_indices():
    """x (B, L, 1, 1, d) with rhs (B, L, K), as the patched block calls it (moe_mlp.py:554-565)."""
    E, K_, d, f = 16, 4, 512, 256
    gate, up = _bank(E, f, d, 4), _bank(E, f, d, 5)
    g = torch.Generator().manual_seed(6)
    x = torch.randn((2, 3, 1, 1, d), generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:K_] for _ in range(6)]).reshape(2, 3, K_).to(torch.int32)
    out = fused_moe.gather_qmm_swiglu(x.to(DEV), *_to(DEV, *gate), *_to(DEV, *up), rhs_indices=idx.to(DEV))
    assert out.shape == (2, 3, K_, 1, f)
    lhs = np.repeat(np.arange(6, dtype=np.int32), K_)
    ref = _oracle_swiglu(t2n(x).reshape(6, d), gate, up, lhs, t2n(idx).reshape(-1)).reshape(2, 3, K_, 1, f)
    assert_close_rel(t2n(out), ref, REL, "moe call shape")
    # uint32 indices (what the routers return) and the per-op SwiGLU contract
    out2 = fused_moe.gather_qmm_swiglu(x.to(DEV), *_to(DEV, *gate), *_to(DEV, *up),
                                       rhs_indices=idx.to(DEV).view(torch.uint32), swiglu_contract="per_op")
    ref2 = _oracle_swiglu(t2n(x).reshape(6, d), gate, up, lhs, t2n(idx).reshape(-1), "per_op").reshape(out2.shape)
    assert_close_rel(t2n(out2), ref2, REL, "per-op contract")
    # no indices at all: x batch (E,) pairs with expert e (tests/test_gather_qmm_swiglu.py "None indices")
    xe = torch.randn((E, 2, d), generator=g).to(torch.bfloat16)
    out3 = fused_moe.gather_qmm_swiglu(xe.to(DEV), *_to(DEV, *gate), *_to(DEV, *up))
    assert out3.shape == (E, 2, f)
    l3 = np.arange(2 * E, dtype=np.int32)
    ref3 = _oracle_swiglu(t2n(xe).reshape(2 * E, d), gate, up, l3, np.repeat(np.arange(E, dtype=np.int32), 2))
    assert_close_rel(t2n(out3), ref3.reshape(E, 2, f), REL, "default indices")


@pytest.mark.parametrize("T", [1, 4, 16, 64, 200])
def test_token_sorted_grouping_many_rows_per_expert(T):
    """Few experts, many tokens: rows per expert exceed one pass, duplicates and ragged counts included."""
    E, K_, d, f = 4, 2, 256, 64
    gate, up, down = _bank(E, f, d, 7), _bank(E, f, d, 8), _bank(E, d, f, 9)
    g = torch.Generator().manual_seed(T)
    x = torch.randn((T, d), generator=g).to(torch.bfloat16)
    idx = torch.randint(0, E, (T, K_), generator=g, dtype=torch.int32)
    idx[:, 0] = 1  # every token also hits expert 1: one expert owns T rows
    h = fused_moe.gather_qmm_swiglu(x.reshape(T, 1, 1, d).to(DEV), *_to(DEV, *gate), *_to(DEV, *up),
                                    rhs_indices=idx.to(DEV))
    assert h.shape == (T, K_, 1, f)
    lhs = np.repeat(np.arange(T, dtype=np.int32), K_)
    ref_h = _oracle_swiglu(t2n(x), gate, up, lhs, t2n(idx).reshape(-1))
    assert_close_rel(t2n(h).reshape(T * K_, f), ref_h, REL, "grouped swiglu")
    # down projection + combine on the kernel's own h (so that the comparison isolates this op)
    hk = h.reshape(T, K_, f)
    gatew = torch.rand((T, K_), generator=g)
    for kw, cmode in (({"streaming": False}, "exact"), ({"output_dtype": torch.float32, "no_fma": True}, "fp32_no_fma"),
                      ({}, "stream_t" if T <= 16 else "exact")):
        gw = gatew.to(torch.bfloat16) if cmode in ("exact", "stream_t") else gatew
        out = moe.gather_qmm_combine_quantized(hk, *_to(DEV, *down), gw.to(DEV), idx.to(DEV).view(torch.uint32), **kw)
        ref = S.gather_qmm_combine_quantized(t2n(hk), *[t2n(t) for t in down], t2n(gw), t2n(idx), combine=cmode)
        assert out.shape == (T, d)
        assert_close_rel(t2n(out), ref, REL, f"gather_qmm_combine {cmode}")


@pytest.mark.parametrize("T,d,f", [(300, 512, 384), (96, 1024, 768), (1024, 256, 256)])
def test_tensor_memory_path_many_rows_per_expert(T, d, f):
    """Hundreds of rows per expert take the tcgen05 / tensor-memory kernel (128 weight rows x up to 128 token rows
    per tile, several token blocks per expert, ragged last block, weight tiles that end beyond N); gate/up +
    SwiGLU and the down projection against the oracle."""
    E, K_ = 4, 2
    gate, up, down = _bank(E, f, d, 21), _bank(E, f, d, 22), _bank(E, d, f, 23)
    g = torch.Generator().manual_seed(T + d)
    x = torch.randn((T, d), generator=g).to(torch.bfloat16)
    idx = torch.randint(0, E, (T, K_), generator=g, dtype=torch.int32)
    idx[:, 0] = 1  # one expert owns T rows
    h = fused_moe.gather_qmm_swiglu(x.reshape(T, 1, 1, d).to(DEV), *_to(DEV, *gate), *_to(DEV, *up),
                                    rhs_indices=idx.to(DEV))
    lhs = np.repeat(np.arange(T, dtype=np.int32), K_)
    ref_h = _oracle_swiglu(t2n(x), gate, up, lhs, t2n(idx).reshape(-1))
    assert_close_rel(t2n(h).reshape(T * K_, f), ref_h, REL, "tensor-memory gate/up + SwiGLU")
    hk = h.reshape(T, K_, f)
    gw = torch.rand((T, K_), generator=g)
    out = moe.gather_qmm_combine_quantized(hk, *_to(DEV, *down), gw.to(DEV), idx.to(DEV).view(torch.uint32),
                                           output_dtype=torch.float32, no_fma=True)
    ref = S.gather_qmm_combine_quantized(t2n(hk), *[t2n(t) for t in down], t2n(gw), t2n(idx), combine="fp32_no_fma")
    assert_close_rel(t2n(out), ref, REL, "tensor-memory down projection + combine")


def test_empty_and_single_expert_cases():
    E, d, f = 4, 128, 32
    gate, up = _bank(E, f, d, 10), _bank(E, f, d, 11)
    x = torch.zeros((0, 1, 1, d), dtype=torch.bfloat16, device=DEV)
    out = fused_moe.gather_qmm_swiglu(x, *_to(DEV, *gate), *_to(DEV, *up),
                                      rhs_indices=torch.zeros((0, 2), dtype=torch.int32, device=DEV))
    assert out.shape == (0, 2, 1, f)
    # all tokens on one expert, other experts idle
    g = torch.Generator().manual_seed(12)
    xs = torch.randn((5, 1, 1, d), generator=g).to(torch.bfloat16)
    idx = torch.full((5, 1), 3, dtype=torch.int32)
    out = fused_moe.gather_qmm_swiglu(xs.to(DEV), *_to(DEV, *gate), *_to(DEV, *up), rhs_indices=idx.to(DEV))
    ref = _oracle_swiglu(t2n(xs).reshape(5, d), gate, up, np.arange(5, dtype=np.int32), np.full(5, 3, np.int32))
    assert_close_rel(t2n(out).reshape(5, f), ref, REL, "single expert")


def test_linearity_and_determinism_at_full_width():
    """Size-independent properties at the Qwen3 shape: the op is linear in x before the activation, so the
    down projection of (a + b) equals the sum of projections up to bf16 rounding; repeated calls are bit-equal."""
    E, d, f = 8, 768, 2048
    down = _bank(E, f, d, 13)  # (E, N=2048, K=768)
    g = torch.Generator().manual_seed(14)
    a = torch.randn((8, d), generator=g).to(torch.bfloat16)
    b = torch.randn((8, d), generator=g).to(torch.bfloat16)
    idx = torch.arange(8, dtype=torch.int32)
    plan = ops.build_plan(idx.to(DEV), E)
    dw, ds, db = _to(DEV, *down)

    def proj(v):
        return ops.gather_qmm_rows(v.to(DEV), dw, ds, db, plan, 8, rows_hint=1)

    pa, pb = proj(a), proj(b)
    s = (a.float() + b.float()).to(torch.bfloat16)
    ps = proj(s)
    assert torch.equal(proj(a), pa)
    resid = (s.float() - a.float() - b.float())  # rounding of a + b itself
    pr = proj(resid.to(torch.bfloat16))
    err = (ps.float() - pa.float() - pb.float() - pr.float()).abs().max().item()
    scale = ps.float().abs().max().item()
    assert err <= 4 * 2 ** -8 * scale


def test_bad_arguments_raise():
    E, d, f = 4, 128, 32
    gate, up = _bank(E, f, d, 15), _bank(E, f, d, 16)
    x = torch.zeros((1, 1, d), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(TypeError):
        fused_moe.gather_qmm_swiglu(x.float(), *_to(DEV, *gate), *_to(DEV, *up))
    with pytest.raises(ValueError):
        fused_moe.gather_qmm_swiglu(x, *_to(DEV, *gate), *_to(DEV, *up), bits=8)
    with pytest.raises(ValueError):
        fused_moe.gather_qmm_swiglu(x, *_to(DEV, *gate), *_to(DEV, *up),
                                    rhs_indices=torch.zeros((1,), device=DEV))  # float indices


@pytest.mark.parametrize("T,K_,d,f", [(1, 4, 2048, 1536), (5, 2, 512, 256), (12, 3, 256, 768), (40, 2, 256, 256)])
def test_mxfp4_swiglu_and_down(T, K_, d, f):
    """mxfp4 expert banks (e2m1 codes, e8m0 scale per 32): fused gate/up + SwiGLU (per-op contract) and down."""
    E = 8
    g = torch.Generator().manual_seed(100 + T)
    banks = []
    for n_out, n_in in ((f, d), (f, d), (d, f)):
        w = torch.randn((E, n_out, n_in), generator=g) * 0.02
        banks.append(quant.quantize_mxfp4(w))
    x = torch.randn((T, 1, 1, d), generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:K_] for _ in range(T)]).to(torch.int32)
    (gw, gs), (uw, us), (dw, ds) = banks
    h = fused_moe.gather_qmm_swiglu(x.to(DEV), gw.to(DEV), gs.to(DEV), None, uw.to(DEV), us.to(DEV), None,
                                    rhs_indices=idx.to(DEV), mode="mxfp4", group_size=32, swiglu_contract="per_op")
    assert h.shape == (T, K_, 1, f)
    lhs = np.repeat(np.arange(T, dtype=np.int32), K_)
    rhs = t2n(idx).reshape(-1)
    gg = F.gather_qmm_rows(t2n(x).reshape(T, d), t2n(gw), t2n(gs), None, lhs, rhs, mode="mxfp4")
    uu = F.gather_qmm_rows(t2n(x).reshape(T, d), t2n(uw), t2n(us), None, lhs, rhs, mode="mxfp4")
    ref_h = S.swiglu_per_op(gg, uu)
    assert_close_rel(t2n(h).reshape(T * K_, f), ref_h, REL, "mxfp4 swiglu")
    gate = torch.rand((T, K_), generator=g)
    out = moe.gather_qmm_combine_quantized(h.reshape(T, K_, f), dw.to(DEV), ds.to(DEV), None, gate.to(DEV),
                                           idx.to(DEV).view(torch.uint32), group_size=32, mode="mxfp4",
                                           output_dtype=torch.float32, no_fma=True)
    ref = S.gather_qmm_combine_quantized(t2n(h).reshape(T, K_, f), t2n(dw), t2n(ds), None, t2n(gate), t2n(idx),
                                         mode="mxfp4", combine="fp32_no_fma")
    assert_close_rel(t2n(out), ref, REL, "mxfp4 down + combine")


@pytest.mark.parametrize("E,P", [(128, 1024), (300, 4096), (1024, 8192), (256, 300)])
def test_plan_with_every_expert_active(E, P):
    """The task list, offsets and row maps stay right when 128 or more experts own rows (the counts of both scans
    of the plan builder pass 127 and 255)."""
    g = torch.Generator().manual_seed(E + P)
    idx = torch.cat([torch.arange(E), torch.randint(0, E, (P - E,), generator=g)])[torch.randperm(P, generator=g)]
    plan = ops.build_plan(idx.to(DEV), E).cpu().numpy()
    counts = np.bincount(idx.numpy(), minlength=E)
    assert plan[0] == int((counts > 0).sum()) and plan[1] == P and plan[2] == 0 and plan[3] == E
    tasks = plan[4:4 + 4 * E].reshape(E, 4)
    n_active = plan[0]
    assert np.array_equal(tasks[:n_active, 0], np.flatnonzero(counts > 0))
    assert np.array_equal(tasks[:n_active, 2], counts[counts > 0])
    offset = plan[4 + 4 * E:4 + 4 * E + E + 1]
    assert np.array_equal(offset, np.concatenate([[0], np.cumsum(counts)]))
    assert np.array_equal(tasks[:n_active, 1], offset[:-1][counts > 0])
    row_src = plan[4 + 4 * E + (E + 1) + E:][:P]
    row_dst = plan[4 + 4 * E + (E + 1) + E + P:][:P]
    assert np.array_equal(np.sort(row_dst), np.arange(P)) and np.array_equal(row_src, row_dst)
    for e in (0, E // 2, E - 1):
        seg = row_dst[offset[e]:offset[e + 1]]
        assert np.array_equal(np.sort(seg), np.flatnonzero(idx.numpy() == e))
