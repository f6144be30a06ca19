"""CPU: the C-ABI library loads and exports what the header declares; host-side
argument checks behave like the reference's; nothing computes without a GPU."""

import os
import re

import pytest
import torch

import zmlx_b200
from zmlx_b200 import _lib, ops
from zmlx_b200.kernels import fused_moe, moe

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "zmoe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zmoe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/zmoe.h but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert lib.zmoe_abi_version() == _lib.ABI_VERSION


def test_argument_errors_do_not_touch_the_gpu():
    lib = _lib.load()
    assert lib.zmoe_plan_bytes(8, 128) == 4 * (4 + 4 * 128 + 129 + 128 + 16)
    rc = lib.zmoe_router_softmax_topk(None, 0, 1, 8, 2, 0, None, 0, None, None, None)
    assert rc == _lib.ERR_SHAPE and "null pointer" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc)
    rc = lib.zmoe_build_plan(None, 0, None, 1, 1, 8, None, 0, None)
    assert rc < 0


def test_cpu_tensors_are_refused():
    x = torch.zeros((1, 8))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        moe.topk_gating_softmax(x, 2)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        moe.moe_combine(torch.zeros((1, 2, 8), dtype=torch.bfloat16), torch.zeros((1, 2)))


def test_reference_validation_messages():
    x = torch.zeros((1, 8))
    with pytest.raises(ValueError, match="k must be > 0"):
        moe.topk_gating_softmax(x, 0)
    with pytest.raises(ValueError, match="exceeds last dimension D=8"):
        moe.topk_gating_softmax(x, 9)
    with pytest.raises(ValueError, match="invalid topk_group"):
        moe.deepseek_router_topk_sigmoid(x, torch.zeros(8), k=2, n_group=2, topk_group=3)
    with pytest.raises(ValueError, match="bias must have shape"):
        moe.deepseek_router_topk_sigmoid(x, torch.zeros(7), k=2)
    with pytest.raises(ValueError, match=r"act must have shape \(B, K, D_in\)"):
        moe.gather_qmm_combine_quantized(torch.zeros((2, 8)), None, None, None, None, None)
    with pytest.raises(ValueError, match=r"act must have shape \(B, K, D_in\)"):
        moe.gather_qmm_combine(torch.zeros((2, 8)), torch.zeros((1, 8, 8)), None, None)
    w = torch.zeros((2, 8, 8), dtype=torch.int32)
    s = torch.zeros((2, 8, 1), dtype=torch.bfloat16)
    xx = torch.zeros((1, 1, 64), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="Only transpose=True"):
        fused_moe.gather_qmm_swiglu(xx, w, s, s, w, s, s, transpose=False)
    with pytest.raises(ValueError, match="matching shapes"):
        fused_moe.gather_qmm_swiglu(xx, w, s, s, w[:, :4], s[:, :4], s[:, :4])
    with pytest.raises(ValueError, match="at least two dimensions"):
        fused_moe.gather_qmm_swiglu(xx[0, 0], w, s, s, w, s, s)


def test_surface_matches_reference_exports():
    assert set(moe.__all__) == {
        "top2_gating_softmax", "topk_gating_softmax", "router_argpartition_logits_topk",
        "deepseek_router_topk_sigmoid", "moe_dispatch", "moe_combine", "moe_combine_no_fma",
        "moe_combine_exact", "moe_combine_fp32", "moe_combine_fp32_no_fma", "gather_mmk_combine",
        "gather_qmmk_combine_quantized", "gather_qmm_combine", "gather_qmm_combine_quantized"}
    assert fused_moe.__all__ == ["gather_qmm_swiglu", "has_gather_qmm_swiglu"]
    assert fused_moe.has_gather_qmm_swiglu() is True
    assert zmlx_b200.__version__
