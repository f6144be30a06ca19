"""GPU: the allocation-free down-projection + combine entry point against the caller-scratch one.

Some callers of this library cannot hand over a scratch buffer or allocate one (capture of a CUDA graph,
serving loops that forbid device-wide synchronising calls, foreign runtimes).  For them
``zmoe_gather_qmm_combine_noalloc`` keeps its scratch inside the library.  This file is named so that pytest
collects it last; it calls both entry points through the C ABI on the same inputs, twice in a row with different
data (the built-in scratch keeps the first call's rows), and expects bit-identical outputs.
"""

import ctypes

import numpy as np
import pytest
import torch

from oracle import semantics as S
from tests.helpers import t2n
from zmlx_b200 import _lib, ops, quant

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, T, K, E, d_in, d_out):
    g = torch.Generator().manual_seed(seed)
    w, s, b = quant.quantize_affine(torch.randn((E, d_out, d_in), generator=g) * 0.02, 64)
    act = torch.randn((T * K, d_in), generator=g).to(torch.bfloat16)
    gate = torch.rand((T, K), generator=g)
    idx = torch.randint(0, E, (T * K,), generator=g, dtype=torch.int32)
    return [t.to(DEV) for t in (w, s, b, act, gate, idx)]


def _run(fn_name, tensors, T, K, E, d_in, d_out, scratch=None):
    w, s, b, act, gate, idx = tensors
    lib = _lib.load()
    p = ops._ptr
    plan = ops.build_plan(idx, E)
    out = torch.full((T, d_out), float("nan"), dtype=torch.float32, device=DEV)
    st = ops._stream()
    args = [p(act), d_in, p(w), p(s), p(b), E, d_out, d_in, 64, _lib.Q_AFFINE4, p(plan), T, K, p(gate), _lib.F32,
            _lib.COMBINE_FP32_NO_FMA]
    if scratch is not None:
        args.append(p(scratch))
    args += [p(out), 0, st]
    _lib.check(getattr(lib, fn_name)(*args))
    torch.cuda.synchronize()
    return out


def test_noalloc_matches_caller_scratch_twice_in_a_row():
    T, K, E, d_in, d_out = 5, 4, 8, 768, 2048
    for seed in (1, 2):  # second call reuses the built-in scratch that the first one filled
        tensors = _case(seed, T, K, E, d_in, d_out)
        scratch = torch.empty((T * K, d_out), dtype=torch.bfloat16, device=DEV)
        want = _run("zmoe_gather_qmm_combine", tensors, T, K, E, d_in, d_out, scratch=scratch)
        if seed == 2:  # the array's address is cached by now: the call itself must not change free memory at all
            plan = ops.build_plan(tensors[5], E)  # (allocations of the test harness happen before the probe)
            del plan
        free_before = torch.cuda.mem_get_info()[0]
        got = _run("zmoe_gather_qmm_combine_noalloc", tensors, T, K, E, d_in, d_out)
        free_after = torch.cuda.mem_get_info()[0]
        assert free_after >= free_before - (1 << 20)  # nothing allocated by the call (torch's own pool aside)
        if seed == 2:  # same shapes as the call before: torch serves its tensors from its pool, so not one byte moves
            assert free_after == free_before
        assert torch.isfinite(got).all()
        assert torch.equal(got, want)
        # and the entry point's own evidence against the CPU oracle: the projections are rounded to T (bfloat16)
        # on both sides before the float32 combine, so a last-bit flip of one projection moves the sum by a
        # bf16 ulp of that term -- the bound is the one for bf16 activations, 2e-2 of the tensor's scale
        w, s_, b, act, gate, idx = tensors
        ref = S.gather_qmm_combine_quantized(t2n(act).reshape(T, K, d_in), t2n(w.view(torch.int32)).view(np.uint32),
                                             t2n(s_), t2n(b), t2n(gate), t2n(idx).reshape(T, K), group_size=64,
                                             combine="fp32_no_fma")
        err = np.abs(t2n(got) - ref).max() / max(float(np.sqrt((ref ** 2).mean())), 1e-30)
        assert err <= 2e-2, f"no-alloc entry vs oracle: {err:.3g} of rms"
    # a smaller call after a larger one: stale rows beyond the used part must not leak in
    tensors = _case(3, 2, 2, 8, 256, 512)
    scratch = torch.empty((4, 512), dtype=torch.bfloat16, device=DEV)
    want = _run("zmoe_gather_qmm_combine", tensors, 2, 2, 8, 256, 512, scratch=scratch)
    got = _run("zmoe_gather_qmm_combine_noalloc", tensors, 2, 2, 8, 256, 512)
    assert torch.equal(got, want)


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    lib = _lib.load()
    dummy = torch.zeros(16, dtype=torch.int32, device=DEV)
    p = ops._ptr
    # T*K*N = 64*8*7168 = 3,670,016 > 2,097,152: refused before anything is enqueued
    rc = lib.zmoe_gather_qmm_combine_noalloc(p(dummy), 2048, p(dummy), p(dummy), p(dummy), 8, 7168, 2048, 64, 0, p(dummy),
                                             64, 8, p(dummy), _lib.F32, _lib.COMBINE_FP32_NO_FMA, p(dummy), 0,
                                             ctypes.c_void_p(0))
    assert rc == _lib.ERR_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
