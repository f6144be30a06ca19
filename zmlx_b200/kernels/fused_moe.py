"""Fused gather + quantised matmul + SwiGLU (the reference's ``zmlx.kernels.fused_moe``).

Same names, arguments and error behaviour as src/zmlx/kernels/fused_moe.py:25-106,
with torch CUDA tensors in place of MLX arrays and a hand-written sm_100a kernel
in place of the MLX primitive (gather_qmm_swiglu.patch:329-510, 695-800).
"""

from __future__ import annotations

import os
from typing import Any

import torch

from .. import _lib, ops

_HAS_GATHER_QMM_SWIGLU: bool | None = None


def has_gather_qmm_swiglu() -> bool:
    """Return True if the fused op is available (the native library is built)."""
    global _HAS_GATHER_QMM_SWIGLU
    if _HAS_GATHER_QMM_SWIGLU is None:
        _HAS_GATHER_QMM_SWIGLU = os.path.exists(_lib.LIB_PATH)
    return _HAS_GATHER_QMM_SWIGLU


def _batch_numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


def _indices_or_default(idx, batch_shape, device):
    if idx is None:
        return torch.arange(_batch_numel(batch_shape), device=device, dtype=torch.int32).reshape(tuple(batch_shape))
    if idx.dtype.is_floating_point or idx.dtype == torch.bool:
        raise ValueError("[gather_qmm_swiglu] Got indices with invalid dtype. Indices must be integral.")
    return idx


def gather_qmm_swiglu(
    x: Any,
    gate_w: Any,
    gate_scales: Any,
    gate_biases: Any,
    up_w: Any,
    up_scales: Any,
    up_biases: Any,
    *,
    lhs_indices: Any | None = None,
    rhs_indices: Any | None = None,
    transpose: bool = True,
    group_size: int = 64,
    bits: int = 4,
    mode: str = "affine",
    swiglu_contract: str = "cpu",
) -> Any:
    """``silu(gather_qmm(x, gate_w, ...)) * gather_qmm(x, up_w, ...)`` in one kernel.

    Args follow src/zmlx/kernels/fused_moe.py:39-106: ``x`` is ``(..., M, K)``;
    the packed weights are ``(E, N, K/8)`` uint32, scales and biases
    ``(E, N, K // group_size)``.  Output shape is
    ``broadcast(lhs_indices, rhs_indices).shape + (M, N)``
    (gather_qmm_swiglu.patch:754-781).  Unlike the reference's Metal kernel there
    is no ``K % 512`` or ``N % 8`` restriction: ``K % 64 == 0`` suffices.

    ``mode="mxfp4"`` (scales are e8m0 bytes per 32, biases ignored) and
    ``swiglu_contract`` ("cpu": the rounding of the reference's CPU evaluation;
    "per_op": every elementwise op rounded to the activation dtype) are
    extensions; the reference op is affine-only.

    Raises ``RuntimeError`` if the native library is missing and ``ValueError``
    for the argument errors the reference's op rejects.
    """
    if not has_gather_qmm_swiglu():
        raise RuntimeError(
            "gather_qmm_swiglu is not available: libzmoe.so has not been built "
            "(python -m zmlx_b200.build)."
        )
    if not transpose:
        raise ValueError("[gather_qmm_swiglu] Only transpose=True is supported.")
    if mode not in ("affine", "mxfp4"):
        raise ValueError("[gather_qmm_swiglu] Only affine and mxfp4 quantization modes are supported.")
    if bits != 4:
        raise ValueError(f"[gather_qmm_swiglu] bits={bits} is not supported by this build (4 only).")
    if x.ndim < 2:
        raise ValueError(
            "[gather_qmm_swiglu] Non-quantized input must have at least two dimensions "
            f"but got input with shape {tuple(x.shape)}."
        )
    if not x.dtype.is_floating_point:
        raise ValueError(f"[gather_qmm_swiglu] Only real floating types are supported but x.dtype == {x.dtype}.")
    if gate_w.shape != up_w.shape or gate_scales.shape != up_scales.shape:
        raise ValueError("[gather_qmm_swiglu] gate and up weights must have matching shapes.")
    if gate_w.ndim < 2:
        raise ValueError("[gather_qmm_swiglu] weights must have at least two dimensions.")
    M, K = int(x.shape[-2]), int(x.shape[-1])
    N = int(gate_w.shape[-2])
    if int(gate_w.shape[-1]) * 8 != K:
        raise ValueError(
            f"[gather_qmm_swiglu] The last dimension of x ({K}) does not match the packed weights "
            f"({int(gate_w.shape[-1])} words of 8 codes)."
        )
    gsz = 32 if mode == "mxfp4" else int(group_size)
    if int(gate_scales.shape[-1]) * gsz != K:
        raise ValueError(
            f"[gather_qmm_swiglu] scales of shape {tuple(gate_scales.shape)} do not match K={K} "
            f"and group_size={gsz}."
        )
    if mode == "affine" and (gate_biases is None or up_biases is None):
        raise ValueError("[gather_qmm_swiglu] affine mode needs biases.")

    dev = x.device
    lhs = _indices_or_default(lhs_indices, x.shape[:-2], dev)
    rhs = _indices_or_default(rhs_indices, gate_w.shape[:-2], dev)
    lhs, rhs = torch.broadcast_tensors(lhs, rhs)
    out_batch = tuple(lhs.shape)
    E = _batch_numel(gate_w.shape[:-2])

    x2 = x.reshape(-1, K)
    if x2.dtype != torch.bfloat16:
        raise TypeError(f"gather_qmm_swiglu: activations must be bfloat16 on this build, got {x2.dtype}")
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) != 0 or x2.data_ptr() % 16 != 0:
        x2 = x2.contiguous()
    gw = gate_w.reshape(E, N, -1)
    uw = up_w.reshape(E, N, -1)
    gs_ = gate_scales.reshape(E, N, -1).contiguous()
    us_ = up_scales.reshape(E, N, -1).contiguous()
    gb_ = None if gate_biases is None else gate_biases.reshape(E, N, -1).contiguous()
    ub_ = None if up_biases is None else up_biases.reshape(E, N, -1).contiguous()

    P = lhs.numel()
    if P * M == 0:
        return torch.empty(out_batch + (M, N), dtype=torch.bfloat16, device=dev)
    plan = ops.build_plan(rhs.reshape(-1), E, M=M, lhs=lhs.reshape(-1))
    sw = _lib.SWIGLU_CPU if swiglu_contract == "cpu" else _lib.SWIGLU_PER_OP
    out = ops.gather_qmm_swiglu_rows(x2, gw.contiguous(), gs_, gb_, uw.contiguous(), us_, ub_, plan, P * M,
                                     rows_hint=P * M, group_size=gsz, mode=mode, swiglu=sw)
    return out.reshape(out_batch + (M, N))


__all__ = [
    "gather_qmm_swiglu",
    "has_gather_qmm_swiglu",
]
