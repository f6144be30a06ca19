"""Quantisers that emit MLX-layout packed expert weights (torch, CPU or CUDA).

The reference never quantises on the hot path: checkpoints arrive packed, and its
tests call ``mx.quantize`` (tests/test_gather_qmm_swiglu.py:27-46).  These
helpers build the same layouts from float weights so that synthetic layers can
be made without MLX:

* affine 4-bit: ``uint32`` words, code ``i`` of a row in word ``i // 8`` at bit
  ``4 * (i % 8)``; ``w ~= q * scale + bias`` with one (scale, bias) pair in the
  scale dtype per ``group_size`` codes (src/zmlx/kernels/quant.py:109-120);
* mxfp4: the same nibble packing of e2m1 codes with one e8m0 byte per 32 codes.

The rounding rule of ``mx.quantize`` itself is not reproduced (it is not stated
anywhere in the reference tree); any packed tensor in this layout is accepted by
the kernels.
"""

from __future__ import annotations

import torch

_E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def pack_u4(q: torch.Tensor) -> torch.Tensor:
    """(..., K) integer codes in [0, 15] -> (..., K/8) uint32 words."""
    if q.shape[-1] % 8 != 0:
        raise ValueError("the packed axis must be a multiple of 8")
    q = q.to(torch.int64).reshape(*q.shape[:-1], q.shape[-1] // 8, 8)
    shifts = torch.arange(8, device=q.device, dtype=torch.int64) * 4
    words = (q << shifts).sum(dim=-1)
    words = torch.where(words >= 2**31, words - 2**32, words).to(torch.int32)
    return words.view(torch.uint32)


def unpack_u4(w: torch.Tensor) -> torch.Tensor:
    """(..., K/8) uint32 words -> (..., K) uint8 codes."""
    wi = w.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(8, device=w.device, dtype=torch.int64) * 4
    q = (wi.unsqueeze(-1) >> shifts) & 0xF
    return q.reshape(*w.shape[:-1], w.shape[-1] * 8).to(torch.uint8)


def quantize_affine(w: torch.Tensor, group_size: int = 64, bits: int = 4,
                    dtype: torch.dtype = torch.bfloat16):
    """Min/max affine quantisation per group along the last axis.

    Returns ``(packed uint32 (..., N, K/8), scales (..., N, K/gs), biases (..., N, K/gs))``.
    Scale and bias are rounded to ``dtype`` first and the codes are chosen against
    the rounded values, so ``q * scale + bias`` is the best 4-bit fit under them.
    """
    if bits != 4:
        raise ValueError("only 4-bit affine quantisation is implemented")
    K = w.shape[-1]
    if K % group_size != 0 or K % 8 != 0:
        raise ValueError(f"K={K} must be a multiple of group_size={group_size} and of 8")
    wf = w.to(torch.float32)
    g = wf.reshape(*wf.shape[:-1], K // group_size, group_size)
    lo = g.amin(dim=-1, keepdim=True)
    hi = g.amax(dim=-1, keepdim=True)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).to(dtype)
    bias = lo.to(dtype)
    q = torch.round((g - bias.to(torch.float32)) / scale.to(torch.float32)).clamp_(0, 15)
    packed = pack_u4(q.reshape(wf.shape))
    return packed, scale.squeeze(-1).contiguous(), bias.squeeze(-1).contiguous()


def dequantize_affine(packed: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                      group_size: int = 64) -> torch.Tensor:
    """float32 ``q * scale + bias`` (src/zmlx/kernels/quant.py:738-745)."""
    q = unpack_u4(packed).to(torch.float32)
    s = scales.to(torch.float32).repeat_interleave(group_size, dim=-1)
    b = biases.to(torch.float32).repeat_interleave(group_size, dim=-1)
    return q * s + b


def quantize_mxfp4(w: torch.Tensor):
    """OCP MX FP4: e2m1 codes with a shared power-of-two (e8m0) scale per 32 along the last axis.

    Returns ``(packed uint32 (..., N, K/8), scales uint8 (..., N, K/32))``.
    """
    K = w.shape[-1]
    if K % 32 != 0:
        raise ValueError(f"K={K} must be a multiple of 32")
    wf = w.to(torch.float32)
    g = wf.reshape(*wf.shape[:-1], K // 32, 32)
    amax = g.abs().amax(dim=-1, keepdim=True)
    # largest e2m1 magnitude is 6 = 1.5 * 2**2: shared exponent = floor(log2(amax)) - 2
    e = torch.floor(torch.log2(amax.clamp_min(2.0**-126))) - 2
    e = e.clamp_(-127, 127)
    scale = torch.exp2(e)
    v = g / scale
    mags = torch.tensor(_E2M1_VALUES, device=w.device, dtype=torch.float32)
    mids = (mags[1:] + mags[:-1]) / 2
    code = torch.bucketize(v.abs().clamp_max(6.0), mids)
    code = code + (v < 0).to(code.dtype) * 8
    packed = pack_u4(code.reshape(wf.shape))
    e8 = (e + 127).to(torch.uint8).squeeze(-1).contiguous()
    return packed, e8


def dequantize_mxfp4(packed: torch.Tensor, scales_e8m0: torch.Tensor) -> torch.Tensor:
    q = unpack_u4(packed).to(torch.int64)
    mags = torch.tensor(_E2M1_VALUES, device=packed.device, dtype=torch.float32)
    v = mags[q & 7] * torch.where((q & 8) != 0, -1.0, 1.0)
    s = torch.exp2(scales_e8m0.to(torch.float32) - 127.0).repeat_interleave(32, dim=-1)
    return v * s
