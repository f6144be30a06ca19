"""Thin torch-tensor front end of the C ABI: pointer plumbing and output allocation.

Every function here enqueues CUDA work on torch's current stream through
``libzmoe.so`` and returns torch tensors.  Tensors must live on a CUDA device;
there is no CPU path.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib

_U32_LIKE = (torch.int32, torch.uint32)


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor | None) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                "zmlx_b200 kernels run on CUDA tensors only (no CPU fallback); got a tensor on " + str(t.device)
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    assert dev is not None
    return dev


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise TypeError(f"unsupported dtype {t.dtype}: this build computes in bfloat16 / float32")


def qmode_code(mode: str) -> int:
    if mode == "affine":
        return _lib.Q_AFFINE4
    if mode == "mxfp4":
        return _lib.Q_MXFP4
    raise ValueError(f"unknown quantisation mode {mode!r}")


def plan_bytes(rows: int, E: int) -> int:
    return int(_lib.load().zmoe_plan_bytes(int(rows), int(E)))


def build_plan(rhs: torch.Tensor, E: int, *, M: int = 1, lhs: torch.Tensor | None = None, lhs_div: int = 1,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """Group (lhs, rhs) gather pairs by expert; returns the int32 plan buffer."""
    dev = _need_cuda(rhs, lhs)
    rhs = rhs.reshape(-1).to(torch.int32).contiguous()
    if lhs is not None:
        lhs = lhs.reshape(-1).to(torch.int32).contiguous()
        if lhs.numel() != rhs.numel():
            raise ValueError("lhs and rhs index counts differ")
    P = rhs.numel()
    nbytes = plan_bytes(P * M, E)
    if out is None:
        out = torch.empty(nbytes // 4, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().zmoe_build_plan(_ptr(lhs), int(lhs_div), _ptr(rhs), P, int(M), int(E), _ptr(out),
                                               out.numel() * 4, _stream()))
    return out


def _check_packed(w: torch.Tensor, name: str) -> None:
    if w.dtype not in _U32_LIKE:
        raise TypeError(f"{name} must be uint32-packed (torch.uint32 or torch.int32), got {w.dtype}")
    if not w.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def gather_qmm_swiglu_rows(x2: torch.Tensor, gate_w, gate_s, gate_b, up_w, up_s, up_b, plan: torch.Tensor, rows: int,
                           *, rows_hint: int, group_size: int = 64, mode: str = "affine",
                           swiglu: int = _lib.SWIGLU_CPU, out: torch.Tensor | None = None) -> torch.Tensor:
    dev = _need_cuda(x2, gate_w, gate_s, gate_b, up_w, up_s, up_b, plan)
    if x2.dtype != torch.bfloat16:
        raise TypeError(f"activations must be bfloat16, got {x2.dtype}")
    _check_packed(gate_w, "gate_w")
    _check_packed(up_w, "up_w")
    E, N, K8 = gate_w.shape
    K = K8 * 8
    if x2.shape[-1] != K or x2.stride(-1) != 1:
        raise ValueError(f"x has inner dimension {x2.shape[-1]}, weights expect {K}")
    if out is None:
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().zmoe_gather_qmm_swiglu(
            _ptr(x2), x2.shape[0], x2.stride(0), _ptr(gate_w), _ptr(gate_s), _ptr(gate_b), _ptr(up_w), _ptr(up_s),
            _ptr(up_b), E, N, K, int(group_size), qmode_code(mode), _ptr(plan), int(rows), int(rows_hint), _ptr(out),
            int(swiglu), _stream()))
    return out


def gather_qmm_rows(x2: torch.Tensor, w, s, b, plan: torch.Tensor, rows: int, *, rows_hint: int,
                    group_size: int = 64, mode: str = "affine", x_by_output_row: bool = False,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    dev = _need_cuda(x2, w, s, b, plan)
    if x2.dtype != torch.bfloat16:
        raise TypeError(f"activations must be bfloat16, got {x2.dtype}")
    _check_packed(w, "w")
    E, N, K8 = w.shape
    K = K8 * 8
    if x2.shape[-1] != K or x2.stride(-1) != 1:
        raise ValueError(f"x has inner dimension {x2.shape[-1]}, weights expect {K}")
    if out is None:
        out = torch.empty((rows, N), dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().zmoe_gather_qmm(
            _ptr(x2), x2.shape[0], x2.stride(0), _ptr(w), _ptr(s), _ptr(b), E, N, K, int(group_size),
            qmode_code(mode), _ptr(plan), int(rows), int(rows_hint), int(bool(x_by_output_row)), _ptr(out),
            _stream()))
    return out


def combine(y: torch.Tensor, w: torch.Tensor, mode: int, *, out_t: bool = False,
            residual: torch.Tensor | None = None) -> torch.Tensor:
    """out[t, d] = sum_i w[t, i] * y[t, i, d]; y (T, K, D), w (T, K)."""
    dev = _need_cuda(y, w, residual)
    T, K, D = y.shape
    y = y.contiguous()
    w = w.contiguous()
    fp32_mode = mode in (_lib.COMBINE_FP32, _lib.COMBINE_FP32_NO_FMA)
    out_dtype = torch.float32 if (fp32_mode and not out_t) else torch.bfloat16
    out = torch.empty((T, D), dtype=out_dtype, device=dev)
    if residual is not None:
        residual = residual.contiguous()
        if residual.dtype != torch.bfloat16 or residual.shape != (T, D):
            raise ValueError("residual must be bfloat16 of shape (T, D)")
    if T == 0:
        return out
    with torch.cuda.device(dev):
        for t0 in range(0, T, 65535):
            n = min(T - t0, 65535)
            _lib.check(_lib.load().zmoe_moe_combine(
                _ptr(y[t0:]), _dtype_code(y), _ptr(w[t0:]), _dtype_code(w), n, K, D, int(mode), _ptr(out[t0:]),
                int(out_t), _ptr(residual[t0:]) if residual is not None else None, _stream()))
    return out


def swiglu(gate: torch.Tensor, up: torch.Tensor, *, mode: int = _lib.SWIGLU_PER_OP) -> torch.Tensor:
    """Elementwise silu(gate) * up on bfloat16 tensors of the same shape (``zmoe_swiglu``)."""
    dev = _need_cuda(gate, up)
    if gate.shape != up.shape:
        raise ValueError("swiglu2: gate and up must have the same shape")
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16:
        raise TypeError(f"swiglu: gate and up must be bfloat16, got {gate.dtype} and {up.dtype}")
    g, u = gate.contiguous(), up.contiguous()
    out = torch.empty_like(g)
    if g.numel() == 0:
        return out
    with torch.cuda.device(dev):
        _lib.check(_lib.load().zmoe_swiglu(_ptr(g), _ptr(u), g.numel(), int(mode), _ptr(out), _stream()))
    return out


def router_softmax_topk(logits: torch.Tensor, k: int, *, flavour: int, bias: torch.Tensor | None = None,
                        renorm: int = 0):
    dev = _need_cuda(logits, bias)
    E = logits.shape[-1]
    l2 = logits.reshape(-1, E).contiguous()
    T = l2.shape[0]
    if bias is not None:
        bias = bias.reshape(-1).to(torch.float32).contiguous()
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        if T > 0:
            _lib.check(_lib.load().zmoe_router_softmax_topk(_ptr(l2), _dtype_code(l2), T, E, int(k), int(flavour),
                                                            _ptr(bias), int(renorm), _ptr(w), _ptr(idx), _stream()))
    shape = logits.shape[:-1] + (k,)
    return w.reshape(shape), idx.view(torch.uint32).reshape(shape)


def router_sigmoid_topk(logits: torch.Tensor, bias: torch.Tensor, k: int, *, n_group: int = 1, topk_group: int = 1,
                        scale: float = 1.0):
    dev = _need_cuda(logits, bias)
    E = logits.shape[-1]
    l2 = logits.reshape(-1, E).contiguous()
    T = l2.shape[0]
    bias = bias.reshape(-1).to(torch.float32).contiguous()
    w = torch.empty((T, k), dtype=torch.float32, device=dev)
    idx = torch.empty((T, k), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        if T > 0:
            _lib.check(_lib.load().zmoe_router_sigmoid_bias_topk(_ptr(l2), _dtype_code(l2), T, E, int(k), _ptr(bias),
                                                                 int(n_group), int(topk_group),
                                                                 ctypes.c_float(float(scale)), _ptr(w), _ptr(idx),
                                                                 _stream()))
    shape = logits.shape[:-1] + (k,)
    return w.reshape(shape), idx.view(torch.uint32).reshape(shape)


def router_logits(x: torch.Tensor, wr: torch.Tensor, *, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    dev = _need_cuda(x, wr)
    if x.dtype != torch.bfloat16 or wr.dtype != torch.bfloat16:
        raise TypeError("router_logits expects bfloat16 activations and weights")
    d = x.shape[-1]
    x2 = x.reshape(-1, d).contiguous()
    wr = wr.contiguous()
    T, E = x2.shape[0], wr.shape[0]
    out = torch.empty((T, E), dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        if T > 0:
            _lib.check(_lib.load().zmoe_router_logits(_ptr(x2), _ptr(wr), T, E, d, _ptr(out), _dtype_code(out),
                                                      _stream()))
    return out.reshape(x.shape[:-1] + (E,))
