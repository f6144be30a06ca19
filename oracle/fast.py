"""ctypes front end of the compiled CPU oracle (TEST INFRASTRUCTURE ONLY).

Wraps ``libzmoe_oracle.so`` (built from ``zmoe_oracle.c`` by ``oracle/Makefile``).
Inputs and outputs use the conventions of :mod:`oracle.semantics`: dtype-T
tensors are float32 arrays holding bfloat16-representable values.
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from . import semantics as S

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile the C restatement next to its source; returns the library path."""
    so = os.path.join(_HERE, "libzmoe_oracle.so")
    src = os.path.join(_HERE, "zmoe_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "libzmoe_oracle.so"], check=True, capture_output=True)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libzmoe_oracle.so")
        if not os.path.exists(so):
            so = build()
        L = ctypes.CDLL(so)
        L.zo_gather_qmm.restype = ctypes.c_int
        L.zo_num_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def num_threads() -> int:
    return int(lib().zo_num_threads())


def set_num_threads(n: int) -> None:
    lib().zo_set_num_threads(int(n))


def gather_qmm_rows(x, w, scales, biases, lhs, rhs, *, group_size: int = 64, mode: str = "affine") -> np.ndarray:
    """out[p] = T(x[lhs[p]] @ dequant(w[rhs[p]]).T); x is (R, K), result (P, N)."""
    xb = np.ascontiguousarray(S.bf16_bits(x))
    R, K = xb.shape
    w = np.ascontiguousarray(w, dtype=np.uint32)
    E, N, _ = w.shape
    lhs = np.ascontiguousarray(lhs, dtype=np.int32).reshape(-1)
    rhs = np.ascontiguousarray(rhs, dtype=np.int32).reshape(-1)
    P = lhs.size
    out = np.empty((P, N), dtype=np.uint16)
    if mode == "affine":
        sc = np.ascontiguousarray(S.bf16_bits(scales))
        bi = np.ascontiguousarray(S.bf16_bits(biases))
        rc = lib().zo_gather_qmm(_p(xb), R, _p(w), _p(sc), _p(bi), E, N, K, int(group_size), 0,
                                 _p(lhs), _p(rhs), P, _p(out))
    elif mode == "mxfp4":
        sc = np.ascontiguousarray(scales, dtype=np.uint8)
        rc = lib().zo_gather_qmm(_p(xb), R, _p(w), _p(sc), None, E, N, K, 32, 1,
                                 _p(lhs), _p(rhs), P, _p(out))
    else:
        raise ValueError(mode)
    if rc != 0:
        raise IndexError("gather index out of range")
    return S.from_bf16_bits(out)


def swiglu_cpu_contract(g, u) -> np.ndarray:
    gb = np.ascontiguousarray(S.bf16_bits(g))
    ub = np.ascontiguousarray(S.bf16_bits(u))
    out = np.empty(gb.shape, dtype=np.uint16)
    lib().zo_swiglu(_p(gb), _p(ub), _p(out), ctypes.c_long(gb.size))
    return S.from_bf16_bits(out)


def experts_forward(x, idx, p, *, group_size: int = 64, mode: str = "affine", swiglu: str = "cpu"):
    """gate/up + SwiGLU + down for every (token, slot): returns y (T, K, d) in T."""
    T_, K = idx.shape
    lhs = np.repeat(np.arange(T_, dtype=np.int32), K)
    rhs = np.asarray(idx, dtype=np.int32).reshape(-1)
    g = gather_qmm_rows(x, p["gate_w"], p["gate_s"], p.get("gate_b"), lhs, rhs, group_size=group_size, mode=mode)
    u = gather_qmm_rows(x, p["up_w"], p["up_s"], p.get("up_b"), lhs, rhs, group_size=group_size, mode=mode)
    h = swiglu_cpu_contract(g, u) if swiglu == "cpu" else S.swiglu_per_op(g, u)
    y = gather_qmm_rows(h, p["down_w"], p["down_s"], p.get("down_b"), np.arange(T_ * K, dtype=np.int32), rhs,
                        group_size=group_size, mode=mode)
    return y.reshape(T_, K, -1), h.reshape(T_, K, -1)
