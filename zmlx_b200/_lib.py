"""ctypes binding of ``libzmoe.so`` (the C ABI declared in ``include/zmoe.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  ``ZmoeError`` carries the library's own message.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libzmoe.so")

OK = 0
ERR_SHAPE, ERR_DTYPE, ERR_ALIGN, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = -1, -2, -3, -4, -5, -6, -7
F32, BF16 = 0, 1
Q_AFFINE4, Q_MXFP4 = 0, 1
SWIGLU_CPU, SWIGLU_PER_OP = 0, 1
COMBINE_FP32, COMBINE_FP32_NO_FMA, COMBINE_T, COMBINE_NO_FMA, COMBINE_EXACT, COMBINE_STREAM_T = range(6)
ROUTER_TOPK_THEN_SOFTMAX, ROUTER_SOFTMAX_THEN_TOPK = 0, 1

COMBINE_MODES = {
    "fp32": COMBINE_FP32,
    "fp32_no_fma": COMBINE_FP32_NO_FMA,
    "t": COMBINE_T,
    "no_fma": COMBINE_NO_FMA,
    "exact": COMBINE_EXACT,
    "stream_t": COMBINE_STREAM_T,
}

# name -> (restype, argtypes); must list every symbol include/zmoe.h declares.
SIGNATURES = {
    "zmoe_abi_version": (c_int, []),
    "zmoe_last_error": (c_char_p, []),
    "zmoe_router_softmax_topk": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                         c_void_p, c_void_p]),
    "zmoe_router_sigmoid_bias_topk": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float,
                                              c_void_p, c_void_p, c_void_p]),
    "zmoe_router_logits": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p]),
    "zmoe_route": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_float,
                           c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p]),
    "zmoe_plan_bytes": (c_size_t, [c_int, c_int]),
    "zmoe_build_plan": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "zmoe_gather_qmm_swiglu": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                       c_int, c_void_p]),
    "zmoe_gather_qmm": (c_int, [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p]),
    "zmoe_moe_combine": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int,
                                 c_void_p, c_void_p]),
    "zmoe_gather_qmm_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                        c_int, c_void_p]),
    "zmoe_gather_qmm_combine_noalloc": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                                c_void_p]),
}


class ZmoeError(RuntimeError):
    """A libzmoe call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libzmoe error {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def load() -> ctypes.CDLL:
    """Load ``libzmoe.so`` (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m zmlx_b200.build` "
                "(there is no CPU or PyTorch fallback for these kernels)"
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        if lib.zmoe_abi_version() != 1:
            raise RuntimeError("libzmoe.so ABI version mismatch; rebuild it")
        _lib = lib
    return _lib


def last_error() -> str:
    return load().zmoe_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Map a status code to the exception type the reference raises for it."""
    if rc == OK:
        return
    msg = last_error()
    if rc in (ERR_SHAPE, ERR_DTYPE):
        # the reference raises ValueError for rank/shape/k violations (moe.py:1169-1178, 1261-1265)
        raise ValueError(msg)
    raise ZmoeError(rc, msg)
