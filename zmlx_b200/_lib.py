"""ctypes binding of ``libzmoe.so`` (the C ABI declared in ``include/zmoe.h``).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  ``ZmoeError`` carries the library's own message.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
# ZMOE_LIB selects another build of the same ABI
LIB_PATH = os.environ.get("ZMOE_LIB") or os.path.join(_HERE, "libzmoe.so")

OK = 0
ABI_VERSION = 2
DEBUG_WITHHOLD_LOGIT = 1
DEBUG_FORCE_INBOX = 2
ERR_SHAPE, ERR_DTYPE, ERR_ALIGN, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_WORKSPACE = -1, -2, -3, -4, -5, -6, -7
F32, BF16 = 0, 1
Q_AFFINE4, Q_MXFP4 = 0, 1
SWIGLU_CPU, SWIGLU_PER_OP, SWIGLU_FP32 = 0, 1, 2
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



class ExpertBank(ctypes.Structure):
    """``zmoe_expert_bank``: device pointers of one bank's packed gate/up/down tensors."""

    _fields_ = [(n, c_void_p) for n in ("gate_w", "gate_scales", "gate_biases", "up_w", "up_scales", "up_biases",
                                        "down_w", "down_scales", "down_biases")]


class LayerDesc(ctypes.Structure):
    """``zmoe_layer_desc``: one MoE block for ``zmoe_layer_decode``."""

    _fields_ = ([(n, ctypes.c_int32) for n in ("E", "d_model", "d_ff", "top_k", "group_size", "qmode",
                                               "router_family", "renorm", "n_group", "topk_group")]
                + [("routed_scale", c_float)]
                + [(n, ctypes.c_int32) for n in ("n_shared", "swiglu_mode", "shared_swiglu_mode", "combine_mode",
                                                 "out_flags", "launch_mode")]
                + [("router_w", c_void_p), ("router_bias", c_void_p), ("routed", ExpertBank), ("shared", ExpertBank)]
                + [("debug_flags", ctypes.c_int32), ("reserved", ctypes.c_int32), ("debug_stamps", c_void_p)]
                + [("ep_world", ctypes.c_int32), ("ep_rank", ctypes.c_int32), ("ep_inbox", c_void_p * 8)])


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
    "zmoe_swiglu": (c_int, [c_void_p, c_void_p, ctypes.c_longlong, c_int, c_void_p, c_void_p]),
    "zmoe_gather_qmm_combine": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                        c_int, c_void_p]),
    "zmoe_gather_qmm_combine_noalloc": (c_int, [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_int,
                                                c_void_p]),
    "zmoe_layer_decode_workspace_bytes": (c_size_t, [ctypes.POINTER(LayerDesc), c_int]),
    "zmoe_layer_decode": (c_int, [ctypes.POINTER(LayerDesc), c_void_p, c_int, c_int, c_void_p, c_size_t, c_void_p,
                                  c_void_p, c_void_p, c_void_p]),
    "zmoe_layer_decode_status": (c_int, [c_void_p, c_int, c_void_p]),
    "zmoe_layer_decode_inbox_bytes": (c_size_t, [ctypes.POINTER(LayerDesc), c_int]),
    "zmoe_ep_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p)]),
    "zmoe_ep_free": (c_int, [c_void_p]),
    "zmoe_ep_export": (c_int, [c_void_p, c_void_p]),
    "zmoe_ep_import": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "zmoe_ep_unmap": (c_int, [c_void_p]),
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
        if lib.zmoe_abi_version() != ABI_VERSION:
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
