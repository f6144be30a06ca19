"""``zmlx.kernels.transformer`` -- the one function of that module that sits on the MoE path.

``swiglu2`` is what the patched block calls between the gate/up and the down projection when it does not take
the fused ``gather_qmm_swiglu`` (src/zmlx/patch/patterns/moe_mlp.py:712-716); the rest of the reference module
(norms, RoPE, attention helpers) is outside this path.
"""

from __future__ import annotations

import warnings
from typing import Any

from .. import _lib, ops

_COMPUTE_DTYPE_DEPRECATION = "compute_dtype is deprecated and ignored: the kernel computes in the tensors' dtype"


def swiglu2(gate: Any, up: Any, *, compute_dtype: Any | None = None) -> Any:
    """y = SiLU(gate) * up for two tensors of the same shape (src/zmlx/kernels/transformer.py:925-1005).

    Arithmetic in the tensors' dtype, op by op, with the reference's stable sigmoid (src/zmlx/msl.py:20-24).
    ``ValueError`` if the shapes differ, as in the reference.
    """
    if compute_dtype is not None:
        warnings.warn(_COMPUTE_DTYPE_DEPRECATION, DeprecationWarning, stacklevel=2)
    if gate.shape != up.shape:
        raise ValueError("swiglu2: gate and up must have the same shape")
    return ops.swiglu(gate, up, mode=_lib.SWIGLU_PER_OP)


__all__ = ["swiglu2"]
