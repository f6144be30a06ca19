"""Hot-path kernels behind the reference's module names (``zmlx.kernels.moe``,
``zmlx.kernels.fused_moe``, ``zmlx.kernels.transformer.swiglu2``, ``zmlx.kernels.discovered``)."""

from . import discovered, fused_moe, moe, transformer  # noqa: F401
