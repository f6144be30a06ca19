"""Hot-path kernels behind the reference's module names (``zmlx.kernels.moe``,
``zmlx.kernels.fused_moe``)."""

from . import fused_moe, moe  # noqa: F401
