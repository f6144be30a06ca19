"""zmlx_b200 -- the MoE decode hot path of ZMLX on NVIDIA B200 (sm_100a).

Router top-k, fused ``gather_qmm_swiglu``, down projection and weighted combine as
hand-written CUDA kernels behind the reference's Python operator surface
(``kernels.moe``, ``kernels.fused_moe``, ``patch``).  The kernels live in
``libzmoe.so`` (C ABI in ``include/zmoe.h``); build it with
``python -m zmlx_b200.build``.  There is no CPU fallback.
"""

__version__ = "0.1.0"

from . import kernels  # noqa: F401,E402
from .kernels import fused_moe, moe  # noqa: F401,E402
from . import patch as _patch_module  # noqa: F401,E402
from .patch import patch, unpatch  # noqa: F401,E402

__all__ = ["kernels", "moe", "fused_moe", "patch", "unpatch", "__version__"]
