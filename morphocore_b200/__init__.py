"""morphocore_b200: B200 (sm_100a) implementation of morphocore's hot path.

Drop-in for the reference's `morphocore.functional.{dilation, erosion, smorph}` and
`morphocore.nn.{Dilation, Erosion, SMorph}` (same signatures, same torch.ops.morphocore schemas).
Everything runs in hand-written CUDA kernels behind a C-ABI (include/morphocore_b200.h); there is no
CPU path and importing the package fails loudly when the native libraries are missing.
"""
__version__ = "0.1.0"

from . import _native  # noqa: F401  (loads the C-ABI library and registers torch.ops.morphocore)
from . import functional, nn  # noqa: F401
from ._native import device_error_count  # noqa: F401

__all__ = ["functional", "nn", "device_error_count", "__version__"]
