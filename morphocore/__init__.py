"""The reference's package name, served by the B200 implementation.

`import morphocore.functional as F` and `import morphocore.nn as Mnn` (the imports of the reference's users and of
its own tests, tests/functional/utils.py:3) resolve to morphocore_b200.functional and morphocore_b200.nn, so that
switching needs no change in user code. Do not install this next to the reference itself: both own the name.
"""
import sys

import morphocore_b200 as _impl
from morphocore_b200 import __version__, functional, nn  # noqa: F401

sys.modules[__name__ + ".functional"] = functional
sys.modules[__name__ + ".nn"] = nn
_C = _impl._native

__all__ = ["functional", "nn", "__version__"]
