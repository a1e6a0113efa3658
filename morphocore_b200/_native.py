"""Loads the native libraries: the C-ABI kernels (ctypes handle in `lib`) and the PyTorch operator
extension, which registers torch.ops.morphocore.{dilation, erosion, smorph, smorph_scm}."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmorphocore_b200.so")
EXT_PATH = os.path.join(_HERE, "_C.so")

for _path in (LIB_PATH, EXT_PATH):
    if not os.path.exists(_path):
        raise ImportError(
            f"morphocore_b200: native library {_path} is missing. Build it with `python morphocore_b200/build.py` "
            "(needs nvcc with sm_100a support); there is no CPU or pure-PyTorch fallback.")

lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
lib.mc_status_string.restype = ctypes.c_char_p
lib.mc_last_error.restype = ctypes.c_char_p
lib.mc_launch_count.restype = ctypes.c_uint64
lib.mc_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
lib.mc_selftest_wait_timeout.argtypes = [ctypes.c_uint64, ctypes.c_void_p]
lib.mc_morpho_backward_workspace_bytes.restype = ctypes.c_size_t
lib.mc_smorph_backward_workspace_bytes.restype = ctypes.c_size_t
lib.mc_smorph_scm_backward_workspace_bytes.restype = ctypes.c_size_t
torch.ops.load_library(EXT_PATH)
ops = torch.ops.morphocore


def device_error_count() -> int:
    """Thread blocks on the current device whose bounded wait on an asynchronous copy ran out (they returned without
    writing their tile): 0 in a healthy run. Synchronises the device; poll it where the host synchronises anyway."""
    count = int(lib.mc_device_error_count())
    if count < 0:
        raise RuntimeError(f"{lib.mc_status_string(count).decode()}: {lib.mc_last_error().decode()}")
    return count


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.mc_launch_count())
