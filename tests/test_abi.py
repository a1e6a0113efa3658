"""The C-ABI library loads, exports every function the header declares and validates its arguments
before touching the GPU. CPU only: no kernel is launched."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    path = os.path.join(ROOT, "morphocore_b200", "libmorphocore_b200.so")
    assert os.path.exists(path), "build the library with `python morphocore_b200/build.py`"
    handle = ctypes.CDLL(path)
    handle.mc_status_string.restype = ctypes.c_char_p
    handle.mc_last_error.restype = ctypes.c_char_p
    handle.mc_morpho_backward_workspace_bytes.restype = ctypes.c_size_t
    handle.mc_smorph_backward_workspace_bytes.restype = ctypes.c_size_t
    return handle


def declared_functions():
    text = open(os.path.join(ROOT, "include", "morphocore_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = declared_functions()
    for expected in ("mc_morpho_forward", "mc_morpho_backward", "mc_smorph_forward", "mc_smorph_backward", "mc_device_error_count",
                     "mc_morpho_backward_workspace_bytes", "mc_smorph_backward_workspace_bytes", "mc_status_string"):
        assert expected in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


class Desc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("Ci", ctypes.c_int32), ("Co", ctypes.c_int32), ("H", ctypes.c_int32),
                ("W", ctypes.c_int32), ("kH", ctypes.c_int32), ("kW", ctypes.c_int32), ("op", ctypes.c_int32),
                ("merge", ctypes.c_int32), ("pad_kind", ctypes.c_int32), ("dtype", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("fill", ctypes.c_double), ("weight_batch_stride", ctypes.c_int64)]


def desc(**kw):
    base = dict(B=1, Ci=2, Co=2, H=8, W=8, kH=3, kW=3, op=0, merge=2, pad_kind=1, dtype=0, reserved=0, fill=0.0, weight_batch_stride=0)
    base.update(kw)
    return Desc(**base)


def test_desc_layout_matches_header():
    assert ctypes.sizeof(Desc) == 12 * 4 + 8 + 8


def test_status_strings(lib):
    assert lib.mc_status_string(0) == b"ok"
    assert lib.mc_status_string(-1) == b"invalid argument"
    assert lib.mc_status_string(-2) == b"unsupported configuration"
    assert lib.mc_status_string(-3) == b"workspace too small"
    assert lib.mc_version() >= 100


def test_validation_happens_before_any_launch(lib):
    one = ctypes.c_void_p(16)  # never dereferenced: every call below fails validation first
    assert lib.mc_morpho_forward(None, one, one, one, None, None) == -1
    assert lib.mc_morpho_forward(ctypes.byref(desc(merge=9)), one, one, one, None, None) == -1
    assert b"Unknown merge mode" in lib.mc_last_error()
    assert lib.mc_morpho_forward(ctypes.byref(desc(merge=4)), one, one, one, None, None) == -2
    assert lib.mc_morpho_forward(ctypes.byref(desc(merge=5, Co=3)), one, one, one, None, None) == -1
    assert b"Identity mode requires" in lib.mc_last_error()
    assert lib.mc_morpho_forward(ctypes.byref(desc(kH=0)), one, one, one, None, None) == -1
    assert lib.mc_morpho_forward(ctypes.byref(desc(dtype=3)), one, one, one, None, None) == -1
    assert lib.mc_morpho_forward(ctypes.byref(desc(kH=300, kW=300)), one, one, one, None, None) == -2
    assert lib.mc_morpho_forward(ctypes.byref(desc()), None, one, one, None, None) == -1
    assert lib.mc_smorph_forward(ctypes.byref(desc(weight_batch_stride=5)), one, one, one, one, None) == -1
    # the entry point with built-in scratch validates before it sizes anything from the descriptor
    assert lib.mc_morpho_backward_noalloc(ctypes.byref(desc(B=-1, merge=0)), one, one, one, one, one, None) == -1
    assert b"sizes must be positive" in lib.mc_last_error()
    assert lib.mc_morpho_backward_noalloc(ctypes.byref(desc(merge=9)), one, one, one, one, one, None) == -1
    assert lib.mc_morpho_forward(ctypes.byref(desc(B=2**20, Co=2**20, H=2**20, W=2**20)), one, one, one, None, None) == -1
    assert b"2^40" in lib.mc_last_error()
    lib.mc_set_wait_limit_ns.argtypes = [ctypes.c_uint64]
    assert lib.mc_set_wait_limit_ns(0) == -1 and lib.mc_set_wait_limit_ns(10**9) == 0
    # an empty batch is a valid no-op
    assert lib.mc_morpho_forward(ctypes.byref(desc(B=0)), None, None, None, None, None) == 0
    assert lib.mc_launch_count() == 0


def test_workspace_sizes(lib):
    d = desc(B=3, Co=5, H=7, W=11, merge=0)
    assert lib.mc_morpho_backward_workspace_bytes(ctypes.byref(d), 0) == 4 * 3 * 5 * 7 * 11
    assert lib.mc_morpho_backward_workspace_bytes(ctypes.byref(d), 1) == 0
    assert lib.mc_morpho_backward_workspace_bytes(ctypes.byref(desc(merge=2)), 0) == 0
    assert lib.mc_smorph_backward_workspace_bytes(ctypes.byref(desc(merge=1, dtype=1))) == 8 * 1 * 2 * 8 * 8
    assert lib.mc_smorph_backward_workspace_bytes(ctypes.byref(desc(merge=3))) == 0
    # a missing workspace is reported, not dereferenced
    one = ctypes.c_void_p(16)
    assert lib.mc_morpho_backward(ctypes.byref(d), one, one, None, one, one, one, None, ctypes.c_size_t(0), None) == -3
