"""numpy front end of the C oracle (libmorpho_oracle.so).

TEST INFRASTRUCTURE ONLY: a CPU restatement of the reference's algorithm used to check the CUDA
kernels. Only tests/, the smoke check and the benchmark's CPU-baseline leg may import this module.

The functions take and return numpy arrays (float32 or float64, C-contiguous NCHW / OIHW) and mirror
the reference's operator level: `weight` is what torch.ops.morphocore.<op> receives, that is the
already flipped structuring element for erosion and the re-parametrised one for smorph.
"""
import ctypes
import os

import numpy as np

MERGES = {"max": 0, "min": 1, "sum": 2, "mean": 3, "identity": 5}
PADDINGS = {"zero": 0, "geodesic": 1, "constant": 2, "replicate": 3}

_lib = None


class _Desc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("Ci", ctypes.c_int32), ("Co", ctypes.c_int32), ("H", ctypes.c_int32),
                ("W", ctypes.c_int32), ("kH", ctypes.c_int32), ("kW", ctypes.c_int32), ("op", ctypes.c_int32),
                ("merge", ctypes.c_int32), ("pad_kind", ctypes.c_int32), ("fill", ctypes.c_double),
                ("weight_batch_stride", ctypes.c_int64)]


def lib():
    global _lib
    if _lib is None:
        here = os.path.dirname(os.path.abspath(__file__))
        path = os.path.join(here, "libmorpho_oracle.so")
        if not os.path.exists(path):
            from . import build_oracle
            build_oracle.build()
        _lib = ctypes.CDLL(path)
    return _lib


def fill_value(op, padding, padding_value, dtype):
    """Border value of the FILL family: 0, the caller's constant, or the neutral element of the
    operation for geodesic padding (reference: csrc/cpp/morpho_padding_policy.hpp:23-33)."""
    if padding == "zero":
        return 0.0
    if padding == "constant":
        return float(np.asarray(padding_value, dtype=dtype))
    return -np.inf if op == "dilation" else np.inf


def _desc(op, x, w, merge, padding="replicate", padding_value=0.0):
    B, Ci, H, W = x.shape
    per_sample = w.ndim == 5
    Co, wCi, kH, kW = w.shape[-4:]
    if merge == "identity":
        assert Co == Ci and wCi == 1, "identity needs weight [C, 1, kH, kW]"
    else:
        assert wCi == Ci
    d = _Desc(B, Ci, Co, H, W, kH, kW, 0 if op == "dilation" else 1, MERGES[merge],
              1 if padding == "replicate" else 0, fill_value(op, padding, padding_value, x.dtype),
              Co * wCi * kH * kW if per_sample else 0)
    return d


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _suffix(x):
    return {np.dtype(np.float32): "_f32", np.dtype(np.float64): "_f64"}[x.dtype]


def morpho_forward(op, x, w, merge="sum", padding="replicate", padding_value=0.0, with_index=False):
    """op in {"dilation", "erosion"}; erosion computes min(x - w) with w as given (already flipped)."""
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    d = _desc(op, x, w, merge, padding, padding_value)
    y = np.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype)
    idx = np.empty(y.shape, dtype=np.int32) if with_index else None
    getattr(lib(), "orc_morpho_forward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(y), _p(idx))
    return (y, idx) if with_index else y


def morpho_backward(op, x, w, gy, merge="sum", padding="replicate", padding_value=0.0, idx=None):
    """Returns (grad_input, grad_weight); grad_weight is with respect to `w` as given."""
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    gy = np.ascontiguousarray(gy, dtype=x.dtype)
    d = _desc(op, x, w, merge, padding, padding_value)
    gx = np.empty_like(x)
    gw = np.empty(w.shape[-4:], dtype=x.dtype)
    if idx is not None:
        idx = np.ascontiguousarray(idx, dtype=np.int32)
    getattr(lib(), "orc_morpho_backward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(idx), _p(gy), _p(gx), _p(gw))
    return gx, gw


def pair_alphas(alpha, Co, Ci, merge, dtype):
    """One alpha per (o, i) pair ([Co] for identity); a single value is broadcast
    (reference: csrc/cpp/smorph_cpu_kernels.hxx:643-649)."""
    pairs = Co if merge == "identity" else Co * Ci
    alpha = np.asarray(alpha, dtype=dtype).reshape(-1)
    if alpha.size == 1:
        return np.full(pairs, alpha[0], dtype=dtype)
    assert alpha.size == pairs, "alpha must have one value or one per channel pair"
    return np.ascontiguousarray(alpha)


def smorph_forward(x, w, alpha, merge="sum"):
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    d = _desc("dilation", x, w, merge)
    a = pair_alphas(alpha, d.Co, d.Ci, merge, x.dtype)
    y = np.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype)
    getattr(lib(), "orc_smorph_forward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(a), _p(y))
    return y


def smorph_backward(x, w, alpha, gy, merge="sum"):
    """Returns (grad_input, grad_weight, grad_alpha_pairs)."""
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    gy = np.ascontiguousarray(gy, dtype=x.dtype)
    d = _desc("dilation", x, w, merge)
    a = pair_alphas(alpha, d.Co, d.Ci, merge, x.dtype)
    gx = np.empty_like(x)
    gw = np.empty_like(w)
    ga = np.empty_like(a)
    getattr(lib(), "orc_smorph_backward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(a), _p(gy), _p(gx), _p(gw), _p(ga))
    return gx, gw, ga


def smorph_weight(w, alpha, merge="sum"):
    """The Python-level re-parametrisation the reference applies before its smorph operator:
    w~ = tanh(a) * ((1 - tanh a)/2 * flip(w) + (1 + tanh a)/2 * w)
    (reference: morphocore/functional/smorph.py:56-70)."""
    alpha = np.asarray(alpha, dtype=w.dtype)
    t = np.tanh(alpha)
    t = t.reshape(-1, 1, 1, 1) if (merge == "identity" or alpha.ndim == 1) else t[..., None, None]
    return (t * ((1 - t) / 2 * w[..., ::-1, ::-1] + (1 + t) / 2 * w)).astype(w.dtype)


def smorph_scm_forward(x, w, alpha, beta):
    """Smorph with the smooth channel merge: `w` is the re-parametrised structuring element, alpha one value per
    pair (or a single value), beta one value per output channel."""
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    d = _desc("dilation", x, w, "sum")
    a = pair_alphas(alpha, d.Co, d.Ci, "sum", x.dtype)
    bt = np.ascontiguousarray(np.asarray(beta, dtype=x.dtype).reshape(-1))
    assert bt.size == d.Co, "beta must have one value per output channel"
    y = np.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype)
    getattr(lib(), "orc_smorph_scm_forward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(a), _p(bt), _p(y))
    return y


def smorph_scm_backward(x, w, alpha, beta, gy):
    """Returns (grad_input, grad_weight, grad_alpha_pairs, grad_beta)."""
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w, dtype=x.dtype)
    gy = np.ascontiguousarray(gy, dtype=x.dtype)
    d = _desc("dilation", x, w, "sum")
    a = pair_alphas(alpha, d.Co, d.Ci, "sum", x.dtype)
    bt = np.ascontiguousarray(np.asarray(beta, dtype=x.dtype).reshape(-1))
    assert bt.size == d.Co, "beta must have one value per output channel"
    gx, gw, ga, gb = np.empty_like(x), np.empty_like(w), np.empty_like(a), np.empty_like(bt)
    getattr(lib(), "orc_smorph_scm_backward" + _suffix(x))(ctypes.byref(d), _p(x), _p(w), _p(a), _p(bt), _p(gy), _p(gx), _p(gw), _p(ga), _p(gb))
    return gx, gw, ga, gb
