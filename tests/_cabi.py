"""Direct ctypes calls into the C-ABI of include/morphocore_b200.h, with torch CUDA tensors as device
memory. The parity tests go through these, not through the PyTorch operators, so that they exercise
exactly what a foreign-language binding would call."""
import ctypes

import torch

from morphocore_b200 import _native

MERGES = {"max": 0, "min": 1, "sum": 2, "mean": 3, "smooth": 4, "identity": 5}


class Desc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("Ci", ctypes.c_int32), ("Co", ctypes.c_int32), ("H", ctypes.c_int32),
                ("W", ctypes.c_int32), ("kH", ctypes.c_int32), ("kW", ctypes.c_int32), ("op", ctypes.c_int32),
                ("merge", ctypes.c_int32), ("pad_kind", ctypes.c_int32), ("dtype", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("fill", ctypes.c_double), ("weight_batch_stride", ctypes.c_int64)]


lib = _native.lib


def check(rc):
    if rc != 0:
        raise RuntimeError(f"{lib.mc_status_string(rc).decode()}: {lib.mc_last_error().decode()}")


def fill_value(op, padding, padding_value, dtype):
    if padding == "zero":
        return 0.0
    if padding == "constant":
        return float(torch.tensor(padding_value, dtype=dtype))
    return float("-inf") if op == "dilation" else float("inf")


def make_desc(op, x, w, merge, padding="replicate", padding_value=0.0):
    B, Ci, H, W = x.shape
    Co, _, kH, kW = w.shape[-4:]
    return Desc(B, Ci, Co, H, W, kH, kW, 0 if op == "dilation" else 1, MERGES[merge], 1 if padding == "replicate" else 0,
                0 if x.dtype == torch.float32 else 1, 0, fill_value(op, padding, padding_value, x.dtype),
                w[0].numel() if w.dim() == 5 else 0)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def morpho_forward(op, x, w, merge="sum", padding="replicate", padding_value=0.0, with_index=False):
    d = make_desc(op, x, w, merge, padding, padding_value)
    y = torch.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype, device=x.device)
    idx = torch.full(y.shape, -1, dtype=torch.int32, device=x.device) if with_index else None
    check(lib.mc_morpho_forward(ctypes.byref(d), ptr(x), ptr(w), ptr(y), ptr(idx), stream()))
    return (y, idx) if with_index else y


def morpho_pair_forward(x, w, merge="sum", padding="replicate", padding_value=0.0):
    """Dilation and erosion (flipped structuring element) of x in one pass; None when the case is not covered."""
    d = make_desc("dilation", x, w, merge, padding, padding_value)
    yd = torch.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype, device=x.device)
    ye = torch.empty_like(yd)
    rc = lib.mc_morpho_pair_forward(ctypes.byref(d), ptr(x), ptr(w), ptr(yd), ptr(ye), stream())
    if rc == -2:   # MC_ERR_UNSUPPORTED
        return None
    check(rc)
    return yd, ye


def morpho_backward(op, x, w, gy, merge="sum", padding="replicate", padding_value=0.0, idx=None):
    d = make_desc(op, x, w, merge, padding, padding_value)
    gx = torch.empty_like(x)
    gw = torch.empty(w.shape[-4:], dtype=x.dtype, device=x.device)
    need = lib.mc_morpho_backward_workspace_bytes(ctypes.byref(d), 1 if idx is not None else 0)
    ws = torch.empty(need, dtype=torch.uint8, device=x.device) if need else None
    check(lib.mc_morpho_backward(ctypes.byref(d), ptr(x), ptr(w), ptr(idx), ptr(gy), ptr(gx), ptr(gw), ptr(ws), ctypes.c_size_t(need), stream()))
    return gx, gw


def pair_alphas(alpha, Co, Ci, merge):
    pairs = Co if merge == "identity" else Co * Ci
    alpha = alpha.reshape(-1)
    return alpha.expand(pairs).contiguous() if alpha.numel() == 1 else alpha.contiguous()


def smorph_forward(x, w, alpha, merge="sum"):
    d = make_desc("dilation", x, w, merge)
    a = pair_alphas(alpha, d.Co, d.Ci, merge)
    y = torch.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype, device=x.device)
    check(lib.mc_smorph_forward(ctypes.byref(d), ptr(x), ptr(w), ptr(a), ptr(y), stream()))
    return y


def smorph_backward(x, w, alpha, y, gy, merge="sum"):
    d = make_desc("dilation", x, w, merge)
    a = pair_alphas(alpha, d.Co, d.Ci, merge)
    gx, gw, ga = torch.empty_like(x), torch.empty_like(w), torch.empty_like(a)
    need = lib.mc_smorph_backward_workspace_bytes(ctypes.byref(d))
    ws = torch.empty(need, dtype=torch.uint8, device=x.device) if need else None
    check(lib.mc_smorph_backward(ctypes.byref(d), ptr(x), ptr(w), ptr(a), ptr(y), ptr(gy), ptr(gx), ptr(gw), ptr(ga), ptr(ws),
                                 ctypes.c_size_t(need), stream()))
    return gx, gw, ga


def smorph_scm_forward(x, w, alpha, beta):
    d = make_desc("dilation", x, w, "smooth")
    a = pair_alphas(alpha, d.Co, d.Ci, "sum")
    y = torch.empty((d.B, d.Co, d.H, d.W), dtype=x.dtype, device=x.device)
    check(lib.mc_smorph_scm_forward(ctypes.byref(d), ptr(x), ptr(w), ptr(a), ptr(beta), ptr(y), stream()))
    return y


def smorph_scm_backward(x, w, alpha, beta, y, gy):
    d = make_desc("dilation", x, w, "smooth")
    a = pair_alphas(alpha, d.Co, d.Ci, "sum")
    gx, gw, ga, gb = torch.empty_like(x), torch.empty_like(w), torch.empty_like(a), torch.empty_like(beta)
    need = lib.mc_smorph_scm_backward_workspace_bytes(ctypes.byref(d))
    ws = torch.empty(need, dtype=torch.uint8, device=x.device)
    check(lib.mc_smorph_scm_backward(ctypes.byref(d), ptr(x), ptr(w), ptr(a), ptr(beta), ptr(y), ptr(gy), ptr(gx), ptr(gw), ptr(ga), ptr(gb),
                                     ptr(ws), ctypes.c_size_t(need), stream()))
    return gx, gw, ga, gb
