"""Synthetic workloads of the five benchmark configurations (shapes, seeds, distributions) and their
tap counts. Pure torch, imports neither the CUDA package nor the oracle, so that the golden-vector
generator, the tests and bench.py all draw bit-identical inputs.

N_taps = B * Co * Ci_eff * H * W * kH * kW, with Ci_eff = 1 for the identity merge, counted once per
forward or per forward+backward pair.
"""
import torch


def _rand(shape, seed, dtype, dist, scale=1.0, lo=0.0, hi=1.0):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        return torch.rand(shape, generator=g, dtype=dtype) * (hi - lo) + lo
    return torch.randn(shape, generator=g, dtype=dtype) * scale


def taps(B, Co, Ci, H, W, kH, kW, identity=False):
    return B * Co * (1 if identity else Ci) * H * W * kH * kW


def cfg1(B=8):
    """dilation forward only, fp32, merge max, replicate padding."""
    x = _rand((B, 3, 128, 128), 0, torch.float32, "uniform")
    w = _rand((16, 3, 3, 3), 1, torch.float32, "normal", 0.1)
    return dict(name="cfg1", op="dilation", merge="max", x=x, w=w, gy=None, n_taps=taps(B, 16, 3, 128, 128, 3, 3))


def cfg2(B=32):
    """erosion forward+backward, fp32, merge sum."""
    x = _rand((B, 16, 256, 256), 0, torch.float32, "uniform")
    w = _rand((32, 16, 5, 5), 1, torch.float32, "normal", 0.1)
    gy = _rand((B, 32, 256, 256), 2, torch.float32, "normal")
    return dict(name="cfg2", op="erosion", merge="sum", x=x, w=w, gy=gy, n_taps=taps(B, 32, 16, 256, 256, 5, 5))


CFG3_ALPHAS = (-8.0, -1.0, 0.0, 2.0, 8.0)


def cfg3(alpha, B=16):
    """smorph forward+backward, fp32, merge mean, alpha tensor (32, 32) filled with one sweep value."""
    x = _rand((B, 32, 128, 128), 0, torch.float32, "normal")
    w = _rand((32, 32, 7, 7), 1, torch.float32, "normal", 0.05)
    gy = _rand((B, 32, 128, 128), 2, torch.float32, "normal")
    a = torch.full((32, 32), float(alpha), dtype=torch.float32)
    return dict(name="cfg3", op="smorph", merge="mean", x=x, w=w, alpha=a, gy=gy, n_taps=taps(B, 32, 32, 128, 128, 7, 7))


def cfg4(op, B=8, C=64, HW=512):
    """dilation or erosion forward+backward, fp64, merge identity. The weight is [:, :1] of the
    (C, C, 11, 11) draw because identity mode takes a (C, 1, kH, kW) structuring element."""
    x = _rand((B, C, HW, HW), 0, torch.float64, "uniform", lo=-1.0, hi=1.0)
    w = _rand((C, C, 11, 11), 1, torch.float64, "normal", 0.1)[:, :1].contiguous()
    gy = _rand((B, C, HW, HW), 2, torch.float64, "normal")
    return dict(name="cfg4", op=op, merge="identity", x=x, w=w, gy=gy, n_taps=taps(B, C, C, HW, HW, 11, 11, identity=True))


CFG5_LAYERS = (
    # kind, Ci, Co, k, merge, init_alpha
    ("dilation", 3, 64, 3, "sum", None),
    ("smorph", 64, 64, 3, "sum", 2.0),
    ("erosion", 64, 64, 5, "max", None),
    ("smorph", 64, 64, 3, "mean", -2.0),
)


def cfg5_weights():
    """The modules initialise their weights to zero, which ties every tap; the workload sets
    w ~ N(0, 0.1^2) with seed 10 + layer instead."""
    return [_rand((co, ci, k, k), 10 + n, torch.float32, "normal", 0.1) for n, (_, ci, co, k, _, _) in enumerate(CFG5_LAYERS)]


def cfg5_taps(B, HW=224):
    return sum(taps(B, co, ci, HW, HW, k, k) for (_, ci, co, k, _, _) in CFG5_LAYERS)


def cfg5_batch(B=256, HW=224, start=0, count=None):
    """Images [start, start+count) of the global batch: x ~ U[0,1) seed 0, target ~ N(0,1) seed 1.
    Each image is drawn from its own generator so that any shard of the batch can be produced alone."""
    count = B - start if count is None else count
    xs, ts = [], []
    for b in range(start, start + count):
        xs.append(_rand((3, HW, HW), 1000003 * b + 0, torch.float32, "uniform"))
        ts.append(_rand((64, HW, HW), 1000003 * b + 1, torch.float32, "normal"))
    return torch.stack(xs), torch.stack(ts)
