"""Generate the golden fixtures of tests/golden/ from the reference's own CPU implementation.

Run once, in a process of its own, where the reference sources are available:

    python oracle/build_ref.py          # compiles the reference's CPU code into oracle/_ref/_C.so
    python tests/golden/make_golden.py  # writes tests/golden/*.npz and manifest.json
    python tests/golden/make_golden.py scm_small   # only the named sets

Every fixture stores the inputs next to the reference's outputs, so the tests need neither the
reference nor a particular RNG. Full-size benchmark configurations are too large to store: for those
the inputs come from workloads.py (seeded) and the fixture keeps a SHA-256 of the forward output
bytes, the full weight / alpha gradients and the input gradient at sampled positions (set "full_size";
the backward pass of config 4 at its full size is the set "cfg4_full").
"""
import hashlib
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import ref_ops as R  # noqa: E402
import workloads as WL  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
SHAPES = [  # B, Ci, Co, H, W, kH, kW
    (2, 3, 4, 9, 11, 3, 3),
    (1, 2, 2, 13, 4, 5, 5),   # odd image, the reference's own 13x4 / 5x5 case
    (1, 2, 2, 3, 3, 9, 9),    # structuring element larger than the image
    (1, 3, 3, 8, 7, 4, 3),    # even / rectangular structuring element
    (1, 3, 4, 10, 17, 7, 7),
]
PADDINGS = [("zero", 0.0), ("geodesic", 0.0), ("constant", -3.5), ("constant", 7.25), ("replicate", 0.0)]
MERGES = ["max", "min", "sum", "mean", "identity"]


def run_morph(op, merge, padding, pv, x, w, gy):
    xr = x.clone().requires_grad_(True)
    wr = w.clone().requires_grad_(True)
    y = (R.dilation if op == "dilation" else R.erosion)(xr, wr, merge, padding, pv)
    y.backward(gy)
    return y.detach().numpy(), xr.grad.numpy(), wr.grad.numpy()


def morph_cases():
    arrays, manifest = {}, []
    n = 0
    gen = torch.Generator().manual_seed(1234)
    for rep in range(2):
        for oi, op in enumerate(("dilation", "erosion")):
            for mi, merge in enumerate(MERGES):
                for pi, (padding, pv) in enumerate(PADDINGS):
                    B, Ci, Co, H, W, kH, kW = SHAPES[(oi + mi + pi + 2 * rep) % len(SHAPES)]
                    dtype = torch.float32 if (mi + pi + rep) % 2 == 0 else torch.float64
                    ties = rep == 1 and pi % 2 == 0
                    if merge == "identity":
                        Co = Ci
                    wshape = (Co, 1 if merge == "identity" else Ci, kH, kW)
                    if ties:  # small integers: many equal candidates, pins the tie-break rules
                        x = torch.randint(0, 3, (B, Ci, H, W), generator=gen).to(dtype)
                        w = torch.randint(-1, 2, wshape, generator=gen).to(dtype)
                    else:
                        x = torch.randn((B, Ci, H, W), generator=gen, dtype=dtype)
                        w = torch.randn(wshape, generator=gen, dtype=dtype)
                    gy = torch.randn((B, Co, H, W), generator=gen, dtype=dtype)
                    y, gx, gw = run_morph(op, merge, padding, pv, x, w, gy)
                    key = f"m{n}"
                    for name, a in (("x", x.numpy()), ("w", w.numpy()), ("gy", gy.numpy()), ("y", y), ("gx", gx), ("gw", gw)):
                        arrays[f"{key}_{name}"] = a
                    manifest.append(dict(key=key, op=op, merge=merge, padding=padding, padding_value=pv, ties=ties,
                                         dtype=str(dtype).split(".")[1]))
                    n += 1
    return arrays, manifest


def smorph_cases():
    arrays, manifest = {}, []
    gen = torch.Generator().manual_seed(4321)
    n = 0
    alphas = (-1000.0, -8.0, -1.0, -0.1, 0.0, 0.5, 2.0, 8.0, 1000.0)
    for mi, merge in enumerate(MERGES):
        for ai, a0 in enumerate(alphas):
            B, Ci, Co, H, W, kH, kW = SHAPES[(mi + ai) % len(SHAPES)]
            dtype = torch.float32 if (mi + ai) % 2 == 0 else torch.float64
            if merge == "identity":
                Co = Ci
            x = torch.randn((B, Ci, H, W), generator=gen, dtype=dtype)
            w = torch.randn((Co, 1 if merge == "identity" else Ci, kH, kW), generator=gen, dtype=dtype) * 0.5
            ashape = (Co,) if merge == "identity" else (Co, Ci)
            if ai % 3 == 2:
                alpha = torch.tensor([a0], dtype=dtype)  # one alpha shared by every pair
            else:
                alpha = a0 + 0.05 * torch.randn(ashape, generator=gen, dtype=dtype)
            gy = torch.randn((B, Co, H, W), generator=gen, dtype=dtype)
            xr, wr, ar = (t.clone().requires_grad_(True) for t in (x, w, alpha))
            y = R.smorph(xr, wr, ar, merge)   # public-level call: includes the tanh re-parametrisation
            y.backward(gy)
            key = f"s{n}"
            for name, a in (("x", x), ("w", w), ("alpha", alpha), ("gy", gy), ("y", y.detach()), ("gx", xr.grad), ("gw", wr.grad),
                            ("galpha", ar.grad)):
                arrays[f"{key}_{name}"] = a.numpy()
            manifest.append(dict(key=key, merge=merge, alpha0=a0, dtype=str(dtype).split(".")[1]))
            n += 1
    return arrays, manifest


def scm_cases():
    """Smorph with the smooth channel merge (beta per output channel): the reference has no test of its own for
    it, so these outputs of its CPU operator are the only pin."""
    arrays, manifest = {}, []
    gen = torch.Generator().manual_seed(2468)
    betas = (-50.0, -3.0, -0.2, 0.0, 0.7, 4.0, 60.0)
    alphas = (-8.0, -1.0, 0.0, 2.0, 8.0)
    for n, b0 in enumerate(betas):
        B, Ci, Co, H, W, kH, kW = SHAPES[n % len(SHAPES)]
        dtype = torch.float32 if n % 2 == 0 else torch.float64
        a0 = alphas[n % len(alphas)]
        x = torch.randn((B, Ci, H, W), generator=gen, dtype=dtype)
        w = torch.randn((Co, Ci, kH, kW), generator=gen, dtype=dtype) * 0.5
        alpha = torch.tensor([a0], dtype=dtype) if n % 3 == 2 else a0 + 0.5 * torch.randn((Co, Ci), generator=gen, dtype=dtype)
        beta = b0 + 0.1 * torch.randn((Co,), generator=gen, dtype=dtype)
        gy = torch.randn((B, Co, H, W), generator=gen, dtype=dtype)
        xr, wr, ar, br = (t.clone().requires_grad_(True) for t in (x, w, alpha, beta))
        y = R.smorph_scm(xr, wr, ar, br)
        y.backward(gy)
        key = f"c{n}"
        for name, a in (("x", x), ("w", w), ("alpha", alpha), ("beta", beta), ("gy", gy), ("y", y.detach()), ("gx", xr.grad), ("gw", wr.grad),
                        ("galpha", ar.grad), ("gbeta", br.grad)):
            arrays[f"{key}_{name}"] = a.numpy()
        manifest.append(dict(key=key, alpha0=a0, beta0=b0, dtype=str(dtype).split(".")[1]))
    return arrays, manifest


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def sample_positions(numel, count=4096, seed=7):
    return np.random.default_rng(seed).integers(0, numel, size=count)


def full_size_cases():
    """BASELINE configurations at full size (configs 1-3; config 4 at full size for the forward hash and
    reduced to 2 x 8 x 256 x 256 for gradients; config 5 at B = 2)."""
    arrays, manifest = {}, []

    c = WL.cfg1()
    y = R.dilation(c["x"], c["w"], "max")
    manifest.append(dict(key="cfg1", y_sha256=sha(y.numpy())))

    c = WL.cfg2()
    xr, wr = c["x"].clone().requires_grad_(True), c["w"].clone().requires_grad_(True)
    y = R.erosion(xr, wr, "sum")
    y.backward(c["gy"])
    pos = sample_positions(xr.numel())
    arrays["cfg2_gw"] = wr.grad.numpy()
    arrays["cfg2_gx_pos"] = pos
    arrays["cfg2_gx_val"] = xr.grad.numpy().reshape(-1)[pos]
    manifest.append(dict(key="cfg2", y_sha256=sha(y.detach().numpy()), gx_sha256=sha(xr.grad.numpy())))

    for alpha in WL.CFG3_ALPHAS:
        c = WL.cfg3(alpha)
        xr, wr, ar = (c[k].clone().requires_grad_(True) for k in ("x", "w", "alpha"))
        y = R.smorph(xr, wr, ar, "mean")
        y.backward(c["gy"])
        key = f"cfg3_a{alpha:g}"
        pos = sample_positions(xr.numel())
        arrays[f"{key}_pos"] = pos
        arrays[f"{key}_y_val"] = y.detach().numpy().reshape(-1)[pos]
        arrays[f"{key}_gx_val"] = xr.grad.numpy().reshape(-1)[pos]
        if alpha in (-8.0, 2.0):
            arrays[f"{key}_gw"] = wr.grad.numpy()
        else:  # the full weight gradient is 200 KB per alpha: keep sampled entries for the others
            wpos = sample_positions(wr.numel(), 2048, seed=11)
            arrays[f"{key}_gw_pos"] = wpos
            arrays[f"{key}_gw_val"] = wr.grad.numpy().reshape(-1)[wpos]
        arrays[f"{key}_galpha"] = ar.grad.numpy()
        manifest.append(dict(key=key, alpha=alpha))

    for op in ("dilation", "erosion"):
        c = WL.cfg4(op)
        f = R.dilation if op == "dilation" else R.erosion
        y = f(c["x"], c["w"], "identity")
        manifest.append(dict(key=f"cfg4_{op}", y_sha256=sha(y.numpy())))
        del y
        c = WL.cfg4(op, B=2, C=8, HW=256)
        xr, wr = c["x"].clone().requires_grad_(True), c["w"].clone().requires_grad_(True)
        y = f(xr, wr, "identity")
        y.backward(c["gy"])
        pos = sample_positions(xr.numel())
        arrays[f"cfg4s_{op}_gw"] = wr.grad.numpy()
        arrays[f"cfg4s_{op}_gx_pos"] = pos
        arrays[f"cfg4s_{op}_gx_val"] = xr.grad.numpy().reshape(-1)[pos]
        manifest.append(dict(key=f"cfg4s_{op}", y_sha256=sha(y.detach().numpy()), gx_sha256=sha(xr.grad.numpy())))

    # config 5: the 4-layer stack at B = 2, MSE loss against the target
    x, target = WL.cfg5_batch(B=256, start=0, count=2)
    ws = [w.clone().requires_grad_(True) for w in WL.cfg5_weights()]
    alphas = {}
    h = x
    for n, (kind, ci, co, k, merge, a0) in enumerate(WL.CFG5_LAYERS):
        if kind == "dilation":
            h = R.dilation(h, ws[n], merge)
        elif kind == "erosion":
            h = R.erosion(h, ws[n], merge)
        else:
            alphas[n] = torch.full((co, ci), a0, dtype=torch.float32, requires_grad=True)
            h = R.smorph(h, ws[n], alphas[n], merge)
    loss = torch.nn.functional.mse_loss(h, target)
    loss.backward()
    arrays["cfg5_loss"] = np.array([loss.item()], dtype=np.float64)
    pos = sample_positions(h.numel())
    arrays["cfg5_out_pos"] = pos
    arrays["cfg5_out_val"] = h.detach().numpy().reshape(-1)[pos]
    for n, w in enumerate(ws):
        arrays[f"cfg5_gw{n}"] = w.grad.numpy()
    for n, a in alphas.items():
        arrays[f"cfg5_galpha{n}"] = a.grad.numpy()
    manifest.append(dict(key="cfg5", B=2))
    return arrays, manifest


def cfg4_full_cases():
    """Config 4 at its full size (8, 64, 512, 512), backward: the whole weight gradient and the input gradient at
    sampled positions, for both operations."""
    arrays, manifest = {}, []
    for op in ("dilation", "erosion"):
        c = WL.cfg4(op)
        f = R.dilation if op == "dilation" else R.erosion
        xr, wr = c["x"].clone().requires_grad_(True), c["w"].clone().requires_grad_(True)
        y = f(xr, wr, "identity")
        y.backward(c["gy"])
        pos = sample_positions(xr.numel(), 8192, seed=13)
        arrays[f"cfg4_{op}_gw"] = wr.grad.numpy()
        arrays[f"cfg4_{op}_gx_pos"] = pos
        arrays[f"cfg4_{op}_gx_val"] = xr.grad.numpy().reshape(-1)[pos]
        manifest.append(dict(key=f"cfg4_{op}", y_sha256=sha(y.detach().numpy()), gx_sha256=sha(xr.grad.numpy())))
        del xr, wr, y
    return arrays, manifest


if __name__ == "__main__":
    torch.set_num_threads(os.cpu_count())
    # Without arguments every set is regenerated; otherwise only the named ones (the manifest keeps the others).
    manifest_path = os.path.join(HERE, "manifest.json")
    out = {}
    if len(sys.argv) > 1 and os.path.exists(manifest_path):
        with open(manifest_path) as f:
            out = json.load(f)
    for name, fn in (("morph_small", morph_cases), ("smorph_small", smorph_cases), ("scm_small", scm_cases), ("full_size", full_size_cases),
                     ("cfg4_full", cfg4_full_cases)):
        if len(sys.argv) > 1 and name not in sys.argv[1:]:
            continue
        arrays, manifest = fn()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **arrays)
        out[name] = manifest
        print(name, len(manifest), "cases", os.path.getsize(os.path.join(HERE, name + ".npz")) // 1024, "KiB", flush=True)
    with open(manifest_path, "w") as f:
        json.dump(out, f, indent=1)
