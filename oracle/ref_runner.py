"""Times the reference's own CPU implementation (oracle/_ref/_C.so) on a benchmark workload.

TEST / BENCHMARK INFRASTRUCTURE ONLY. Runs in a process of its own because the reference registers the
same torch.ops.morphocore namespace as the CUDA package. Prints one JSON object:
{"seconds": [per-step times], "n_taps": taps per step, "cores": threads used, "sample": "..."}.

Usage: python oracle/ref_runner.py --workload cfg5 --batch 8 --steps 1 --warmup 1
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import ref_ops as R  # noqa: E402
import workloads as WL  # noqa: E402


def step_fn(workload, batch):
    if workload == "cfg1":
        c = WL.cfg1(B=batch)
        return (lambda: R.dilation(c["x"], c["w"], "max")), c["n_taps"], f"config 1 at B={batch}, forward only"
    if workload == "cfg2":
        c = WL.cfg2(B=batch)

        def run():
            x, w = c["x"].requires_grad_(True), c["w"].requires_grad_(True)
            x.grad = w.grad = None
            R.erosion(x, w, "sum").backward(c["gy"])
        return run, c["n_taps"], f"config 2 at B={batch}, forward+backward"
    if workload == "cfg3":
        c = WL.cfg3(2.0, B=batch)

        def run():
            x, w, a = c["x"].requires_grad_(True), c["w"].requires_grad_(True), c["alpha"].requires_grad_(True)
            x.grad = w.grad = a.grad = None
            R.smorph(x, w, a, "mean").backward(c["gy"])
        return run, c["n_taps"], f"config 3 (alpha=2) at B={batch}, forward+backward"
    if workload == "cfg4":
        c = WL.cfg4("dilation", B=batch)

        def run():
            x, w = c["x"].requires_grad_(True), c["w"].requires_grad_(True)
            x.grad = w.grad = None
            R.dilation(x, w, "identity").backward(c["gy"])
        return run, c["n_taps"], f"config 4 (dilation) at B={batch}, forward+backward"
    if workload == "cfg5":
        x, target = WL.cfg5_batch(B=256, start=0, count=batch)
        ws = [w.clone().requires_grad_(True) for w in WL.cfg5_weights()]
        alphas = {n: torch.full((co, ci), a0, requires_grad=True) for n, (kind, ci, co, k, m, a0) in enumerate(WL.CFG5_LAYERS) if kind == "smorph"}
        params = ws + list(alphas.values())

        def run():
            for p in params:
                p.grad = None
            h = x
            for n, (kind, ci, co, k, merge, a0) in enumerate(WL.CFG5_LAYERS):
                if kind == "dilation":
                    h = R.dilation(h, ws[n], merge)
                elif kind == "erosion":
                    h = R.erosion(h, ws[n], merge)
                else:
                    h = R.smorph(h, ws[n], alphas[n], merge)
            torch.nn.functional.mse_loss(h, target).backward()
            with torch.no_grad():
                for p in params:
                    p -= 1e-3 * p.grad
        return run, WL.cfg5_taps(batch), f"config 5 training step at B={batch} of 256 (the metric is per tap; batch elements are independent)"
    raise SystemExit(f"unknown workload {workload}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="cfg5")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    args = ap.parse_args()
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    torch.set_num_threads(cores)
    run, n_taps, sample = step_fn(args.workload, args.batch)
    for _ in range(args.warmup):
        run()
    seconds = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run()
        seconds.append(time.perf_counter() - t0)
    print(json.dumps({"seconds": seconds, "n_taps": n_taps, "cores": cores, "sample": sample, "threads": torch.get_num_threads()}))
