#!/usr/bin/env python
"""Benchmark of the dilation / erosion / smorph hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg5|cfg2|cfg3|cfg4|cfg1]

Headline workload (default): config 5, one training step (forward, MSE loss, backward, gradient
all-reduce, SGD update) of the 4-layer stack Dilation(3->64,3x3,sum) -> SMorph(64->64,3x3,sum,alpha=2) ->
Erosion(64->64,5x5,max) -> SMorph(64->64,3x3,mean,alpha=-2) on a global batch of 256 x 3 x 224 x 224
synthetic images, the batch sharded over the N GPUs (strong scaling). Metric: forward+backward Gtaps/s,
N_taps = sum over layers of B*Co*Ci*H*W*kH*kW counted once per forward+backward pair.

One JSON line is printed by rank 0. `value` is timed with the shard resident in HBM; `e2e` copies the
shard's inputs from pinned host memory and reads the loss back every step, through the public Python
API. `configs` holds the single-GPU results of configurations 1-4, `roofline` the dominant kernel of
the headline workload timed alone with CUDA events, `cpu_baseline` the reference's own CPU code timed
on this host's cores on a bounded sample (in a subprocess: it owns the same operator namespace).

--impl reference times the reference's CPU implementation instead (oracle/_ref/_C.so when it was
built, else the C oracle port), each step a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import workloads as WL  # noqa: E402

METRIC = "fwd+bwd Gtaps/s"
UNIT = "Gtaps/s"

# Roofline denominators in Gtaps/s: instruction-mix ceilings of the CUDA cores, measured LIVE at the start of
# the run by ./probe_rates (source probe_rates.cu: register-only kernels, every operand loop carried, the SM clock
# sampled inside each kernel). The values
# below are an earlier measurement on this pool's B200 (profiles/probe_rates_b200.md), used only when the
# probe binary is missing. A dilation / erosion tap is one add and one max; the float peak is the best mix
# found (packed add.f32x2 + 3-input max), the double peak DADD + compare/select; a smorph tap costs three
# fused multiply-adds forward (factorised exponentials) and ten FP32 operations plus one ex2 backward. Packed
# two-lane instructions halve the issue slots of an operation, not its time on the FP32 pipe: both count per lane.
PEAK_GTAPS = {"morph_f32": 27300.0, "morph_f64": 5750.0, "smorph_fwd_f32": 10844.0, "smorph_bwd_f32": 3253.0, "smorph_fwdbwd_f32": 2502.0}
PEAK_SOURCE = "earlier measurement on this pool (probe binary missing)"


def measure_peaks():
    """Run the instruction-rate probe on the current GPU and fill PEAK_GTAPS; returns the raw rates."""
    global PEAK_SOURCE
    exe = os.path.join(ROOT, "probe_rates")
    if not os.path.exists(exe):
        return None
    try:
        out = subprocess.run([exe], capture_output=True, text=True, timeout=120).stdout.strip().splitlines()[-1]
        r = json.loads(out)
        PEAK_GTAPS["morph_f32"] = max(r["add_max_taps"], r["add_max3_taps"], r["add2_max3_taps"])
        PEAK_GTAPS["morph_f64"] = max(r["f64_add_fmax_taps"], r["f64_add_select_taps"])
        # smorph forward (sum / mean / identity merges): the factorised kernel needs 3 fused multiply-adds per tap and
        # no exponential; smorph backward: 10 FP32 operations (the exponent t, sum e, e t, sum e t, sum e t^2, two for
        # c_k, grad_input and grad_weight accumulation: nine per tap, plus one fma per window element and six
        # operations per pixel, together one more per tap at 3 x 3) and one ex2 per tap.
        fma = max(r["fma_ops"], r.get("fma2_ops", 0.0))
        PEAK_GTAPS["smorph_fwd_f32"] = fma / 3
        PEAK_GTAPS["smorph_bwd_f32"] = min(r["ex2_ops"], fma / 10)
        PEAK_GTAPS["smorph_fwdbwd_f32"] = 1.0 / (1.0 / PEAK_GTAPS["smorph_fwd_f32"] + 1.0 / PEAK_GTAPS["smorph_bwd_f32"])
        PEAK_SOURCE = "of measured (instruction-rate probe run on this GPU at the start of this bench)"
        return r
    except (OSError, ValueError, KeyError, IndexError, subprocess.TimeoutExpired):
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p.get("hbm_gbs", 6650.0)), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max = float(parts[2])
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        # samples under load are the upper half of the clock distribution (idle samples bracket the region)
        sm.sort()
        loaded = sm[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(loaded) if loaded else None, "sm_max_mhz": sm_max, "reasons": sorted(reasons), "samples": len(sm)}


def event_ms(fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def flush_l2(buf):
    buf.add_(1.0)  # 512 MB written: larger than the 126 MB L2


# ------------------------------------------------------------------------------------------------
# config 5
# ------------------------------------------------------------------------------------------------
def build_cfg5(device):
    import morphocore_b200.nn as Mnn
    layers = []
    for (kind, ci, co, k, merge, a0) in WL.CFG5_LAYERS:
        if kind == "dilation":
            layers.append(Mnn.Dilation(ci, co, k, merge))
        elif kind == "erosion":
            layers.append(Mnn.Erosion(ci, co, k, merge))
        else:
            layers.append(Mnn.SMorph(ci, co, k, merge, init_alpha=a0))
    model = torch.nn.Sequential(*layers).to(device)
    with torch.no_grad():
        for layer, w in zip(model, WL.cfg5_weights()):
            layer.weight.copy_(w)
    return model


def run_cfg5(args, rank, world, device):
    import torch.distributed as dist
    from morphocore_b200 import _native
    from morphocore_b200.parallel import GradBucket, shard_range

    B = args.batch
    start, count = shard_range(B, rank, world)
    x_host, t_host = WL.cfg5_batch(B=B, start=start, count=count)
    x_host, t_host = x_host.pin_memory(), t_host.pin_memory()
    model = build_cfg5(device)
    bucket = GradBucket(model.parameters())
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    x_dev, t_dev = x_host.to(device), t_host.to(device)

    def step(x, t):
        bucket.zero()
        loss = torch.nn.functional.mse_loss(model(x), t)
        loss.backward()
        bucket.all_reduce(average=True)
        opt.step()
        return loss

    # End to end: every step's inputs cross PCIe from pinned host memory and its loss is read back. As in any
    # input pipeline, the copy of step i + 1 runs on a copy stream into the other of two device buffers while
    # step i computes; the first copy of a run is exposed.
    copy_stream = torch.cuda.Stream(device=device)
    staged = [(torch.empty_like(x_dev), torch.empty_like(t_dev)) for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]

    def prefetch(i):
        with torch.cuda.stream(copy_stream):
            staged[i % 2][0].copy_(x_host, non_blocking=True)
            staged[i % 2][1].copy_(t_host, non_blocking=True)
            ready[i % 2].record(copy_stream)

    def run_e2e(steps):
        last = None
        prefetch(0)
        for i in range(steps):
            torch.cuda.current_stream().wait_event(ready[i % 2])
            loss = step(*staged[i % 2])
            if i + 1 < steps:
                prefetch(i + 1)   # the buffer it overwrites was last read by step i - 1, which .item() below has waited for
            last = loss.item()
        return last

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    for _ in range(args.warmup):
        step(x_dev, t_dev)
    barrier()
    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else 0)
    sampler.start()
    launches0 = _native.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(x_dev, t_dev)   # per-rank working set (activations of ~3.3 GB per layer) far exceeds the 126 MB L2
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = _native.launch_count() - launches0
    clocks = sampler.stop()

    run_e2e(1)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    last_loss = run_e2e(args.steps)
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / args.steps

    n_taps = WL.cfg5_taps(B)
    out = {
        "value": n_taps / ms / 1e6, "ms_per_step": ms, "gpu_launches": int(launches), "clocks": clocks,
        "e2e": {"value": n_taps / ms_e2e / 1e6, "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(x_host.numel() * 4 + t_host.numel() * 4), "d2h_bytes_per_step": 4,
                "pipeline": "copy of step i+1 on a copy stream overlaps step i (two device buffers); first copy exposed"},
        "config": {"workload": "config 5: training step of Dilation(3->64,3x3,sum)->SMorph(64->64,3x3,sum,alpha=2)->Erosion(64->64,5x5,max)->"
                               "SMorph(64->64,3x3,mean,alpha=-2), MSE loss, grad all-reduce, SGD",
                   "global_batch": B, "per_gpu_batch": count, "image": "3x224x224", "n_taps_per_step": n_taps,
                   "parallelism": f"dp{world}", "l2": "inputs larger than L2 (per-layer activations of %.1f GB per rank)" % (count * 64 * 224 * 224 * 4 / 1e9)},
        "loss": last_loss,
    }
    if rank == 0:
        out["roofline"] = cfg5_roofline(model, x_dev[:min(count, 16)], device)
    return out


def cfg5_roofline(model, x, device):
    """Times each layer's forward and backward kernels alone (CUDA events on the launching stream, one
    warm-up, L2 flushed in between) and reports the one taking the largest share of the step."""
    flush = torch.zeros(128 * 1024 * 1024, device=device)
    B = x.shape[0]
    rows = []
    h = x
    for n, (layer, (kind, ci, co, k, merge, a0)) in enumerate(zip(model, WL.CFG5_LAYERS)):
        inp = h.detach().requires_grad_(True)
        out = layer(inp)
        gy = torch.randn_like(out)
        out.backward(gy)     # warm-up
        flush_l2(flush)
        holder = {}
        t_f = event_ms(lambda: holder.__setitem__("out", layer(inp)))
        flush_l2(flush)
        t_b = event_ms(lambda: holder["out"].backward(gy))
        taps = WL.taps(B, co, ci, 224, 224, k, k)
        smorph = kind == "smorph"
        fwd_kernel = "smorph_forward_lean_kernel" if smorph else ("morpho_forward_kernel + morpho_find_tap_tiled_kernel" if merge in ("max", "min")
                                                                  else "morpho_forward_kernel")
        rows.append((t_f, f"L{n + 1} {kind} forward ({fwd_kernel})", taps,
                     PEAK_GTAPS["smorph_fwd_f32" if smorph else "morph_f32"], (ci + co) * 224 * 224 * 4 * B))
        bwd_kernel = "smorph_backward_kernel" if smorph else ("morpho_backward_scatter_kernel" if merge in ("max", "min")
                                                              else "morpho_backward_pairs_regs_kernel")
        rows.append((t_b, f"L{n + 1} {kind} backward ({bwd_kernel})", taps, PEAK_GTAPS["smorph_bwd_f32" if smorph else "morph_f32"],
                     2 * (ci + co) * 224 * 224 * 4 * B))
        h = holder["out"].detach()
    total = sum(r[0] for r in rows)
    t, name, taps, peak, alg_bytes = max(rows)
    hbm_peak, which = measured_peaks()
    return {
        "kernel": name, "share_of_step": t / total, "bound": "cuda_core", "achieved": taps / t / 1e6, "peak": peak, "unit": UNIT,
        "frac": taps / t / 1e6 / peak, "peak_source": PEAK_SOURCE,
        "hbm": {"bound": "hbm", "achieved": alg_bytes / t / 1e6, "peak": hbm_peak, "unit": "GB/s", "frac": alg_bytes / t / 1e6 / hbm_peak,
                "peak_source": f"of {which}", "algorithmic_bytes_per_launch": alg_bytes},
        "traffic": load_traffic(name, taps),
        "layers_ms": {r[1]: round(r[0], 3) for r in rows}, "sample_batch": B,
    }


def load_traffic(kernel_name, taps):
    """DRAM bytes read + written by one launch of the named kernel: the bytes per tap of the committed ncu
    capture (profiles/traffic.json, a smaller batch of the same layer; traffic grows in proportion to the
    batch) times the taps of this launch. null when no capture of this kernel is recorded."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    for key, value in table.items():
        if key in kernel_name:
            return value["dram_bytes_per_tap"] * taps
    return None


# ------------------------------------------------------------------------------------------------
# configs 1-4 (single GPU)
# ------------------------------------------------------------------------------------------------
def run_single(name, device, steps, warmup):
    import morphocore_b200.functional as F
    flush = torch.zeros(128 * 1024 * 1024, device=device)
    results = {}

    def timed(fwd, bwd_inputs, n_taps, peak_key, extra):
        for _ in range(warmup):
            out = fwd()
            if bwd_inputs is not None:
                out.backward(bwd_inputs)
        tf, tb = [], []
        for _ in range(steps):
            flush_l2(flush)
            holder = {}
            tf.append(event_ms(lambda: holder.__setitem__("y", fwd())))
            if bwd_inputs is not None:
                flush_l2(flush)
                tb.append(event_ms(lambda: holder["y"].backward(bwd_inputs)))
        f_ms, b_ms = statistics.median(tf), (statistics.median(tb) if tb else 0.0)
        g = n_taps / (f_ms + b_ms) / 1e6
        r = {"gtaps_per_s": g, "fwd_ms": f_ms, "bwd_ms": b_ms, "n_taps": n_taps, "frac_of_peak": g / PEAK_GTAPS[peak_key],
             "peak_gtaps": PEAK_GTAPS[peak_key], "fwd_gtaps_per_s": n_taps / f_ms / 1e6}
        if bwd_inputs is not None and peak_key.startswith("morph"):
            # The dilation / erosion backward has to evaluate every tap again (no winner is saved for sum / mean / identity
            # merges): a forward+backward pair is two passes at the add + max rate.
            r["pair_peak_gtaps"] = PEAK_GTAPS[peak_key] / 2
            r["frac_of_pair_peak"] = g / r["pair_peak_gtaps"]
        r.update(extra)
        return r

    if name in ("cfg1", "all"):
        c = WL.cfg1()
        x, w = c["x"].to(device), c["w"].to(device)
        g = torch.cuda.CUDAGraph()
        F.dilation(x, w, "max", save_indices=False)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for _ in range(20):
                y = F.dilation(x, w, "max", save_indices=False)
        g.replay()
        ms = event_ms(g.replay) / 20
        r = timed(lambda: F.dilation(x, w, "max", save_indices=False), None, c["n_taps"], "morph_f32", {"note": "forward only, launch-latency bound"})
        r["graph_ms"] = ms
        r["graph_gtaps_per_s"] = c["n_taps"] / ms / 1e6
        results["cfg1 dilation fwd fp32 max (8,3,128,128)x(16,3,3,3)"] = r
    if name in ("cfg2", "all"):
        c = WL.cfg2()
        x, w, gy = c["x"].to(device).requires_grad_(True), c["w"].to(device).requires_grad_(True), c["gy"].to(device)
        results["cfg2 erosion fwd+bwd fp32 sum (32,16,256,256)x(32,16,5,5)"] = timed(lambda: F.erosion(x, w, "sum"), gy, c["n_taps"], "morph_f32", {})
        del x, w, gy
    if name in ("cfg3", "all"):
        for alpha in WL.CFG3_ALPHAS:
            c = WL.cfg3(alpha)
            x, w, a, gy = c["x"].to(device).requires_grad_(True), c["w"].to(device).requires_grad_(True), c["alpha"].to(device).requires_grad_(True), c["gy"].to(device)
            results[f"cfg3 smorph fwd+bwd fp32 mean alpha={alpha:g} (16,32,128,128)x(32,32,7,7)"] = timed(
                lambda: F.smorph(x, w, a, channel_merge_mode="mean"), gy, c["n_taps"], "smorph_fwdbwd_f32",
                {"peak_note": "peak of a forward+backward pair: 3 FMA per tap forward, 10 FP32 operations + 1 ex2 per tap backward"})
            del x, w, a, gy
    if name in ("cfg4", "all"):
        for op in ("dilation", "erosion"):
            c = WL.cfg4(op)
            x, w, gy = c["x"].to(device).requires_grad_(True), c["w"].to(device).requires_grad_(True), c["gy"].to(device)
            fn = F.dilation if op == "dilation" else F.erosion
            results[f"cfg4 {op} fwd+bwd fp64 identity (8,64,512,512)x(64,1,11,11)"] = timed(lambda: fn(x, w, "identity"), gy, c["n_taps"], "morph_f64",
                                                                                         {"note": "weight is [:, :1] of the (64,64,11,11) draw: identity takes (C,1,kH,kW)"})
            del x, w, gy
    return results


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm
# ------------------------------------------------------------------------------------------------
def run_reference_cpu(workload, batch, steps, warmup, timeout=900):
    """Reference CPU code in a subprocess; falls back to the C oracle port when it was not built."""
    ref = os.path.join(ROOT, "oracle", "_ref", "_C.so")
    if os.path.exists(ref):
        cmd = [sys.executable, os.path.join(ROOT, "oracle", "ref_runner.py"), "--workload", workload, "--batch", str(batch), "--steps", str(steps),
               "--warmup", str(warmup)]
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
        if proc.returncode == 0:
            r = json.loads(proc.stdout.strip().splitlines()[-1])
            r["kind"] = "reference"
            return r
        sys.stderr.write(proc.stderr[-2000:])
    return run_oracle_port(workload, batch, steps, warmup)


def run_oracle_port(workload, batch, steps, warmup):
    """The C oracle (a port, OpenMP over the batch) on config 2's erosion forward+backward."""
    from oracle import oracle as O
    c = WL.cfg2(B=batch)
    x, w, gy = c["x"].numpy(), c["w"].flip((-2, -1)).contiguous().numpy(), c["gy"].numpy()
    seconds = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.morpho_forward("erosion", x, w, "sum")
        O.morpho_backward("erosion", x, w, gy, "sum")
        if i >= warmup:
            seconds.append(time.perf_counter() - t0)
    return {"seconds": seconds, "n_taps": c["n_taps"], "cores": os.cpu_count(), "kind": "port", "sample": f"config 2 at B={batch} (C oracle port)"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    batch = args.ref_batch
    r = run_reference_cpu(args.workload if args.workload != "all" else "cfg5", batch, args.steps, args.warmup)
    ms = statistics.mean(r["seconds"]) * 1e3
    value = r["n_taps"] / ms / 1e6
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": r["sample"], "device": "host CPU"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def run_case(name, batch, device):
    """One operator of one configuration at a reduced batch, run twice (warm-up + the launch to capture
    under ncu): the small cases behind the summaries in profiles/."""
    import morphocore_b200.functional as F
    part, direction = name.rsplit("_", 1)
    if part == "cfg2":
        c = WL.cfg2(B=batch)
        args, fn = (c["x"], c["w"]), (lambda x, w: F.erosion(x, w, "sum"))
    elif part == "cfg3":
        c = WL.cfg3(2.0, B=batch)
        args, fn = (c["x"], c["w"], c["alpha"]), (lambda x, w, a: F.smorph(x, w, a, channel_merge_mode="mean"))
    elif part == "cfg4":
        c = WL.cfg4("dilation", B=batch)
        args, fn = (c["x"], c["w"]), (lambda x, w: F.dilation(x, w, "identity"))
    elif part in ("cfg5l2", "cfg5l2pp", "cfg5l3"):
        g = torch.Generator().manual_seed(0)
        x = torch.rand((batch, 64, 224, 224), generator=g)
        if part in ("cfg5l2", "cfg5l2pp"):
            # "pp": one alpha per pair, as after the first optimiser step of a training run
            alpha = torch.full((64, 64), 2.0) + (0.01 * torch.randn((64, 64), generator=g) if part == "cfg5l2pp" else 0.0)
            args = (x, 0.1 * torch.randn((64, 64, 3, 3), generator=g), alpha)
            fn = lambda x, w, a: F.smorph(x, w, a, channel_merge_mode="sum")
        else:
            args, fn = (x, 0.1 * torch.randn((64, 64, 5, 5), generator=g)), (lambda x, w: F.erosion(x, w, "max"))
        c = {"gy": torch.randn((batch, 64, 224, 224), generator=g)}
    elif part == "sigma":
        # sigma_layer on the tensors of configuration 2: its two halves through the paired operator (one fused forward pass)
        # against the reference's formulation, erosion and dilation called one after the other; timed with CUDA events.
        c = WL.cfg2(B=batch)
        x, w, gy = c["x"].to(device), c["w"].to(device), c["gy"].to(device)
        alpha = torch.zeros((w.shape[0], w.shape[1]), device=device)

        def separate(x, w, a):
            soft = torch.sigmoid(a.mean(dim=1)).view(1, -1, 1, 1)
            return F.erosion(x, w, "sum") * (1.0 - soft) + F.dilation(x, w, "sum") * soft

        flush = torch.empty(64 * 1024 * 1024, dtype=torch.float32, device=device)
        result = {"case": name, "batch": batch}
        for label, fn in (("paired_ms", lambda x, w, a: F.sigma_layer(x, w, a, "sum")), ("separate_ms", separate)):
            best = float("inf")
            for _ in range(4):
                args = [t.clone().requires_grad_(direction == "bwd") for t in (x, w, alpha)]
                flush.zero_()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                y = fn(*args)
                if direction == "bwd":
                    y.backward(gy)
                stop.record()
                torch.cuda.synchronize()
                best = min(best, start.elapsed_time(stop))
            result[label] = best
        emit(result)
        return
    else:
        raise SystemExit(f"unknown case {name}")
    args = [t.to(device).requires_grad_(direction == "bwd") for t in args]
    gy = c["gy"].to(device)
    for _ in range(2):
        y = fn(*args)
        if direction == "bwd":
            y.backward(gy)
    torch.cuda.synchronize()
    emit({"case": name, "batch": batch, "done": True})


def emit(line):
    """Write the one JSON line to the process's original stdout."""
    os.write(RESULT_FD, (json.dumps(line) + "\n").encode())


# Libraries (NCCL's version banner, for one) print to stdout from native code. The contract is ONE JSON line
# on stdout, so everything else is sent to stderr and the result line goes to a duplicate of the original fd.
sys.stdout.flush()
RESULT_FD = os.dup(1)
os.dup2(2, 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=["cfg5", "cfg1", "cfg2", "cfg3", "cfg4", "all"])
    ap.add_argument("--batch", type=int, default=256, help="global batch of config 5")
    ap.add_argument("--ref-batch", type=int, default=8, help="images per step of the CPU reference sample (the metric is per tap and batch "
                    "elements are independent: eight images give every host core whole bands of work)")
    ap.add_argument("--no-configs", action="store_true", help="skip configurations 1-4")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--case", default=None, help="profiling helper: run one operator twice and exit, e.g. cfg2_fwd, cfg2_bwd, cfg3_fwd, "
                    "cfg3_bwd, cfg4_fwd, cfg4_bwd, cfg5l2_fwd, cfg5l2_bwd, cfg5l2pp_fwd, cfg5l2pp_bwd, cfg5l3_fwd, cfg5l3_bwd (with --case-batch); "
                    "sigma_fwd / sigma_bwd time sigma_layer through the paired operator against the two separate operators")
    ap.add_argument("--case-batch", type=int, default=4)
    args = ap.parse_args()

    if args.impl == "reference":
        reference_arm(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    if args.case:
        run_case(args.case, args.case_batch, device)
        return
    probe = measure_peaks() if rank == 0 else None
    line = {"metric": METRIC, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
    if args.workload == "cfg5":
        line.update(run_cfg5(args, rank, world, device))
    else:
        res = run_single(args.workload, device, args.steps, args.warmup)
        first = next(iter(res.values()))
        line.update({"value": first["gtaps_per_s"], "ms_per_step": first["fwd_ms"] + first["bwd_ms"], "config": {"workload": next(iter(res))},
                     "configs": res})
    if rank == 0:
        if world == 1 and args.workload == "cfg5" and not args.no_configs:
            torch.cuda.empty_cache()
            line["configs"] = run_single("all", device, 3, 2)
        if world == 1 and not args.no_cpu:
            r = run_reference_cpu("cfg5", args.ref_batch, 1, 1)
            ms = statistics.mean(r["seconds"]) * 1e3
            line["cpu_baseline"] = {"value": r["n_taps"] / ms / 1e6, "unit": UNIT, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"],
                                    "ms_per_step": ms}
        line["probe_gunits_per_s"] = probe
        line["peaks_gtaps"] = dict(PEAK_GTAPS)
        # A thread block whose bounded wait on a TMA copy ran out returns without writing its tile: a run with such a
        # block is not a measurement.
        import morphocore_b200
        line["device_errors"] = morphocore_b200.device_error_count()
        if line["device_errors"] != 0:
            raise SystemExit(f"{line['device_errors']} thread blocks gave up waiting for a TMA copy: the results are invalid")
        emit(line)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
