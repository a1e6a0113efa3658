"""Data-parallel plumbing on CPU: world_size-2 gloo ranks (no GPU). The flat gradient bucket must give
every rank the mean of the per-rank gradients, shards must tile the batch, a rank whose bucket
differs must be reported on the host instead of hanging a collective, a rank that leaves between two
steps must end its peer's next all-reduce with an error instead of a hang, and a gradient that no
longer aliases the bucket must be refused."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT  # noqa: F401


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def worker(rank, world, port, mode, results):
    import importlib.util
    spec = importlib.util.spec_from_file_location("mc_parallel", os.path.join(ROOT, "morphocore_b200", "parallel.py"))
    par = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(par)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8 if mode == "leaver" else 120))
    try:
        torch.manual_seed(0)
        extra = 1 if (mode == "mismatch" and rank == 1) else 0
        params = [torch.nn.Parameter(torch.randn(4, 3, 3, 3)), torch.nn.Parameter(torch.randn(4, 3 + extra))]
        bucket = par.GradBucket(params)
        # a "model": loss = sum_b (x_b . p)^2 over this rank's shard of a global batch of 6
        start, count = par.shard_range(6, rank, world)
        data = torch.arange(6, dtype=torch.float32) + 1.0
        bucket.zero()
        loss = sum((data[b] * p).pow(2).sum() for b in range(start, start + count) for p in params) / count
        loss.backward()
        assert params[0].grad.data_ptr() == bucket.flat.data_ptr(), "gradients must accumulate inside the flat bucket"
        if mode == "rebound":
            for p in params:
                p.grad = None               # what optimizer.zero_grad() does by default
            params[0].grad = torch.ones_like(params[0])
        try:
            bucket.all_reduce(average=True)
            results[rank] = ("ok", bucket.flat.clone())
        except RuntimeError as err:
            results[rank] = ("error", str(err))
        if mode == "leaver":
            # Step 1 is done on both ranks. Rank 1 leaves between the steps, with no collective in flight; rank 0 starts
            # step 2 and must come back with an error within the group's time-out instead of waiting for ever.
            if rank == 1:
                os._exit(0)
            started = time.monotonic()
            try:
                bucket.all_reduce(average=True)
                results["step2"] = ("ok", time.monotonic() - started)
            except Exception as err:  # gloo reports a lost peer as RuntimeError or DistBackendError
                results["step2"] = ("error", time.monotonic() - started, type(err).__name__)
            os._exit(0)                     # the process group cannot be torn down cleanly without its peer
    finally:
        if mode != "leaver":
            dist.destroy_process_group()


def run(mode):
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    if mode == "leaver":
        # the ranks end with os._exit: join them by hand instead of through mp.spawn's error handling
        ctx = mp.get_context("spawn")
        port = free_port()
        procs = [ctx.Process(target=worker, args=(r, world, port, mode, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            if p.is_alive():
                p.kill()
                p.join()
                results["step2"] = ("hang", 120.0)
        return dict(results)
    mp.spawn(worker, args=(world, free_port(), mode, results), nprocs=world, join=True)
    return dict(results)


def test_shard_range_tiles_the_batch():
    import importlib.util
    spec = importlib.util.spec_from_file_location("mc_parallel", os.path.join(ROOT, "morphocore_b200", "parallel.py"))
    par = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(par)
    for total in (1, 7, 256):
        for world in (1, 2, 3, 8):
            spans = [par.shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == total
            for (s0, c0), (s1, _) in zip(spans, spans[1:]):
                assert s0 + c0 == s1
    assert par.shard_range(256, 3, 8) == (96, 32)
    with pytest.raises(ValueError):
        par.shard_range(8, 2, 2)


def test_bucket_all_reduce_gives_the_global_mean_gradient():
    results = run("normal")
    assert results[0][0] == "ok" and results[1][0] == "ok"
    assert torch.equal(results[0][1], results[1][1])
    # single-process reference: mean over the two shards of the per-shard mean gradients
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.randn(4, 3, 3, 3)), torch.nn.Parameter(torch.randn(4, 3))]
    data = torch.arange(6, dtype=torch.float32) + 1.0
    loss = sum((data[b] * p).pow(2).sum() for b in range(6) for p in params) / 6
    loss.backward()
    want = torch.cat([p.grad.reshape(-1) for p in params])
    torch.testing.assert_close(results[0][1], want, rtol=1e-6, atol=1e-6)


def test_rebound_gradients_are_refused():
    results = run("rebound")
    for rank in (0, 1):
        assert results[rank][0] == "error" and "no longer a view of the flat buffer" in results[rank][1]


def test_rank_leaving_between_steps_ends_the_next_all_reduce_with_an_error():
    results = run("leaver")
    assert results[0][0] == "ok", "step 1 ran with both ranks present"
    outcome = results["step2"]
    assert outcome[0] == "error", f"the all-reduce without its peer returned {outcome}"
    assert outcome[1] < 60, f"took {outcome[1]:.1f} s: that is a hang, not a time-out"


def test_mismatched_buckets_are_reported_not_hung():
    results = run("mismatch")
    assert results[0][0] == "error" and results[1][0] == "error"
    assert "differ across ranks" in results[0][1]
