"""Data-parallel gradient exchange, host-side logic, on CPU with the gloo backend (2 ranks):
bucket planning, one collective per bucket, sum and mean, equality with the sum over shards."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from ngraph_python_b200 import comm as C


def test_bucket_plan_splits_in_production_order():
    sizes = [("a", 1000), ("b", 7_000_000), ("c", 10), ("d", 3_000_000), ("e", 64)]
    plan = C.BucketPlan(sizes, bucket_bytes=25 * 1024 * 1024)
    # 25 MB = 6 553 600 fp32: "a" alone, then "b" (larger than the limit) alone, then c+d+e
    assert [k for _, _, k in plan.buckets] == [["a"], ["b"], ["c", "d", "e"]]
    for key, n in sizes:
        assert plan.offsets[key] % C.ALIGN_ELEMS == 0
    starts = [plan.offsets[k] for k, _ in sizes]
    assert starts == sorted(starts)
    assert plan.total >= sum(n for _, n in sizes)
    small = C.BucketPlan([("x", 10), ("y", 20)], bucket_bytes=1 << 30)
    assert len(small.buckets) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        comm = C.TorchDistComm()
        sizes = [("g0", 300), ("g1", 5000), ("g2", 77)]
        plan = C.BucketPlan(sizes, bucket_bytes=4 * 4096)        # forces several buckets
        arena = torch.zeros(plan.total, dtype=torch.float32)
        rng = np.random.RandomState(rank)
        grads = {k: rng.standard_normal(n).astype(np.float32) for k, n in sizes}
        for k, n in sizes:
            arena[plan.offsets[k]:plan.offsets[k] + n] = torch.from_numpy(grads[k])
        funcs = {"g0": "sum", "g1": "sum", "g2": "mean"}
        ar = C.BucketedAllReduce(comm, plan, arena, funcs)
        ar.begin_call()
        # g0 is needed before its bucket is complete: the produced part is exchanged early
        ar.produced("g0")
        ar.wait_for("g0")
        early = ar.started
        ar.produced("g1")
        ar.produced("g2")
        for b in range(len(plan.buckets)):
            ar.bucket_ready(b)
        for k, _ in sizes:
            ar.wait_for(k)
        assert early == 1
        res = {k: arena[plan.offsets[k]:plan.offsets[k] + n].numpy().copy() for k, n in sizes}
        if rank == 0:
            out.put((res, ar.started, len(plan.buckets)))
    finally:
        dist.destroy_process_group()


def test_bucketed_allreduce_two_ranks_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res, started, nb = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert started >= nb >= 2          # one collective per bucket (+1 for the early part)
    sizes = [("g0", 300), ("g1", 5000), ("g2", 77)]
    shards = [{k: np.random.RandomState(r).standard_normal(n).astype(np.float32)
               for k, n in sizes} for r in range(world)]
    # RandomState(r) is consumed in order g0, g1, g2 per rank: rebuild exactly
    shards = []
    for r in range(world):
        rng = np.random.RandomState(r)
        shards.append({k: rng.standard_normal(n).astype(np.float32) for k, n in sizes})
    for k, _ in sizes:
        total = shards[0][k] + shards[1][k]
        if k == "g2":
            total = total / world
        np.testing.assert_allclose(res[k], total, rtol=1e-6, atol=1e-6)


def test_single_process_comm_is_identity():
    comm = C.SingleProcessComm()
    x = torch.arange(8, dtype=torch.float32)
    comm.all_reduce_async(x, "sum").wait()
    assert torch.equal(x, torch.arange(8, dtype=torch.float32))
    with pytest.raises(ValueError):
        comm.all_reduce_async(x, "max")


def _leaver(rank, world, port, out):
    """Rank 1 leaves between two exchanges (on the host, with nothing in flight); rank 0's next
    collective must end with CommError within its time limit instead of waiting for ever."""
    import time
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = C.TorchDistComm(timeout_s=3.0)
    plan = C.BucketPlan([("g", 256)])
    arena = torch.ones(plan.total, dtype=torch.float32)
    ar = C.BucketedAllReduce(comm, plan, arena, {"g": "sum"})
    ar.begin_call()
    ar.produced("g")
    ar.bucket_ready(0)
    ar.wait_for("g")                       # first step: both ranks take part
    ok_first = bool(torch.all(arena[:256] == 2.0))
    if rank == 1:
        out.put(("left", ok_first, 0.0))
        return                             # leaves without a word (no destroy, no second step)
    t0 = time.monotonic()
    try:
        ar.begin_call()
        ar.produced("g")
        ar.bucket_ready(0)
        ar.wait_for("g")
        ar.finish()
        out.put(("no error", ok_first, time.monotonic() - t0))
    except C.CommError as e:
        out.put(("CommError", ok_first, time.monotonic() - t0))


def test_a_replica_that_leaves_ends_the_exchange_with_an_error():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        got = [q.get(timeout=120) for _ in range(world)]
    finally:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
    by = dict((g[0], g) for g in got)
    assert "left" in by and by["left"][1]
    assert "CommError" in by, got
    assert by["CommError"][1] and by["CommError"][2] < 60.0


def _sampler_rank(rank, world, port, out):
    """One replica of the benchmark's keep-the-GPU-loaded loop, with a load that exchanges."""
    import datetime
    import torch.distributed as dist
    import bench
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=20))
    sampler = bench.ClockSampler(0)
    sampler.proc = object()                       # "nvidia-smi is running"
    # replica 0 already has its samples; replica 1 gets them only after 40 calls
    sampler.samples = [["0"]] * 4 if rank == 0 else []
    calls = [0]

    def load():
        calls[0] += 1
        dist.all_reduce(torch.ones(1))            # a step that holds a collective
        if rank == 1 and calls[0] == 40:
            sampler.samples.extend([["0"]] * 4)
    sampler.keep_loaded(load, lambda: None, want=4, limit_s=30.0, dist=dist, torch=torch,
                        device="cpu")
    out.put((rank, calls[0]))
    dist.destroy_process_group()


def test_replicas_agree_on_how_long_the_benchmark_keeps_them_loaded():
    """bench.py keeps a GPU busy until its clock sampler has samples.  When the workload holds a
    collective every replica must run it equally often, whatever its own sampler says: a replica
    that stopped on its own would leave the others waiting in an exchange for ever."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sampler_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=30)
    assert got[0] == got[1] == 40


def _bare_nccl_comm(timeout_s):
    """An NcclComm without a library behind it: only the watchdog's own logic is exercised."""
    import threading
    c = object.__new__(C.NcclComm)
    c.timeout_s, c.handle = timeout_s, object()
    c._deadline, c._failed, c._stop, c._watcher = None, None, threading.Event(), None
    c.aborted = []
    c.abort = lambda: c.aborted.append(True)
    return c


def test_watchdog_ends_a_step_whose_collective_never_completes():
    """The main thread synchronises; the watchdog aborts the communicator when the time limit
    passes (which makes the kernels in flight return) and the call ends with CommError."""
    import time
    c = _bare_nccl_comm(0.1)
    c.poll_error = lambda: None                      # NCCL reports nothing: a peer is just absent
    c.watch()
    time.sleep(0.4)                                  # "the synchronisation"
    with pytest.raises(C.CommError, match="time limit"):
        c.unwatch()
    assert c.aborted == [True]
    with pytest.raises(C.CommError):                 # the communicator stays failed
        c.watch()
    c._stop.set()


def test_watchdog_reports_an_asynchronous_nccl_error_and_stays_quiet_otherwise():
    import time
    c = _bare_nccl_comm(30.0)
    state = {"bad": False}

    def poll():
        if state["bad"]:
            raise C.CommError("a collective failed asynchronously: remote process exited")
    c.poll_error = poll
    c.watch()
    time.sleep(0.1)
    c.unwatch()                                      # a healthy step: nothing raised, no abort
    assert c.aborted == []
    c.watch()
    state["bad"] = True
    time.sleep(0.2)
    with pytest.raises(C.CommError, match="remote process exited"):
        c.unwatch()
    assert c.aborted == [True]
    c._stop.set()
