"""Shared driver of the example scripts: policy name -> executor, timed runs with
CUDA events, and the batch-size sweep that stops at the first OutOfHBMBudget
(the reference's sweep loops until its executor asserts,
``examples/imagenet_vgg.py:159-178``)."""
from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np                                            # noqa: E402

from tsplit_b200 import ndarray, gpu_ops as ad                # noqa: E402
from tsplit_b200.runtime.pool import MemoryPool               # noqa: E402

POLICIES = ["None", "base", "vdnnconv", "vdnnall", "superneurons", "recompute_memory", "recompute_speed",
            "capuchin", "simulator", "profiler", "planner", "tsplit"]


#: set by ``--graph``: 1 = replay fixed steps from a CUDA graph, 2 = from the native tape of recorded calls
#: (``"tape"``; the memory executors only: it also covers steps with the multi-GPU gradient exchange)
USE_GRAPH = [False]


def make_executor(policy, nodes, ctx):
    g = USE_GRAPH[0]
    if policy in ("None", "base"):
        return ad.Executor(nodes, ctx=ctx, use_graph=g is True)
    if policy == "vdnnconv":
        return ad.vdnnExecutor(nodes, ctx=ctx, policy="conv")
    if policy == "vdnnall":
        return ad.vdnnExecutor(nodes, ctx=ctx, policy="all")
    if policy == "superneurons":
        return ad.superNeuronsExecutor(nodes, ctx=ctx)
    if policy == "recompute_memory":
        return ad.recomputeExecutor(nodes, ctx=ctx, policy="memory", use_graph=g)
    if policy == "recompute_speed":
        return ad.recomputeExecutor(nodes, ctx=ctx, policy="speed", use_graph=g)
    if policy == "capuchin":
        return ad.capuchinExecutor(nodes, ctx=ctx)
    if policy == "simulator":
        return ad.microopOptimizer(nodes, ctx=ctx)
    if policy == "profiler":
        return ad.profileExecutor(nodes, ctx=ctx)
    if policy == "planner":
        return ad.microopPlanner(nodes, ctx=ctx)
    if policy == "tsplit":
        return ad.microopExecutor(nodes, ctx=ctx, use_graph=g)
    raise NotImplementedError(policy)


def default_ctx():
    import torch
    if torch.cuda.is_available():
        return ndarray.gpu(int(os.environ.get("LOCAL_RANK", "0")))
    return ndarray.simgpu(0)


# -- data-parallel runs: `python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 examples/X.py ...`
_DIST = [None]


def dist_setup():
    """Join the process group when launched by torchrun (one process per GPU); returns (rank, world)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    from tsplit_b200.utils.affinity import bind_to_gpu
    bind_to_gpu(local)                 # pinned swap buffers on the NUMA node of this rank's GPU
    if not dist.is_initialized():
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _DIST[0] = dist
    return dist.get_rank(), world


def attach(opt, mode="fused"):
    """Data-parallel gradient exchange for ``opt`` (the fused NVLink all-reduce + update kernel by default)."""
    if _DIST[0] is not None:
        from tsplit_b200.parallel import ddp
        ddp.attach(opt, _DIST[0], mode=mode)
    return opt


def max_over_ranks(value):
    if _DIST[0] is None:
        return value
    import torch
    t = torch.tensor([float(value)], device="cuda", dtype=torch.float64)
    _DIST[0].all_reduce(t, op=_DIST[0].ReduceOp.MAX)
    return float(t.item())


def timed_run(executor, feed, iters=3):
    """Warm-up (one run; three with ``--graph``, whose capture happens on the third), then ``iters``
    timed runs; seconds per iteration.  On a CUDA context the time is taken on the device with events on the
    executor's stream, and with several ranks it is the maximum over the ranks."""
    out = executor.run(feed)
    if not isinstance(out, list):
        return out
    if USE_GRAPH[0]:
        executor.run(feed)
        executor.run(feed)
    on_device = getattr(executor, "on_device", False)
    if on_device:
        import torch
        if _DIST[0] is not None:
            _DIST[0].barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(executor.stream.torch_stream)
        for _ in range(iters):
            executor.run(feed)
        e1.record(executor.stream.torch_stream)
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / 1e3 / iters)
    t0 = time.time()
    for _ in range(iters):
        executor.run(feed)
    return (time.time() - t0) / iters


def sweep(run_at_batch, batches, out_path=None):
    """Call ``run_at_batch(b)`` for growing b until the budget is exceeded (on any rank)."""
    results = []
    for b in batches:
        failed = 0
        try:
            t = run_at_batch(b)
        except ndarray.OutOfHBMBudget as e:
            print("Batch size: %d does not fit: %s" % (b, e))
            failed, t = 1, None
        if _DIST[0] is None and failed:
            break
        if _DIST[0] is not None and max_over_ranks(failed):
            break
        if int(os.environ.get("RANK", "0")) != 0:
            continue
        print("Batch size: {} , time: {} s".format(b, t))
        results.append((b, t))
        if out_path:
            with open(out_path, "a") as f:
                f.write("Batch size: {} , time: {} s\n".format(b, t))
    return results


def parse(description, extra=None):
    p = argparse.ArgumentParser(description=description)
    p.add_argument("-l", "--layer", type=int, default=0)
    p.add_argument("-p", "--policy", default="None", choices=POLICIES)
    p.add_argument("-b", "--batch", type=int, default=0, help="single batch size (0 = sweep)")
    p.add_argument("--cap-gib", type=float, default=16.0, help="HBM budget of the activation pool")
    p.add_argument("--out", default=None, help="append results to this file")
    p.add_argument("--graph", type=int, default=0, help="1 = replay fixed steps from a CUDA graph, 2 = from the native tape of recorded calls")
    p.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                   help="gradient exchange when launched with several ranks")
    if extra:
        extra(p)
    args = p.parse_args()
    USE_GRAPH[0] = {0: False, 1: True, 2: "tape"}[int(args.graph)]
    return args


def with_pool(ctx, cap_gib):
    pool = MemoryPool(ctx, int(cap_gib * 2**30))
    ndarray.set_pool(ctx, pool)
    return pool
