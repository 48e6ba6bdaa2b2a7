"""Bandwidth of the fused all-reduce + momentum-SGD + parameter-broadcast kernel
against its NVLink roofline, and against the NCCL all-reduce + separate update it
replaces.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        --master-port 29555 -m tsplit_b200.parallel.bench_allreduce --mb 100 400

For a bucket of S bytes on N GPUs every GPU receives 2*S*(N-1)/N bytes (the
peers' gradients for its own shard, which it reads, and the peers' updated
shards, which they store into it) and sends as many (the answers to the peers'
reads of its gradients and its own updated shard stored to the peers).  The two
directions run concurrently, so the link-time floor is 2*S*(N-1)/N divided by
the per-direction peer bandwidth (770 GB/s measured copy, 900 GB/s nominal).
Timed on the device with CUDA events, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.distributed as dist

from .. import ndarray
from ..graph import Node
from ..stream import current_stream
from .fused_allreduce import FusedCommunicator

LINK_GBS_MEASURED = 770.0
LINK_GBS_NOMINAL = 900.0


def _recorded(stream, ctx):
    from ..stream import Event
    ev = Event(ctx)
    ev.record(stream)
    return ev


class _Opt(object):
    """The three things the communicator needs from an optimizer."""
    kind, initial_accumulator_value = 1, 0.0

    def __init__(self, n, ctx):
        node = Node()
        node.tensor_value = ndarray.empty((n,), ctx, use_pool=False)
        node.tensor_value.t.normal_()
        self.tensors = [node]

    @property
    def params(self):
        return [n.tensor_value for n in self.tensors]

    def hyper(self):
        return [0.01, 0.9]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=float, nargs="+", default=[100.0, 553.0])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nvls", type=int, default=0, help="1 = multimem.ld_reduce / multimem.st through NVSwitch")
    args = ap.parse_args()
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    own_group = not dist.is_initialized()
    if own_group:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    ctx = ndarray.gpu(local)
    st = current_stream(ctx)
    for mb in args.mb:
        n = int(mb * 2**20 / 4) // (4 * world) * (4 * world)
        opt = _Opt(n, ctx)
        comm = FusedCommunicator(opt, dist, use_multimem=bool(args.nvls), bucket_mb=1 << 20)   # one bucket
        grad = ndarray.empty((n,), ctx, use_pool=False)
        grad.t.normal_()
        # one checked step first: rank-dependent gradients, zero velocity; the fused kernel must leave
        # p - lr * mean(g) on every rank (first momentum step), compared with an NCCL all-reduce of the same data
        g_chk = torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(100 + rank))
        dist.broadcast(comm.param_bucket, src=0)       # as data-parallel training starts: the same parameters everywhere
        p_before = comm.param_bucket.clone()
        comm.grad_bucket.copy_(g_chk)
        torch.cuda.synchronize()
        dist.barrier()
        comm.begin_step()
        comm.launch_bucket(0, opt, st, overlapped=False)
        st.wait_event(_recorded(comm.comm_stream, ctx))
        torch.cuda.synchronize()
        dist.all_reduce(g_chk)
        want = p_before - 0.01 * g_chk / world
        err = (comm.param_bucket - want).abs().max()
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        max_err = float(err.item())
        dist.barrier()
        # the kernel proper (gradients already in the symmetric array): time launches back to back
        comm.grad_bucket.copy_(grad.t)

        def fused_once():
            comm.begin_step()
            comm.launch_bucket(0, opt, st, overlapped=False)
            st.wait_event(_recorded(comm.comm_stream, ctx))

        vel = torch.zeros(n, device="cuda")
        par = torch.randn(n, device="cuda")

        def nccl_once():
            dist.all_reduce(grad.t)
            grad.t.mul_(1.0 / world)
            vel.mul_(0.9).add_(grad.t, alpha=-0.01)
            par.add_(vel)

        results = {}
        for name, fn in (("fused", fused_once), ("nccl+update", nccl_once)):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1) / args.iters], device="cuda")
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            results[name] = float(ms.item())
        comm.check(st)
        if rank == 0:
            s_bytes = n * 4
            floor_ms = 2.0 * s_bytes * (world - 1) / world / (LINK_GBS_MEASURED * 1e6)
            bus = 2.0 * s_bytes * (world - 1) / world / (results["fused"] * 1e6)
            print(json.dumps({"bucket_mb": round(s_bytes / 2**20, 1), "world": world, "nvls": args.nvls,
                              "fused_ms": round(results["fused"], 4), "nccl_plus_update_ms":
                              round(results["nccl+update"], 4), "link_floor_ms": round(floor_ms, 4),
                              "fraction_of_link_roofline_of_measured": round(floor_ms / results["fused"], 3),
                              "fraction_of_link_roofline_of_nominal": round(
                                  floor_ms * LINK_GBS_MEASURED / LINK_GBS_NOMINAL / results["fused"], 3),
                              "bus_gbs": round(bus, 1), "checked_step_max_abs_err": max_err}))
        del comm, opt
    if own_group:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
