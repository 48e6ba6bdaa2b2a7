#!/usr/bin/env python
"""Headline benchmark: VGG-16 training throughput (img/s) at the maximum trainable
batch under a per-GPU HBM cap, 1..8 B200.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference ...                     # the reference arm

One step = forward + backward + momentum-SGD update of VGG-16 with batch-norm
(13 conv3x3 + 3 FC, 1000 classes, fp32 storage, TF32 tensor-core math with fp32
accumulation) on synthetic [B,3,224,224] ~ N(0,1) images with uniform labels.
Activations live in a capped pool (``--cap-gib`` per GPU); the TSplit planner
chooses swap / recompute / micro-tensor split per tensor to fit, and the batch is
the largest one whose plan fits (bounded by ``--max-batch``).  With N > 1 every
rank runs the same per-GPU batch (weak scaling) and gradients are reduced and
applied by the fused NVSwitch all-reduce + optimizer kernel.

Timing: W untimed warm-up steps, then K steps bracketed by barrier +
``cuda.synchronize`` and CUDA events on the compute stream, max over ranks.  The
activations touched per step exceed the 126 MB L2 by orders of magnitude, so no
extra L2 flush is needed between iterations.  ``e2e`` repeats the measurement
through the public ``executor.run(feed_dict)`` call with pinned host arrays as
feeds (copied host->device every step) and a device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=8)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="vgg16", choices=["vgg16", "resnet50"])
    p.add_argument("--policy", default="tsplit",
                   choices=["base", "tsplit", "vdnnall", "vdnnconv", "recompute_speed", "recompute_memory",
                            "superneurons", "capuchin"])
    p.add_argument("--cap-gib", type=float, default=16.0, help="activation pool (HBM cap) per GPU")
    p.add_argument("--batch", type=int, default=0, help="per-GPU batch; 0 = largest batch whose plan fits")
    p.add_argument("--max-batch", type=int, default=2048, help="upper bound of the max-batch search")
    p.add_argument("--host-link-gbs", type=float, default=0.0,
                   help="host link bandwidth the planner assumes; 0 = measure it (pinned copies, both directions busy)")
    p.add_argument("--also-batch", type=int, default=256,
                   help="after the headline run, time this smaller batch with the same policy (0 = skip)")
    p.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    p.add_argument("--graph", type=int, default=0,
                   help="1 = replay the step from a CUDA graph (single GPU); 2 = replay it from the native tape "
                        "of recorded calls (any number of GPUs)")
    return p.parse_args()


def reference_arm(args):
    """The reference cannot be installed: it has no setup.py / pyproject.toml (pip:
    "Neither 'setup.py' nor 'pyproject.toml' found"), no build files for its C++/CUDA
    runtime, Python-2 sources and cuDNN-7-only calls."""
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is not installable offline: no setup.py/pyproject.toml, no build "
                                     "system for libc_runtime_api.so, Python 2 sources, cuDNN-7-only API, and its "
                                     "TSplit planner modules are missing from the tree"}))
    return 0


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.idx = device_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for name, val in zip(names, r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_model(name):
    from tsplit_b200.models import vgg, resnet
    return vgg(16) if name == "vgg16" else resnet(50)


def make_executor(args, model, train_op, ctx):
    from tsplit_b200 import gpu_ops as ad
    nodes = [model.loss, train_op]
    pol = args.policy
    graph = {0: False, 1: True, 2: "tape"}[int(getattr(args, "graph", 0))]
    if pol == "base":
        return ad.MemoryExecutor(nodes, ctx=ctx, use_graph=graph)
    if pol == "tsplit":
        return ad.microopExecutor(nodes, ctx=ctx, host_link_gbs=args.host_link_gbs, use_graph=graph,
                                  budget_bytes=args.plan_budget, max_split=32)
    if pol in ("vdnnall", "vdnnconv"):
        return ad.vdnnExecutor(nodes, ctx=ctx, policy=pol[4:])
    if pol.startswith("recompute"):
        return ad.recomputeExecutor(nodes, ctx=ctx, policy=pol.split("_")[1])
    if pol == "superneurons":
        return ad.superNeuronsExecutor(nodes, ctx=ctx)
    return ad.capuchinExecutor(nodes, ctx=ctx, host_link_gbs=args.host_link_gbs)


def batch_ladder(limit):
    """Candidate batches, largest first: multiples of 256 above 1024, of 128 above 512, of 64 above 256, of 32
    below."""
    out, b = [], limit
    while b >= 8:
        out.append(b)
        step = 256 if b > 1024 else 128 if b > 512 else 64 if b > 256 else 32 if b > 32 else 8
        b = (b - 1) // step * step if b % step else b - step
    return out


def find_max_batch(args, model, train_op, ctx, log):
    """Largest batch on the ladder (<= --max-batch) for which the TSplit planner finds a plan inside the
    budget (its replay is byte-exact and every allocation is placed ahead of time, so a plan that fits runs).
    The ladder is walked downward and the first batch that fits is taken: the result never drops below a
    batch that was found to fit.  Other policies have no dry run and are probed by running (see main)."""
    from tsplit_b200 import gpu_ops as ad
    nodes = [model.loss, train_op]
    for b in batch_ladder(max(8, args.max_batch)):
        sim = ad.microopOptimizer(nodes, ctx=ctx, budget_bytes=args.plan_budget, host_link_gbs=args.host_link_gbs,
                                  max_split=32)
        x = np.empty((b,) + model.input_shape, dtype=np.float32)
        y = np.empty((b, model.num_classes), dtype=np.float32)
        r = sim.run({model.X: x, model.y_: y})
        log.append({"batch": b, "fits": bool(r["fits"]), "pieces": r["pieces"],
                    "predicted_ms": round(r["predicted_ms"], 1)})
        if r["fits"]:
            return b
    return 0


def library_scratch_bytes():
    """Bytes the kernel library holds as scratch obtained with cudaMalloc (split-K partial sums, padded and
    transposed operand copies, column partial sums): outside the pool and outside torch's allocator."""
    import ctypes
    from tsplit_b200 import _base
    lib = _base.kernels()
    raw = object.__getattribute__(lib, "_lib") if not isinstance(lib, ctypes.CDLL) else lib
    fn = raw.tsb_scratch_bytes
    fn.restype = ctypes.c_longlong
    return int(fn())


def time_steps(ex, feed, steps, barrier):
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(ex.stream.torch_stream)
    loss = None
    for _ in range(steps):
        loss = ex.run(feed)[0]
    e1.record(ex.stream.torch_stream)
    barrier()
    return e0.elapsed_time(e1), loss


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local_rank)
    cpus = None
    if world > 1:      # pinned swap buffers on the NUMA node of this rank's GPU
        from tsplit_b200.utils.affinity import bind_to_gpu
        cpus = bind_to_gpu(local_rank)

    from tsplit_b200 import ndarray, optimizer, _base
    from tsplit_b200.runtime.pool import MemoryPool
    from tsplit_b200.utils import launch_counter, hostlink

    dist = comm = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()          # all ranks measure at the same time: they share the host's memory bandwidth during training too
    link = hostlink.measure(local_rank, repeats=8 if world > 1 else 4, shared=world > 1)
    if not args.host_link_gbs:
        args.host_link_gbs = min(link["bidir_h2d_gbs"], link["bidir_d2h_gbs"])
    if dist is not None:                    # every rank plans with the same figure
        t = torch.tensor([args.host_link_gbs], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        args.host_link_gbs = float(t.item())

    ctx = ndarray.gpu(local_rank)
    model = build_model(args.model)
    opt = optimizer.MomentumOptimizer(learning_rate=0.001, momentum=0.9, ctx=ctx)
    train_op = opt.minimize(model.loss)
    if world > 1:
        from tsplit_b200.parallel import ddp
        comm = ddp.attach(opt, dist, mode=args.comm)
        if hasattr(comm, "exposed_ms"):
            comm.timing = True

    cap_bytes = int(args.cap_gib * 2**30)
    args.plan_budget = cap_bytes - (1 << 20)           # the results of a step (loss) live beside the placed region
    search_log = []
    t_plan = time.time()
    batch = args.batch or (find_max_batch(args, model, train_op, ctx, search_log) if args.policy == "tsplit"
                           else args.max_batch)
    plan_seconds = time.time() - t_plan
    if world > 1:                      # every rank must agree
        t = torch.tensor([batch], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        batch = int(t.item())
    assert batch > 0, "no batch fits the cap"

    # ---- build + warm-up at the chosen batch.  Policies without a dry run (and a TSplit plan that meets
    # something its replay did not see) step down the ladder until the steps run.
    ladder = [b for b in batch_ladder(max(8, args.max_batch)) if b <= batch] or [batch]
    pool = ex = None
    for batch in ladder:
        pool = MemoryPool(ctx, cap_bytes)          # a fresh arena per attempt: an aborted step may leave blocks behind
        ndarray.set_pool(ctx, pool)
        ex = make_executor(args, model, train_op, ctx)
        x_np, y_np = model.synthetic_batch(batch, seed=rank)
        x_dev = ndarray.array(x_np, ctx, use_pool=False)
        y_dev = ndarray.array(y_np, ctx, use_pool=False)
        feed_dev = {model.X: x_dev, model.y_: y_dev}
        failed = 0
        try:
            for _ in range(max(args.warmup, 3)):
                loss = ex.run(feed_dev)[0]
        except (ndarray.OutOfHBMBudget, RuntimeError) as e:
            if args.batch:
                raise
            failed = 1
            search_log.append({"batch": batch, "ran": False, "why": str(e)[:120]})
        if dist is not None:
            t = torch.tensor([failed], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            failed = int(t.item())
        if not failed:
            break
        del ex, x_dev, y_dev, feed_dev, pool
        ndarray.set_pool(ctx, None)
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    assert not failed, "no batch on the ladder runs under the cap"
    barrier()

    # ---- device-timed region
    sampler = ClockSampler(local_rank)
    sampler.start()
    launch_counter.reset()
    dev_ms, loss = time_steps(ex, feed_dev, args.steps, barrier)
    exposed_comm_ms = None
    if comm is not None and hasattr(comm, "exposed_ms"):
        v = comm.exposed_ms(last=args.steps)
        exposed_comm_ms = round(sum(v) / max(len(v), 1), 3) if v else None
    launches = launch_counter.count()
    clocks = sampler.stop()
    loss_val = float(loss.asnumpy().reshape(-1)[0])
    stats = {k: int(v) for k, v in ex.stats.items()}
    plan = getattr(ex, "plan_result", None)
    plan_repr, plan_pieces = repr(plan), getattr(plan, "pieces", None)
    peak_in_pool = pool.stats()["peak"]
    torch_bytes = int(torch.cuda.max_memory_allocated())

    # ---- end-to-end through the public API: every step copies its inputs host -> device from
    # pinned host memory (the caller's own pinned NDArrays) and reads the loss back to the host
    from tsplit_b200 import ndarray as nd
    x_pin = nd.empty(x_np.shape, nd.cpu(0), pinned=True)
    y_pin = nd.empty(y_np.shape, nd.cpu(0), pinned=True)
    x_pin.t.copy_(torch.from_numpy(x_np))
    y_pin.t.copy_(torch.from_numpy(y_np))
    feed_pin = {model.X: x_pin, model.y_: y_pin}
    # two alternating pinned batches, as an input pipeline would hand them over; the copy of the next
    # batch is started before the current step runs (it overlaps the step) and belongs to the timed region
    x_pin2 = nd.empty(x_np.shape, nd.cpu(0), pinned=True)
    y_pin2 = nd.empty(y_np.shape, nd.cpu(0), pinned=True)
    x_pin2.t.copy_(x_pin.t)
    y_pin2.t.copy_(y_pin.t)
    feeds = [feed_pin, {model.X: x_pin2, model.y_: y_pin2}]
    for i in range(2):
        ex.run(feeds[i % 2], convert_to_numpy_ret_vals=True)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record(ex.stream.torch_stream)
    ex.prefetch_feeds(feeds[0])
    for i in range(args.steps):
        if i + 1 < args.steps:
            ex.prefetch_feeds(feeds[(i + 1) % 2])
        out = ex.run(feeds[i % 2], convert_to_numpy_ret_vals=True)
        _ = float(out[0].reshape(-1)[0])
    s1.record(ex.stream.torch_stream)
    torch.cuda.synchronize()
    e2e_ms = s0.elapsed_time(s1)

    # ---- multi-GPU correctness bit: after the same number of steps every rank must hold the same parameters
    params_equal = None
    if dist is not None:
        chk = torch.zeros(2, device="cuda", dtype=torch.float64)
        for p_ in opt.params:
            chk[0] += p_.t.double().sum()
            chk[1] += p_.t.double().abs().sum()
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        params_equal = bool(torch.equal(lo, hi))

    # ---- the same policy at a smaller reference batch (shows what the larger batch costs per image)
    also = None
    if args.also_batch and args.also_batch < batch:
        try:
            xa, ya = model.synthetic_batch(args.also_batch, seed=rank)
            fa = {model.X: ndarray.array(xa, ctx, use_pool=False), model.y_: ndarray.array(ya, ctx, use_pool=False)}
            for _ in range(3):
                ex.run(fa)
            ms_a, _ = time_steps(ex, fa, args.steps, barrier)
            if dist is not None:
                t = torch.tensor([ms_a], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms_a = float(t.item())
            also = {"per_gpu_batch": args.also_batch, "ms_per_step": round(ms_a / args.steps, 3),
                    "img_s": round(args.also_batch * world / (ms_a / args.steps) * 1e3, 1),
                    "plan": repr(getattr(ex, "plan_result", None))}
        except Exception as e:                       # the headline stands without it
            also = {"per_gpu_batch": args.also_batch, "error": str(e)[:160]}

    if dist is not None:
        t = torch.tensor([dev_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0].item()), float(t[1].item())

    global_batch = batch * world
    ms_per_step = dev_ms / args.steps
    value = global_batch / ms_per_step * 1e3
    e2e_value = global_batch / (e2e_ms / args.steps) * 1e3
    h2d = int(x_np.nbytes + y_np.nbytes)
    swap_bytes = stats.get("swap_out_bytes", 0) + stats.get("swap_in_bytes", 0)
    # host-link roofline of the swap traffic: the busier direction's bytes over that direction's measured
    # bandwidth (both directions busy), as a fraction of the step
    link_ms = max(stats.get("swap_out_bytes", 0) / (link["bidir_d2h_gbs"] * 1e6),
                  stats.get("swap_in_bytes", 0) / (link["bidir_h2d_gbs"] * 1e6))
    if rank == 0:
        print(json.dumps({
            "metric": "img/s at max batch under HBM cap (VGG-16)" if args.model == "vgg16" else
                      "img/s at max batch under HBM cap (ResNet-50)",
            "value": round(value, 2), "unit": "img/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "tf32 (fp32 storage, fp32 accumulate)",
            "data": "synthetic N(0,1) images, uniform labels, random-init weights",
            "impl": "ours",
            "config": {"model": args.model, "global_batch": global_batch, "per_gpu_batch": batch,
                       "max_batch_found": batch if not args.batch else None,
                       "image": "3x224x224", "parallelism": "dp%d" % world, "optimizer": "momentum-sgd",
                       "hbm_cap_gib_per_gpu": args.cap_gib, "policy": args.policy,
                       "max_batch_search_limit": args.max_batch, "max_batch_search": search_log,
                       "plan_seconds": round(plan_seconds, 1),
                       "l2": "inputs and activations per step exceed the 126 MB L2; no explicit flush",
                       "plan": plan_repr, "loss": loss_val, "executor_stats": stats,
                       "exposed_comm_ms_per_step": exposed_comm_ms,
                       "exchange_path": (None if comm is None else "multimem (NVSwitch)" if getattr(comm, "grad_mc", 0)
                                         else "peer loads / stores" if hasattr(comm, "grad_bucket") else "nccl"),
                       "cpus_bound_to_gpu": len(cpus) if cpus else 0,
                       "step_replay": {0: "python loop", 1: "cuda graph", 2: "native tape"}[int(args.graph)],
                       "native_replay_host_us_and_actions": (ex.replay_host_us() if hasattr(ex, "replay_host_us")
                                                             else None),
                       "pieces": plan_pieces, "micro_ops": stats.get("micro_ops", 0),
                       "swap_bytes_per_step": swap_bytes,
                       "swap_link_ms_per_step": round(link_ms, 2),
                       "swap_roofline_fraction": round(link_ms / ms_per_step, 3),
                       "host_link_gbs_measured": link,
                       "peak_bytes_in_pool": int(peak_in_pool),
                       "bytes_outside_cap": max(0, torch_bytes - cap_bytes),
                       "bytes_outside_cap_what": "parameters, momentum slots, feed buffers, batch-norm side buffers, "
                                                 "kernel scratch (torch.cuda.max_memory_allocated minus the pool arena); "
                                                 "plus library scratch obtained with cudaMalloc, see library_scratch_bytes",
                       "library_scratch_bytes": library_scratch_bytes(),
                       "params_equal_across_ranks": params_equal,
                       "same_policy_at_smaller_batch": also},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "img/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
        }))
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
