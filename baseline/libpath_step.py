#!/usr/bin/env python
"""Library-path stand-in for the reference's training step (NOT the reference).

The reference cannot be built offline, so this script measures what its library
calls amount to on this machine: the same VGG-16 (with batch-norm) or ResNet-50
architecture as plain ``torch.nn`` modules in channels-last fp32 storage with TF32
allowed, i.e. cuDNN convolutions / batch-norm, cuBLAS GEMMs, momentum SGD, and
NCCL ``DistributedDataParallel`` when launched with more than one rank.  Same
synthetic data shape, same batch, CUDA-event timing (max over ranks) and clock
sampling as ``bench.py``; no memory cap (the whole HBM is available to it), so it
is the *speed* anchor for a given batch and, with ``--find-max``, shows the largest
batch a keep-everything library path trains under the same byte cap (enforced with
``torch.cuda.set_per_process_memory_fraction``).

    python baseline/libpath_step.py --model vgg16 --batch 256 --steps 10
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        baseline/libpath_step.py --model resnet50 --batch 256

Prints one JSON line with ``"impl": "library-path stand-in"``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def vgg16_bn(num_classes=1000):
    cfg = [(2, 64), (2, 128), (3, 256), (3, 512), (3, 512)]
    layers, cin = [], 3
    for reps, cout in cfg:
        for _ in range(reps):
            layers += [nn.Conv2d(cin, cout, 3, padding=1, bias=False), nn.BatchNorm2d(cout, eps=0.01, momentum=0.01),
                       nn.ReLU(inplace=True)]
            cin = cout
        layers.append(nn.MaxPool2d(2, 2))
    return nn.Sequential(*layers, nn.Flatten(), nn.Linear(512 * 49, 4096, bias=False), nn.ReLU(inplace=True),
                         nn.Linear(4096, 4096, bias=False), nn.ReLU(inplace=True),
                         nn.Linear(4096, num_classes, bias=False))


class Bottleneck(nn.Module):
    def __init__(self, cin, mid, stride):
        super().__init__()
        cout = mid * 4
        self.a = nn.Sequential(nn.Conv2d(cin, mid, 1, bias=False), nn.BatchNorm2d(mid), nn.ReLU(inplace=True),
                               nn.Conv2d(mid, mid, 3, stride=stride, padding=1, bias=False), nn.BatchNorm2d(mid),
                               nn.ReLU(inplace=True), nn.Conv2d(mid, cout, 1, bias=False), nn.BatchNorm2d(cout))
        self.short = None
        if stride != 1 or cin != cout:
            self.short = nn.Sequential(nn.Conv2d(cin, cout, 1, stride=stride, bias=False), nn.BatchNorm2d(cout))

    def forward(self, x):
        s = x if self.short is None else self.short(x)
        return torch.relu(self.a(x) + s)


def resnet50(num_classes=1000):
    layers = [nn.Conv2d(3, 64, 7, stride=2, padding=3, bias=False), nn.BatchNorm2d(64), nn.ReLU(inplace=True),
              nn.MaxPool2d(3, 2, 1)]
    cin = 64
    for i, (mid, reps) in enumerate(zip([64, 128, 256, 512], [3, 4, 6, 3])):
        for r in range(reps):
            layers.append(Bottleneck(cin, mid, 2 if (r == 0 and i > 0) else 1))
            cin = mid * 4
    return nn.Sequential(*layers, nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(cin, num_classes))


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="vgg16", choices=["vgg16", "resnet50"])
    p.add_argument("--batch", type=int, default=256, help="per-GPU batch")
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--cap-gib", type=float, default=0.0, help="if > 0, cap this process's device memory")
    p.add_argument("--find-max", type=int, default=0,
                   help="1 = double / bisect the batch upward until the capped allocator refuses")
    args = p.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.benchmark = True
    if args.cap_gib > 0:
        total = torch.cuda.get_device_properties(local).total_memory
        torch.cuda.set_per_process_memory_fraction(min(1.0, args.cap_gib * 2**30 / total), local)

    net = (vgg16_bn() if args.model == "vgg16" else resnet50()).cuda().to(memory_format=torch.channels_last)
    model = net
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(net, device_ids=[local])
    opt = torch.optim.SGD(net.parameters(), lr=0.001, momentum=0.9)
    lossf = nn.CrossEntropyLoss()

    def step(x, y):
        opt.zero_grad(set_to_none=True)
        loss = lossf(model(x), y)
        loss.backward()
        opt.step()
        return loss

    def trainable(b):
        try:
            x = torch.randn(b, 3, 224, 224, device="cuda").contiguous(memory_format=torch.channels_last)
            y = torch.randint(0, 1000, (b,), device="cuda")
            for _ in range(2):
                step(x, y)
            torch.cuda.synchronize()
            return True
        except torch.OutOfMemoryError:
            return False
        finally:
            x = y = None
            opt.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()

    max_batch = None
    if args.find_max:
        lo, hi = 8, 16
        assert trainable(lo), "batch 8 does not fit"
        while hi <= 8192 and trainable(hi):
            lo, hi = hi, hi * 2
        while hi - lo > 8:
            mid = (lo + hi) // 16 * 8
            if trainable(mid):
                lo = mid
            else:
                hi = mid
        max_batch = lo
        args.batch = lo

    from bench import ClockSampler
    b = args.batch
    while True:
        try:
            x = torch.randn(b, 3, 224, 224, device="cuda").contiguous(memory_format=torch.channels_last)
            y = torch.randint(0, 1000, (b,), device="cuda")
            for _ in range(max(args.warmup, 3) + args.steps):      # as many steps as the timed loop will run
                loss = step(x, y)
            torch.cuda.synchronize()
            break
        except torch.OutOfMemoryError:
            if not args.find_max or b <= 8:
                raise
            x = y = loss = None
            opt.zero_grad(set_to_none=True)
            torch.cuda.empty_cache()
            b -= 8                      # the probe passed with a cold allocator; the steady state needs a little more
            max_batch = b
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        loss = step(x, y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    peak = torch.cuda.max_memory_allocated()
    if dist is not None:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        per = ms / args.steps
        print(json.dumps({"impl": "library-path stand-in", "what": "torch.nn + cuDNN/cuBLAS (TF32 allowed, "
                          "channels-last fp32) + momentum SGD" + (" + NCCL DDP" if world > 1 else ""),
                          "metric": "img/s", "model": args.model, "n_gpus": world, "per_gpu_batch": b,
                          "ms_per_step": round(per, 3), "value": round(b * world / per * 1e3, 1),
                          "peak_allocated_gib": round(peak / 2**30, 2), "cap_gib": args.cap_gib or None,
                          "max_batch_found": max_batch, "loss": float(loss.item()), "clocks": clocks,
                          "steps": args.steps, "warmup": max(args.warmup, 3)}))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
