"""Attach a gradient communicator to an optimizer for one-process-per-GPU
data-parallel training.

``attach(optimizer, dist, mode)`` broadcasts the parameters from rank 0 and
installs ``optimizer.communicator``; from then on ``Optimizer.update`` hands the
gradients to ``communicator.reduce_and_update`` instead of running the local
optimizer kernel.

* ``mode="nccl"``  — the baseline the reference's communicators amount to
  (``ncclAllReduce`` per gradient tensor, ``src/communication/mpi_nccl_communication.cu:101-120``,
  followed by a separate update kernel).
* ``mode="fused"`` — one hand-written kernel per bucket that reads every peer's
  gradient shard over NVLink, averages in a fixed rank order, applies the
  optimizer to the owned parameter shard and writes the new parameters to all
  peers (``parallel/fused_allreduce.py``).
"""
from __future__ import annotations

import torch

from ..ops import _gpu as G


class NcclCommunicator(object):
    def __init__(self, dist):
        self.dist = dist
        self.world = dist.get_world_size()

    def reduce_and_update(self, optimizer, grads, stream):
        ts = stream.torch_stream
        with torch.cuda.stream(ts):
            for g in grads:
                flat = g.t.as_strided((g.t.numel(),), (1,))
                self.dist.all_reduce(flat)
                flat.mul_(1.0 / self.world)
        s1, s2 = optimizer.slots()
        params = optimizer.params
        for lo in range(0, len(grads), 64):
            hi = lo + 64
            G.optimizer_step(optimizer.kind, params[lo:hi], grads[lo:hi], s1[lo:hi] if s1 else None,
                             s2[lo:hi] if s2 else None, optimizer.hyper(), stream)


def broadcast_parameters(optimizer, dist):
    for p in optimizer.params:
        flat = p.t.as_strided((p.t.numel(),), (1,))
        dist.broadcast(flat, src=0)


def attach(optimizer, dist, mode="fused"):
    broadcast_parameters(optimizer, dist)
    if mode == "nccl":
        optimizer.communicator = NcclCommunicator(dist)
    else:
        from .fused_allreduce import FusedCommunicator
        optimizer.communicator = FusedCommunicator(optimizer, dist)
    return optimizer.communicator
