"""Host side of the fused all-reduce + optimizer kernel
(``csrc/comm/fused_allreduce.cu``).

``FusedCommunicator`` lays all parameters out in one flat bucket (each tensor
padded to 4 floats), allocates the gradient bucket, the parameter bucket and the
flag words in peer-mapped symmetric memory (``torch.distributed._symmetric_memory``
does the handle exchange), re-binds every variable to a view of the parameter
bucket, and shards the optimizer state N ways.  One step = copy the gradients
into the bucket, launch one kernel.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import numpy as np
import torch

from .. import _base, ndarray
from ..ops import _gpu as G


class CollectiveTimeout(RuntimeError):
    """A peer never signalled within the kernel's bounded wait."""


def bucket_layout(numels, align=4):
    """Offsets of tensors in the flat bucket (each padded to ``align`` elements)."""
    offs, total = [], 0
    for n in numels:
        offs.append(total)
        total += (int(n) + align - 1) // align * align
    return offs, total


def _lib():
    lib = _base.comm()
    raw = object.__getattribute__(lib, "_lib")
    raw.tsb_fused_shard_elems.restype = c_longlong
    raw.tsb_fused_shard_begin.restype = c_longlong
    return lib


class FusedCommunicator(object):
    def __init__(self, optimizer, dist, use_multimem=None):
        import torch.distributed._symmetric_memory as symm
        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.lib = _lib()
        params = optimizer.params
        self.offsets, self.n = bucket_layout([p.t.numel() for p in params])
        dev = params[0].t.device
        group = dist.group.WORLD
        self.grad_bucket = symm.empty(self.n, dtype=torch.float32, device=dev)
        self.param_bucket = symm.empty(self.n, dtype=torch.float32, device=dev)
        self.flags = symm.empty(64, dtype=torch.int32, device=dev)
        self.grad_bucket.zero_()
        self.param_bucket.zero_()
        self.flags.zero_()
        self.h_grad = symm.rendezvous(self.grad_bucket, group)
        self.h_param = symm.rendezvous(self.param_bucket, group)
        self.h_flags = symm.rendezvous(self.flags, group)
        if use_multimem is None:
            use_multimem = os.environ.get("TSPLIT_NVLS", "0") == "1"
        self.grad_mc = int(self.h_grad.multicast_ptr) if use_multimem and self.h_grad.has_multicast_support else 0
        self.param_mc = int(self.h_param.multicast_ptr) if self.grad_mc else 0
        # move parameters into the bucket and re-bind the variables to views of it
        for node, p, off in zip(optimizer.tensors, params, self.offsets):
            n = p.t.numel()
            seg = self.param_bucket[off:off + n]
            seg.copy_(p.t.as_strided((n,), (1,)))
            view = seg.as_strided(tuple(p.t.shape), tuple(p.t.stride()))
            node.tensor_value = ndarray.NDArray(view, p.ctx, owns=False)
        shard = int(self.lib.tsb_fused_shard_elems(c_longlong(self.n), c_int(self.rank), c_int(self.world)))
        self.shard_begin = int(self.lib.tsb_fused_shard_begin(c_longlong(self.n), c_int(self.rank),
                                                              c_int(self.world)))
        self.shard_elems = shard
        init1 = getattr(optimizer, "initial_accumulator_value", 0.0)
        self.slot1 = torch.full((max(shard, 4),), float(init1), dtype=torch.float32, device=dev)
        self.slot2 = torch.zeros(max(shard, 4), dtype=torch.float32, device=dev)
        self.epoch = 0
        self._ptr_arrays()
        dist.barrier()
        torch.cuda.synchronize()

    def _ptr_arrays(self):
        PT = c_void_p * self.world
        self.grad_ptrs = PT(*[int(p) for p in self.h_grad.buffer_ptrs])
        self.param_ptrs = PT(*[int(p) for p in self.h_param.buffer_ptrs])
        self.flag_ptrs = PT(*[int(p) for p in self.h_flags.buffer_ptrs])

    def reduce_and_update(self, optimizer, grads, stream):
        base = self.grad_bucket.data_ptr()
        for g, off in zip(grads, self.offsets):
            n = g.t.numel()
            G.copy_raw(g.ptr, [1], base + 4 * off, [1], [n], stream)
        self.epoch += 1
        hv = (c_float * 8)(*(list(optimizer.hyper()) + [0.0] * (8 - len(optimizer.hyper()))))
        rc = self.lib.tsb_fused_allreduce_update(
            c_int(optimizer.kind), c_int(self.rank), c_int(self.world), self.grad_ptrs, self.param_ptrs,
            self.flag_ptrs, c_void_p(self.grad_mc), c_void_p(self.param_mc), c_void_p(self.slot1.data_ptr()),
            c_void_p(self.slot2.data_ptr()), c_longlong(self.n), hv, c_uint(self.epoch),
            c_void_p(stream.handle if stream is not None else 0))
        if rc & 0xFF == 4:
            raise CollectiveTimeout("fused all-reduce: a peer did not signal in time (code %x)" % (rc >> 8))
        if rc:
            raise RuntimeError("fused all-reduce failed: " + _base.error_string(rc))

    def check(self, stream):
        st = self.lib.tsb_comm_status(c_void_p(stream.handle if stream is not None else 0))
        if st:
            raise CollectiveTimeout("fused all-reduce: bounded wait ran out (code %x)" % st)


def emulate(kind, grads, params, slot1, slot2, hyper, stream_handle=0):
    """All ranks on one GPU (tests): ``grads`` / ``params`` are lists of flat
    fp32 CUDA tensors of equal length (one per emulated rank)."""
    lib = _lib()
    world = len(grads)
    n = grads[0].numel()
    PT = c_void_p * world
    hv = (c_float * 8)(*(list(hyper) + [0.0] * (8 - len(hyper))))
    rc = lib.tsb_fused_allreduce_emulate(
        c_int(kind), c_int(world), PT(*[g.data_ptr() for g in grads]), PT(*[p.data_ptr() for p in params]),
        c_void_p(slot1.data_ptr() if slot1 is not None else 0),
        c_void_p(slot2.data_ptr() if slot2 is not None else 0), c_longlong(n), hv, c_void_p(stream_handle))
    if rc:
        raise RuntimeError("emulation failed: " + _base.error_string(rc))
