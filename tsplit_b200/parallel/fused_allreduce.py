"""Host side of the fused all-reduce + optimizer kernel
(``csrc/comm/fused_allreduce.cu``).

``FusedCommunicator`` lays all parameters out in one flat array (each tensor
padded to 4 floats), allocates the gradient array, the parameter array and the
flag words in peer-mapped symmetric memory (``torch.distributed._symmetric_memory``
does the handle exchange), re-binds every variable to a view of the parameter
array, and shards the optimizer state N ways.

The flat array is cut into buckets of consecutive tensors.  Executors allocate
each parameter gradient as a view of the gradient array (``grad_array``), so the
backward pass writes gradients where the kernel reads them and no staging copy
exists; as soon as the last gradient of a bucket has been produced the executor
calls ``launch_bucket``, which runs the fused kernel for that bucket on the
communication stream while the backward pass continues.  The optimizer node at
the end of the step only launches what is left and makes the compute stream wait.
The reference reduces one tensor at a time after a stream sync
(``src/communication/mpi_nccl_communication.cu:101-120``).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import numpy as np
import torch

from .. import _base, ndarray
from ..ops import _gpu as G
from ..runtime import tape as _tape


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
    def __init__(self, optimizer, dist, use_multimem=None, bucket_mb=None, overlap_blocks=None):
        import torch.distributed._symmetric_memory as symm
        from ..stream import create_stream_handle
        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.lib = _lib()
        params = optimizer.params
        self.ctx = params[0].ctx
        numels = [p.t.numel() for p in params]
        self.offsets, self.n = bucket_layout(numels)
        dev = params[0].t.device
        group = dist.group.WORLD
        # buckets: consecutive tensors up to `bucket_mb` (a tensor larger than that is a bucket of its own)
        if bucket_mb is None:
            bucket_mb = float(os.environ.get("TSPLIT_BUCKET_MB", "64"))
        limit = int(bucket_mb * 2**20 / 4)
        self.buckets = []                      # (first tensor, last tensor + 1, lo, hi) in flat elements
        first, lo = 0, 0
        for i, n in enumerate(numels):
            end = self.offsets[i] + (n + 3) // 4 * 4
            nxt = i + 1
            if end - lo >= limit or nxt == len(numels):
                self.buckets.append((first, nxt, lo, end))
                first, lo = nxt, end
        self.bucket_of = {}
        for k, (f, l, _, _) in enumerate(self.buckets):
            for i in range(f, l):
                self.bucket_of[i] = k
        nb = len(self.buckets)
        self.grad_bucket = symm.empty(self.n, dtype=torch.float32, device=dev)
        self.param_bucket = symm.empty(self.n, dtype=torch.float32, device=dev)
        self.flags = symm.empty(64 * nb, dtype=torch.int32, device=dev)
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
        # move parameters into the array and re-bind the variables to views of it
        self._shapes = []
        for node, p, off in zip(optimizer.tensors, params, self.offsets):
            n = p.t.numel()
            seg = self.param_bucket[off:off + n]
            seg.copy_(p.t.as_strided((n,), (1,)))
            view = seg.as_strided(tuple(p.t.shape), tuple(p.t.stride()))
            node.tensor_value = ndarray.NDArray(view, p.ctx, owns=False)
            self._shapes.append((tuple(p.t.shape), tuple(p.t.stride())))
        init1 = getattr(optimizer, "initial_accumulator_value", 0.0)
        # optimizer state: one shard per bucket (the kernel indexes it from the start of the owned shard)
        self.slot1, self.slot2 = [], []
        for (_, _, lo, hi) in self.buckets:
            shard = int(self.lib.tsb_fused_shard_elems(c_longlong(hi - lo), c_int(self.rank), c_int(self.world)))
            self.slot1.append(torch.full((max(shard, 4),), float(init1), dtype=torch.float32, device=dev))
            self.slot2.append(torch.zeros(max(shard, 4), dtype=torch.float32, device=dev))
        self.epoch = 0
        self._launched = set()
        self._step_open = False
        self._grad_views = {}
        self.comm_stream = create_stream_handle(self.ctx)
        self.timing = False           # True: time the compute stream's wait for the exchange (exposed_ms)
        self._exposed = []
        #: thread blocks of a bucket kernel that runs beside the backward pass (the last bucket of a step
        #: has nothing left to overlap with and takes the whole GPU)
        self.overlap_blocks = int(os.environ.get("TSPLIT_OVERLAP_BLOCKS", "48")) if overlap_blocks is None \
            else int(overlap_blocks)
        self._ptr_arrays()
        dist.barrier()
        torch.cuda.synchronize()

    def _ptr_arrays(self):
        PT = c_void_p * self.world
        self._ptrs = []
        for k, (_, _, lo, _) in enumerate(self.buckets):
            self._ptrs.append((PT(*[int(p) + 4 * lo for p in self.h_grad.buffer_ptrs]),
                               PT(*[int(p) + 4 * lo for p in self.h_param.buffer_ptrs]),
                               PT(*[int(p) + 4 * 64 * k for p in self.h_flags.buffer_ptrs])))

    # -- gradients in place ----------------------------------------------------------
    def grad_array(self, i):
        """Array for the gradient of parameter ``i`` that lives inside the symmetric gradient array (same
        shape and strides as the parameter), for executors to hand to the node that produces it."""
        a = self._grad_views.get(i)
        if a is None:
            shape, stride = self._shapes[i]
            n = 1
            for d in shape:
                n *= d
            seg = self.grad_bucket[self.offsets[i]:self.offsets[i] + n]
            a = self._grad_views[i] = ndarray.NDArray(seg.as_strided(shape, stride), self.ctx, owns=False)
        return a

    def _stage(self, grads, tensors, stream):
        """Copy the gradients of ``tensors`` that were not produced in place."""
        base = self.grad_bucket.data_ptr()
        for i in tensors:
            g = grads[i]
            if g.ptr != base + 4 * self.offsets[i]:
                G.copy_raw(g.ptr, [1], base + 4 * self.offsets[i], [1], [g.t.numel()], stream)

    # -- launches ----------------------------------------------------------------------
    def open_step(self):
        """Start a step: no bucket launched yet, next epoch of the flag words.  Executors that launch buckets
        during backward call it before the first launch; otherwise the optimizer node does."""
        self._launched = set()
        self.epoch += 1
        self._step_open = True

    begin_step = open_step

    def replay_epoch(self):
        """Next epoch of the flag words for a step that is replayed from a recording instead of issued here."""
        self.epoch += 1
        self._step_open = False
        return c_uint(self.epoch)

    def launch_bucket(self, k, optimizer, compute_stream, overlapped=True):
        """Run the fused kernel for bucket ``k`` on the communication stream, after everything issued so far
        on ``compute_stream`` (which must include the producers of the bucket's gradients)."""
        if k in self._launched:
            return
        self._launched.add(k)
        from ..stream import Event
        ev = Event(self.ctx)
        ev.record(compute_stream)
        self.comm_stream.wait_event(ev)
        first, last, lo, hi = self.buckets[k]
        gp, pp, fp = self._ptrs[k]
        hv = (c_float * 8)(*(list(optimizer.hyper()) + [0.0] * (8 - len(optimizer.hyper()))))
        rc = self.lib.tsb_fused_allreduce_update(
            c_int(optimizer.kind), c_int(self.rank), c_int(self.world), gp, pp, fp,
            c_void_p(self.grad_mc + 4 * lo if self.grad_mc else 0),
            c_void_p(self.param_mc + 4 * lo if self.param_mc else 0), c_void_p(self.slot1[k].data_ptr()),
            c_void_p(self.slot2[k].data_ptr()), c_longlong(hi - lo), hv, _tape.dyn("comm_epoch", c_uint(self.epoch)),
            c_int(self.overlap_blocks if overlapped else 0), c_void_p(self.comm_stream.handle))
        if rc & 0xFF == 4:
            raise CollectiveTimeout("fused all-reduce: a peer did not signal in time (code %x)" % (rc >> 8))
        if rc:
            raise RuntimeError("fused all-reduce failed: " + _base.error_string(rc))

    def reduce_and_update(self, optimizer, grads, stream):
        """Called by the optimizer node: launch the buckets the executor has not launched during backward
        (all of them for an executor that does not know about buckets) and order the compute stream after
        the communication stream."""
        if not self._step_open:
            self.open_step()
        pending = [k for k in range(len(self.buckets)) if k not in self._launched]
        for k in pending:
            first, last, _, _ = self.buckets[k]
            self._stage(grads, range(first, last), stream)
            self.launch_bucket(k, optimizer, stream, overlapped=(k != pending[-1]))
        from ..stream import Event
        if self.timing:
            t0 = Event(self.ctx, timing=True)
            t0.record(stream)
        ev = Event(self.ctx)
        ev.record(self.comm_stream)
        stream.wait_event(ev)
        if self.timing:
            t1 = Event(self.ctx, timing=True)
            t1.record(stream)
            self._exposed.append((t0, t1))
            del self._exposed[:-64]
        self._step_open = False

    def exposed_ms(self, last=None):
        """Time the compute stream spent waiting for the communication stream at the optimizer node in each of
        the ``last`` most recent steps (all recorded ones if None): the part of the gradient exchange that backward
        did not hide.  Needs ``self.timing = True`` before those steps; synchronises."""
        torch.cuda.synchronize()
        pairs = self._exposed if last is None else self._exposed[-int(last):]
        return [a.elapsed_ms(b) for a, b in pairs]

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
