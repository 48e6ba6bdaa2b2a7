"""Parameter server with GPU-resident shards on one NVLink / NVSwitch box.

Same contract as the host server (``parallel/ps.py``; reference: ``src/ps/worker.cc:108-133``, graph
hook ``python/athena/autodiff.py:264-327``): a worker pushes ``-lr / workers * gradient`` for a key and
pulls the key's value back, with a barrier in between (``BSP``) or without (``ASP``).  Here every rank
of a ``torch.distributed`` job is a worker AND serves one slice of every key: the values live in one
flat array in symmetric (peer-mapped) memory, and a push / pull is one kernel that adds into, and reads
from, the serving ranks' memory over NVLink — no host copy, no NumPy round trip.

* ``BSP``: push + barrier + pull of all workers is an all-reduce of the deltas applied to the served slice
  and broadcast back: the fused all-reduce + SGD kernel (``csrc/comm/fused_allreduce.cu``) on the key.
* ``ASP``: ``csrc/comm/ps_shards_gpu.cu`` — ``red.add`` of the worker's delta into the serving ranks,
  then a read of every slice; no wait on any peer.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p

import torch

from .. import _base, ndarray
from ..ops import _gpu as G
from .fused_allreduce import CollectiveTimeout, _lib, bucket_layout


class GpuParameterServer(object):
    def __init__(self, dist):
        self.dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.num_workers = self.world
        self.num_servers = self.world
        self.lib = _lib()
        self._pending = []            # (name, flat fp32 CUDA tensor) until finalize()
        self.keys = {}
        self.ready = False

    # -- key space -----------------------------------------------------------------
    def init(self, name, value):
        """Register a key with its initial value (a CUDA ``NDArray`` or anything ``ndarray.array`` takes).
        All ranks must register the same keys in the same order, then call :meth:`finalize`."""
        assert not self.ready, "keys are registered before the first push"
        t = value.t if isinstance(value, ndarray.NDArray) else torch.as_tensor(value, dtype=torch.float32).cuda()
        self._pending.append((name, t, tuple(t.shape), tuple(t.stride())))

    def finalize(self):
        """Allocate the key array (values), the delta array and the flag words in symmetric memory, copy the
        initial values of rank 0 in, and exchange the peer handles."""
        if self.ready:
            return
        import torch.distributed._symmetric_memory as symm
        numels = [t.numel() for _, t, _, _ in self._pending]
        offs, self.n = bucket_layout(numels)
        # every key is padded so that its slices are 16-byte aligned for any rank count
        dev = self._pending[0][1].device
        group = self.dist.group.WORLD
        self.values = symm.empty(self.n, dtype=torch.float32, device=dev)      # served values (and, BSP, the local copy)
        self.deltas = symm.empty(self.n, dtype=torch.float32, device=dev)      # what this worker pushes (BSP)
        self.flags = symm.empty(64 * len(numels), dtype=torch.int32, device=dev)
        self.local = torch.zeros(self.n, dtype=torch.float32, device=dev)      # ASP: this worker's pulled copy
        self.values.zero_()
        self.deltas.zero_()
        self.flags.zero_()
        for (name, t, shape, stride), off, n in zip(self._pending, offs, numels):
            flat = t.as_strided((n,), (1,)) if t.dim() else t.reshape(1)
            self.values[off:off + n].copy_(flat)
            self.keys[name] = (len(self.keys), off, n, shape, stride)
        self.dist.broadcast(self.values, src=0)
        self.local.copy_(self.values)
        self.h_values = symm.rendezvous(self.values, group)
        self.h_deltas = symm.rendezvous(self.deltas, group)
        self.h_flags = symm.rendezvous(self.flags, group)
        self.epochs = [0] * len(numels)
        self.dist.barrier()
        torch.cuda.synchronize()
        self._pending = []
        self.ready = True

    def value_array(self, name, asp=False):
        """This rank's view of a key's value (the array a variable is re-bound to)."""
        _, off, n, shape, stride = self.keys[name]
        src = self.local if asp else self.values
        return ndarray.NDArray(src[off:off + n].as_strided(shape, stride), ndarray.gpu(src.device.index), owns=False)

    # -- push / pull ---------------------------------------------------------------------
    def push_pull_device(self, name, grad, lr, mode="BSP", stream=None):
        """Push ``-lr / workers * grad`` for ``name`` and pull the value; returns the NDArray that now holds
        this worker's view of the value.  Everything stays on the device and on ``stream``."""
        self.finalize()
        idx, off, n, shape, stride = self.keys[name]
        n4 = (n + 3) // 4 * 4
        sh = c_void_p(stream.handle if stream is not None else 0)
        PT = c_void_p * self.world
        if mode == "BSP":
            # stage the gradient where the peers read it, then all-reduce + SGD + broadcast on the key's slice
            G.copy_raw(grad.ptr, [1], self.deltas.data_ptr() + 4 * off, [1], [n], stream)
            self.epochs[idx] += 1
            hv = (c_float * 8)(float(lr), 0, 0, 0, 0, 0, 0, 0)
            rc = self.lib.tsb_fused_allreduce_update(
                c_int(0), c_int(self.rank), c_int(self.world),
                PT(*[int(p) + 4 * off for p in self.h_deltas.buffer_ptrs]),
                PT(*[int(p) + 4 * off for p in self.h_values.buffer_ptrs]),
                PT(*[int(p) + 4 * 64 * idx for p in self.h_flags.buffer_ptrs]), c_void_p(0), c_void_p(0),
                c_void_p(0), c_void_p(0), c_longlong(n4), hv, c_uint(self.epochs[idx]), c_int(0), sh)
            if rc & 0xFF == 4:
                raise CollectiveTimeout("parameter server (BSP): a worker did not push in time (code %x)" % (rc >> 8))
            if rc:
                raise RuntimeError("parameter server push/pull failed: " + _base.error_string(rc))
            return self.value_array(name)
        assert mode == "ASP", mode
        # staged into the (4-float padded, zero-tailed) delta array so the kernel may read whole 16-byte pieces
        G.copy_raw(grad.ptr, [1], self.deltas.data_ptr() + 4 * off, [1], [n], stream)
        rc = _base.comm().tsb_ps_gpu_asp(
            PT(*[int(p) + 4 * off for p in self.h_values.buffer_ptrs]), c_void_p(self.deltas.data_ptr() + 4 * off),
            c_void_p(self.local.data_ptr() + 4 * off), c_longlong(n4), c_int(self.world),
            c_float(-float(lr) / self.world), sh)
        if rc:
            raise RuntimeError("parameter server push/pull failed: " + _base.error_string(rc))
        return self.value_array(name, asp=True)

    def barrier(self):
        self.dist.barrier()

    def pull_device(self, name):
        """Fresh copy of a key's value read from its serving ranks (zero delta push)."""
        self.finalize()
        _, off, n, _, _ = self.keys[name]
        zero = ndarray.NDArray(torch.zeros((n + 3) // 4 * 4, device=self.values.device), ndarray.gpu(
            self.values.device.index), owns=False)
        return self.push_pull_device(name, zero, 0.0, mode="ASP")
