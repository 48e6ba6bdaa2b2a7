"""Capped activation pool: one arena tensor + the native offset allocator.

``MemoryPool(ctx, capacity_bytes)`` reserves the whole budget up front (device
memory on a CUDA context, host memory on the simulated device) and serves
``ndarray.empty`` through ``ndarray.set_pool(ctx, pool)``.  Running out raises
:class:`tsplit_b200.ndarray.OutOfHBMBudget`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int64, c_void_p

import torch

from .. import _base
from .. import ndarray

_ALIGN = 256


def _lib():
    lib = _base.runtime()
    if not getattr(lib, "_pool_typed", False):
        lib.tsb_pool_create.restype = c_void_p
        lib.tsb_pool_create.argtypes = [c_int64, c_int64]
        lib.tsb_pool_destroy.argtypes = [c_void_p]
        lib.tsb_pool_alloc.argtypes = [c_void_p, c_int64, ctypes.POINTER(c_int64)]
        lib.tsb_pool_alloc_high.argtypes = [c_void_p, c_int64, ctypes.POINTER(c_int64)]
        lib.tsb_pool_free.argtypes = [c_void_p, c_int64]
        lib.tsb_pool_compact.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, ctypes.c_int]
        lib.tsb_pool_try.argtypes = [c_void_p, c_int64]
        lib.tsb_pool_stats.argtypes = [c_void_p, ctypes.POINTER(c_int64)]
        lib.tsb_pool_reset_peak.argtypes = [c_void_p]
        lib.tsb_pool_block_size.restype = c_int64
        lib.tsb_pool_block_size.argtypes = [c_void_p, c_int64]
        lib._pool_typed = True
    return lib


class PoolCorruption(RuntimeError):
    """A guard zone behind a pool block was overwritten (a kernel or copy ran past the end of its tensor)."""


CANARY_BYTES = 256
_CANARY_VALUE = -6.259853398707798e18        # 0xDEADBEEF as an fp32 bit pattern


class MemoryPool(object):
    """``canary=True`` (or ``TSPLIT_POOL_CANARY=1``) is the debug mode that stands in for a memory checker:
    every block gets a 256-byte guard zone behind it, filled with a pattern at allocation and verified when the
    block is freed and by ``check_canaries()``; a damaged zone raises :class:`PoolCorruption` naming the block.
    The check reads device memory back, so it synchronises: not for timed runs."""

    def __init__(self, ctx, capacity_bytes, canary=None):
        import os
        self.canary = bool(int(os.environ.get("TSPLIT_POOL_CANARY", "0"))) if canary is None else bool(canary)
        self._guards = {}            # block offset -> (first float of the guard zone, floats)
        self.ctx = ctx
        self.capacity = int(capacity_bytes) // _ALIGN * _ALIGN
        n_floats = self.capacity // 4
        dev = ctx.torch_device if ctx.device_type == 2 else torch.device("cpu")
        self.arena = torch.empty(n_floats, dtype=torch.float32, device=dev)
        self._views = {}
        self._live = set()
        self.lib = _lib()
        self.handle = self.lib.tsb_pool_create(self.capacity, _ALIGN)
        assert self.handle, "pool creation failed"

    def __del__(self):
        try:
            if self.handle:
                self.lib.tsb_pool_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # -- allocator interface used by ndarray.empty --------------------------------
    def alloc(self, nbytes, long_lived=False):
        """Long-lived blocks and small blocks (< 1/256 of the pool) are carved from the
        top, large short-lived activations from the bottom, so the small ones do not
        pin holes between the large ones."""
        off = c_int64()
        high = long_lived or nbytes * 256 < self.capacity
        fn = self.lib.tsb_pool_alloc_high if high else self.lib.tsb_pool_alloc
        want = int(nbytes) + (CANARY_BYTES + 3 if self.canary else 0)
        rc = fn(self.handle, want, ctypes.byref(off))
        if rc == 0 and self.canary:
            self._arm(off.value, int(nbytes))
        if rc == 5:
            st = self.stats()
            raise ndarray.OutOfHBMBudget(
                "GPU available memory is not enough! need %.1f MB, free %.1f MB (largest block %.1f MB) "
                "of a %.1f MB budget" % (nbytes / 2**20, st["free"] / 2**20, st["largest_free"] / 2**20,
                                         st["capacity"] / 2**20))
        assert rc == 0, "pool alloc error %d" % rc
        o = off.value // 4
        n = max((int(nbytes) + 3) // 4, 1)
        self._live.add(off.value)
        return off.value, self.arena[o:o + n]

    def alloc_view(self, nbytes, shape, channels_last, long_lived=False):
        """``alloc`` plus the shaped tensor view of the block.  A training step asks for the
        same (offset, shape, layout) combinations every iteration, so the views are cached:
        the steady state costs one native call and a dictionary lookup per tensor."""
        off = c_int64()
        high = long_lived or nbytes * 256 < self.capacity
        fn = self.lib.tsb_pool_alloc_high if high else self.lib.tsb_pool_alloc
        want = int(nbytes) + (CANARY_BYTES + 3 if self.canary else 0)
        rc = fn(self.handle, want, ctypes.byref(off))
        if rc == 0 and self.canary:
            self._arm(off.value, int(nbytes))
        if rc != 0:
            if rc == 5:
                st = self.stats()
                raise ndarray.OutOfHBMBudget(
                    "GPU available memory is not enough! need %.1f MB, free %.1f MB (largest block %.1f MB) "
                    "of a %.1f MB budget" % (nbytes / 2**20, st["free"] / 2**20, st["largest_free"] / 2**20,
                                             st["capacity"] / 2**20))
            raise AssertionError("pool alloc error %d" % rc)
        self._live.add(off.value)
        key = (off.value, shape, channels_last)
        view = self._views.get(key)
        if view is None:
            if len(self._views) > 65536:
                self._views.clear()
            o = off.value // 4
            n = max((int(nbytes) + 3) // 4, 1)
            view = self._views[key] = ndarray._make_view(self.arena[o:o + n][:ndarray._numel(shape)], shape,
                                                         channels_last)
        return off.value, view

    def _arm(self, offset, nbytes):
        first = (offset + nbytes + 3) // 4
        n = CANARY_BYTES // 4
        self.arena[first:first + n].fill_(_CANARY_VALUE)
        self._guards[offset] = (first, n)

    def _verify(self, offset):
        g = self._guards.get(offset)
        if g is None:
            return
        zone = self.arena[g[0]:g[0] + g[1]]
        bad = int((zone != _CANARY_VALUE).sum().item())
        if bad:
            raise PoolCorruption("guard zone behind pool block at offset %d damaged (%d of %d words): something wrote "
                                 "past the end of that tensor" % (offset, bad, g[1]))

    def check_canaries(self):
        """Verify the guard zone of every live block (debug mode only)."""
        for off in list(self._guards):
            self._verify(off)

    def free(self, block):
        if self.canary and int(block) in self._guards:
            try:
                self._verify(int(block))
            finally:
                self._guards.pop(int(block), None)
        if self.handle:
            rc = self.lib.tsb_pool_free(self.handle, int(block))
            assert rc == 0, "pool free of unknown block %r" % (block,)
            self._live.discard(int(block))

    def compact(self, max_moves=65536, stream=None):
        """Defragment: pack all live blocks to the bottom and move their bytes.
        Returns {old_block: new_block}; holders of views into the arena must re-bind
        (``NDArray._rebind``).  The caller guarantees that no kernel or copy is in flight.
        ``stream``: the framework stream the moves are issued on (the caller's compute stream, so
        that later launches on it are ordered after the moves); default = torch's current stream."""
        old = (c_int64 * max_moves)()
        new = (c_int64 * max_moves)()
        size = (c_int64 * max_moves)()
        n = self.lib.tsb_pool_compact(self.handle, old, new, size, max_moves)
        moves = {}
        with ndarray._stream_scope(stream):
            for i in range(n):
                o, d, b = old[i] // 4, new[i] // 4, size[i] // 4
                if d + b <= o:
                    self.arena[d:d + b].copy_(self.arena[o:o + b])
                else:                                   # overlapping ranges: go through a temporary
                    self.arena[d:d + b].copy_(self.arena[o:o + b].clone())
                moves[int(old[i])] = int(new[i])
        self._views.clear()
        self._live = {moves.get(b, b) for b in self._live}
        return moves

    def live_blocks(self):
        """Offsets of the blocks that are allocated right now."""
        return set(self._live)

    def try_alloc(self, nbytes):
        return bool(self.lib.tsb_pool_try(self.handle, int(nbytes)))

    def stats(self):
        out = (c_int64 * 7)()
        self.lib.tsb_pool_stats(self.handle, out)
        keys = ("capacity", "used", "free", "largest_free", "peak", "allocs", "fails")
        return dict(zip(keys, [int(v) for v in out]))

    def reset_peak(self):
        self.lib.tsb_pool_reset_peak(self.handle)

    def address_of(self, block):
        return self.arena.data_ptr() + int(block)


class use_pool(object):
    """``with use_pool(ctx, capacity_bytes) as pool:`` — install a capped pool for
    the duration of the block."""

    def __init__(self, ctx, capacity_bytes):
        self.ctx = ctx
        self.pool = MemoryPool(ctx, capacity_bytes)

    def __enter__(self):
        self.prev = ndarray.get_pool(self.ctx)
        ndarray.set_pool(self.ctx, self.pool)
        return self.pool

    def __exit__(self, *a):
        ndarray.set_pool(self.ctx, self.prev)
