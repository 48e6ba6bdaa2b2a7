"""Parameter server: Python face of ``csrc/runtime/ps_shards.cc``.

``ParameterServer(num_servers, num_workers)`` hosts the shards; workers call
``push`` / ``pull`` (asynchronous, return a timestamp), ``wait``, ``barrier``,
``push_pull`` with ``mode="BSP"`` (push, barrier among workers, pull — the
reference's ``DL_Communicate_BSP``, ``src/ps/worker.cc:108-112``) or
``mode="ASP"`` (push, pull whatever has arrived).  ``PSVector`` / ``PSMatrix``
mirror the user objects of ``ps-lite/include/ps/psmodel``.  Keys are strings
here and hashed to the 64-bit ids of the native layer.
"""
from __future__ import annotations

import ctypes
import zlib
from ctypes import c_double, c_float, c_int, c_int64, c_void_p

import numpy as np

from .. import _base


def _lib():
    lib = _base.runtime()
    if not getattr(lib, "_ps_typed", False):
        lib.tsb_ps_create.restype = c_void_p
        lib.tsb_ps_create.argtypes = [c_int, c_int, c_int, c_int]
        lib.tsb_ps_destroy.argtypes = [c_void_p]
        lib.tsb_ps_init.argtypes = [c_void_p, c_int64, c_void_p, c_int64]
        lib.tsb_ps_push.restype = c_int64
        lib.tsb_ps_push.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_int64]
        lib.tsb_ps_pull.restype = c_int64
        lib.tsb_ps_pull.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_int64]
        lib.tsb_ps_wait.argtypes = [c_void_p, c_int64]
        lib.tsb_ps_barrier.argtypes = [c_void_p]
        lib.tsb_ps_sparse_push.argtypes = [c_void_p, c_int, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        lib.tsb_ps_sparse_pull.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64]
        lib.tsb_ps_cols.argtypes = [c_void_p, c_int, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p, c_int]
        lib.tsb_ps_norm2.restype = c_double
        lib.tsb_ps_norm2.argtypes = [c_void_p, c_int64]
        lib.tsb_ps_nnz.restype = c_int64
        lib.tsb_ps_nnz.argtypes = [c_void_p, c_int64]
        lib.tsb_ps_dot.restype = c_double
        lib.tsb_ps_dot.argtypes = [c_void_p, c_int64, c_int64]
        lib.tsb_ps_axpy.argtypes = [c_void_p, c_int64, c_int64, c_float]
        lib.tsb_ps_heartbeat.argtypes = [c_void_p, c_int]
        lib.tsb_ps_dead_nodes.argtypes = [c_void_p, c_int, c_void_p, c_int]
        lib.tsb_ps_stats.argtypes = [c_void_p, c_void_p]
        lib._ps_typed = True
    return lib


def _key(name):
    return name if isinstance(name, int) else zlib.crc32(str(name).encode()) | (len(str(name)) << 32)


class ParameterServer(object):
    def __init__(self, num_servers=2, num_workers=1, drop_percent=0, resend_timeout_ms=2):
        self.lib = _lib()
        self.num_servers, self.num_workers = num_servers, num_workers
        self.handle = self.lib.tsb_ps_create(num_servers, num_workers, drop_percent, resend_timeout_ms)
        assert self.handle
        self._keep = {}          # timestamp -> buffers that must outlive the asynchronous request

    def __del__(self):
        try:
            if self.handle:
                self.lib.tsb_ps_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    # -- dense ------------------------------------------------------------------
    def init(self, name, value=None, length=None):
        """Create a key from an array, or as zeros of ``length`` (InitAllZeros)."""
        if value is not None:
            v = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
            rc = self.lib.tsb_ps_init(self.handle, _key(name), v.ctypes.data, v.size)
        else:
            rc = self.lib.tsb_ps_init(self.handle, _key(name), None, int(length))
        assert rc == 0

    def push(self, name, value, worker=0):
        v = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
        ts = self.lib.tsb_ps_push(self.handle, worker, _key(name), v.ctypes.data, v.size)
        assert ts > 0, "push to unknown key or wrong length"
        self._keep[ts] = v
        return ts

    def pull(self, name, out, worker=0):
        assert out.dtype == np.float32 and out.flags.c_contiguous
        ts = self.lib.tsb_ps_pull(self.handle, worker, _key(name), out.ctypes.data, out.size)
        assert ts > 0, "pull of unknown key or wrong length"
        self._keep[ts] = out
        return ts

    def wait(self, ts):
        self.lib.tsb_ps_wait(self.handle, ts)
        self._keep.pop(ts, None)

    def barrier(self):
        self.lib.tsb_ps_barrier(self.handle)

    def push_pull(self, name, delta, mode="BSP", worker=0):
        """Push ``delta`` and return the pulled value (BSP: after every worker pushed)."""
        self.wait(self.push(name, delta, worker))
        if mode == "BSP":
            self.barrier()
        out = np.empty(np.asarray(delta).size, dtype=np.float32)
        self.wait(self.pull(name, out, worker))
        if mode == "BSP":
            self.barrier()       # nobody starts the next round's pushes before all pulled
        return out

    # -- sparse / columns -----------------------------------------------------------
    def sparse_push(self, name, rows, values, worker=0):
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        values = np.ascontiguousarray(values, dtype=np.float32)
        rc = self.lib.tsb_ps_sparse_push(self.handle, worker, _key(name), rows.ctypes.data, rows.size,
                                         values.ctypes.data, values.shape[1])
        assert rc == 0

    def sparse_pull(self, name, rows, cols):
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        out = np.empty((rows.size, cols), dtype=np.float32)
        rc = self.lib.tsb_ps_sparse_pull(self.handle, _key(name), rows.ctypes.data, rows.size, out.ctypes.data, cols)
        assert rc == 0
        return out

    def push_cols(self, name, shape, c0, c1, values, worker=0):
        v = np.ascontiguousarray(values, dtype=np.float32)
        assert self.lib.tsb_ps_cols(self.handle, worker, _key(name), shape[0], shape[1], c0, c1, v.ctypes.data, 1) == 0

    def pull_cols(self, name, shape, c0, c1):
        out = np.empty((shape[0], c1 - c0), dtype=np.float32)
        assert self.lib.tsb_ps_cols(self.handle, 0, _key(name), shape[0], shape[1], c0, c1, out.ctypes.data, 0) == 0
        return out

    # -- server-side functions ---------------------------------------------------------
    def norm2(self, name):
        return self.lib.tsb_ps_norm2(self.handle, _key(name))

    def nnz(self, name):
        return self.lib.tsb_ps_nnz(self.handle, _key(name))

    def dot(self, a, b):
        return self.lib.tsb_ps_dot(self.handle, _key(a), _key(b))

    def axpy(self, x, y, alpha):
        assert self.lib.tsb_ps_axpy(self.handle, _key(x), _key(y), alpha) == 0

    def add_to(self, src, dst):
        self.axpy(src, dst, 1.0)

    def minus(self, src, dst):
        self.axpy(src, dst, -1.0)

    # -- liveness ------------------------------------------------------------------------
    def heartbeat(self, node_id):
        self.lib.tsb_ps_heartbeat(self.handle, node_id)

    def dead_nodes(self, timeout_ms):
        out = (c_int * 256)()
        n = self.lib.tsb_ps_dead_nodes(self.handle, timeout_ms, out, 256)
        return [out[i] for i in range(n)]

    def stats(self):
        out = (c_int64 * 4)()
        self.lib.tsb_ps_stats(self.handle, out)
        return dict(zip(("sent", "dropped", "resent", "duplicates"), [int(v) for v in out]))


class PSVector(object):
    """A dense vector living on the servers."""

    def __init__(self, ps, name, length=None, value=None):
        self.ps, self.name = ps, name
        ps.init(name, value, length)
        self.length = length if value is None else np.asarray(value).size

    def push(self, delta, worker=0):
        return self.ps.push(self.name, delta, worker)

    def pull(self, worker=0):
        out = np.empty(self.length, dtype=np.float32)
        self.ps.wait(self.ps.pull(self.name, out, worker))
        return out


class PSMatrix(object):
    """A [rows, cols] matrix on the servers with column-range access."""

    def __init__(self, ps, name, rows, cols, value=None):
        self.ps, self.name, self.shape = ps, name, (rows, cols)
        ps.init(name, value, rows * cols)

    def push_cols(self, c0, c1, values, worker=0):
        self.ps.push_cols(self.name, self.shape, c0, c1, values, worker)

    def pull_cols(self, c0, c1):
        return self.ps.pull_cols(self.name, self.shape, c0, c1)

    def pull_rows(self, rows):
        return self.ps.sparse_pull(self.name, rows, self.shape[1])

    def push_rows(self, rows, values, worker=0):
        self.ps.sparse_push(self.name, rows, values, worker)
