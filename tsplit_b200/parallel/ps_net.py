"""Parameter server across processes: a server process hosts the shards (``ParameterServer``) and serves them
over TCP (``csrc/runtime/ps_net.cc``); workers in other processes use :class:`RemoteParameterServer`, which has the
dense / sparse push-pull face of :class:`~tsplit_b200.parallel.ps.ParameterServer` and can therefore stand behind
``ps_gradients`` (``parallel/graph_hooks.py``).  Roles as in the reference (``DMLC_ROLE`` = server / worker,
``src/ps/worker.cc:20-60``); the scheduler's job (rendezvous) is the listening port.

The requests carry no authentication, so the listener binds the loopback interface (127.0.0.1) unless the caller
names another address of the machine.

    # server process                                 # every worker process
    srv = serve(num_servers=2, num_workers=2)        ps = RemoteParameterServer("127.0.0.1", port, worker=rank)
    print(srv.port); srv.wait_for_workers()          ps.init("w", w0) ... ps.push_pull("w", delta, "BSP") ...
"""
from __future__ import annotations

import time
from ctypes import byref, c_char_p, c_int, c_int64, c_void_p

import numpy as np

from .. import _base
from .ps import ParameterServer, _key

OP_INIT, OP_PUSH, OP_PULL, OP_BARRIER, OP_SPARSE_PUSH, OP_SPARSE_PULL, OP_HEARTBEAT, OP_DEAD, OP_BYE = range(1, 10)


class PSConnectionError(RuntimeError):
    """The server did not answer within the worker's timeout (it is gone, or a barrier is waiting for a worker
    that never arrives)."""


def _lib():
    lib = _base.runtime()
    if not getattr(lib, "_psnet_typed", False):
        lib.tsb_psnet_serve.restype = c_void_p
        lib.tsb_psnet_serve.argtypes = [c_void_p, c_int, c_char_p]
        lib.tsb_psnet_port.argtypes = [c_void_p]
        lib.tsb_psnet_connected.argtypes = [c_void_p]
        lib.tsb_psnet_accepted.argtypes = [c_void_p]
        lib.tsb_psnet_gone.argtypes = [c_void_p]
        lib.tsb_psnet_stop.argtypes = [c_void_p]
        lib.tsb_psnet_connect.restype = c_void_p
        lib.tsb_psnet_connect.argtypes = [c_char_p, c_int, c_int]
        lib.tsb_psnet_request.argtypes = [c_void_p, c_int, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                          c_int64, c_void_p, c_int64, c_void_p, c_void_p]
        lib.tsb_psnet_close.argtypes = [c_void_p, c_int]
        lib._psnet_typed = True
    return lib


class ServedParameterServer(object):
    """The shards plus their listener; lives in the server process."""

    def __init__(self, num_servers=2, num_workers=1, port=0, bind_addr="127.0.0.1", **kw):
        self.store = ParameterServer(num_servers=num_servers, num_workers=num_workers, **kw)
        self.lib = _lib()
        self.handle = self.lib.tsb_psnet_serve(self.store.handle, port, str(bind_addr).encode())
        if not self.handle:
            raise RuntimeError("could not listen on %s:%d" % (bind_addr, port))
        self.port = self.lib.tsb_psnet_port(self.handle)
        self.num_workers = num_workers

    def connected(self):
        return self.lib.tsb_psnet_connected(self.handle)

    def gone(self):
        """Workers whose connection ended without a goodbye (crashed or killed)."""
        return self.lib.tsb_psnet_gone(self.handle)

    def wait_for_workers(self, timeout=30.0):
        """Block until every worker has connected and left again (the life of a training job)."""
        t0 = time.time()
        while time.time() - t0 < timeout:
            if self.lib.tsb_psnet_accepted(self.handle) >= self.num_workers and self.connected() == 0:
                return True
            time.sleep(0.02)
        return False

    def stop(self):
        if self.handle:
            self.lib.tsb_psnet_stop(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.stop()
        except Exception:
            pass


def serve(num_servers=2, num_workers=1, port=0, bind_addr="127.0.0.1", **kw):
    return ServedParameterServer(num_servers, num_workers, port, bind_addr, **kw)


class RemoteParameterServer(object):
    """Worker-side handle.  Requests are synchronous (the reply is the completion), so ``wait`` is a no-op and the
    timestamps returned by ``push`` / ``pull`` are the server's."""

    def __init__(self, host, port, worker=0, num_workers=1, timeout=30.0):
        self.lib = _lib()
        self.worker, self.num_workers = int(worker), int(num_workers)
        self.handle = self.lib.tsb_psnet_connect(str(host).encode(), int(port), int(timeout * 1000))
        if not self.handle:
            raise PSConnectionError("no parameter server at %s:%d" % (host, port))

    def _request(self, op, key=0, n=0, aux=0, rows=None, data=None, out=None):
        ts, out_n = c_int64(0), c_int64(0)
        rc = self.lib.tsb_psnet_request(
            self.handle, op, self.worker, key, n, aux,
            rows.ctypes.data if rows is not None else None, data.ctypes.data if data is not None else None,
            data.size if data is not None else 0, out.ctypes.data if out is not None else None,
            out.size if out is not None else 0, byref(ts), byref(out_n))
        if rc < 0:
            raise PSConnectionError("the parameter server did not answer (request %d)" % op)
        return rc, ts.value, out_n.value

    # -- dense ------------------------------------------------------------------
    def init(self, name, value=None, length=None):
        if value is not None:
            v = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
            rc, _, _ = self._request(OP_INIT, _key(name), v.size, 1, data=v)
        else:
            rc, _, _ = self._request(OP_INIT, _key(name), int(length), 0)
        assert rc == 0

    def push(self, name, value, worker=None):
        v = np.ascontiguousarray(value, dtype=np.float32).reshape(-1)
        rc, ts, _ = self._request(OP_PUSH, _key(name), v.size, data=v)
        assert rc == 0 and ts > 0, "push to unknown key or wrong length"
        return ts

    def pull(self, name, out, worker=None):
        assert out.dtype == np.float32 and out.flags.c_contiguous
        rc, ts, n = self._request(OP_PULL, _key(name), out.size, out=out.reshape(-1))
        assert rc == 0 and n == out.size, "pull of unknown key or wrong length"
        return ts

    def wait(self, ts):
        return None

    def barrier(self):
        rc, _, _ = self._request(OP_BARRIER)
        if rc == 5:
            raise PSConnectionError("a worker left the job: the barrier was released without it")
        assert rc == 0

    def push_pull(self, name, delta, mode="BSP", worker=None):
        self.push(name, delta)
        if mode == "BSP":
            self.barrier()
        out = np.empty(np.asarray(delta).size, dtype=np.float32)
        self.pull(name, out)
        if mode == "BSP":
            self.barrier()
        return out

    # -- sparse -----------------------------------------------------------------------
    def sparse_push(self, name, rows, values, worker=None):
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        values = np.ascontiguousarray(values, dtype=np.float32)
        rc, _, _ = self._request(OP_SPARSE_PUSH, _key(name), rows.size, values.shape[1], rows=rows, data=values)
        assert rc == 0

    def sparse_pull(self, name, rows, cols):
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        out = np.empty((rows.size, cols), dtype=np.float32)
        rc, _, n = self._request(OP_SPARSE_PULL, _key(name), rows.size, cols, rows=rows, out=out.reshape(-1))
        assert rc == 0 and n == out.size
        return out

    # -- liveness ---------------------------------------------------------------------
    def heartbeat(self):
        self._request(OP_HEARTBEAT)

    def dead_nodes(self, timeout_ms):
        out = np.empty(64, dtype=np.float32)
        _, _, n = self._request(OP_DEAD, aux=int(timeout_ms), out=out)
        return [int(v) for v in out[:n]]

    def close(self, say_bye=True):
        if self.handle:
            self.lib.tsb_psnet_close(self.handle, int(bool(say_bye)))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
