"""Host ring all-reduce over TCP (Python face of ``csrc/runtime/ring_allreduce.cc``;
the reference's ``DL_Connect_Init`` / ``DL_Communicate_*`` ZeroMQ ring,
``src/communication/c_communication_nthread.cc:39-125,478-496``)."""
from __future__ import annotations

from ctypes import c_char_p, c_int, c_int64, c_void_p

import numpy as np

from .. import _base


class RingError(RuntimeError):
    pass


class RingAllReduce(object):
    def __init__(self, world, rank, host="127.0.0.1", base_port=29700, timeout_ms=10000):
        lib = _base.runtime()
        lib.tsb_ring_connect.restype = c_void_p
        lib.tsb_ring_connect.argtypes = [c_int, c_int, c_char_p, c_int, c_int]
        lib.tsb_ring_allreduce.argtypes = [c_void_p, c_void_p, c_int64, c_int]
        lib.tsb_ring_close.argtypes = [c_void_p]
        self.lib = lib
        self.nRanks, self.myRank = world, rank
        self.handle = lib.tsb_ring_connect(world, rank, host.encode(), base_port, timeout_ms)
        if not self.handle:
            raise RingError("rank %d could not join the ring (neighbour not reachable within %d ms)"
                            % (rank, timeout_ms))

    def allReduce(self, arr, average=False):
        assert isinstance(arr, np.ndarray) and arr.dtype == np.float32 and arr.flags.c_contiguous
        rc = self.lib.tsb_ring_allreduce(self.handle, arr.ctypes.data, arr.size, int(average))
        if rc == 4:
            raise RingError("a neighbour in the ring went away")
        assert rc == 0
        return arr

    def close(self):
        if self.handle:
            self.lib.tsb_ring_close(self.handle)
            self.handle = None
