"""Capture a launch sequence on a framework stream into a CUDA graph and replay it."""
from __future__ import annotations

import ctypes

from .. import _base


class CapturedGraph(object):
    def __init__(self, handle):
        self.handle = handle

    def launch(self, stream):
        rc = _base.kernels().tsb_graph_launch(self.handle, ctypes.c_void_p(stream.handle))
        if rc:
            raise RuntimeError("graph launch failed: " + _base.error_string(rc))

    def __del__(self):
        try:
            if self.handle:
                _base.kernels().tsb_graph_destroy(self.handle)
        except Exception:
            pass


def capture(stream, fn):
    """Run ``fn()`` (which must only enqueue work on ``stream``) under stream
    capture and return the instantiated graph.  Nothing executes during capture."""
    lib = _base.kernels()
    rc = lib.tsb_graph_begin(ctypes.c_void_p(stream.handle))
    if rc:
        raise RuntimeError("graph capture could not start: " + _base.error_string(rc))
    try:
        fn()
    except Exception:
        dummy = ctypes.c_void_p()
        lib.tsb_graph_end(ctypes.c_void_p(stream.handle), ctypes.byref(dummy))
        raise
    exec_handle = ctypes.c_void_p()
    rc = lib.tsb_graph_end(ctypes.c_void_p(stream.handle), ctypes.byref(exec_handle))
    if rc:
        raise RuntimeError("graph capture failed: " + _base.error_string(rc))
    return CapturedGraph(exec_handle)
