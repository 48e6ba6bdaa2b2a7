"""Counts kernel launches issued through the native kernel libraries.

Every call of a ``tsb_*`` entry point goes through a thin proxy that adds the
number of kernels that entry launches (a lower bound: conditional extra kernels
such as a split-K reduction are not counted)."""
from __future__ import annotations

from ..runtime import tape as _tape

_count = [0]

#: kernels launched per entry point (entries not listed launch one)
KERNELS_PER_ENTRY = {
    "tsb_bn_forward": 3, "tsb_bn_backward": 3, "tsb_softmax_ce": 2, "tsb_layer_norm_grad": 3,
    "tsb_graph_begin": 0, "tsb_graph_end": 0, "tsb_graph_destroy": 0, "tsb_device_status": 0,
    "tsb_mem_info": 0, "tsb_scratch_bytes": 0, "tsb_scratch_trim": 0, "tsb_graph_launch": 0,
    "tsb_event_record": 0, "tsb_stream_wait_event": 0, "tsb_memcpy_async": 0,
}


def reset():
    _count[0] = 0


def count():
    return _count[0]


def add(n):
    """Kernels launched without an entry-point call (a replayed CUDA graph launches what it captured)."""
    _count[0] += int(n)


class CountingLib(object):
    """Proxy around a ``ctypes.CDLL`` that counts launches per call."""

    def __init__(self, lib, count=True):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_wrapped", {})
        object.__setattr__(self, "_counts", bool(count))      # False: a host library (its calls launch no kernel)

    def __getattr__(self, name):
        w = self._wrapped.get(name)
        if w is not None:
            return w
        fn = getattr(self._lib, name)
        k = KERNELS_PER_ENTRY.get(name, 1) if self._counts else 0
        if not name.startswith("tsb_") or name in _tape.NOT_ACTIONS:
            return fn

        def call(*a, _fn=fn, _k=k, _name=name, _active=_tape.ACTIVE):
            _count[0] += _k
            rc = _fn(*a)
            if _active[0] is not None:
                _active[0].record(_name, _fn, a, _k)      # a step is being recorded for native replay
            return rc
        self._wrapped[name] = call
        return call
