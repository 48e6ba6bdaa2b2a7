"""Streams and events (reference: ``python/athena/stream.py:10-53``).

On a CUDA context these wrap ``torch.cuda.Stream`` / ``torch.cuda.Event`` so the
raw ``cudaStream_t`` can be handed to the hand-written kernels.  On host and
simulated-GPU contexts they are logical objects: every record / wait is appended
to an ordering log that the happens-before checker (``runtime/hbcheck.py``)
inspects, so stream discipline is testable without a GPU.
"""
from __future__ import annotations

import itertools
from ctypes import c_void_p

import torch

from . import _base
from .runtime import tape as _tape

_ids = itertools.count()
ORDER_LOG = []          # (kind, stream_id, event_id) tuples, host contexts only
LOGGING = [False]


def _native(name):
    """The raw library entry (not the counting proxy): the call is only recorded here, torch has made it."""
    return getattr(_base.kernels()._lib, name)


def _is_cuda(ctx):
    return ctx is not None and ctx.device_type == 2


class Stream(object):
    def __init__(self, ctx, torch_stream=None, priority=0):
        self.ctx = ctx
        self.id = next(_ids)
        self.torch_stream = None
        if _is_cuda(ctx):
            self.torch_stream = torch_stream or torch.cuda.Stream(
                device=ctx.torch_device, priority=priority)

    @property
    def handle(self):
        """Raw ``cudaStream_t`` as an integer (0 on host contexts)."""
        return self.torch_stream.cuda_stream if self.torch_stream is not None else 0

    def sync(self):
        if self.torch_stream is not None:
            self.torch_stream.synchronize()
        elif LOGGING[0]:
            ORDER_LOG.append(("sync", self.id, -1))

    def wait_event(self, event):
        if self.torch_stream is not None:
            if event.recorded:
                self.torch_stream.wait_event(event.torch_event)
                rec = _tape.ACTIVE[0]
                if rec is not None:              # a step is being recorded: the same wait as a native action
                    rec.record("tsb_stream_wait_event", _native("tsb_stream_wait_event"),
                               (c_void_p(self.handle), c_void_p(event.torch_event.cuda_event)), 0)
                    rec.hold(event)
        elif LOGGING[0]:
            ORDER_LOG.append(("wait", self.id, event.id))


def create_stream_handle(ctx, priority=0):
    return Stream(ctx, priority=priority)


def current_stream(ctx):
    if _is_cuda(ctx):
        return Stream(ctx, torch_stream=torch.cuda.current_stream(ctx.torch_device))
    return Stream(ctx)


class Event(object):
    def __init__(self, ctx, timing=False):
        self.ctx = ctx
        self.id = next(_ids)
        self.recorded = False
        self._timing = timing
        self.torch_event = None

    def _ensure(self):
        if self.torch_event is None and _is_cuda(self.ctx):
            self.torch_event = torch.cuda.Event(enable_timing=self._timing)

    def record(self, stream_handle=None):
        self._ensure()
        self.recorded = True
        if self.torch_event is not None:
            ts = getattr(stream_handle, "torch_stream", None)
            ts = ts if ts is not None else torch.cuda.current_stream()
            self.torch_event.record(ts)
            rec = _tape.ACTIVE[0]
            if rec is not None:
                rec.record("tsb_event_record", _native("tsb_event_record"),
                           (c_void_p(self.torch_event.cuda_event), c_void_p(ts.cuda_stream)), 0)
                rec.hold(self)
        elif LOGGING[0]:
            ORDER_LOG.append(("record", getattr(stream_handle, "id", -1), self.id))

    def sync(self):
        if self.torch_event is not None and self.recorded:
            self.torch_event.synchronize()

    def query(self):
        if self.torch_event is not None and self.recorded:
            return bool(self.torch_event.query())
        return True

    def elapsed_ms(self, later):
        return self.torch_event.elapsed_time(later.torch_event)


def create_event_handle(ctx, timing=False):
    return Event(ctx, timing)
