"""Chrome-trace export of an executor's event log.

``MemoryExecutor(trace=[])`` appends ``(kind, node_desc, op_name, t0, t1)``
records (host clock, seconds) for every op launch, swap-out, swap-in and
recompute: when the HOST issued them.  On a CUDA context the executor also
brackets every action with a pair of timing events on the stream it runs on;
``executor.device_trace()`` resolves them to ``(kind, node, op, stream, start ms,
end ms)`` ON THE DEVICE, which is the picture that shows whether the copies of a
swap plan hide behind the kernels.  ``to_chrome_trace`` turns either (or both)
into the JSON that chrome://tracing and Perfetto read: process 0 = host issue
times, process 1 = device times with one track per stream.  While tracing, every
launch is also wrapped in an NVTX range (``nvtx_range``) named after its node."""
from __future__ import annotations

import contextlib
import json

_TRACKS = {"op": 0, "recompute": 0, "swap_in": 1, "swap_out": 2}


def to_chrome_trace(records, path=None, device_records=None):
    events = []
    if records:
        base = min(r[3] for r in records)
        for kind, desc, op, t0, t1 in records:
            events.append({"name": "%s:%s" % (kind, op), "cat": kind, "ph": "X", "pid": 0,
                           "tid": _TRACKS.get(kind, 3), "ts": (t0 - base) * 1e6,
                           "dur": max((t1 - t0) * 1e6, 0.01), "args": {"node": desc}})
    if device_records:
        streams = {}
        for kind, desc, op, sid, a, b in device_records:
            tid = streams.setdefault(sid, len(streams))
            events.append({"name": "%s:%s" % (kind, op), "cat": "device:" + kind, "ph": "X", "pid": 1, "tid": tid,
                           "ts": a * 1e3, "dur": max((b - a) * 1e3, 0.01), "args": {"node": desc, "stream": sid}})
    doc = {"traceEvents": events, "displayTimeUnit": "ms"}
    if path:
        with open(path, "w") as f:
            json.dump(doc, f)
    return doc


@contextlib.contextmanager
def nvtx_range(name):
    try:
        import torch
        pushed = torch.cuda.is_available()
        if pushed:
            torch.cuda.nvtx.range_push(name)
    except Exception:
        pushed = False
    try:
        yield
    finally:
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()
