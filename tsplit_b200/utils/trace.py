"""Chrome-trace export of an executor's event log.

``MemoryExecutor(trace=[])`` appends ``(kind, node_desc, op_name, t0, t1)``
records (host clock, seconds) for every op launch, swap-out, swap-in and
recompute.  ``to_chrome_trace`` turns them into the JSON that chrome://tracing
and Perfetto read; ``nvtx_range`` wraps a region in an NVTX range when the CUDA
profiler tools are attached."""
from __future__ import annotations

import contextlib
import json

_TRACKS = {"op": 0, "recompute": 0, "swap_in": 1, "swap_out": 2}


def to_chrome_trace(records, path=None):
    events = []
    if records:
        base = min(r[3] for r in records)
        for kind, desc, op, t0, t1 in records:
            events.append({"name": "%s:%s" % (kind, op), "cat": kind, "ph": "X", "pid": 0,
                           "tid": _TRACKS.get(kind, 3), "ts": (t0 - base) * 1e6,
                           "dur": max((t1 - t0) * 1e6, 0.01), "args": {"node": desc}})
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
