"""Per-op profile record and swap-cost constants.

The record mirrors the reference's C ``Profiler{time, input_memory,
output_memory, workspace_memory}`` (``src/common/profiler.h:13-22``,
``python/athena/profiler.py:8-32``): time in ms, sizes in MB.  The constants
describe THIS machine class (B200 + PCIe Gen5 host link) instead of the PCIe-3
values the reference hard-codes (``BandWidth = 16*1024/1000`` MB/ms).
"""
from __future__ import annotations

from ._base import get_array_memory

#: host link (pinned host memory <-> device), GB/s per direction with both directions busy; measured on a
#: B200 with ``python -m tsplit_b200.utils.hostlink`` (55.5 / 57.2 GB/s one direction at a time, 49.9 / 50.4
#: GB/s with both).  The one figure every swap cost model in the package uses.
HOST_LINK_GBS = 50.0
#: the same in the reference's unit (MB per ms), ``python/athena/profiler.py:14``
BandWidth = HOST_LINK_GBS * 1024 / 1000
PAGEIN_LATENCY = 0.010e-3
PAGEOUT_LATENCY = 0.010e-3
#: sustained TF32 tensor-core rate of the wide-tile convolution / GEMM kernels (FLOP per ms), the HBM rate the
#: batch-norm / pooling / element-wise passes reach (bytes per ms) and the cost of a launch (ms): the static
#: cost model of every executor (the role of the reference's ``FLOPS_PER_SECOND``, ``profiler.py:8``)
FLOPS_PER_MS = 7.0e11
HBM_BYTES_PER_MS = 5.5e9
LAUNCH_MS = 0.004


class Profiler(object):
    __slots__ = ["time", "input_memory", "output_memory", "workspace_memory"]

    def __init__(self):
        self.time = 0.0
        self.input_memory = 0.0
        self.output_memory = 0.0
        self.workspace_memory = 0.0

    def swap_time(self):
        return self.output_memory / BandWidth


def CreateProfiler():
    return Profiler()


def PrintProfiler(profiler):
    print("time: %.4f ms, input: %.3f MB, output: %.3f MB, workspace: %.3f MB, swap_time: %.4f ms" % (
        profiler.time, profiler.input_memory, profiler.output_memory, profiler.workspace_memory,
        profiler.swap_time()))


def profile_node(node, input_shapes, output_shape, is_static=True, measured_ms=None):
    """Fill ``node.profiler`` (``Op.profile`` role: static estimate or measured time)."""
    p = node.profiler = node.profiler or CreateProfiler()
    p.input_memory = sum(get_array_memory(s) for s in input_shapes if s is not None)
    p.output_memory = get_array_memory(output_shape) if output_shape is not None else 0.0
    p.workspace_memory = node.op.workspace_bytes(node, input_shapes, output_shape) / 2**20
    if is_static or measured_ms is None:
        flops = node.op.flops(node, input_shapes, output_shape)
        p.time = max(flops / FLOPS_PER_MS, (p.input_memory + p.output_memory) * 2**20 / HBM_BYTES_PER_MS) + LAUNCH_MS
    else:
        p.time = measured_ms
    return p
