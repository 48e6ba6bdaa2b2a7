"""Memory-profile executor (reference ``gpu_ops/profileExecutor.py:19-141``):
shape inference only; reports the total bytes of all node outputs and, beyond
the reference, the liveness peak and a per-op static cost table."""
from __future__ import annotations

from ..ops.misc import PlaceholderOp
from .base import Executor


class profileExecutor(Executor):
    def __init__(self, eval_node_list, ctx=None, streams=None, policy=None):
        Executor.__init__(self, eval_node_list, ctx=None, policy=policy)
        self.total_memory_usage = 0
        self.peak_memory_usage = 0

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        feed_shapes = {n: tuple(v.shape) for n, v in feed_dict.items()}
        self.infer_shape(feed_shapes)
        self.feed_shapes = feed_shapes
        total, live, peak = 0, 0, 0
        users = {}
        for i, n in enumerate(self.topo_order):
            for u in n.inputs:
                users[u] = i
        free_at = {}
        for n in self.topo_order:
            free_at.setdefault(users.get(n, len(self.topo_order)), []).append(n)

        def size(n):
            shp = self.node_to_shape_map[n]
            if shp is None:
                return 0
            b = 4
            for s in shp:
                b *= s
            return b
        for i, n in enumerate(self.topo_order):
            total += size(n)
            if not isinstance(n.op, PlaceholderOp) and n not in feed_shapes:
                live += size(n)
            peak = max(peak, live)
            for t in free_at.get(i, ()):
                if not isinstance(t.op, PlaceholderOp) and t not in feed_shapes and t not in self.eval_node_list:
                    live -= size(t)
        self.total_memory_usage = total / 2**20
        self.peak_memory_usage = peak / 2**20
        print("total_memory_usage: %.3f MB (liveness peak %.3f MB)" % (self.total_memory_usage,
                                                                     self.peak_memory_usage))
        return [None for _ in self.eval_node_list]
