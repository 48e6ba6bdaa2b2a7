"""Memory policies expressed as classifications for the plan-driven engine."""
from __future__ import annotations

import math

from .engine import MemoryExecutor, KEEP, SWAP, DROP


def _is_conv(n):
    return n.op.name == "Conv2d"


class vdnnExecutor(MemoryExecutor):
    """vDNN (reference ``gpu_ops/vdnnExecutor.py:132-157,202-330``).

    ``policy="all"``: every forward activation that backward needs is offloaded
    at its last forward use; ``policy="conv"``: only the inputs of forward
    convolutions.  In backward each offloaded tensor is prefetched while the
    previous one's consumer computes (the reference's ``findPrefetchNode``
    look-ahead, ``vdnnExecutor.py:121-130``), otherwise fetched on demand."""
    policy_name = "vdnn"

    def classify(self):
        self.cls, self.prefetch_at = {}, {}
        mode = self.policy or "all"
        assert mode in ("all", "conv"), "vdnn policy must be 'all' or 'conv'"
        if mode == "all":
            for n in self.managed:
                self.cls[n] = SWAP
        else:
            conv_inputs = set()
            for n in self.topo_order:
                if _is_conv(n) and self.is_fwd[n]:
                    conv_inputs.add(n.inputs[0])
            for n in self.managed:
                if n in conv_inputs:
                    self.cls[n] = SWAP
        swapped = sorted((n for n, c in self.cls.items() if c == SWAP), key=lambda n: self.first_bwd_use[n])
        for prev, nxt in zip(swapped, swapped[1:]):
            self.prefetch_at.setdefault(self.first_bwd_use[prev], []).append(nxt)
        if swapped:
            self.prefetch_at.setdefault(self.first_bwd_index, []).append(swapped[0])


class recomputeExecutor(MemoryExecutor):
    """Chen-style sub-linear recompute (reference
    ``gpu_ops/recomputeExecutor.py:118-165,186-260``): checkpoints are chosen so
    that no segment between two checkpoints exceeds B = sqrt(x*y) bytes, where x
    is the total size of forward activations and y the largest one; everything
    else is dropped after its last forward use and rebuilt on demand.
    ``policy="speed"`` keeps rebuilt intermediates until their last use,
    ``policy="memory"`` frees them at once (and rebuilds again when needed)."""
    policy_name = "recompute"

    def __init__(self, *a, **kw):
        MemoryExecutor.__init__(self, *a, **kw)
        assert (self.policy or "speed") in ("speed", "memory"), "recompute policy must be 'speed' or 'memory'"
        self.recompute_mode = self.policy or "speed"

    def classify(self):
        self.cls, self.prefetch_at = {}, {}
        sizes = [self.tensor_bytes(n) for n in self.managed]
        if not sizes:
            return
        budget = math.sqrt(float(sum(sizes)) * float(max(sizes)))
        acc = 0.0
        self.checkpoints = []
        for n in self.managed:
            acc += self.tensor_bytes(n)
            if acc > budget:
                self.checkpoints.append(n)
                acc = 0.0
            else:
                self.cls[n] = DROP


class superNeuronsExecutor(MemoryExecutor):
    """SuperNeurons (reference ``gpu_ops/superNeuronsExecutor.py:193-220,395-595``):
    convolution outputs are offloaded but stay in an LRU tensor cache on the
    device until memory is actually needed; every other forward activation is
    dropped and recomputed from the nearest resident tensors, freeing rebuilt
    intermediates as soon as they are consumed."""
    policy_name = "superneurons"
    lazy_evict = True
    recompute_mode = "memory"

    def classify(self):
        self.cls, self.prefetch_at = {}, {}
        for n in self.managed:
            self.cls[n] = SWAP if _is_conv(n) else DROP
        swapped = sorted((n for n, c in self.cls.items() if c == SWAP), key=lambda n: self.first_bwd_use[n])
        # prefetch the next offloaded tensor at each filter-gradient node
        wgrads = [i for i, n in enumerate(self.topo_order) if n.op.name == "Conv2dGradFilter"]
        for t in swapped:
            before = [i for i in wgrads if i < self.first_bwd_use[t]]
            if before:
                self.prefetch_at.setdefault(before[-1], []).append(t)


class capuchinExecutor(MemoryExecutor):
    """Capuchin-style executor (the reference ships only a dead draft,
    ``gpu_ops/capuchinExecutor.py:129-168,302-318``).  The first iteration runs
    in a measuring mode (every candidate is offloaded lazily, evicted only under
    pressure) and records when each tensor is accessed; later iterations use
    those measurements: a tensor is swapped when its idle interval hides the
    transfer, recomputed when that is cheaper per byte saved, and only as many
    tensors are evicted as the budget requires.  Swap-ins are triggered early
    enough (by measured time) to arrive before the first backward use."""
    policy_name = "capuchin"
    lazy_evict = True
    spill_on_pressure = True

    def __init__(self, *a, host_link_gbs=None, **kw):
        MemoryExecutor.__init__(self, *a, **kw)
        from ..profiler import HOST_LINK_GBS
        self.host_link_gbs = HOST_LINK_GBS if host_link_gbs is None else host_link_gbs
        self.measured = None

    def classify(self):
        self.cls, self.prefetch_at = {}, {}
        if self.measured is None:
            for n in self.managed:                 # measuring mode
                self.cls[n] = SWAP
            return
        t_of = self.measured                        # schedule index -> start time (ms)
        need = self.required_saving
        bw = self.host_link_gbs * 1e6               # bytes per ms
        cands = []
        for n in self.managed:
            b = self.tensor_bytes(n)
            idle = t_of[self.first_bwd_use[n]] - t_of[self.last_fwd_use[n]]
            swap_overhead = max(0.0, 2.0 * b / bw - idle)
            rec_cost = self.op_ms.get(n, 0.0) if getattr(n.op, "cheap", False) or n.op.name in (
                "BatchNorm", "MaxPool2d", "AvgPool2d") else float("inf")
            if swap_overhead <= rec_cost:
                cands.append((b / (swap_overhead + 1e-3), n, SWAP, b))
            else:
                cands.append((b / (rec_cost + 1e-3), n, DROP, b))
        cands.sort(key=lambda c: -c[0])
        saved = 0
        for _, n, c, b in cands:
            if saved >= need:
                break
            self.cls[n] = c
            saved += b
        for n, c in self.cls.items():
            if c != SWAP:
                continue
            due = t_of[self.first_bwd_use[n]] - self.tensor_bytes(n) / bw
            trig = self.first_bwd_use[n]
            while trig > self.first_bwd_index and t_of[trig] > due:
                trig -= 1
            self.prefetch_at.setdefault(trig, []).append(n)

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        if self.measured is None:
            self.trace = []
            out = MemoryExecutor.run(self, feed_dict, convert_to_numpy_ret_vals)
            self._digest_trace()
            self.trace = None
            self._planned_for = None
            self.plan()                             # re-plan with measurements
            return out
        return MemoryExecutor.run(self, feed_dict, convert_to_numpy_ret_vals)

    def _digest_trace(self):
        """Turn the first iteration's op records into per-position start times.
        On a CUDA context the per-op device time comes from an event-timed replay
        (``profile_ops``); the host trace only provides the order."""
        desc_index = {n.desc: i for i, n in enumerate(self.topo_order)}
        self.op_ms = self.profile_ops()
        t, acc = [0.0] * (len(self.topo_order) + 1), 0.0
        for i, n in enumerate(self.topo_order):
            t[i] = acc
            acc += self.op_ms.get(n, 0.0)
        t[len(self.topo_order)] = acc
        self.measured = t
        pool_stats = self.stats.get("peak_bytes", 0)
        total = sum(self.tensor_bytes(n) for n in self.managed)
        budget = self.budget_bytes
        if budget is None:
            from .. import ndarray
            pool = ndarray.get_pool(self.ctx)
            budget = pool.capacity if pool is not None else None
        keep_all_peak = self.estimate_keep_all_peak()
        self.required_saving = max(0, keep_all_peak - int(0.95 * budget)) if budget else 0
        _ = (desc_index, pool_stats, total)

    def estimate_keep_all_peak(self):
        """Peak bytes of the schedule when nothing is evicted (liveness frees only)."""
        live, peak = 0, 0
        free_at = {}
        for n in self.topo_order:
            free_at.setdefault(self.last_use[n], []).append(n)
        from ..ops.misc import PlaceholderOp
        for i, n in enumerate(self.topo_order):
            if not isinstance(n.op, PlaceholderOp) and n not in self.feed_shapes:
                live += self.tensor_bytes(n)
            peak = max(peak, live)
            for t in free_at.get(i, ()):
                if not isinstance(t.op, PlaceholderOp) and t not in self.feed_shapes:
                    live -= self.tensor_bytes(t)
        return peak
