"""TSplit: micro-tensor planning and execution.

The reference imports ``microopExecutor`` / ``microopOptimizer`` /
``microopPlanner`` (``gpu_ops/__init__.py:9``, ``examples/imagenet_vgg.py:4-5,
123-130``) but does not ship them; only their runtime hooks exist (micro-tensor
views ``src/common/c_runtime_api.cc:212-271``, swap events on every array
``python/athena/ndarray.py:94-119``, per-op profiler structs).  This module is a
fresh implementation on top of the plan-driven engine:

* ``microopPlanner``   (policy name ``planner``)   — builds the plan only;
* ``microopOptimizer`` (policy name ``simulator``) — dry run: predicted step
  time, peak bytes and feasibility from the native timeline simulator;
* ``microopExecutor``  (policy name ``tsplit``)    — plans, then runs.

Plan = per forward tensor {keep | swap | recompute}, a micro-tensor count k for
swapped tensors, and a prefetch trigger.  A tensor with k > 1 moves over the
host link as k batch slices with one event each; batch-separable consumers
(convolution forward / data gradient, ReLU and its gradient, pooling, add,
dropout) then run as k micro-ops, each waiting only for its own slice, so the
transfer of slice j+1 overlaps the compute on slice j.
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_int64

import numpy as np

from .. import _base, ndarray
from ..ops.misc import PlaceholderOp
from ..stream import Event
from .engine import MemoryExecutor, KEEP, SWAP, DROP

#: ops whose batch slices can be computed independently (all batch-sized inputs are sliced alike)
BATCH_SEPARABLE = {"Conv2d", "Conv2dGradData", "Relu", "ReluGradient", "Add", "Mul", "MaxPool2d", "AvgPool2d",
                   "MaxPool2dGradient", "AvgPool2dGradient", "Dropout", "DropoutGradient", "AddConst", "MulConst"}
#: ops that are cheap enough to rebuild instead of moving their output over the host link
RECOMPUTABLE = {"Relu", "BatchNorm", "BatchNormRelu", "MaxPool2d", "AvgPool2d", "Add", "Mul", "AddConst", "MulConst", "Reshape",
                "Transpose", "Dropout", "Concat", "Slice", "Pad", "Sigmoid", "Tanh", "BroadcastTo",
                "BroadcastShape", "BroadcastToTF", "AddBroadcast", "Conv2dBroadcastTo", "LayerNorm", "Softmax", "Opposite"}


def _arr(ctype, values):
    return (ctype * len(values))(*values)


class Plan(object):
    """Outcome of planning: decisions per schedule position and the simulator's
    prediction for them."""

    def __init__(self, cls, split, prefetch, summary, fits):
        self.cls, self.split, self.prefetch = cls, split, prefetch
        self.predicted_ms, self.predicted_peak_bytes = summary[0], int(summary[1])
        self.first_over_budget, self.stall_ms, self.peak_position = int(summary[2]), summary[3], int(summary[4])
        self.fits = fits

    def counts(self):
        return {"keep": self.cls.count(KEEP), "swap": self.cls.count(SWAP), "recompute": self.cls.count(DROP),
                "split_tensors": sum(1 for k in self.split if k > 1)}

    def __repr__(self):
        return "Plan(%s, predicted %.2f ms, peak %.1f MB, fits=%s)" % (
            self.counts(), self.predicted_ms, self.predicted_peak_bytes / 2**20, self.fits)


class microopExecutor(MemoryExecutor):
    policy_name = "tsplit"
    spill_on_pressure = True

    def __init__(self, eval_node_list, ctx=None, streams=None, policy=None, budget_bytes=None,
                 host_link_gbs=50.0, max_split=8, trace=None, use_graph=False):
        MemoryExecutor.__init__(self, eval_node_list, ctx=ctx, streams=streams, policy=policy,
                                budget_bytes=budget_bytes, trace=trace, use_graph=use_graph)
        self.host_link_gbs = float(host_link_gbs)
        self.max_split = int(max_split)
        self.plan_result = None
        self.split = {}
        #: every forward op may be rebuilt (the planner prices it by the op's time); False restricts
        #: recomputation to the cheap, memory-bound operators
        self.recompute_any = True

    # ------------------------------------------------------------------ planning
    def _budget(self):
        if self.budget_bytes is not None:
            return int(self.budget_bytes)
        pool = ndarray.get_pool(self.ctx)
        return int(pool.capacity * 0.9) if pool is not None else 1 << 62

    def planning_budget(self):
        return self._budget()

    def _graph_arrays(self):
        order = self.topo_order
        idx = self.index
        ms = self.profile_ops()
        evals = set(self.eval_node_list)
        managed = set(self.managed)
        out_bytes, time_ms, phase, mg, rc, sp, ws, pinned = [], [], [], [], [], [], [], []
        in_ptr, in_idx = [0], []
        for n in order:
            external = isinstance(n.op, PlaceholderOp) or n in self.feed_shapes
            out_bytes.append(0 if external else self.tensor_bytes(n))
            time_ms.append(float(ms.get(n, 0.0)))
            phase.append(0 if self.is_fwd[n] else 1)
            mg.append(1 if n in managed else 0)
            rc.append(1 if (n.op.name in RECOMPUTABLE or self.recompute_any) else 0)
            batch_like = self.node_to_shape_map[n] is not None and len(self.node_to_shape_map[n]) >= 1
            sp.append(1 if batch_like else 0)
            try:
                w = n.op.workspace_bytes(n, [self.node_to_shape_map[i] for i in n.inputs],
                                         self.node_to_shape_map[n])
            except Exception:
                w = 0
            ws.append(int(w))
            pinned.append(1 if n in evals else 0)
            for i in n.inputs:
                in_idx.append(idx[i])
            in_ptr.append(len(in_idx))
        return dict(n=len(order), out_bytes=out_bytes, time_ms=time_ms, phase=phase, managed=mg,
                    recomputable=rc, splittable=sp, ws=ws, in_ptr=in_ptr, in_idx=in_idx or [0], pinned=pinned)

    def search_plan(self):
        g = self._graph_arrays()
        n = g["n"]
        lib = _base.runtime()
        cls, split, pre = (c_int * n)(), (c_int * n)(), (c_int * n)()
        out = (c_double * 5)()
        rc = lib.tsb_plan_search(
            c_int(n), _arr(c_int64, g["out_bytes"]), _arr(c_double, g["time_ms"]), _arr(c_int, g["phase"]),
            _arr(c_int, g["managed"]), _arr(c_int, g["recomputable"]), _arr(c_int, g["splittable"]),
            _arr(c_int64, g["ws"]), _arr(c_int, g["in_ptr"]), _arr(c_int, g["in_idx"]), _arr(c_int, g["pinned"]),
            c_int64(self._budget()), c_double(self.host_link_gbs * 1e6), c_int(self.max_split), cls, split, pre,
            out)
        assert rc in (0, 5), "planner error %d" % rc
        return Plan(list(cls), list(split), list(pre), list(out), rc == 0)

    def simulate_plan(self, plan, budget=None):
        g = self._graph_arrays()
        n = g["n"]
        out = (c_double * 5)()
        mem = (c_int64 * n)()
        rc = _base.runtime().tsb_plan_simulate(
            c_int(n), _arr(c_int64, g["out_bytes"]), _arr(c_double, g["time_ms"]), _arr(c_int, g["phase"]),
            _arr(c_int, g["managed"]), _arr(c_int, g["recomputable"]), _arr(c_int, g["splittable"]),
            _arr(c_int64, g["ws"]), _arr(c_int, g["in_ptr"]), _arr(c_int, g["in_idx"]), _arr(c_int, g["pinned"]),
            c_int64(self._budget() if budget is None else int(budget)), c_double(self.host_link_gbs * 1e6),
            _arr(c_int, plan.cls), _arr(c_int, plan.split), _arr(c_int, plan.prefetch), out, mem)
        assert rc == 0
        return list(out), list(mem)

    def classify(self):
        self.plan_result = plan = self.search_plan()
        self.cls, self.prefetch_at, self.split = {}, {}, {}
        for i, n in enumerate(self.topo_order):
            if plan.cls[i] != KEEP:
                self.cls[n] = plan.cls[i]
            if plan.split[i] > 1:
                self.split[n] = plan.split[i]
            if plan.cls[i] == SWAP and plan.prefetch[i] >= 0:
                self.prefetch_at.setdefault(plan.prefetch[i], []).append(n)

    # ------------------------------------------------------------------ micro-tensor transfers
    def _reset_state(self):
        MemoryExecutor._reset_state(self)
        self.micro_events = {}          # node -> [event per batch slice] of an in-flight swap-in
        self.stats["micro_transfers"] = 0
        self.stats["micro_ops"] = 0

    def _slices(self, node, k):
        b = self.node_to_shape_map[node][0]
        k = max(1, min(k, b))
        return [ndarray._split_bounds(b, k, j) for j in range(k)]

    def _copy_slice(self, dst, src, lo, hi, batch, stream):
        """Copy batch rows [lo, hi) of a dense array (the batch is outermost in
        both layouts, so a slice is one contiguous byte range)."""
        n = dst.t.numel()
        per = n // batch
        if self.on_device:
            import torch
            with torch.cuda.stream(stream.torch_stream):
                d = dst.t.as_strided((n,), (1,)) if dst.is_cuda else dst.t.reshape(-1)
                s = src.t.as_strided((n,), (1,)) if src.is_cuda else src.t.reshape(-1)
                d[lo * per:hi * per].copy_(s[lo * per:hi * per], non_blocking=True)
        else:
            dst.t.reshape(-1)[lo * per:hi * per] = src.t.reshape(-1)[lo * per:hi * per]

    def _swap_out(self, node):
        k = self.split.get(node, 1)
        if k <= 1:
            return MemoryExecutor._swap_out(self, node)
        a, h = self.arr[node], self._host_buffer(node)
        ev = Event(self.ctx)
        ev.record(self.stream)
        self.d2h_stream.wait_event(ev)
        batch = a.shape[0]
        for lo, hi in self._slices(node, k):
            self._copy_slice(h, a, lo, hi, batch, self.d2h_stream)
            self.stats["micro_transfers"] += 1
        a.gpu2cpu_event.record(self.d2h_stream)
        self.host[node] = h
        self.stats["swap_out_bytes"] += a.nbytes
        self._log("swap_out", node)

    def _swap_in(self, node, prefetch=False):
        k = self.split.get(node, 1)
        if k <= 1:
            return MemoryExecutor._swap_in(self, node, prefetch)
        if node in self.arr or node in self.swapin_event:
            return
        a, h = self._alloc(node), self.host[node]
        ev = Event(self.ctx)
        ev.record(self.stream)
        self.h2d_stream.wait_event(ev)
        batch, evs = a.shape[0], []
        for lo, hi in self._slices(node, k):
            self._copy_slice(a, h, lo, hi, batch, self.h2d_stream)
            e = Event(self.ctx)
            e.record(self.h2d_stream)
            evs.append(e)
            self.stats["micro_transfers"] += 1
        a.cpu2gpu_event.record(self.h2d_stream)
        self.arr[node] = a
        self.swapin_event[node] = a.cpu2gpu_event
        self.micro_events[node] = evs
        self.stats["swap_in_bytes"] += a.nbytes
        self.stats["prefetch_hits" if prefetch else "on_demand_swapins"] += 1
        self._log("swap_in", node)

    def _release(self, node, final=False):
        self.micro_events.pop(node, None)
        MemoryExecutor._release(self, node, final)

    # ------------------------------------------------------------------ micro-ops
    def _launch(self, node, out):
        streamed = [i for i in node.inputs if i in self.micro_events]
        if (not streamed or node.op.name not in BATCH_SEPARABLE or out is None or len(out.shape) < 1):
            for i in streamed:
                self.micro_events.pop(i, None)
            return MemoryExecutor._launch(self, node, out)
        batch = out.shape[0]
        k = max(len(self.micro_events[i]) for i in streamed)
        if any(len(self.micro_events[i]) != k or self.arr[i].shape[0] != batch for i in streamed):
            for i in streamed:
                self.micro_events.pop(i, None)
            return MemoryExecutor._launch(self, node, out)
        ins = [self.arr[i] for i in node.inputs]
        for i in node.inputs:                      # whole-tensor events of inputs that are not streamed
            if i not in streamed:
                ev = self.swapin_event.pop(i, None)
                if ev is not None:
                    self.stream.wait_event(ev)
        for j in range(k):
            for i in streamed:
                self.stream.wait_event(self.micro_events[i][j])
            lo, hi = ndarray._split_bounds(batch, k, j)
            sl_in = []
            for a, i in zip(ins, node.inputs):
                sliced = isinstance(a, ndarray.NDArray) and len(a.shape) >= 1 and a.shape[0] == batch and \
                    not isinstance(i.op, PlaceholderOp)
                sl_in.append(ndarray.NDArray(a.t.narrow(0, lo, hi - lo), a.ctx, owns=False) if sliced else a)
            sl_out = ndarray.NDArray(out.t.narrow(0, lo, hi - lo), out.ctx, owns=False)
            if self.on_device:
                node.op.compute(node, sl_in, sl_out, False, self.stream)
            else:
                node.op.compute(node, [a.numpy_view() for a in sl_in], sl_out.numpy_view(), True, self.stream)
            self.stats["micro_ops"] += 1
        for i in streamed:
            self.micro_events.pop(i, None)
            self.swapin_event.pop(i, None)


class microopPlanner(microopExecutor):
    """Plan only (example-level policy ``planner``): ``run`` returns the plan."""
    policy_name = "planner"

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        feed_shapes = {n: tuple(np.asarray(v).shape if not hasattr(v, "shape") else v.shape)
                       for n, v in feed_dict.items()}
        self.feed_shapes = feed_shapes
        self.infer_shape(feed_shapes)
        self.plan()
        return self.plan_result


class microopOptimizer(microopPlanner):
    """Dry run (example-level policy ``simulator``): returns a dict with the
    predicted step time, peak bytes and whether the budget is met."""
    policy_name = "simulator"

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        plan = microopPlanner.run(self, feed_dict)
        summary, mem = self.simulate_plan(plan)
        return {"predicted_ms": summary[0], "predicted_peak_bytes": int(summary[1]), "fits": summary[2] < 0,
                "stall_ms": summary[3], "plan": plan, "memory_curve": mem}


def max_batch_search(build_executor, feeds_for_batch, lo=1, hi=4096):
    """Largest batch for which ``build_executor().run(feeds_for_batch(b))``
    does not raise ``OutOfHBMBudget`` (the reference sweeps upward until its
    executor asserts, ``examples/imagenet_vgg.py:174-177``; this bisects)."""
    def ok(b):
        try:
            build_executor().run(feeds_for_batch(b))
            return True
        except ndarray.OutOfHBMBudget:
            return False
    if not ok(lo):
        return 0
    while lo < hi:
        mid = (lo + hi + 1) // 2
        if ok(mid):
            lo = mid
        else:
            hi = mid - 1
    return lo
