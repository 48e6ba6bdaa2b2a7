"""TSplit: micro-tensor planning and execution.

The reference imports ``microopExecutor`` / ``microopOptimizer`` /
``microopPlanner`` (``gpu_ops/__init__.py:9``, ``examples/imagenet_vgg.py:4-5,
123-130``) but does not ship them; only their runtime hooks exist (micro-tensor
views ``src/common/c_runtime_api.cc:212-271``, the input/output overlap allocation
``c_runtime_api.cc:164-210``, swap events on every array
``python/athena/ndarray.py:94-119``, ``SplitOp``, per-op profiler structs).  This
module is a fresh implementation on top of the plan-driven engine:

* ``microopPlanner``   (policy name ``planner``)   — builds the plan only;
* ``microopOptimizer`` (policy name ``simulator``) — dry run: predicted step
  time, peak bytes and feasibility from the native replay;
* ``microopExecutor``  (policy name ``tsplit``)    — plans, then runs.

Planning, once per feed shape:

1. the differentiated graph is lowered to micro-ops over k batch pieces
   (``lowering.py``): operators run piece by piece, every piece of every tensor is
   a tensor of its own (a micro-tensor);
2. the native planner (``csrc/planner/planner.cc``) decides keep / swap /
   recompute per micro-tensor by replaying the step against the real pool
   allocator, and returns the plan as a list of events at schedule positions
   (release, start copy-out, free copied-out block, prefetch);
3. k is chosen among powers of two: the smallest predicted step time among the
   plans that fit.

Execution follows the event list literally.  A copied-out block is freed at its
planned position after the compute stream has been made to wait for the copy's
event, so the sequence of pool operations — and with it the placement of every
block — is the one the planner replayed, whatever the copy timing.
"""
from __future__ import annotations

from ctypes import byref, c_double, c_int, c_int64

import numpy as np

from .. import _base, ndarray
from ..ndarray import OutOfHBMBudget
from ..ops.misc import PlaceholderOp
from ..stream import Event
from .. import stream as _stream
from . import lowering
from .engine import MemoryExecutor, KEEP, SWAP, DROP

F_EVICTABLE, F_RECOMPUTABLE, F_PINNED, F_EXTERNAL = 1, 2, 4, 8
EV_RELEASE, EV_SWAPOUT, EV_FREE, EV_PREFETCH = 0, 1, 2, 3


#: (graph, feed shapes, budget, link, ...) -> (piece count, gap) chosen by an earlier search in this process
_CHOICES = {}


def _arr(ctype, values):
    return (ctype * len(values))(*values)


class Plan(object):
    """Outcome of planning: per-tensor decisions, the event list and the replay's prediction."""

    def __init__(self, cls, last_use, events, summary, fits, pieces=1, micro_ops=0):
        self.cls, self.last_use, self.events = cls, last_use, events
        self.predicted_ms, self.predicted_peak_bytes = summary[0], int(summary[1])
        self.first_over_budget, self.stall_ms = int(summary[2]), summary[3]
        self.fail_need_bytes = int(summary[4])
        self.swap_out_bytes, self.swap_in_bytes = int(summary[5]), int(summary[6])
        self.rebuild_ms, self.rebuilds, self.on_demand = summary[7], int(summary[8]), int(summary[9])
        self.fits = fits
        self.fail_free_bytes = int(summary[10])
        self.footprint_bytes = int(summary[11])
        self.allocs = []
        self.pieces = pieces
        self.micro_ops = micro_ops
        self.memory_curve = None

    def counts(self):
        return {"keep": self.cls.count(KEEP), "swap": self.cls.count(SWAP), "recompute": self.cls.count(DROP),
                "pieces": self.pieces, "micro_ops": self.micro_ops,
                "split_tensors": self.micro_ops}

    def __repr__(self):
        return ("Plan(%s, predicted %.2f ms, peak %.1f MB in a placed region of %.1f MB, swap out/in %.0f/%.0f MB, "
                "rebuilds %d, fits=%s)" % (
                    self.counts(), self.predicted_ms, self.predicted_peak_bytes / 2**20, self.footprint_bytes / 2**20,
                    self.swap_out_bytes / 2**20, self.swap_in_bytes / 2**20, self.rebuilds, self.fits))


class microopExecutor(MemoryExecutor):
    policy_name = "tsplit"
    spill_on_pressure = True
    recompute_mode = "planned"

    def __init__(self, eval_node_list, ctx=None, streams=None, policy=None, budget_bytes=None,
                 host_link_gbs=None, max_split=16, trace=None, use_graph=False, pieces=None,
                 min_split_bytes=None, allow_swap=True, min_gap=None):
        MemoryExecutor.__init__(self, eval_node_list, ctx=ctx, streams=streams, policy=policy,
                                budget_bytes=budget_bytes, trace=trace, use_graph=use_graph)
        from ..profiler import HOST_LINK_GBS
        self.host_link_gbs = float(host_link_gbs if host_link_gbs is not None else HOST_LINK_GBS)
        self.max_split = int(max_split)
        self.fixed_pieces = pieces           # None: chosen by the planner
        self.min_split_bytes = min_split_bytes
        self.allow_swap = bool(allow_swap)
        #: uses closer than this many schedule positions keep a tensor resident (None: chosen by the planner)
        self.fixed_gap = min_gap is not None
        self.min_gap = int(min_gap) if min_gap is not None else 3
        self.plan_result = None
        self.lowered = None
        self.orig_topo_order = list(self.topo_order)
        self.orig_eval_node_list = list(self.eval_node_list)

    # ------------------------------------------------------------------ shapes / lowering
    def infer_shape(self, feed_shapes):
        """Shapes are inferred on the original graph; the plan then installs the lowered schedule."""
        self.topo_order = self.orig_topo_order
        self.eval_node_list = self.orig_eval_node_list
        MemoryExecutor.infer_shape(self, feed_shapes)
        self.orig_shapes, self.orig_layout = self.node_to_shape_map, self.node_layout
        self._graph_ok = None

    def _install(self, low):
        self.lowered = low
        self.topo_order = low.order
        self.node_to_shape_map = low.shapes
        self.node_layout = low.layout
        self.eval_node_list = low.evals
        self.index = {n: i for i, n in enumerate(self.topo_order)}
        self._setup_comm()

    def _lower(self, k):
        msb = self.min_split_bytes
        if msb is None:
            msb = max(self._budget() // 256, 1 << 20)
        return lowering.lower(self.orig_topo_order, self.orig_shapes, self.orig_layout, self.orig_eval_node_list,
                              self.feed_shapes, k, msb)

    # ------------------------------------------------------------------ planning
    def _budget(self):
        if self.budget_bytes is not None:
            return int(self.budget_bytes)
        pool = ndarray.get_pool(self.ctx)
        return int(pool.capacity) if pool is not None else 1 << 60

    def planning_budget(self):
        return self._budget()

    def _graph_arrays(self):
        order = self.topo_order
        idx = self.index
        ms = self.profile_ops()
        evals = set(self.eval_node_list)
        low = self.lowered
        out_bytes, time_ms, flags = [], [], []
        in_ptr, in_idx = [0], []
        for n in order:
            external = isinstance(n.op, PlaceholderOp) or n in self.feed_shapes
            shp = self.node_to_shape_map.get(n)
            f = 0
            if external:
                f |= F_EXTERNAL
            elif shp is not None:
                if n in evals:
                    f |= F_PINNED
                elif n not in low.no_evict:
                    f |= F_EVICTABLE
                    if n not in low.no_rebuild and n.inputs:
                        f |= F_RECOMPUTABLE
            # a gradient that is produced inside the communicator's symmetric array takes no bytes of the region
            out_bytes.append(0 if external or shp is None or n in self._direct else self.tensor_bytes(n))
            time_ms.append(float(ms.get(n, 0.0)))
            flags.append(f)
            for i in n.inputs:
                in_idx.append(idx[i])
            in_ptr.append(len(in_idx))
        return dict(n=len(order), out_bytes=out_bytes, time_ms=time_ms, flags=flags, in_ptr=in_ptr,
                    in_idx=in_idx or [0])

    def _call_planner(self, cls_in=None, budget=None, from_in=None, arrays=None, gap=None, low=None):
        """One native planning call.  ``arrays`` / ``gap`` / ``low``: graph arrays, residency gap and lowering to
        plan for instead of the installed ones (then nothing of ``self`` that a lowering changes is read, so calls
        for different lowerings may run in parallel threads; the native planner keeps no global state)."""
        g = self._graph_arrays() if arrays is None else arrays
        gap = self.min_gap if gap is None else gap
        low = self.lowered if low is None else low
        n = g["n"]
        lib = _base.runtime()
        cap = 64 * (len(g["in_idx"]) + n) + 64
        acap = 32 * n + 64
        while True:
            cls, last, frm = (c_int * n)(), (c_int * n)(), (c_int * n)()
            ek, ep, et = (c_int * cap)(), (c_int * cap)(), (c_int * cap)()
            at, ao = (c_int * acap)(), (c_int64 * acap)()
            cnt, acnt = c_int(0), c_int(0)
            summ = (c_double * 12)()
            mem = (c_int64 * n)()
            rbc = (c_int * n)()
            common = (c_int(n), _arr(c_int64, g["out_bytes"]), _arr(c_double, g["time_ms"]), _arr(c_int, g["flags"]),
                      _arr(c_int, g["in_ptr"]), _arr(c_int, g["in_idx"]),
                      c_int64(self._budget() if budget is None else int(budget)), c_int64(int(gap)),
                      c_double(self.host_link_gbs * 1e6))
            tail = (last, c_int(cap), ek, ep, et, byref(cnt), c_int(acap), at, ao, byref(acnt), summ, mem, rbc)
            if cls_in is None:
                rc = lib.tsb_plan2_search(*common, c_int(int(self.allow_swap)), cls, frm, *tail)
            else:
                cls = _arr(c_int, cls_in)
                frm = _arr(c_int, from_in if from_in is not None else [0] * n)
                rc = lib.tsb_plan2_simulate(*common, cls, frm, *tail)
            if rc == 6:                                  # an output array was too small: the counts say how large
                cap, acap = max(cap, cnt.value + 64), max(acap, acnt.value + 64)
                continue
            break
        assert rc in (0, 5), "planner error %d" % rc
        events = [(ek[i], ep[i], et[i]) for i in range(cnt.value)]
        plan = Plan(list(cls), list(last), events, list(summ), summ[2] < 0, low.pieces, low.micro_ops)
        plan.memory_curve = list(mem)
        plan.active_from = list(frm)
        plan.rebuild_count = list(rbc)
        plan.allocs = [(at[i], ao[i]) for i in range(acnt.value)]
        plan.footprint_bytes = int(summ[11])
        return plan

    def _choice_key(self):
        return (tuple(id(n) for n in self.orig_eval_node_list), tuple(sorted((id(n), tuple(s)) for n, s in
                                                                              self.feed_shapes.items())),
                self._budget(), round(self.host_link_gbs, 3), self.allow_swap, self.max_split, self.min_split_bytes,
                self.fixed_pieces, self.min_gap if self.fixed_gap else None, self._comm is not None)

    def search_plan(self):
        """Lower for each candidate piece count, plan with each candidate residency gap, keep the fastest plan
        that fits (or, when none fits, the one that got furthest).  Installs the chosen lowering.  The chosen
        (piece count, gap) is remembered per graph, feed shape and budget, so that an executor built after a dry
        run (``microopOptimizer``) of the same configuration plans once instead of searching again."""
        key = self._choice_key()
        known = _CHOICES.get(key)
        if known is not None:
            k, gap = known
            low = self._lower(k)
            self._install(low)
            self.min_gap = gap
            plan = self._call_planner()
            plan.min_gap = gap
            if plan.fits:
                return plan
            _CHOICES.pop(key, None)             # not this configuration after all: search
        plan = self._search_plan()
        if plan.fits:
            _CHOICES[key] = (plan.pieces, plan.min_gap)
        return plan

    def _search_plan(self):
        batch = self._batch()
        if self.fixed_pieces is not None:
            cand = [int(self.fixed_pieces)]
        else:
            cand, k = [1], 2
            while k <= min(self.max_split, batch):
                cand.append(k)
                k *= 2
        best = None

        def consider(low, gap):
            nonlocal best
            self.min_gap = gap
            plan = self._call_planner()
            plan.min_gap = gap
            key = (0, plan.predicted_ms) if plan.fits else (1, -plan.first_over_budget)
            if best is None or key < best[0]:
                best = (key, low, plan)
            return plan, key

        first_gap = self.min_gap if self.fixed_gap else 6
        worse = 0
        for k in cand:
            low = self._lower(k)
            self._install(low)
            plan, key = consider(low, first_gap)
            if plan.fits and k == 1 and not any(c != KEEP for c in plan.cls):
                break                                   # everything fits whole: nothing to gain from pieces
            # more pieces cost launches: once a plan fits and finer splits come out slower, stop refining
            if best[0][0] == 0:
                worse = worse + 1 if key > best[0] else 0
                if worse >= 2:
                    break
        if best[1].pieces > 1 and (self.fixed_pieces is None or not self.fixed_gap) and \
                (best[0][0] != 0 or any(c != KEEP for c in best[2].cls)):
            # The predicted time is not smooth in the residency gap (the greedy search lands in different plans):
            # plan the best piece count with the other gaps too, the planner calls in parallel threads.  (Piece
            # counts between the powers of two were tried as well: VGG-16 at 2048 predicted 7 % faster with 24
            # pieces than with 16 and measured 1 % slower, with a third more swap traffic; they are not searched.)
            k0 = best[1].pieces
            ks = [k0]
            gaps = [first_gap] if self.fixed_gap else [3, 6, 12]
            jobs = []
            for k in ks:
                low = best[1] if k == k0 else self._lower(k)
                self._install(low)
                arrays = self._graph_arrays()
                jobs += [(low, arrays, gap) for gap in gaps if not (k == k0 and gap == first_gap)]
            import os
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1, 12))) as pool:
                plans = list(pool.map(lambda j: self._call_planner(arrays=j[1], gap=j[2], low=j[0]), jobs))
            for (low, _, gap), plan in zip(jobs, plans):
                plan.min_gap = gap
                key = (0, plan.predicted_ms) if plan.fits else (1, -plan.first_over_budget)
                if key < best[0]:
                    best = (key, low, plan)
        _, low, plan = best
        self.min_gap = plan.min_gap
        self._install(low)
        return plan

    def _batch(self):
        for n in self.orig_topo_order:
            if n in self.feed_shapes:
                return int(self.feed_shapes[n][0])
        return 1

    def simulate_plan(self, plan, budget=None):
        p = self._call_planner(cls_in=plan.cls, budget=budget, from_in=getattr(plan, "active_from", None))
        return [p.predicted_ms, p.predicted_peak_bytes, p.first_over_budget, p.stall_ms], p.memory_curve

    def plan(self):
        self.plan_result = plan = self.search_plan()
        self.analyze()
        order = self.topo_order
        flags = self._graph_arrays()["flags"]
        self._managed_set = {n for n, f in zip(order, flags) if f & F_EVICTABLE}      # what an emergency spill may take
        self.cls = {order[i]: c for i, c in enumerate(plan.cls) if c != KEEP}
        self.last_use = {order[i]: lu for i, lu in enumerate(plan.last_use)}
        self.evict_at, self.free_at, self.prefetch_at = {}, {}, {}
        for kind, pos, t in plan.events:
            node = order[t]
            if kind == EV_PREFETCH:
                self.prefetch_at.setdefault(pos, []).append(node)
            elif kind == EV_FREE:
                self.free_at.setdefault(pos, []).append(node)
            else:
                self.evict_at.setdefault(pos, []).append((node, kind))
        self.release_at = {}
        for n in order:
            self.release_at.setdefault(self.last_use[n], []).append(n)
        self.fwd_release_at = {}
        self._use_pos = {}
        for i, n in enumerate(order):
            for u in n.inputs:
                self._use_pos.setdefault(u, []).append(i)

    def _manageable(self, n, evals):
        return False            # the planner manages every tensor through its own flags

    # ------------------------------------------------------------------ planned execution
    def _reset_state(self):
        MemoryExecutor._reset_state(self)
        self.evicting = {}              # node -> device array whose copy-out is in flight (freed at its planned position)
        self.stats["micro_ops"] = 0
        self.stats["micro_transfers"] = 0
        self.stats["planned_frees"] = 0
        self._alloc_seq = 0
        self.hb_accesses, self._hb_blocks, self._hb_overlaps = [], [], {}

    # The plan gives every allocation of the step its byte offset inside one region (the planner's
    # offline placement).  The region is taken from the context's pool as a single block for the
    # duration of the step (or owned by the executor when no pool is installed), so no allocator
    # runs while the step executes and the footprint is known before the first launch.
    def _open_region(self):
        if self.__dict__.get("_region") is not None:
            return
        nbytes = max(int(self.plan_result.footprint_bytes), 256)
        pool = ndarray.get_pool(self.ctx)
        if pool is not None:
            blk, flat = pool.alloc(nbytes)
            self._region, self._region_block, self._region_pool = flat, blk, pool
        else:
            own = self.__dict__.get("_own_region")
            if own is None or own.numel() * 4 < nbytes:
                import torch
                own = self._own_region = torch.empty((nbytes + 3) // 4, dtype=torch.float32,
                                                     device=self.ctx.torch_device)
            self._region, self._region_block, self._region_pool = own, None, None
        self._region_views = self.__dict__.get("_region_views_cache", {}) if (
            self.__dict__.get("_region_key") == (self._region.data_ptr(), id(self.plan_result))) else {}
        self._region_views_cache = self._region_views
        self._region_key = (self._region.data_ptr(), id(self.plan_result))

    def _close_region(self):
        if self.__dict__.get("_region") is None:
            return
        if self._region_pool is not None and self._region_block is not None:
            self._region_pool.free(self._region_block)
        self._region = None

    def _alloc(self, node):
        direct = self._direct.get(node)
        if direct is not None:
            return direct
        shape = self.node_to_shape_map[node]
        cl = bool(self.node_layout.get(node)) and len(shape) == 4 and ndarray.is_cuda_ctx(self.ctx)
        if self.last_use.get(node, 0) >= len(self.topo_order):        # a result: outlives the step and its region
            return ndarray.empty(shape, self.ctx, channels_last=cl, long_lived=True)
        seq = self._alloc_seq
        self._alloc_seq += 1
        allocs = self.plan_result.allocs
        if seq >= len(allocs) or self.topo_order[allocs[seq][0]] is not node:
            raise RuntimeError("step diverged from its plan at allocation %d (%s)" % (seq, node.desc))
        off = allocs[seq][1]
        key = (off, shape, cl)
        view = self._region_views.get(key)
        if view is None:
            n = ndarray._numel(shape)
            o = off // 4
            view = self._region_views[key] = ndarray._make_view(self._region[o:o + max(n, 1)][:n], shape, cl)
        arr = ndarray.NDArray(view, self.ctx, owns=False)
        if _stream.LOGGING[0]:
            self._hb_new_block(arr, seq, off, ndarray._numel(shape) * 4)
        return arr

    # -- happens-before evidence (simulated device, stream logging on): which stream touched which planned
    # block when, and which earlier blocks a new block lies on top of.  `runtime/hbcheck.check(log,
    # executor.hb_accesses)` then proves that every reuse of region bytes is ordered after the last access to
    # the block that held them before (by a record -> wait chain), whatever the copies' timing.
    def _hb_new_block(self, arr, seq, off, size):
        arr._hb_id = seq
        earlier = [i for (i, o, sz) in self._hb_blocks if o < off + size and off < o + sz]
        self._hb_blocks.append((seq, off, size))
        self._hb_overlaps[seq] = earlier

    def _hb_access(self, arr, stream, write):
        if not _stream.LOGGING[0]:
            return
        bid = getattr(arr, "_hb_id", None)
        if bid is None:
            return
        pos = len(_stream.ORDER_LOG)
        for prev in self._hb_overlaps.pop(bid, ()):          # first touch of the block: it overwrites what lay there
            self.hb_accesses.append((pos, stream.id, prev, True))
        self.hb_accesses.append((pos, stream.id, bid, bool(write)))

    def _launch(self, node, out):
        MemoryExecutor._launch(self, node, out)
        if _stream.LOGGING[0]:
            # the launch is submitted after the waits on its inputs' prefetches: its accesses take the place
            # behind them in the ordering log, and the launch an entry of its own
            for i in node.inputs:
                a = self.arr.get(i)
                if a is not None:
                    # an accumulating micro-op writes into its last input
                    mutates = node.attrs.get("first") is False and i is node.inputs[-1]
                    self._hb_access(a, self.stream, mutates)
            if out is not None:
                self._hb_access(out, self.stream, True)
            _stream.ORDER_LOG.append(("launch", self.stream.id, -1))

    def _raw_copy(self, dst, src, stream):
        if _stream.LOGGING[0]:
            self._hb_access(src, stream, False)
            self._hb_access(dst, stream, True)
        MemoryExecutor._raw_copy(self, dst, src, stream)
        if _stream.LOGGING[0]:
            _stream.ORDER_LOG.append(("copy", stream.id, -1))

    def _release(self, node, final=False):
        if node in self._direct:                 # lives in the communicator's array, not in the region
            self.arr.pop(node, None)
            return
        a = self.evicting.pop(node, None)
        if a is not None:
            self.stream.wait_event(a.gpu2cpu_event)      # the copy-out has read the block before it is reused
        a = self.arr.pop(node, None)
        self.swapin_event.pop(node, None)
        if a is not None:
            if node in self.host and a.gpu2cpu_event.recorded:
                self.stream.wait_event(a.gpu2cpu_event)
            a._release()
        if final:
            self.host.pop(node, None)

    def _ensure(self, node, temps):
        if node in self.arr:
            return
        if node in self.evicting:
            self.arr[node] = self.evicting.pop(node)         # needed again before its planned free
            return
        if node in self.host:
            self._swap_in(node)
            return
        assert node.inputs, "tensor %s was released and cannot be rebuilt" % node.desc
        for i in node.inputs:
            self._ensure(i, temps)
            self._lock(i)                      # a nested rebuild must not send it away again
        for i in node.inputs:
            self._unlock(i)
        out = self._alloc(node)
        self.arr[node] = out
        state = getattr(node, "state", None)
        if isinstance(state, dict):
            state["rematerialise"] = True      # ops with per-step side results (batch-norm statistics) reuse them
        try:
            self._launch(node, out)
        finally:
            if isinstance(state, dict):
                state.pop("rematerialise", None)
        self.stats["recomputed_nodes"] += 1
        temps.append(node)
        # inputs that were only needed for this rebuild leave at once (same rule as the planner's replay)
        cur = self.topo_order[self._cursor]
        for i in node.inputs:
            if i in self._leaving and i in self.arr and i not in cur.inputs and i not in self.locked \
                    and i not in self.feed_shapes \
                    and not isinstance(i.op, PlaceholderOp):
                self._release(i)               # its host copy (if any) stays valid until the position's final releases

    def _execute(self):
        if not self.plan_result.fits:
            p = self.plan_result
            raise OutOfHBMBudget(
                "GPU available memory is not enough! no keep / swap / recompute plan over %d batch pieces fits a "
                "budget of %.1f MB (first position that does not fit: %d of %d, %.1f MB requested, %.1f MB free)" % (
                    p.pieces, self._budget() / 2**20, p.first_over_budget, len(p.cls), p.fail_need_bytes / 2**20,
                    p.fail_free_bytes / 2**20))
        self._open_region()
        try:
            self._execute_plan()
        finally:
            if not self.use_graph:
                self.stream.sync() if self.on_device else None
                self._close_region()

    def _execute_plan(self):
        self._advance_device_step()
        if self._comm is not None:
            self._comm.open_step()
        order = self.topo_order
        feeds = self.feed_shapes
        micro = 0
        for idx, node in enumerate(order):
            self._cursor = idx
            if node in self.arr:
                continue
            if isinstance(node.op, PlaceholderOp):
                self.arr[node] = self._placeholder_value(node)
                continue
            for t in self.prefetch_at.get(idx, ()):
                if t in self.host and t not in self.arr and t not in self.evicting:
                    self._swap_in(t, prefetch=True)
            temps = []
            self._leaving = {t for t, kind in self.evict_at.get(idx, ()) if kind == EV_RELEASE}
            self._leaving.update(self.release_at.get(idx, ()))
            for i in node.inputs:
                if i not in feeds:
                    self._ensure(i, temps)
            shape = self.node_to_shape_map[node]
            out = self._alloc(node) if shape is not None else None
            if out is not None:
                self.arr[node] = out
            self._launch(node, out)
            if self._bucket_ready_at:
                self._after_launch(idx)
            if node.attrs.get("piece") is not None:
                micro += 1
            for t, kind in self.evict_at.get(idx, ()):
                if t not in self.arr:
                    continue
                if kind == EV_SWAPOUT:
                    if t not in self.host:
                        self._swap_out(t)
                        self.stats["micro_transfers"] += 1
                    self.evicting[t] = self.arr.pop(t)
                    self.swapin_event.pop(t, None)
                else:
                    self._release(t)
            for t in self.free_at.get(idx, ()):
                if t in self.evicting:
                    self._release(t)
                    self.stats["planned_frees"] += 1
            for t in self.release_at.get(idx, ()):
                if not isinstance(t.op, PlaceholderOp) and t not in feeds:
                    self._release(t, final=True)
        for t in list(self.evicting):
            self._release(t)
        # the copy streams end the step joined to the compute stream (nothing of this step is left in flight on
        # them when the compute stream's work is done; a capture needs that to close)
        for side in (self.d2h_stream, self.h2d_stream):
            if side not in self._side_used:     # (a stream without work of this step is not part of a capture)
                continue
            ev = Event(self.ctx)
            ev.record(side)
            self.stream.wait_event(ev)
        self.stats["micro_ops"] += micro
        assert self._alloc_seq == len(self.plan_result.allocs), "step made %d of %d planned allocations" % (
            self._alloc_seq, len(self.plan_result.allocs))

    def _graph_eligible(self):
        """A planned step is a fixed sequence of launches, copies and event waits at fixed addresses (every
        allocation has its offset in the region, every copy its pinned host buffer), so the whole step, swaps
        included, is captured into one CUDA graph across the three streams and replayed.  Not while tracing; with a
        communicator only as a native tape (``use_graph="tape"``): the fused exchange is a cooperative launch whose
        epoch argument changes every step, which a captured graph cannot hold and the tape supplies at replay."""
        ok = self.__dict__.get("_graph_ok")
        if ok is None:
            ok = self.trace is None
            for n in self.topo_order:
                if n.op.name == "Optimizer":
                    opt = n.attrs.get("optimizer") or n.attrs["orig"].attrs.get("optimizer")
                    if opt is None or (getattr(opt, "communicator", None) is not None and self.replay_mode != "tape"):
                        ok = False
            self._graph_ok = bool(ok) and self._replay_backend_ok()
        return self._graph_ok


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
        return {"predicted_ms": plan.predicted_ms, "predicted_peak_bytes": plan.predicted_peak_bytes,
                "fits": plan.fits, "stall_ms": plan.stall_ms, "plan": plan, "memory_curve": plan.memory_curve,
                "pieces": plan.pieces, "swap_out_bytes": plan.swap_out_bytes, "swap_in_bytes": plan.swap_in_bytes}


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
