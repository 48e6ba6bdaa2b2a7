"""Plan-driven memory-saving execution engine.

One engine runs every memory policy of the reference — vDNN
(``gpu_ops/vdnnExecutor.py:21-340``), SuperNeurons
(``superNeuronsExecutor.py:23-616``), Chen-style recompute
(``recomputeExecutor.py:21-384``), Capuchin (``capuchinExecutor.py:67-364``)
and the TSplit micro-tensor plan.  A policy only *classifies* forward tensors
(keep / swap / drop) and places prefetch triggers; the engine owns liveness,
allocation under the HBM budget, the three streams and the event discipline:

* compute, H2D and D2H streams; a consumer waits on the producer's or the
  swap-in's event, never on the host (the reference synchronises both streams
  after every node, ``vdnnExecutor.py:273-274``);
* device memory read by an in-flight D2H copy is released only when that copy's
  event has completed (event-deferred free), so blocks can be re-used without a
  stream sync;
* running out of budget raises ``OutOfHBMBudget`` instead of asserting.

It runs unchanged on the simulated device (host storage, NumPy kernels), which
is how the policies are tested without a GPU.
"""
from __future__ import annotations

import time
from collections import OrderedDict

import numpy as np

from .. import ndarray
from ..ndarray import OutOfHBMBudget
from ..stream import create_stream_handle, Event
from ..ops.misc import PlaceholderOp
from ..ops import _gpu as G
from .base import Executor

KEEP, SWAP, DROP = 0, 1, 2


def nbytes(shape):
    n = 4
    for s in shape:
        n *= int(s)
    return n


class _TapedStep(object):
    """A step recorded by ``runtime/tape.py``; same ``launch`` face as a captured CUDA graph."""

    def __init__(self, tape, executor):
        self.tape, self.executor = tape, executor

    def launch(self, stream):
        from ..runtime.tape import TapeError
        values = {}
        comm = self.executor._comm
        if comm is not None:
            values["comm_epoch"] = comm.replay_epoch()
        try:
            self.tape.replay(values)
        except TapeError as e:
            if e.entry == "tsb_fused_allreduce_update" and e.status & 0xFF == 4:
                from ..parallel.fused_allreduce import CollectiveTimeout
                raise CollectiveTimeout("fused all-reduce: a peer did not signal in time (code %x)" % (e.status >> 8))
            raise


class MemoryExecutor(Executor):
    """Base of all memory-saving executors."""

    policy_name = "keep"
    lazy_evict = False           # swap-class tensors stay resident until memory is needed (LRU)
    recompute_mode = "speed"     # "speed": keep rematerialised intermediates; "memory": free them at once

    def __init__(self, eval_node_list, ctx=None, streams=None, policy=None, budget_bytes=None, trace=None,
                 use_graph=False):
        Executor.__init__(self, eval_node_list, ctx=ctx, policy=policy)
        # replay of the whole step without the interpreter (see _graph_eligible): use_graph=True / "graph" captures
        # a CUDA graph; use_graph="tape" records the native calls and replays them from a C++ loop
        # (csrc/runtime/step_tape.cc), which also covers steps with a gradient exchange between GPUs
        self.use_graph = bool(use_graph) and self.on_device
        self.replay_mode = "tape" if use_graph == "tape" else "graph"
        self._step_graph = None
        self._graph_steps_seen = 0
        assert ctx is not None and ndarray.is_gpu_ctx(ctx), "memory executors need a (simulated) GPU context"
        if streams is None:
            streams = [self.stream, create_stream_handle(ctx), create_stream_handle(ctx)]
        self.streams = streams
        self.stream, self.h2d_stream, self.d2h_stream = streams[0], streams[1], streams[2]
        self.budget_bytes = budget_bytes
        self.trace = trace
        self.index = {n: i for i, n in enumerate(self.topo_order)}
        self.stats = {}
        self._planned_for = None
        self._direct, self._bucket_ready_at, self._comm, self._comm_opt = {}, {}, None, None

    # ------------------------------------------------------------------ analysis
    def analyze(self):
        """Liveness facts per tensor, in schedule positions."""
        order = self.topo_order
        self.users = {n: [] for n in order}
        for n in order:
            for i in set(n.inputs):
                self.users[i].append(n)
        self.is_fwd = {n: n.phase == "forward" for n in order}
        first_bwd = next((self.index[n] for n in order if n.phase != "forward"), len(order))
        self.first_bwd_index = first_bwd
        self.last_use, self.last_fwd_use, self.first_bwd_use = {}, {}, {}
        evals = set(self.eval_node_list)
        for n in order:
            idx = [self.index[u] for u in self.users[n]]
            self.last_use[n] = max(idx) if idx else self.index[n]
            f = [j for j in idx if j < first_bwd]
            b = [j for j in idx if j >= first_bwd]
            self.last_fwd_use[n] = max(f) if f else self.index[n]
            self.first_bwd_use[n] = min(b) if b else None
            if n in evals:
                self.last_use[n] = len(order)          # never released
        self.managed = [n for n in order if self._manageable(n, evals)]
        self._managed_set = set(self.managed)

    def _manageable(self, n, evals):
        """Forward activations that are needed again in backward."""
        return (self.is_fwd[n] and not isinstance(n.op, PlaceholderOp) and n not in self.feed_shapes
                and self.first_bwd_use.get(n) is not None and n not in evals
                and self.node_to_shape_map[n] is not None)

    def classify(self):
        """Policy hook: fill ``self.cls`` (node -> KEEP/SWAP/DROP) and
        ``self.prefetch_at`` (schedule index -> tensors to swap in early)."""
        self.cls = {}
        self.prefetch_at = {}

    def _extend_sources(self):
        """A dropped tensor is rebuilt from its inputs, so those must stay
        recoverable until the dropped tensor's last use."""
        for n in reversed(self.topo_order):
            if self.cls.get(n, KEEP) == DROP:
                for u in n.inputs:
                    if self.last_use[u] < self.last_use[n]:
                        self.last_use[u] = self.last_use[n]

    def plan(self):
        self._setup_comm()
        self.analyze()
        self.classify()
        self._extend_sources()
        self.release_at = {}
        for n in self.topo_order:
            self.release_at.setdefault(self.last_use[n], []).append(n)
        self.fwd_release_at = {}
        for n, c in self.cls.items():
            if c != KEEP:
                self.fwd_release_at.setdefault(self.last_fwd_use[n], []).append(n)

    # ------------------------------------------------------------------ gradient exchange hooks
    def _setup_comm(self):
        """When the optimizer has a bucketed communicator (``parallel/fused_allreduce.py``): allocate each
        parameter gradient inside the communicator's symmetric gradient array (no staging copy), and note
        after which schedule position each bucket is complete, so that its fused all-reduce + update can be
        launched there and overlap the rest of the backward pass."""
        self._direct, self._bucket_ready_at, self._comm, self._comm_opt = {}, {}, None, None
        if not self.on_device:
            return
        for pos, n in enumerate(self.topo_order):
            if n.op.name != "Optimizer":
                continue
            opt = n.attrs.get("optimizer") or n.attrs.get("orig").attrs.get("optimizer")
            comm = getattr(opt, "communicator", None)
            if comm is None or not hasattr(comm, "launch_bucket"):
                return
            self._comm, self._comm_opt = comm, opt
            index = {m: i for i, m in enumerate(self.topo_order)}
            users = {}
            for m in self.topo_order:
                for i in m.inputs:
                    users.setdefault(i, []).append(m)
            ready = {}
            for i, g in enumerate(n.inputs):
                arr = comm.grad_array(i)
                shp = self.node_to_shape_map.get(g)
                want = ndarray._make_view(arr.t.as_strided((arr.t.numel(),), (1,)), shp,
                                          bool(self.node_layout.get(g)) and len(shp) == 4)
                if tuple(arr.shape) == tuple(shp) and arr.strides == tuple(want.stride()) and g not in self.feed_shapes \
                        and not isinstance(g.op, PlaceholderOp) and g not in self.eval_node_list:
                    self._direct[g] = arr
                # complete after its producer and after every micro-op that accumulates into it
                last = max([index[g]] + [index[u] for u in users.get(g, ()) if index[u] < pos])
                k = comm.bucket_of[i]
                ready[k] = max(ready.get(k, -1), last)
            for k, p in ready.items():
                self._bucket_ready_at.setdefault(p, []).append(k)
            return

    def _after_launch(self, idx):
        """Launch the gradient buckets that are complete once position ``idx`` has been issued."""
        for k in self._bucket_ready_at.get(idx, ()):
            self._comm.launch_bucket(k, self._comm_opt, self.stream)

    # ------------------------------------------------------------------ memory state
    def _reset_state(self):
        self.arr = {}                 # node -> device NDArray (resident)
        self.host = {}                # node -> pinned host NDArray holding a valid copy
        self.pending = []             # (event, NDArray) device arrays waiting for their D2H copy
        self.swapin_event = {}        # node -> event of an in-flight H2D copy
        self.lru = OrderedDict()      # lazy-evict cache: node -> True (MRU last)
        self._prefetch_queue = []
        self.locked = {}              # node -> lock count (an input of the running node and of a nested rebuild)
        self._side_used = set()       # copy streams this step has put work on
        self.stats = dict(swap_out_bytes=0, swap_in_bytes=0, recomputed_nodes=0, evictions=0,
                          peak_bytes=0, prefetch_hits=0, on_demand_swapins=0)

    def _reap(self, block=False):
        """Release device arrays whose D2H copy has completed."""
        keep = []
        for ev, a in self.pending:
            if block:
                ev.sync()
            if block or ev.query():
                a._release()
            else:
                keep.append((ev, a))
        self.pending = keep

    def _evict_one(self):
        """LRU eviction for lazy-evict policies: drop the least recently used
        unlocked cache entry whose host copy is complete."""
        for n in list(self.lru.keys()):
            if n in self.locked or n not in self.arr:
                continue
            a = self.arr[n]
            a.gpu2cpu_event.sync()
            del self.arr[n]
            del self.lru[n]
            a._release()
            self.stats["evictions"] += 1
            return True
        return False

    def _alloc(self, node):
        direct = self._direct.get(node)
        if direct is not None:
            return direct
        shape = self.node_to_shape_map[node]
        cl = self.node_layout.get(node)
        self._reap(False)
        while True:
            try:
                a = ndarray.empty(shape, self.ctx, channels_last=cl,
                                  long_lived=self.last_use.get(node, 0) >= len(self.topo_order))
                break
            except OutOfHBMBudget:
                if self.pending:
                    self._reap(True)
                    continue
                if self._evict_one():
                    continue
                if self._emergency_free(node):
                    continue
                if self._compact(nbytes(shape)):
                    continue
                raise
        return a

    def _compact(self, need):
        """Defragment the pool when the bytes exist but no single hole is large
        enough: drain the streams, pack live blocks, re-bind the arrays."""
        pool = ndarray.get_pool(self.ctx)
        if pool is None or getattr(self, "_no_spill", False):
            return False
        st = pool.stats()
        if st["free"] < need + 256 or st["largest_free"] >= need:
            return False
        for s in self.streams:
            s.sync()
        self._reap(True)
        # every live block has to be one this executor can re-bind: results still held by the caller,
        # another executor's arrays or blocks awaiting a planned free would keep a stale address
        mine = {a._block for a in self.arr.values()
                if isinstance(a, ndarray.NDArray) and a._pool is pool and a._block is not None}
        if pool.live_blocks() - mine:
            return False
        moves = pool.compact(stream=self.stream)
        if not moves:
            return False
        for a in self.arr.values():
            if isinstance(a, ndarray.NDArray) and a._pool is pool and a._block in moves:
                a._rebind(moves[a._block])
        self.stream.sync()          # the moved bytes have landed before anything is launched on them
        self.stats["compactions"] = self.stats.get("compactions", 0) + 1
        return True

    spill_on_pressure = False     # planned executors spill an idle activation instead of failing

    def _emergency_free(self, node):
        """Last resort when the plan fits in bytes but not in contiguous blocks
        (fragmentation) or a prefetch arrived early: spill the resident managed
        activation whose next use is farthest away.  It comes back on demand."""
        if not self.spill_on_pressure or getattr(self, "_no_spill", False):
            return False
        cur = self._cursor
        best, best_next = None, -1
        for t in self.arr:
            if t in self.locked or t not in self._managed_set or t in self.swapin_event:
                continue
            nxt = min((self.index[u] for u in self.users[t] if self.index[u] >= cur), default=None)
            if nxt is None or nxt == cur:
                continue
            if nxt > best_next:
                best, best_next = t, nxt
        if best is None:
            return self._cancel_prefetch()
        if best not in self.host:
            self._swap_out(best)
        a = self.arr[best]
        a.gpu2cpu_event.sync()
        self._release(best)
        self._reap(True)
        self.stats["evictions"] += 1
        return True

    def _cancel_prefetch(self):
        """Give back the prefetched tensor whose use is farthest away: its host copy
        stays valid, so it returns on demand (or by a later trigger)."""
        cur = self._cursor
        best, best_next = None, -1
        for t, ev in self.swapin_event.items():
            if t in self.locked or t not in self.arr:
                continue
            nxt = min((self.index[u] for u in self.users[t] if self.index[u] >= cur), default=None)
            if nxt is None or nxt == cur:
                continue
            if nxt > best_next:
                best, best_next = t, nxt
        if best is None:
            return False
        self.swapin_event[best].sync()            # the copy must not land in a freed block
        self._release(best)
        self.stats["evictions"] += 1
        return True

    def _lock(self, node):
        self.locked[node] = self.locked.get(node, 0) + 1

    def _unlock(self, node):
        c = self.locked.get(node, 0) - 1
        if c <= 0:
            self.locked.pop(node, None)
        else:
            self.locked[node] = c

    def _host_buffer(self, node):
        h = self.host_bufs.get(node)
        if h is None:
            need = 4 * ndarray._numel(self.node_to_shape_map[node])
            if self.host_bytes + need > self.host_budget_bytes:
                raise ndarray.OutOfHostSwapSpace(
                    "host swap space is not enough! need %.1f MB more on top of %.1f MB pinned, budget %.1f MB" % (
                        need / 2**20, self.host_bytes / 2**20, self.host_budget_bytes / 2**20))
            self.host_bytes += need
            h = self.host_bufs[node] = ndarray.empty(self.node_to_shape_map[node], ndarray.cpu(0),
                                                     pinned=self.on_device)
        return h

    def _raw_copy(self, dst, src, stream):
        """Byte copy of a dense array between device and pinned host (same element order)."""
        if self.on_device:
            # both sides are dense with the same logical shape; physical order may differ (channels-last on
            # the device, row-major on the host), so the copy is one run of bytes between the two storages.
            # It is an entry of the kernel library (cudaMemcpyAsync) so that a recorded step replays it.
            dev = src if src.is_cuda else dst
            nbytes = 4 * dev.t.numel()
            G.memcpy_async(dst.t.data_ptr(), src.t.data_ptr(), nbytes, stream)
        else:
            dst.t.reshape(-1)[...] = src.t.reshape(-1)

    def _swap_out(self, node):
        a = self.arr[node]
        h = self._host_buffer(node)
        ev = Event(self.ctx)
        ev.record(self.stream)                       # data is complete at this point of compute
        self.d2h_stream.wait_event(ev)
        mark = self._device_mark(self.d2h_stream) if self.trace is not None else None
        self._raw_copy(h, a, self.d2h_stream)
        self._side_used.add(self.d2h_stream)
        a.gpu2cpu_event.record(self.d2h_stream)
        self.host[node] = h
        self.stats["swap_out_bytes"] += a.nbytes
        self._log("swap_out", node)
        self._device_span("swap_out", node, mark, self.d2h_stream)

    def _swap_in(self, node, prefetch=False):
        if node in self.arr or node in self.swapin_event:
            return
        a = self._alloc(node)
        h = self.host[node]
        ev = Event(self.ctx)
        ev.record(self.stream)                       # the block's previous owner is done here
        self.h2d_stream.wait_event(ev)
        mark = self._device_mark(self.h2d_stream) if self.trace is not None else None
        self._raw_copy(a, h, self.h2d_stream)
        self._side_used.add(self.h2d_stream)
        a.cpu2gpu_event.record(self.h2d_stream)
        self.arr[node] = a
        self.swapin_event[node] = a.cpu2gpu_event
        self.stats["swap_in_bytes"] += a.nbytes
        self.stats["prefetch_hits" if prefetch else "on_demand_swapins"] += 1
        self._log("swap_in", node)
        self._device_span("swap_in", node, mark, self.h2d_stream)

    def _release(self, node, final=False):
        if node in self._direct:                 # lives in the communicator's array, not in the pool
            self.arr.pop(node, None)
            return
        a = self.arr.pop(node, None)
        self.lru.pop(node, None)
        self.swapin_event.pop(node, None)
        if a is None:
            return
        if node in self.host and a.gpu2cpu_event.recorded and not a.gpu2cpu_event.query():
            self.pending.append((a.gpu2cpu_event, a))     # D2H still reading it
        else:
            a._release()
        if final:
            self.host.pop(node, None)

    # ------------------------------------------------------------------ execution helpers
    def _value(self, node):
        return self.arr[node]

    def _launch(self, node, out):
        ins = [self.arr[i] for i in node.inputs]
        for i in node.inputs:
            ev = self.swapin_event.pop(i, None)
            if ev is not None:
                self.stream.wait_event(ev)
        tracing = self.trace is not None
        t0 = time.perf_counter() if tracing else 0
        dev = self._device_mark(self.stream) if tracing else None
        if self.on_device:
            if tracing:
                from ..utils.trace import nvtx_range
                with nvtx_range("%s:%s" % (node.op.name, node.desc)):
                    node.op.compute(node, ins, out, False, self.stream)
            else:
                node.op.compute(node, ins, out, False, self.stream)
        else:
            node.op.compute(node, [a.numpy_view() if isinstance(a, ndarray.NDArray) else a for a in ins],
                            out.numpy_view() if out is not None else None, True, self.stream)
        if tracing:
            self.trace.append(("op", node.desc, node.op.name, t0, time.perf_counter()))
            self._device_span("op", node, dev, self.stream)

    def _log(self, kind, node):
        if self.trace is not None:
            self.trace.append((kind, node.desc, node.op.name, time.perf_counter(), time.perf_counter()))

    # -- device timeline: a timing event before and after every action on the stream it runs on ----------
    def _device_mark(self, stream):
        if not self.on_device:
            return None
        ev = Event(self.ctx, timing=True)
        ev.record(stream)
        return ev

    def _device_span(self, kind, node, start, stream):
        """Close a span opened by ``_device_mark``: the pair of events gives the action's time ON THE DEVICE
        (kernel or copy duration and its position relative to the other streams), which the host clock of the
        launch cannot.  Resolved by ``device_trace`` after the step."""
        if start is None:
            return
        end = Event(self.ctx, timing=True)
        end.record(stream)
        self.__dict__.setdefault("_device_spans", []).append((kind, node.desc, node.op.name, stream.id, start, end))

    def device_trace(self):
        """Device-time records of the traced steps: ``(kind, node, op, stream id, start ms, end ms)`` relative
        to the first recorded event.  Synchronises."""
        spans = self.__dict__.get("_device_spans", [])
        if not spans:
            return []
        for s in self.streams:
            s.sync()
        origin = spans[0][4]
        out = []
        for kind, desc, op, sid, a, b in spans:
            out.append((kind, desc, op, sid, origin.elapsed_ms(a), origin.elapsed_ms(b)))
        return out

    def _ensure(self, node, temps):
        """Make ``node`` resident: cache hit, swap-in, or recompute from its inputs."""
        if node in self.arr:
            if node in self.lru:
                self.lru.move_to_end(node)
            return
        if node in self.host:
            self._swap_in(node)
            return
        assert node.inputs, "tensor %s was released and cannot be rebuilt" % node.desc
        for i in node.inputs:
            self._ensure(i, temps)
            self._lock(i)
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
        for i in node.inputs:
            self._unlock(i)
        self.stats["recomputed_nodes"] += 1
        temps.append(node)
        self._log("recompute", node)

    # ------------------------------------------------------------------ run
    def memory_plan(self, feed_shapes):
        self.node_to_arr_map = {}
        if self.__dict__.get("_step_graph") is not None or self.__dict__.get("_graph_steps_seen"):
            # a new feed shape: the captured graph / recorded tape holds the old shapes and addresses
            if self.on_device:
                self.stream.sync()
            self._step_graph, self._graph_steps_seen, self._graph_ok = None, 0, None
            self._graph_keep, self._graph_feeds = [], None
            if hasattr(self, "_close_region"):
                self._close_region()
        had = bool(getattr(self, "host_bufs", None))
        self.host_bufs = {}
        self.host_bytes = 0
        if had and self.on_device:
            # page-locked buffers of the previous feed shape go back to the OS, not to torch's host cache:
            # a batch sweep would otherwise pin the sum over its trials
            import torch
            getattr(torch._C, "_host_emptyCache", lambda: None)()
        self.host_budget_bytes = ndarray.host_swap_budget_bytes()
        self.plan()

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        self._begin_step()
        node_to_val = self._ingest(feed_dict)
        feed_shapes = {n: tuple(v.shape) for n, v in node_to_val.items()}
        if feed_shapes != self.feed_shapes:
            self.feed_shapes = feed_shapes
            self.infer_shape(feed_shapes)
            self.memory_plan(feed_shapes)
        if self.use_graph and self._graph_eligible():
            return self._run_graphed(node_to_val, convert_to_numpy_ret_vals)
        return self._run_with_values(node_to_val, convert_to_numpy_ret_vals)

    def _run_with_values(self, node_to_val, convert_to_numpy_ret_vals):
        self._reset_state()
        for n, v in node_to_val.items():
            self.arr[n] = v
        pool = ndarray.get_pool(self.ctx)
        if pool is not None:
            pool.reset_peak()
        self._execute()
        self.stream.sync()
        self._reap(True)
        if pool is not None:
            self.stats["peak_bytes"] = pool.stats()["peak"]
        outs = [self.arr.get(n) for n in self.eval_node_list]
        if convert_to_numpy_ret_vals:
            outs = [o.asnumpy() if isinstance(o, ndarray.NDArray) else o for o in outs]
        # drop everything that is not a result, a feed or a parameter
        for n in list(self.arr.keys()):
            if n not in self.eval_node_list and not isinstance(n.op, PlaceholderOp) and n not in node_to_val:
                self._release(n, final=True)
        self._reap(True)
        return outs

    # ------------------------------------------------------------------ CUDA-graph replay
    def _graph_eligible(self):
        """A step can be replayed from a captured graph when its launch list is fixed: no swaps (their
        event queries and host-side frees cannot be captured), no lazily evicted cache, no trace, no
        collective (its epoch counter is a kernel argument), no op whose kernel arguments change from
        step to step (the step index of dropout and Adam's bias-correction powers live on the device for this reason)."""
        ok = self.__dict__.get("_graph_ok")
        if ok is None:
            ok = self.trace is None and not self.lazy_evict
            ok = ok and not any(c == SWAP for c in getattr(self, "cls", {}).values())
            for n in self.topo_order:
                if n.op.name == "Optimizer":
                    opt = n.attrs.get("optimizer")
                    if opt is None or (getattr(opt, "communicator", None) is not None and self.replay_mode != "tape"):
                        ok = False
            self._graph_ok = bool(ok) and self._replay_backend_ok()
        return self._graph_ok

    def _replay_backend_ok(self):
        if self.replay_mode != "tape":
            return True
        from ..runtime import tape
        return tape.available()

    def _record_tape(self):
        """Run the step once the ordinary way while every native call is recorded; returns the replayable step."""
        from ..runtime import tape
        with tape.recording() as rec:
            self._execute()
        if rec.invalid is not None:
            raise RuntimeError("step cannot be replayed natively: " + rec.invalid)
        return _TapedStep(tape.Tape(rec), self), rec.kernels

    def _run_graphed(self, node_to_val, convert):
        """Two eager steps (they size every library scratch buffer, tensor map and side buffer and let
        the pool settle), then one capture, then replays.  Feeds are copied into fixed device arrays
        first, because staged feeds alternate between two buffers."""
        from ..runtime import cudagraph
        if self._step_graph is None and self._graph_steps_seen < 2:
            self._graph_steps_seen += 1
            return self._run_eager_step(node_to_val, convert)
        if self._step_graph is None:
            self._graph_feeds = {n: ndarray.empty(v.shape, self.ctx, use_pool=False,
                                                  channels_last=v.is_channels_last() if len(v.shape) == 4 else None)
                                 for n, v in node_to_val.items() if isinstance(v, ndarray.NDArray)}
        fixed = dict(node_to_val)
        for n, buf in self._graph_feeds.items():
            G.copy(node_to_val[n], buf, self.stream)
            fixed[n] = buf
        if self._step_graph is None:
            self._reset_state()
            for n, v in fixed.items():
                self.arr[n] = v
            self.stream.sync()
            from ..utils import launch_counter
            before = launch_counter.count()
            try:
                if self.replay_mode == "tape":
                    self._step_graph, self._graph_launches = self._record_tape()
                    self._just_recorded = True      # the recording ran the step: nothing to launch this time
                else:
                    self._step_graph = cudagraph.capture(self.stream, self._execute)
                    self._graph_launches = launch_counter.count() - before      # kernels one replay launches
            except Exception as e:
                # something in this step cannot be captured (an allocation path that synchronises, a
                # library buffer that had to grow): stay on the eager path for good
                self.replay_failure = "%s: %s" % (type(e).__name__, e)
                self.use_graph = False
                self._step_graph = None
                return self._run_with_values(node_to_val, convert)
            self._just_captured = True          # this step's Python side (optimizer bookkeeping) ran during capture
            self._graph_outs = [self.arr.get(n) for n in self.eval_node_list]
            # The captured launches keep the addresses of every intermediate of the step.  Arrays that are
            # still resident at the end of the capture stay reserved for as long as the graph exists; blocks
            # that the step itself freed and re-used belong to the pool again, which is safe only while this
            # executor is the pool's sole user during a replay (a second executor on the same pool must not
            # run between a replay's launch and its completion).
            self._graph_keep = [a for n, a in self.arr.items()
                                if n not in self.eval_node_list and not isinstance(n.op, PlaceholderOp)
                                and n not in fixed]
            for n in list(self.arr.keys()):
                if n not in self.eval_node_list and not isinstance(n.op, PlaceholderOp) and n not in fixed:
                    self.arr.pop(n)
                    self.host.pop(n, None)
        captured_now = self.__dict__.pop("_just_captured", False)
        if not self.__dict__.pop("_just_recorded", False):
            self._step_graph.launch(self.stream)
            from ..utils import launch_counter
            launch_counter.add(self.__dict__.get("_graph_launches", 0))
        self.stream.sync()
        if not captured_now:
            # the optimizer's Python side did not run: keep its host-side step bookkeeping (checkpoints) in step.
            # Hyper-parameters are kernel arguments of the captured launch: a changed learning rate needs a new capture.
            for n in self.topo_order:
                if n.op.name == "Optimizer":
                    opt = n.attrs.get("optimizer") or n.attrs["orig"].attrs["optimizer"]
                    opt.step_count += 1
                    opt._begin_step()
        outs = self._graph_outs
        if convert:
            outs = [o.asnumpy() if isinstance(o, ndarray.NDArray) else o for o in outs]
        return outs

    def replay_host_us(self):
        """Host time of the last native replay in microseconds and its number of actions (``use_graph="tape"``)."""
        g = self._step_graph
        if isinstance(g, _TapedStep):
            return g.tape.last_host_ns / 1e3, len(g.tape)
        return None

    def _run_eager_step(self, node_to_val, convert):
        saved, self.use_graph = self.use_graph, False
        try:
            return self._run_with_values(node_to_val, convert)
        finally:
            self.use_graph = saved

    def _execute(self):
        self._advance_device_step()
        if self._comm is not None:
            self._comm.open_step()
        order = self.topo_order
        self._cursor = 0
        for idx, node in enumerate(order):
            self._cursor = idx
            if node in self.arr:
                continue
            if isinstance(node.op, PlaceholderOp):
                self.arr[node] = self._placeholder_value(node)
                continue
            # prefetches that found no room stay queued and are retried before every later node
            self._prefetch_queue.extend(self.prefetch_at.get(idx, ()))
            if self._prefetch_queue:
                self._reap(False)
                waiting = []
                for t in self._prefetch_queue:
                    if t not in self.host or t in self.arr:
                        continue
                    if waiting or not self._room_for_prefetch(t, idx):
                        waiting.append(t)          # keep the order: earlier uses first
                        continue
                    self._no_spill = True
                    try:
                        self._swap_in(t, prefetch=True)
                    except OutOfHBMBudget:
                        waiting.append(t)
                    finally:
                        self._no_spill = False
                self._prefetch_queue = waiting
            temps = []
            for i in node.inputs:
                self._ensure(i, temps)
                self._lock(i)
            shape = self.node_to_shape_map[node]
            out = self._alloc(node) if shape is not None else None
            if out is not None:
                self.arr[node] = out
            self._launch(node, out)
            if self._bucket_ready_at:
                self._after_launch(idx)
            for i in node.inputs:
                self._unlock(i)
            self._after_node(idx, node, temps)

    def _room_for_prefetch(self, t, idx):
        """Prefetch only when the pool keeps head-room for what the schedule
        allocates before ``t`` is used (the largest output on the way)."""
        pool = ndarray.get_pool(self.ctx)
        if pool is None:
            return True
        use = self.first_bwd_use.get(t) or idx
        reserve = max((self.tensor_bytes(n) for n in self.topo_order[idx:use + 1]), default=0)
        st = pool.stats()
        need = self.tensor_bytes(t)
        if st["largest_free"] < need:
            return False
        plan_budget = self.planning_budget()
        if plan_budget is not None:          # same rule as the planner's simulator
            return st["used"] + need + 2 * reserve <= plan_budget
        return st["free"] >= need + reserve

    def planning_budget(self):
        """Bytes the plan was made for (None: no plan-level budget)."""
        return None

    def _after_node(self, idx, node, temps):
        # forward: offload / drop policy-managed tensors at their last forward use
        for t in self.fwd_release_at.get(idx, ()):
            if t not in self.arr:
                continue
            c = self.cls[t]
            if c == SWAP:
                if t not in self.host:
                    self._swap_out(t)
                if self.lazy_evict:
                    self.lru[t] = True
                    self.lru.move_to_end(t)
                else:
                    self._release(t)
            elif c == DROP:
                self._release(t)
        # rematerialised intermediates
        for t in temps:
            if t in self.arr and t not in node.inputs:
                if self.recompute_mode == "memory" or self.last_use[t] <= idx:
                    self._release(t)
        if self.recompute_mode == "memory" and idx >= self.first_bwd_index:
            for t in node.inputs:
                if self.cls.get(t, KEEP) == DROP and self.last_use[t] > idx and t in self.arr:
                    self._release(t)
        # final releases
        for t in self.release_at.get(idx, ()):
            if t in self.arr and not isinstance(t.op, PlaceholderOp) and t not in self.feed_shapes:
                self._release(t, final=True)
        if node not in self.users or (not self.users[node] and node not in self.eval_node_list):
            if node in self.arr:
                self._release(node, final=True)

    # ------------------------------------------------------------------ cost model
    from ..profiler import FLOPS_PER_MS as TF32_FLOP_PER_MS, HBM_BYTES_PER_MS, LAUNCH_MS

    def profile_ops(self):
        """Per-node time in ms.  Static roofline estimate (the reference's
        ``Op.profile(is_static=True)`` role, ``gpu_ops/Conv2d.py:80-90``); a
        measured table can be supplied through ``self.measured_op_ms``."""
        measured = getattr(self, "measured_op_ms", None)
        est = {}
        for n in self.topo_order:
            if isinstance(n.op, PlaceholderOp) or n in self.feed_shapes:
                continue
            if measured and n in measured:
                est[n] = measured[n]
                continue
            out = self.node_to_shape_map.get(n)
            # a micro-op states the shapes its operator really sees (batch pieces of whole inputs)
            ins = n.attrs.get("op_in_shapes") or [self.node_to_shape_map.get(i) for i in n.inputs]
            try:
                fl = float(n.op.flops(n, ins, out))
            except Exception:
                fl = 0.0
            by = sum(nbytes(s) for s in ins if s is not None) + (nbytes(out) if out is not None else 0)
            est[n] = max(fl / self.TF32_FLOP_PER_MS, by / self.HBM_BYTES_PER_MS) + self.LAUNCH_MS
        return est

    def measure_ops(self, feed_dict, repeats=2):
        """Event-timed per-node device time (ms) from a keep-everything run; the
        role of the reference's ``Op.profile(is_static=False)``."""
        assert self.on_device, "measured profiling needs a CUDA context"
        import torch
        base = Executor(self.eval_node_list, ctx=self.ctx)
        base.run(feed_dict)
        vals = dict(base._last_vals)
        table = {}
        for n in base.topo_order:
            if isinstance(n.op, PlaceholderOp) or n in feed_dict or n.op.name == "Optimizer":
                continue
            ins = [vals[i] for i in n.inputs]
            out = base.node_to_arr_map.get(n)
            best = None
            for _ in range(repeats):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(base.stream.torch_stream)
                n.op.compute(n, ins, out, False, base.stream)
                b.record(base.stream.torch_stream)
                b.synchronize()
                ms = a.elapsed_time(b)
                best = ms if best is None else min(best, ms)
            table[n] = best
        self.measured_op_ms = table
        return table

    def tensor_bytes(self, node):
        shp = self.node_to_shape_map.get(node)
        return nbytes(shp) if shp is not None else 0

    def show_tensor_in_gpu(self):
        return [(n.desc, self.tensor_bytes(n)) for n in self.arr]
