"""Baseline executors: ``Executor``, ``StreamExecutor``, ``MultiStreamExecutor``.

Capability parity: ``gpu_ops/executor.py:21-158`` (allocate every node output
once per feed shape and keep it), ``StreamExecutor.py:68-214`` (user-supplied
stream) and ``MultiStreamExecutor.py:68-252`` (feeds copied on an H2D stream
with one event per feed node).

B200-first differences: feeds are staged through cached pinned buffers and one
layout kernel instead of a fresh synchronous allocation+copy per run; the
compute stream waits on events instead of the host; and the steady-state step
can be captured once per feed shape into a CUDA graph and replayed
(``use_graph=True``), which removes the per-node host work the reference pays on
every iteration.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ndarray
from ..graph import schedule_order
from ..stream import create_stream_handle, Event
from ..ops.misc import PlaceholderOp


def _shape_of(v):
    return tuple(v.shape)


class FeedStager(object):
    """Host -> device feed path: a pinned staging buffer and a device buffer per
    fed node, reused across runs while the shape stays the same.  A feed that is
    already a pinned host ``NDArray`` (``ndarray.empty(shape, ndarray.cpu(0),
    pinned=True)``) is copied to the device straight from the caller's buffer."""

    def __init__(self, ctx):
        self.ctx = ctx
        self.slots = {}
        self.staged = {}          # node -> {id(value): (value object, device array, event)} copied ahead of its step
                                  # (at most two per node: one per device buffer)
        self._flip = {}           # node -> which of the two device buffers the next copy uses

    def stage(self, node, value, copy_stream, channels_last=None):
        """Copy the NEXT step's feed while the current step computes: the copy goes to the other of
        two device buffers on ``copy_stream`` and leaves an event; ``put`` with the same value
        object later only waits for that event.  The caller must not modify ``value`` in between."""
        if not (ndarray.is_gpu_ctx(self.ctx) and self.ctx.device_type == 2):
            return
        if isinstance(value, ndarray.NDArray) and value.ctx.device_type == self.ctx.device_type:
            return
        self._flip[node] = 1 - self._flip.get(node, 0)
        dev = self._copy(("ahead", node, self._flip[node]), value, copy_stream, channels_last)
        ev = Event(self.ctx)
        ev.record(copy_stream)
        self.staged.setdefault(node, {})[id(value)] = (value, dev, ev)

    def put(self, node, value, stream, channels_last=None):
        ahead = self.staged.get(node, {}).pop(id(value), None)
        if ahead is not None and ahead[0] is value:
            stream.wait_event(ahead[2])
            return ahead[1]
        if isinstance(value, ndarray.NDArray) and (
                value.ctx == self.ctx or value.ctx.device_type == self.ctx.device_type):
            return value
        return self._copy(node, value, stream, channels_last)

    def _copy(self, node, value, stream, channels_last=None):
        user_pinned = None
        if isinstance(value, ndarray.NDArray):
            if value.ctx == self.ctx or value.ctx.device_type == self.ctx.device_type:
                return value
            t = getattr(value, "t", None)
            if (ndarray.is_gpu_ctx(self.ctx) and self.ctx.device_type == 2 and t is not None and not t.is_cuda
                    and t.is_pinned() and t.is_contiguous() and t.dtype == torch.float32):
                user_pinned = t.reshape(-1)       # the caller's own pinned buffer: no staging copy
            else:
                value = value.asnumpy()
        if user_pinned is None:
            value = np.asarray(value)
            if not ndarray.is_gpu_ctx(self.ctx) or self.ctx.device_type == 3:
                return ndarray.array(value, self.ctx, use_pool=False)
        shape = tuple(value.shape)
        slot = self.slots.get(node)
        if slot is None or slot[0] != shape or slot[2].is_channels_last() != bool(
                len(shape) == 4 and (channels_last is None or channels_last)):
            n = int(np.prod(shape)) if shape else 1
            pinned = None
            dev = ndarray.empty(shape, self.ctx, use_pool=False, channels_last=channels_last)
            raw = None
            if dev.is_channels_last() and not dev.t.is_contiguous():   # land row-major bytes first
                raw = torch.empty(max(n, 1), dtype=torch.float32, device=self.ctx.torch_device)
            slot = [shape, pinned, dev, raw]
            self.slots[node] = slot
        _, pinned, dev, raw = slot
        n = int(np.prod(shape)) if shape else 1
        if user_pinned is not None:
            src = user_pinned
        else:
            if pinned is None:
                pinned = slot[1] = torch.empty(max(n, 1), dtype=torch.float32, pin_memory=True)
            pinned[:n].numpy()[...] = value.reshape(-1)
            src = pinned
        with torch.cuda.stream(stream.torch_stream):
            if raw is None:
                dev.t.view(-1)[:n].copy_(src[:n], non_blocking=True) if dev.t.is_contiguous() \
                    else dev.t.copy_(src[:n].view(shape), non_blocking=True)
            else:
                raw[:n].copy_(src[:n], non_blocking=True)
                from ..ops import _gpu as G
                rm = []
                acc = 1
                for d in reversed(shape):
                    rm.insert(0, acc)
                    acc *= d
                G.copy_raw(raw.data_ptr(), rm, dev.ptr, dev.strides, shape, stream)
        return dev

    def bytes_per_step(self, feed_dict):
        return sum(int(np.prod(v.shape)) * 4 for v in feed_dict.values()
                   if not (isinstance(v, ndarray.NDArray) and ndarray.is_gpu_ctx(v.ctx)))


class Executor(object):
    """Executor computes values for given set of nodes in a computation graph."""

    def __init__(self, eval_node_list, ctx=None, stream=None, policy=None, use_graph=False):
        self.eval_node_list = list(eval_node_list)
        self.ctx = ctx
        self.policy = policy
        self.topo_order = schedule_order(self.eval_node_list)
        self.use_numpy = ctx is None
        self.on_device = ndarray.is_gpu_ctx(ctx) and ctx.device_type == 2
        self.stream = stream
        if self.stream is None and ctx is not None:
            self.stream = create_stream_handle(ctx)
        self.node_to_shape_map = None
        self.node_to_arr_map = None
        self.feed_shapes = None
        self.stager = FeedStager(ctx) if ctx is not None else None
        self.use_graph = bool(use_graph) and self.on_device
        self._graph = None
        self._graph_feed_arrs = None
        # a CPU-context executor can replay its step from the native tape too (use_graph="tape"): every operator
        # of the step must have a host kernel (csrc/runtime/cpu_ops.cc), else it keeps its Python loop
        self.cpu_tape = use_graph == "tape" and ctx is not None and ctx.device_type == 1
        self._cpu_tape, self._cpu_tape_state = None, "warm"

    # -- shapes ---------------------------------------------------------------
    def infer_shape(self, feed_shapes):
        self.node_to_shape_map = {}
        for node in self.topo_order:
            if node in feed_shapes:
                shp = tuple(feed_shapes[node])
            elif isinstance(node.op, PlaceholderOp):
                shp = node.op.infer_shape(node, [])
            else:
                shp = node.op.infer_shape(node, [self.node_to_shape_map[i] for i in node.inputs])
            if shp is not None:
                shp = tuple(int(s) for s in shp)
            self.node_to_shape_map[node] = shp
            node.inferred_shape = shp
        from .. import layout
        self.node_layout = layout.resolve(self.topo_order, self.node_to_shape_map)

    def memory_plan(self, feed_shapes):
        """One array per computed node, kept until the feed shapes change."""
        self.node_to_arr_map = {}
        for node, shape in self.node_to_shape_map.items():
            if node in feed_shapes or isinstance(node.op, PlaceholderOp) or shape is None:
                continue
            self.node_to_arr_map[node] = ndarray.empty(shape, ctx=self.ctx,
                                                       channels_last=self.node_layout.get(node))

    # -- feeds ---------------------------------------------------------------
    def _ingest(self, feed_dict):
        vals = {}
        for node, value in feed_dict.items():
            if isinstance(value, ndarray.ND_Sparse_Array):
                vals[node] = value
            elif self.use_numpy:
                if isinstance(value, ndarray.NDArray):
                    value = value.asnumpy()
                assert isinstance(value, np.ndarray), "feed_dict value type not supported"
                vals[node] = value
            else:
                assert isinstance(value, (np.ndarray, ndarray.NDArray)), "feed_dict value type not supported"
                vals[node] = self.stager.put(node, value, self.stream, self._feed_layout(node, value))
        return vals

    def prefetch_feeds(self, feed_dict):
        """Start the host -> device copies of the NEXT step's feeds now, on the copy stream, so that
        they overlap the step that is about to run: ``ex.prefetch_feeds(next); ex.run(cur)``.  The
        next ``run`` must be given the same value objects, unmodified.  No-op off the GPU."""
        if not self.on_device or self.stager is None:
            return
        stream = getattr(self, "h2d_stream", None)
        if stream is None:
            stream = self.__dict__.get("_prefetch_stream")
            if stream is None:
                stream = self._prefetch_stream = create_stream_handle(self.ctx)
        for node, value in feed_dict.items():
            if isinstance(value, ndarray.ND_Sparse_Array):
                continue
            self.stager.stage(node, value, stream, self._feed_layout(node, value))

    def _feed_layout(self, node, value):
        """Channels-last only for 4-D feeds consumed by an image operator."""
        if len(getattr(value, "shape", ())) != 4:
            return False
        cache = self.__dict__.setdefault("_feed_layout_cache", {})
        if node not in cache:
            from .. import layout
            cache[node] = any(node in u.inputs and u.op.name in layout.IMAGE_OPS for u in self.topo_order)
        return cache[node]

    def _placeholder_value(self, node):
        v = node.tensor_value
        assert v is not None, "placeholder %s values provided by feed_dict" % node.name
        if self.use_numpy:
            return v.asnumpy() if isinstance(v, ndarray.NDArray) else v
        if isinstance(v, np.ndarray):
            v = ndarray.array(v, self.ctx, use_pool=False, channels_last=self._feed_layout(node, v))
            node.tensor_value = v
        return v

    def _val(self, arr):
        """What ops receive: NumPy views on host-backed contexts, NDArrays on CUDA."""
        if self.use_numpy or self.on_device:
            return arr
        return arr.numpy_view() if isinstance(arr, ndarray.NDArray) else arr

    # -- run ---------------------------------------------------------------------
    def _begin_step(self):
        """Publish this executor's step index to the ops that draw per-step random numbers."""
        from ..ops import misc
        misc.STEP[0] = self.__dict__.get("_run_index", 0)
        misc.RUN_ID[0] += 1
        self._run_index = misc.STEP[0] + 1
        if self.on_device:
            # the same index on the device, advanced by a one-thread kernel at the start of every step
            # (see _advance_device_step), so that a step replayed from a CUDA graph still moves on
            if self.__dict__.get("_step_dev") is None:
                self._step_dev = torch.full((1,), misc.STEP[0] - 1, dtype=torch.int64,
                                            device=self.ctx.torch_device)
            misc.STEP_DEV[0] = self._step_dev.data_ptr()
        else:
            misc.STEP_DEV[0] = 0

    def _advance_device_step(self):
        if self.on_device and self.__dict__.get("_step_dev") is not None:
            from ..ops import _gpu as G
            G.step_advance(self._step_dev.data_ptr(), self.stream)

    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        from .. import graph
        native = self.ctx is not None and self.ctx.device_type == 1       # CPU context: native host kernels
        prev, graph.CPU_NATIVE[0] = graph.CPU_NATIVE[0], native
        try:
            return self._run(feed_dict, convert_to_numpy_ret_vals)
        finally:
            graph.CPU_NATIVE[0] = prev

    def _run(self, feed_dict, convert_to_numpy_ret_vals=False):
        self._begin_step()
        node_to_val = self._ingest(feed_dict)
        feed_shapes = {n: _shape_of(v) for n, v in node_to_val.items()}
        if feed_shapes != self.feed_shapes:
            self.infer_shape(feed_shapes)
            self.feed_shapes = feed_shapes
            if not self.use_numpy:
                self.memory_plan(feed_shapes)
            self._graph = None
            self._graph_warm = False
            self._cpu_tape, self._cpu_tape_state = None, "warm"

        if self.use_graph:
            self._run_graph(node_to_val)
        elif self.cpu_tape and self._cpu_tape_state != "off":
            self._run_cpu_tape(node_to_val)
        else:
            self._run_eager(node_to_val)

        if self.stream is not None:
            self.stream.sync()
        outs = [node_to_val.get(n) for n in self.eval_node_list]
        if convert_to_numpy_ret_vals and not self.use_numpy:
            return [o.asnumpy() if isinstance(o, ndarray.NDArray) else o for o in outs]
        return outs

    def _run_eager(self, node_to_val):
        self._advance_device_step()
        host_like = not self.on_device
        for node in self.topo_order:
            if node in node_to_val:
                continue
            if isinstance(node.op, PlaceholderOp):
                node_to_val[node] = self._placeholder_value(node)
                continue
            ins = [node_to_val[i] for i in node.inputs]
            if self.use_numpy:
                out = np.empty(self.node_to_shape_map[node], dtype=np.float32) \
                    if self.node_to_shape_map[node] is not None else None
                node.op.compute(node, ins, out, True, None)
            elif host_like:
                out = self.node_to_arr_map.get(node)
                node.op.compute(node, [self._val(i) for i in ins],
                                out.numpy_view() if out is not None else None, True, self.stream)
            else:
                out = self.node_to_arr_map.get(node)
                node.op.compute(node, ins, out, False, self.stream)
            node_to_val[node] = out
        self._last_vals = node_to_val

    # -- native replay of a CPU-context step ------------------------------------------
    def _run_cpu_tape(self, node_to_val):
        """First step eager, second step recorded (it runs the ordinary way while every host-library call is
        appended to a tape), later steps one call of the C++ replay loop.  Feeds are copied into fixed host
        arrays first, because the recorded calls hold addresses."""
        from .. import graph
        from ..runtime import tape
        if self._cpu_tape_state == "warm" or not tape.available():
            self._cpu_tape_state = "record" if tape.available() else "off"
            return self._run_eager(node_to_val)
        if self._cpu_tape is None:
            self._cpu_feed_arrs = {n: ndarray.empty(_shape_of(v), self.ctx) for n, v in node_to_val.items()
                                   if not isinstance(v, ndarray.ND_Sparse_Array)}
        fixed = dict(node_to_val)
        for n, buf in self._cpu_feed_arrs.items():
            v = node_to_val[n]
            buf.numpy_view()[...] = v.numpy_view() if isinstance(v, ndarray.NDArray) else v
            fixed[n] = buf
        if self._cpu_tape is None:
            before = graph.NUMPY_FALLBACKS[0]
            with tape.recording() as rec:
                self._run_eager(fixed)
            if rec.invalid is None and graph.NUMPY_FALLBACKS[0] != before:
                rec.invalid = "%d operators of the step have no host kernel" % (graph.NUMPY_FALLBACKS[0] - before)
            if rec.invalid is not None or not rec.fns:
                self.replay_failure = rec.invalid or "nothing was recorded"
                self._cpu_tape_state = "off"
                node_to_val.update(self._last_vals)
                return
            self._cpu_tape = tape.Tape(rec)
            self._cpu_tape_vals = self._last_vals
            node_to_val.update(self._last_vals)
            return
        self._cpu_tape.replay()
        for n in self.topo_order:            # the optimizer's Python side did not run: keep its step count in step
            if n.op.name == "Optimizer":
                opt = n.attrs["optimizer"]
                opt.step_count += 1
                opt._begin_step()
        self._last_vals = self._cpu_tape_vals
        node_to_val.update(self._cpu_tape_vals)

    # -- CUDA-graph replay ---------------------------------------------------------
    def _run_graph(self, node_to_val):
        """Capture the whole step once per feed shape and replay it afterwards.  The captured launches
        read the feeds from fixed device buffers (not from whatever buffer a feed arrived in: staged
        feeds alternate between two, and a caller may hand a different device array every step), so
        every step first copies its feeds into those buffers on the stream."""
        from ..runtime import cudagraph
        from ..ops import _gpu as G
        if self._graph is None and not getattr(self, "_graph_warm", False):
            # first step with these shapes runs eagerly: it creates the lazily allocated side
            # buffers, tensor maps and workspaces that a capture must not allocate
            self._run_eager(node_to_val)
            self._graph_warm = True
            return
        if self._graph is None:
            self._graph_feed_arrs = {
                n: ndarray.empty(v.shape, self.ctx, use_pool=False,
                                 channels_last=v.is_channels_last() if len(v.shape) == 4 else None)
                for n, v in node_to_val.items() if isinstance(v, ndarray.NDArray)}
        fixed = dict(node_to_val)
        for n, buf in self._graph_feed_arrs.items():
            G.copy(node_to_val[n], buf, self.stream)
            fixed[n] = buf
        captured_now = False
        if self._graph is None:
            self.stream.sync()
            self._graph = cudagraph.capture(self.stream, lambda: self._run_eager(dict(fixed)))
            self._graph_vals = self._last_vals
            captured_now = True              # the optimizer's host side ran during the capture
        self._graph.launch(self.stream)
        if not captured_now:
            # a replay runs no Python: keep the host-side step bookkeeping (checkpoints, Adam's powers) in step
            for n in self.topo_order:
                if n.op.name == "Optimizer":
                    opt = n.attrs["optimizer"]
                    opt.step_count += 1
                    opt._begin_step()
        self._last_vals = self._graph_vals
        node_to_val.update(self._graph_vals)


class StreamExecutor(Executor):
    """Same as :class:`Executor` with a caller-owned stream (``streams=`` may be a
    single stream or a one-element list)."""

    def __init__(self, eval_node_list, ctx=None, stream=None, streams=None, policy=None, use_graph=False):
        if stream is None and streams is not None:
            stream = streams[0] if isinstance(streams, (list, tuple)) else streams
        Executor.__init__(self, eval_node_list, ctx=ctx, stream=stream, policy=policy, use_graph=use_graph)


class MultiStreamExecutor(Executor):
    """Three streams — H2D, compute, D2H.  Each feed is copied on the H2D stream
    and followed by an event; the compute stream waits for a feed's event right
    before the first node that consumes it, so later feeds overlap with earlier
    compute."""

    def __init__(self, eval_node_list, ctx=None, streams=None, policy=None):
        Executor.__init__(self, eval_node_list, ctx=ctx, policy=policy)
        if streams is None and ctx is not None:
            streams = [create_stream_handle(ctx) for _ in range(3)]
        self.streams = streams
        if streams is not None:
            self.h2d_stream, self.stream, self.d2h_stream = streams[0], streams[1], streams[2]
        self.feed_events = {}

    def _ingest(self, feed_dict):
        if self.use_numpy:
            return Executor._ingest(self, feed_dict)
        vals = {}
        for node, value in feed_dict.items():
            vals[node] = self.stager.put(node, value, self.h2d_stream, self._feed_layout(node, value))
            ev = self.feed_events.get(node)
            if ev is None:
                ev = self.feed_events[node] = Event(self.ctx)
            ev.record(self.h2d_stream)
        return vals

    def _run_eager(self, node_to_val):
        waited = set()
        fed = set(self.feed_events) & set(node_to_val)
        host_like = not self.on_device
        for node in self.topo_order:
            if node in node_to_val:
                continue
            if isinstance(node.op, PlaceholderOp):
                node_to_val[node] = self._placeholder_value(node)
                continue
            for i in node.inputs:
                if i in fed and i not in waited:
                    self.stream.wait_event(self.feed_events[i])
                    waited.add(i)
            ins = [node_to_val[i] for i in node.inputs]
            out = self.node_to_arr_map.get(node) if not self.use_numpy else \
                np.empty(self.node_to_shape_map[node], dtype=np.float32)
            if self.use_numpy:
                node.op.compute(node, ins, out, True, None)
            elif host_like:
                node.op.compute(node, [self._val(i) for i in ins],
                                out.numpy_view() if out is not None else None, True, self.stream)
            else:
                node.op.compute(node, ins, out, False, self.stream)
            node_to_val[node] = out
        self._last_vals = node_to_val
