"""Lowering of a differentiated graph to micro-ops over batch pieces (TSplit).

The reference's runtime hooks exist so that an operator can run as k micro-ops over
micro-tensors: ``DLArraySliceForMicroTensor`` (``src/common/c_runtime_api.cc:212-271``),
``NDArray.split_tensor / slice_for_micro_tensor`` (``python/athena/ndarray.py:121-145,
372-409``) and ``SplitOp`` (``python/athena/gpu_ops/Split.py:7-69``); the planner
that used them is not in its tree.  Here the split is a graph transformation done
once per feed shape, after autodiff and before planning:

* a batch-separable operator (convolution, its data gradient, pooling, element-wise
  ops, reshapes that keep the batch, ...) becomes k independent micro-ops; piece j
  reads piece j of every batch-sized input and produces piece j of the output as a
  tensor of its own, so the memory planner decides keep / swap / recompute per
  micro-tensor and the whole-batch tensor never has to exist;
* a batch reduction (filter gradient, bias gradient) becomes k micro-ops that
  accumulate into one output;
* batch norm needs whole-batch statistics: k statistics micro-ops fill a partial-sum
  buffer, one finalise micro-op produces mean / inverse deviation (and the running
  statistics, once), then k normalise micro-ops run; its backward is split the same
  way (sums of dy and dy*xhat, finalise, k dx micro-ops);
* everything else runs whole; pieces that feed a whole operator are merged first,
  whole tensors that feed a split operator are read through batch views.

Micro-ops are emitted piece-major between the whole-batch barriers (a piece runs
through a chain of operators before the next piece starts), alternating the piece
order from one barrier to the next so that the pieces produced last are consumed
first.
"""
from __future__ import annotations

import numpy as np

from .. import ndarray
from ..graph import Node, Op
from ..ops.misc import PlaceholderOp
from ..ops import _gpu as G

#: operators whose batch pieces are independent (every batch-sized input is cut alike)
SEPARABLE = {
    "Conv2d", "Conv2dGradData", "Relu", "ReluGradient", "Add", "AddRelu", "ReluOutGradient", "Mul", "Div",
    "AddConst", "MulConst", "DivConst", "Opposite", "Sqrt", "Rsqrt", "Sigmoid", "Tanh", "Where",
    "MaxPool2d", "AvgPool2d", "MaxPool2dGradient", "AvgPool2dGradient", "Reshape", "ReshapeGradient",
    "AddBroadcast", "Conv2dBroadcastTo", "Dropout", "DropoutGradient", "BatchNormGradData",
}
#: operators that sum over the batch: k micro-ops accumulate into one output
REDUCING = {"Conv2dGradFilter", "Conv2dReduceSum"}
BN_FWD = {"BatchNorm", "BatchNormRelu"}
BN_BWD = {"BatchNormGradient", "BatchNormReluGradient"}


def _nbytes(shape):
    n = 4
    for s in shape:
        n *= int(s)
    return n


def _piece(a, lo, hi):
    """Batch rows [lo, hi) of a NumPy array or an NDArray (a view, no copy)."""
    if isinstance(a, ndarray.NDArray):
        return ndarray.NDArray(a.t.narrow(0, lo, hi - lo), a.ctx, owns=False)
    return a[lo:hi]


def _mk(op, inputs, orig, **attrs):
    node = Node()
    node.op = op
    node.inputs = list(inputs)
    node.phase = orig.phase
    node.attrs = dict(attrs, orig=orig)
    node.name = op.name
    node.fwd_node = orig.fwd_node
    if isinstance(op, WholeOp) and isinstance(getattr(orig, "state", None), dict):
        node.state = orig.state          # the engine flags a rebuild ("rematerialise") through the node's state
    j = attrs.get("piece")
    node.desc = "%s%s" % (orig.desc, "" if j is None else "[%d/%d]" % (j, attrs.get("pieces", 0)))
    return node


class _MicroBase(Op):
    """Common part of the micro-op wrappers: they act for an original node (``attrs["orig"]``)."""
    recomputable = True

    def __init__(self, name):
        self.name = name

    def _ins(self, node, ins):
        cut = node.attrs.get("cut")
        if not cut:
            return list(ins)
        lo, hi = node.attrs["bounds"]
        return [_piece(a, lo, hi) if c else a for a, c in zip(ins, cut)]

    def flops(self, node, input_shapes, output_shape):
        orig = node.attrs["orig"]
        out = node.attrs.get("op_out_shape", output_shape)
        try:
            return float(orig.op.flops(orig, node.attrs.get("op_in_shapes", input_shapes), out))
        except Exception:
            return 0.0

    def infer_shape(self, node, s):
        return node.attrs.get("shape")

    def gradient(self, node, g):
        raise NotImplementedError("micro-ops are created after differentiation")


class WholeOp(_MicroBase):
    """The original operator on whole tensors."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        return orig.op.compute(orig, ins, out, use_numpy, stream)


class FillOp(_MicroBase):
    """``OnesLike`` / ``ZerosLike`` of a whole tensor.  The result depends on the operand's SHAPE only, which is
    known when the graph is lowered, so the micro-op takes no input: the ones that seed the backward pass do not
    wait for the loss to be accumulated over all pieces, and a network without whole-batch statistics lowers to a
    single level in which every piece runs forward AND backward before the next one starts."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        value = node.attrs["orig"].op.value
        if use_numpy:
            out[...] = value
        else:
            G.fill(out, value, stream)
        return None

    def flops(self, node, input_shapes, output_shape):
        return float(np.prod(output_shape)) if output_shape else 1.0


class PieceOp(_MicroBase):
    """Piece j of k of a batch-separable operator."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        ins = self._ins(node, ins)
        if orig.op.name in ("Dropout", "DropoutGradient"):
            lo, _ = node.attrs["bounds"]
            per = int(np.prod(node.attrs["shape"][1:])) if len(node.attrs["shape"]) > 1 else 1
            orig.attrs["element_offset"] = lo * per       # the mask is a function of the element's index in the WHOLE tensor
            try:
                return orig.op.compute(orig, ins, out, use_numpy, stream)
            finally:
                orig.attrs.pop("element_offset", None)
        bn = node.attrs.get("stat_for")
        if bn is not None and not use_numpy and self._conv_with_stats(node, orig, bn, ins, out, stream):
            return None
        return orig.op.compute(orig, ins, out, use_numpy, stream)

    @staticmethod
    def _open_stats(st, first):
        """Start the piece-wise sums of a new step (the first piece that arrives in a run does it)."""
        from ..ops import misc
        if first and st.get("opened_run") != misc.RUN_ID[0]:
            st["opened_run"] = misc.RUN_ID[0]
            st["micro_chunks"], st["micro_rows"] = 0, 0
            st["stats_open"] = True
            st["conv_stat_pieces"] = set()
        return st.get("stats_open") and st.get("opened_run") == misc.RUN_ID[0]

    def _conv_with_stats(self, node, orig, bn, ins, out, stream):
        """Piece j of a convolution whose output feeds a batch norm that is computed piece by piece: the
        epilogue leaves the piece's column sums in the batch norm's piece-wise buffer, so the separate
        statistics pass over this piece (``BnStatOp``) has nothing left to do.  Only in the forward pass of the
        step: a rebuild of the piece after the statistics were finalised is a plain convolution."""
        from ..ops.conv import _pads
        x, w = ins
        j, k = node.attrs["piece"], node.attrs["pieces"]
        st = _bn_state(bn)
        if not self._open_stats(st, node.attrs.get("stat_first", False)) or j in st["conv_stat_pieces"]:
            return False
        o = out.shape[1]
        if o % 4 or x.shape[1] % 4 or not (x.is_channels_last() and w.is_channels_last() and out.is_channels_last()):
            return False
        plane = k * G.BN_PIECE_CHUNKS * o
        part = st.get("micro_part")
        if part is None or part.shape != (2 * plane,):
            part = st["micro_part"] = _side((2 * plane,), out.ctx)
        ph, pw = _pads(orig)
        room = k * G.BN_PIECE_CHUNKS - st["micro_chunks"]
        chunks = G.conv2d_fwd_stats(x, w, out, ph, pw, orig.attrs["stride"], part, stream,
                                    chunk_offset=st["micro_chunks"], plane=plane,
                                    max_chunks=min(G.BN_PIECE_CHUNKS, room))
        if chunks:
            st["micro_chunks"] += chunks
            st["micro_rows"] += out.shape[0] * out.shape[2] * out.shape[3]
            st["conv_stat_pieces"].add(j)
        return True


class AccumulateOp(_MicroBase):
    """Piece j of a batch reduction.  The first micro-op that runs owns the output; the others compute
    their contribution into a scratch array of the same shape and add it to that output (their own
    ``out`` is None, the accumulator is their last input)."""
    recomputable = False
    _scratch = {}

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        if node.attrs["first"]:
            return orig.op.compute(orig, self._ins(node, ins), out, use_numpy, stream)
        acc = ins[-1]
        ins = self._ins(node, ins[:-1])
        if use_numpy:
            acc += orig.op.np_compute(orig, ins)
            return None
        key = (acc.ctx.device_id, tuple(acc.shape), acc.strides)
        tmp = AccumulateOp._scratch.get(key)
        if tmp is None:
            import torch
            tmp = AccumulateOp._scratch[key] = ndarray.NDArray(torch.empty_like(acc.t), acc.ctx)
        orig.op.compute(orig, ins, tmp, False, stream)
        G.binary(G.BIN_ADD, acc, tmp, acc, stream)
        return None


class MergeOp(_MicroBase):
    """k batch pieces -> one whole tensor (in front of an operator that runs whole)."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        lo = 0
        for a in ins:
            n = a.shape[0]
            if use_numpy:
                out[lo:lo + n] = a
            else:
                G.copy(a, _piece(out, lo, lo + n), stream)
            lo += n

    def flops(self, node, input_shapes, output_shape):
        return 0.0


def _bn_state(orig):
    st = getattr(orig, "state", None)
    if st is None:
        st = orig.state = {}
    return st


def _side(shape, ctx, value=None):
    a = ndarray.empty(shape, ctx, use_pool=False)
    if value is not None:
        a.t.fill_(value)
    return a


class BnStatOp(_MicroBase):
    """Column sums of one piece of a batch norm's input (no output tensor)."""
    recomputable = False

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig, j, k = node.attrs["orig"], node.attrs["piece"], node.attrs["pieces"]
        x = self._ins(node, ins)[0]
        st = _bn_state(orig)
        if use_numpy:
            if node.attrs["first"]:
                st["np_sum"] = np.zeros(x.shape[1], np.float64)
                st["np_sq"] = np.zeros(x.shape[1], np.float64)
                st["np_rows"] = 0
            st["np_sum"] += x.sum(axis=(0, 2, 3), dtype=np.float64)
            st["np_sq"] += np.square(x, dtype=np.float64).sum(axis=(0, 2, 3))
            st["np_rows"] += x.shape[0] * x.shape[2] * x.shape[3]
            return None
        c = x.shape[1]
        plane = k * G.BN_PIECE_CHUNKS * c
        PieceOp._open_stats(st, node.attrs["first"])
        if j in st.get("conv_stat_pieces", ()):
            return None                 # the convolution that produced this piece left its sums in the epilogue
        part = st.get("micro_part")
        if part is None or part.shape != (2 * plane,):
            part = st["micro_part"] = _side((2 * plane,), x.ctx)
        st["micro_chunks"] += G.bn_stats_partial(x, part, plane, st["micro_chunks"], stream)
        st["micro_rows"] += x.shape[0] * x.shape[2] * x.shape[3]
        return None


class BnFinalizeOp(_MicroBase):
    """Mean / inverse deviation of the whole batch from the pieces' sums; running statistics once."""
    recomputable = False

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        st = _bn_state(orig)
        eps, mom = orig.attrs["eps"], orig.attrs["momentum"]
        if use_numpy:
            m = st["np_sum"] / st["np_rows"]
            var = np.maximum(st["np_sq"] / st["np_rows"] - m * m, 0.0)
            st["np_mean"], st["np_invstd"] = m.astype(np.float32), (1.0 / np.sqrt(var + eps)).astype(np.float32)
            st["np_run_mean"] = mom * st.get("np_run_mean", np.zeros_like(st["np_mean"])) + (1 - mom) * st["np_mean"]
            st["np_run_var"] = mom * st.get("np_run_var", np.ones_like(st["np_mean"])) + (1 - mom) * var.astype(
                np.float32)
            return None
        scale = ins[0]
        c = int(np.prod(scale.shape))
        if "mean" not in st or st["mean"].shape != (c,):
            st["mean"], st["invstd"] = _side((c,), scale.ctx), _side((c,), scale.ctx)
            st["run_mean"], st["run_var"] = _side((c,), scale.ctx, 0.0), _side((c,), scale.ctx, 1.0)
        G.bn_stats_finalize(st["micro_part"], st["micro_part"].shape[0] // 2, st["micro_chunks"], st["micro_rows"], c,
                            eps, mom, st["mean"], st["invstd"], st["run_mean"], st["run_var"], stream)
        st["stats_open"] = False        # pieces rebuilt from here on are plain convolutions
        return None


class BnApplyOp(_MicroBase):
    """Normalise / scale / shift (/ReLU) one piece with the whole-batch statistics."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        x, scale, bias = self._ins(node, ins)
        st = _bn_state(orig)
        relu = orig.op.name == "BatchNormRelu"
        if use_numpy:
            bc = (1, -1, 1, 1)
            y = (x - st["np_mean"].reshape(bc)) * st["np_invstd"].reshape(bc) * scale.reshape(bc) + bias.reshape(bc)
            out[...] = np.maximum(y, 0) if relu else y
            return None
        G.bn_apply(x, scale, bias, out, st["mean"], st["invstd"], relu, stream)
        return None

    def flops(self, node, input_shapes, output_shape):
        return 4.0 * float(np.prod(output_shape))


class BnBwdStatOp(_MicroBase):
    """Sums of dy and dy * xhat of one piece (dy masked by the ReLU of the fused forward)."""
    recomputable = False

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig, k = node.attrs["orig"], node.attrs["pieces"]
        vals = self._ins(node, ins)
        g, x, scale = vals[0], vals[1], vals[2]
        bias = vals[3] if orig.op.name == "BatchNormReluGradient" else None
        fst, st = _bn_state(orig.attrs["fwd"]), _bn_state(orig)
        if use_numpy:
            bc = (1, -1, 1, 1)
            xn = (x - fst["np_mean"].reshape(bc)) * fst["np_invstd"].reshape(bc)
            if bias is not None:
                g = g * ((xn * scale.reshape(bc) + bias.reshape(bc)) > 0)
            if node.attrs["first"]:
                st["np_ds"] = np.zeros(x.shape[1], np.float64)
                st["np_db"] = np.zeros(x.shape[1], np.float64)
                st["np_rows"] = 0
            st["np_ds"] += (g * xn).sum(axis=(0, 2, 3), dtype=np.float64)
            st["np_db"] += g.sum(axis=(0, 2, 3), dtype=np.float64)
            st["np_rows"] += x.shape[0] * x.shape[2] * x.shape[3]
            return None
        c = x.shape[1]
        plane = k * G.BN_PIECE_CHUNKS * c
        part = st.get("micro_part")
        if part is None or part.shape != (2 * plane,):
            part = st["micro_part"] = _side((2 * plane,), x.ctx)
        if node.attrs["first"]:
            st["micro_chunks"], st["micro_rows"] = 0, 0
        st["micro_chunks"] += G.bn_bwd_partial(g, x, fst["mean"], fst["invstd"], scale if bias is not None else None,
                                               bias, part, plane, st["micro_chunks"], stream)
        st["micro_rows"] += x.shape[0] * x.shape[2] * x.shape[3]
        return None


class BnBwdFinalizeOp(_MicroBase):
    recomputable = False

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        st = _bn_state(orig)
        scale = ins[0]
        if use_numpy:
            st["np_dscale"] = st["np_ds"].astype(np.float32).reshape(scale.shape)
            st["np_dbias"] = st["np_db"].astype(np.float32).reshape(scale.shape)
            return None
        if "dscale" not in st or st["dscale"].shape != tuple(scale.shape):
            st["dscale"], st["dbias"] = _side(scale.shape, scale.ctx), _side(scale.shape, scale.ctx)
        G.bn_bwd_finalize(st["micro_part"], st["micro_part"].shape[0] // 2, st["micro_chunks"],
                          int(np.prod(scale.shape)), st["dscale"], st["dbias"], stream)
        return None


class BnBwdApplyOp(_MicroBase):
    """dx of one piece from the whole-batch sums."""

    def compute(self, node, ins, out, use_numpy=True, stream=None):
        orig = node.attrs["orig"]
        vals = self._ins(node, ins)
        g, x, scale = vals[0], vals[1], vals[2]
        bias = vals[3] if orig.op.name == "BatchNormReluGradient" else None
        fst, st = _bn_state(orig.attrs["fwd"]), _bn_state(orig)
        if use_numpy:
            bc = (1, -1, 1, 1)
            m = float(st["np_rows"])
            xn = (x - fst["np_mean"].reshape(bc)) * fst["np_invstd"].reshape(bc)
            if bias is not None:
                g = g * ((xn * scale.reshape(bc) + bias.reshape(bc)) > 0)
            out[...] = (scale.reshape(bc) * fst["np_invstd"].reshape(bc)) * (
                g - st["np_db"].reshape(bc) / m - xn * st["np_ds"].reshape(bc) / m)
            return None
        G.bn_bwd_apply(g, x, scale, bias, fst["mean"], fst["invstd"], st["dscale"], st["dbias"], out,
                       st["micro_rows"], stream)
        return None

    def flops(self, node, input_shapes, output_shape):
        return 8.0 * float(np.prod(output_shape))


class Lowered(object):
    """Result of :func:`lower`: the micro-op schedule and what the engine needs to run it."""

    def __init__(self):
        self.order = []            # micro-nodes in execution order (placeholders included)
        self.shapes = {}           # micro-node -> shape (None = no output tensor)
        self.layout = {}           # micro-node -> channels-last?
        self.evals = []            # micro-nodes standing for the original eval nodes, same order
        self.pieces = 1
        self.micro_ops = 0         # micro-ops that act on a batch piece
        self.no_evict = set()      # accumulators: mutated after they were produced
        self.no_rebuild = set()


def lower(topo_order, shapes, layout, eval_nodes, feed_nodes, pieces, min_split_bytes=0):
    """Lower the scheduled graph ``topo_order`` to micro-ops over ``pieces`` batch pieces.

    ``shapes`` / ``layout`` are the inferred shape and layout maps of the original nodes,
    ``feed_nodes`` the fed placeholders (the batch size is the leading extent of the first 4-D
    or otherwise first feed).  Operators whose largest batch-sized operand is below
    ``min_split_bytes`` run whole."""
    k = int(pieces)
    feeds = [n for n in topo_order if n in feed_nodes]
    assert feeds, "lowering needs a fed placeholder to read the batch size from"
    batch = int(shapes[feeds[0]][0])
    k = max(1, min(k, batch))

    # which original tensors carry the batch in their leading dimension
    carries = {}
    for n in topo_order:
        shp = shapes.get(n)
        if n in feed_nodes:
            carries[n] = shp is not None and len(shp) >= 1 and shp[0] == batch
        elif isinstance(n.op, PlaceholderOp) or shp is None or n.op.name in REDUCING:
            carries[n] = False
        else:
            carries[n] = len(shp) >= 1 and shp[0] == batch and any(carries.get(i, False) for i in n.inputs)

    def kind_of(n):
        if isinstance(n.op, PlaceholderOp) or n in feed_nodes:
            return "ext"
        if k == 1:
            return "whole"
        name = n.op.name
        shp = shapes.get(n)
        big = max([_nbytes(shapes[i]) for i in n.inputs if carries.get(i)] + [_nbytes(shp) if shp and carries[n] else 0])
        if big < max(min_split_bytes, 1):
            return "whole"
        cut_in = [i for i in n.inputs if carries.get(i)]
        if not cut_in:
            return "whole"
        if name in SEPARABLE and carries[n]:
            if name in ("Reshape", "ReshapeGradient") and not all(shapes[i][0] == batch for i in cut_in):
                return "whole"
            return "sep"
        if name in REDUCING:
            return "red"
        if name in BN_FWD and shp is not None and len(shp) == 4 and carries.get(n.inputs[0]):
            return "bnf"
        if name in BN_BWD and shp is not None and len(shp) == 4 and carries.get(n.inputs[0]) and \
                carries.get(n.inputs[1]) and n.attrs.get("fwd") is not None:
            return "bnb"
        return "whole"

    kind = {n: kind_of(n) for n in topo_order}
    for n in topo_order:
        if kind[n] == "whole" and k > 1 and n.op.name in ("OnesLike", "ZerosLike") and shapes.get(n) is not None:
            kind[n] = "fill"
    # a split batch-norm backward needs its forward split too (the statistics live in the forward's state either way),
    # and the pick node that only renames dx follows its producer
    for n in topo_order:
        if n.op.name == "BatchNormGradData":
            kind[n] = "alias" if kind[n.inputs[0]] == "bnb" else "whole"
    split_out = {n: kind[n] in ("sep", "bnf", "bnb", "alias") for n in topo_order}

    # barrier levels: a stage that needs ALL pieces of something starts one level later
    level, avail = {}, {}
    for n in topo_order:
        kd = kind[n]
        if kd == "ext":
            level[n], avail[n] = 0, 0
            continue
        lv = 0
        for i in (n.inputs if kd != "fill" else ()):
            a = avail[i]
            if split_out[i] and kd in ("whole",):
                a += 1                      # merge of all pieces
            lv = max(lv, a)
        level[n] = lv
        if kd in ("sep", "whole", "alias", "fill"):
            avail[n] = lv
        elif kd == "red":
            avail[n] = lv + 1               # all pieces accumulated
        else:                               # bnf / bnb: statistics at lv, finalise + apply at lv + 1
            avail[n] = lv + 1
    out = Lowered()
    out.pieces = k
    bounds = [ndarray._split_bounds(batch, k, j) for j in range(k)]
    whole_of, piece_of, merged = {}, {}, {}

    def pshape(shp, j):
        lo, hi = bounds[j]
        return (hi - lo,) + tuple(shp[1:])

    def emit(node, shape, like):
        out.order.append(node)
        out.shapes[node] = tuple(shape) if shape is not None else None
        out.layout[node] = layout.get(like, False)
        node.attrs["shape"] = out.shapes[node]
        node.inferred_shape = out.shapes[node]
        return node

    def whole_input(i):
        """Micro-node holding original tensor ``i`` whole (merging its pieces when it is split)."""
        if not split_out[i]:
            return whole_of[i]
        if i not in merged:
            m = _mk(MergeOp("MicroMerge"), [piece_of[(i, j)] for j in range(k)], i)
            merged[i] = emit(m, shapes[i], i)
        return merged[i]

    def piece_inputs(n, j):
        """(micro inputs, cut flags, shapes as the original op sees them) for piece j of n."""
        ins, cut, seen = [], [], []
        for i in n.inputs:
            if carries.get(i) and split_out[i]:
                ins.append(piece_of[(i, j)]); cut.append(False); seen.append(pshape(shapes[i], j))
            elif carries.get(i):
                ins.append(whole_of[i]); cut.append(True); seen.append(pshape(shapes[i], j))
            else:
                ins.append(whole_input(i) if split_out.get(i) else whole_of[i]); cut.append(False)
                seen.append(shapes[i])
        return ins, cut, seen

    for n in topo_order:
        if kind[n] == "ext":
            whole_of[n] = n
            out.order.append(n)
            out.shapes[n] = shapes.get(n)
            out.layout[n] = layout.get(n, False)

    max_level = max(level.values()) if level else 0
    acc_owner = {}
    stat_started, bstat_started = set(), set()
    for lv in range(max_level + 1):
        here = [n for n in topo_order if kind[n] != "ext"]
        # 1. whole operators and finalise stages of this level
        for n in here:
            kd = kind[n]
            if kd == "fill" and level[n] == lv:
                whole_of[n] = emit(_mk(FillOp(n.op.name), [], n), shapes[n], n)
            elif kd == "whole" and level[n] == lv:
                if n.op.name in ("BatchNormGradScale", "BatchNormGradBias") and kind.get(n.inputs[0]) == "bnb":
                    ins = [whole_of[n.inputs[1]]]       # the sums are read from the gradient node's state
                else:
                    ins = [whole_input(i) for i in n.inputs]
                node = _mk(WholeOp(n.op.name), ins, n)
                whole_of[n] = emit(node, shapes.get(n), n)
                if n.op.name == "Optimizer" or shapes.get(n) is None:
                    out.no_rebuild.add(node)
            elif kd == "bnf" and level[n] + 1 == lv:
                fin = _mk(BnFinalizeOp(n.op.name + "Finalize"), [whole_of[n.inputs[1]]], n)
                emit(fin, None, n)
            elif kd == "bnb" and level[n] + 1 == lv:
                fin = _mk(BnBwdFinalizeOp(n.op.name + "Finalize"), [whole_of[n.inputs[2]]], n)
                emit(fin, None, n)
        # 2. piece stages, piece-major, alternating direction
        js = range(k) if lv % 2 == 0 else range(k - 1, -1, -1)
        staged = [n for n in here if (kind[n] in ("sep", "red", "alias") and level[n] == lv) or
                  (kind[n] in ("bnf", "bnb") and level[n] in (lv, lv - 1))]
        if not staged:
            continue
        for j in js:
            for n in staged:
                kd = kind[n]
                if kd == "alias":
                    piece_of[(n, j)] = piece_of[(n.inputs[0], j)]
                    continue
                ins, cut, seen = piece_inputs(n, j)
                common = dict(piece=j, pieces=k, bounds=bounds[j], cut=cut, op_in_shapes=seen)
                if kd == "sep":
                    node = _mk(PieceOp(n.op.name), ins, n, **common)
                    piece_of[(n, j)] = emit(node, pshape(shapes[n], j), n)
                    node.attrs["op_out_shape"] = out.shapes[node]
                    out.micro_ops += 1
                elif kd == "red":
                    first = n not in acc_owner
                    if first:
                        node = _mk(AccumulateOp(n.op.name), ins, n, first=True, **common)
                        acc_owner[n] = whole_of[n] = emit(node, shapes[n], n)
                        out.no_evict.add(node)
                    else:
                        common["cut"] = cut
                        node = _mk(AccumulateOp(n.op.name), ins + [acc_owner[n]], n, first=False, **common)
                        emit(node, None, n)
                    node.attrs["op_out_shape"] = shapes[n]
                    out.no_rebuild.add(node)
                    out.micro_ops += 1
                elif kd == "bnf":
                    if level[n] == lv:          # statistics stage
                        src = n.inputs[0]
                        if kind.get(src) == "sep" and src.op.name == "Conv2d" and (src, j) in piece_of and \
                                src.attrs.get("bn_consumer") is n:
                            # the convolution piece right before this stage takes the sums in its epilogue
                            piece_of[(src, j)].attrs["stat_for"] = n
                            piece_of[(src, j)].attrs["stat_first"] = n not in stat_started
                        node = _mk(BnStatOp(n.op.name + "Stats"), ins[:1], n, first=n not in stat_started,
                                   **dict(common, cut=cut[:1], op_in_shapes=seen[:1]))
                        stat_started.add(n)
                        emit(node, None, n)
                    else:                       # normalise stage
                        node = _mk(BnApplyOp(n.op.name), ins, n, **common)
                        piece_of[(n, j)] = emit(node, pshape(shapes[n], j), n)
                    out.micro_ops += 1
                elif kd == "bnb":
                    if level[n] == lv:
                        node = _mk(BnBwdStatOp(n.op.name + "Stats"), ins, n, first=n not in bstat_started, **common)
                        bstat_started.add(n)
                        emit(node, None, n)
                    else:
                        node = _mk(BnBwdApplyOp(n.op.name), ins, n, **common)
                        piece_of[(n, j)] = emit(node, pshape(shapes[n], j), n)
                    out.micro_ops += 1
    for n in out.order:
        if isinstance(n.op, _MicroBase) and not n.op.recomputable:
            out.no_rebuild.add(n)
        if n.op.name == "Optimizer":
            out.no_rebuild.update(n.inputs)     # a finished parameter gradient may be copied out, never recomputed
    out.evals = [whole_input(n) if kind[n] != "ext" else n for n in eval_nodes]
    return out
