"""Placeholders, fills, one-hot, embedding, dropout and the swap / split nodes.

Capability parity: ``gpu_ops/Variable.py:7-59``, ``OnesLike.py``, ``ZerosLike.py``,
``OneHot.py``, ``EmbeddingLookUp.py:36-93``, ``Dropout.py:51-143``,
``SwapOut.py:8-114`` and ``Split.py:7-69``.

The embedding kernels honour the index tensor (the reference kernel uses the
thread index instead of ``ids``, ``src/ops/EmbeddingLookup.cu:6-7,59-60``), and
dropout draws a counter-based (Philox-style) mask from a per-node seed and step
counter, so the backward pass regenerates the mask instead of storing a
reserve buffer (``src/ops/CudnnDropout.cu:4-152``).
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from .. import ndarray
from . import _gpu as G


# -- placeholders -----------------------------------------------------------------
class PlaceholderOp(Op):
    name = "Placeholder"

    def __call__(self, value=None, trainable=True):
        node = Op.__call__(self)
        if value is not None:
            assert isinstance(value, (np.ndarray, ndarray.NDArray))
        else:
            trainable = False
        node.tensor_value = value
        node.trainable = trainable
        return node

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        assert node.tensor_value is not None, "placeholder %s values provided by feed_dict" % node.name
        return node.tensor_value

    def gradient(self, node, g):
        return None

    def infer_shape(self, node, s):
        assert node.tensor_value is not None, "placeholder %s shape provided by feed_shape" % node.name
        return tuple(node.tensor_value.shape)


_placeholder = PlaceholderOp()


def placeholder_op(value=None, trainable=True):
    return _placeholder(value, trainable)


def Variable(name, value=None, trainable=True, swap=False):
    """User-defined variable, e.g. ``x = Variable(name="x")``."""
    node = placeholder_op(value, trainable)
    node.name = name
    node.desc = "%s_%d" % (name, node.id)
    node.swap = swap
    return node


# -- fills ---------------------------------------------------------------------------
class _FillLike(Op):
    value, cheap = 0.0, True

    def __call__(self, x):
        return Op.__call__(self, x)

    def np_compute(self, node, iv):
        return np.full(iv[0].shape, self.value, dtype=np.float32)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(out):
            return False
        cpu_links.array_set(out, self.value)
        return True

    def gpu_compute(self, node, iv, out, stream):
        G.fill(out, self.value, stream)

    def gradient(self, node, g):
        return [zeroslike_op(node.inputs[0])]

    def infer_shape(self, node, s):
        return tuple(s[0])


class OnesLikeOp(_FillLike):
    name, value = "OnesLike", 1.0


class ZerosLikeOp(_FillLike):
    name, value = "ZerosLike", 0.0


_ones, _zeros = OnesLikeOp(), ZerosLikeOp()


def oneslike_op(node):
    return _ones(node)


def zeroslike_op(node):
    return _zeros(node)


# -- one-hot ---------------------------------------------------------------------------
class OneHotOp(Op):
    name = "OneHot"

    def __call__(self, x, num_classes):
        return Op.__call__(self, x, num_classes=num_classes)

    def np_compute(self, node, iv):
        idx = iv[0].astype(np.int64)
        return np.eye(node.attrs["num_classes"], dtype=np.float32)[idx]

    def gpu_compute(self, node, iv, out, stream):
        G.one_hot(iv[0], out, node.attrs["num_classes"], stream)

    def gradient(self, node, g):
        return [None]

    def infer_shape(self, node, s):
        return tuple(s[0]) + (node.attrs["num_classes"],)


_onehot = OneHotOp()


def one_hot_op(node, num_classes):
    return _onehot(node, num_classes)


# -- embedding ---------------------------------------------------------------------------
class EmbeddingLookUpOp(Op):
    name = "EmbeddingLookUp"

    def __call__(self, table, index):
        return Op.__call__(self, table, index)

    def np_compute(self, node, iv):
        flat = iv[1].reshape(-1).astype(np.int64)
        return iv[0][flat].reshape(tuple(iv[1].shape) + (iv[0].shape[1],))

    def gpu_compute(self, node, iv, out, stream):
        G.embedding(iv[0], iv[1], out, stream)

    def gradient(self, node, g):
        return [embedding_lookup_gradient_op(g, node.inputs[1], node.inputs[0]), None]

    def infer_shape(self, node, s):
        return tuple(s[1]) + (s[0][1],)


class EmbeddingLookUpGradientOp(Op):
    name = "EmbeddingLookUpGradient"

    def __call__(self, vectors, index, table):
        return Op.__call__(self, vectors, index, like=table)

    def np_compute(self, node, iv):
        shape = node.attrs["like"].inferred_shape
        out = np.zeros(shape, dtype=np.float32)
        np.add.at(out, iv[1].reshape(-1).astype(np.int64), iv[0].reshape(-1, shape[1]))
        return out

    def gpu_compute(self, node, iv, out, stream):
        G.fill(out, 0.0, stream)
        G.embedding_grad(iv[0], iv[1], out, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(node.attrs["like"].inferred_shape)


_emb, _embg = EmbeddingLookUpOp(), EmbeddingLookUpGradientOp()


def embedding_lookup_op(embedding, index):
    return _emb(embedding, index)


def embedding_lookup_gradient_op(vectors, index, embedding):
    return _embg(vectors, index, embedding)


# -- dropout ---------------------------------------------------------------------------
def philox_like_mask(shape, keep_prob, seed, offset=0):
    """Host twin of the device mask generator: element i is kept when
    ``hash(seed, i)`` maps below ``keep_prob`` (same integer mix as
    ``csrc/kernels/misc.cu``).  ``offset``: index of the first element in the whole
    tensor when ``shape`` is a batch piece of it."""
    n = int(np.prod(shape))
    i = np.arange(n, dtype=np.uint64) + np.uint64(offset)
    with np.errstate(over="ignore"):
        x = i + np.uint64(seed) * np.uint64(0x9E3779B97F4A7C15)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    u = (x >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / (1 << 24))
    return (u < np.float32(keep_prob)).reshape(shape)


#: index of the training step that is executing; executors set it at the start of ``run`` so that
#: dropout draws a fresh mask every step while forward, recompute and backward of one step agree
STEP = [0]
#: device address of the running executor's step counter (0 = none: the host index above is used)
STEP_DEV = [0]
#: bumped at the start of every ``run`` of every executor: per-step side state of an operator (batch-norm sums
#: collected piece by piece) tells a new step from a rebuild inside the same step by it
RUN_ID = [0]


def step_seed(node):
    return (int(node.attrs["seed"]) + 0x632BE5AB * int(STEP[0])) & 0x7FFFFFFFFFFFFFFF


class DropoutOp(Op):
    """``x * mask / keep_prob`` with a mask that is a pure function of
    (node seed, step index, element index), so forward, recompute and backward
    of one step agree and every step draws a new mask."""
    name = "Dropout"

    def __call__(self, x, keep_prob, seed=None):
        node = Op.__call__(self, x, keep_prob=float(keep_prob))
        node.attrs["seed"] = (0x5EED0000 + node.id) if seed is None else int(seed)
        return node

    def np_compute(self, node, iv):
        kp = node.attrs["keep_prob"]
        m = philox_like_mask(iv[0].shape, kp, step_seed(node), node.attrs.get("element_offset", 0))
        return (iv[0] * m / kp).astype(np.float32)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out):
            return False
        cpu_links.dropout(iv[0], out, node.attrs["keep_prob"], step_seed(node), int(node.attrs.get("element_offset", 0)))
        return True

    def gpu_compute(self, node, iv, out, stream):
        assert iv[0].is_dense() and iv[0].same_layout(out)
        off = int(node.attrs.get("element_offset", 0))
        if STEP_DEV[0]:
            G.dropout(iv[0], out, node.attrs["keep_prob"], int(node.attrs["seed"]), stream, step_dev=STEP_DEV[0],
                      offset=off)
        else:
            G.dropout(iv[0], out, node.attrs["keep_prob"], step_seed(node), stream, offset=off)

    def gradient(self, node, g):
        return [dropout_gradient_op(g, node.attrs["keep_prob"], node)]

    def infer_shape(self, node, s):
        return tuple(s[0])


class DropoutGradientOp(Op):
    name = "DropoutGradient"

    def __call__(self, g, keep_prob, forward_node):
        return Op.__call__(self, g, keep_prob=float(keep_prob), seed=forward_node.attrs["seed"])

    np_compute = DropoutOp.np_compute
    cpu_compute = DropoutOp.cpu_compute
    gpu_compute = DropoutOp.gpu_compute

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(s[0])


_drop, _dropg = DropoutOp(), DropoutGradientOp()


def dropout_op(node_in, keep_prob, seed=None):
    return _drop(node_in, keep_prob, seed)


def dropout_gradient_op(node_in, keep_prob, forward_node):
    return _dropg(node_in, keep_prob, forward_node)


# -- explicit swap / split nodes -------------------------------------------------------------
class SwapOutOp(Op):
    """Device -> pinned host copy on the executor's D2H stream."""
    name = "SwapOut"

    def __call__(self, x):
        return Op.__call__(self, x)

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        if use_numpy:
            output_val[...] = input_vals[0]
        else:
            output_val.async_d2h(input_vals[0], stream_handle, output_val.gpu2cpu_event
                                 if hasattr(output_val, "gpu2cpu_event") else None)

    def gradient(self, node, g):
        return [g]

    def infer_shape(self, node, s):
        return tuple(s[0])


class SwapInOp(Op):
    """Pinned host -> device copy on the executor's H2D stream."""
    name = "SwapIn"

    def __call__(self, x):
        return Op.__call__(self, x)

    def compute(self, node, input_vals, output_val, use_numpy=True, stream_handle=None):
        if use_numpy:
            output_val[...] = input_vals[0]
        else:
            output_val.async_h2d(input_vals[0], stream_handle, output_val.cpu2gpu_event)

    def gradient(self, node, g):
        return [g]

    def infer_shape(self, node, s):
        return tuple(s[0])


class SplitOp(Op):
    """Micro-tensor ``sub_index`` of ``total_num`` along batch or channel."""
    name, cheap = "Split", True

    def __call__(self, x, sub_index, total_num, dimension="batch"):
        return Op.__call__(self, x, sub_index=sub_index, total_num=total_num, dimension=dimension)

    def _bounds(self, node, shape):
        dim = 0 if node.attrs["dimension"] == "batch" else 1
        b, e = ndarray._split_bounds(shape[dim], node.attrs["total_num"], node.attrs["sub_index"])
        return dim, b, e

    def np_compute(self, node, iv):
        dim, b, e = self._bounds(node, iv[0].shape)
        sl = [slice(None)] * iv[0].ndim
        sl[dim] = slice(b, e)
        return iv[0][tuple(sl)]

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        dim, b, e = self._bounds(node, x.shape)
        G.copy_raw(x.ptr + 4 * b * x.strides[dim], x.strides, out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        from .shape import slice_gradient_op
        raise NotImplementedError("split nodes are inserted after differentiation")

    def infer_shape(self, node, s):
        dim, b, e = self._bounds(node, s[0])
        out = list(s[0])
        out[dim] = e - b
        return tuple(out)


_swapout, _swapin, _split = SwapOutOp(), SwapInOp(), SplitOp()


def swap_out_op(node):
    return _swapout(node)


def swap_in_op(node):
    return _swapin(node)


def split_op(node, sub_index, total_num, dimension="batch"):
    return _split(node, sub_index, total_num, dimension)
