"""Data-movement family: reshape, transpose, slice, concat, pad, the three
broadcast flavours and the two reductions.

Capability parity: ``gpu_ops/Reshape.py:42-155``, ``Transpose.py:44-76``,
``Slice.py:47-155``, ``Concat.py:47-141``, ``Pad.py:48-150``,
``Broadcast.py:45-74``, ``BroadcastShape.py:48-97``, ``BroadcastTF.py:46-87``,
``ReduceSum.py:54-95``, ``ReduceSumAxisZero.py``.

GPU path: every op here is one launch of a generic strided-copy or
strided-reduce kernel whose shape/stride tables travel as kernel parameters —
the reference instead does pool allocations plus blocking host-to-device copies
of the tables on every call (``src/ops/Slice.cu:48-57``, ``Transpose.cu:47-52``).
"""
from __future__ import annotations

import numpy as np

from ..graph import Op
from . import _gpu as G


def _numel(s):
    n = 1
    for d in s:
        n *= d
    return n


def _row_major(shape):
    st, acc = [], 1
    for d in reversed(shape):
        st.insert(0, acc)
        acc *= d
    return st


# -- reshape ---------------------------------------------------------------------
def _resolve(shape, numel):
    shape = list(shape)
    if -1 in shape:
        i = shape.index(-1)
        rest = 1
        for j, d in enumerate(shape):
            if j != i:
                rest *= d
        shape[i] = numel // rest
    assert _numel(shape) == numel, "reshape to %s does not keep %d elements" % (shape, numel)
    return tuple(shape)


def _reshape_gpu(x, out, stream):
    """Logical (row-major) element order is preserved whatever the two physical
    layouts are: walk the finer of the two index spaces.  When both sides are
    row-major this is a flat copy."""
    if x.is_contiguous() and out.is_contiguous():
        G.copy_raw(x.ptr, [1], out.ptr, [1], [_numel(x.shape)], stream)
    elif out.is_contiguous():
        G.copy_raw(x.ptr, x.strides, out.ptr, _row_major(x.shape), x.shape, stream)
    elif x.is_contiguous():
        G.copy_raw(x.ptr, _row_major(out.shape), out.ptr, out.strides, out.shape, stream)
    else:
        raise NotImplementedError("reshape between two non-row-major layouts")


class ReshapeOp(Op):
    name, cheap = "Reshape", True

    def __call__(self, x, output_shape):
        return Op.__call__(self, x, output_shape=tuple(output_shape))

    def np_compute(self, node, iv):
        shp = tuple(node.attrs["output_shape"])
        if -1 not in shp and int(np.prod(shp)) != iv[0].size:      # a batch piece of an explicitly shaped reshape
            shp = (-1,) + shp[1:]
        return iv[0].reshape(_resolve(shp, iv[0].size))

    def gpu_compute(self, node, iv, out, stream):
        _reshape_gpu(iv[0], out, stream)

    def gradient(self, node, g):
        return [array_reshape_gradient_op(node.inputs[0], g)]

    def infer_shape(self, node, s):
        return _resolve(node.attrs["output_shape"], _numel(s[0]))


class ReshapeGradientOp(Op):
    name, cheap = "ReshapeGradient", True

    def __call__(self, like, g):
        return Op.__call__(self, g, like=like)

    def np_compute(self, node, iv):
        shp = tuple(node.attrs["like"].inferred_shape)
        if int(np.prod(shp)) != iv[0].size:        # a batch piece: the leading extent follows the input
            shp = (-1,) + shp[1:]
        return iv[0].reshape(shp)

    def gpu_compute(self, node, iv, out, stream):
        _reshape_gpu(iv[0], out, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(node.attrs["like"].inferred_shape)


# -- transpose ---------------------------------------------------------------------
class TransposeOp(Op):
    name, cheap = "Transpose", True

    def __call__(self, x, perm=None):
        return Op.__call__(self, x, perm=None if perm is None else tuple(perm))

    def _perm(self, node, ndim):
        p = node.attrs["perm"]
        return tuple(reversed(range(ndim))) if p is None else p

    def np_compute(self, node, iv):
        return np.transpose(iv[0], self._perm(node, iv[0].ndim))

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out) or iv[0].ndim > 8:
            return False
        cpu_links.transpose(iv[0], out, self._perm(node, iv[0].ndim))
        return True

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        perm = self._perm(node, len(x.shape))
        G.copy_raw(x.ptr, [x.strides[p] for p in perm], out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        p = node.attrs["perm"]
        if p is None:
            return [transpose_op(g)]
        inv = [0] * len(p)
        for i, a in enumerate(p):
            inv[a] = i
        return [transpose_op(g, inv)]

    def infer_shape(self, node, s):
        perm = self._perm(node, len(s[0]))
        return tuple(s[0][p] for p in perm)


# -- slice ---------------------------------------------------------------------------
def _slice_sizes(begin, size, shape):
    return [shape[i] - begin[i] if size[i] == -1 else size[i] for i in range(len(shape))]


class SliceOp(Op):
    name, cheap = "Slice", True

    def __call__(self, x, begin, size):
        return Op.__call__(self, x, begin=tuple(begin), size=tuple(size))

    def np_compute(self, node, iv):
        b = node.attrs["begin"]
        sz = _slice_sizes(b, node.attrs["size"], iv[0].shape)
        return iv[0][tuple(slice(bi, bi + si) for bi, si in zip(b, sz))]

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        off = sum(bi * st for bi, st in zip(node.attrs["begin"], x.strides))
        G.copy_raw(x.ptr + 4 * off, x.strides, out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        return [slice_gradient_op(g, node.attrs["begin"], node.attrs["size"], like=node.inputs[0])]

    def infer_shape(self, node, s):
        b = node.attrs["begin"]
        sz = _slice_sizes(b, node.attrs["size"], s[0])
        for bi, si, di in zip(b, sz, s[0]):
            assert 0 <= bi and bi + si <= di, "slice out of range"
        return tuple(sz)


class SliceGradientOp(Op):
    """Zero-pad the gradient back to the sliced tensor's shape."""
    name, cheap = "SliceGradient", True

    def __call__(self, g, begin, size, like=None, output_shape=None):
        return Op.__call__(self, g, begin=tuple(begin), size=tuple(size), like=like,
                           output_shape=output_shape)

    def _shape(self, node):
        if node.attrs["like"] is not None:
            return tuple(node.attrs["like"].inferred_shape)
        return tuple(node.attrs["output_shape"])

    def np_compute(self, node, iv):
        out = np.zeros(self._shape(node), dtype=np.float32)
        b = node.attrs["begin"]
        out[tuple(slice(bi, bi + si) for bi, si in zip(b, iv[0].shape))] = iv[0]
        return out

    def gpu_compute(self, node, iv, out, stream):
        g = iv[0]
        G.fill(out, 0.0, stream)
        off = sum(bi * st for bi, st in zip(node.attrs["begin"], out.strides))
        G.copy_raw(g.ptr, g.strides, out.ptr + 4 * off, out.strides, g.shape, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return self._shape(node)


# -- concat ---------------------------------------------------------------------------
class ConcatOp(Op):
    name, cheap = "Concat", True

    def __call__(self, a, b, axis=0):
        return Op.__call__(self, a, b, axis=axis)

    def np_compute(self, node, iv):
        return np.concatenate(iv, axis=node.attrs["axis"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], iv[1], out):
            return False
        ax = node.attrs["axis"]
        outer = int(np.prod(out.shape[:ax], dtype=np.int64))
        ycols, off = out.size // max(outer, 1), 0
        for x in iv:
            xcols = x.size // max(outer, 1)
            cpu_links.copy_block(x, out, outer, xcols, ycols, off)
            off += xcols
        return True

    def gpu_compute(self, node, iv, out, stream):
        ax = node.attrs["axis"]
        off = 0
        for x in iv:
            G.copy_raw(x.ptr, x.strides, out.ptr + 4 * off * out.strides[ax], out.strides, x.shape, stream)
            off += x.shape[ax]

    def gradient(self, node, g):
        ax = node.attrs["axis"]
        return [concat_gradient_op(g, node.inputs[0], ax, 0), concat_gradient_op(g, node.inputs[1], ax, 1)]

    def infer_shape(self, node, s):
        ax = node.attrs["axis"]
        out = list(s[0])
        for i, (p, q) in enumerate(zip(s[0], s[1])):
            assert i == ax or p == q, "concat: shapes %s / %s differ off-axis" % (s[0], s[1])
        out[ax] = s[0][ax] + s[1][ax]
        return tuple(out)


class ConcatGradientOp(Op):
    """Slice of the concat gradient that belongs to input ``idx``.  The offset
    is the size of the *other* operand when idx == 1, resolved from the inferred
    shape of ``like`` (kept as an attribute, not a dependency)."""
    name, cheap = "ConcatGradient", True

    def __call__(self, g, like, axis, idx):
        return Op.__call__(self, g, like=like, axis=axis, idx=idx)

    def _range(self, node, gshape):
        ax, idx = node.attrs["axis"], node.attrs["idx"]
        mine = node.attrs["like"].inferred_shape[ax]
        begin = 0 if idx == 0 else gshape[ax] - mine
        return ax, begin, mine

    def np_compute(self, node, iv):
        ax, b, n = self._range(node, iv[0].shape)
        sl = [slice(None)] * iv[0].ndim
        sl[ax] = slice(b, b + n)
        return iv[0][tuple(sl)]

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        g = iv[0]
        if not cpu_links.ok(g, out):
            return False
        ax, b, n = self._range(node, g.shape)
        outer = int(np.prod(g.shape[:ax], dtype=np.int64))
        inner = int(np.prod(g.shape[ax + 1:], dtype=np.int64))
        cpu_links.copy_block(out, g, outer, n * inner, g.shape[ax] * inner, b * inner, grad=True)
        return True

    def gpu_compute(self, node, iv, out, stream):
        g = iv[0]
        ax, b, n = self._range(node, g.shape)
        G.copy_raw(g.ptr + 4 * b * g.strides[ax], g.strides, out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        return tuple(node.attrs["like"].inferred_shape)


# -- pad ---------------------------------------------------------------------------------
class PadOp(Op):
    name, cheap = "Pad", True

    def __call__(self, x, paddings, mode="CONSTANT", constant_values=0):
        assert mode == "CONSTANT", "only CONSTANT padding is implemented (as in the reference, src/ops/Pad.cu:46-52)"
        return Op.__call__(self, x, paddings=[tuple(p) for p in paddings], mode=mode,
                           constant_values=constant_values)

    def _full(self, node, ndim):
        p = node.attrs["paddings"]
        return [(0, 0)] * (ndim - len(p)) + list(p)

    def np_compute(self, node, iv):
        return np.pad(iv[0], self._full(node, iv[0].ndim), mode="constant",
                      constant_values=node.attrs["constant_values"])

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        pads = self._full(node, iv[0].ndim)
        if not cpu_links.ok(iv[0], out) or iv[0].ndim < 2 or any(p != (0, 0) for p in pads[:-2]):
            return False                       # the native kernel pads the two trailing axes
        cpu_links.pad2d(iv[0], out, pads[-2], pads[-1], float(node.attrs["constant_values"]))
        return True

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        pads = self._full(node, len(x.shape))
        G.fill(out, float(node.attrs["constant_values"]), stream)
        off = sum(p[0] * st for p, st in zip(pads, out.strides))
        G.copy_raw(x.ptr, x.strides, out.ptr + 4 * off, out.strides, x.shape, stream)

    def gradient(self, node, g):
        return [pad_gradient_op(g, node.attrs["paddings"], node.attrs["mode"])]

    def infer_shape(self, node, s):
        pads = self._full(node, len(s[0]))
        return tuple(d + p[0] + p[1] for d, p in zip(s[0], pads))


class PadGradientOp(Op):
    name, cheap = "PadGradient", True

    def __call__(self, g, paddings, mode="CONSTANT"):
        return Op.__call__(self, g, paddings=[tuple(p) for p in paddings], mode=mode)

    def _full(self, node, ndim):
        p = node.attrs["paddings"]
        return [(0, 0)] * (ndim - len(p)) + list(p)

    def np_compute(self, node, iv):
        pads = self._full(node, iv[0].ndim)
        return iv[0][tuple(slice(p[0], d - p[1]) for p, d in zip(pads, iv[0].shape))]

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        pads = self._full(node, iv[0].ndim)
        if not cpu_links.ok(iv[0], out) or iv[0].ndim < 2 or any(p != (0, 0) for p in pads[:-2]):
            return False
        cpu_links.pad2d(out, iv[0], pads[-2], pads[-1], grad=True)
        return True

    def gpu_compute(self, node, iv, out, stream):
        g = iv[0]
        pads = self._full(node, len(g.shape))
        off = sum(p[0] * st for p, st in zip(pads, g.strides))
        G.copy_raw(g.ptr + 4 * off, g.strides, out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        raise NotImplementedError

    def infer_shape(self, node, s):
        pads = self._full(node, len(s[0]))
        return tuple(d - p[0] - p[1] for d, p in zip(s[0], pads))


# -- broadcasts -------------------------------------------------------------------------------
def _bcast_strides(in_shape, in_strides, out_shape, add_axes=None):
    """Strides of the input seen through the output's index space."""
    nd = len(out_shape)
    if add_axes:
        if list(in_shape) == [1] and nd - len(add_axes) != 1:
            return [0] * nd
        st, j = [], 0
        for i in range(nd):
            if i in add_axes:
                st.append(0)
            else:
                st.append(in_strides[j] if in_shape[j] != 1 else 0)
                j += 1
        return st
    diff = nd - len(in_shape)
    return [0] * diff + [in_strides[i] if in_shape[i] != 1 else 0 for i in range(len(in_shape))]


class BroadcastToOp(Op):
    """Prepend/tile leading dims: out[i, ...] = in[...] (reference
    ``Broadcast.cu:4-8``: ``out[i] = in[i % in_size]``)."""
    name, cheap = "BroadcastTo", True

    def __call__(self, x, like):
        return Op.__call__(self, x, like)

    def np_compute(self, node, iv):
        return np.broadcast_to(iv[0], iv[1].shape)

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        x = iv[0]
        # the native kernel tiles the whole input along new leading dimensions (the reference's form)
        if not cpu_links.ok(x, out) or x.size == 0 or tuple(out.shape[out.ndim - x.ndim:]) != tuple(x.shape):
            return False
        cpu_links.broadcast_rows(x, out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.copy_raw(x.ptr, _bcast_strides(x.shape, x.strides, out.shape), out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        return [reducesumaxiszero_op(g), None]

    def infer_shape(self, node, s):
        return tuple(s[1])


class BroadcastShapeOp(Op):
    name, cheap = "BroadcastShape", True

    def __call__(self, x, shape, add_axes=None):
        return Op.__call__(self, x, shape=None if shape is None else tuple(shape),
                           add_axes=None if add_axes is None else list(add_axes), grad_node=None)

    def np_compute(self, node, iv):
        shape, add = node.attrs["shape"], node.attrs["add_axes"]
        ishape = list(shape)
        x = iv[0]
        if add:
            if x.size == 1:
                return np.broadcast_to(x.reshape([1] * len(shape)), shape)
            ishape = [1 if i in add else d for i, d in enumerate(shape)]
            return np.broadcast_to(x.reshape(ishape), shape)
        return np.broadcast_to(x, shape)

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.copy_raw(x.ptr, _bcast_strides(x.shape, x.strides, out.shape, node.attrs["add_axes"]),
                   out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        gn = reduce_sum_op(g, None, None)
        node.attrs["grad_node"] = gn
        return [gn]

    def infer_shape(self, node, s):
        shape, add = node.attrs["shape"], node.attrs["add_axes"]
        assert shape is not None
        in_shape = list(s[0])
        diff = len(shape) - len(in_shape)
        if add:
            axes, keep = list(add), [False] * len(add)
        else:
            axes, keep = list(range(diff)), [False] * diff
            padded = [1] * diff + in_shape
            for i in range(diff, len(shape)):
                assert padded[i] in (1, shape[i])
                if padded[i] == 1 and shape[i] > 1:
                    axes.append(i)
                    keep.append(True)
        gn = node.attrs.get("grad_node")
        if gn is not None:
            gn.attrs["axes"], gn.attrs["keepdims"] = axes, keep
        return tuple(shape)


class BroadcastToTFOp(Op):
    """NumPy-style broadcast of A to the shape of B."""
    name, cheap = "BroadcastToTF", True

    def __call__(self, a, b):
        return Op.__call__(self, a, b, grad_node=None)

    def np_compute(self, node, iv):
        return np.broadcast_to(iv[0], iv[1].shape)

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.copy_raw(x.ptr, _bcast_strides(x.shape, x.strides, out.shape), out.ptr, out.strides, out.shape, stream)

    def gradient(self, node, g):
        gn = reduce_sum_op(g, None, None)
        node.attrs["grad_node"] = gn
        return [gn, None]

    def infer_shape(self, node, s):
        in_shape, shape = list(s[0]), list(s[1])
        diff = len(shape) - len(in_shape)
        axes, keep = list(range(diff)), [False] * diff
        padded = [1] * diff + in_shape
        for i in range(diff, len(shape)):
            assert padded[i] in (1, shape[i])
            if padded[i] == 1 and shape[i] > 1:
                axes.append(i)
                keep.append(True)
        gn = node.attrs.get("grad_node")
        if gn is not None:
            gn.attrs["axes"], gn.attrs["keepdims"] = axes, keep
        return tuple(shape)


class AddBroadcastOp(Op):
    """``x + broadcast(b)`` in one kernel.  ``add_op`` builds it for ``x + broadcasttoTF_op(b, x)`` (the
    bias of a dense layer, an attention mask), so the broadcast is never materialised."""
    name, cheap = "AddBroadcast", True

    def __call__(self, x, b):
        return Op.__call__(self, x, b, grad_node=None)

    def np_compute(self, node, iv):
        return (iv[0] + np.broadcast_to(iv[1], iv[0].shape)).astype(np.float32)

    def gpu_compute(self, node, iv, out, stream):
        x, b = iv
        G.add_broadcast(x, b, _bcast_strides(b.shape, b.strides, out.shape), out, stream)

    def gradient(self, node, g):
        gn = reduce_sum_op(g, None, None)
        node.attrs["grad_node"] = gn
        return [g, gn]

    def infer_shape(self, node, s):
        shape, in_shape = list(s[0]), list(s[1])
        diff = len(shape) - len(in_shape)
        assert diff >= 0, "AddBroadcast: %s does not broadcast to %s" % (in_shape, shape)
        axes, keep = list(range(diff)), [False] * diff
        padded = [1] * diff + in_shape
        for i in range(diff, len(shape)):
            assert padded[i] in (1, shape[i])
            if padded[i] == 1 and shape[i] > 1:
                axes.append(i)
                keep.append(True)
        gn = node.attrs.get("grad_node")
        if gn is not None:
            gn.attrs["axes"], gn.attrs["keepdims"] = axes, keep
        return tuple(shape)


# -- reductions ---------------------------------------------------------------------------------
class ReduceSumOp(Op):
    name = "ReduceSum"

    def __call__(self, x, axes, keepdims=False):
        if axes is not None:
            axes = [axes] if isinstance(axes, int) else list(axes)
            if keepdims is True or keepdims is False:
                keepdims = [keepdims] * len(axes)
            else:
                keepdims = list(keepdims)
                assert len(keepdims) == len(axes)
        return Op.__call__(self, x, axes=axes, keepdims=keepdims, grad_node=None)

    def _out_shape(self, node, in_shape):
        axes, keep = node.attrs["axes"], node.attrs["keepdims"]
        assert axes is not None and keep is not None, "reduce_sum axes not resolved"
        shape = list(in_shape)
        for a, k in zip(axes, keep):
            shape[a % len(in_shape)] = 1 if k else 0
        shape = [d for d in shape if d > 0]
        return tuple(shape) if shape else (1,)

    def np_compute(self, node, iv):
        x = iv[0]
        axes = tuple(a % x.ndim for a in node.attrs["axes"])
        return x.sum(axis=axes).reshape(self._out_shape(node, x.shape))

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.reduce_sum(x.ptr, list(x.shape), list(x.strides), node.attrs["axes"], out, stream)

    def gradient(self, node, g):
        gn = broadcast_shape_op(g, None)
        node.attrs["grad_node"] = gn
        return [gn]

    def infer_shape(self, node, s):
        in_shape = list(s[0])
        axes, keep = node.attrs["axes"], node.attrs["keepdims"]
        gn = node.attrs.get("grad_node")
        if gn is not None:
            gn.attrs["shape"] = tuple(in_shape)
            gn.attrs["add_axes"] = [a % len(in_shape) for a, k in zip(axes, keep) if not k] or None
            if gn.attrs["add_axes"] is None and len(self._out_shape(node, in_shape)) != len(in_shape):
                gn.attrs["add_axes"] = [a % len(in_shape) for a in axes]
        return self._out_shape(node, in_shape)


class ReduceSumAxisZeroOp(Op):
    name = "ReduceSumAxisZero"

    def __call__(self, x):
        return Op.__call__(self, x)

    def np_compute(self, node, iv):
        r = iv[0].sum(axis=0)
        return r.reshape((1,)) if r.ndim == 0 else r

    def cpu_compute(self, node, iv, out):
        from .. import cpu_links
        if not cpu_links.ok(iv[0], out) or iv[0].ndim < 1:
            return False
        cpu_links.reduce_sum_axis_zero(iv[0], out)
        return True

    def gpu_compute(self, node, iv, out, stream):
        x = iv[0]
        G.reduce_sum(x.ptr, list(x.shape), list(x.strides), [0], out, stream)

    def gradient(self, node, g):
        return [broadcastto_op(g, node.inputs[0])]

    def infer_shape(self, node, s):
        return tuple(s[0][1:]) if len(s[0]) > 1 else (1,)


_reshape, _reshape_g, _transpose = ReshapeOp(), ReshapeGradientOp(), TransposeOp()
_slice, _slice_g, _concat, _concat_g, _pad, _pad_g = (SliceOp(), SliceGradientOp(), ConcatOp(),
                                                      ConcatGradientOp(), PadOp(), PadGradientOp())
_bto, _bshape, _btf, _rsum, _rsum0 = (BroadcastToOp(), BroadcastShapeOp(), BroadcastToTFOp(), ReduceSumOp(),
                                      ReduceSumAxisZeroOp())
_addb = AddBroadcastOp()


def array_reshape_op(node, output_shape):
    return _reshape(node, output_shape)


def array_reshape_gradient_op(node_in, node_out):
    return _reshape_g(node_in, node_out)


def transpose_op(node_A, perm=None):
    return _transpose(node_A, perm)


def slice_op(node, begin, size):
    return _slice(node, begin, size)


def slice_gradient_op(node, begin, size, like=None, output_shape=None):
    return _slice_g(node, begin, size, like, output_shape)


def concat_op(node_A, node_B, axis=0):
    return _concat(node_A, node_B, axis)


def concat_gradient_op(grad_node, input_node, axis, idx):
    return _concat_g(grad_node, input_node, axis, idx)


def pad_op(node_A, paddings, mode="CONSTANT", constant_values=0):
    return _pad(node_A, paddings, mode, constant_values)


def pad_gradient_op(node_A, paddings, mode="CONSTANT"):
    return _pad_g(node_A, paddings, mode)


def broadcastto_op(node_A, node_B):
    return _bto(node_A, node_B)


def broadcast_shape_op(node_A, shape, add_axes=None):
    return _bshape(node_A, shape, add_axes)


def broadcasttoTF_op(node_A, node_B):
    return _btf(node_A, node_B)


def add_broadcast_op(node_x, node_b):
    return _addb(node_x, node_b)


def reduce_sum_op(node, axes, keepdims=False):
    return _rsum(node, axes, keepdims)


def reducesumaxiszero_op(node):
    return _rsum0(node)
