"""Python entry points of the hand-written sm_100a kernel library.

One thin function per C entry of ``libtsplit_kernels.so`` (the role the
reference's ``python/athena/gpu_links/*.py`` plays for ``libc_runtime_api.so``):
checks types, passes raw device pointers, logical shapes, element strides and
the ``cudaStream_t``.  Every kernel accepts strided operands, so channels-last
arrays and channel-dimension micro-tensors need no packing.

There is no fallback: on a CUDA context a missing library is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_int64, c_float

from .. import _base

# unary codes
(UN_COPY, UN_RELU, UN_SIGMOID, UN_TANH, UN_SQRT, UN_RSQRT, UN_NEG, UN_ADDC, UN_MULC, UN_CDIV,
 UN_FILL) = range(11)
# binary codes
BIN_ADD, BIN_MUL, BIN_DIV, BIN_RELU_GRAD, BIN_SUB, BIN_ADD_RELU, BIN_RELU_GRAD_OUT = range(7)

MAX_DIMS = 8
_I64x8 = c_int64 * MAX_DIMS


def lib():
    return _base.kernels()


def _s(stream):
    return c_void_p(stream.handle if stream is not None else 0)


def _p(arr):
    return c_void_p(arr.ptr)


def _check(rc, what):
    if rc != 0:
        raise RuntimeError("%s failed: %s" % (what, _base.error_string(rc)))


def _vec(vals):
    v = list(vals) + [0] * (MAX_DIMS - len(vals))
    return _I64x8(*v)


def _numel(shape):
    n = 1
    for s in shape:
        n *= s
    return n


def _flat_ok(*arrs):
    """All operands dense with identical shape and strides -> treat as 1-D."""
    a0 = arrs[0]
    if not a0.is_dense():
        return False
    return all(a.same_layout(a0) for a in arrs[1:])


def _collapse(shape, *strides_list):
    """Drop size-1 dims and merge adjacent dims that are contiguous in every
    operand; returns (shape, [strides...])."""
    dims = [i for i, s in enumerate(shape) if s != 1]
    if not dims:
        return [1], [[1] for _ in strides_list]
    shp = [shape[i] for i in dims]
    sts = [[st[i] for i in dims] for st in strides_list]
    out_shape, out_sts = [shp[0]], [[st[0]] for st in sts]
    for k in range(1, len(shp)):
        if all(o[-1] == st[k] * shp[k] for o, st in zip(out_sts, sts)):
            out_shape[-1] *= shp[k]
            for o, st in zip(out_sts, sts):
                o[-1] = st[k]
        else:
            out_shape.append(shp[k])
            for o, st in zip(out_sts, sts):
                o.append(st[k])
    return out_shape, out_sts


# ---------------------------------------------------------------------------
def unary(code, x, y, stream, alpha=0.0):
    if _flat_ok(x, y):
        rc = lib().tsb_ew_unary(c_int(code), _p(x), _p(y), c_int64(_numel(x.shape)),
                                c_float(alpha), _s(stream))
    else:
        shape, (xs, ys) = _collapse(list(y.shape), list(x.strides), list(y.strides))
        rc = lib().tsb_strided_unary(c_int(code), _p(x), _p(y), c_int(len(shape)), _vec(shape),
                                     _vec(xs), _vec(ys), c_float(alpha), _s(stream))
    _check(rc, "unary")


def fill(y, value, stream):
    if y.is_dense():
        rc = lib().tsb_ew_unary(c_int(UN_FILL), _p(y), _p(y), c_int64(_numel(y.shape)),
                                c_float(value), _s(stream))
        _check(rc, "fill")
    else:
        unary(UN_FILL, y, y, stream, alpha=value)


def copy(x, y, stream):
    """y <- x with arbitrary strides on both sides (same logical shape)."""
    unary(UN_COPY, x, y, stream)


def memcpy_async(dst_ptr, src_ptr, nbytes, stream):
    """Byte copy between device memory and pinned host memory on ``stream`` (the swap path)."""
    rc = lib().tsb_memcpy_async(c_void_p(dst_ptr), c_void_p(src_ptr), ctypes.c_longlong(nbytes), _s(stream))
    _check(rc, "memcpy_async")


def copy_raw(x_ptr, x_strides, y_ptr, y_strides, shape, stream):
    shape, (xs, ys) = _collapse(list(shape), list(x_strides), list(y_strides))
    rc = lib().tsb_strided_unary(c_int(UN_COPY), c_void_p(x_ptr), c_void_p(y_ptr), c_int(len(shape)),
                                 _vec(shape), _vec(xs), _vec(ys), c_float(0.0), _s(stream))
    _check(rc, "copy_raw")


def binary(code, a, b, y, stream):
    if _flat_ok(a, b, y):
        rc = lib().tsb_ew_binary(c_int(code), _p(a), _p(b), _p(y), c_int64(_numel(y.shape)), _s(stream))
    else:
        assert a.shape == b.shape == y.shape
        shape, (sa, sb, sy) = _collapse(list(y.shape), list(a.strides), list(b.strides), list(y.strides))
        rc = lib().tsb_strided_binary(c_int(code), _p(a), _p(b), _p(y), c_int(len(shape)), _vec(shape),
                                      _vec(sa), _vec(sb), _vec(sy), _s(stream))
    _check(rc, "binary")


def add_broadcast(x, b, b_strides, y, stream):
    """y <- x + b, b seen through ``b_strides`` (zeros where it is broadcast) in y's index space."""
    cols = y.shape[-1]
    if (x.is_contiguous() and y.is_contiguous() and cols % 4 == 0 and b_strides[-1] == 1
            and all(s == 0 for s in b_strides[:-1])):
        rc = lib().tsb_bias_add(_p(x), _p(b), _p(y), c_int64(_numel(y.shape) // cols), c_int64(cols), _s(stream))
        if rc == 0:
            return
        if rc != 2:      # 2: operands not 16-byte aligned, take the strided kernel
            _check(rc, "bias_add")
    binary_bcast(BIN_ADD, x.ptr, x.strides, b.ptr, b_strides, y, stream)


def binary_bcast(code, a_ptr, a_strides, b_ptr, b_strides, y, stream):
    """Binary op where operand strides (possibly 0) are given for y's shape."""
    shape, (sa, sb, sy) = _collapse(list(y.shape), list(a_strides), list(b_strides), list(y.strides))
    rc = lib().tsb_strided_binary(c_int(code), c_void_p(a_ptr), c_void_p(b_ptr), _p(y), c_int(len(shape)),
                                  _vec(shape), _vec(sa), _vec(sb), _vec(sy), _s(stream))
    _check(rc, "binary_bcast")


def binary_dev_scalar(code, a, scalar, y, stream, scalar_first=False):
    """``a (op) scalar[0]`` with the scalar read on the device (stride-0 operand)."""
    zero = [0] * len(y.shape)
    if scalar_first:
        binary_bcast(code, scalar.ptr, zero, a.ptr, a.strides, y, stream)
    else:
        binary_bcast(code, a.ptr, a.strides, scalar.ptr, zero, y, stream)


def where(c, a, b, y, stream):
    assert _flat_ok(c, a, b, y), "where: operands must share one dense layout"
    _check(lib().tsb_where(_p(c), _p(a), _p(b), _p(y), c_int64(_numel(y.shape)), _s(stream)), "where")


def reduce_sum(x_ptr, x_shape, x_strides, axes, y, stream):
    """y[keep...] = sum over ``axes`` of x.  ``y`` has the kept dims in order."""
    axes = sorted(a % len(x_shape) for a in axes)
    keep = [i for i in range(len(x_shape)) if i not in axes and x_shape[i] != 1]
    kshape = [x_shape[i] for i in keep] or [1]
    kxs = [x_strides[i] for i in keep] or [0]
    # y holds the kept dims in order, possibly with extra size-1 dims
    ydims = [(s, st) for s, st in zip(y.shape, y.strides) if s != 1]
    assert [d[0] for d in ydims] == [x_shape[i] for i in keep], "reduce_sum: output shape mismatch"
    ys = [d[1] for d in ydims] or [0]
    rshape = [x_shape[i] for i in axes] or [1]
    rxs = [x_strides[i] for i in axes] or [0]
    rc = lib().tsb_reduce_sum(c_void_p(x_ptr), _p(y), c_int(len(kshape)), _vec(kshape), _vec(kxs), _vec(ys),
                              c_int(len(rshape)), _vec(rshape), _vec(rxs), _s(stream))
    _check(rc, "reduce_sum")


def softmax(x, y, stream):
    rows, cols = _numel(x.shape[:-1]), x.shape[-1]
    _check(lib().tsb_softmax(_p(x), _p(y), c_int64(rows), c_int64(cols), _s(stream)), "softmax")


def softmax_grad(y, dy, dx, stream):
    rows, cols = _numel(y.shape[:-1]), y.shape[-1]
    _check(lib().tsb_softmax_grad(_p(y), _p(dy), _p(dx), c_int64(rows), c_int64(cols), _s(stream)),
           "softmax_grad")


def masked_softmax(x, key_tokens, y, scale, causal, stream):
    """y = softmax(scale * x + padding mask [+ causal mask]) over the last axis of x [N, H, Tq, Tk]."""
    n, h, tq, tk = x.shape
    rc = lib().tsb_masked_softmax(_p(x), c_void_p(key_tokens.ptr if key_tokens is not None else 0), _p(y),
                                  c_int64(n * h * tq), c_int64(tk), c_int64(h * tq), c_int(tq), c_float(scale),
                                  c_int(int(causal)), _s(stream))
    _check(rc, "masked_softmax")


def scaled_softmax_grad(y, dy, dx, scale, stream):
    rows, cols = _numel(y.shape[:-1]), y.shape[-1]
    _check(lib().tsb_scaled_softmax_grad(_p(y), _p(dy), _p(dx), c_int64(rows), c_int64(cols), c_float(scale),
                                         _s(stream)), "scaled_softmax_grad")


def softmax_ce(logits, labels, loss, stream):
    rows, cols = logits.shape
    _check(lib().tsb_softmax_ce(_p(logits), _p(labels), _p(loss), c_int64(rows), c_int64(cols),
                                _s(stream)), "softmax_ce")


def softmax_ce_grad(logits, labels, g, dx, stream):
    rows, cols = logits.shape
    _check(lib().tsb_softmax_ce_grad(_p(logits), _p(labels), _p(g), _p(dx), c_int64(rows), c_int64(cols),
                                     _s(stream)), "softmax_ce_grad")


def one_hot(idx, y, num_classes, stream):
    _check(lib().tsb_one_hot(_p(idx), _p(y), c_int64(_numel(idx.shape)), c_int64(num_classes), _s(stream)),
           "one_hot")


def embedding(table, idx, y, stream):
    _check(lib().tsb_embedding(_p(table), _p(idx), _p(y), c_int64(_numel(idx.shape)),
                               c_int64(table.shape[0]), c_int64(table.shape[1]), _s(stream)), "embedding")


def embedding_grad(g, idx, dtable, stream):
    _check(lib().tsb_embedding_grad(_p(g), _p(idx), _p(dtable), c_int64(_numel(idx.shape)),
                                    c_int64(dtable.shape[0]), c_int64(dtable.shape[1]), _s(stream)),
           "embedding_grad")


def dropout(x, y, keep_prob, seed, stream, step_dev=0, offset=0):
    """``step_dev``: device address of the executor's step counter (0 = ``seed`` is already step-mixed);
    ``offset``: index of ``x``'s first element in the whole tensor when ``x`` is a batch piece of it."""
    _check(lib().tsb_dropout(_p(x), _p(y), c_int64(_numel(x.shape)), c_float(keep_prob),
                             ctypes.c_uint64(seed), c_void_p(step_dev or None), ctypes.c_uint64(offset),
                             _s(stream)), "dropout")


def step_advance(step_dev, stream):
    _check(lib().tsb_step_advance(c_void_p(step_dev), _s(stream)), "step_advance")


# -- normalisation ------------------------------------------------------------
def _rows_c(x):
    """(rows, C, row stride) of a channels-last 4-D array or a 2-D array."""
    if len(x.shape) == 4:
        n, c, h, w = x.shape
        st = x.strides
        assert st[1] == 1 and st[3] >= c and st[2] == w * st[3] and st[0] == h * st[2], \
            "batch-norm kernels need a channels-last (possibly channel-sliced) operand"
        return n * h * w, c, st[3]
    r, c = x.shape
    assert x.strides[1] == 1
    return r, c, x.strides[0]


def bn_forward(x, scale, bias, y, save_mean, save_invstd, run_mean, run_var, momentum, eps, relu, stream):
    rows, c, ldx = _rows_c(x)
    _, _, ldy = _rows_c(y)
    _check(lib().tsb_bn_forward(_p(x), _p(scale), _p(bias), _p(y), _p(save_mean), _p(save_invstd),
                                _p(run_mean), _p(run_var), c_int64(rows), c_int64(c), c_int64(ldx),
                                c_int64(ldy), c_float(momentum), c_float(eps), c_int(int(relu)),
                                _s(stream)), "bn_forward")


def bn_backward(dy, x, scale, save_mean, save_invstd, dx, dscale, dbias, stream):
    rows, c, ldx = _rows_c(x)
    _, _, lddy = _rows_c(dy)
    _, _, lddx = _rows_c(dx)
    _check(lib().tsb_bn_backward(_p(dy), _p(x), _p(scale), _p(save_mean), _p(save_invstd), _p(dx),
                                 _p(dscale), _p(dbias), c_int64(rows), c_int64(c), c_int64(ldx),
                                 c_int64(lddy), c_int64(lddx), _s(stream)), "bn_backward")


def bn_apply(x, scale, bias, y, save_mean, save_invstd, relu, stream):
    """Normalise with known statistics (rematerialisation of a batch-norm output)."""
    rows, c, ldx = _rows_c(x)
    _, _, ldy = _rows_c(y)
    _check(lib().tsb_bn_apply(_p(x), _p(scale), _p(bias), _p(y), _p(save_mean), _p(save_invstd), c_int64(rows),
                              c_int64(c), c_int64(ldx), c_int64(ldy), c_int(int(relu)), _s(stream)), "bn_apply")


def bn_relu_backward(dy, x, scale, bias, save_mean, save_invstd, dx, dscale, dbias, stream):
    rows, c, ldx = _rows_c(x)
    _, _, lddy = _rows_c(dy)
    _, _, lddx = _rows_c(dx)
    _check(lib().tsb_bn_relu_backward(_p(dy), _p(x), _p(scale), _p(bias), _p(save_mean), _p(save_invstd), _p(dx),
                                      _p(dscale), _p(dbias), c_int64(rows), c_int64(c), c_int64(ldx),
                                      c_int64(lddy), c_int64(lddx), _s(stream)), "bn_relu_backward")


BN_PIECE_CHUNKS = 256      # chunk rows a batch piece may fill in a piece-wise statistics buffer


def bn_stats_partial(x, part, plane, chunk_offset, stream):
    """Column sums / sums of squares of one batch piece into ``part`` (two planes of ``plane`` floats);
    returns the number of chunk rows written from ``chunk_offset`` on."""
    rows, c, ldx = _rows_c(x)
    n = c_int(0)
    _check(lib().tsb_bn_stats_partial(_p(x), _p(part), c_int64(plane), c_int(chunk_offset), c_int(BN_PIECE_CHUNKS),
                                      c_int64(rows), c_int64(c), c_int64(ldx), ctypes.byref(n), _s(stream)),
           "bn_stats_partial")
    return int(n.value)


def bn_stats_finalize(part, plane, chunks, count, c, eps, momentum, mean, invstd, run_mean, run_var, stream):
    _check(lib().tsb_bn_stats_finalize(_p(part), c_int64(plane), c_int(chunks), ctypes.c_double(count), c_int64(c),
                                       c_float(eps), c_float(momentum), _p(mean), _p(invstd), _p(run_mean),
                                       _p(run_var), _s(stream)), "bn_stats_finalize")


def bn_bwd_partial(dy, x, mean, invstd, rscale, rbias, part, plane, chunk_offset, stream):
    rows, c, ldx = _rows_c(x)
    _, _, lddy = _rows_c(dy)
    n = c_int(0)
    _check(lib().tsb_bn_bwd_partial(_p(dy), _p(x), _p(mean), _p(invstd),
                                    c_void_p(rscale.ptr if rscale is not None else 0),
                                    c_void_p(rbias.ptr if rbias is not None else 0), _p(part), c_int64(plane),
                                    c_int(chunk_offset), c_int(BN_PIECE_CHUNKS), c_int64(rows), c_int64(c),
                                    c_int64(lddy), c_int64(ldx), ctypes.byref(n), _s(stream)), "bn_bwd_partial")
    return int(n.value)


def bn_bwd_finalize(part, plane, chunks, c, dscale, dbias, stream):
    _check(lib().tsb_bn_bwd_finalize(_p(part), c_int64(plane), c_int(chunks), c_int64(c), _p(dscale), _p(dbias),
                                     _s(stream)), "bn_bwd_finalize")


def bn_bwd_apply(dy, x, scale, rbias, mean, invstd, dscale, dbias, dx, total_rows, stream):
    rows, c, ldx = _rows_c(x)
    _, _, lddy = _rows_c(dy)
    _, _, lddx = _rows_c(dx)
    _check(lib().tsb_bn_bwd_apply(_p(dy), _p(x), _p(scale), c_void_p(rbias.ptr if rbias is not None else 0),
                                  _p(mean), _p(invstd), _p(dscale), _p(dbias), _p(dx), c_int64(rows), c_int64(c),
                                  c_int64(lddy), c_int64(ldx), c_int64(lddx), ctypes.c_double(total_rows),
                                  _s(stream)), "bn_bwd_apply")


def layer_norm(x, scale, bias, y, mean, invstd, eps, stream):
    rows, cols = _numel(x.shape[:-1]), x.shape[-1]
    _check(lib().tsb_layer_norm(_p(x), _p(scale), _p(bias), _p(y), _p(mean), _p(invstd), c_int64(rows),
                                c_int64(cols), c_float(eps), _s(stream)), "layer_norm")


def layer_norm_grad(dy, x, scale, mean, invstd, dx, dscale, dbias, stream):
    rows, cols = _numel(x.shape[:-1]), x.shape[-1]
    _check(lib().tsb_layer_norm_grad(_p(dy), _p(x), _p(scale), _p(mean), _p(invstd), _p(dx), _p(dscale),
                                     _p(dbias), c_int64(rows), c_int64(cols), _s(stream)), "layer_norm_grad")


# -- pooling (channels-last) ------------------------------------------------------
def _nhwc(x):
    n, c, h, w = x.shape
    st = x.strides
    assert st[1] == 1, "pooling kernels need a channels-last operand"
    return n, c, h, w, st[0], st[2], st[3]


def pool(kind, x, y, kh, kw, pad, stride, stream):
    """kind: 0 = max, 1 = average (count includes padding)."""
    n, c, h, w, xsn, xsh, xsw = _nhwc(x)
    _, _, oh, ow, ysn, ysh, ysw = _nhwc(y)
    _check(lib().tsb_pool_fwd(c_int(kind), _p(x), _p(y), c_int(n), c_int(c), c_int(h), c_int(w), c_int(oh),
                              c_int(ow), c_int(kh), c_int(kw), c_int(pad), c_int(stride),
                              c_int64(xsn), c_int64(xsh), c_int64(xsw), c_int64(ysn), c_int64(ysh),
                              c_int64(ysw), _s(stream)), "pool_fwd")


def pool_grad(kind, x, y, dy, dx, kh, kw, pad, stride, stream):
    n, c, h, w, xsn, xsh, xsw = _nhwc(dx)
    _, _, oh, ow, ysn, ysh, ysw = _nhwc(dy)
    assert x is None or (x.same_layout(dx) and y.same_layout(dy))
    _check(lib().tsb_pool_bwd(c_int(kind), c_void_p(x.ptr if x is not None else 0),
                              c_void_p(y.ptr if y is not None else 0), _p(dy), _p(dx),
                              c_int(n), c_int(c), c_int(h), c_int(w), c_int(oh), c_int(ow), c_int(kh),
                              c_int(kw), c_int(pad), c_int(stride), c_int64(xsn), c_int64(xsh),
                              c_int64(xsw), c_int64(ysn), c_int64(ysh), c_int64(ysw), _s(stream)),
           "pool_bwd")


# -- tensor-core contractions -------------------------------------------------------
def gemm(a, b, c, trans_a, trans_b, stream, batch=1, sa=0, sb=0, sc=0, m=None, n=None, k=None,
         lda=None, ldb=None, ldc=None, accumulate=False, heads=0, head_mask=0):
    """C[m,n] (+)= op(A)·op(B), row-major operands, TF32 tensor cores
    (tcgen05, fp32 accumulate in TMEM).  ``heads`` / ``head_mask`` (bit 0 A, 1 B, 2 C): that operand is in head
    layout ``[outer][row][head][col]`` and is given with its head stride as batch stride."""
    if head_mask:
        rc = lib().tsb_gemm_tf32_heads(_p(a), _p(b), _p(c), c_int(m), c_int(n), c_int(k), c_int64(lda),
                                       c_int64(ldb), c_int64(ldc), c_int(int(trans_a)), c_int(int(trans_b)),
                                       c_int(batch), c_int64(sa), c_int64(sb), c_int64(sc),
                                       c_int(int(accumulate)), c_int(heads), c_int(head_mask), _s(stream))
        _check(rc, "gemm_tf32_heads")
        return
    rc = lib().tsb_gemm_tf32(_p(a), _p(b), _p(c), c_int(m), c_int(n), c_int(k), c_int64(lda),
                             c_int64(ldb), c_int64(ldc), c_int(int(trans_a)), c_int(int(trans_b)),
                             c_int(batch), c_int64(sa), c_int64(sb), c_int64(sc),
                             c_int(int(accumulate)), _s(stream))
    _check(rc, "gemm_tf32")


def conv2d(kind, x, w, y, ph, pw, stride, stream):
    """kind 0: y = conv(x, w); 1: x(dx) = dgrad(y(dy), w); 2: w(dw) = wgrad(x, y(dy)).
    All operands channels-last; logical shapes x[N,C,H,W], w[O,C,KH,KW], y[N,O,OH,OW]."""
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    _, _, oh, ow = y.shape
    # inputs that arrive row-major (e.g. straight out of a transpose) are re-laid-out once
    if kind != 1 and not x.is_channels_last():
        x = _as_channels_last(x, "cl_x", stream)
    if kind != 2 and not w.is_channels_last():
        w = _as_channels_last(w, "cl_w", stream)
    if kind != 0 and not y.is_channels_last():
        y = _as_channels_last(y, "cl_y", stream)
    assert x.is_channels_last() and w.is_channels_last() and y.is_channels_last(), \
        "conv kernels need dense channels-last operands"
    if c % 4:
        return _conv2d_padded_channels(kind, x, w, y, ph, pw, stride, stream)
    rc = lib().tsb_conv2d(c_int(kind), _p(x), _p(w), _p(y), c_int(n), c_int(c), c_int(h), c_int(wd),
                          c_int(o), c_int(kh), c_int(kw), c_int(oh), c_int(ow), c_int(ph), c_int(pw),
                          c_int(stride), _s(stream))
    _check(rc, "conv2d kind %d" % kind)


CONV_STAT_MAX_CHUNKS = 304      # upper bound of per-CTA partial-sum slots a forward convolution may fill


def conv2d_fwd_stats(x, w, y, ph, pw, stride, part, stream, chunk_offset=0, plane=None, max_chunks=None):
    """Forward convolution that also leaves per-CTA column sums / sums of squares of ``y`` in
    ``part`` (flat array of 2 * CONV_STAT_MAX_CHUNKS * O floats) for the batch norm that follows.
    Returns the number of chunks written; 0 = no statistics (the plain kernel ran).
    ``chunk_offset`` / ``plane`` / ``max_chunks``: write the chunk rows from that row on into a buffer whose two
    planes are ``plane`` floats apart and that has room for ``max_chunks`` more rows (the piece-wise statistics
    buffer of a batch norm whose input is computed piece by piece)."""
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    _, _, oh, ow = y.shape
    if c % 4 or not (x.is_channels_last() and w.is_channels_last() and y.is_channels_last()):
        conv2d(0, x, w, y, ph, pw, stride, stream)
        return 0
    chunks = c_int(0)
    rc = lib().tsb_conv2d_fwd_stats(_p(x), _p(w), _p(y), c_int(n), c_int(c), c_int(h), c_int(wd), c_int(o),
                                    c_int(kh), c_int(kw), c_int(oh), c_int(ow), c_int(ph), c_int(pw),
                                    c_int(stride), c_void_p(part.ptr + 4 * int(chunk_offset) * o),
                                    c_int64(CONV_STAT_MAX_CHUNKS * o if plane is None else plane),
                                    c_int(CONV_STAT_MAX_CHUNKS if max_chunks is None else max_chunks),
                                    ctypes.byref(chunks), _s(stream))
    _check(rc, "conv2d_fwd_stats")
    return int(chunks.value)


def bn_forward_from_partials(part, chunks, x, scale, bias, y, save_mean, save_invstd, run_mean, run_var, momentum,
                             eps, relu, stream):
    rows, c, ldx = _rows_c(x)
    _, _, ldy = _rows_c(y)
    _check(lib().tsb_bn_forward_from_partials(_p(part), c_int(chunks), c_int64(CONV_STAT_MAX_CHUNKS * c), _p(x),
                                              _p(scale), _p(bias), _p(y), _p(save_mean), _p(save_invstd),
                                              _p(run_mean), _p(run_var), c_int64(rows), c_int64(c), c_int64(ldx),
                                              c_int64(ldy), c_float(momentum), c_float(eps), c_int(int(relu)),
                                              _s(stream)), "bn_forward_from_partials")


_PAD_CACHE = {}


def _as_channels_last(arr, tag, stream):
    from .. import ndarray
    key = (tag, arr.shape, arr.ctx.device_id)
    buf = _PAD_CACHE.get(key)
    if buf is None:
        buf = _PAD_CACHE[key] = ndarray.empty(arr.shape, arr.ctx, use_pool=False, channels_last=True)
    copy(arr, buf, stream)
    return buf


def _padded(arr, c4, tag):
    """Cached channels-last scratch with the channel count rounded up to a
    multiple of 4 (the gather moves 16-byte pieces).  The padding lanes are
    zeroed once at creation; every use rewrites only the real channels."""
    from .. import ndarray
    shape = (arr.shape[0], c4, arr.shape[2], arr.shape[3])
    key = (tag, shape, arr.ctx.device_id)
    buf = _PAD_CACHE.get(key)
    if buf is None:
        buf = ndarray.empty(shape, arr.ctx, use_pool=False)
        buf.t.zero_()
        _PAD_CACHE[key] = buf
    return buf


def _conv2d_padded_channels(kind, x, w, y, ph, pw, stride, stream):
    """Input-channel count not a multiple of 4 (the RGB stem): run the kernel on
    zero-padded copies of x and w; only the real channels are copied back.

    Stride-1 "same" convolutions with at most 4 channels take the packed route
    instead: eight pixels of a row are read as one pixel with 32 channels (same
    memory), which turns the stem into an ordinary 32 -> 8*O channel convolution
    for the TMA kernels (see ``stem_pack_filters`` in the kernel source)."""
    c = x.shape[1]
    c4 = (c + 3) // 4 * 4
    if kind in (0, 2) and _packed_stem_ok(x, w, y, c4, pw, stride):
        return _conv2d_packed_stem(kind, x, w, y, ph, pw, stream)
    x4, w4 = _padded(x, c4, "x"), _padded(w, c4, "w")
    xs, ws = x4.strides, w4.strides
    if kind in (0, 2):
        copy_raw(x.ptr, x.strides, x4.ptr, xs, x.shape, stream)
    if kind in (0, 1):
        copy_raw(w.ptr, w.strides, w4.ptr, ws, w.shape, stream)
    conv2d(kind, x4, w4, y, ph, pw, stride, stream)
    if kind == 1:
        copy_raw(x4.ptr, xs, x.ptr, x.strides, x.shape, stream)
    elif kind == 2:
        copy_raw(w4.ptr, ws, w.ptr, w.strides, w.shape, stream)


def _packed_stem_ok(x, w, y, c4, pw, stride):
    kw = w.shape[3]
    return (stride == 1 and c4 == 4 and x.shape[3] % 8 == 0 and y.shape[3] == x.shape[3] and kw <= 9 and pw <= 8
            and kw - 1 - pw <= 8 and y.shape[1] % 4 == 0)


def _conv2d_packed_stem(kind, x, w, y, ph, pw, stream):
    from .. import ndarray
    n, c, h, wd = x.shape
    o, _, kh, kw = w.shape
    _, _, oh, ow = y.shape
    x4 = _padded(x, 4, "x")
    copy_raw(x.ptr, x.strides, x4.ptr, x4.strides, x.shape, stream)
    key = ("stem_w", (o, kh), x.ctx.device_id)
    packed = _PAD_CACHE.get(key)
    if packed is None:
        packed = _PAD_CACHE[key] = ndarray.empty((8 * o * kh * 3 * 32,), x.ctx, use_pool=False)
    so, sc, sh, sw = w.strides
    if kind == 0:
        _check(lib().tsb_stem_pack_filters(_p(w), c_int64(so), c_int64(sc), c_int64(sh), c_int64(sw), _p(packed),
                                           c_int(o), c_int(c), c_int(kh), c_int(kw), c_int(pw), _s(stream)),
               "stem_pack_filters")
    rc = lib().tsb_conv2d(c_int(kind), _p(x4), _p(packed), _p(y), c_int(n), c_int(32), c_int(h), c_int(wd // 8),
                          c_int(8 * o), c_int(kh), c_int(3), c_int(oh), c_int(ow // 8), c_int(ph), c_int(1),
                          c_int(1), _s(stream))
    _check(rc, "conv2d (packed stem) kind %d" % kind)
    if kind == 2:
        _check(lib().tsb_stem_unpack_filter_grads(_p(packed), _p(w), c_int64(so), c_int64(sc), c_int64(sh),
                                                  c_int64(sw), c_int(o), c_int(c), c_int(kh), c_int(kw), c_int(pw),
                                                  _s(stream)), "stem_unpack_filter_grads")


def csrmm(vals, rowptr, colidx, nrow, ncol, dense, out, trans_a, ncols_dense, stream):
    _check(lib().tsb_csrmm(_p(vals), _p(rowptr), _p(colidx), c_int64(nrow), c_int64(ncol), _p(dense),
                           _p(out), c_int(int(trans_a)), c_int64(ncols_dense), _s(stream)), "csrmm")


# -- optimizers (multi-tensor) ----------------------------------------------------------
def adam_advance(hdev, beta1, beta2, stream):
    _check(lib().tsb_adam_advance(_p(hdev), c_float(beta1), c_float(beta2), _s(stream)), "adam_advance")


def optimizer_step(kind, params, grads, slot1, slot2, hyper, stream, hyper_dev=None):
    """One launch per chunk of up to 64 tensors.  kind: 0 sgd, 1 momentum,
    2 nesterov, 3 adagrad, 4 adam.  ``hyper`` is up to 6 floats."""
    n = len(params)
    PT = c_void_p * n
    SZ = c_int64 * n
    z = [None] * n
    hv = (c_float * 8)(*(list(hyper) + [0.0] * (8 - len(hyper))))
    rc = lib().tsb_optimizer_step_dev(
        c_int(kind), c_int(n), PT(*[p.ptr for p in params]), PT(*[g.ptr for g in grads]),
        PT(*[(s.ptr if s is not None else None) for s in (slot1 or z)]),
        PT(*[(s.ptr if s is not None else None) for s in (slot2 or z)]),
        SZ(*[_numel(p.shape) for p in params]), hv, c_void_p(hyper_dev.ptr if hyper_dev is not None else None),
        _s(stream))
    _check(rc, "optimizer_step")
