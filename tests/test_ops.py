"""Every graph op: the sm_100a kernel path against the NumPy oracle path, through
the public Executor API (so layouts, strides and feed staging are covered too)."""
import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad
from helpers import run_graph, assert_close, assert_close_per_channel



@pytest.fixture(params=[pytest.param("cpu"), pytest.param("gpu", marks=pytest.mark.gpu)])
def ctx(request):
    return ndarray.cpu(0) if request.param == "cpu" else ndarray.gpu(0)

R = np.random.RandomState(7)


@pytest.fixture(autouse=True)
def _same_data_whatever_the_selection(request):
    """Every test draws from a generator seeded by its own name, so its data does not depend on which tests ran
    before it (a tolerance that holds in the full run then holds for any ``-k`` selection too)."""
    import zlib
    R.seed(zlib.crc32(request.node.name.split("[")[0].encode()) & 0x7FFFFFFF)


def f32(*shape, scale=1.0):
    return (R.standard_normal(shape) * scale).astype(np.float32)


def both(build, feeds, ctx, rtol=2e-3):
    ref = run_graph(build, feeds, None)
    got = run_graph(build, feeds, ctx)
    for i, (g, r) in enumerate(zip(got, ref)):
        if r is not None:
            assert_close(g, r, rtol=rtol, what="output %d" % i)


def unary_graph(fn):
    def build():
        x = ad.Variable("x")
        return {"x": x}, [fn(x)]
    return build


@pytest.mark.parametrize("shape", [(5, 7), (2, 8, 6, 6), (1000,), (3, 4, 5)])
def test_elementwise_unary(shape, ctx):
    x = np.abs(f32(*shape)) + 0.5
    for fn in (ad.relu_op, ad.sigmoid_op, ad.tanh_op, ad.sqrt_op, ad.rsqrt_op, ad.opposite_op,
               lambda n: ad.addbyconst_op(n, 1.5), lambda n: ad.mul_byconst_op(n, -2.0),
               lambda n: ad.div_const_op(3.0, n), ad.oneslike_op, ad.zeroslike_op):
        both(unary_graph(fn), {"x": x - 0.7 if fn is ad.relu_op else x}, ctx)


@pytest.mark.parametrize("shape", [(6, 10), (2, 4, 5, 5)])
def test_elementwise_binary_and_where(shape, ctx):
    a, b = f32(*shape), np.abs(f32(*shape)) + 0.5

    def build():
        x, y = ad.Variable("a"), ad.Variable("b")
        c = ad.relu_op(x)
        return {"a": x, "b": y}, [x + y, x * y, ad.div_op(x, y), ad.relu_gradient_op(x, y),
                                  ad.where_op(c, x, y)]
    both(build, {"a": a, "b": b}, ctx)


def test_scalar_broadcast_add_mul(ctx):
    def build():
        x, s = ad.Variable("x"), ad.Variable("s")
        return {"x": x, "s": s}, [ad.add_op(x, s), ad.mul_op(s, x)]
    both(build, {"x": f32(4, 9), "s": np.array([2.5], np.float32)}, ctx)


def test_fused_add_relu_matches_add_then_relu(ctx):
    av, bv = f32(3, 8, 5, 7), f32(3, 8, 5, 7)

    def build():
        a, b = ad.Variable("a"), ad.Variable("b")
        y = ad.add_relu_op(a, b)
        ref = ad.relu_op(ad.add_op(a, b))
        w = ad.Variable("w")
        ga, gb = ad.gradients(ad.reduce_sum_op(ad.mul_op(y, w), [0, 1, 2, 3]), [a, b])
        ra, rb = ad.gradients(ad.reduce_sum_op(ad.mul_op(ref, w), [0, 1, 2, 3]), [a, b])
        return {"a": a, "b": b, "w": w}, [y, ref, ga, gb, ra, rb]
    feeds = {"a": av, "b": bv, "w": f32(3, 8, 5, 7)}
    both(build, feeds, ctx)
    y, ref, ga, gb, ra, rb = [np.asarray(o) for o in run_graph(build, feeds, ctx)]
    np.testing.assert_allclose(y, ref, rtol=1e-6)
    np.testing.assert_allclose(ga, ra, rtol=1e-6)
    np.testing.assert_allclose(gb, rb, rtol=1e-6)


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_matmul_and_grads(ta, tb, ctx):
    m, k, n = 96, 64, 80
    a = f32(k, m) if ta else f32(m, k)
    b = f32(n, k) if tb else f32(k, n)

    def build():
        A, B = ad.Variable("a"), ad.Variable("b")
        C = ad.matmul_op(A, B, ta, tb)
        loss = ad.reduce_sum_op(ad.mul_op(C, C), [0, 1])
        ga, gb = ad.gradients(loss, [A, B])
        return {"a": A, "b": B}, [C, ga, gb]
    both(build, {"a": a, "b": b}, ctx, rtol=5e-3)


@pytest.mark.parametrize("n,h,tq,tk,d", [(2, 4, 40, 40, 32), (3, 2, 37, 45, 64), (2, 8, 255, 255, 64), (1, 2, 8, 130, 20)])
def test_batch_matmul_in_head_layout_with_gradients(n, h, tq, tk, d, ctx):
    """The attention products on operands stored [N, T, H, d]: scores = Q K^T (both operands in head layout),
    context = P V (V and the result in head layout), and through ``ad.gradients`` the four products of the backward
    pass (dQ, dK: result in head layout; dV: MN-major operand in head layout; dP: both operands in head layout)."""
    q, k, v = f32(n, tq, h, d), f32(n, tk, h, d), f32(n, tk, h, d)

    def build():
        Q, K, V = ad.Variable("q"), ad.Variable("k"), ad.Variable("v")
        scores = ad.batch_matmul_op(Q, K, trans_B=True, heads_A=True, heads_B=True)
        probs = ad.softmax_op(scores * 0.2)
        ctxv = ad.batch_matmul_op(probs, V, heads_B=True, heads_out=True)
        loss = ad.reduce_sum_op(ad.mul_op(ctxv, ctxv), [0, 1, 2, 3])
        gq, gk, gv = ad.gradients(loss, [Q, K, V])
        return {"q": Q, "k": K, "v": V}, [scores, ctxv, gq, gk, gv]
    # the gradients pass through three TF32 products and the soft-max: 1e-2 of each tensor's scale
    both(build, {"q": q, "k": k, "v": v}, ctx, rtol=1e-2)


@pytest.mark.parametrize("n,h,tq,tk,causal,masked", [(2, 3, 16, 16, True, True), (2, 2, 37, 45, False, True),
                                                     (1, 4, 255, 255, True, False), (2, 2, 8, 600, False, True)])
def test_masked_softmax_and_gradient(n, h, tq, tk, causal, masked, ctx):
    scores = f32(n, h, tq, tk, scale=3.0)
    tokens = (np.random.RandomState(3).rand(n, tk) > 0.3).astype(np.float32) * 7.0
    tokens[:, 0] = 5.0                       # at least one real key per row
    g = f32(n, h, tq, tk)

    def build():
        S, T, Gv = ad.Variable("s"), ad.Variable("t"), ad.Variable("g")
        p = ad.masked_softmax_op(S, T if masked else None, scale=0.125, causal=causal)
        loss = ad.reduce_sum_op(ad.mul_op(p, Gv), [0, 1, 2, 3])
        ds, = ad.gradients(loss, [S])
        return {"s": S, "t": T, "g": Gv}, [p, ds]
    both(build, {"s": scores, "t": tokens, "g": g}, ctx, rtol=2e-3)


def test_masked_softmax_equals_the_operator_chain():
    n, h, tq, tk = 2, 3, 6, 6
    scores, tokens = f32(n, h, tq, tk), np.array([[3, 1, 0, 2, 0, 0], [4, 4, 4, 0, 1, 2]], np.float32)

    def chain(S, T):
        s = S * 0.5
        zeros = ad.zeroslike_op(T)
        mask = ad.array_reshape_op(ad.where_op(T, zeros, ad.addbyconst_op(zeros, -1e9)), (n, 1, 1, tk))
        s = s + ad.broadcasttoTF_op(mask, s)
        tril = ad.Variable("tril", value=np.tril(np.ones((tq, tk), np.float32)), trainable=False)
        s = ad.where_op(ad.broadcast_shape_op(tril, (n, h, tq, tk)), s, ad.addbyconst_op(ad.zeroslike_op(s), -1e9))
        return ad.softmax_op(s)
    outs = []
    for fused in (True, False):
        S, T = ad.Variable("s"), ad.Variable("t")
        p = ad.masked_softmax_op(S, T, scale=0.5, causal=True) if fused else chain(S, T)
        loss = ad.reduce_sum_op(ad.mul_op(p, p), [0, 1, 2, 3])
        outs.append(ad.Executor([p] + ad.gradients(loss, [S]), ctx=None).run({S: scores, T: tokens},
                                                                              convert_to_numpy_ret_vals=True))
    for a, b in zip(*outs):
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-7)


def test_head_layout_equals_transposed_heads():
    """NumPy oracle: the head-layout products equal the transpose -> batched product -> transpose chain."""
    q, k, v = f32(2, 5, 3, 4), f32(2, 7, 3, 4), f32(2, 7, 3, 4)

    def build(head_layout):
        Q, K, V = ad.Variable("q"), ad.Variable("k"), ad.Variable("v")
        if head_layout:
            s = ad.batch_matmul_op(Q, K, trans_B=True, heads_A=True, heads_B=True)
            c = ad.batch_matmul_op(ad.softmax_op(s), V, heads_B=True, heads_out=True)
        else:
            tq, tk, tv = (ad.transpose_op(x, (0, 2, 1, 3)) for x in (Q, K, V))
            s = ad.batch_matmul_op(tq, tk, trans_B=True)
            c = ad.transpose_op(ad.batch_matmul_op(ad.softmax_op(s), tv), (0, 2, 1, 3))
        loss = ad.reduce_sum_op(ad.mul_op(c, c), [0, 1, 2, 3])
        return [s, c] + ad.gradients(loss, [Q, K, V]), {Q: q, K: k, V: v}
    outs = []
    for hl in (True, False):
        nodes, feed = build(hl)
        outs.append(ad.Executor(nodes, ctx=None).run(feed, convert_to_numpy_ret_vals=True))
    for a, b in zip(*outs):
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)


def test_batch_matmul(ctx):
    def build():
        A, B = ad.Variable("a"), ad.Variable("b")
        return {"a": A, "b": B}, [ad.batch_matmul_op(A, B), ad.batch_matmul_op(A, A, False, True)]
    both(build, {"a": f32(2, 3, 64, 32), "b": f32(2, 3, 32, 48)}, ctx, rtol=5e-3)


CONVS = [
    # n, c, h, w, o, k, pad, stride
    (2, 8, 12, 12, 16, 3, 1, 1),
    (3, 3, 16, 16, 64, 3, 1, 1),       # RGB stem (padded-channel path)
    (2, 64, 14, 14, 128, 3, 1, 1),
    (2, 32, 9, 9, 64, 1, 0, 1),
    (2, 16, 15, 15, 32, 3, 1, 2),
    (1, 3, 32, 32, 64, 7, 3, 2),
    (2, 72, 7, 7, 200, 3, 1, 1),       # ragged channel counts
    (4, 256, 8, 8, 512, 3, 1, 1),      # wide tiles (BN = 256)
    # channel counts that are multiples of 32 take the TMA im2col path on the GPU
    (2, 32, 13, 11, 96, 3, 1, 2),      # strided, non-square image
    (2, 64, 10, 10, 32, 5, 2, 1),      # 5x5 window
    (1, 32, 40, 40, 32, 3, 0, 1),      # no padding, several tiles of pixels
    (3, 96, 6, 6, 160, 3, 1, 1),       # pixel tiles that span images
    (5, 128, 7, 9, 64, 3, 1, 1),
    # enough 256-pixel x 256-channel tiles for the CTA-pair (cta_group::2) kernel
    (10, 32, 32, 32, 256, 3, 1, 1),    # forward on pairs
    (10, 256, 32, 32, 64, 3, 1, 1),    # dgrad on pairs (forward kernel with flipped filters)
    (12, 64, 56, 56, 320, 3, 1, 2),    # strided, ragged channel tile
    (4, 64, 14, 14, 128, 1, 0, 2),     # 1x1 stride-2 projection (strided dgrad through zero insertion)
    (2, 32, 15, 17, 64, 3, 1, 3),      # stride 3, sizes that leave a remainder
    (2, 64, 35, 35, 96, 3, 0, 2),      # stride 2 without padding on an odd image (parity classes of unequal size)
    (2, 32, 28, 28, 64, 5, 2, 2),      # stride 2, 5x5: three and two taps per parity
    (2, 32, 16, 12, 64, 2, 0, 2),      # stride 2, 2x2: one tap per parity, no padding taps
    (3, 32, 9, 9, 32, 1, 0, 2),        # 1x1 stride 2 on an odd image: three of the four parities are zero
]


@pytest.mark.parametrize("n,c,h,w,o,k,pad,stride", CONVS)
def test_conv2d_forward_and_gradients(n, c, h, w, o, k, pad, stride, ctx):
    xv, wv = f32(n, c, h, w), f32(o, c, k, k, scale=0.2)

    def build():
        x, f = ad.Variable("x"), ad.Variable("w")
        y = ad.conv2d_op(x, f, padding=pad, stride=stride)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        gx, gf = ad.gradients(loss, [x, f])
        return {"x": x, "w": f}, [y, gx, gf]
    both(build, {"x": xv, "w": wv}, ctx, rtol=6e-3)


def test_conv_asymmetric_kernel_and_padding(ctx):
    def build():
        x, f = ad.Variable("x"), ad.Variable("w")
        y = ad.conv2d_op(x, f, padding=0, padding2=3, stride=1)
        loss = ad.reduce_sum_op(y, [0, 1, 2, 3])
        gx, gf = ad.gradients(loss, [x, f])
        return {"x": x, "w": f}, [y, gx, gf]
    both(build, {"x": f32(2, 16, 10, 10), "w": f32(24, 16, 1, 7, scale=0.2)}, ctx, rtol=6e-3)


@pytest.mark.parametrize("n,c,hw,o,relu", [
    (4, 32, 16, 64, True),        # one-CTA tiles of 64 columns, two CTAs per SM
    (3, 64, 12, 128, False),      # tiles of 128 columns
    (6, 64, 24, 512, True),       # one-CTA tiles of 256 columns, two column tiles
    (10, 32, 32, 256, True),      # CTA pairs
    (16, 64, 32, 512, False),     # CTA pairs, two column tiles
    (2, 8, 10, 24, True),         # channel count off the TMA path: statistics from the separate kernel
])
def test_conv_then_batch_norm_takes_statistics_from_the_conv_epilogue(n, c, hw, o, relu, ctx):
    xv, wv = f32(n, c, hw, hw), f32(o, c, 3, 3, scale=0.2)
    sv, bv = 1.0 + 0.1 * f32(1, o, 1, 1), 0.1 * f32(1, o, 1, 1)

    def build():
        x, f = ad.Variable("x"), ad.Variable("w")
        s, b = ad.Variable("s"), ad.Variable("b")
        y = ad.conv2d_op(x, f, padding=1, stride=1)
        z = ad.batch_normalization_relu_op(y, s, b) if relu else ad.batch_normalization_op(y, s, b)
        loss = ad.reduce_sum_op(ad.mul_op(z, z), [0, 1, 2, 3])
        gx, gf, gs, gb = ad.gradients(loss, [x, f, s, b])
        return {"x": x, "w": f, "s": s, "b": b}, [z, gx, gf, gs, gb]
    feeds = {"x": xv, "w": wv, "s": sv, "b": bv}
    both(build, feeds, ctx, rtol=2e-2)
    # and channel by channel: activations and their gradient per channel, the filter gradient per output channel,
    # the scale / bias gradients element by element
    ref = run_graph(build, feeds, None)
    got = run_graph(build, feeds, ctx)
    for i, axis in ((0, 1), (1, 1), (2, 0), (3, 1), (4, 1)):
        assert_close_per_channel(got[i], ref[i], axis, rtol=5e-2, what="output %d per channel" % i)


def test_conv_bias_helpers(ctx):
    def build():
        b, x = ad.Variable("b"), ad.Variable("x")
        return {"b": b, "x": x}, [ad.conv2d_broadcastto_op(b, x), ad.conv2d_reducesum_op(x)]
    both(build, {"b": f32(8), "x": f32(3, 8, 5, 5)}, ctx)


@pytest.mark.parametrize("kind", ["max", "avg"])
@pytest.mark.parametrize("k,pad,stride,hw", [(2, 0, 2, 8), (3, 1, 2, 9), (3, 1, 1, 6), (7, 0, 7, 7)])
def test_pooling(kind, k, pad, stride, hw, ctx):
    def build():
        x = ad.Variable("x")
        op = ad.max_pool2d_op if kind == "max" else ad.avg_pool2d_op
        y = op(x, k, k, pad, stride)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        gx, = ad.gradients(loss, [x])
        return {"x": x}, [y, gx]
    both(build, {"x": np.round(f32(2, 8, hw, hw) * 2) / 2}, ctx)    # ties on purpose


def test_batch_norm_forward_backward(ctx):
    def build():
        x, s, b = ad.Variable("x"), ad.Variable("s"), ad.Variable("b")
        y = ad.batch_normalization_op(x, s, b)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        gx, gs, gb = ad.gradients(loss, [x, s, b])
        return {"x": x, "s": s, "b": b}, [y, gx, gs, gb]
    both(build, {"x": f32(4, 16, 6, 6) + 0.5, "s": f32(1, 16, 1, 1) + 1, "b": f32(1, 16, 1, 1)}, ctx, rtol=5e-3)


@pytest.mark.parametrize("shape", [(3, 5, 64), (40, 33, 512), (7, 9, 30)])
def test_layer_norm(ctx, shape):
    d = shape[-1]

    def build():
        x, s, b = ad.Variable("x"), ad.Variable("s"), ad.Variable("b")
        y = ad.layer_normalization_op(x, s, b)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2])
        gx, gs, gb = ad.gradients(loss, [x, s, b])
        return {"x": x, "s": s, "b": b}, [y, gx, gs, gb]
    both(build, {"x": f32(*shape), "s": f32(d) + 1, "b": f32(d)}, ctx, rtol=5e-3)


@pytest.mark.parametrize("rows,cols", [(32, 1000), (70, 256), (19, 64), (5, 1023), (9, 4100), (6, 33000)])
def test_softmax_and_cross_entropy(ctx, rows, cols):
    # short rows take the warp-per-row kernel, rows whose length is no multiple of 4 the scalar one,
    # long rows the 16-byte one-pass kernels
    logits = f32(rows, cols) * 3
    labels = np.eye(cols, dtype=np.float32)[R.randint(0, cols, rows)]

    def build():
        y, y_ = ad.Variable("y"), ad.Variable("y_")
        loss = ad.softmaxcrossentropy_op(y, y_)
        g, = ad.gradients(loss, [y])
        return {"y": y, "y_": y_}, [ad.softmax_op(y), loss, g]
    both(build, {"y": logits, "y_": labels}, ctx)


@pytest.mark.parametrize("shape", [(2, 4, 24, 256), (3, 2, 7, 64), (2, 3, 9, 255), (11, 100), (5, 1030), (4, 4100)])
def test_softmax_backward(ctx, shape):
    # rows up to 1024 long take the warp-per-row kernel, others the CTA-per-row one
    def build():
        x, w = ad.Variable("x"), ad.Variable("w")
        y = ad.softmax_op(x)
        loss = ad.reduce_sum_op(ad.mul_op(y, w), list(range(len(shape))))
        gx, = ad.gradients(loss, [x])
        return {"x": x, "w": w}, [y, gx]
    both(build, {"x": f32(*shape) * 2, "w": f32(*shape)}, ctx)


@pytest.mark.parametrize("xs,bs", [((6, 10, 64), (64,)), ((5, 30), (30,)), ((3, 4, 9, 15), (3, 1, 1, 15)),
                                   ((4, 8, 12), (8, 1)), ((7, 36), (7, 36)), ((3, 2, 5, 100), (3, 1, 1, 100)),
                                   ((2, 3, 66, 70), (66, 70)), ((2, 3, 9, 255), (2, 1, 1, 255))])
def test_add_of_a_broadcast_is_one_op(ctx, xs, bs):
    # x + broadcasttoTF_op(b, x) is built as one AddBroadcast node; b's gradient sums over the broadcast axes
    def build():
        x, b, w = ad.Variable("x"), ad.Variable("b"), ad.Variable("w")
        y = x + ad.broadcasttoTF_op(b, x)
        assert y.op.name == "AddBroadcast"
        z = ad.broadcasttoTF_op(b, x) + x
        assert z.op.name == "AddBroadcast"
        loss = ad.reduce_sum_op(ad.mul_op(y, w), list(range(len(xs))))
        gx, gb = ad.gradients(loss, [x, b])
        # the bare broadcast and a product with it run the strided copy / binary kernels (row form when the
        # innermost dimension is long)
        bc = ad.broadcasttoTF_op(b, x)
        return {"x": x, "b": b, "w": w}, [y, z, gx, gb, bc, ad.mul_op(x, bc)]
    both(build, {"x": f32(*xs), "b": f32(*bs), "w": f32(*xs)}, ctx)


@pytest.mark.parametrize("rows,cols", [(300, 128), (2050, 36), (100, 30), (64, 4)])
def test_column_sums(ctx, rows, cols):
    # [rows, cols] -> [cols]: the two-stage kernels (16-byte lanes when cols is a multiple of 4)
    def build():
        x = ad.Variable("x")
        return {"x": x}, [ad.reduce_sum_op(x, [0]), ad.reducesumaxiszero_op(x)]
    both(build, {"x": f32(rows, cols)}, ctx)


def test_shape_family(ctx):
    def build():
        x, z = ad.Variable("x"), ad.Variable("z")
        outs = [ad.array_reshape_op(x, (-1, 6 * 5 * 5)), ad.transpose_op(x, (0, 2, 3, 1)),
                ad.transpose_op(z), ad.slice_op(x, (0, 1, 1, 0), (2, 3, -1, 4)),
                ad.concat_op(x, x, axis=1), ad.pad_op(x, [(0, 0), (0, 0), (1, 2), (2, 1)]),
                ad.reduce_sum_op(x, [0, 2, 3]), ad.reduce_sum_op(z, [1], keepdims=True),
                ad.reducesumaxiszero_op(z), ad.broadcastto_op(z, ad.Variable("w", value=np.zeros((3, 7, 9), np.float32))),
                ad.broadcast_shape_op(ad.reduce_sum_op(z, [1]), (7, 9), add_axes=[1])]
        loss = ad.reduce_sum_op(ad.mul_op(outs[3], outs[3]), [0, 1, 2, 3]) + \
            ad.reduce_sum_op(ad.pad_op(x, [(0, 0), (0, 0), (1, 1), (1, 1)]), [0, 1, 2, 3]) + \
            ad.reduce_sum_op(ad.mul_op(outs[4], outs[4]), [0, 1, 2, 3]) + \
            ad.reduce_sum_op(ad.mul_op(outs[0], outs[0]), [0, 1])
        gx, = ad.gradients(loss, [x])
        return {"x": x, "z": z}, outs + [gx]
    both(build, {"x": f32(2, 6, 5, 5), "z": f32(7, 9)}, ctx)


def test_embedding_onehot_dropout(ctx):
    idx = R.randint(0, 50, (4, 6)).astype(np.float32)

    def build():
        t, i, x = ad.Variable("t"), ad.Variable("i"), ad.Variable("x")
        e = ad.embedding_lookup_op(t, i)
        loss = ad.reduce_sum_op(ad.mul_op(e, e), [0, 1, 2])
        gt, = ad.gradients(loss, [t])
        d = ad.dropout_op(x, 0.7, seed=1234)
        gd, = ad.gradients(ad.reduce_sum_op(d, [0, 1]), [x])
        # 50 classes: scalar one-hot kernel; 1032: the 16-byte row kernel
        return {"t": t, "i": i, "x": x}, [e, gt, ad.one_hot_op(i, 50), d, gd, ad.one_hot_op(i, 1032)]
    both(build, {"t": f32(50, 16), "i": idx, "x": f32(8, 32)}, ctx)


def test_csrmm_and_csrmv(ctx):
    import scipy.sparse
    dense = f32(20, 8)
    m = scipy.sparse.random(12, 20, density=0.3, random_state=3, dtype=np.float32).tocoo()
    for ctx in (ctx,):
        sp = ndarray.sparse_array(m.data, (m.row, m.col), (12, 20), ctx)
        A, B = ad.Variable("A"), ad.Variable("B")
        out = ad.csrmm_op(A, B)
        ex = ad.Executor([out], ctx=ctx)
        got = ex.run({A: sp, B: dense}, convert_to_numpy_ret_vals=True)[0]
        assert_close(got, m.toarray() @ dense, rtol=1e-4)


def test_fused_batch_norm_relu_forward_backward(ctx):
    def build(fused):
        def b():
            x, s, bb = ad.Variable("x"), ad.Variable("s"), ad.Variable("b")
            y = ad.batch_normalization_relu_op(x, s, bb) if fused else ad.relu_op(ad.batch_normalization_op(x, s, bb))
            loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
            gx, gs, gb = ad.gradients(loss, [x, s, bb])
            return {"x": x, "s": s, "b": bb}, [y, gx, gs, gb]
        return b
    feeds = {"x": f32(4, 16, 6, 6) + 0.2, "s": f32(1, 16, 1, 1) + 1, "b": f32(1, 16, 1, 1)}
    ref = run_graph(build(False), feeds, None)
    got = run_graph(build(True), feeds, ctx)
    for i, (g, r) in enumerate(zip(got, ref)):
        assert_close(g, r, rtol=5e-3, what="output %d" % i)
