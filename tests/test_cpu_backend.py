"""Host operator library (csrc/runtime/cpu_ops.cc) behind ``Op.cpu_compute``: every operator that has a native
kernel gives what its NumPy path gives, and a CPU-context training step of each model family runs its forward AND
backward operators through the library."""
import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad, cpu_links, graph


def f32(*shape, seed=0, scale=1.0):
    return (np.random.RandomState(seed + sum(shape)).randn(*shape) * scale).astype(np.float32)


def run_both(build, feeds):
    """Same graph on the NumPy oracle (ctx=None) and on the CPU context; returns (oracle, native, native calls)."""
    outs = []
    calls = 0
    for ctx in (None, ndarray.cpu(0)):
        ph, nodes = build()
        ex = ad.Executor(nodes, ctx=ctx)
        before = cpu_links.CALLS[0]
        outs.append([np.asarray(o) for o in ex.run({ph[k]: v for k, v in feeds.items()}, convert_to_numpy_ret_vals=True)])
        calls = cpu_links.CALLS[0] - before
    return outs[0], outs[1], calls


def check(build, feeds, min_calls, rtol=2e-4, atol=2e-5):
    ref, got, calls = run_both(build, feeds)
    assert calls >= min_calls, "only %d native calls" % calls
    for a, b in zip(got, ref):
        np.testing.assert_allclose(a, b, rtol=rtol, atol=atol)


@pytest.mark.parametrize("stride,pad,k", [(1, 1, 3), (2, 1, 3), (2, 0, 1), (1, 0, 2)])
def test_convolution_gradients(stride, pad, k):
    def build():
        x, w = ad.Variable("x"), ad.Variable("w")
        y = ad.conv2d_op(x, w, padding=pad, stride=stride)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        return {"x": x, "w": w}, [y] + ad.gradients(loss, [x, w])
    check(build, {"x": f32(2, 3, 9, 8), "w": f32(4, 3, k, k, scale=0.3)}, 3, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("kind", ["max", "avg"])
@pytest.mark.parametrize("k,pad,stride,hw", [(2, 0, 2, 8), (3, 1, 2, 9), (3, 1, 1, 6)])
def test_pooling_gradients(kind, k, pad, stride, hw):
    op = ad.max_pool2d_op if kind == "max" else ad.avg_pool2d_op

    def build():
        x = ad.Variable("x")
        y = op(x, k, k, pad, stride)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        return {"x": x}, [y] + ad.gradients(loss, [x])
    check(build, {"x": f32(2, 3, hw, hw)}, 2)


@pytest.mark.parametrize("relu", [False, True])
def test_batch_norm_forward_and_backward(relu):
    def build():
        x, s, b = ad.Variable("x"), ad.Variable("s"), ad.Variable("b")
        y = ad.batch_normalization_op(x, s, b)
        y = ad.relu_op(y) if relu else y
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1, 2, 3])
        return {"x": x, "s": s, "b": b}, [y] + ad.gradients(loss, [x, s, b])
    check(build, {"x": f32(4, 5, 6, 6), "s": f32(5) + 1.5, "b": f32(5, seed=1)}, 2, rtol=2e-3, atol=2e-4)


def test_softmax_transpose_concat_pad_broadcast_reduce_fill():
    def build():
        a, b = ad.Variable("a"), ad.Variable("b")
        sm = ad.softmax_op(a)
        t = ad.transpose_op(a, (1, 0, 2))
        cat = ad.concat_op(a, b, axis=1)
        pad = ad.pad_op(a, [(0, 0), (1, 2), (3, 0)])
        red = ad.reducesumaxiszero_op(a)
        bc = ad.broadcastto_op(red, a)
        loss = ad.reduce_sum_op(ad.mul_op(sm, sm), [0, 1, 2]) + ad.reduce_sum_op(ad.mul_op(cat, cat), [0, 1, 2]) \
            + ad.reduce_sum_op(ad.mul_op(pad, pad), [0, 1, 2]) + ad.reduce_sum_op(ad.mul_op(t, bc_t(bc)), [0, 1, 2])
        return {"a": a, "b": b}, [sm, t, cat, pad, red, bc, ad.oneslike_op(a)] + ad.gradients(loss, [a, b])

    def bc_t(bc):
        return ad.transpose_op(bc, (1, 0, 2))
    check(build, {"a": f32(3, 4, 5), "b": f32(3, 2, 5, seed=2)}, 10)


def test_dropout_mask_matches_the_oracle():
    def build():
        x = ad.Variable("x")
        y = ad.dropout_op(x, 0.7, seed=1234)
        loss = ad.reduce_sum_op(ad.mul_op(y, y), [0, 1])
        return {"x": x}, [y] + ad.gradients(loss, [x])
    ref, got, calls = run_both(build, {"x": f32(64, 33)})
    assert calls >= 2
    assert 0.55 < float((got[0] != 0).mean()) < 0.85
    for a, b in zip(got, ref):
        np.testing.assert_allclose(a, b, rtol=1e-6)


@pytest.mark.parametrize("family", ["vgg", "resnet", "transformer"])
def test_training_step_runs_forward_and_backward_natively(family):
    """Which operator classes went through the library during one CPU-context step."""
    from tsplit_b200.models import vgg, resnet, transformer
    seen = set()
    orig = graph.Op.compute

    def spy(self, node, iv, out, use_numpy=True, stream_handle=None):
        before = cpu_links.CALLS[0]
        r = orig(self, node, iv, out, use_numpy, stream_handle)
        if cpu_links.CALLS[0] > before:
            seen.add(self.name)
        return r
    graph.Op.compute = spy
    try:
        if family == "transformer":
            t = transformer(vocab_size=40, d_model=16, num_heads=2, d_ff=32, num_blocks=1, maxlen1=6, maxlen2=6,
                            batch_size=2, seed=3)
            loss, variables, feed = t.loss, t.variables, t.synthetic_batch()
        else:
            m = vgg(16, num_classes=10, image=32, width_div=16, fc_width=32, seed=3) if family == "vgg" else \
                resnet(26, num_classes=10, image=32, width_div=8, seed=3)
            x, y = m.synthetic_batch(4, seed=1)
            loss, variables, feed = m.loss, m.variables, {m.X: x, m.y_: y}
        grads = ad.gradients(loss, variables)
        outs = []
        for ctx in (None, ndarray.cpu(0)):
            seen.clear()
            ex = ad.Executor([loss] + grads, ctx=ctx)
            outs.append([np.asarray(o) for o in ex.run(feed, convert_to_numpy_ret_vals=True)])
        native = set(seen)
    finally:
        graph.Op.compute = orig
    if family == "transformer":
        assert {"MatMul", "Softmax", "SoftmaxGradient", "Transpose"} <= native or {"MatMul", "Add"} <= native, native
    else:
        assert {"Conv2d", "Conv2dGradData", "Conv2dGradFilter", "MatMul", "SoftmaxCrossEntropy"} <= native, native
        assert {"BatchNormRelu", "BatchNormReluGradient"} <= native or {"BatchNorm", "BatchNormGradient"} <= native, native
        assert ("MaxPool2dGradient" in native) or ("AvgPool2dGradient" in native), native
    for a, b in zip(outs[1], outs[0]):       # fp32 sums in another order through 10-26 layers: compare to the tensor's scale
        assert np.abs(a - b).max() <= 2e-3 * max(np.abs(b).max(), 1e-3)


@pytest.mark.parametrize("make", [
    lambda ctx: __import__("tsplit_b200").optimizer.SGDOptimizer(0.05, ctx=ctx),
    lambda ctx: __import__("tsplit_b200").optimizer.MomentumOptimizer(0.05, 0.9, ctx=ctx),
    lambda ctx: __import__("tsplit_b200").optimizer.MomentumOptimizer(0.05, 0.9, nesterov=True, ctx=ctx),
    lambda ctx: __import__("tsplit_b200").optimizer.AdaGradOptimizer(0.005, ctx=ctx),
    lambda ctx: __import__("tsplit_b200").optimizer.AdamOptimizer(0.01, ctx=ctx),
], ids=["sgd", "momentum", "nesterov", "adagrad", "adam"])
def test_optimizers_update_natively_on_a_cpu_context(make):
    """Four training steps of an MLP on ``ndarray.cpu(0)`` (update kernels of the host library) give the losses and
    parameters of the NumPy oracle."""
    from tsplit_b200.models import mlp
    runs = []
    for ctx in (None, ndarray.cpu(0)):
        m = mlp(seed=11)
        opt = make(ctx)
        train = opt.minimize(m.loss)
        ex = ad.Executor([m.loss, train], ctx=ctx)
        x, y = m.synthetic_batch(32, seed=4)
        before = cpu_links.CALLS[0]
        losses = [float(np.asarray(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0]).reshape(-1)[0])
                  for _ in range(4)]
        calls = cpu_links.CALLS[0] - before
        assert (calls > 0) == (ctx is not None)
        runs.append((losses, [np.asarray(p.asnumpy() if hasattr(p, "asnumpy") else p).copy() for p in opt.params]))
    np.testing.assert_allclose(runs[1][0], runs[0][0], rtol=5e-4)
    # AdaGrad and Adam divide by the root of an accumulator that is tiny where the gradient is: there the update
    # is lr * sign-ish and a last-bit difference of the gradient moves it by a fraction of lr: absolute floor
    for a, b in zip(runs[1][1], runs[0][1]):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=5e-4)
    assert runs[0][0][-1] < runs[0][0][0]
