"""Memory policies on a real GPU: pinned-host swaps on the copy streams,
event-ordered reuse of pool blocks, recompute and micro-tensor transfers must
reproduce the keep-everything executor."""
import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
from tsplit_b200.models import vgg, resnet
from tsplit_b200.runtime.pool import use_pool
from helpers import assert_close

pytestmark = pytest.mark.gpu


def net():
    return vgg(16, num_classes=32, image=64, width_div=4, fc_width=256, seed=5)


def run(cls, policy, cap, batch=16, steps=2, **kw):
    ctx = ndarray.gpu(0)
    m = net()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(batch, seed=2)
    with use_pool(ctx, cap) as pool:
        ex = cls([m.loss] + grads, ctx=ctx, policy=policy, **kw)
        for _ in range(steps):
            pool.reset_peak()
            outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        return outs, pool.stats()["peak"], ex


@pytest.fixture(scope="module")
def keep_all():
    outs, peak, _ = run(ad.MemoryExecutor, None, 4 << 30)
    return outs, peak


@pytest.mark.parametrize("cls,policy", [(ad.vdnnExecutor, "all"), (ad.vdnnExecutor, "conv"),
                                        (ad.recomputeExecutor, "speed"), (ad.recomputeExecutor, "memory"),
                                        (ad.superNeuronsExecutor, None)])
def test_policy_on_gpu_matches_keep_all(cls, policy, keep_all):
    ref, peak_keep = keep_all
    outs, peak, ex = run(cls, policy, 4 << 30)
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=2e-3, what="%s/%s output %d" % (cls.__name__, policy, i))
    assert peak < peak_keep
    assert ex.stats["swap_out_bytes"] > 0 or ex.stats["recomputed_nodes"] > 0


def test_tsplit_and_capuchin_under_a_tight_cap(keep_all):
    ref, peak_keep = keep_all
    cap = int(peak_keep * 0.7)
    with pytest.raises(ndarray.OutOfHBMBudget):
        run(ad.MemoryExecutor, None, cap, steps=1)
    for cls, kw in ((ad.microopExecutor, dict(host_link_gbs=20.0, max_split=4)), (ad.capuchinExecutor, {})):
        outs, peak, ex = run(cls, None, cap, steps=3, **kw)
        assert peak <= cap
        for i, (o, r) in enumerate(zip(outs, ref)):
            assert_close(o, r, rtol=2e-3, what="%s output %d" % (cls.__name__, i))


def test_training_with_graph_replay_matches_eager():
    ctx = ndarray.gpu(0)
    losses = {}
    for use_graph in (False, True):
        m = net()
        opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        ex = ad.Executor([m.loss, train], ctx=ctx, use_graph=use_graph)
        x, y = m.synthetic_batch(16, seed=2)
        xd, yd = ndarray.array(x, ctx), ndarray.array(y, ctx)
        losses[use_graph] = [float(ex.run({m.X: xd, m.y_: yd})[0].asnumpy()[0]) for _ in range(5)]
    assert_close(np.array(losses[True]), np.array(losses[False]), rtol=5e-3)
    assert losses[False][-1] < losses[False][0]


def test_graph_replay_of_a_swap_free_step_matches_eager():
    """The engine replays a step without swaps from a CUDA graph after two eager steps; the losses
    of six training steps equal those of the eager executor step by step."""
    ctx = ndarray.gpu(0)
    outs = []
    for use_graph in (False, True):
        m = net()
        opt = optimizer.MomentumOptimizer(learning_rate=0.01, momentum=0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        x, y = m.synthetic_batch(16, seed=2)
        with use_pool(ctx, 4 << 30):
            ex = ad.MemoryExecutor([m.loss, train], ctx=ctx, use_graph=use_graph)
            vals = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0].reshape(-1)[0])
                    for _ in range(6)]
        outs.append(vals)
        if use_graph:
            assert ex._step_graph is not None, "the step was not captured"
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-5)
    assert outs[0][-1] < outs[0][0]


def test_graph_replay_with_adam_keeps_the_bias_correction_in_step():
    ctx = ndarray.gpu(0)
    outs = []
    for use_graph in (False, True):
        m = net()
        opt = optimizer.AdamOptimizer(learning_rate=0.001, ctx=ctx)
        train = opt.minimize(m.loss)
        x, y = m.synthetic_batch(16, seed=2)
        with use_pool(ctx, 4 << 30):
            ex = ad.MemoryExecutor([m.loss, train], ctx=ctx, use_graph=use_graph)
            vals = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0].reshape(-1)[0])
                    for _ in range(6)]
        outs.append(vals)
        assert opt.step_count == 6
        if use_graph:
            assert ex._step_graph is not None, "the step was not captured"
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-4)


def test_prefetched_pinned_feeds_give_the_same_steps():
    """``prefetch_feeds`` copies the next step's pinned host arrays on the copy stream into the second
    device buffer; results equal those of feeding the same arrays step by step."""
    import torch
    ctx = ndarray.gpu(0)
    batches = []
    m0 = net()
    for seed in (2, 9):
        x, y = m0.synthetic_batch(16, seed=seed)
        xp = ndarray.empty(x.shape, ndarray.cpu(0), pinned=True)
        yp = ndarray.empty(y.shape, ndarray.cpu(0), pinned=True)
        xp.t.copy_(torch.from_numpy(x))
        yp.t.copy_(torch.from_numpy(y))
        batches.append((xp, yp))
    outs = []
    for ahead in (False, True):
        m = net()
        opt = optimizer.MomentumOptimizer(learning_rate=0.01, momentum=0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        with use_pool(ctx, 4 << 30):
            ex = ad.MemoryExecutor([m.loss, train], ctx=ctx)
            feeds = [{m.X: b[0], m.y_: b[1]} for b in batches]
            vals = []
            if ahead:
                ex.prefetch_feeds(feeds[0])
            for i in range(5):
                if ahead and i + 1 < 5:
                    ex.prefetch_feeds(feeds[(i + 1) % 2])
                vals.append(float(ex.run(feeds[i % 2], convert_to_numpy_ret_vals=True)[0].reshape(-1)[0]))
        outs.append(vals)
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-5)
    assert abs(outs[0][0] - outs[0][1]) > 1e-6        # the two batches really differ
