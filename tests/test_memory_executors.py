"""Every memory policy must reproduce the base executor's losses and gradients
(fp32 tolerance) on the simulated device under a budget the base executor
cannot meet."""
import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
from tsplit_b200.models import vgg, resnet
from tsplit_b200.runtime.pool import use_pool
from helpers import assert_close


def small_cnn():
    return vgg(16, num_classes=10, image=64, width_div=8, fc_width=64, seed=3)


def reference_run(model_fn, batch, steps=2):
    m = model_fn()
    grads = ad.gradients(m.loss, m.variables)
    ex = ad.Executor([m.loss] + grads, ctx=None)
    x, y = m.synthetic_batch(batch, seed=1)
    outs = None
    for _ in range(steps):
        outs = ex.run({m.X: x, m.y_: y})
    return [np.asarray(o) for o in outs]


def base_peak_bytes(model_fn, batch):
    m = model_fn()
    grads = ad.gradients(m.loss, m.variables)
    ex = ad.MemoryExecutor([m.loss] + grads, ctx=ndarray.simgpu(0))
    x, y = m.synthetic_batch(batch, seed=1)
    with use_pool(ndarray.simgpu(0), 1 << 30) as pool:
        ex.run({m.X: x, m.y_: y})
        return pool.stats()["peak"]


POLICIES = [
    (ad.vdnnExecutor, "all"), (ad.vdnnExecutor, "conv"), (ad.recomputeExecutor, "speed"),
    (ad.recomputeExecutor, "memory"), (ad.superNeuronsExecutor, None), (ad.capuchinExecutor, None),
]


@pytest.mark.parametrize("cls,policy", POLICIES)
def test_policy_matches_base_and_saves_memory(cls, policy):
    batch = 8
    ref = reference_run(small_cnn, batch)
    peak_keep = base_peak_bytes(small_cnn, batch)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    ctx = ndarray.simgpu(0)
    ex = cls([m.loss] + grads, ctx=ctx, policy=policy)
    x, y = m.synthetic_batch(batch, seed=1)
    cap = int(peak_keep * 0.8) if cls is ad.capuchinExecutor else 1 << 30
    with use_pool(ctx, cap) as pool:
        for _ in range(2):
            pool.reset_peak()
            outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        peak = pool.stats()["peak"]
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-4, what="%s/%s output %d" % (cls.__name__, policy, i))
    st = ex.stats
    assert st["swap_out_bytes"] > 0 or st["recomputed_nodes"] > 0
    if cls is not ad.capuchinExecutor:      # capuchin only evicts what the budget requires
        assert peak < peak_keep, "%s/%s did not lower the peak (%d vs %d)" % (cls.__name__, policy, peak,
                                                                             peak_keep)


def test_budget_too_small_raises_typed_error():
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    ctx = ndarray.simgpu(0)
    ex = ad.MemoryExecutor([m.loss] + grads, ctx=ctx)
    x, y = m.synthetic_batch(8, seed=1)
    with use_pool(ctx, 64 << 10):
        with pytest.raises(ndarray.OutOfHBMBudget):
            ex.run({m.X: x, m.y_: y})


def test_vdnn_runs_under_a_cap_that_breaks_keep_all():
    batch = 8
    peak_keep = base_peak_bytes(small_cnn, batch)
    cap = int(peak_keep * 0.75)
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(batch, seed=1)
    with use_pool(ctx, cap):
        with pytest.raises(ndarray.OutOfHBMBudget):
            ad.MemoryExecutor([m.loss] + grads, ctx=ctx).run({m.X: x, m.y_: y})
    with use_pool(ctx, cap):
        outs = ad.vdnnExecutor([m.loss] + grads, ctx=ctx, policy="all").run({m.X: x, m.y_: y},
                                                                            convert_to_numpy_ret_vals=True)
    ref = reference_run(small_cnn, batch, steps=1)
    assert_close(outs[0], ref[0], rtol=1e-4)


def test_optimizer_inside_memory_executor_trains():
    m = small_cnn()
    ctx = ndarray.simgpu(0)
    opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
    train = opt.minimize(m.loss)
    ex = ad.recomputeExecutor([m.loss, train], ctx=ctx, policy="speed")
    x, y = m.synthetic_batch(8, seed=1)
    losses = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]) for _ in range(6)]
    assert losses[-1] < losses[0]


def test_tsplit_plan_fits_budget_and_matches_base():
    batch = 8
    ref = reference_run(small_cnn, batch, steps=1)
    peak_keep = base_peak_bytes(small_cnn, batch)
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(batch, seed=1)
    cap = int(peak_keep * 0.8)
    with use_pool(ctx, cap) as pool:
        ex = ad.microopExecutor([m.loss] + grads, ctx=ctx, host_link_gbs=0.05, max_split=4)
        outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        plan = ex.plan_result
        assert plan.fits and plan.predicted_peak_bytes <= cap
        assert pool.stats()["peak"] <= cap
        c = plan.counts()
        assert c["swap"] + c["recompute"] > 0
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-4, what="tsplit output %d" % i)


def test_tsplit_micro_tensors_are_streamed():
    batch = 8
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(batch, seed=1)
    peak_keep = base_peak_bytes(small_cnn, batch)
    ref = reference_run(small_cnn, batch, steps=1)
    with use_pool(ctx, int(peak_keep * 0.8)):
        # a slow link makes every swapped tensor worth splitting
        ex = ad.microopExecutor([m.loss] + grads, ctx=ctx, host_link_gbs=0.001, max_split=4)
        ex.TF32_FLOP_PER_MS = 1e13      # make recompute look expensive so the plan prefers swapping
        ex.HBM_BYTES_PER_MS = 1e3
        outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
    assert ex.stats["swap_out_bytes"] > 0
    if ex.plan_result.counts()["split_tensors"]:
        assert ex.stats["micro_transfers"] > 0
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-4, what="tsplit output %d" % i)


def test_simulator_and_planner_entry_points():
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(8, seed=1)
    peak_keep = base_peak_bytes(small_cnn, 8)
    plan = ad.microopPlanner([m.loss] + grads, ctx=ctx, budget_bytes=int(peak_keep * 0.8)).run({m.X: x, m.y_: y})
    assert plan.fits
    sim = ad.microopOptimizer([m.loss] + grads, ctx=ctx, budget_bytes=int(peak_keep * 0.8)).run({m.X: x, m.y_: y})
    assert sim["fits"] and sim["predicted_peak_bytes"] <= int(peak_keep * 0.8) and sim["predicted_ms"] > 0
    loose = ad.microopOptimizer([m.loss] + grads, ctx=ctx, budget_bytes=1 << 40).run({m.X: x, m.y_: y})
    assert loose["plan"].counts()["swap"] == 0 and loose["plan"].counts()["recompute"] == 0
    assert loose["predicted_ms"] <= sim["predicted_ms"] + 1e-9


def test_max_batch_search_finds_the_boundary():
    ctx = ndarray.simgpu(0)
    peak8 = base_peak_bytes(small_cnn, 8)

    def build():
        m = small_cnn()
        build.m = m
        return ad.MemoryExecutor([m.loss] + ad.gradients(m.loss, m.variables), ctx=ctx)

    def feeds(b):
        x, y = build.m.synthetic_batch(b, seed=1)
        return {build.m.X: x, build.m.y_: y}
    with use_pool(ctx, peak8 + 4096):
        best = ad.max_batch_search(build, feeds, lo=1, hi=32)
    assert 8 <= best < 16
