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


def _tsplit_case(frac, ref, peak_keep, **kw):
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(8, seed=1)
    cap = int(peak_keep * frac)
    with use_pool(ctx, cap) as pool:
        ex = ad.microopExecutor([m.loss] + grads, ctx=ctx, min_split_bytes=1, **kw)
        for _ in range(2):
            pool.reset_peak()
            outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        peak = pool.stats()["peak"]
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-4, what="tsplit %s output %d" % (kw, i))
    return ex, peak, cap


@pytest.mark.parametrize("pieces", [1, 2, 4, 8])
def test_tsplit_micro_ops_match_base_for_every_piece_count(pieces):
    """The lowered graph (every operator as `pieces` micro-ops, batch norm as statistics / finalise /
    normalise stages, reductions accumulated) computes what the whole-batch graph computes."""
    ref = reference_run(small_cnn, 8)
    peak_keep = base_peak_bytes(small_cnn, 8)
    ex, peak, cap = _tsplit_case(1.0, ref, peak_keep, pieces=pieces)
    assert ex.plan_result.pieces == pieces
    assert (ex.stats["micro_ops"] > 0) == (pieces > 1)
    assert ex.stats["micro_ops"] == ex.plan_result.micro_ops


def test_tsplit_plan_fits_half_the_keep_all_peak_and_is_replayed_exactly():
    ref = reference_run(small_cnn, 8)
    peak_keep = base_peak_bytes(small_cnn, 8)
    ex, peak, cap = _tsplit_case(0.5, ref, peak_keep, pieces=4, host_link_gbs=0.5)
    plan = ex.plan_result
    assert plan.fits and plan.footprint_bytes <= cap
    assert ex.stats["micro_ops"] > 0
    assert ex.stats["recomputed_nodes"] + ex.stats["swap_out_bytes"] > 0
    assert ex.stats["recomputed_nodes"] == plan.rebuilds
    assert ex.stats["swap_out_bytes"] == plan.swap_out_bytes and ex.stats["swap_in_bytes"] == plan.swap_in_bytes
    # the step ran inside the region the planner placed it in, plus the results it returns
    results = sum(int(np.prod(o.shape)) * 4 for o in ex.run.__self__.orig_eval_node_list and
                  [np.empty(s) for s in [ex.node_to_shape_map[n] for n in ex.eval_node_list]])
    assert plan.footprint_bytes <= peak <= plan.footprint_bytes + results + 256 * len(ex.eval_node_list)
    assert peak <= cap


def test_tsplit_swaps_micro_tensors_when_the_link_is_fast():
    """With a host link that costs nothing the planner evicts by copying out; every copied-out micro-tensor
    is one transfer with its own event, freed at its planned position and fetched back before its use."""
    ref = reference_run(small_cnn, 8)
    peak_keep = base_peak_bytes(small_cnn, 8)
    ex, peak, cap = _tsplit_case(0.5, ref, peak_keep, pieces=4, host_link_gbs=1e6)
    st = ex.stats
    assert st["micro_ops"] > 0 and st["micro_transfers"] > 0 and st["swap_out_bytes"] > 0
    assert st["planned_frees"] == st["micro_transfers"]
    assert st["swap_in_bytes"] >= st["swap_out_bytes"]
    assert ex.plan_result.counts()["swap"] > 0


@pytest.mark.parametrize("pieces,frac,swap", [(8, 0.3, True), (16, 0.15, True), (16, 0.15, False)])
def test_tsplit_deep_rebuild_chains_replay_the_plan_exactly(pieces, frac, swap):
    """Budgets far below the keep-all peak force rebuild chains that nest several levels deep (a rebuilt
    tensor's inputs are themselves rebuilt, shared inputs are released early and fetched again).  The executor
    must perform exactly the allocations the planner replayed (it raises when it diverges) and compute the
    keep-all results."""
    batch = 16
    ref = reference_run(small_cnn, batch)
    peak_keep = base_peak_bytes(small_cnn, batch)
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(batch, seed=1)
    with use_pool(ctx, int(peak_keep * frac)) as pool:
        ex = ad.microopExecutor([m.loss] + grads, ctx=ctx, pieces=pieces, min_split_bytes=1, allow_swap=swap,
                                host_link_gbs=0.05)
        for _ in range(2):
            outs = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        assert pool.stats()["peak"] <= int(peak_keep * frac)
    assert ex.stats["recomputed_nodes"] == ex.plan_result.rebuilds > len(ex.topo_order) // 8
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-4, what="pieces=%d frac=%s output %d" % (pieces, frac, i))


def test_tsplit_without_a_fitting_plan_raises_the_typed_error():
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    ctx = ndarray.simgpu(0)
    x, y = m.synthetic_batch(8, seed=1)
    with use_pool(ctx, 256 << 10):
        ex = ad.microopExecutor([m.loss] + grads, ctx=ctx, min_split_bytes=1)
        with pytest.raises(ndarray.OutOfHBMBudget):
            ex.run({m.X: x, m.y_: y})


def test_tsplit_dropout_pieces_draw_the_whole_tensor_mask():
    """A dropout computed piece by piece (and rebuilt piece by piece in backward) uses the mask of the
    unsplit tensor: the element index counts from the start of the whole tensor."""
    def build():
        X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
        rs = np.random.RandomState(4)
        w1 = ad.Variable(name="w1", value=rs.normal(scale=0.3, size=(16, 3, 3, 3)).astype(np.float32))
        w2 = ad.Variable(name="w2", value=rs.normal(scale=0.1, size=(16, 16, 3, 3)).astype(np.float32))
        w3 = ad.Variable(name="w3", value=rs.normal(scale=0.1, size=(16 * 4 * 4, 5)).astype(np.float32))
        h = ad.relu_op(ad.conv2d_op(X, w1, padding=1, stride=1))
        h = ad.dropout_op(h, 0.6, seed=77)
        h = ad.relu_op(ad.conv2d_op(h, w2, padding=1, stride=1))
        h = ad.dropout_op(h, 0.8, seed=78)
        h = ad.avg_pool2d_op(h, 4, 4, 0, 4)
        h = ad.array_reshape_op(h, (-1, 16 * 4 * 4))
        loss = ad.softmaxcrossentropy_op(ad.matmul_op(h, w3), y_)
        return X, y_, loss, [w1, w2, w3]
    rs = np.random.RandomState(0)
    x = rs.standard_normal((8, 3, 16, 16)).astype(np.float32)
    y = np.eye(5, dtype=np.float32)[rs.randint(0, 5, 8)]
    ctx = ndarray.simgpu(0)
    X, y_, loss, ws = build()
    base = ad.MemoryExecutor([loss] + ad.gradients(loss, ws), ctx=ctx)
    with use_pool(ctx, 1 << 20) as pool:
        ref = base.run({X: x, y_: y}, convert_to_numpy_ret_vals=True)
        keep_all = pool.stats()["peak"]
    X, y_, loss, ws = build()
    with use_pool(ctx, 1 << 20):
        ex = ad.microopExecutor([loss] + ad.gradients(loss, ws), ctx=ctx, pieces=4, min_split_bytes=1, allow_swap=False,
                                budget_bytes=int(keep_all * 0.6))
        outs = ex.run({X: x, y_: y}, convert_to_numpy_ret_vals=True)
    assert ex.stats["micro_ops"] > 0 and ex.stats["recomputed_nodes"] > 0
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=1e-5, what="dropout under tsplit, output %d" % i)


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


def test_tsplit_region_reuse_is_ordered_by_events_not_by_timing():
    """Every planned block lies on bytes other blocks held before it.  With stream logging on, the executor
    records which stream touched which block when; the happens-before checker then proves that each reuse is
    ordered after the last access to the previous holder by a record -> wait chain (the copy-out of a swapped
    micro-tensor before the planned free, the compute stream's event before a prefetch writes).  Dropping the
    wait in front of a planned free must be caught."""
    from tsplit_b200.runtime import hbcheck
    from tsplit_b200.executors.microop import microopExecutor
    peak_keep = base_peak_bytes(small_cnn, 8)

    def run_logged(ex_cls):
        ctx = ndarray.simgpu(0)
        m = small_cnn()
        grads = ad.gradients(m.loss, m.variables)
        x, y = m.synthetic_batch(8, seed=1)
        with use_pool(ctx, int(peak_keep * 0.5)):
            ex = ex_cls([m.loss] + grads, ctx=ctx, pieces=4, min_split_bytes=1, host_link_gbs=1e6)
            with hbcheck.logging_streams() as log:
                ex.run({m.X: x, m.y_: y})
                log = list(log)
        assert ex.stats["micro_transfers"] > 0 and ex.stats["planned_frees"] > 0
        assert len(ex.hb_accesses) > 1000
        return hbcheck.check(log, ex.hb_accesses)

    assert run_logged(microopExecutor) == []

    class Careless(microopExecutor):
        def _release(self, node, final=False):               # frees a copied-out block without waiting for its copy
            a = self.evicting.pop(node, None)
            if a is not None:
                self.arr.pop(node, None)
                return
            microopExecutor._release(self, node, final)
    violations = run_logged(Careless)
    assert violations and any(v[0] == "write unordered after read" for v in violations)


def test_host_swap_space_is_bounded_with_a_typed_error(monkeypatch):
    """A swap-everything policy whose host copies exceed the host swap budget fails with an error the batch
    sweep catches (a subclass of OutOfHBMBudget), not by exhausting page-locked host memory."""
    from tsplit_b200.ndarray import OutOfHostSwapSpace, OutOfHBMBudget
    monkeypatch.setenv("TSPLIT_HOST_SWAP_GIB", "0.00001")          # ~10 KB
    ctx = ndarray.simgpu(0)
    m = small_cnn()
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(8, seed=1)
    ex = ad.vdnnExecutor([m.loss] + grads, ctx=ctx, policy="all")
    with pytest.raises(OutOfHostSwapSpace) as e:
        ex.run({m.X: x, m.y_: y})
    assert isinstance(e.value, OutOfHBMBudget) and "host swap space" in str(e.value)
    monkeypatch.delenv("TSPLIT_HOST_SWAP_GIB")
    ex2 = ad.vdnnExecutor([m.loss] + grads, ctx=ctx, policy="all")
    ex2.run({m.X: x, m.y_: y})
    assert ex2.host_bytes > 0
