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


def assert_same_training_signal(outs, ref, what):
    """Loss to TF32 tolerance; gradients by relative L2 distance.  A convolution over a batch piece accumulates
    in another order than over the whole batch, the last bits of an activation differ, and a ReLU whose input
    sits at zero may then switch for one sample: that changes that sample's gradient contribution entirely
    (measured on this 16-sample net: 3-7 % of the gradient norm from one switched unit), which an element-wise
    comparison cannot tell from an error.  The exact element-wise comparison of the same lowering runs on the
    simulated device in fp32 NumPy (tests/test_memory_executors.py); a wrong kernel moves the gradient by far more
    than this bound."""
    assert_close(outs[0], ref[0], rtol=2e-3, what=what + " loss")
    for i, (o, r) in enumerate(zip(outs[1:], ref[1:])):
        o, r = np.asarray(o, np.float64), np.asarray(r, np.float64)
        rel = np.linalg.norm(o - r) / max(np.linalg.norm(r), 1e-12)
        assert rel < 0.15, "%s gradient %d: relative L2 distance %.3f" % (what, i, rel)


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


def test_capuchin_under_a_tight_cap(keep_all):
    ref, peak_keep = keep_all
    cap = int(peak_keep * 0.7)
    with pytest.raises(ndarray.OutOfHBMBudget):
        run(ad.MemoryExecutor, None, cap, steps=1)
    outs, peak, ex = run(ad.capuchinExecutor, None, cap, steps=3)
    assert peak <= cap
    for i, (o, r) in enumerate(zip(outs, ref)):
        assert_close(o, r, rtol=2e-3, what="capuchin output %d" % i)


@pytest.mark.parametrize("pieces", [1, 2, 4])
def test_tsplit_micro_ops_on_gpu_match_keep_all(pieces, keep_all):
    """Every operator as `pieces` micro-ops on the hand-written kernels: convolutions on batch views,
    piece-wise batch-norm statistics combined by one finalise launch, accumulated filter gradients."""
    ref, peak_keep = keep_all
    outs, peak, ex = run(ad.microopExecutor, None, 4 << 30, steps=2, pieces=pieces, min_split_bytes=1)
    assert ex.plan_result.pieces == pieces
    assert (ex.stats["micro_ops"] > 0) == (pieces > 1)
    if pieces == 1:
        for i, (o, r) in enumerate(zip(outs, ref)):
            assert_close(o, r, rtol=2e-3, what="tsplit pieces=1 output %d" % i)
    else:
        assert_same_training_signal(outs, ref, "tsplit pieces=%d" % pieces)


def test_tsplit_swaps_and_rebuilds_micro_tensors_under_a_tight_cap(keep_all):
    """Half of the keep-all peak: the plan must move micro-tensors over the host link (fast link assumed, so
    the planner prefers copies) and the step must stay inside the region the planner placed it in."""
    ref, peak_keep = keep_all
    cap = int(peak_keep * 0.5)
    outs, peak, ex = run(ad.microopExecutor, None, cap, steps=3, pieces=4, min_split_bytes=1, host_link_gbs=1e5)
    st, plan = ex.stats, ex.plan_result
    assert plan.fits and peak <= cap
    assert st["micro_ops"] > 0
    assert st["swap_out_bytes"] > 0 and st["micro_transfers"] > 0 and st["planned_frees"] == st["micro_transfers"]
    assert st["swap_out_bytes"] == plan.swap_out_bytes and st["swap_in_bytes"] == plan.swap_in_bytes
    assert_same_training_signal(outs, ref, "tsplit with swaps")
    # and with the real link figure the planner rebuilds instead
    outs, peak, ex = run(ad.microopExecutor, None, cap, steps=3, pieces=4, min_split_bytes=1, allow_swap=False)
    assert ex.stats["recomputed_nodes"] > 0 and ex.stats["micro_ops"] > 0 and peak <= cap
    assert_same_training_signal(outs, ref, "tsplit with rebuilds")


def test_tsplit_chooses_pieces_and_trains(keep_all):
    ctx = ndarray.gpu(0)
    _, peak_keep = keep_all
    m = net()
    opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
    train = opt.minimize(m.loss)
    x, y = m.synthetic_batch(32, seed=2)
    with use_pool(ctx, int(peak_keep * 0.9)):          # batch 32 in less than what batch 16 needs to keep everything
        ex = ad.microopExecutor([m.loss, train], ctx=ctx, min_split_bytes=1)
        losses = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]) for _ in range(6)]
    plan = ex.plan_result
    assert plan.fits and plan.pieces in (1, 2, 4, 8, 16)
    assert ex.stats["recomputed_nodes"] + ex.stats["swap_out_bytes"] > 0
    assert losses[-1] < losses[0]


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
            assert ex._step_graph is not None, "the step was not captured: %s" % getattr(ex, "replay_failure", "")
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
            assert ex._step_graph is not None, "the step was not captured: %s" % getattr(ex, "replay_failure", "")
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


def test_base_executor_graph_replay_reads_each_steps_feeds():
    """The base executor's captured step reads its feeds from fixed buffers that are refreshed every step:
    feeding two different batches (as different device arrays) gives the eager results, and the optimizer's
    step count keeps counting through the replays."""
    ctx = ndarray.gpu(0)
    outs = []
    for use_graph in (False, True):
        m = net()
        opt = optimizer.MomentumOptimizer(learning_rate=0.01, momentum=0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        ex = ad.Executor([m.loss, train], ctx=ctx, use_graph=use_graph)
        feeds = []
        for seed in (2, 9):
            x, y = m.synthetic_batch(16, seed=seed)
            feeds.append({m.X: ndarray.array(x, ctx), m.y_: ndarray.array(y, ctx)})
        vals = [float(ex.run(feeds[i % 2])[0].asnumpy().reshape(-1)[0]) for i in range(6)]
        outs.append(vals)
        assert opt.step_count == 6
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-4)
    assert abs(outs[0][0] - outs[0][1]) > 1e-6


def test_tsplit_step_with_swaps_replays_from_one_cuda_graph(keep_all):
    """A planned step is static (fixed offsets, fixed pinned buffers, planned events), so the whole step with
    its copy-outs, planned frees and prefetches on the copy streams is captured into one CUDA graph; the
    replayed steps train exactly like the eager ones."""
    ctx = ndarray.gpu(0)
    _, peak_keep = keep_all
    runs = []
    for use_graph in (False, True):
        m = net()
        opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        x, y = m.synthetic_batch(16, seed=2)
        with use_pool(ctx, int(peak_keep * 0.5)):
            ex = ad.microopExecutor([m.loss, train], ctx=ctx, pieces=4, min_split_bytes=1, host_link_gbs=1e5,
                                    use_graph=use_graph)
            losses = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]) for _ in range(7)]
        assert ex.stats["swap_out_bytes"] > 0 and ex.stats["micro_ops"] > 0
        if use_graph:
            assert ex._step_graph is not None, "the step was not captured: %s" % getattr(ex, "replay_failure", "")
        assert opt.step_count == 7
        runs.append(losses)
    np.testing.assert_allclose(runs[1], runs[0], rtol=1e-5)
    assert runs[0][-1] < runs[0][0]


def test_tsplit_step_with_swaps_replays_from_the_native_tape(keep_all):
    """The same planned step recorded as a list of native calls (kernel entries, event records, stream waits,
    copies) and replayed by the C++ loop: steps train exactly like the eager ones, and the replay's host time per
    action is reported."""
    from tsplit_b200.runtime import tape
    assert tape.available()
    ctx = ndarray.gpu(0)
    _, peak_keep = keep_all
    runs = []
    for use_graph in (False, "tape"):
        m = net()
        opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
        train = opt.minimize(m.loss)
        x, y = m.synthetic_batch(16, seed=2)
        with use_pool(ctx, int(peak_keep * 0.5)):
            ex = ad.microopExecutor([m.loss, train], ctx=ctx, pieces=4, min_split_bytes=1, host_link_gbs=1e5,
                                    use_graph=use_graph)
            losses = [float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]) for _ in range(7)]
        assert ex.stats["swap_out_bytes"] > 0 and ex.stats["micro_ops"] > 0
        if use_graph:
            assert ex._step_graph is not None, "the step was not recorded: %s" % getattr(ex, "replay_failure", "")
            us, actions = ex.replay_host_us()
            names = set(ex._step_graph.tape.names)
            assert {"tsb_memcpy_async", "tsb_event_record", "tsb_stream_wait_event"} <= names
            assert actions > 100 and 0 < us / actions < 50.0
            print("native replay: %d actions, %.1f us host time, %.2f us per action" % (actions, us, us / actions))
        assert opt.step_count == 7
        runs.append(losses)
    np.testing.assert_allclose(runs[1], runs[0], rtol=1e-5)
    assert runs[0][-1] < runs[0][0]


def test_native_tape_replay_with_adam_matches_eager():
    ctx = ndarray.gpu(0)
    outs = []
    for use_graph in (False, "tape"):
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
            assert ex._step_graph is not None, "the step was not recorded: %s" % getattr(ex, "replay_failure", "")
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-4)


def test_device_timeline_of_a_swap_plan(tmp_path):
    """Tracing brackets every launch and copy with timing events on its own stream: the device records carry
    kernel / copy durations and show copies on streams other than the compute stream."""
    from tsplit_b200.utils import trace
    recs = []
    outs, peak, ex = run(ad.vdnnExecutor, "conv", 4 << 30, steps=1, trace=recs)
    dev = ex.device_trace()
    kinds = {r[0] for r in dev}
    assert {"op", "swap_out", "swap_in"} <= kinds
    assert all(r[5] >= r[4] >= 0.0 for r in dev)
    op_streams = {r[3] for r in dev if r[0] == "op"}
    copy_streams = {r[3] for r in dev if r[0] in ("swap_out", "swap_in")}
    assert len(op_streams) == 1 and not (op_streams & copy_streams)
    assert sum(r[5] - r[4] for r in dev if r[0] == "op") > 0.0
    doc = trace.to_chrome_trace(recs, str(tmp_path / "t.json"), device_records=dev)
    assert any(e["pid"] == 1 and e["cat"].startswith("device:") for e in doc["traceEvents"])
