"""Auxiliary subsystems: checkpoint format, metrics, graph DOT, trace export,
happens-before checker, profiler records, pool semantics, micro-tensor helpers."""
import json
import pickle

import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad, optimizer, model, metrics, graphboard, profiler
from tsplit_b200.models import mlp
from tsplit_b200.runtime import hbcheck
from tsplit_b200.runtime.pool import MemoryPool
from tsplit_b200.utils import trace


def test_saver_loader_roundtrip_and_python2_pickles(tmp_path):
    path = str(tmp_path / "ckpt.pkl")
    s = model.Saver(path)
    s.append("w", np.arange(6, dtype=np.float32).reshape(2, 3))
    s.append("step", 7)
    s.save()
    l = model.Loader(path)
    np.testing.assert_array_equal(l.load("w"), np.arange(6, dtype=np.float32).reshape(2, 3))
    assert l.load("step") == 7
    with open(path, "rb") as f:
        assert isinstance(pickle.load(f), dict)        # one pickled dict, as in the reference
    # protocol-0 file with a latin1 byte string, as Python 2 would write it
    p2 = str(tmp_path / "py2.pkl")
    with open(p2, "wb") as f:
        f.write(b"(dp0\nS'name'\np1\nS'caf\\xe9'\np2\ns.")
    assert model.Loader(p2).load("name") == "caf\xe9"


def test_optimizer_state_checkpoint_resume(tmp_path):
    def make():
        m = mlp((16, 8, 4), seed=1)
        opt = optimizer.AdamOptimizer(0.01)
        train = opt.minimize(m.loss)
        return m, opt, ad.Executor([m.loss, train], ctx=None)
    m, opt, ex = make()
    x, y = m.synthetic_batch(8)
    for _ in range(3):
        ex.run({m.X: x, m.y_: y})
    path = str(tmp_path / "state.pkl")
    s = model.Saver(path)
    s.append_variables(m.variables)
    s.append_optimizer(opt)
    s.save()
    cont = [float(ex.run({m.X: x, m.y_: y})[0][0]) for _ in range(2)]
    m2, opt2, ex2 = make()
    l = model.Loader(path)
    l.restore_variables(m2.variables)
    l.restore_optimizer(opt2)
    resumed = [float(ex2.run({m2.X: x, m2.y_: y})[0][0]) for _ in range(2)]
    np.testing.assert_allclose(resumed, cont, rtol=1e-5)


def test_metrics_against_direct_definitions():
    r = np.random.RandomState(0)
    labels = np.eye(4)[r.randint(0, 4, 64)]
    preds = metrics.softmax_func(r.randn(64, 4))
    assert abs(metrics.accuracy(labels, preds) - np.mean(labels.argmax(1) == preds.argmax(1))) < 1e-12
    cm = metrics.confusion_matrix_one_hot(labels, preds)
    assert np.all(cm["tp"] + cm["fn"] == labels.sum(0))
    p = metrics.precision_score_one_hot(labels, preds)
    rcl = metrics.recall_score_one_hot(labels, preds)
    f = metrics.f_score_one_hot(labels, preds)
    np.testing.assert_allclose(f, 2 * p * rcl / (p + rcl), rtol=1e-5)
    assert 0 <= metrics.precision_score_one_hot(labels, preds, average="micro") <= 1
    assert 0 <= metrics.recall_score_one_hot(labels, preds, average="macro") <= 1
    y = r.randint(0, 2, 500)
    score = np.clip(y * 0.3 + r.rand(500) * 0.7, 0, 1)
    auc = metrics.auc(y, score, num_thresholds=200)
    order = np.argsort(score)
    ranks = np.empty(500)
    ranks[order] = np.arange(1, 501)
    exact = (ranks[y == 1].sum() - y.sum() * (y.sum() + 1) / 2) / (y.sum() * (500 - y.sum()))
    assert abs(auc - exact) < 0.02
    with pytest.raises(ValueError):
        metrics.confusion_matrix_at_thresholds(y, score, [0.5], includes=("xx",))


def test_graphboard_dot_and_trace_export(tmp_path):
    m = mlp((16, 8, 4))
    ex = ad.Executor([m.loss], ctx=None)
    x, y = m.synthetic_batch(4)
    ex.run({m.X: x, m.y_: y})
    dot = graphboard.to_dot(ex)
    assert dot.startswith("digraph") and "MatMul" in dot and "->" in dot
    path, _ = graphboard.show(ex, out_dir=str(tmp_path), serve=False)
    assert open(path).read() == dot
    recs = []
    grads = ad.gradients(m.loss, m.variables)
    ex2 = ad.vdnnExecutor([m.loss] + grads, ctx=ndarray.simgpu(0), policy="all", trace=recs)
    ex2.run({m.X: x, m.y_: y})
    doc = trace.to_chrome_trace(recs, str(tmp_path / "t.json"))
    kinds = {e["cat"] for e in doc["traceEvents"]}
    assert "op" in kinds and "swap_out" in kinds and "swap_in" in kinds
    json.load(open(str(tmp_path / "t.json")))


def test_happens_before_checker_flags_missing_wait():
    # stream 1 writes buffer A then records e; stream 2 reads A with and without waiting on e
    good = [("record", 1, 10), ("wait", 2, 10), ("record", 2, 11)]
    assert hbcheck.check(good, [(0, 1, "A", True), (2, 2, "A", False)]) == []
    bad = [("record", 1, 10), ("record", 2, 11)]
    v = hbcheck.check(bad, [(0, 1, "A", True), (1, 2, "A", False)])
    assert v and v[0][0] == "unordered after write"
    synced = [("record", 1, 10), ("sync", 1, -1), ("record", 2, 11)]
    assert hbcheck.check(synced, [(0, 1, "A", True), (2, 2, "A", False)]) == []


def test_executor_streams_follow_record_wait_discipline():
    m = mlp((16, 8, 4))
    grads = ad.gradients(m.loss, m.variables)
    x, y = m.synthetic_batch(4)
    with hbcheck.logging_streams() as log:
        ex = ad.vdnnExecutor([m.loss] + grads, ctx=ndarray.simgpu(0), policy="all")
        ex.run({m.X: x, m.y_: y})
        kinds = [k for k, _, _ in log]
    # every swap copy is bracketed by a record on the producer stream and a wait on the copy stream
    assert kinds.count("wait") >= 2 and kinds.count("record") >= kinds.count("wait")


def test_profiler_record_and_constants():
    m = mlp((16, 8, 4))
    ex = ad.Executor([m.loss], ctx=None)
    x, y = m.synthetic_batch(4)
    ex.run({m.X: x, m.y_: y})
    node = [n for n in ex.topo_order if n.op.name == "MatMul"][0]
    p = profiler.profile_node(node, [ex.node_to_shape_map[i] for i in node.inputs], ex.node_to_shape_map[node])
    assert p.time > 0 and p.output_memory > 0 and p.swap_time() == p.output_memory / profiler.BandWidth
    profiler.PrintProfiler(p)


def test_pool_best_fit_coalescing_and_two_ended_allocation():
    pool = MemoryPool(ndarray.simgpu(0), 1 << 20)
    a, _ = pool.alloc(100 * 1024)
    b, _ = pool.alloc(200 * 1024)
    c, _ = pool.alloc(100 * 1024)
    hi, _ = pool.alloc(64 * 1024, long_lived=True)
    assert hi > c                                   # carved from the top
    pool.free(b)
    d, _ = pool.alloc(150 * 1024)                   # best fit re-uses b's hole
    assert d == b
    pool.free(a), pool.free(c), pool.free(d), pool.free(hi)
    st = pool.stats()
    assert st["used"] == 0 and st["largest_free"] == st["capacity"]      # fully coalesced
    assert pool.try_alloc(1 << 20) and not pool.try_alloc((1 << 20) + 256)
    with pytest.raises(ndarray.OutOfHBMBudget):
        pool.alloc(2 << 20)


def test_micro_tensor_helpers():
    a = ndarray.array(np.arange(2 * 10 * 3 * 3, dtype=np.float32).reshape(2, 10, 3, 3), ndarray.cpu(0))
    parts = a.split_tensor(3, "channel")
    assert [p.shape[1] for p in parts] == [4, 3, 3]
    np.testing.assert_array_equal(parts[1].asnumpy(), a.asnumpy()[:, 4:7])
    assert ndarray.split_shape((7, 5), 3, "batch") == [[3, 5], [2, 5], [2, 5]]
    m = ndarray.slice_for_micro_tensor(a, 1, 2, "batch")
    np.testing.assert_array_equal(m.asnumpy(), a.asnumpy()[1:2])
    inp, out = ndarray.tensor_reuse((8, 4), (8, 4), pieces=4, overlap_pieces=3, ctx=ndarray.cpu(0))
    assert inp._holder.shape[0] == 32 + 8 * (4 - 3)       # output + one un-overlapped input piece
    assert inp.shape == (8, 4) and out.shape == (8, 4)


def test_dropout_draws_a_new_mask_every_step_and_backward_reuses_it():
    from tsplit_b200 import gpu_ops as ad
    x = ad.Variable("x")
    y = ad.dropout_op(x, 0.5, seed=11)
    (gx,) = ad.gradients(ad.reduce_sum_op(y, [0, 1]), [x])
    ex = ad.Executor([y, gx], ctx=None)
    xv = np.ones((8, 64), np.float32)
    y0, g0 = ex.run({x: xv})
    y1, g1 = ex.run({x: xv})
    assert np.array_equal(y0 != 0, g0 != 0) and np.array_equal(y1 != 0, g1 != 0)    # same mask within a step
    assert not np.array_equal(y0 != 0, y1 != 0)                                     # a new one the next step
    assert 0.3 < (y0 != 0).mean() < 0.7


def test_pool_compaction_moves_live_blocks_and_keeps_their_values():
    """Fragment a simulated-device pool, compact it through an executor that owns every live block and check
    that the arrays were re-bound to their bytes; a pool with blocks the executor does not own is left alone."""
    from tsplit_b200.runtime.pool import use_pool
    from tsplit_b200.models import vgg
    ctx = ndarray.simgpu(0)
    m = vgg(16, num_classes=10, image=32, width_div=16, fc_width=32, seed=3)
    ex = ad.MemoryExecutor([m.loss], ctx=ctx)
    with use_pool(ctx, 64 << 10) as pool:
        ex._reset_state()                            # the executor only lends its compaction logic here
        keep, holes = {}, []
        for i in range(8):
            a = ndarray.empty((1024,), ctx)          # 4 KiB each
            a.numpy_view()[...] = float(i)
            if i % 2 == 0:
                keep[i] = a
            else:
                holes.append(a)
        for a in holes:
            a._release()
        st = pool.stats()
        assert st["largest_free"] < st["free"]          # fragmented
        ex.arr = {("t", i): a for i, a in keep.items()}
        ex._no_spill = False
        assert ex._compact(st["largest_free"] + 4096)
        assert pool.stats()["largest_free"] == pool.stats()["free"]
        for i, a in keep.items():
            assert np.all(a.numpy_view() == float(i)), "block %d lost its bytes" % i
        # a block held by somebody else: the executor must refuse to move anything
        other = ndarray.empty((1024,), ctx)
        other.numpy_view()[...] = 99.0
        hole = ndarray.empty((1024,), ctx)
        tail = ndarray.empty((1024,), ctx)
        ex.arr[("t", "tail")] = tail
        hole._release()
        assert not ex._compact(pool.stats()["free"])
        assert np.all(other.numpy_view() == 99.0)


def test_pool_guard_zones_catch_a_write_past_the_end():
    """Debug mode of the pool (the stand-in for a memory checker): a write that runs past a tensor's end
    lands in the guard zone behind its block and is reported when the block is freed."""
    from tsplit_b200.runtime.pool import MemoryPool, PoolCorruption
    ctx = ndarray.simgpu(0)
    pool = MemoryPool(ctx, 1 << 20, canary=True)
    ndarray.set_pool(ctx, pool)
    try:
        a = ndarray.empty((100,), ctx)
        b = ndarray.empty((100,), ctx)
        a.numpy_view()[...] = 1.0
        pool.check_canaries()                      # clean
        a._release()                               # clean free
        flat = pool.arena.numpy()
        start = b._block // 4
        flat[start:start + 104] = 7.0              # 4 floats too many
        with pytest.raises(PoolCorruption):
            pool.check_canaries()
        with pytest.raises(PoolCorruption):
            b._release()
    finally:
        ndarray.set_pool(ctx, None)


def test_rank_binds_its_threads_to_the_cpus_next_to_its_gpu(monkeypatch):
    """``bind_to_gpu`` applies NVML's CPU set of the GPU to the calling thread (a fake NVML here: no GPU setting is
    read or changed), leaves the thread alone when NVML is missing or the set is not usable, and honours the switch."""
    import os
    import sys
    import types
    from tsplit_b200.utils.affinity import bind_to_gpu
    if not hasattr(os, "sched_setaffinity"):
        pytest.skip("no sched_setaffinity on this platform")
    before = os.sched_getaffinity(0)
    want = set(sorted(before)[:max(1, len(before) // 2)])
    if want == before:
        pytest.skip("only one CPU available")
    asked = []
    fake = types.ModuleType("pynvml")
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: asked.append(i) or ("gpu", i)
    fake.nvmlDeviceGetHandleByUUID = lambda u: ("gpu", u)
    mask = [sum(1 << (c - 64 * w) for c in want if 64 * w <= c < 64 * (w + 1)) for w in range((max(before) // 64) + 1)]
    fake.nvmlDeviceGetCpuAffinity = lambda h, n: (mask + [0] * n)[:n]
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    try:
        assert bind_to_gpu(3) == sorted(want) and asked == [3]
        assert os.sched_getaffinity(0) == want
        os.sched_setaffinity(0, before)
        monkeypatch.setenv("TSPLIT_BIND_CPUS", "0")
        assert bind_to_gpu(3) is None and os.sched_getaffinity(0) == before
        monkeypatch.delenv("TSPLIT_BIND_CPUS")
        fake.nvmlDeviceGetCpuAffinity = lambda h, n: [0] * n          # a CPU set outside this process's cpuset
        assert bind_to_gpu(0) is None and os.sched_getaffinity(0) == before
    finally:
        os.sched_setaffinity(0, before)
