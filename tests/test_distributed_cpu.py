"""Host-side distributed pieces, exercised with threads / gloo ranks on CPU:
parameter-server semantics against a dict oracle (BSP = sum of pushes, ASP
eventual), at-least-once delivery under message loss, heartbeats, the TCP ring
all-reduce (including a neighbour that never joins), communicator classes, the
in-graph gradient exchange nodes and the CPU operator library."""
import os
import sys
import socket
import threading
import time

import numpy as np
import pytest

from tsplit_b200 import ndarray, gpu_ops as ad, cpu_links
from tsplit_b200.models import mlp
from tsplit_b200.parallel.ps import ParameterServer, PSVector, PSMatrix
from tsplit_b200.parallel.ring import RingAllReduce, RingError
from tsplit_b200.parallel import graph_hooks


def test_ps_dense_bsp_equals_sum_of_pushes():
    workers, n = 4, 1001
    ps = ParameterServer(num_servers=3, num_workers=workers)
    ps.init("w", np.zeros(n, np.float32))
    r = np.random.RandomState(0)
    deltas = [r.randn(n).astype(np.float32) for _ in range(workers)]
    results = [None] * workers

    def work(i):
        results[i] = ps.push_pull("w", deltas[i], mode="BSP", worker=i)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(workers)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    oracle = np.sum(deltas, axis=0)
    for res in results:                       # every worker sees every push after the barrier
        np.testing.assert_allclose(res, oracle, rtol=1e-5, atol=1e-5)


def test_ps_asp_is_eventually_consistent():
    ps = ParameterServer(num_servers=2, num_workers=2)
    ps.init("w", length=64)
    seen = []

    def work(i):
        for k in range(5):
            seen.append(ps.push_pull("w", np.full(64, 1.0, np.float32), mode="ASP", worker=i).copy())
    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    final = PSVector.pull(type("V", (), {"ps": ps, "name": "w", "length": 64})())
    np.testing.assert_allclose(final, np.full(64, 10.0))
    assert all(1.0 <= s[0] <= 10.0 for s in seen)


def test_ps_survives_dropped_messages_exactly_once():
    ps = ParameterServer(num_servers=4, num_workers=1, drop_percent=30, resend_timeout_ms=1)
    ps.init("w", length=4000)
    total = np.zeros(4000, np.float32)
    r = np.random.RandomState(1)
    for _ in range(10):
        d = r.randn(4000).astype(np.float32)
        total += d
        ps.wait(ps.push("w", d))
    out = np.empty(4000, np.float32)
    ps.wait(ps.pull("w", out))
    np.testing.assert_allclose(out, total, rtol=1e-5, atol=1e-5)      # applied once despite re-sends
    st = ps.stats()
    assert st["dropped"] > 0 and st["resent"] > 0


def test_ps_functions_sparse_and_columns():
    ps = ParameterServer(num_servers=3, num_workers=1)
    a = np.arange(12, dtype=np.float32)
    b = np.ones(12, np.float32)
    ps.init("a", a)
    ps.init("b", b)
    assert abs(ps.norm2("a") - np.linalg.norm(a)) < 1e-4
    assert ps.nnz("a") == 11
    assert abs(ps.dot("a", "b") - a.sum()) < 1e-4
    ps.axpy("a", "b", 2.0)
    out = np.empty(12, np.float32)
    ps.wait(ps.pull("b", out))
    np.testing.assert_allclose(out, 1 + 2 * a)
    m = PSMatrix(ps, "m", 4, 6)
    m.push_rows([1, 3], np.ones((2, 6), np.float32))
    m.push_cols(2, 4, np.full((4, 2), 5.0, np.float32))
    full = m.pull_rows([0, 1, 2, 3])
    expect = np.zeros((4, 6), np.float32)
    expect[[1, 3]] += 1
    expect[:, 2:4] += 5
    np.testing.assert_allclose(full, expect)
    np.testing.assert_allclose(m.pull_cols(2, 4), expect[:, 2:4])


def test_ps_heartbeat_detects_a_silent_node():
    ps = ParameterServer(1, 1)
    ps.heartbeat(7)
    ps.heartbeat(9)
    time.sleep(0.06)
    ps.heartbeat(9)
    assert ps.dead_nodes(timeout_ms=40) == [7]


def _free_port_base(n):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port if port + n < 65000 else 30000


def test_ring_allreduce_over_tcp_matches_numpy():
    world, n = 3, 1000
    base = _free_port_base(world)
    r = np.random.RandomState(2)
    data = [r.randn(n).astype(np.float32) for _ in range(world)]
    outs, errs = [None] * world, []

    def work(i):
        try:
            ring = RingAllReduce(world, i, base_port=base)
            outs[i] = ring.allReduce(data[i].copy(), average=True)
            ring.close()
        except Exception as e:      # pragma: no cover
            errs.append(e)
    ts = [threading.Thread(target=work, args=(i,)) for i in range(world)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    assert not errs, errs
    for o in outs:
        np.testing.assert_allclose(o, np.mean(data, axis=0), rtol=1e-5, atol=1e-6)


def test_ring_reports_a_rank_that_never_joins():
    base = _free_port_base(2)
    with pytest.raises(RingError):
        RingAllReduce(2, 0, base_port=base, timeout_ms=300)       # rank 1 never starts


def test_ps_gradients_train_through_the_server():
    m = mlp((16, 8, 4), seed=2)
    ps = ParameterServer(num_servers=2, num_workers=1)
    pulled = graph_hooks.ps_gradients(m.loss, m.variables, ps, lr=0.1)
    ex = ad.Executor([m.loss] + pulled, ctx=None)
    x, y = m.synthetic_batch(16)
    losses = [float(ex.run({m.X: x, m.y_: y})[0][0]) for _ in range(8)]
    assert losses[-1] < losses[0]


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    from tsplit_b200.communicator import mpi_communicator
    comm = mpi_communicator()
    comm.MPI_Init()
    arr = np.full(5, float(rank + 1), np.float32)
    comm.allReduce(arr)
    m = mlp((8, 4, 2), seed=3)
    grads = graph_hooks.distributed_gradients(m.loss, m.variables, comm)
    ex = ad.Executor(grads, ctx=None)
    x, y = m.synthetic_batch(4, seed=rank)
    g = ex.run({m.X: x, m.y_: y})
    q.put((rank, arr.tolist(), [np.asarray(t).copy() for t in g]))
    dist.barrier()
    comm.finish()


def test_gloo_ranks_allreduce_and_distributed_gradients():
    import torch.multiprocessing as mp
    world, port = 2, _free_port_base(1)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    [p.start() for p in procs]
    got = sorted([q.get(timeout=120) for _ in range(world)], key=lambda t: t[0])
    [p.join(timeout=60) for p in procs]
    assert got[0][1] == [3.0] * 5 and got[1][1] == [3.0] * 5
    for a, b in zip(got[0][2], got[1][2]):          # averaged gradients are identical on both ranks
        np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)


def test_cpu_operator_library_against_numpy():
    r = np.random.RandomState(4)
    a, b = r.randn(17, 9).astype(np.float32), r.randn(9, 13).astype(np.float32)
    c = np.empty((17, 13), np.float32)
    cpu_links.matrix_multiply(a, b, c)
    np.testing.assert_allclose(c, a @ b, rtol=1e-4, atol=1e-5)
    at = np.ascontiguousarray(a.T)
    cpu_links.matrix_multiply(at, b, c, trans_a=True)
    np.testing.assert_allclose(c, a @ b, rtol=1e-4, atol=1e-5)
    from tsplit_b200.ops.conv import np_conv2d
    x, w = r.randn(2, 3, 9, 9).astype(np.float32), r.randn(4, 3, 3, 3).astype(np.float32)
    y = np.empty((2, 4, 5, 5), np.float32)
    cpu_links.conv2d(x, w, y, padding=1, stride=2)
    np.testing.assert_allclose(y, np_conv2d(x, w, 1, 1, 2), rtol=1e-4, atol=1e-4)
    from tsplit_b200.ops.pool import np_max_pool, np_avg_pool
    yp = np.empty((2, 3, 4, 4), np.float32)
    cpu_links.pool2d(0, x, yp, 3, 3, 0, 2)
    np.testing.assert_allclose(yp, np_max_pool(x, 3, 3, 0, 2))
    cpu_links.pool2d(1, x, yp, 3, 3, 0, 2)
    np.testing.assert_allclose(yp, np_avg_pool(x, 3, 3, 0, 2), rtol=1e-5, atol=1e-6)
    logits = r.randn(6, 10).astype(np.float32)
    labels = np.eye(10, dtype=np.float32)[r.randint(0, 10, 6)]
    loss, dx = np.empty(1, np.float32), np.empty((6, 10), np.float32)
    cpu_links.softmax_crossentropy(logits, labels, loss, dx)
    sm = np.exp(logits - logits.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    np.testing.assert_allclose(loss[0], np.mean(-np.sum(labels * np.log(sm), 1)), rtol=1e-5)
    np.testing.assert_allclose(dx, (sm - labels) / 6, rtol=1e-4, atol=1e-6)
    p, g = r.randn(100).astype(np.float32), r.randn(100).astype(np.float32)
    m_, v_ = np.zeros(100, np.float32), np.zeros(100, np.float32)
    p0 = p.copy()
    cpu_links.optimizer_update(4, p, g, m_, v_, [0.01, 0.9, 0.999, 0.9, 0.999, 1e-7])
    m_ref, v_ref = 0.1 * g, 0.001 * g * g
    np.testing.assert_allclose(p, p0 - 0.01 * (m_ref / 0.1) / (np.sqrt(v_ref / 0.001) + 1e-7), rtol=1e-4)


def test_cpu_context_executor_runs_on_the_native_host_kernels():
    """``Executor(ctx=ndarray.cpu(0))`` sends matmul / conv / pool / element-wise / cross-entropy through the
    OpenMP library and gives what the NumPy oracle (``ctx=None``) gives."""
    from tsplit_b200.models import vgg
    outs = []
    for ctx in (None, ndarray.cpu(0)):
        m = vgg(16, num_classes=10, image=32, width_div=16, fc_width=32, seed=3)
        grads = ad.gradients(m.loss, m.variables)
        ex = ad.Executor([m.loss] + grads, ctx=ctx)
        x, y = m.synthetic_batch(4, seed=1)
        before = cpu_links.CALLS[0]
        outs.append([np.asarray(o) for o in ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)])
        used = cpu_links.CALLS[0] - before
        assert (used > 20) == (ctx is not None), "native kernel calls: %d" % used
    for a, b in zip(outs[1], outs[0]):
        np.testing.assert_allclose(a, b, rtol=2e-4, atol=2e-5)


def _run_ps_workers(port, workers, mode, env=None):
    import subprocess
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ps_net_worker.py")
    e = dict(os.environ, **(env or {}))
    procs = [subprocess.Popen([sys.executable, worker, str(port), str(r), str(workers), mode], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True, env=e) for r in range(workers)]
    return [(p.wait(timeout=120), p.stdout.read()) for p in procs]


def test_parameter_server_across_processes_over_tcp():
    """Server in this process (listening on the loopback interface), two workers in child processes: BSP push-pull
    sums every worker's delta each step, sparse rows arrive, and both workers say goodbye."""
    from tsplit_b200.parallel import ps_net
    srv = ps_net.serve(num_servers=2, num_workers=2)
    try:
        res = _run_ps_workers(srv.port, 2, "train")
        for rc, out in res:
            assert rc == 0 and "WORKER_OK" in out, out
        assert srv.wait_for_workers(timeout=10) and srv.gone() == 0
        w = np.empty(1000, np.float32)
        srv.store.wait(srv.store.pull("w", w))
        np.testing.assert_allclose(w, (1 + 2) * (1 + 2 + 3))
    finally:
        srv.stop()


def test_a_worker_that_leaves_is_seen_by_the_server_and_times_out_the_others():
    """Rank 1 exits between steps without a goodbye: the server counts it as gone and releases (or refuses) the
    barrier rank 0 waits in, so rank 0's BSP step ends with PSConnectionError (at the latest after its own request
    timeout) instead of hanging."""
    from tsplit_b200.parallel import ps_net
    srv = ps_net.serve(num_servers=1, num_workers=2)
    try:
        res = _run_ps_workers(srv.port, 2, "leave_early", env={"PS_TIMEOUT": "2"})
        assert res[1][0] == 0
        assert res[0][0] == 3 and "TIMEOUT" in res[0][1], res[0]
        t0 = time.time()
        while srv.gone() < 1 and time.time() - t0 < 5:
            time.sleep(0.05)
        assert srv.gone() >= 1
    finally:
        srv.stop()
