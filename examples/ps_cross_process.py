"""Parameter-server training across processes on one machine (CPU): one server process hosts the shards and serves
them over TCP on the loopback interface, ``--workers`` worker processes train an MLP on synthetic data and exchange
``-lr / workers * gradient`` through it (BSP or ASP), as the reference's ``DMLC_ROLE`` = server / worker launch does
(``src/ps/worker.cc:20-60``, ``python/athena/autodiff.py:264-327``).

    python examples/ps_cross_process.py --workers 2 --mode BSP --steps 20
"""
import argparse
import multiprocessing as mp
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def worker(rank, workers, port, mode, steps, out):
    from tsplit_b200 import gpu_ops as ad
    from tsplit_b200.models import mlp
    from tsplit_b200.parallel.ps_net import RemoteParameterServer
    ps = RemoteParameterServer("127.0.0.1", port, worker=rank, num_workers=workers)
    m = mlp(seed=5)                                   # same initial weights on every worker
    grads = ad.gradients(m.loss, m.variables)
    ex = ad.Executor([m.loss] + grads, ctx=None)
    if rank == 0:
        for i, v in enumerate(m.variables):
            ps.init("w%d" % i, v.tensor_value)
    ps.barrier()
    lr, losses = 0.1, []
    for step in range(steps):
        x, y = m.synthetic_batch(128, seed=1000 * rank + step)
        res = ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)
        losses.append(float(np.asarray(res[0]).reshape(-1)[0]))
        for i, (v, g) in enumerate(zip(m.variables, res[1:])):
            new = ps.push_pull("w%d" % i, (-lr / workers) * np.asarray(g, np.float32), mode=mode)
            v.tensor_value = new.reshape(np.asarray(v.tensor_value).shape)
    ps.barrier()
    ps.close()
    out.put((rank, losses[0], losses[-1]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workers", type=int, default=2)
    ap.add_argument("--mode", default="BSP", choices=["BSP", "ASP"])
    ap.add_argument("--steps", type=int, default=20)
    args = ap.parse_args()
    from tsplit_b200.parallel import ps_net
    srv = ps_net.serve(num_servers=2, num_workers=args.workers)        # listens on 127.0.0.1
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, args.workers, srv.port, args.mode, args.steps, out))
             for r in range(args.workers)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=300) for _ in procs)
    for p in procs:
        p.join()
    srv.stop()
    for rank, first, last in results:
        print("worker %d: loss %.4f -> %.4f" % (rank, first, last))
    assert all(last < first for _, first, last in results)


if __name__ == "__main__":
    main()
