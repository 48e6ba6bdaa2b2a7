"""Worker for the 2-GPU parameter-server test (launched by torchrun).

BSP: a small MLP trained through ``ps_gradients`` with GPU-resident shards must follow plain SGD on the
mean gradient (computed here with an NCCL all-reduce).  ASP: after every rank pushed once and a barrier,
the pulled values equal the initial values plus the sum of all pushed deltas."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tsplit_b200 import ndarray, gpu_ops as ad                      # noqa: E402
from tsplit_b200.parallel.graph_hooks import ps_gradients           # noqa: E402
from tsplit_b200.parallel.ps_gpu import GpuParameterServer          # noqa: E402


def build(ctx, seed=3):
    rs = np.random.RandomState(seed)
    X, y_ = ad.Variable(name="X"), ad.Variable(name="y_")
    w1 = ad.Variable(name="w1", value=ndarray.array(rs.normal(scale=0.2, size=(20, 33)).astype(np.float32), ctx,
                                                    use_pool=False))
    w2 = ad.Variable(name="w2", value=ndarray.array(rs.normal(scale=0.2, size=(33, 7)).astype(np.float32), ctx,
                                                    use_pool=False))
    h = ad.relu_op(ad.matmul_op(X, w1))
    loss = ad.softmaxcrossentropy_op(ad.matmul_op(h, w2), y_)
    return X, y_, loss, [w1, w2]


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    world = dist.get_world_size()
    ctx = ndarray.gpu(local)
    rs = np.random.RandomState(100 + rank)
    x = rs.standard_normal((16, 20)).astype(np.float32)
    y = np.eye(7, dtype=np.float32)[rs.randint(0, 7, 16)]
    lr = 0.1

    # ---- BSP through the graph hook
    X, y_, loss, ws = build(ctx)
    ps = GpuParameterServer(dist)
    new_w = ps_gradients(loss, ws, ps, lr=lr, mode="BSP")
    ex = ad.Executor([loss] + new_w, ctx=ctx)
    # yardstick: the same model, gradients averaged with NCCL, plain SGD on the host
    Xr, yr, lossr, wsr = build(ctx)
    exr = ad.Executor([lossr] + ad.gradients(lossr, wsr), ctx=ctx)
    ref_w = [w.tensor_value.asnumpy() for w in wsr]
    for step in range(4):
        outs = ex.run({X: x, y_: y}, convert_to_numpy_ret_vals=True)
        for w, v in zip(wsr, ref_w):
            w.tensor_value = ndarray.array(v, ctx, use_pool=False)
        r = exr.run({Xr: x, yr: y}, convert_to_numpy_ret_vals=True)
        for i, g in enumerate(r[1:]):
            t = torch.from_numpy(np.ascontiguousarray(g)).cuda()
            dist.all_reduce(t)
            ref_w[i] = ref_w[i] - lr * (t.cpu().numpy() / world)
        for got, want in zip(outs[1:], ref_w):
            np.testing.assert_allclose(got, want, rtol=2e-3, atol=2e-4, err_msg="BSP step %d" % step)
        for w, want in zip(ws, ref_w):                       # the variables were re-bound to the served values
            np.testing.assert_allclose(w.tensor_value.asnumpy(), want, rtol=2e-3, atol=2e-4)

    # ---- ASP: one push per rank, then everybody must see the sum
    ps2 = GpuParameterServer(dist)
    w0 = np.arange(1003, dtype=np.float32) * 0.01
    ps2.init("k", ndarray.array(w0, ctx, use_pool=False))
    ps2.finalize()
    g = ndarray.array(np.full(1003, float(rank + 1), np.float32), ctx, use_pool=False)
    mine = ps2.push_pull_device("k", g, lr, mode="ASP").asnumpy()
    # what a worker pulls right after its own push contains at least its own delta
    assert np.all(mine <= w0 - lr / world * (rank + 1) + 1e-4)
    torch.cuda.synchronize()
    dist.barrier()
    final = ps2.pull_device("k").asnumpy()
    want = w0 - lr / world * sum(range(1, world + 1))
    np.testing.assert_allclose(final, want, rtol=1e-5, atol=1e-5)
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("PS_GPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
