"""Worker for the 2-GPU data-parallel test (launched by torchrun): trains a small
CNN for a few steps with the fused all-reduce + optimizer kernel and with the
NCCL all-reduce + local update baseline from identical initial weights and data;
parameters must agree."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from tsplit_b200 import ndarray, gpu_ops as ad, optimizer      # noqa: E402
from tsplit_b200.models import vgg                              # noqa: E402
from tsplit_b200.parallel import ddp                            # noqa: E402


def train(mode, rank, ctx, steps=4, executor="plain"):
    m = vgg(16, num_classes=16, image=32, width_div=8, fc_width=64, seed=11)
    opt = optimizer.MomentumOptimizer(0.05, 0.9, ctx=ctx)
    train_op = opt.minimize(m.loss)
    comm = ddp.attach(opt, dist, mode=mode)
    x, y = m.synthetic_batch(8, seed=100 + rank)
    losses = []
    if executor == "plain":
        # an executor that knows nothing about buckets: the optimizer node stages the gradients and launches
        # every bucket itself
        ex = ad.Executor([m.loss, train_op], ctx=ctx)
        for _ in range(steps):
            losses.append(float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]))
    else:
        # the memory engine: gradients are produced inside the symmetric array and every bucket is launched
        # on the communication stream as soon as its last gradient exists
        from tsplit_b200.runtime.pool import use_pool
        with use_pool(ctx, 256 << 20):
            ex = ad.microopExecutor([m.loss, train_op], ctx=ctx, pieces=1 if executor == "engine" else 2,
                                    min_split_bytes=1,
                                    use_graph="tape" if executor == "tape" and mode == "fused" else False)
            for _ in range(steps):
                losses.append(float(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0][0]))
            if mode == "fused":
                assert len(comm.buckets) > 1, "the test is meant to exercise several buckets"
                assert ex._direct, "no gradient was produced in place"
                assert ex._bucket_ready_at, "no bucket was scheduled inside the backward pass"
            if executor == "tape" and mode == "fused":
                # two eager steps, one recorded, the rest replayed by the C++ loop, cooperative launches included
                assert ex._step_graph is not None, getattr(ex, "replay_failure", "")
                assert "tsb_fused_allreduce_update" in ex._step_graph.tape.names
    if hasattr(comm, "check"):
        comm.check(ex.stream)
    torch.cuda.synchronize()
    return losses, [p.asnumpy() for p in opt.params]


def main():
    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = ndarray.gpu(local)
    os.environ["TSPLIT_BUCKET_MB"] = "0.02"          # several buckets even for this small net
    l_ref, p_ref = train("nccl", rank, ctx)
    l_fused, p_fused = train("fused", rank, ctx)
    for a, b in zip(p_fused, p_ref):
        np.testing.assert_allclose(a, b, rtol=5e-3, atol=5e-4)
    for kind in ("engine", "tsplit", "tape"):
        # same executor, NCCL all-reduce + local update as the yardstick (a different executor may legitimately
        # differ by a switched ReLU, see tests/test_memory_executors_gpu.py)
        steps = 7 if kind == "tape" else 4
        _, p_base = train("nccl", rank, ctx, steps=steps, executor=kind)
        l_e, p_e = train("fused", rank, ctx, steps=steps, executor=kind)
        for a, b in zip(p_e, p_base):
            np.testing.assert_allclose(a, b, rtol=5e-3, atol=5e-4, err_msg="overlapped buckets, executor " + kind)
        flat_e = torch.cat([torch.from_numpy(p).reshape(-1) for p in p_e]).cuda()
        other_e = flat_e.clone()
        dist.broadcast(other_e, src=0)
        assert torch.equal(flat_e, other_e), "ranks diverged (%s)" % kind
    # every rank must hold identical parameters after the fused update
    flat = torch.cat([torch.from_numpy(p).reshape(-1) for p in p_fused]).cuda()
    other = flat.clone()
    dist.broadcast(other, src=0)
    assert torch.equal(flat, other), "ranks diverged"
    # the NVSwitch path: multimem.ld_reduce of the gradients and multimem.st of the new parameters through the
    # switch instead of one load / store per peer.  The switch adds in its own order, so equality is to rounding.
    nvls_used = False
    if os.environ.get("TSPLIT_TEST_NVLS", "1") == "1":
        os.environ["TSPLIT_NVLS"] = "1"
        m = vgg(16, num_classes=16, image=32, width_div=8, fc_width=64, seed=11)
        opt = optimizer.MomentumOptimizer(0.05, 0.9, ctx=ctx)
        train_op = opt.minimize(m.loss)
        comm = ddp.attach(opt, dist, mode="fused")
        nvls_used = bool(comm.grad_mc)
        if nvls_used:
            ex = ad.Executor([m.loss, train_op], ctx=ctx)
            x, y = m.synthetic_batch(8, seed=100 + rank)
            for _ in range(4):
                ex.run({m.X: x, m.y_: y})
            comm.check(ex.stream)
            torch.cuda.synchronize()
            for a, b in zip([p.asnumpy() for p in opt.params], p_fused):
                np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-4, err_msg="multimem path vs peer loads")
        os.environ["TSPLIT_NVLS"] = "0"
    dist.barrier()
    if rank == 0:
        print("losses nccl", l_ref, "fused", l_fused)
        print("NVLS path exercised:", nvls_used)
        print("DDP_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
