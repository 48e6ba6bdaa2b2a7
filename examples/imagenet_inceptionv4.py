"""Inception-v4.

    python examples/imagenet_inceptionv4.py -p tsplit -b 64        # one batch size
    python examples/imagenet_inceptionv4.py -p vdnnall             # sweep the batch size until the budget is exceeded
Policies: None | base | vdnnconv | vdnnall | superneurons | recompute_memory | recompute_speed |
capuchin | simulator | profiler | planner | tsplit.
Data parallel on N GPUs of one node (momentum SGD, fused NVLink all-reduce + update):
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/imagenet_inceptionv4.py -p tsplit -b 64"""
from common import parse, make_executor, default_ctx, timed_run, sweep, with_pool, dist_setup, attach

from tsplit_b200 import gpu_ops as ad, optimizer
from tsplit_b200.models import inception_v4


def run(batch_size, args, ctx):
    m = inception_v4()
    if world > 1:
        # data parallel: every rank trains on its own batch, gradients are reduced and applied by the fused kernel
        opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
        nodes = [m.loss, opt.minimize(m.loss)]
        attach(opt, args.comm)
    else:
        grads = ad.gradients(m.loss, m.variables)
        nodes = [m.loss] + grads + [m.y]
    ex = make_executor(args.policy, nodes, ctx)
    x, y = m.synthetic_batch(batch_size, seed=rank)
    return timed_run(ex, {m.X: x, m.y_: y})


if __name__ == "__main__":
    args = parse(__doc__.splitlines()[0])
    rank, world = dist_setup()
    ctx = default_ctx()
    with_pool(ctx, args.cap_gib)
    if args.batch:
        t = run(args.batch, args, ctx)
        if rank == 0:
            print({"policy": args.policy, "per_gpu_batch": args.batch, "gpus": world, "s_per_step": t,
                   "img_s": (args.batch * world / t) if isinstance(t, float) else None})
    else:
        sweep(lambda b: run(b, args, ctx), range(32, 2000, 32), args.out)
