"""ResNet-50/101.

    python examples/imagenet_resnet.py -p tsplit -b 64        # one batch size
    python examples/imagenet_resnet.py -p vdnnall             # sweep the batch size until the budget is exceeded
Policies: None | base | vdnnconv | vdnnall | superneurons | recompute_memory | recompute_speed |
capuchin | simulator | profiler | planner | tsplit."""
from common import parse, make_executor, default_ctx, timed_run, sweep, with_pool

from tsplit_b200 import gpu_ops as ad
from tsplit_b200.models import resnet


def run(batch_size, args, ctx):
    m = resnet(args.layer or 50)
    grads = ad.gradients(m.loss, m.variables)
    ex = make_executor(args.policy, [m.loss] + grads + [m.y], ctx)
    x, y = m.synthetic_batch(batch_size)
    return timed_run(ex, {m.X: x, m.y_: y})


if __name__ == "__main__":
    args = parse(__doc__.splitlines()[0])
    ctx = default_ctx()
    with_pool(ctx, args.cap_gib)
    if args.batch:
        print(run(args.batch, args, ctx))
    else:
        sweep(lambda b: run(b, args, ctx), range(32, 2000, 32), args.out)
