"""Transformer encoder-decoder (6+6, d_model 512, 8 heads, FFN 2048) with Adam.

    python examples/transformer.py -p recompute_speed -b 32 --maxlen1 256 --maxlen2 256
Data parallel on N GPUs of one node:
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/transformer.py -p recompute_speed -b 32"""
from common import parse, make_executor, default_ctx, timed_run, sweep, with_pool, dist_setup, attach

from tsplit_b200 import optimizer
from tsplit_b200.models import transformer


def extra(p):
    p.add_argument("--vocab_size", type=int, default=32000)
    p.add_argument("--d_model", type=int, default=512)
    p.add_argument("--d_ff", type=int, default=2048)
    p.add_argument("--num_blocks", type=int, default=6)
    p.add_argument("--num_heads", type=int, default=8)
    p.add_argument("--maxlen1", type=int, default=256)
    p.add_argument("--maxlen2", type=int, default=256)
    p.add_argument("--dropout_rate", type=float, default=0.0)
    p.add_argument("--lr", type=float, default=0.0003)


def run(batch_size, args, ctx):
    t = transformer(vocab_size=args.vocab_size, d_model=args.d_model, d_ff=args.d_ff, num_blocks=args.num_blocks,
                    num_heads=args.num_heads, maxlen1=args.maxlen1, maxlen2=args.maxlen2,
                    dropout_rate=args.dropout_rate, batch_size=batch_size)
    opt = optimizer.AdamOptimizer(args.lr, ctx=ctx)
    train = opt.minimize(t.loss)
    attach(opt, args.comm)
    ex = make_executor(args.policy, [t.loss, train], ctx)
    return timed_run(ex, t.synthetic_batch())


if __name__ == "__main__":
    args = parse(__doc__.splitlines()[0], extra)
    rank, world = dist_setup()
    ctx = default_ctx()
    with_pool(ctx, args.cap_gib)
    if args.batch:
        t = run(args.batch, args, ctx)
        if rank == 0:
            print({"policy": args.policy, "per_gpu_batch": args.batch, "gpus": world, "s_per_step": t,
                   "target_tokens_s": (args.batch * world * args.maxlen2 / t) if isinstance(t, float) else None})
    else:
        sweep(lambda b: run(b, args, ctx), range(8, 1000, 8), args.out)
