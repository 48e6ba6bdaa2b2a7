"""Per-operator time sweeps over batch, channel and spatial size (the role of the
reference's ``kernel_profile/{conv2d,matmul,bn,maxpool,relu}.py``): each point is
measured with CUDA events after a warm-up, reported as ms and achieved TFLOP/s or
GB/s.

    python -m tsplit_b200.kernel_profile conv2d --sweep batch
"""
from __future__ import annotations

import argparse

import numpy as np


def _time(fn, iters=5):
    import torch
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def sweep(op, axis, points=None):
    from . import ndarray
    from .ops import _gpu as G
    from .stream import current_stream
    ctx = ndarray.gpu(0)
    st = current_stream(ctx)
    base = dict(batch=32, channel=128, hw=56)
    points = points or {"batch": [1, 8, 32, 64, 128, 256], "channel": [16, 64, 128, 256, 512, 1024],
                        "hw": [8, 14, 28, 56, 112, 224]}[axis]
    rows = []
    for v in points:
        cfg = dict(base)
        cfg[axis] = v
        n, c, hw = cfg["batch"], cfg["channel"], cfg["hw"]
        if op == "matmul":
            a, b, out = (ndarray.empty(s, ctx) for s in ((n * 64, c * 8), (c * 8, c * 8), (n * 64, c * 8)))
            for t in (a, b):
                t.t.normal_()
            ms = _time(lambda: G.gemm(a, b, out, False, False, st, m=n * 64, n=c * 8, k=c * 8, lda=c * 8,
                                      ldb=c * 8, ldc=c * 8))
            rows.append((v, ms, 2.0 * n * 64 * (c * 8) ** 2 / ms / 1e9, "TFLOP/s"))
            continue
        x = ndarray.empty((n, c, hw, hw), ctx)
        x.t.normal_()
        y = ndarray.empty((n, c, hw, hw), ctx)
        if op == "conv2d":
            w = ndarray.empty((c, c, 3, 3), ctx)
            w.t.normal_()
            ms = _time(lambda: G.conv2d(0, x, w, y, 1, 1, 1, st))
            rows.append((v, ms, 2.0 * n * hw * hw * c * c * 9 / ms / 1e9, "TFLOP/s"))
        elif op == "relu":
            ms = _time(lambda: G.unary(G.UN_RELU, x, y, st))
            rows.append((v, ms, 2.0 * x.nbytes / ms / 1e6, "GB/s"))
        elif op == "bn":
            s, b = ndarray.empty((1, c, 1, 1), ctx), ndarray.empty((1, c, 1, 1), ctx)
            s.t.fill_(1.0)
            b.t.zero_()
            stats = [ndarray.empty((c,), ctx) for _ in range(4)]
            ms = _time(lambda: G.bn_forward(x, s, b, y, stats[0], stats[1], stats[2], stats[3], 0.99, 0.01,
                                            False, st))
            rows.append((v, ms, 3.0 * x.nbytes / ms / 1e6, "GB/s"))
        elif op == "maxpool":
            yo = ndarray.empty((n, c, hw // 2, hw // 2), ctx)
            ms = _time(lambda: G.pool(0, x, yo, 2, 2, 0, 2, st))
            rows.append((v, ms, 1.25 * x.nbytes / ms / 1e6, "GB/s"))
        else:
            raise ValueError(op)
    return rows


def single(op, batch, channel, hw, iters):
    """One configuration, ``iters`` launches after one warm-up: the small case a
    profiler capture is taken on.  Prints ms and the achieved rate."""
    import torch
    from . import ndarray
    from .ops import _gpu as G
    from .stream import current_stream
    ctx = ndarray.gpu(0)
    st = current_stream(ctx)
    n, c = batch, channel
    if op == "matmul":
        m = batch * 64
        a, b, out = (ndarray.empty(s, ctx) for s in ((m, c * 8), (c * 8, c * 8), (m, c * 8)))
        a.t.normal_(), b.t.normal_()
        fn = lambda: G.gemm(a, b, out, False, False, st, m=m, n=c * 8, k=c * 8, lda=c * 8, ldb=c * 8, ldc=c * 8)
        work, unit = 2.0 * m * (c * 8) ** 2 / 1e9, "TFLOP/s"
    elif op in ("softmax", "softmax_grad", "ce_grad"):
        # rows = batch * channel, row length = hw
        rows, cols = n * c, hw
        x, y, z = (ndarray.empty((rows, cols), ctx) for _ in range(3))
        x.t.normal_(), y.t.normal_()
        if op == "softmax":
            fn = lambda: G.softmax(x, z, st)
            work = 2.0 * x.nbytes / 1e6
        elif op == "softmax_grad":
            G.softmax(x, y, st)
            fn = lambda: G.softmax_grad(y, x, z, st)
            work = 3.0 * x.nbytes / 1e6
        else:
            y.t.zero_()
            y.t[:, 0] = 1.0
            g = ndarray.empty((1,), ctx)
            g.t.fill_(1.0)
            fn = lambda: G.softmax_ce_grad(x, y, g, z, st)
            work = 3.0 * x.nbytes / 1e6
        unit = "GB/s"
    elif op in ("masked_softmax", "attention_scores", "attention_context"):
        # batch = N, channel = heads, hw = sequence length; head size 64
        heads, t, d = c, hw, 64
        q, k, v = (ndarray.empty((n, t, heads, d), ctx) for _ in range(3))
        sc, pr = ndarray.empty((n, heads, t, t), ctx), ndarray.empty((n, heads, t, t), ctx)
        ctxv = ndarray.empty((n, t, heads, d), ctx)
        tok = ndarray.empty((n, t), ctx)
        for a in (q, k, v, sc):
            a.t.normal_()
        tok.t.fill_(1.0)
        if op == "masked_softmax":
            fn = lambda: G.masked_softmax(sc, tok, pr, 0.125, True, st)
            work, unit = 2.0 * sc.nbytes / 1e6, "GB/s"                  # read the scores, write the probabilities
        elif op == "attention_scores":     # Q K^T, both operands read in the [N, T, heads, d] projection layout
            fn = lambda: G.gemm(q, k, sc, False, True, st, batch=n * heads, m=t, n=t, k=d, sa=d, sb=d, sc=t * t,
                                lda=heads * d, ldb=heads * d, ldc=t, heads=heads, head_mask=3)
            work, unit = (q.nbytes + k.nbytes + sc.nbytes) / 1e6, "GB/s"
        else:                              # P V, V and the result in the projection layout
            fn = lambda: G.gemm(sc, v, ctxv, False, False, st, batch=n * heads, m=t, n=d, k=t, sa=t * t, sb=d, sc=d,
                                lda=t, ldb=heads * d, ldc=heads * d, heads=heads, head_mask=6)
            work, unit = (sc.nbytes + v.nbytes + ctxv.nbytes) / 1e6, "GB/s"
    elif op in ("allreduce_emulate", "optimizer"):
        # elements = batch * channel * hw * hw
        elems = n * c * hw * hw // 4 * 4
        if op == "allreduce_emulate":
            # every rank's gradient / parameter array on ONE device, the shards processed one after the other by
            # one launch: the reduce + momentum update + parameter store code of the fused all-reduce without
            # links (what a single-GPU profiler capture can see of it).  Two ranks.
            from .parallel import fused_allreduce as fa
            grads = [torch.randn(elems, device="cuda") for _ in range(2)]
            params = [torch.zeros(elems, device="cuda") for _ in range(2)]
            s1, s2 = torch.zeros(elems, device="cuda"), torch.zeros(elems, device="cuda")
            fn = lambda: fa.emulate(1, grads, params, s1, s2, [0.01, 0.9], st.handle)
            work, unit = (2 + 1 + 2 + 2) * elems * 4 / 1e6, "GB/s"   # read 2 grads + param + slot, write slot + 2 params
        else:
            from . import optimizer as O
            ps = [ndarray.empty((elems // 8,), ctx) for _ in range(8)]
            gs = [ndarray.empty((elems // 8,), ctx) for _ in range(8)]
            ss = [ndarray.empty((elems // 8,), ctx) for _ in range(8)]
            for t in ps + gs + ss:
                t.t.normal_()
            fn = lambda: G.optimizer_step(1, ps, gs, ss, None, [0.01, 0.9], st)
            work, unit = 5.0 * elems * 4 / 1e6, "GB/s"               # read p, g, slot; write p, slot
    elif op in ("maxpool_fwd", "maxpool_bwd"):
        x = ndarray.empty((n, c, hw, hw), ctx)
        yo = ndarray.empty((n, c, hw // 2, hw // 2), ctx)
        x.t.normal_()
        G.pool(0, x, yo, 2, 2, 0, 2, st)
        if op == "maxpool_fwd":
            fn = lambda: G.pool(0, x, yo, 2, 2, 0, 2, st)
            work, unit = 1.25 * x.nbytes / 1e6, "GB/s"
        else:
            dy = ndarray.empty((n, c, hw // 2, hw // 2), ctx)
            dy.t.normal_()
            dx = ndarray.empty((n, c, hw, hw), ctx)
            fn = lambda: G.pool_grad(0, x, yo, dy, dx, 2, 2, 0, 2, st)
            work, unit = 2.5 * x.nbytes / 1e6, "GB/s"                # read x, y, dy; write dx
    else:
        x = ndarray.empty((n, c, hw, hw), ctx)
        y = ndarray.empty((n, c, hw, hw), ctx)
        x.t.normal_(), y.t.normal_()
        if op in ("conv_dgrad_s2", "conv_dgrad_s2_1x1"):
            # data gradient of a stride-2 layer (3x3 / pad 1, or the 1x1 projection): dx is hw x hw, dy half that;
            # the rate counts the layer's useful FLOPs only
            k = 3 if op == "conv_dgrad_s2" else 1
            w = ndarray.empty((c, c, k, k), ctx)
            w.t.normal_()
            dy = ndarray.empty((n, c, hw // 2, hw // 2), ctx)
            dy.t.normal_()
            fn = lambda: G.conv2d(1, x, w, dy, k // 2, k // 2, 2, st)
            work, unit = 2.0 * n * (hw // 2) ** 2 * c * c * k * k / 1e9, "TFLOP/s"
        elif op.startswith("conv"):
            w = ndarray.empty((c, c, 3, 3), ctx)
            w.t.normal_()
            kind = {"conv_fwd": 0, "conv_dgrad": 1, "conv_wgrad": 2}[op]
            fn = lambda: G.conv2d(kind, x, w, y, 1, 1, 1, st)
            work, unit = 2.0 * n * hw * hw * c * c * 9 / 1e9, "TFLOP/s"
        else:
            s_, b_ = ndarray.empty((1, c, 1, 1), ctx), ndarray.empty((1, c, 1, 1), ctx)
            s_.t.fill_(1.0), b_.t.zero_()
            stats = [ndarray.empty((c,), ctx) for _ in range(4)]
            G.bn_forward(x, s_, b_, y, stats[0], stats[1], stats[2], stats[3], 0.99, 0.01, True, st)
            if op == "bn":
                fn = lambda: G.bn_forward(x, s_, b_, y, stats[0], stats[1], stats[2], stats[3], 0.99, 0.01, True, st)
                work, unit = 3.0 * x.nbytes / 1e6, "GB/s"
            else:   # bnrelu_bwd
                dx = ndarray.empty((n, c, hw, hw), ctx)
                ds, db = ndarray.empty((1, c, 1, 1), ctx), ndarray.empty((1, c, 1, 1), ctx)
                g = ndarray.empty((n, c, hw, hw), ctx)
                g.t.normal_()
                fn = lambda: G.bn_relu_backward(g, x, s_, b_, stats[0], stats[1], dx, ds, db, stream=st)
                work, unit = 5.0 * x.nbytes / 1e6, "GB/s"   # dy and x read twice, dx written once
    ms = _time(fn, iters)
    print("%s batch=%d channel=%d hw=%d: %.4f ms, %.1f %s" % (op, batch, channel, hw, ms, work / ms, unit))
    return ms


def main():
    p = argparse.ArgumentParser()
    p.add_argument("op", choices=["conv2d", "matmul", "bn", "maxpool", "relu", "conv_fwd", "conv_dgrad",
                                  "conv_wgrad", "bnrelu_bwd", "softmax", "softmax_grad", "ce_grad",
                                  "allreduce_emulate", "optimizer", "maxpool_fwd", "maxpool_bwd",
                                  "conv_dgrad_s2", "conv_dgrad_s2_1x1", "masked_softmax", "attention_scores",
                                  "attention_context"])
    p.add_argument("--sweep", default="batch", choices=["batch", "channel", "hw"])
    p.add_argument("--single", action="store_true", help="one configuration (for profiler captures)")
    p.add_argument("--batch", type=int, default=32)
    p.add_argument("--channel", type=int, default=256)
    p.add_argument("--hw", type=int, default=56)
    p.add_argument("--iters", type=int, default=3)
    a = p.parse_args()
    if a.single or a.op in ("conv_fwd", "conv_dgrad", "conv_wgrad", "bnrelu_bwd", "conv_dgrad_s2", "conv_dgrad_s2_1x1"):
        single(a.op if a.op != "conv2d" else "conv_fwd", a.batch, a.channel, a.hw, a.iters)
        return
    for v, ms, rate, unit in sweep(a.op, a.sweep):
        print("%s=%-6d %9.4f ms  %9.1f %s" % (a.sweep, v, ms, rate, unit))


if __name__ == "__main__":
    main()
