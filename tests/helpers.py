"""Shared helpers: run the same graph on two contexts and compare every output."""
import numpy as np

from tsplit_b200 import ndarray, gpu_ops as ad


def run_graph(build, feeds, ctx, executor=None, **kw):
    """``build(ad)`` returns (placeholders dict name->node, list of eval nodes)."""
    ph, outs = build()
    ex_cls = executor or ad.Executor
    ex = ex_cls(outs, ctx=ctx, **kw)
    res = ex.run({ph[k]: v for k, v in feeds.items()}, convert_to_numpy_ret_vals=True)
    return [np.asarray(r) if r is not None else None for r in res]


def assert_close(a, b, rtol=2e-3, atol=None, what=""):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, a.shape, b.shape)
    scale = max(np.abs(b).max(), 1e-6)
    err = np.abs(a - b).max()
    tol = rtol * scale if atol is None else atol
    assert err <= tol, "%s: max err %.3e > %.3e (scale %.3e)" % (what, err, tol, scale)


def assert_close_per_channel(a, b, axis, rtol=2e-2, what=""):
    """Like :func:`assert_close`, but every slice along ``axis`` (a channel of an activation, an output
    channel of a filter) is compared against ITS OWN magnitude, so a wrong channel with small values cannot
    hide behind a large one.  Channels whose reference is all zero are compared absolutely against the
    tensor's scale."""
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    assert a.shape == b.shape, "%s: shape %s vs %s" % (what, a.shape, b.shape)
    a, b = np.moveaxis(a, axis, 0).reshape(a.shape[axis], -1), np.moveaxis(b, axis, 0).reshape(b.shape[axis], -1)
    floor = 1e-3 * max(np.abs(b).max(), 1e-6)
    scale = np.maximum(np.abs(b).max(axis=1), floor)
    err = np.abs(a - b).max(axis=1)
    worst = int(np.argmax(err / scale))
    assert np.all(err <= rtol * scale), "%s: channel %d max err %.3e > %.3e (channel scale %.3e)" % (
        what, worst, err[worst], rtol * scale[worst], scale[worst])
