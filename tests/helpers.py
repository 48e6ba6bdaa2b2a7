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
