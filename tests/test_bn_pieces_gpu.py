"""Batch norm over batch pieces on the GPU: statistics taken piece by piece into one partial-sum buffer,
one finalise launch, then piece-wise normalise (forward) / dx (backward) must equal the whole-batch
kernels and a plain fp32 PyTorch reference of the same op."""
import numpy as np
import pytest
import torch

from tsplit_b200 import ndarray
from tsplit_b200.ops import _gpu as G

pytestmark = pytest.mark.gpu


def _cl(t, ctx):
    """NDArray over a channels-last copy of an NCHW torch tensor."""
    return ndarray.NDArray(t.contiguous(memory_format=torch.channels_last), ctx, owns=False)


@pytest.mark.parametrize("n,c,hw,pieces,relu", [(12, 64, 14, 3, True), (8, 32, 9, 4, False), (5, 128, 7, 5, True)])
def test_piecewise_batch_norm_matches_whole_batch(n, c, hw, pieces, relu):
    ctx = ndarray.gpu(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3)
    x = torch.randn(n, c, hw, hw, device=dev, generator=g) * 1.7 + 0.3
    dy = torch.randn(n, c, hw, hw, device=dev, generator=g)
    scale = torch.rand(c, device=dev, generator=g) + 0.5
    bias = torch.randn(c, device=dev, generator=g) * 0.2
    eps, mom = 0.01, 0.99
    X, DY = _cl(x, ctx), _cl(dy, ctx)
    S, B = ndarray.NDArray(scale, ctx, owns=False), ndarray.NDArray(bias, ctx, owns=False)

    def vec(v=None):
        t = torch.empty(c, device=dev) if v is None else torch.full((c,), float(v), device=dev)
        return ndarray.NDArray(t, ctx, owns=False)
    # whole-batch kernels
    Yw = _cl(torch.empty_like(x), ctx)
    mean_w, inv_w, rm_w, rv_w = vec(), vec(), vec(0), vec(1)
    G.bn_forward(X, S, B, Yw, mean_w, inv_w, rm_w, rv_w, mom, eps, relu, None)
    DXw, ds_w, db_w = _cl(torch.empty_like(x), ctx), vec(), vec()
    if relu:
        G.bn_relu_backward(DY, X, S, B, mean_w, inv_w, DXw, ds_w, db_w, None)
    else:
        G.bn_backward(DY, X, S, mean_w, inv_w, DXw, ds_w, db_w, None)
    # piece-wise
    bounds = [ndarray._split_bounds(n, pieces, j) for j in range(pieces)]
    plane = pieces * G.BN_PIECE_CHUNKS * c
    part = ndarray.NDArray(torch.empty(2 * plane, device=dev), ctx, owns=False)
    piece = lambda a, lo, hi: ndarray.NDArray(a.t.narrow(0, lo, hi - lo), ctx, owns=False)
    chunks = 0
    for lo, hi in bounds:
        chunks += G.bn_stats_partial(piece(X, lo, hi), part, plane, chunks, None)
    mean_p, inv_p, rm_p, rv_p = vec(), vec(), vec(0), vec(1)
    G.bn_stats_finalize(part, plane, chunks, n * hw * hw, c, eps, mom, mean_p, inv_p, rm_p, rv_p, None)
    Yp = _cl(torch.empty_like(x), ctx)
    for lo, hi in bounds:
        G.bn_apply(piece(X, lo, hi), S, B, piece(Yp, lo, hi), mean_p, inv_p, relu, None)
    chunks = 0
    for lo, hi in bounds:
        chunks += G.bn_bwd_partial(piece(DY, lo, hi), piece(X, lo, hi), mean_p, inv_p, S if relu else None,
                                   B if relu else None, part, plane, chunks, None)
    ds_p, db_p = vec(), vec()
    G.bn_bwd_finalize(part, plane, chunks, c, ds_p, db_p, None)
    DXp = _cl(torch.empty_like(x), ctx)
    for lo, hi in bounds:
        G.bn_bwd_apply(piece(DY, lo, hi), piece(X, lo, hi), S, B if relu else None, mean_p, inv_p, ds_p, db_p,
                       piece(DXp, lo, hi), n * hw * hw, None)
    torch.cuda.synchronize()
    # plain PyTorch fp32 reference
    mu = x.mean(dim=(0, 2, 3))
    var = x.var(dim=(0, 2, 3), unbiased=False)
    inv = 1.0 / torch.sqrt(var + eps)
    bc = (1, c, 1, 1)
    xn = (x - mu.view(bc)) * inv.view(bc)
    y = xn * scale.view(bc) + bias.view(bc)
    gm = dy * (y > 0) if relu else dy
    if relu:
        y = y.clamp_min(0)
    m = float(n * hw * hw)
    ds = (gm * xn).sum(dim=(0, 2, 3))
    db = gm.sum(dim=(0, 2, 3))
    dx = scale.view(bc) * inv.view(bc) * (gm - db.view(bc) / m - xn * ds.view(bc) / m)

    def close(a, b, what, rtol=2e-4):
        a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
        err, sc = np.abs(a - b).max(), max(np.abs(b).max(), 1e-6)
        assert err <= rtol * sc, "%s: max err %.3e (scale %.3e)" % (what, err, sc)
    for got, whole, ref, what in ((mean_p.t, mean_w.t, mu, "mean"), (inv_p.t, inv_w.t, inv, "invstd"),
                                  (Yp.t, Yw.t, y, "y"), (ds_p.t, ds_w.t, ds, "dscale"), (db_p.t, db_w.t, db, "dbias"),
                                  (DXp.t, DXw.t, dx, "dx"), (rm_p.t, rm_w.t, (1 - mom) * mu, "running mean")):
        close(got, whole, what + " vs whole-batch kernel")
        close(got, ref, what + " vs PyTorch fp32")
