"""Stride-2 data gradient by output-pixel parity (csrc/kernels/conv_tcgen05.cu: run_dgrad_parity): the host
geometry of the library, checked in one dimension against the definition of the gradient.  For every parity a the
class is a stride-1 correlation of dy with the flipped sub-filter w[2t + r], dy padded by `lead` in front and
`trail` behind (a negative `trail` drops rows no window reaches); interleaving the two classes must give the
strided layer's data gradient."""
import ctypes
import itertools

import numpy as np
import pytest

from tsplit_b200 import _base


def axis(H, OH, K, pad, a):
    out = (ctypes.c_int * 7)()
    ok = _base.kernels()._lib.tsb_conv_parity_axis(H, OH, K, pad, a, out)
    return bool(ok), dict(zip(("r", "T", "q", "R", "lead", "trail", "empty"), list(out)))


def dgrad_by_definition(dy, w, H, pad):
    dx = np.zeros(H)
    for o in range(len(dy)):
        for k in range(len(w)):
            x = 2 * o + k - pad
            if 0 <= x < H:
                dx[x] += dy[o] * w[k]
    return dx


def dgrad_by_parity(dy, w, H, pad):
    OH, dx = len(dy), np.zeros(H)
    for a in (0, 1):
        ok, g = axis(H, OH, len(w), pad, a)
        if not ok:
            return None
        if g["empty"] or g["R"] == 0:
            continue
        sub = w[g["r"]::2][:g["T"]]
        assert len(sub) == g["T"]
        body = dy if g["trail"] >= 0 else dy[:g["trail"]]
        padded = np.concatenate([np.zeros(g["lead"]), body, np.zeros(max(g["trail"], 0))])
        assert len(padded) - g["T"] + 1 == g["R"], "the stride-1 launch must produce exactly the class's rows"
        dx[a::2] = [np.dot(padded[i:i + g["T"]], sub[::-1]) for i in range(g["R"])]
    return dx


def test_parity_classes_reproduce_the_strided_gradient():
    rng = np.random.RandomState(0)
    covered = 0
    for K, pad, H in itertools.product([1, 2, 3, 5, 7], [0, 1, 2, 3], range(4, 40)):
        if pad > K - 1 or H + 2 * pad < K:
            continue
        OH = (H + 2 * pad - K) // 2 + 1
        dy, w = rng.randn(OH), rng.randn(K)
        got = dgrad_by_parity(dy, w, H, pad)
        if got is None:
            continue
        np.testing.assert_allclose(got, dgrad_by_definition(dy, w, H, pad), atol=1e-12)
        covered += 1
    assert covered > 400


@pytest.mark.parametrize("K,pad,H", [(3, 1, 56), (3, 1, 13), (1, 0, 14), (1, 0, 13), (3, 0, 35), (7, 3, 224), (5, 2, 28)])
def test_layer_shapes_of_the_model_zoo_are_supported(K, pad, H):
    OH = (H + 2 * pad - K) // 2 + 1
    for a in (0, 1):
        ok, g = axis(H, OH, K, pad, a)
        assert ok
    ok0, g0 = axis(H, OH, K, pad, 0)
    ok1, g1 = axis(H, OH, K, pad, 1)
    assert sum(g["T"] for g in (g0, g1)) == K          # every tap runs in exactly one class, none is padding
