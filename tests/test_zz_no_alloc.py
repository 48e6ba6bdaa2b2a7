"""tsb_bn_forward_static: the batch-norm forward for callers that cannot allocate
device memory (a trainer whose HBM budget is fully reserved by its pool, a
latency-bound loop that cannot afford cudaMalloc's device-wide sync, a host that
owns the allocator).  It is called here through its exported C symbol, and its
outputs must equal those of the regular entry point — twice in a row, because
both calls share the library's static scratch array and the second one runs on
whatever the first left there.  Collected last on purpose (file name), so a run
that stops at the first failure has already exercised everything else."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tsplit_b200", "lib",
                   "libtsplit_kernels.so")


def _call(fn, x, scale, bias, rows, c, momentum, eps, relu, run_mean, run_var):
    y = torch.empty_like(x)
    mean = torch.empty(c, device="cuda")
    invstd = torch.empty(c, device="cuda")
    vp = ctypes.c_void_p
    rc = fn(vp(x.data_ptr()), vp(scale.data_ptr()), vp(bias.data_ptr()), vp(y.data_ptr()), vp(mean.data_ptr()),
            vp(invstd.data_ptr()), vp(run_mean.data_ptr()), vp(run_var.data_ptr()), ctypes.c_longlong(rows),
            ctypes.c_longlong(c), ctypes.c_longlong(c), ctypes.c_longlong(c), ctypes.c_float(momentum),
            ctypes.c_float(eps), ctypes.c_int(relu), vp(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, "entry point returned %d" % rc
    torch.cuda.synchronize()
    return y, mean, invstd


def test_static_scratch_entry_matches_regular_entry_twice():
    lib = ctypes.CDLL(LIB)
    static_fn, regular_fn = lib.tsb_bn_forward_static, lib.tsb_bn_forward
    g = torch.Generator(device="cuda").manual_seed(5)
    # two different problems back to back: the second call sees the first one's partial sums in the array
    for rows, c, relu in ((4096, 256, 0), (1000, 64, 1)):
        x = torch.randn(rows, c, device="cuda", generator=g) * 2 + 0.5
        scale = torch.rand(c, device="cuda", generator=g) + 0.5
        bias = torch.randn(c, device="cuda", generator=g)
        rm_a, rv_a = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        rm_b, rv_b = rm_a.clone(), rv_a.clone()
        ya, ma, ia = _call(static_fn, x, scale, bias, rows, c, 0.99, 0.01, relu, rm_a, rv_a)
        yb, mb, ib = _call(regular_fn, x, scale, bias, rows, c, 0.99, 0.01, relu, rm_b, rv_b)
        for got, ref in ((ya, yb), (ma, mb), (ia, ib), (rm_a, rm_b), (rv_a, rv_b)):
            scale_ref = ref.abs().max().item() + 1e-6
            assert (got - ref).abs().max().item() <= 2e-3 * scale_ref
        # and against plain fp32 PyTorch
        mu, var = x.mean(0), x.var(0, unbiased=False)
        ref = (x - mu) / torch.sqrt(var + 0.01) * scale + bias
        if relu:
            ref = ref.clamp_min(0)
        assert (ya - ref).abs().max().item() <= 2e-3 * (ref.abs().max().item() + 1e-6)


def test_static_scratch_entry_rejects_sizes_beyond_its_limit():
    lib = ctypes.CDLL(LIB)
    c = 8192 + 4
    x = torch.zeros(8, c, device="cuda")
    p = torch.zeros(c, device="cuda")
    vp = ctypes.c_void_p
    rc = lib.tsb_bn_forward_static(vp(x.data_ptr()), vp(p.data_ptr()), vp(p.data_ptr()), vp(x.data_ptr()),
                                   vp(p.data_ptr()), vp(p.data_ptr()), vp(p.data_ptr()), vp(p.data_ptr()),
                                   ctypes.c_longlong(8), ctypes.c_longlong(c), ctypes.c_longlong(c),
                                   ctypes.c_longlong(c), ctypes.c_float(0.9), ctypes.c_float(1e-5),
                                   ctypes.c_int(0), vp(0))
    assert rc == 7
