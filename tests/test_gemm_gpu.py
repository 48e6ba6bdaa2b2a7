"""tcgen05 TF32 GEMM against a plain fp32 PyTorch reference."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(m, n, k, ta, tb, batch=1, splits=0, accumulate=False):
    from tsplit_b200 import _base
    lib = _base.kernels()
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n * 3 + k)
    a_shape = (batch, k, m) if ta else (batch, m, k)
    b_shape = (batch, n, k) if tb else (batch, k, n)
    a = torch.randn(a_shape, device="cuda", generator=g)
    b = torch.randn(b_shape, device="cuda", generator=g)
    c0 = torch.randn((batch, m, n), device="cuda", generator=g)
    c = c0.clone()
    st = torch.cuda.current_stream().cuda_stream
    if splits:
        rc = lib.tsb_gemm_tf32_splitk(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                                      ctypes.c_void_p(c.data_ptr()), m, n, k, ctypes.c_longlong(a.shape[-1]),
                                      ctypes.c_longlong(b.shape[-1]), ctypes.c_longlong(n), int(ta), int(tb),
                                      splits, ctypes.c_void_p(st))
    else:
        rc = lib.tsb_gemm_tf32(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                               ctypes.c_void_p(c.data_ptr()), m, n, k, ctypes.c_longlong(a.shape[-1]),
                               ctypes.c_longlong(b.shape[-1]), ctypes.c_longlong(n), int(ta), int(tb), batch,
                               ctypes.c_longlong(a.shape[-1] * a.shape[-2]),
                               ctypes.c_longlong(b.shape[-1] * b.shape[-2]), ctypes.c_longlong(m * n),
                               int(accumulate), ctypes.c_void_p(st))
    assert rc == 0, _base.error_string(rc)
    assert lib.tsb_device_status(ctypes.c_void_p(st)) == 0
    ad = a.double().transpose(-1, -2) if ta else a.double()
    bd = b.double().transpose(-1, -2) if tb else b.double()
    ref = ad @ bd
    if accumulate:
        ref = ref + c0.double()
    err = (c.double() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    return err / scale


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 512), (300, 200, 100), (64, 1000, 4096),
                                   (1024, 64, 128), (130, 72, 36)])
def test_gemm_layouts(m, n, k, ta, tb):
    assert _run(m, n, k, ta, tb) < 5e-3


def test_gemm_batched():
    assert _run(256, 128, 64, 0, 1, batch=12) < 5e-3
    assert _run(100, 100, 64, 0, 0, batch=5) < 5e-3
    assert _run(64, 256, 256, 1, 0, batch=3) < 5e-3


def test_gemm_splitk_and_accumulate():
    assert _run(128, 128, 4096, 0, 0, splits=4) < 5e-3
    assert _run(256, 64, 2048, 1, 0, splits=7) < 5e-3
    assert _run(200, 136, 512, 0, 1, accumulate=True) < 5e-3
    assert _run(128, 256, 8192, 1, 0) < 5e-3        # auto split-K (few tiles, long K)


def test_gemm_row_strides_that_tma_cannot_address():
    assert _run(37, 10, 256, 0, 0) < 5e-3           # ldb = 10 floats: padded into scratch, then tensor cores
    assert _run(128, 10, 255, 0, 0) < 5e-3


def test_gemm_large_many_tiles():
    assert _run(4096, 4096, 1024, 0, 0) < 5e-3


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(2048, 2048, 320), (2304, 2560, 96), (2112, 4128, 40)])
def test_gemm_cta_pair_tiles(m, n, k, ta, tb):
    """Problems with many 256 x 256 tiles and no split-K run the cta_group::2 kernel."""
    assert _run(m, n, k, ta, tb) < 5e-3


def test_gemm_cta_pair_ragged_batched_accumulate():
    assert _run(3000, 1800, 72, 0, 1) < 5e-3                     # rows / columns that are not tile multiples
    assert _run(1024, 1024, 128, 0, 0, batch=8) < 5e-3
    assert _run(1024, 768, 64, 1, 1, batch=16) < 5e-3
    assert _run(2048, 2048, 64, 0, 1, accumulate=True) < 5e-3


def test_gemm_odd_row_stride_is_padded_not_simt():
    """Row strides that are not multiples of four floats (255-wide attention matrices) are padded
    into scratch and still run on the tensor cores; results match in every transpose mode."""
    assert _run(255, 64, 255, 0, 0, batch=16) < 5e-3
    assert _run(255, 64, 255, 1, 0, batch=16) < 5e-3
    assert _run(130, 255, 64, 0, 1, batch=3) < 5e-3
    assert _run(100, 37, 72, 0, 0) < 5e-3            # ldb = 37
