"""Fused all-reduce + optimizer: bucket layout on CPU, all-ranks-on-one-GPU
emulation of the reduce/update/broadcast math, and a real 2-GPU run against
NCCL all-reduce + a local update."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tsplit_b200.parallel.fused_allreduce import bucket_layout

HERE = os.path.dirname(os.path.abspath(__file__))


def test_bucket_layout_pads_every_tensor_to_four_floats():
    offs, total = bucket_layout([5, 8, 1, 1024])
    assert offs == [0, 8, 16, 20] and total == 20 + 1024
    assert all(o % 4 == 0 for o in offs)


def _np_update(kind, p, g, s1, s2, h):
    if kind == 0:
        return p - h[0] * g, s1, s2
    if kind == 1:
        s1 = h[1] * s1 - h[0] * g
        return p + s1, s1, s2
    if kind == 2:
        lr_g = -h[0] * g
        s1 = h[1] * (s1 + lr_g)
        return p + s1 + lr_g, s1, s2
    if kind == 3:
        s1 = s1 + g * g
        return p - h[0] * g / (np.sqrt(s1) + h[1]), s1, s2
    s1 = h[1] * s1 + (1 - h[1]) * g
    s2 = h[2] * s2 + (1 - h[2]) * g * g
    return p - h[0] * (s1 / (1 - h[3])) / (np.sqrt(s2 / (1 - h[4])) + h[5]), s1, s2


@pytest.mark.gpu
@pytest.mark.parametrize("kind,hyper", [(0, [0.1]), (1, [0.1, 0.9]), (2, [0.1, 0.9]), (3, [0.1, 1e-7]),
                                        (4, [0.01, 0.9, 0.999, 0.9, 0.999, 1e-7])])
@pytest.mark.parametrize("world,n", [(2, 4096), (8, 1000004), (3, 52)])
def test_all_ranks_emulated_on_one_gpu(kind, hyper, world, n):
    from tsplit_b200.parallel.fused_allreduce import emulate
    g = torch.Generator(device="cuda").manual_seed(kind * 10 + world)
    grads = [torch.randn(n, device="cuda", generator=g) for _ in range(world)]
    p0 = torch.randn(n, device="cuda", generator=g)
    params = [p0.clone() for _ in range(world)]
    s1 = torch.rand(n, device="cuda", generator=g)
    s2 = torch.rand(n, device="cuda", generator=g)
    s1_0, s2_0 = s1.clone(), s2.clone()
    emulate(kind, grads, params, s1, s2, hyper)
    torch.cuda.synchronize()
    gm = sum(x.double() for x in grads).cpu().numpy() / world
    ref_p, ref_s1, ref_s2 = _np_update(kind, p0.double().cpu().numpy(), gm, s1_0.double().cpu().numpy(),
                                       s2_0.double().cpu().numpy(), hyper)
    for r in range(world):
        np.testing.assert_allclose(params[r].cpu().numpy(), ref_p, rtol=2e-5, atol=2e-6)
    if kind >= 1:
        np.testing.assert_allclose(s1.cpu().numpy(), ref_s1, rtol=2e-5, atol=2e-6)
    if kind == 4:
        np.testing.assert_allclose(s2.cpu().numpy(), ref_s2, rtol=2e-5, atol=2e-6)


@pytest.mark.gpu
def test_two_gpu_training_matches_nccl_baseline():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    # no rank leaves this test early, so the NVSwitch (multimem) path may be exercised next to the peer-load path
    env = dict(os.environ, TSPLIT_NVLS="0", TSPLIT_TEST_NVLS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29613", os.path.join(HERE, "ddp_worker.py")]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "DDP_OK" in res.stdout, res.stdout[-4000:]


@pytest.mark.gpu
def test_two_gpu_parameter_server_with_gpu_resident_shards():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TSPLIT_NVLS="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29617", os.path.join(HERE, "ps_gpu_worker.py")]
    res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-4000:]
    assert "PS_GPU_OK" in res.stdout, res.stdout[-4000:]


@pytest.mark.gpu
def test_bounded_wait_reports_a_peer_that_never_signals():
    """Failure detection on the device: rank 0 of a 2-rank exchange whose peer never writes its flag.
    The kernel's flag wait gives up after about a second, leaves a status code that the host turns
    into an error, and the context stays usable (a following launch works)."""
    from ctypes import c_int, c_void_p, c_longlong, c_float, c_uint
    from tsplit_b200.parallel import fused_allreduce as fa
    lib = fa._lib()
    dev = torch.device("cuda", 0)
    n = 4096
    grads = [torch.ones(n, device=dev), torch.ones(n, device=dev)]
    params = [torch.zeros(n, device=dev), torch.zeros(n, device=dev)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev), torch.zeros(64, dtype=torch.int32, device=dev)]
    slot1, slot2 = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    PT = c_void_p * 2
    hv = (c_float * 8)(0.1, 0, 0, 0, 0, 0, 0, 0)
    torch.cuda.synchronize()
    rc = lib.tsb_fused_allreduce_update(
        c_int(0), c_int(0), c_int(2), PT(*[g.data_ptr() for g in grads]), PT(*[p.data_ptr() for p in params]),
        PT(*[f.data_ptr() for f in flags]), c_void_p(0), c_void_p(0), c_void_p(slot1.data_ptr()),
        c_void_p(slot2.data_ptr()), c_longlong(n), hv, c_uint(1), c_int(0), c_void_p(0))
    assert rc & 0xFF in (0, 4), rc          # the launch itself succeeds; a late status may already be visible
    status = lib.tsb_comm_status(c_void_p(0))          # synchronises, reads and clears the status word
    assert (status & 0xF00) == 0x300, hex(status)      # a flag wait of the exchange ran out
    # the rank that gave up must not have reduced anything: parameters and optimizer state are untouched
    # (momentum SGD would have written slot1, plain SGD the parameters)
    assert float(params[0].abs().max()) == 0.0 and float(params[1].abs().max()) == 0.0
    assert float(slot1.abs().max()) == 0.0 and float(slot2.abs().max()) == 0.0
    # the context is still healthy: the one-GPU emulation of two ranks runs and gives the SGD result
    g2 = [torch.full((n,), 1.0, device=dev), torch.full((n,), 3.0, device=dev)]
    p2 = [torch.zeros(n, device=dev), torch.zeros(n, device=dev)]
    fa.emulate(0, g2, p2, torch.zeros(n, device=dev), torch.zeros(n, device=dev), [0.1])
    torch.cuda.synchronize()
    assert lib.tsb_comm_status(c_void_p(0)) == 0
    np.testing.assert_allclose(p2[0].cpu().numpy(), np.full(n, -0.2, np.float32), rtol=1e-6)
