"""Native replay of recorded calls (csrc/runtime/step_tape.cc), exercised on the host kernels of the runtime
library: every argument class the GPU entries use (pointers, 32/64-bit ints, floats, by-pointer host arrays) and
arguments that change between replays."""
import ctypes
from ctypes import c_float, c_int, c_int64, c_uint, c_void_p

import numpy as np
import pytest

from tsplit_b200 import _base
from tsplit_b200.runtime import tape
from tsplit_b200.utils.launch_counter import CountingLib

pytestmark = pytest.mark.skipif(not tape.available(), reason="libffi is not on this machine")


def ptr(a):
    return c_void_p(a.ctypes.data)


def test_recorded_host_kernels_replay_with_the_same_result():
    lib = CountingLib(_base.runtime())
    rng = np.random.RandomState(0)
    a, b = rng.randn(1000).astype(np.float32), rng.randn(1000).astype(np.float32)
    y, z = np.zeros(1000, np.float32), np.zeros(1000, np.float32)
    p, g, s1 = rng.randn(1000).astype(np.float32), rng.randn(1000).astype(np.float32), np.zeros(1000, np.float32)
    p0 = p.copy()
    hyper = (c_float * 8)(0.1, 0.9, 0, 0, 0, 0, 0, 0)
    with tape.recording() as rec:
        assert lib.tsb_cpu_binary(c_int(1), ptr(a), ptr(b), ptr(y), c_int64(1000)) == 0
        assert lib.tsb_cpu_unary(c_int(8), ptr(y), ptr(z), c_int64(1000), c_float(0.25)) == 0
        assert lib.tsb_cpu_unary(7, ptr(z), ptr(z), c_int64(1000), c_float(-1.5)) == 0      # bare Python int
        assert lib.tsb_cpu_optimizer(c_int(1), ptr(p), ptr(g), ptr(s1), None, c_int64(1000), hyper) == 0
    assert rec.invalid is None and len(rec.fns) == 4
    want_z = a * b * 0.25 - 1.5
    np.testing.assert_allclose(z, want_z, rtol=1e-6)
    p1, s1_1 = p.copy(), s1.copy()
    t = tape.Tape(rec)
    hyper[0] = 123.0                       # the recorded copy of a by-pointer argument is what replays
    z[:] = 0
    a *= 2
    t.replay()
    np.testing.assert_allclose(z, a * b * 0.25 - 1.5, rtol=1e-6)
    np.testing.assert_allclose(s1, 0.9 * s1_1 - 0.1 * g, rtol=1e-6)
    np.testing.assert_allclose(p, p1 + s1, rtol=1e-6)
    assert len(t) == 4 and t.last_host_ns > 0 and not np.allclose(p, p0)


def test_dynamic_arguments_take_their_value_at_replay_and_a_status_stops_the_tape():
    lib = CountingLib(_base.runtime())
    x, y = np.arange(8, dtype=np.float32), np.zeros(8, np.float32)
    with tape.recording() as rec:
        lib.tsb_cpu_unary(c_int(8), ptr(x), ptr(y), c_int64(8), tape.dyn("alpha", c_float(2.0)))
        lib.tsb_cpu_unary(c_int(7), ptr(y), ptr(y), tape.dyn("n", c_int64(8)), c_float(1.0))
    t = tape.Tape(rec)
    assert t.dyn_keys == ["alpha", "n"]
    t.replay({"alpha": c_float(3.0), "n": c_int64(4)})
    np.testing.assert_allclose(y, np.concatenate([x[:4] * 3 + 1, x[4:] * 3]))
    # a failing action: the ring all-reduce rejects a null handle with a non-zero status
    with tape.recording() as rec:
        lib.tsb_cpu_unary(c_int(8), ptr(x), ptr(y), c_int64(8), c_float(1.0))
        lib.tsb_ring_allreduce(None, None, c_int64(4), c_int(0))
        lib.tsb_cpu_unary(c_int(8), ptr(x), ptr(y), c_int64(8), c_float(5.0))
    t = tape.Tape(rec)
    with pytest.raises(tape.TapeError) as e:
        t.replay()
    assert e.value.index == 1 and e.value.entry == "tsb_ring_allreduce"
    np.testing.assert_allclose(y, x)            # the action behind the failing one did not run


def test_result_pointers_replay_into_the_tapes_own_storage_and_objects_make_a_recording_invalid():
    lib = CountingLib(_base.runtime())
    x, y = np.arange(1, 5, dtype=np.float32), np.zeros(4, np.float32)
    res = c_float(0)
    with tape.recording() as rec:
        lib.tsb_cpu_unary(c_int(8), ptr(x), ctypes.byref(res), c_int64(1), c_float(2.0))
    assert rec.invalid is None and res.value == 2.0 and bytes(rec.types) == b"ipbqf"
    x[0] = 5
    tape.Tape(rec).replay()
    assert res.value == 2.0                      # the replay wrote into the tape's copy
    with tape.recording() as rec:
        lib.tsb_cpu_unary(c_int(8), ptr(x), ptr(y), c_int64(4), c_float(1.0))
        lib.tsb_cpu_unary(c_int(8), ptr(x), ctypes.pointer(res), c_int64(1), c_float(1.0))
    assert rec.invalid is not None and "cannot be stored" in rec.invalid
    with pytest.raises(AssertionError):
        tape.Tape(rec)


def test_cpu_context_training_step_replays_from_the_tape():
    """``Executor(ctx=ndarray.cpu(0), use_graph="tape")``: one eager step, one recorded step, then the C++ loop.
    An MLP with momentum SGD runs entirely on host kernels, so its step is recorded; losses and parameters equal
    those of the Python loop.  A different batch is read every step (the feeds go through fixed buffers)."""
    from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
    from tsplit_b200.models import mlp
    runs = []
    for mode in (False, "tape"):
        m = mlp(seed=11)
        opt = optimizer.MomentumOptimizer(0.05, 0.9, ctx=ndarray.cpu(0))
        train = opt.minimize(m.loss)
        ex = ad.Executor([m.loss, train], ctx=ndarray.cpu(0), use_graph=mode)
        losses = []
        for step in range(6):
            x, y = m.synthetic_batch(32, seed=step % 2)
            losses.append(float(np.asarray(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0]).reshape(-1)[0]))
        if mode:
            assert ex._cpu_tape is not None, getattr(ex, "replay_failure", "")
            assert len(ex._cpu_tape) > 8 and "tsb_cpu_optimizer" in ex._cpu_tape.names
        assert opt.step_count == 6
        runs.append((losses, [np.asarray(p.asnumpy() if hasattr(p, "asnumpy") else p).copy() for p in opt.params]))
    np.testing.assert_allclose(runs[1][0], runs[0][0], rtol=1e-6)
    for a, b in zip(runs[1][1], runs[0][1]):
        np.testing.assert_allclose(a, b, rtol=1e-6, atol=1e-7)
    assert abs(runs[0][0][2] - runs[0][0][3]) > 1e-6          # the two batches really differ


def test_cpu_step_with_an_operator_without_host_kernel_keeps_the_python_loop():
    from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
    from tsplit_b200.models import mlp
    m = mlp(seed=11)
    opt = optimizer.AdamOptimizer(0.01, ctx=ndarray.cpu(0))          # hyper-parameters change every step
    train = opt.minimize(m.loss)
    ex = ad.Executor([m.loss, train], ctx=ndarray.cpu(0), use_graph="tape")
    x, y = m.synthetic_batch(16, seed=0)
    losses = [float(np.asarray(ex.run({m.X: x, m.y_: y}, convert_to_numpy_ret_vals=True)[0]).reshape(-1)[0])
              for _ in range(4)]
    assert ex._cpu_tape is None and "Adam" in ex.replay_failure
    assert losses[-1] < losses[0] and opt.step_count == 4
