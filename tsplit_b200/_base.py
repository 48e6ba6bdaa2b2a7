"""Native library loader (role of the reference's ``python/athena/_base.py:9-113``).

Three shared objects are built in-tree under ``tsplit_b200/lib/`` by
``tsplit_b200/build.py``:

* ``libtsplit_runtime.so`` — host-only C++: capped best-fit pool, planner core,
  schedule log and happens-before checker, parameter-server shards, ring
  all-reduce.  Needs no CUDA and is used by the CPU test-suite.
* ``libtsplit_kernels.so`` — every sm_100a kernel (tcgen05 GEMM / conv,
  normalisation, pooling, softmax-CE, element-wise, optimizers).
* ``libtsplit_comm.so`` — peer-memory collectives fused with the optimizer.

A CUDA context without its kernel library is a hard error: there is no eager
fallback on the GPU.
"""
from __future__ import annotations

import ctypes
import os

LIB_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib")
_cache = {}

ERRORS = {
    0: "ok",
    1: "invalid argument",
    2: "unsupported shape or alignment",
    3: "CUDA launch error",
    4: "device-side wait ran out (peer or pipeline never signalled)",
    5: "out of memory budget",
    6: "tensor-map encode failed",
    7: "size beyond the static scratch limit",
}


def error_string(rc):
    base = ERRORS.get(rc & 0xFF, "error %d" % rc)
    if rc >> 8:
        base += " (cuda error %d)" % (rc >> 8)
    return base


def _load(name):
    if name in _cache:
        return _cache[name]
    path = os.path.join(LIB_DIR, name)
    if not os.path.exists(path):
        raise RuntimeError(
            "%s is not built; run `python -m tsplit_b200.build` (needs nvcc for the CUDA libraries)" % path)
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    _cache[name] = lib
    return lib


def runtime():
    lib = _load("libtsplit_runtime.so")
    return lib


def _counted(name):
    key = "counted:" + name
    if key not in _cache:
        from .utils.launch_counter import CountingLib
        _cache[key] = CountingLib(_load(name))
    return _cache[key]


def kernels():
    return _counted("libtsplit_kernels.so")


def comm():
    return _counted("libtsplit_comm.so")


def have(name):
    return os.path.exists(os.path.join(LIB_DIR, name))


def check_call(ret):
    assert ret == 0, error_string(ret)


def get_array_memory(shape):
    """Size in MB of an fp32 array of ``shape``."""
    n = 1
    for s in shape:
        n *= s
    return n * 4.0 / (1024 * 1024)
