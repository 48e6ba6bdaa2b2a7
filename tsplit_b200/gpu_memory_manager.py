"""Memory queries (reference: ``python/athena/gpu_memory_manager.py:6-40``):
``get_gpu_memory``, ``print_gpu_memory``, ``judge_malloc``, ``print_usage``,
``judge_usage`` — answered by the context's capped pool when one is installed,
otherwise by the CUDA driver."""
from __future__ import annotations

from . import ndarray
from ._base import get_array_memory


def _pool(ctx):
    return ndarray.get_pool(ctx)


def get_gpu_memory(ctx=None):
    """(used_MB, free_MB) of the active budget on ``ctx``."""
    ctx = ctx or ndarray.gpu(0)
    pool = _pool(ctx)
    if pool is not None:
        st = pool.stats()
        return st["used"] / 2**20, st["free"] / 2**20
    if ctx.device_type == 2:
        import torch
        free_b, total_b = torch.cuda.mem_get_info(ctx.torch_device)
        return (total_b - free_b) / 2**20, free_b / 2**20
    return 0.0, float("inf")


def print_gpu_memory(ctx=None):
    used, free = get_gpu_memory(ctx)
    print("GPU memory: used %.1f MB, available %.1f MB" % (used, free))


def judge_malloc(shape, ctx=None):
    """1 when an fp32 array of ``shape`` fits right now, else 0."""
    ctx = ctx or ndarray.gpu(0)
    pool = _pool(ctx)
    nbytes = int(get_array_memory(shape) * 2**20)
    if pool is not None:
        return 1 if pool.try_alloc(nbytes) else 0
    _, free = get_gpu_memory(ctx)
    return 1 if nbytes / 2**20 <= free else 0


def print_usage(ctx=None):
    ctx = ctx or ndarray.gpu(0)
    pool = _pool(ctx)
    if pool is None:
        return print_gpu_memory(ctx)
    st = pool.stats()
    print("pool: used %.1f MB, free %.1f MB (largest %.1f MB), peak %.1f MB, capacity %.1f MB" % tuple(
        st[k] / 2**20 for k in ("used", "free", "largest_free", "peak", "capacity")))


def judge_usage(ctx=None):
    """Fraction of the budget in use."""
    ctx = ctx or ndarray.gpu(0)
    pool = _pool(ctx)
    if pool is None:
        used, free = get_gpu_memory(ctx)
        return used / max(used + free, 1e-9)
    st = pool.stats()
    return st["used"] / max(st["capacity"], 1)
