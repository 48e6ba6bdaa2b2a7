"""Bind a rank's host threads to the CPUs next to its GPU.

With one process per GPU, pinned swap buffers should live on the NUMA node the GPU hangs off: page-locked memory is
placed where the allocating thread runs, and a copy that crosses the inter-socket link shares it with every other
rank's traffic.  ``bind_to_gpu`` asks NVML for the GPU's CPU set and applies it to the calling thread (threads
started later inherit it).  This changes an attribute of this PROCESS only; nothing about the GPU is set.
Best effort: without NVML, or inside a cpuset that excludes those CPUs, it does nothing and returns None."""
from __future__ import annotations

import os


def bind_to_gpu(device_index):
    """Returns the sorted CPU list the thread is now bound to, or None if nothing was changed."""
    if os.environ.get("TSPLIT_BIND_CPUS", "1") == "0" or not hasattr(os, "sched_setaffinity"):
        return None
    try:
        import pynvml
        pynvml.nvmlInit()
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        if visible:
            entry = visible.split(",")[device_index].strip()
            handle = (pynvml.nvmlDeviceGetHandleByUUID(entry) if entry.startswith("GPU-")
                      else pynvml.nvmlDeviceGetHandleByIndex(int(entry)))
        else:
            handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        cpus = {64 * w + b for w, mask in enumerate(words) for b in range(64) if (mask >> b) & 1}
        allowed = os.sched_getaffinity(0)
        target = cpus & allowed
        if not target or target == allowed:
            return None
        os.sched_setaffinity(0, target)
        return sorted(target)
    except Exception:
        return None
