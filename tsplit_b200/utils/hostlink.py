"""Measured bandwidth of the host link (pinned host memory <-> device).

The swap cost model of the planner needs the bytes per millisecond that a
``cudaMemcpyAsync`` between pinned host memory and the device sustains, in each
direction and with both directions busy at once (swap-out of one tensor overlaps
the swap-in of another).  The reference hard-codes a PCIe-3 figure
(``python/athena/profiler.py:14``); here it is measured once per process with
CUDA events and cached.

    python -m tsplit_b200.utils.hostlink          # prints one JSON line
"""
from __future__ import annotations

import json

_CACHE = {}


def measure(device=0, mbytes=256, repeats=4, shared=False):
    """Returns {"h2d_gbs", "d2h_gbs", "bidir_h2d_gbs", "bidir_d2h_gbs"} for pinned copies of
    ``mbytes`` MiB (best of ``repeats``); the bidirectional figures are per direction while
    both run on their own streams.  ``shared``: other processes of the box copy at the same time (one rank per
    GPU measuring together); then the MEDIAN repeat counts, because the best one is the moment the others paused."""
    import torch
    key = (device, mbytes, bool(shared))
    if key in _CACHE:
        return _CACHE[key]
    n = mbytes * 2**20 // 4
    dev = torch.device("cuda", device)
    h_a = torch.empty(n, dtype=torch.float32, pin_memory=True)
    h_b = torch.empty(n, dtype=torch.float32, pin_memory=True)
    d_a = torch.empty(n, dtype=torch.float32, device=dev)
    d_b = torch.empty(n, dtype=torch.float32, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    gb = n * 4 / 1e9

    def timed(fn_in, fn_out):
        best_in = best_out = None
        all_in, all_out = [], []
        for _ in range(repeats + 1):
            torch.cuda.synchronize(dev)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            if fn_in:
                with torch.cuda.stream(s_in):
                    ev[0].record()
                    fn_in()
                    ev[1].record()
            if fn_out:
                with torch.cuda.stream(s_out):
                    ev[2].record()
                    fn_out()
                    ev[3].record()
            torch.cuda.synchronize(dev)
            if fn_in:
                t = ev[0].elapsed_time(ev[1])
                best_in = t if best_in is None else min(best_in, t)
                all_in.append(t)
            if fn_out:
                t = ev[2].elapsed_time(ev[3])
                best_out = t if best_out is None else min(best_out, t)
                all_out.append(t)
        if shared:
            return (sorted(all_in)[len(all_in) // 2] if all_in else None,
                    sorted(all_out)[len(all_out) // 2] if all_out else None)
        return best_in, best_out

    h2d = lambda: d_a.copy_(h_a, non_blocking=True)
    d2h = lambda: h_b.copy_(d_b, non_blocking=True)
    t_in, _ = timed(h2d, None)
    _, t_out = timed(None, d2h)
    b_in, b_out = timed(h2d, d2h)
    res = {"h2d_gbs": round(gb / t_in * 1e3, 2), "d2h_gbs": round(gb / t_out * 1e3, 2),
           "bidir_h2d_gbs": round(gb / b_in * 1e3, 2), "bidir_d2h_gbs": round(gb / b_out * 1e3, 2),
           "mbytes": mbytes}
    _CACHE[key] = res
    return res


def planning_gbs(device=0):
    """Per-direction bandwidth the planner should assume: the slower direction with both busy."""
    m = measure(device)
    return min(m["bidir_h2d_gbs"], m["bidir_d2h_gbs"])


if __name__ == "__main__":
    print(json.dumps(measure()))
