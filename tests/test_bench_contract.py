"""The parts of ``bench.py`` that run without a GPU: the reference arm's line, the batch ladder, and the dry-run
maximum-batch search (the planner on the simulated device)."""
import importlib.util
import json
import os
import subprocess
import sys
import types

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_json_line_and_exits_zero():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "3", "--warmup", "3"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    assert res.returncode == 0
    lines = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    j = json.loads(lines[0])
    assert j["impl"] == "reference" and "\n" not in j["unavailable"] and len(j["unavailable"]) > 20


def test_batch_ladder_is_strictly_decreasing_and_starts_at_the_limit():
    bench = load_bench()
    for limit in (2048, 1000, 300, 64, 8):
        lad = bench.batch_ladder(limit)
        assert lad[0] == limit and lad[-1] >= 8
        assert all(a > b for a, b in zip(lad, lad[1:]))
    assert bench.batch_ladder(2048)[:4] == [2048, 1792, 1536, 1280]


def test_max_batch_search_takes_the_largest_batch_whose_plan_fits():
    """The search walks the ladder downward with dry runs of the planner and returns the first batch that fits:
    with a budget between the needs of two neighbouring rungs it must return the lower one, and log both."""
    bench = load_bench()
    from tsplit_b200 import ndarray, gpu_ops as ad, optimizer
    from tsplit_b200.models import vgg
    ctx = ndarray.simgpu(0)
    m = vgg(16, num_classes=10, image=32, width_div=8, fc_width=64, seed=3)
    opt = optimizer.MomentumOptimizer(0.01, 0.9, ctx=ctx)
    train = opt.minimize(m.loss)

    def need(batch):         # smallest budget at which the planner finds a plan for this batch (bisection)
        lo, hi = 1 << 16, 1 << 30
        while hi - lo > (1 << 16):
            mid = (lo + hi) // 2
            sim = ad.microopOptimizer([m.loss, train], ctx=ctx, budget_bytes=mid, host_link_gbs=50.0, max_split=32)
            x = np.empty((batch,) + m.input_shape, np.float32)
            y = np.empty((batch, m.num_classes), np.float32)
            if sim.run({m.X: x, m.y_: y})["fits"]:
                hi = mid
            else:
                lo = mid
        return hi
    lad = bench.batch_ladder(64)
    upper, lower = lad[0], lad[1]
    budget = (need(upper) + need(lower)) // 2
    assert need(lower) < budget < need(upper)
    args = types.SimpleNamespace(max_batch=64, plan_budget=budget, host_link_gbs=50.0)
    log = []
    got = bench.find_max_batch(args, m, train, ctx, log)
    assert got == lower
    assert [e["batch"] for e in log] == [upper, lower] and [e["fits"] for e in log] == [False, True]
