#!/usr/bin/env python
"""Maximum trainable batch and throughput per memory policy under one HBM cap.

The reference's drivers sweep the batch upward for one policy until the executor
refuses (``examples/imagenet_vgg.py:159-178``).  This script does that for every
policy of this framework by calling ``bench.py`` (one process per policy, so that
an aborted attempt cannot leave anything behind) and prints a Markdown table:

    python examples/max_batch_table.py --model vgg16 --cap-gib 16 --max-batch 2048

TSplit's maximum comes from its planner's dry run (confirmed by running it); the
other policies have no dry run and are probed by running down a ladder of batches.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
POLICIES = ["base", "vdnnall", "vdnnconv", "superneurons", "recompute_speed", "recompute_memory", "capuchin", "tsplit"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="vgg16", choices=["vgg16", "resnet50"])
    ap.add_argument("--cap-gib", type=float, default=16.0)
    ap.add_argument("--max-batch", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--policies", nargs="+", default=POLICIES)
    ap.add_argument("--json", default="", help="also write the raw bench lines to this file")
    args = ap.parse_args()
    rows, raw = [], []
    for pol in args.policies:
        cmd = [sys.executable, os.path.join(HERE, "bench.py"), "--model", args.model, "--policy", pol, "--cap-gib",
               str(args.cap_gib), "--max-batch", str(args.max_batch), "--steps", str(args.steps), "--warmup", "3",
               "--also-batch", "0"]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        line = next((ln for ln in reversed(res.stdout.splitlines()) if ln.startswith("{")), None)
        if res.returncode != 0 or line is None:
            why = (res.stderr.strip().splitlines() or ["no output"])[-1][:80]
            rows.append((pol, None, None, None, "did not finish (exit code %d): %s" % (res.returncode, why)))
            continue
        j = json.loads(line)
        raw.append(j)
        st = j["config"]["executor_stats"]
        note = "swap out %.1f GB, rebuilt %d, micro-ops %d" % (st.get("swap_out_bytes", 0) / 1e9,
                                                               st.get("recomputed_nodes", 0), st.get("micro_ops", 0))
        rows.append((pol, j["config"]["per_gpu_batch"], j["ms_per_step"], j["value"], note))
    print("| policy | max batch | ms / step | img/s | notes |")
    print("|---|---|---|---|---|")
    for pol, b, ms, v, note in rows:
        print("| %s | %s | %s | %s | %s |" % (pol, b if b is not None else "-", ms if ms is not None else "-",
                                              v if v is not None else "-", note))
    if args.json:
        with open(args.json, "w") as f:
            for j in raw:
                f.write(json.dumps(j) + "\n")


if __name__ == "__main__":
    main()
