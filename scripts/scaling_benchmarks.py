#!/usr/bin/env python
"""Sweep parallel layouts of one node and tabulate throughput (capability parity: reference scripts/scaling_benchmarks.py, which
generates slurm jobs over dp / tp / pp / batch-accumulation grids and collects tokens/s and MFU into a CSV).

    python scripts/scaling_benchmarks.py --gpus 8 --model llama3-8b --out results/scaling.csv [--layouts dp8 dp4tp2 dp2tp4 tp8 dp4pp2]

Each layout is one ``torchrun`` of ``bench.py`` (same timing rules: CUDA events, barrier + synchronize, max over ranks); its JSON
line becomes one CSV row.  A layout that fails or runs out of memory is recorded with its exit code and the sweep continues.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import re
import subprocess
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def parse_layout(name: str):
    parts = dict(dp=1, tp=1, pp=1)
    for key, val in re.findall(r"(dp|tp|pp)(\d+)", name):
        parts[key] = int(val)
    return parts


def default_layouts(gpus: int):
    out = []
    tp = 1
    while tp <= gpus:
        pp = 1
        while tp * pp <= gpus:
            dp = gpus // (tp * pp)
            if dp * tp * pp == gpus:
                out.append(f"dp{dp}tp{tp}pp{pp}")
            pp *= 2
        tp *= 2
    return out


def run_layout(args, layout: str, port: int):
    p = parse_layout(layout)
    world = p["dp"] * p["tp"] * p["pp"]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(port),
           os.path.join(REPO, "bench.py"), "--gpus", str(world), "--steps", str(args.steps), "--warmup", str(args.warmup), "--model", args.model, "--seq", str(args.seq),
           "--mbs", str(args.mbs), "--accum", str(args.accum), "--tp", str(p["tp"]), "--pp", str(p["pp"])]
    if args.recompute:
        cmd.append("--recompute")
    if world == 1:
        cmd = [sys.executable] + cmd[cmd.index(os.path.join(REPO, "bench.py")):]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=args.timeout, cwd=REPO)
    line = next((l for l in reversed(r.stdout.splitlines()) if l.startswith("{")), None)
    row = {"layout": layout, "returncode": r.returncode}
    if line:
        d = json.loads(line)
        row.update(tokens_per_s=d["value"], tokens_per_s_per_gpu=d["tokens_per_sec_per_gpu"], ms_per_step=d["ms_per_step"], model_tflops_per_gpu=d["model_tflops_per_gpu"],
                   mfu=d["mfu_of_measured_sustained_peak"], peak_mem_gb=d.get("peak_mem_gb"), parallelism=d["config"]["parallelism"], sm_mhz=(d.get("clocks") or {}).get("sm_mhz"))
    else:
        row["error"] = (r.stderr or r.stdout)[-300:].replace("\n", " ")
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--mbs", type=int, default=1)
    ap.add_argument("--accum", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--timeout", type=int, default=1200)
    ap.add_argument("--layouts", nargs="*", default=None, help="e.g. dp8 dp4tp2 dp2tp2pp2 (default: every power-of-two factorisation of --gpus)")
    ap.add_argument("--out", default="scaling.csv")
    args = ap.parse_args()
    layouts = args.layouts or default_layouts(args.gpus)
    rows = []
    for i, layout in enumerate(layouts):
        row = run_layout(args, layout, 29600 + i)
        rows.append(row)
        print(json.dumps(row), flush=True)
    keys = sorted({k for r in rows for k in r}, key=lambda k: (k != "layout", k))
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    with open(args.out, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=keys)
        w.writeheader()
        w.writerows(rows)
    print(f"wrote {args.out}")


if __name__ == "__main__":
    main()
