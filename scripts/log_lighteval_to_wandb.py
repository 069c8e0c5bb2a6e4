"""Replays a folder of evaluation results, one sub-folder per checkpoint step, into Weights & Biases (or a JSON-lines file)
(capability parity: reference scripts/log_lighteval_to_wandb.py).

    python scripts/log_lighteval_to_wandb.py --eval-path evals/ --wandb-project my_evals --wandb-name run7
    python scripts/log_lighteval_to_wandb.py --eval-path evals/ --jsonl evals/curve.jsonl        # no wandb needed

Layout read:  ``<eval-path>/<step>/results*.json`` where the file is either a lighteval result file (``results`` maps task
names to metric dicts, ``config_general.config.general`` carries ``step`` / ``consumed_train_samples``) or the file
``run_evals.py`` of this repository writes (same ``results`` shape).  Per step the row holds every task's accuracy, the
mean over each benchmark family (``family:subset`` task names: mmlu, arc, ...) and the mean over all tasks.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
from collections import defaultdict
from typing import Callable, Dict, Iterable, List, Optional

ACC_KEYS = ("acc", "acc_norm", "accuracy", "acc_token", "acc_char")


def _accuracy(metrics: dict) -> Optional[float]:
    for key in ACC_KEYS:
        if isinstance(metrics.get(key), (int, float)):
            return float(metrics[key])
    return None


def _family(task: str) -> Optional[str]:
    """``custom|mmlu:anatomy|0`` -> ``mmlu``; tasks without a subset have no family."""
    core = task.split("|")[1] if task.count("|") >= 2 else task
    return core.split(":")[0] if ":" in core else None


def summarise(results: Dict[str, dict]) -> Dict[str, float]:
    """One row of numbers from the ``results`` section of a result file."""
    row: Dict[str, float] = {}
    by_family: Dict[str, List[float]] = defaultdict(list)
    everything: List[float] = []
    for task, metrics in results.items():
        if task == "all" or not isinstance(metrics, dict):
            continue
        acc = _accuracy(metrics)
        if acc is None:
            continue
        row[f"{task}_acc"] = acc
        everything.append(acc)
        fam = _family(task)
        if fam is not None:
            by_family[fam].append(acc)
    for fam, values in by_family.items():
        row[f"{fam}:average_acc"] = sum(values) / len(values)
    if everything:
        row["all:average_acc"] = sum(everything) / len(everything)
    return row


def iter_steps(eval_path: str) -> Iterable[tuple]:
    """(step, path of its single result file), in increasing step order; folders with zero or several files are reported and skipped."""
    steps = sorted((d for d in os.listdir(eval_path) if d.isdigit() and os.path.isdir(os.path.join(eval_path, d))), key=int)
    for d in steps:
        files = sorted(glob.glob(os.path.join(eval_path, d, "*.json")))
        if len(files) != 1:
            print(f"step {d}: expected one result file, found {len(files)} - skipped")
            continue
        yield int(d), files[0]


def replay(eval_path: str, sink: Callable[[dict], None]) -> int:
    """Feeds one row per checkpoint step to ``sink``; returns the number of rows."""
    n = 0
    for step, path in iter_steps(eval_path):
        with open(path) as f:
            data = json.load(f)
        general = data.get("config_general", {}).get("config", {}).get("general", {}) if isinstance(data.get("config_general"), dict) else {}
        row = summarise(data.get("results", {}))
        row["iteration_step"] = int(general.get("step", step))
        if "consumed_train_samples" in general:
            row["consumed_train_samples"] = int(general["consumed_train_samples"])
        sink(row)
        n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--eval-path", required=True, help="folder with one sub-folder of results per checkpoint step")
    ap.add_argument("--wandb-project", default="nanotron_evals")
    ap.add_argument("--wandb-name", default=None, help="run name; required unless --jsonl is given")
    ap.add_argument("--jsonl", default=None, help="write the rows to this file instead of logging them to wandb")
    args = ap.parse_args(argv)
    if args.jsonl:
        with open(args.jsonl, "w") as out:
            n = replay(args.eval_path, lambda row: out.write(json.dumps(row, sort_keys=True) + "\n"))
    else:
        if not args.wandb_name:
            ap.error("--wandb-name is required when logging to wandb")
        import wandb

        wandb.init(project=args.wandb_project, name=args.wandb_name, config={"eval_path": args.eval_path})
        n = replay(args.eval_path, wandb.log)
        wandb.finish()
    print(f"{n} checkpoint steps replayed")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
