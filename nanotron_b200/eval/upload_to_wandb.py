"""Pushes lighteval result files to Weights & Biases (parity: reference src/nanotron/eval/upload_to_wandb.py)."""
from __future__ import annotations

import argparse
import glob
import json
import os


def collect_results(results_path: str) -> dict:
    """Flatten every ``results*.json`` under ``results_path`` into ``{task/metric: value}``."""
    flat = {}
    for path in sorted(glob.glob(os.path.join(results_path, "**", "results*.json"), recursive=True)):
        with open(path) as f:
            data = json.load(f)
        for task, metrics in data.get("results", {}).items():
            for metric, value in metrics.items():
                if isinstance(value, (int, float)):
                    flat[f"{task}/{metric}"] = value
    return flat


def push_to_wandb(wandb_project, wandb_entity, model_name, results_path, train_step, consumed_tokens=None):
    import wandb

    flat = collect_results(results_path)
    wandb.init(project=wandb_project, entity=wandb_entity or None, name=model_name, id=model_name, resume="allow")
    payload = {**flat, "train_step": int(train_step)}
    if consumed_tokens is not None:
        payload["consumed_tokens"] = int(consumed_tokens)
    wandb.log(payload)
    wandb.finish()
    return flat


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--wandb_project", required=True)
    ap.add_argument("--wandb_entity", default=None)
    ap.add_argument("--model_name", required=True)
    ap.add_argument("--results_path", required=True)
    ap.add_argument("--train_step", type=int, required=True)
    ap.add_argument("--consumed_tokens", type=int, default=None)
    a = ap.parse_args()
    push_to_wandb(a.wandb_project, a.wandb_entity, a.model_name, a.results_path, a.train_step, a.consumed_tokens)
