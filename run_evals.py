#!/usr/bin/env python
"""Evaluate a checkpoint with lighteval (parity: reference run_evals.py).  Needs the optional ``lighteval`` package.

    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 run_evals.py --checkpoint-config-path ckpt/10/config.yaml
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def get_parser():
    p = argparse.ArgumentParser()
    p.add_argument("--checkpoint-config-path", type=str, required=True, help="config.yaml inside the checkpoint folder")
    p.add_argument("--lighteval-override", type=str, default=None, help="YAML file overriding the `lighteval` section")
    p.add_argument("--cache-dir", type=str, default=None)
    return p


if __name__ == "__main__":
    args, unknown = get_parser().parse_known_args()
    try:
        from lighteval.main_nanotron import main  # type: ignore
    except ImportError:
        raise SystemExit("run_evals.py needs the `lighteval` package, which is not installed in this environment")
    main(args.checkpoint_config_path, args.lighteval_override, args.cache_dir)
