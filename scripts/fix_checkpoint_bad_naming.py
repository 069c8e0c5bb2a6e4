#!/usr/bin/env python
"""Renames parameter shard files written by old versions that put ``.safetensors`` in the middle of the file name
(parity: reference scripts/fix_checkpoint_bad_naming.py).

    python scripts/fix_checkpoint_bad_naming.py /path/to/checkpoints/10
"""
import argparse
import os
import re
from pathlib import Path


def fixed_name(name: str):
    """``model_weight.safetensors_pp-rank-0-of-1_tp-rank-0-of-2`` -> ``model_weight_pp-rank-0-of-1_tp-rank-0-of-2.safetensors``."""
    m = re.match(r"^(.*)\.safetensors(_pp-rank-.*)$", name)
    if not m:
        return None
    tail = m.group(2)
    tail = tail[: -len(".safetensors")] if tail.endswith(".safetensors") else tail
    return f"{m.group(1)}{tail}.safetensors"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("path", type=Path)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args()
    n = 0
    for root, _, files in os.walk(a.path):
        for f in files:
            new = fixed_name(f)
            if new and new != f:
                print(f"{os.path.join(root, f)} -> {new}")
                if not a.dry_run:
                    os.rename(os.path.join(root, f), os.path.join(root, new))
                n += 1
    print(f"{n} file(s) renamed")


if __name__ == "__main__":
    main()
