"""Dataset warm-up on tiered storage before a run (capability parity: reference scripts/weka.py).

Token files that were tiered out to object storage make the first epoch crawl.  ``warmup`` pulls every file of the given
dataset folders back to the fast tier, ``status`` reports how much of each folder is there already.

    python scripts/weka.py status  /data/tokenized/fineweb /data/tokenized/code
    python scripts/weka.py warmup  --from-config examples/config_llama3_8b.yaml      # folders of every data stage
    python scripts/weka.py warmup  --backend read /data/tokenized/fineweb             # any file system: read through the page cache

Backends: ``weka`` drives the ``weka fs tier`` command line (``location`` for the status, ``fetch`` for the warm-up, files in
batches of 512 over a pool of workers); ``read`` needs no tooling: it streams the files with a thread pool, which pulls them
through whatever cache the file system has, and reports the status as unknown (-1).  ``auto`` picks ``weka`` when the command
exists.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Union

Runner = Callable[[List[str]], str]


def _run(cmd: List[str]) -> str:
    return subprocess.check_output(cmd, text=True)


def parse_paths(spec: Union[str, Sequence[str]]) -> List[str]:
    """A list of folders, or a block of text with one folder per line (YAML list items are accepted)."""
    if not isinstance(spec, str):
        return [p.rstrip("/") for p in spec if p]
    out = []
    for line in spec.splitlines():
        line = line.strip()
        if line.startswith("-"):
            line = line[1:].strip()
        if line and not line.startswith("#"):
            out.append(line.rstrip("/"))
    return out


def folders_of_config(config_path: str) -> List[str]:
    """Dataset folders named by the data stages of a training config (nanoset ``dataset_folder`` entries)."""
    import yaml

    with open(config_path) as f:
        cfg = yaml.safe_load(f)
    found: List[str] = []
    for stage in cfg.get("data_stages") or []:
        ds = ((stage or {}).get("data") or {}).get("dataset") or {}
        folder = ds.get("dataset_folder")
        if isinstance(folder, str):
            found.append(folder)
        elif isinstance(folder, (list, tuple)):
            found.extend(folder)
    seen, out = set(), []
    for p in found:
        p = p.rstrip("/")
        if p not in seen:
            seen.add(p)
            out.append(p)
    return out


def _files(folder: str) -> List[str]:
    out = []
    for root, _, names in os.walk(folder, followlinks=True):
        out.extend(os.path.join(root, n) for n in names)
    return sorted(out)


def _batches(items: List[str], n: int) -> Iterable[List[str]]:
    for i in range(0, len(items), n):
        yield items[i : i + n]


def pick_backend(name: str = "auto") -> str:
    if name != "auto":
        return name
    return "weka" if shutil.which("weka") else "read"


# ------------------------------------------------------------------------------------------------ status
def tier_status(folders: Union[str, Sequence[str]], backend: str = "auto", run: Runner = _run) -> Dict[str, float]:
    """Percentage of each folder's bytes on the fast tier (-1: could not be determined, 0 for an empty folder)."""
    backend = pick_backend(backend)
    result: Dict[str, float] = {}
    for folder in parse_paths(folders):
        files = _files(folder)
        if not files:
            result[folder] = 0.0
            continue
        if backend != "weka":
            result[folder] = -1.0
            continue
        total = cached = 0.0
        try:
            for batch in _batches(files, 512):
                out = run(["weka", "fs", "tier", "location", *batch, "--no-header", "--raw-units", "-o", "path,size,ssdRead"])
                for line in out.splitlines():
                    parts = line.split()
                    # "<path> <size> B <bytes on ssd> B"; the path may contain blanks, the numbers are counted from the end
                    if len(parts) >= 5 and parts[-1] == "B" and parts[-3] == "B":
                        total += float(parts[-4])
                        cached += float(parts[-2])
        except (subprocess.CalledProcessError, OSError, ValueError):
            result[folder] = -1.0
            continue
        result[folder] = round(100.0 * cached / total, 2) if total > 0 else 0.0
    return result


# ------------------------------------------------------------------------------------------------ warm-up
def _read_through(path: str, block: int = 8 << 20) -> int:
    n = 0
    with open(path, "rb", buffering=0) as f:
        while True:
            chunk = f.read(block)
            if not chunk:
                return n
            n += len(chunk)


def warmup(folders: Union[str, Sequence[str]], backend: str = "auto", workers: int = 64, run: Runner = _run) -> Dict[str, int]:
    """Fetches every file under the folders to the fast tier.  Returns the number of files handled per folder (-1 on error)."""
    backend = pick_backend(backend)
    done: Dict[str, int] = {}
    for folder in parse_paths(folders):
        files = _files(folder)
        try:
            with ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
                if backend == "weka":
                    list(pool.map(lambda batch: run(["weka", "fs", "tier", "fetch", *batch]), _batches(files, 512)))
                else:
                    list(pool.map(_read_through, files))
            done[folder] = len(files)
        except (subprocess.CalledProcessError, OSError):
            done[folder] = -1
    return done


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("command", choices=["status", "warmup"])
    ap.add_argument("folders", nargs="*")
    ap.add_argument("--from-config", default=None, help="take the dataset folders from the data stages of this training config")
    ap.add_argument("--backend", default="auto", choices=["auto", "weka", "read"])
    ap.add_argument("--workers", type=int, default=64)
    args = ap.parse_intermixed_args(argv)
    folders = list(args.folders) + (folders_of_config(args.from_config) if args.from_config else [])
    if not folders:
        ap.error("no folders given")
    if args.command == "warmup":
        for folder, n in warmup(folders, args.backend, args.workers).items():
            print(f"{folder}: {'failed' if n < 0 else f'{n} files fetched'}")
    for folder, pct in tier_status(folders, args.backend).items():
        print(f"{folder}: {'unknown' if pct < 0 else f'{pct:.2f} % on the fast tier'}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
