"""Builds the in-tree native libraries with nvcc / g++ (no JIT cache: the ``.so`` files sit beside the sources).

    python -m nanotron_b200.ops.build            # build what is out of date
    python -m nanotron_b200.ops.build --force

``libntb_kernels.so``: every CUDA kernel, compiled for sm_100a only, plain C ABI (called through ctypes).
``libntb_dataidx.so``: C++17 dataset index builders (CPU).
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB_DIR = Path(__file__).resolve().parent
KERNEL_LIB = LIB_DIR / "libntb_kernels.so"
DATA_LIB = LIB_DIR.parent / "data" / "libntb_dataidx.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    if not force and not _newer(KERNEL_LIB, sources + headers):
        return KERNEL_LIB
    obj_dir = CSRC / "build"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or _newer(obj, [src] + headers):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)] + (["-Xptxas", "-v"] if verbose else [])
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                print(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as ex:
        objs = list(ex.map(compile_one, sources))
    tmp = KERNEL_LIB.with_suffix(".so.tmp")
    r = subprocess.run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart", "-Xcompiler", "-fPIC"], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, KERNEL_LIB)
    return KERNEL_LIB


def build_data_helpers(force: bool = False) -> Path:
    src = LIB_DIR.parent / "data" / "csrc" / "index_helpers.cpp"
    if not src.exists():
        return DATA_LIB
    if not force and not _newer(DATA_LIB, [src]):
        return DATA_LIB
    tmp = DATA_LIB.with_suffix(".so.tmp")
    r = subprocess.run(["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-o", str(tmp), str(src)], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, DATA_LIB)
    return DATA_LIB


def build_all(force: bool = False, verbose: bool = False):
    return build_kernels(force=force, verbose=verbose), build_data_helpers(force=force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(*build_all(force=a.force, verbose=a.verbose), sep="\n")
