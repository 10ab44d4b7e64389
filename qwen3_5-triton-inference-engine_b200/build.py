"""Builds libb200attn.so (sm_100a only) from csrc/*.cu with nvcc, in-tree, next to this file.

    python build.py            # incremental: recompiles sources newer than their object
    python build.py --force
    python build.py --verbose  # adds -Xptxas -v (registers / spills / shared memory per kernel)

nvcc cross-compiles, so this runs on a machine without a GPU.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
OBJ = HERE / "build"
LIB = HERE / "libb200attn.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    OBJ.mkdir(exist_ok=True)
    hdr_time = _newest_header()
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            cmd = [_nvcc(), *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", str(src), "-o", str(obj)]
            jobs.append((src, cmd))

    def run(job):
        src, cmd = job
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for src, res in pool.map(run, jobs):
            if verbose or res.returncode != 0:
                sys.stderr.write(f"--- {src.name}\n{res.stdout}{res.stderr}\n")
            failed |= res.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed (see stderr)")
    objs = [str(OBJ / (s.stem + ".o")) for s in sources]
    if jobs or not LIB.exists():
        link = [_nvcc(), "-shared", "-o", str(LIB), *objs, "-gencode", "arch=compute_100a,code=sm_100a",
                "-Xcompiler", "-fPIC", "-lcudart"]
        res = subprocess.run(link, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
