"""Builds libthrift_sm100.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE.parent / "libthrift_sm100.so"
OBJ = HERE / "_obj"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcudafe", "--diag_suppress=550"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    sources = sorted(HERE.glob("*.cu"))
    headers = sorted(HERE.glob("*.cuh"))
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [NVCC, *FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            results = list(pool.map(lambda c: subprocess.run(c, capture_output=True, text=True), jobs))
        for cmd, res in zip(jobs, results):
            if verbose or res.returncode != 0:
                sys.stderr.write(res.stdout + res.stderr)
            if res.returncode != 0:
                raise RuntimeError("nvcc failed: " + " ".join(cmd))
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(OUT, objs):
        subprocess.run([NVCC, "-shared", "-o", str(OUT), *map(str, objs), "-gencode",
                        "arch=compute_100a,code=sm_100a"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
