"""Build libhi2_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension).

    python -m hi2_b200.build [--force] [--verbose]

The library is compiled without FMA contraction (-fmad=false): the exact-arithmetic kernels rely
on every product and sum being rounded separately, and the GEMM-like kernels spell their fused
multiply-adds out.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libhi2_b200.so"
OBJ_DIR = HERE / "build"
SOURCES = [
    "common.cu",
    "rotate.cu",
    "pack.cu",
    "dequant.cu",
    "ladder.cu",
    "gptq.cu",
    "lazy_tc.cu",
    "refine.cu",
    "sigma.cu",
    "cholinv.cu",
    "hessian.cu",
    "hessian2.cu",
    "allocate.cu",
]
FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-fmad=false",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    cc = nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "hi2_b200.h"]
    jobs = []
    for name in SOURCES:
        src = CSRC / name
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [cc, *FLAGS, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        return res.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for log in pool.map(run, jobs):
            if verbose and log:
                print(log, file=sys.stderr)
    objs = [OBJ_DIR / (Path(n).stem + ".o") for n in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([cc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode",
             "arch=compute_100a,code=sm_100a", "-cudart", "static"])
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
