"""Build libbwmoe.so (sm_100a only) in-tree with nvcc.

    python blackwell-moe_b200/build.py [--force]

The library links the CUDA runtime statically and resolves the one driver
entry point it needs (cuTensorMapEncodeTiled) at run time, so it loads on a
machine without a GPU (for symbol checks) and needs nothing but the driver on
a B200 box.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libbwmoe.so"
SOURCES = ["api.cu", "router.cu", "permute_quant.cu", "grouped_gemm_sm100.cu", "grouped_gemm_block_sm100.cu", "grouped_gemm_block_small_sm100.cu",
           "router_tc.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "bwmoe.h"]
    OBJ.mkdir(exist_ok=True)
    jobs = []
    for src in SOURCES:
        obj = OBJ / (src + ".o")
        if force or _stale(obj, [CSRC / src, *headers]):
            jobs.append([NVCC, *FLAGS, "-c", str(CSRC / src), "-o", str(obj)])

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=4) as pool:
        logs = list(pool.map(run, jobs))
    if verbose:
        for log in logs:
            print(log)
    objs = [str(OBJ / (s + ".o")) for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([NVCC, "-shared", "-o", str(LIB), *objs, "-cudart", "static"])
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
