"""Builds libnntrain_grad_b200.so in-tree from nntrain_b200/csrc/*.cu.

sm_100a only; no fast-math, no FMA contraction (the codec has to agree bit
for bit with a CPU that does neither).  `python -m nntrain_b200.build` or
`build()` from Python; `-v` adds ptxas resource usage.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
OBJ = os.path.join(_HERE, "build")
LIBRARY = os.path.join(_HERE, "libnntrain_grad_b200.so")

NVCC_FLAGS = [
    "-O3", "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-fmad=false",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    stamp = os.path.getmtime(target)
    return any(os.path.getmtime(s) > stamp for s in sources)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every translation unit and link the shared library."""
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = sorted(glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
                     + glob.glob(os.path.join(_HERE, "..", "include", "*.h")))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    include = ["-I", os.path.join(_HERE, "..", "include"), "-I", CSRC]

    def compile_one(source: str) -> str:
        obj = os.path.join(OBJ, os.path.basename(source)[:-3] + ".o")
        if force or verbose or _stale(obj, [source, *headers, __file__]):
            cmd = [nvcc, *NVCC_FLAGS, *extra, *include, "-c", source, "-o", obj]
            done = subprocess.run(cmd, capture_output=True, text=True)
            if done.returncode != 0:
                raise RuntimeError(f"nvcc failed for {source}:\n{done.stdout}\n{done.stderr}")
            if verbose:
                sys.stderr.write(done.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))
    if force or _stale(LIBRARY, objects):
        cmd = [nvcc, "-shared", "-o", LIBRARY, *objects, "-lcudart", "-ldl"]
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
