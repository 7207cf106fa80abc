"""In-tree build of the sm_100a kernel library (``libprism_b200.so``).

Plain ``nvcc``: every ``csrc/*.cu`` is compiled to an object with
``-gencode arch=compute_100a,code=sm_100a -lineinfo`` (cross-compiles without a GPU) and
linked into one shared library next to this file.  The library exports ``extern "C"``
entry points only and is loaded with ``ctypes`` (see ``native.py``), so there is no
dependency on the PyTorch C++ ABI and a rebuild takes seconds.  The reference JIT-builds
its single CUDA source with ``torch.utils.cpp_extension.load``
(``prism_infer/ops/cutlass_swiglu.py:44-79``).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libprism_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or add it to PATH")


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose: bool = False, force: bool = False) -> str:
    """Compile what changed, link, return the library path."""
    os.makedirs(BUILD, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    jobs = []
    objects = []
    for src in _sources():
        obj = os.path.join(BUILD, src[:-3] + ".o")
        objects.append(obj)
        if force or _stale(obj, [os.path.join(CSRC, src), *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd: list[str]) -> tuple[list[str], subprocess.CompletedProcess]:
        return cmd, subprocess.run(cmd, capture_output=True, text=True)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for cmd, res in pool.map(run, jobs):
                if verbose or res.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
                if res.returncode:
                    raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    if jobs or force or _stale(LIB, objects):
        cmd = [nvcc, "-shared", "-o", LIB, *objects, "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
