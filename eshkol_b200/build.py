"""Build recipe for libeshkol_gpu_b200.so (in-tree, sm_100a only).

nvcc compiles the CUDA translation units and links them with the C host layer
into one shared object next to this file.  Nothing is cached outside the tree,
so the built library travels with a copy of the repository.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libeshkol_gpu_b200.so")

CU_SOURCES = ["b200_modgemm.cu", "b200_modgemm2.cu", "b200_ozaki2.cu", "b200_tiers.cu", "b200_shim.cu", "b200_static_scratch.cu", "b200_staging.cu", "b200_sharded.cu", "b200_operators.cu"]
C_SOURCES = ["gpu_memory_b200.c", "rt_conv2d_b200.c"]
HEADERS = ["b200_common.cuh", "b200_internal.h", "b200_ozaki2.h", "b200_residue.cuh", "b200_tiers.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _sources() -> list[str]:
    return [os.path.join(CSRC, s) for s in CU_SOURCES + C_SOURCES]


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = _sources() + [os.path.join(CSRC, h) for h in HEADERS]
    inc = os.path.join(os.path.dirname(HERE), "include")
    deps += [os.path.join(inc, f) for f in os.listdir(inc)]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if any source is newer than it; return its path."""
    if not force and not is_stale():
        return LIB
    objs = []
    bdir = os.path.join(HERE, "build")
    os.makedirs(bdir, exist_ok=True)
    nvcc = _nvcc()
    log = []
    for src in _sources():
        obj = os.path.join(bdir, os.path.basename(src) + ".o")
        if src.endswith(".c"):
            cmd = ["gcc", "-O2", "-fPIC", "-std=c11", "-Wall", "-c", src, "-o", obj]
        else:
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log.append(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            sys.stderr.write(log[-1])
            raise RuntimeError(f"compile failed: {src}")
        objs.append(obj)
    cmd = [nvcc, "-shared", "-o", LIB, *objs, "-lcudart", "-lpthread", "-lm", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.append(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        sys.stderr.write(log[-1])
        raise RuntimeError("link failed")
    with open(os.path.join(bdir, "build.log"), "w") as f:
        f.write("\n".join(log))
    if verbose:
        sys.stderr.write("\n".join(log))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
