"""Generates tests/golden/reference_cuda_1024.npz on a GPU box.

Runs the reference's own CUDA backend (oracle/_ref/libref_gpu_cuda.so, built by oracle/Makefile
from the reference's lib/backend/gpu/gpu_memory_cuda.cpp and gpu_cuda_kernels.cu) through
tests/ref_gpu_runner.py on 1024^3 products of seeded operands and keeps 8 rows of each result:

    slice_T4, slice_T6   its INT8 slice tier (ESHKOL_CUDA_F64_KERNEL=ozaki-int8) at T = 4 and 6
    dgemm                its default cublasDgemm path

Operands are eshkol_b200.inputs.uniform(seed_a, (1024, 1024)) and uniform(seed_b, ...) with the
seeds stored in the file.  The slice-tier rows are integer-exact products reconstructed in a
fixed order, so they are bit patterns to be matched; the dgemm rows are a tolerance reference.

    python tests/golden/make_golden.py          # needs a GPU and the built reference library
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ROWS = [0, 1, 127, 128, 511, 640, 1000, 1023]
SEED_A, SEED_B, N = 601, 602, 1024


def run(kernel: str, T: int) -> np.ndarray:
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "c.npy")
        subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_gpu_runner.py"), kernel, str(T), str(N),
                        str(N), str(N), str(SEED_A), str(SEED_B), out], check=True, timeout=300)
        return np.load(out)[ROWS]


def main() -> None:
    np.savez_compressed(os.path.join(HERE, "reference_cuda_1024.npz"), rows=np.array(ROWS), seed_a=SEED_A,
                        seed_b=SEED_B, n=N, slice_T4=run("ozaki-int8", 4), slice_T6=run("ozaki-int8", 6),
                        dgemm=run("dgemm", 0))


if __name__ == "__main__":
    main()
