"""TEST INFRASTRUCTURE: runs the reference's own CUDA backend (built by oracle/Makefile into
oracle/_ref/libref_gpu_cuda.so from lib/backend/gpu/gpu_memory_cuda.cpp and gpu_cuda_kernels.cu
of the reference project) on one GEMM and writes C to a .npy file.

    python tests/ref_gpu_runner.py <kernel> <T> <M> <K> <N> <seedA> <seedB> <out.npy>

kernel: "ozaki-int8" (the INT8 slice tier at fixed T) or "dgemm" (cublasDgemm).  Run as a
process of its own: the reference library exports the same symbol names as this repository's.
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> int:
    kernel, T, M, K, N, sa, sb, out = sys.argv[1], *map(int, sys.argv[2:8]), sys.argv[8]
    if kernel == "ozaki-int8":
        os.environ["ESHKOL_CUDA_F64_KERNEL"] = "ozaki-int8"
        os.environ["ESHKOL_OZAKI_CUDA_T"] = str(T)
    from eshkol_b200 import inputs
    from eshkol_b200.abi import EshkolGPUBuffer
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_gpu_cuda.so"))
    lib.eshkol_gpu_init.restype = ctypes.c_int
    if lib.eshkol_gpu_init() != 1:
        print("reference backend found no GPU")
        return 2
    A = inputs.uniform(sa, (M, K))
    B = inputs.uniform(sb, (K, N))
    C = np.zeros((M, N), dtype=np.float64)
    bufs = [EshkolGPUBuffer() for _ in range(3)]
    wrap = lib.eshkol_gpu_wrap_host
    wrap.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(EshkolGPUBuffer)]
    wrap.restype = ctypes.c_int
    for arr, buf in zip((A, B, C), bufs):
        if wrap(arr.ctypes.data, arr.nbytes, ctypes.byref(buf)) != 0:
            print("wrap_host failed")
            return 3
    mm = lib.eshkol_gpu_matmul_f64
    mm.argtypes = [ctypes.POINTER(EshkolGPUBuffer)] * 3 + [ctypes.c_uint64] * 3
    mm.restype = ctypes.c_int
    rc = mm(ctypes.byref(bufs[0]), ctypes.byref(bufs[1]), ctypes.byref(bufs[2]), M, K, N)
    if os.environ.get("REF_GPU_TIME"):
        # wall-clock of a second and third call (the first carries cuBLAS initialisation)
        import time
        for _ in range(2):
            t0 = time.perf_counter()
            mm(ctypes.byref(bufs[0]), ctypes.byref(bufs[1]), ctypes.byref(bufs[2]), M, K, N)
            dt = time.perf_counter() - t0
            print(f"reference {kernel} T={T} {M}x{K}x{N}: {dt * 1e3:.2f} ms, {2.0 * M * K * N / dt / 1e12:.2f} TFLOP/s")
    sync = lib.eshkol_gpu_sync
    sync.argtypes = [ctypes.POINTER(EshkolGPUBuffer), ctypes.c_int]
    sync.restype = ctypes.c_int
    sync(ctypes.byref(bufs[2]), 2)  # ESHKOL_SYNC_DEVICE_TO_HOST (gpu_memory.h:50)
    free = lib.eshkol_gpu_free
    free.argtypes = [ctypes.POINTER(EshkolGPUBuffer)]
    for buf in bufs:
        free(ctypes.byref(buf))
    if rc != 0:
        print("reference matmul returned", rc)
        return 4
    np.save(out, C)
    return 0


if __name__ == "__main__":
    sys.exit(main())
