"""TEST INFRASTRUCTURE: runs the reference's own CUDA backend (built by oracle/Makefile into
oracle/_ref/libref_gpu_cuda.so from lib/backend/gpu/gpu_memory_cuda.cpp and gpu_cuda_kernels.cu
of the reference project) on one GEMM and writes C to a .npy file.

    python tests/ref_gpu_runner.py <kernel> <T> <M> <K> <N> <seedA> <seedB> <out.npy>
    python tests/ref_gpu_runner.py conv-backward <batch> <C_in> <H> <W> <C_out> <kH> <kW> <sH> <sW> <out.npz>

kernel: "ozaki-int8" (the INT8 slice tier at fixed T) or "dgemm" (cublasDgemm).  conv-backward
runs the reference's two conv2d gradient kernels (lib/backend/gpu/gpu_cuda_kernels.cu:413-486)
through eshkol_gpu_conv2d_backward_input_f64 / _kernel_f64 on the operands of seeds 401 (input),
402 (weights), 403 (upstream gradient) and writes grad_input and grad_kernel.  Run as a process
of its own: the reference library exports the same symbol names as this repository's.
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def conv_backward() -> int:
    batch, C_in, H, W, C_out, kH, kW, sH, sW = map(int, sys.argv[2:11])
    out = sys.argv[11]
    from eshkol_b200 import inputs
    from eshkol_b200.abi import EshkolGPUBuffer
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_gpu_cuda.so"))
    lib.eshkol_gpu_init.restype = ctypes.c_int
    if lib.eshkol_gpu_init() != 1:
        print("reference backend found no GPU")
        return 2
    oH, oW = (H - kH) // sH + 1, (W - kW) // sW + 1
    X = inputs.uniform(401, (batch, C_in, H, W))
    Wt = inputs.uniform(402, (C_out, C_in, kH, kW))
    G = inputs.normal(403, (batch, C_out, oH, oW))
    gX = np.zeros_like(X)
    gK = np.zeros_like(Wt)
    bufp = ctypes.POINTER(EshkolGPUBuffer)
    wrap = lib.eshkol_gpu_wrap_host
    wrap.argtypes = [ctypes.c_void_p, ctypes.c_size_t, bufp]
    wrap.restype = ctypes.c_int
    bufs = {}
    for name, arr in (("X", X), ("W", Wt), ("G", G), ("gX", gX), ("gK", gK)):
        bufs[name] = EshkolGPUBuffer()
        if wrap(arr.ctypes.data, arr.nbytes, ctypes.byref(bufs[name])) != 0:
            print("wrap_host failed")
            return 3
    dims = [H, W, kH, kW, oH, oW, sH, sW, C_in, C_out, batch]
    rcs = []
    for fn, a, b, c in (("eshkol_gpu_conv2d_backward_input_f64", "G", "W", "gX"),
                        ("eshkol_gpu_conv2d_backward_kernel_f64", "G", "X", "gK")):
        f = getattr(lib, fn)
        f.argtypes = [bufp] * 3 + [ctypes.c_uint64] * 11
        f.restype = ctypes.c_int
        rcs.append(f(ctypes.byref(bufs[a]), ctypes.byref(bufs[b]), ctypes.byref(bufs[c]), *dims))
    sync = lib.eshkol_gpu_sync
    sync.argtypes = [bufp, ctypes.c_int]
    sync.restype = ctypes.c_int
    for name in ("gX", "gK"):
        sync(ctypes.byref(bufs[name]), 2)  # ESHKOL_SYNC_DEVICE_TO_HOST (gpu_memory.h:50)
    free = lib.eshkol_gpu_free
    free.argtypes = [bufp]
    for buf in bufs.values():
        free(ctypes.byref(buf))
    if any(rcs):
        print("reference conv2d backward returned", rcs)
        return 4
    np.savez(out, grad_input=gX, grad_kernel=gK)
    return 0


def main() -> int:
    if sys.argv[1] == "conv-backward":
        return conv_backward()
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
