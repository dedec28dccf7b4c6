"""Host-side mirror of the reference's matmul / conv2d entry points.

Each function is a thin call through the C ABI; names and argument meaning
follow the reference (eshkol_matmul_dispatch, eshkol_batch_matmul_dispatch:
lib/backend/gpu/gpu_memory_cuda.cpp:1107-1175; conv2d:
lib/backend/tensor_conv_kernel.h:66-105).  Arrays are numpy float64, C-contiguous.
"""
from __future__ import annotations

import ctypes

import numpy as np

from .abi import GemmOpts, load_library

_MODULI = (256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193)


def init() -> bool:
    """eshkol_gpu_init: True when the B200 backend is active."""
    return load_library().eshkol_gpu_init() == 1


def _f64(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float64)
    return a


def matmul_dispatch(A, B, dtype: int = 0) -> np.ndarray:
    """C = A @ B through eshkol_matmul_dispatch (host pointers in, host pointer out)."""
    A, B = _f64(A), _f64(B)
    M, K = A.shape
    K2, N = B.shape
    if K != K2:
        raise ValueError("inner dimensions differ")
    C = np.empty((M, N), dtype=np.float64)
    load_library().eshkol_matmul_dispatch(A.ctypes.data, B.ctypes.data, C.ctypes.data, M, K, N, dtype)
    return C


matmul = matmul_dispatch


def matmul_backward(G, A, B):
    """(grad_A, grad_B) of C = A @ B for the upstream gradient G, through
    eshkol_gpu_matmul_backward_f64 on host arrays; raises when the GPU path declines or fails."""
    G, A, B = _f64(G), _f64(A), _f64(B)
    M, K = A.shape
    N = B.shape[1]
    if G.shape != (M, N) or B.shape[0] != K:
        raise ValueError("shapes do not match")
    gA = np.empty((M, K), dtype=np.float64)
    gB = np.empty((K, N), dtype=np.float64)
    rc = load_library().eshkol_gpu_matmul_backward_f64(G.ctypes.data, A.ctypes.data, B.ctypes.data,
                                                      gA.ctypes.data, gB.ctypes.data, M, K, N)
    if rc != 0:
        raise RuntimeError("eshkol_gpu_matmul_backward_f64 returned -1")
    return gA, gB


def batch_matmul_dispatch(a, b, dtype: int = 0) -> np.ndarray:
    a, b = _f64(a), _f64(b)
    batch, M, K = a.shape
    _, _, N = b.shape
    c = np.empty((batch, M, N), dtype=np.float64)
    load_library().eshkol_batch_matmul_dispatch(a.ctypes.data, b.ctypes.data, c.ctypes.data, batch, M, K, N, dtype)
    return c


def conv_out_dim(in_dim: int, k_dim: int, stride: int, pad: int) -> int:
    """eshkol_conv_out_dim (lib/backend/tensor_conv_kernel.h:49-56)."""
    if stride <= 0:
        stride = 1
    if pad < 0:
        pad = 0
    span = in_dim + 2 * pad - k_dim
    return 0 if span < 0 else span // stride + 1


def conv2d(inp, ker, stride: int = 1, pad: int = 0, activation: int = 0) -> np.ndarray:
    """NCHW cross-correlation on host arrays through eshkol_gpu_conv2d_f64."""
    inp, ker = _f64(inp), _f64(ker)
    batch, in_c, H, W = inp.shape
    out_c, in_c2, kH, kW = ker.shape
    if in_c != in_c2:
        raise ValueError("channel counts differ")
    oH, oW = conv_out_dim(H, kH, stride, pad), conv_out_dim(W, kW, stride, pad)
    out = np.zeros((batch, out_c, oH, oW), dtype=np.float64)
    if oH == 0 or oW == 0:
        return out
    rc = load_library().eshkol_gpu_conv2d_f64(inp.ctypes.data, batch, in_c, H, W, ker.ctypes.data,
                                              out_c, kH, kW, stride, pad, out.ctypes.data, activation)
    if rc != 0:
        raise RuntimeError("eshkol_gpu_conv2d_f64 failed")
    return out


def make_opts(tier: int = 0, param: int = 0, activation: int = 0, bias_ptr: int = 0, bias_mode: int = 0,
              use_simt: bool = False, tile_n: int = 0, ldc: int = 0, trans_a: bool = False,
              trans_b: bool = False) -> GemmOpts:
    o = GemmOpts()
    o.tier, o.param, o.activation = tier, param, activation
    o.bias_mode, o.bias = (bias_mode if bias_ptr else 0), (bias_ptr or None)
    o.pixels_per_image = 0
    o.use_simt_products = 1 if use_simt else 0
    o.gemm_tile_n = tile_n
    o.ldc = ldc
    o.trans_a, o.trans_b = (1 if trans_a else 0), (1 if trans_b else 0)
    return o


def gemm_device(dA: int, dB: int, dC: int, M: int, K: int, N: int, opts: GemmOpts | None = None) -> None:
    """eshkol_b200_gemm_f64_device on raw device pointers (asynchronous)."""
    lib = load_library()
    if lib.eshkol_b200_init(_current_device()) != 0:
        raise RuntimeError("eshkol_b200_init failed: no usable sm_100 device")
    rc = lib.eshkol_b200_gemm_f64_device(dA, dB, dC, M, K, N, ctypes.byref(opts) if opts is not None else None)
    if rc != 0:
        raise RuntimeError(f"eshkol_b200_gemm_f64_device failed ({rc})")


def conv2d_device(d_in: int, shape_in, d_ker: int, shape_ker, stride: int, pad: int, d_out: int,
                  opts: GemmOpts | None = None) -> None:
    lib = load_library()
    if lib.eshkol_b200_init(_current_device()) != 0:
        raise RuntimeError("eshkol_b200_init failed: no usable sm_100 device")
    b, ic, H, W = shape_in
    oc, _, kH, kW = shape_ker
    rc = lib.eshkol_b200_conv2d_f64_device(d_in, b, ic, H, W, d_ker, oc, kH, kW, stride, pad, d_out,
                                           ctypes.byref(opts) if opts is not None else None)
    if rc != 0:
        raise RuntimeError(f"eshkol_b200_conv2d_f64_device failed ({rc})")


_device = None


def set_device(index: int) -> None:
    """Device the library binds to on first use (one process per GPU)."""
    global _device
    _device = index


def _current_device() -> int:
    import os
    if _device is not None:
        return _device
    return int(os.environ.get("ESHKOL_B200_DEVICE", os.environ.get("LOCAL_RANK", "0")))


def sync_status() -> int:
    return load_library().eshkol_b200_sync_status()


def stream_handle() -> int:
    return load_library().eshkol_b200_stream() or 0


def launch_count() -> int:
    return int(load_library().eshkol_b200_launch_count())


def debug_fetch(what: int, index: int = 0):
    """Intermediate of the last Ozaki-II GEMM as a numpy array (tests only)."""
    lib = load_library()
    info = (ctypes.c_uint64 * 6)()
    cap = 1 << 20
    while True:
        buf = np.empty(cap, dtype=np.uint8)
        rc = lib.eshkol_b200_debug_fetch(what, index, buf.ctypes.data, cap, info)
        if rc == -2:
            cap *= 4
            continue
        if rc != 0:
            raise RuntimeError("eshkol_b200_debug_fetch failed")
        break
    rows, pitch, esz, n_chunks, last_seg, nbytes = (int(x) for x in info)
    dt = {1: np.int8, 2: np.int16, 4: np.int32}[esz]
    arr = buf[:nbytes].view(dt).reshape(rows, pitch).copy()
    return arr, {"n_chunks": n_chunks, "last_seg": last_seg}
