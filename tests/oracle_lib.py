"""ctypes access to the CPU oracle (oracle/liboracle.so) and to the reference's own
CPU code compiled into oracle/_ref/.  Test infrastructure only."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
UNFUSED, EXPFIELD = 1, 2

_dp = ctypes.POINTER(ctypes.c_double)
_ip = ctypes.POINTER(ctypes.c_int)
_fp = ctypes.POINTER(ctypes.c_float)
_lib = None


def build() -> None:
    subprocess.run(["make", "-C", ORACLE_DIR, "-s"], check=True, capture_output=True)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(ORACLE_DIR, "liboracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < max(
                os.path.getmtime(os.path.join(ORACLE_DIR, f)) for f in ("ozaki2_ref.cpp", "reduced_ref.cpp")):
            build()
        L = ctypes.CDLL(path)
        i64, ci = ctypes.c_int64, ctypes.c_int
        L.oracle_oz2_constants.argtypes = [ci, _dp, _dp, _dp, _dp, _dp, _dp, _ip]
        L.oracle_oz2_E.argtypes = [_dp, _dp, i64, i64, i64, ci, _dp, _dp]
        L.oracle_oz2_exact_sub.argtypes = [_dp, _dp, _dp, i64, i64, i64, ci, ci, ci, _ip, _ip, _fp, _fp, _fp]
        L.oracle_oz1.argtypes = [_dp, _dp, _dp, i64, i64, i64, ci, ci]
        L.oracle_fast_integerise.argtypes = [_dp, _dp, i64, i64, i64, ctypes.c_double, _ip, _ip,
                                             ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
        L.oz2_floor_log2_model.argtypes = [ctypes.c_double]
        L.oz2_floor_log2_model.restype = ci
        _lib = L
    return _lib


def _p(a, t=_dp):
    return a.ctypes.data_as(t)


def oz2_E(A, B, n_mod=16) -> int:
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    return lib().oracle_oz2_E(_p(A), _p(B), A.shape[0], A.shape[1], B.shape[1], n_mod, None, None)


def oz2_exact(A, B, E=None, n_mod=16, flags=EXPFIELD, debug=False):
    """Exact-tier product of the given rows of A and columns of B (both already
    sliced).  E defaults to the value for these operands taken as the whole problem."""
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    m, K = A.shape
    n = B.shape[1]
    if E is None:
        E = oz2_E(A, B, n_mod)
    C = np.empty((m, n), dtype=np.float64)
    if not debug:
        rc = lib().oracle_oz2_exact_sub(_p(A), _p(B), _p(C), m, K, n, E, n_mod, flags, None, None, None, None, None)
        assert rc == 0
        return C
    mu = np.empty(m, dtype=np.int32)
    nu = np.empty(n, dtype=np.int32)
    W = np.empty((n_mod, m, n), dtype=np.float32)
    Ar = np.empty((n_mod, m, K), dtype=np.float32)
    Br = np.empty((n_mod, K, n), dtype=np.float32)
    rc = lib().oracle_oz2_exact_sub(_p(A), _p(B), _p(C), m, K, n, E, n_mod, flags, _p(mu, _ip), _p(nu, _ip),
                                    _p(W, _fp), _p(Ar, _fp), _p(Br, _fp))
    assert rc == 0
    return C, {"mu": mu, "nu": nu, "W": W, "Ares": Ar, "Bres": Br, "E": E}


def oz1(A, B, T=6, max_pairs=8):
    """Ozaki-I restatement; max_pairs models the library's per-accumulator pair limit."""
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    C = np.empty((A.shape[0], B.shape[1]), dtype=np.float64)
    rc = lib().oracle_oz1(_p(A), _p(B), _p(C), A.shape[0], A.shape[1], B.shape[1], T, max_pairs)
    assert rc == 0
    return C


MODULI = (256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193)


def fast_exact_reference(A, B, n_mod=11):
    """What an error-free fast tier returns: the exact integer product of the
    round-half-up integerised operands, reduced to the centred residue modulo P and
    scaled back (python integers; small shapes only)."""
    import math
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    M, K = A.shape
    N = B.shape[1]
    P = 1
    for p in MODULI[:n_mod]:
        P *= p
    log2P = math.log2(float(P))
    er = np.empty(M, dtype=np.int32)
    ec = np.empty(N, dtype=np.int32)
    Ai = np.empty((M, K), dtype=np.int64)
    Bi = np.empty((K, N), dtype=np.int64)
    i64p = ctypes.POINTER(ctypes.c_int64)
    E = lib().oracle_fast_integerise(_p(A), _p(B), M, K, N, log2P, _p(er, _ip), _p(ec, _ip), _p(Ai, i64p), _p(Bi, i64p))
    X = Ai.astype(object) @ Bi.astype(object)
    C = np.empty((M, N), dtype=np.float64)
    for i in range(M):
        for j in range(N):
            x = int(X[i, j]) % P
            if 2 * x >= P:
                x -= P
            C[i, j] = math.ldexp(float(x), int(er[i]) + int(ec[j]) - 2 * E)
    return C, E


def floor_log2_model(x: float) -> int:
    return lib().oz2_floor_log2_model(float(x))


def ref_lib(name: str):
    """One of the reference-compiled libraries under oracle/_ref, or None if absent."""
    path = os.path.join(ORACLE_DIR, "_ref", name)
    if not os.path.exists(path):
        return None
    return ctypes.CDLL(path)


def set_threads(n: int) -> int:
    """Thread count of the oracle's OpenMP loops (libgomp reads OMP_NUM_THREADS only when it is
    loaded, and launchers such as torch.distributed.run export OMP_NUM_THREADS=1).  Returns the
    count in force."""
    L = lib()
    if n > 0:
        L.omp_set_num_threads(int(n))
    return int(L.omp_get_max_threads())


def ref_blas_threads(n: int = 0) -> int:
    """Set (n > 0) and read back the thread count of the OpenBLAS the reference's cblas path is
    linked against; 0 when that library is not built."""
    L = ref_lib("libref_matmul_blas.so")
    if L is None:
        return 0
    if n > 0:
        L.openblas_set_num_threads(int(n))
    return int(L.openblas_get_num_threads())


def ref_matmul(A, B, blas: bool = False):
    L = ref_lib("libref_matmul_blas.so" if blas else "libref_matmul_simd.so")
    if L is None:
        return None
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    C = np.zeros((A.shape[0], B.shape[1]), dtype=np.float64)
    u64 = ctypes.c_uint64
    L.eshkol_matmul_f64.argtypes = [_dp, _dp, _dp, u64, u64, u64]
    L.eshkol_matmul_f64.restype = None
    L.eshkol_matmul_f64(_p(A), _p(B), _p(C), A.shape[0], A.shape[1], B.shape[1])
    return C


def ref_matmul_backward(G, A, B, blas: bool = True):
    """The reference's own eshkol_matmul_backward_f64 (lib/backend/blas_backend.cpp:924), CPU build."""
    L = ref_lib("libref_matmul_blas.so" if blas else "libref_matmul_simd.so")
    if L is None or not hasattr(L, "eshkol_matmul_backward_f64"):
        return None
    G = np.ascontiguousarray(G, dtype=np.float64)
    A = np.ascontiguousarray(A, dtype=np.float64)
    B = np.ascontiguousarray(B, dtype=np.float64)
    gA = np.zeros_like(A)
    gB = np.zeros_like(B)
    u64 = ctypes.c_uint64
    L.eshkol_matmul_backward_f64.argtypes = [_dp, _dp, _dp, _dp, _dp, u64, u64, u64]
    L.eshkol_matmul_backward_f64.restype = None
    L.eshkol_matmul_backward_f64(_p(G), _p(A), _p(B), _p(gA), _p(gB), A.shape[0], A.shape[1], B.shape[1])
    return gA, gB


def ref_conv2d(inp, ker, stride=1, pad=0):
    L = ref_lib("libref_conv.so")
    if L is None:
        return None
    inp = np.ascontiguousarray(inp, dtype=np.float64)
    ker = np.ascontiguousarray(ker, dtype=np.float64)
    b, ic, H, W = inp.shape
    oc, _, kH, kW = ker.shape
    i64 = ctypes.c_int64
    L.ref_conv_out_dim.argtypes = [i64] * 4
    L.ref_conv_out_dim.restype = i64
    oH, oW = L.ref_conv_out_dim(H, kH, stride, pad), L.ref_conv_out_dim(W, kW, stride, pad)
    out = np.zeros((b, oc, oH, oW), dtype=np.float64)
    L.ref_conv2d.argtypes = [_dp, i64, i64, i64, i64, _dp, i64, i64, i64, i64, i64, _dp]
    L.ref_conv2d.restype = None
    L.ref_conv2d(_p(inp), b, ic, H, W, _p(ker), oc, kH, kW, stride, pad, _p(out))
    return out
