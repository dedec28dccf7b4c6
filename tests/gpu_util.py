"""Helpers for the -m gpu tests: device memory through torch, compute through the C ABI."""
from __future__ import annotations

import numpy as np

import eshkol_b200 as eb
from eshkol_b200 import api


def gemm(A, B, tier=eb.TIER_OZAKI2, param=0, simt=False, tile_n=0, activation=0, bias=None, bias_mode=0,
         trans_a=False, trans_b=False):
    """C = op(A) @ op(B) on the GPU via eshkol_b200_gemm_f64_device; numpy in, numpy out.
    With trans_a / trans_b the array passed is the transposed storage (K x M, N x K)."""
    import torch
    dA = torch.from_numpy(np.ascontiguousarray(A, dtype=np.float64)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B, dtype=np.float64)).cuda()
    M, K = (dA.shape[1], dA.shape[0]) if trans_a else dA.shape
    N = dB.shape[0] if trans_b else dB.shape[1]
    dC = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    dbias = None
    if bias is not None:
        dbias = torch.from_numpy(np.ascontiguousarray(bias, dtype=np.float64)).cuda()
    torch.cuda.synchronize()
    opts = api.make_opts(tier, param, activation, dbias.data_ptr() if dbias is not None else 0, bias_mode,
                         simt, tile_n, 0, trans_a, trans_b)
    api.gemm_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, K, N, opts)
    st = api.sync_status()
    assert st == 0, f"kernel status {st}"
    return dC.cpu().numpy()


def decode_plane0(p0: np.ndarray, K: int):
    """modulus-256 plane (1024 bytes per 1008-element chunk) -> rows x K residue bytes"""
    k = np.arange(K)
    return p0[:, (k // 1008) * 1024 + (k % 1008)]


def decode_flags(units: np.ndarray, K: int):
    """flag bit-plane (64 16-bit units per chunk, bit b of unit u = element 16u + b) -> rows x K of 0/1"""
    k = np.arange(K)
    c, off = k // 1008, k % 1008
    u = units.view(np.uint16)[:, c * 64 + off // 16]
    return ((u >> (off % 16).astype(np.uint16)) & 1).astype(np.int32)


def same_bits(x: np.ndarray, y: np.ndarray) -> bool:
    return np.array_equal(np.ascontiguousarray(x).view(np.uint64), np.ascontiguousarray(y).view(np.uint64))
