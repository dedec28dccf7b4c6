"""Helpers for the -m gpu tests: device memory through torch, compute through the C ABI."""
from __future__ import annotations

import numpy as np

import eshkol_b200 as eb
from eshkol_b200 import api


def gemm(A, B, tier=eb.TIER_OZAKI2, param=0, simt=False, tile_n=0, activation=0, bias=None, bias_mode=0):
    """C = A @ B on the GPU via eshkol_b200_gemm_f64_device; numpy in, numpy out."""
    import torch
    dA = torch.from_numpy(np.ascontiguousarray(A, dtype=np.float64)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B, dtype=np.float64)).cuda()
    M, K = dA.shape
    N = dB.shape[1]
    dC = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    dbias = None
    if bias is not None:
        dbias = torch.from_numpy(np.ascontiguousarray(bias, dtype=np.float64)).cuda()
    torch.cuda.synchronize()
    opts = api.make_opts(tier, param, activation, dbias.data_ptr() if dbias is not None else 0, bias_mode,
                         simt, tile_n)
    api.gemm_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, K, N, opts)
    st = api.sync_status()
    assert st == 0, f"kernel status {st}"
    return dC.cpu().numpy()


def decode_plane0(p0: np.ndarray, K: int, meta: dict, operand: str):
    """modulus-256 plane -> (byte residue, +128 flag, odd flag), each rows x K"""
    CH, SEG, EXT = 1008, 1024, 3072
    k = np.arange(K)
    c = k // CH
    off = k % CH
    seglen = np.where(c == meta["n_chunks"] - 1, meta["last_seg"], SEG)
    col = c * EXT + off
    lo = p0[:, col]
    s1 = p0[:, col + seglen]
    s2 = p0[:, col + 2 * seglen]
    if operand == "A":
        return lo, s1, s2      # A: segment 1 = +128 flags, segment 2 = odd flags
    return lo, s2, s1          # B: segment 1 = odd flags, segment 2 = +128 flags


def same_bits(x: np.ndarray, y: np.ndarray) -> bool:
    return np.array_equal(np.ascontiguousarray(x).view(np.uint64), np.ascontiguousarray(y).view(np.uint64))
