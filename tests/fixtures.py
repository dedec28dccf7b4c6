"""Generators of the reference's own test fixtures, re-implemented from its test
sources (plain arithmetic, cited per function)."""
from __future__ import annotations

import math

import numpy as np


def certificate_operands(n: int = 512):
    """tests/gpu/ozaki_certification_test.esk:30-38: integer-valued 512x512 witness."""
    r = np.arange(n, dtype=np.int64)[:, None]
    c = np.arange(n, dtype=np.int64)[None, :]
    a = (16777216 + (r * 97 + c * 53) % 257) * np.where((r * 131 + c * 13) % 2 == 0, 1, -1)
    b = (16777216 + (r * 71 + c * 29 + r * c) % 257) * np.where((r * 73 + c * 23) % 2 == 0, 1, -1)
    return a, b


CERT_POINTS = (0, 128, 256, 384, 511)  # ozaki_certification_test.esk:19


def exact_dot(a_int, b_int, i, j) -> int:
    return sum(int(x) * int(y) for x, y in zip(a_int[i, :].tolist(), b_int[:, j].tolist()))


def regime_operands(regime: int, n: int):
    """tests/gpu/ozaki_correctness_test.esk:36-47: the four deterministic regimes."""
    i = np.arange(n * n, dtype=np.int64)
    if regime == 0:
        a = ((i % 7) - 3).astype(np.float64)
        b = ((i % 5) - 2).astype(np.float64)
    elif regime == 1:
        a = 1.0 + 0.5 * (i % 7).astype(np.float64)
        b = 0.5 + 0.25 * (i % 5).astype(np.float64)
    elif regime == 2:
        a = 3.141592653589793 * (1.0 + (i % 11).astype(np.float64))
        b = 2.718281828459045 * ((i % 9).astype(np.float64) - 4.0)
    else:
        a = np.power(2.0, ((i % 20) - 10).astype(np.float64)) * (1.0 + 0.1 * (i % 3).astype(np.float64))
        b = np.power(2.0, ((i % 18) - 9).astype(np.float64)) * (1.0 + 0.1 * (i % 4).astype(np.float64))
    return a.reshape(n, n), b.reshape(n, n)


def probe_grid(n: int):
    """ozaki_correctness_test.esk:56-57: the 5x5 probe positions."""
    return [(pr * (n - 1)) // 4 for pr in range(5)]


def naive_dot(A, B, i, j) -> float:
    """the probe's in-order f64 accumulation (ozaki_correctness_test.esk:59-62)"""
    ref = 0.0
    col = B[:, j]
    row = A[i, :]
    for k in range(A.shape[1]):
        ref += float(row[k]) * float(col[k])
    return ref


def rel_err(got: float, ref: float) -> float:
    """denominator rule of ozaki_correctness_test.esk:64-65"""
    denom = abs(ref) if abs(ref) > 1e-9 else 1.0
    return abs(got - ref) / denom


# tests/ml/conv_correctness_test.esk:38-106: (input shape, input, kernel shape, kernel, stride, pad, out shape, out);
# all seven cases, the second one in the 2-D single-plane form (:46-52)
CONV_CASES = [
    ((1, 1, 3, 3), [1.0] * 9, (1, 1, 2, 2), [1.0] * 4, 1, 0, (1, 1, 2, 2), [4.0] * 4),
    ((3, 3), [1.0] * 9, (2, 2), [1.0] * 4, 1, 0, (2, 2), [4.0] * 4),
    ((1, 1, 3, 3), [1, 2, 3, 4, 5, 6, 7, 8, 9], (1, 1, 2, 2), [1, 0, 0, 1], 1, 0, (1, 1, 2, 2), [6, 8, 12, 14]),
    ((1, 2, 2, 2), [1, 2, 3, 4, 5, 6, 7, 8], (1, 2, 2, 2), [1.0] * 8, 1, 0, (1, 1, 1, 1), [36.0]),
    ((1, 1, 2, 2), [1, 2, 3, 4], (2, 1, 2, 2), [1, 1, 1, 1, 1, 0, 0, 0], 1, 0, (1, 2, 1, 1), [10.0, 1.0]),
    ((1, 1, 4, 4), list(range(1, 17)), (1, 1, 2, 2), [1.0] * 4, 2, 0, (1, 1, 2, 2), [14, 22, 46, 54]),
    ((1, 1, 3, 3), [1.0] * 9, (1, 1, 3, 3), [1.0] * 9, 1, 1, (1, 1, 3, 3), [4, 6, 4, 6, 9, 6, 4, 6, 4]),
]


def conv_promote(ishape, kshape):
    """NCHW shapes the runtime entry point gives the kernel (lib/backend/tensor_conv_kernel.cpp:58-79):
    a kernel of rank >= 4 is [out_c, in_c, kH, kW] and every leading input dimension is a batch
    index; a kernel of lower rank is a single plane, every leading input dimension a plane."""
    ishape, kshape = tuple(ishape), tuple(kshape)
    H, W = ishape[-2:]
    kH, kW = kshape[-2:]
    if len(kshape) >= 4:
        batch = int(np.prod(ishape[:-3], dtype=np.int64)) if len(ishape) > 3 else 1
        return (batch, kshape[1], H, W), (kshape[0], kshape[1], kH, kW)
    batch = int(np.prod(ishape[:-2], dtype=np.int64)) if len(ishape) > 2 else 1
    return (batch, 1, H, W), (1, 1, kH, kW)


def conv2d_numpy(inp, ker, stride=1, pad=0):
    """Restatement of eshkol_conv2d_kernel (lib/backend/tensor_conv_kernel.h:66-105)
    with the same (ic, kh, kw) accumulation order."""
    inp = np.asarray(inp, dtype=np.float64)
    ker = np.asarray(ker, dtype=np.float64)
    b, ic, H, W = inp.shape
    oc, _, kH, kW = ker.shape
    stride = 1 if stride <= 0 else stride
    pad = 0 if pad < 0 else pad
    oH = 0 if H + 2 * pad - kH < 0 else (H + 2 * pad - kH) // stride + 1
    oW = 0 if W + 2 * pad - kW < 0 else (W + 2 * pad - kW) // stride + 1
    out = np.zeros((b, oc, oH, oW))
    for c in range(ic):
        for kh in range(kH):
            for kw in range(kW):
                for oh in range(oH):
                    ih = oh * stride + kh - pad
                    if ih < 0 or ih >= H:
                        continue
                    for ow in range(oW):
                        iw = ow * stride + kw - pad
                        if iw < 0 or iw >= W:
                            continue
                        out[:, :, oh, ow] += inp[:, c, ih, iw][:, None] * ker[:, c, kh, kw][None, :]
    return out


def im2col(inp, kH, kW, stride, pad):
    """[ic*kH*kW, batch*oH*oW] operand of the conv2d lowering (same ordering as the library)."""
    inp = np.asarray(inp, dtype=np.float64)
    b, ic, H, W = inp.shape
    oH = (H + 2 * pad - kH) // stride + 1
    oW = (W + 2 * pad - kW) // stride + 1
    padded = np.zeros((b, ic, H + 2 * pad, W + 2 * pad))
    padded[:, :, pad:pad + H, pad:pad + W] = inp
    col = np.empty((ic, kH, kW, b, oH, oW))
    for kh in range(kH):
        for kw in range(kW):
            col[:, kh, kw] = padded[:, :, kh:kh + stride * oH:stride, kw:kw + stride * oW:stride].transpose(1, 0, 2, 3)
    return col.reshape(ic * kH * kW, b * oH * oW), oH, oW
