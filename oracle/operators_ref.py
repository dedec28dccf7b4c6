"""CPU restatement (test infrastructure, not part of the product) of the reference's tensor
operators beside the matrix product, lib/backend/gpu/gpu_cuda_kernels.cu: reduce :76-141 and its
CPU twin lib/backend/gpu/gpu_memory_cuda.cpp:1247-1268, axis reduce :147-180, transpose :189-213,
softmax :319-343, normalize :364-389, batchnorm backward :489-521, layernorm backward :524-555.

numpy sums are pairwise where the reference's loops are serial, and the GPU kernels under test
share each sum between threads: the three agree to rounding, which is what the tests assert.
"""
import numpy as np

SUM, PROD, MIN, MAX, MEAN = range(5)


def reduce_all(x, op):
    x = np.asarray(x, dtype=np.float64).ravel()
    if op == SUM:
        return float(np.sum(x))
    if op == PROD:
        return float(np.prod(x))
    if op == MIN:
        return float(np.fmin.reduce(x, initial=np.inf))   # fmin / fmax: a NaN operand is ignored
    if op == MAX:
        return float(np.fmax.reduce(x, initial=-np.inf))
    if op == MEAN:
        return float(np.sum(x) / x.size)
    raise ValueError(op)


def reduce_axis(x, axis, op):
    x = np.asarray(x, dtype=np.float64)
    if op == SUM:
        return np.sum(x, axis=axis)
    if op == PROD:
        return np.prod(x, axis=axis)
    if op == MIN:
        return np.fmin.reduce(x, axis=axis, initial=np.inf)
    if op == MAX:
        return np.fmax.reduce(x, axis=axis, initial=-np.inf)
    if op == MEAN:
        return np.sum(x, axis=axis) / x.shape[axis]
    raise ValueError(op)


def softmax(x):
    """x: [slices, len]; the maximum is subtracted first and a zero sum divides by 1."""
    x = np.asarray(x, dtype=np.float64)
    m = np.fmax.reduce(x, axis=1, keepdims=True)
    e = np.exp(x - m)
    s = e.sum(axis=1, keepdims=True)
    s[s == 0.0] = 1.0
    return e / s


def normalize(x, gamma, beta, eps):
    """x: [slices, len]; scalar gamma / beta, population variance."""
    x = np.asarray(x, dtype=np.float64)
    n = x.shape[1]
    mean = x.sum(axis=1, keepdims=True) / n
    var = ((x - mean) ** 2).sum(axis=1, keepdims=True) / n
    return gamma * (x - mean) * (1.0 / np.sqrt(var + eps)) + beta


def batchnorm_backward(grad_out, x, mean, inv_std, gamma):
    """grad_out, x: [batch, features]; mean, inv_std, gamma: [features].
    Returns grad_input, grad_gamma, grad_beta."""
    N = grad_out.shape[0]
    nz = (x - mean) * inv_std
    sum_g = grad_out.sum(axis=0)
    sum_gn = (grad_out * nz).sum(axis=0)
    coeff = gamma * inv_std / N
    return coeff * (N * grad_out - sum_g - nz * sum_gn), sum_gn, sum_g


def layernorm_backward(grad_out, x, mean, inv_std, gamma):
    """grad_out, x: [samples, features]; mean, inv_std: [samples]; gamma: [features]."""
    D = grad_out.shape[1]
    g = grad_out * gamma
    nz = (x - mean[:, None]) * inv_std[:, None]
    sum_g = g.sum(axis=1, keepdims=True)
    sum_gn = (g * nz).sum(axis=1, keepdims=True)
    return (inv_std[:, None] / D) * (D * g - sum_g - nz * sum_gn)
