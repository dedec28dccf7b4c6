"""The vectorised restatement of the reference's tensor operators (oracle/operators_ref.py)
against the reference's own serial loops written out one statement at a time, on small cases."""
import math

import numpy as np

from eshkol_b200 import inputs
from oracle import operators_ref as ref


def test_softmax_and_normalize_follow_the_serial_loops():
    x = inputs.normal(1, (6, 17)) * 5.0
    sm, nm = np.empty_like(x), np.empty_like(x)
    for s in range(x.shape[0]):                 # lib/backend/gpu/gpu_cuda_kernels.cu:319-343
        m = x[s, 0]
        for k in range(1, x.shape[1]):
            m = max(m, x[s, k])
        tot = 0.0
        for k in range(x.shape[1]):
            sm[s, k] = math.exp(x[s, k] - m)
            tot += sm[s, k]
        if tot == 0.0:
            tot = 1.0
        sm[s] /= tot
        mean = sum(x[s]) / x.shape[1]           # :364-389
        var = sum((v - mean) ** 2 for v in x[s]) / x.shape[1]
        nm[s] = 0.7 * (x[s] - mean) * (1.0 / math.sqrt(var + 1e-5)) + 0.1
    assert np.allclose(ref.softmax(x), sm, rtol=1e-14, atol=0)
    assert np.allclose(ref.normalize(x, 0.7, 0.1, 1e-5), nm, rtol=1e-13, atol=1e-15)


def test_axis_reduce_follows_the_index_arithmetic():
    shape, axis = (3, 4, 5), 1
    x = inputs.normal(2, shape)
    flat = x.ravel()
    inner = 5
    out = np.empty(15)
    for idx in range(15):                       # gpu_cuda_kernels.cu:147-180
        o, r = divmod(idx, inner)
        acc = 0.0
        for k in range(shape[axis]):
            acc += flat[o * shape[axis] * inner + k * inner + r]
        out[idx] = acc
    assert np.allclose(ref.reduce_axis(x, axis, ref.SUM).ravel(), out, rtol=1e-14)
    y = x.copy()
    y[1, 2, 3] = np.nan
    assert np.isfinite(ref.reduce_axis(y, axis, ref.MIN)).all()      # fmin ignores the NaN
    assert ref.reduce_all(y, ref.MAX) == np.nanmax(y)


def test_normalisation_gradients_follow_the_serial_loops():
    g = inputs.normal(3, (5, 7))
    x = inputs.normal(4, (5, 7))
    gamma = 1.0 + 0.1 * inputs.normal(5, (7,))
    mean, inv_std = x.mean(axis=0), 1.0 / np.sqrt(x.var(axis=0) + 1e-5)
    gin, ggam, gbeta = ref.batchnorm_backward(g, x, mean, inv_std, gamma)
    for f in range(7):                          # gpu_cuda_kernels.cu:489-521
        sg = sgn = 0.0
        for b in range(5):
            nz = (x[b, f] - mean[f]) * inv_std[f]
            sg += g[b, f]
            sgn += g[b, f] * nz
        assert math.isclose(gbeta[f], sg, rel_tol=1e-13, abs_tol=1e-15)
        assert math.isclose(ggam[f], sgn, rel_tol=1e-13, abs_tol=1e-15)
        for b in range(5):
            nz = (x[b, f] - mean[f]) * inv_std[f]
            want = gamma[f] * inv_std[f] / 5.0 * (5.0 * g[b, f] - sg - nz * sgn)
            assert math.isclose(gin[b, f], want, rel_tol=1e-12, abs_tol=1e-14)
    mean, inv_std = x.mean(axis=1), 1.0 / np.sqrt(x.var(axis=1) + 1e-5)
    got = ref.layernorm_backward(g, x, mean, inv_std, gamma)
    for s in range(5):                          # :524-555
        sg = sgn = 0.0
        for f in range(7):
            gg = g[s, f] * gamma[f]
            nz = (x[s, f] - mean[s]) * inv_std[s]
            sg += gg
            sgn += gg * nz
        for f in range(7):
            gg = g[s, f] * gamma[f]
            nz = (x[s, f] - mean[s]) * inv_std[s]
            want = inv_std[s] / 7.0 * (7.0 * gg - sg - nz * sgn)
            assert math.isclose(got[s, f], want, rel_tol=1e-12, abs_tol=1e-14)
