"""The backend's tensor operators beside the matrix product, on the GPU, against the CPU
restatement of the reference's kernels (oracle/operators_ref.py).  Sums are associated
differently on the three sides, so sums are compared to rounding; min, max and transpose exactly."""
import ctypes

import numpy as np
import pytest

import eshkol_b200 as eb
from eshkol_b200 import api, inputs
from oracle import operators_ref as ref

pytestmark = pytest.mark.gpu


def dev(x):
    """x on the device, complete before the library's own (non-blocking) stream may read it"""
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    torch.cuda.synchronize()
    return t


def empty(shape):
    """NaN-filled output, the fill complete before the library's stream writes into it"""
    import torch
    t = torch.full(tuple(shape), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    return t


def done():
    assert api.sync_status() == 0


def close(got, want, cond=1.0):
    """|got - want| <= 64 ulp of the larger magnitude involved in the sum (cond scales it)"""
    got, want = np.asarray(got), np.asarray(want)
    return bool(np.all(np.abs(got - want) <= 64 * np.finfo(np.float64).eps * cond * np.maximum(1.0, np.abs(want))))


@pytest.mark.parametrize("n", [1, 7, 255, 4096, 1_000_003, 20_000_000])
@pytest.mark.parametrize("op", [ref.SUM, ref.PROD, ref.MIN, ref.MAX, ref.MEAN])
def test_full_reduce(gpu_lib, n, op):
    x = inputs.normal(11, (n,))
    if op == ref.PROD:
        x = 1.0 + x * 1e-4 / max(1.0, np.sqrt(n))  # keeps the product finite and well-conditioned
    if op in (ref.MIN, ref.MAX) and n > 3:
        x[3] = np.nan  # ignored by fmin / fmax
    dx, out = dev(x), empty((1,))
    assert gpu_lib.eshkol_b200_reduce_f64_device(dx.data_ptr(), out.data_ptr(), n, op) == 0
    done()
    got, want = float(out.cpu()[0]), ref.reduce_all(x, op)
    if op in (ref.MIN, ref.MAX):
        assert got == want
    else:
        eps = np.finfo(np.float64).eps
        if op == ref.PROD:
            # n - 1 roundings on either side, each half an ulp of the running product
            assert abs(got - want) <= max(64, n) * eps * abs(want)
        else:
            cond = float(np.sum(np.abs(x)))
            scale = cond / n if op == ref.MEAN else cond
            assert abs(got - want) <= 64 * eps * max(scale, abs(want), 1e-300)


@pytest.mark.parametrize("shape,axis", [((37, 1000), 1), ((3, 5000), 1), ((100000, 12), 1), ((64, 33, 70), 1),
                                        ((5000, 48), 0), ((200000, 4), 0), ((2, 3, 4, 5), 2), ((9, 1, 7), 1),
                                        ((70, 64, 33), 0), ((1, 1), 0)])
@pytest.mark.parametrize("op", [ref.SUM, ref.PROD, ref.MIN, ref.MAX, ref.MEAN])
def test_axis_reduce_through_the_buffer_api(gpu_lib, shape, axis, op):
    x = inputs.normal(12, shape)
    if op == ref.PROD:
        x = 1.0 + x * 1e-4
    want = ref.reduce_axis(x, axis, op)
    bi, bo = eb.EshkolGPUBuffer(), eb.EshkolGPUBuffer()
    assert gpu_lib.eshkol_gpu_alloc(x.nbytes, 3, ctypes.byref(bi)) == 0   # unified: host_ptr == device_ptr
    assert gpu_lib.eshkol_gpu_alloc(max(want.nbytes, 8), 3, ctypes.byref(bo)) == 0
    np.ctypeslib.as_array(ctypes.cast(bi.host_ptr, ctypes.POINTER(ctypes.c_double)), shape=(x.size,))[:] = x.ravel()
    dims = (ctypes.c_uint64 * len(shape))(*shape)
    assert gpu_lib.eshkol_gpu_reduce_axis_f64(ctypes.byref(bi), ctypes.byref(bo), len(shape), dims, axis, op) == 0
    got = np.ctypeslib.as_array(ctypes.cast(bo.host_ptr, ctypes.POINTER(ctypes.c_double)), shape=(want.size,)).copy()
    # too small an output, and an axis outside the rank, are refused
    if want.size > 1:
        small = eb.EshkolGPUBuffer()
        assert gpu_lib.eshkol_gpu_alloc(8, 3, ctypes.byref(small)) == 0
        assert gpu_lib.eshkol_gpu_reduce_axis_f64(ctypes.byref(bi), ctypes.byref(small), len(shape), dims, axis, op) == -1
        gpu_lib.eshkol_gpu_free(ctypes.byref(small))
    assert gpu_lib.eshkol_gpu_reduce_axis_f64(ctypes.byref(bi), ctypes.byref(bo), len(shape), dims, len(shape), op) == -1
    gpu_lib.eshkol_gpu_free(ctypes.byref(bi))
    gpu_lib.eshkol_gpu_free(ctypes.byref(bo))
    got = got.reshape(want.shape)
    if op in (ref.MIN, ref.MAX):
        assert np.array_equal(got, want)
    else:
        eps = np.finfo(np.float64).eps
        if op == ref.PROD:
            assert np.all(np.abs(got - want) <= max(64, shape[axis]) * eps * np.abs(want))
        else:
            cond = np.sum(np.abs(x), axis=axis)
            if op == ref.MEAN:
                cond = cond / shape[axis]
            assert np.all(np.abs(got - want) <= 64 * eps * np.maximum(cond, np.abs(want)))


@pytest.mark.parametrize("rows,cols", [(1, 1), (1, 999), (31, 33), (1000, 17), (4096, 4096), (5, 70001)])
def test_transpose_is_exact(gpu_lib, rows, cols):
    x = inputs.normal(13, (rows, cols))
    dx, out = dev(x), empty((cols, rows))
    assert gpu_lib.eshkol_b200_transpose_f64_device(dx.data_ptr(), out.data_ptr(), rows, cols) == 0
    done()
    assert np.array_equal(out.cpu().numpy(), x.T)
    assert gpu_lib.eshkol_b200_transpose_f64_device(dx.data_ptr(), dx.data_ptr(), rows, cols) == -1  # not in place


@pytest.mark.parametrize("slices,length", [(1, 1), (5, 3), (1000, 10), (4096, 512), (300, 1024), (9, 1025), (3, 50000),
                                           (100000, 32)])
def test_softmax_and_normalize(gpu_lib, slices, length):
    x = inputs.normal(14, (slices, length)) * 8.0
    if length > 2:
        x[0, 1] = 700.0   # exp would overflow without the maximum subtracted
    dx, out = dev(x), empty((slices, length))
    assert gpu_lib.eshkol_b200_softmax_f64_device(dx.data_ptr(), out.data_ptr(), slices, length) == 0
    done()
    got = out.cpu().numpy()
    assert close(got, ref.softmax(x), cond=4.0)
    assert np.all(np.abs(got.sum(axis=1) - 1.0) < 1e-12)
    # in place
    assert gpu_lib.eshkol_b200_softmax_f64_device(dx.data_ptr(), dx.data_ptr(), slices, length) == 0
    done()
    assert np.array_equal(dx.cpu().numpy(), got)
    # layer normalisation with scalar gamma / beta
    x = inputs.normal(15, (slices, length)) * 3.0 + 0.5
    dx = dev(x)
    assert gpu_lib.eshkol_b200_normalize_f64_device(dx.data_ptr(), out.data_ptr(), slices, length, 1.5, -0.25, 1e-5) == 0
    done()
    want = ref.normalize(x, 1.5, -0.25, 1e-5)
    assert np.all(np.abs(out.cpu().numpy() - want) <= 1e-12 * np.maximum(1.0, np.abs(want)))


def test_softmax_of_a_slice_of_minus_infinity_follows_the_reference(gpu_lib):
    """exp(-inf - -inf) is NaN in the reference's kernel too (gpu_cuda_kernels.cu:333): the slice
    comes out NaN, the other slices are untouched by it."""
    x = inputs.normal(16, (4, 40))
    x[2, :] = -np.inf
    dx, out = dev(x), empty((4, 40))
    assert gpu_lib.eshkol_b200_softmax_f64_device(dx.data_ptr(), out.data_ptr(), 4, 40) == 0
    done()
    got = out.cpu().numpy()
    assert np.isnan(got[2]).all()
    keep = [0, 1, 3]
    assert close(got[keep], ref.softmax(x[keep]), cond=4.0)


@pytest.mark.parametrize("batch,features", [(1, 1), (7, 5), (64, 1000), (5000, 33), (3, 100000), (100000, 3)])
def test_normalisation_gradients(gpu_lib, batch, features):
    g = inputs.normal(17, (batch, features))
    x = inputs.normal(18, (batch, features)) * 2.0 + 1.0
    gamma = 1.0 + 0.1 * inputs.normal(19, (features,))
    # batch norm: statistics per feature
    mean = x.mean(axis=0)
    inv_std = 1.0 / np.sqrt(x.var(axis=0) + 1e-5)
    dg, dx, dm, di, dgam = dev(g), dev(x), dev(mean), dev(inv_std), dev(gamma)
    gin, ggam, gbeta = empty((batch, features)), empty((features,)), empty((features,))
    assert gpu_lib.eshkol_b200_batchnorm_backward_f64_device(dg.data_ptr(), dx.data_ptr(), dm.data_ptr(), di.data_ptr(),
                                                             dgam.data_ptr(), gin.data_ptr(), ggam.data_ptr(),
                                                             gbeta.data_ptr(), batch, features) == 0
    done()
    w_in, w_gam, w_beta = ref.batchnorm_backward(g, x, mean, inv_std, gamma)
    scale = 1e-11 * max(1.0, float(np.abs(g).sum(axis=0).max()))
    assert np.all(np.abs(gbeta.cpu().numpy() - w_beta) <= scale)
    assert np.all(np.abs(ggam.cpu().numpy() - w_gam) <= scale * max(1.0, float(np.abs((x - mean) * inv_std).max())))
    assert np.all(np.abs(gin.cpu().numpy() - w_in) <= 1e-10 * np.maximum(1.0, np.abs(w_in).max()))
    # layer norm: statistics per sample
    mean = x.mean(axis=1)
    inv_std = 1.0 / np.sqrt(x.var(axis=1) + 1e-5)
    dm, di = dev(mean), dev(inv_std)
    gin = empty((batch, features))
    assert gpu_lib.eshkol_b200_layernorm_backward_f64_device(dg.data_ptr(), dx.data_ptr(), dm.data_ptr(), di.data_ptr(),
                                                             dgam.data_ptr(), gin.data_ptr(), batch, features) == 0
    done()
    want = ref.layernorm_backward(g, x, mean, inv_std, gamma)
    assert np.all(np.abs(gin.cpu().numpy() - want) <= 1e-10 * np.maximum(1.0, np.abs(want).max()))


def test_operators_through_wrapped_host_buffers(gpu_lib):
    """The buffer-level entry points on wrapped host arrays: upload, operator, download on sync."""
    lib = gpu_lib
    x = inputs.normal(20, (300, 200))
    y = np.zeros_like(x)
    t = np.zeros((200, 300))
    r = np.zeros(1)
    bx, by, bt, br = (eb.EshkolGPUBuffer() for _ in range(4))
    for arr, b in ((x, bx), (y, by), (t, bt), (r, br)):
        assert lib.eshkol_gpu_wrap_host(arr.ctypes.data, arr.nbytes, ctypes.byref(b)) == 0
    assert lib.eshkol_gpu_softmax_f64(ctypes.byref(bx), ctypes.byref(by), 300, 200) == 0
    assert lib.eshkol_gpu_transpose_f64(ctypes.byref(bx), ctypes.byref(bt), 300, 200) == 0
    assert lib.eshkol_gpu_reduce_f64(ctypes.byref(bx), ctypes.byref(br), x.size, ref.MAX) == 0
    assert lib.eshkol_gpu_reduce_f64(ctypes.byref(bx), ctypes.byref(br), x.size + 1, ref.MAX) == -1   # beyond the buffer
    assert lib.eshkol_gpu_transpose_f64(ctypes.byref(bx), ctypes.byref(br), 300, 200) == -1           # output too small
    for b in (by, bt, br):
        assert lib.eshkol_gpu_sync(ctypes.byref(b), 2) == 0   # ESHKOL_SYNC_DEVICE_TO_HOST
    assert close(y, ref.softmax(x), cond=4.0)
    assert np.array_equal(t, x.T)
    assert r[0] == x.max()
    assert lib.eshkol_gpu_normalize_f64(ctypes.byref(bx), ctypes.byref(by), 300, 200, 2.0, 1.0, 1e-6) == 0
    assert lib.eshkol_gpu_sync(ctypes.byref(by), 2) == 0
    want = ref.normalize(x, 2.0, 1.0, 1e-6)
    assert np.all(np.abs(y - want) <= 1e-12 * np.maximum(1.0, np.abs(want)))
    # a host-only buffer is refused: the caller's CPU path runs instead (no CPU fallback in here)
    host_only = eb.EshkolGPUBuffer()
    host_only.host_ptr = x.ctypes.data
    host_only.size_bytes = x.nbytes
    assert lib.eshkol_gpu_softmax_f64(ctypes.byref(host_only), ctypes.byref(by), 300, 200) == -1
    for b in (bx, by, bt, br):
        lib.eshkol_gpu_free(ctypes.byref(b))
