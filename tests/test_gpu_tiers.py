"""Reduced-precision tiers, conv2d and the host-pointer dispatchers on the GPU."""
import ctypes

import numpy as np
import pytest

import eshkol_b200 as eb
from eshkol_b200 import api, inputs
import fixtures as fx
import gpu_util as gu
import oracle_lib as ol

pytestmark = pytest.mark.gpu

# guaranteed relative error of the slice tiers (lib/backend/gpu/gpu_memory_cuda.cpp:485-487)
OZAKI_TOL = {1: 1e-3, 2: 1e-5, 3: 1e-7, 4: 1e-9, 5: 1e-11, 6: 1e-13, 7: 1e-14}
# published worst-case errors of the fast tier (docs/breakdown/GPU_ACCELERATION.md:173-179)
FAST_TOL = {10: 2.2e-7, 11: 2.4e-8, 12: 4.0e-8, 14: 6e-11}


def normwise(got, ref):
    return float(np.linalg.norm((got - ref).astype(np.float64)) / np.linalg.norm(ref.astype(np.float64)))


def true_product(A, B):
    """the product in 80-bit arithmetic: the 'exact f64 reference' the tier bounds are stated against"""
    return (A.astype(np.longdouble) @ B.astype(np.longdouble))


@pytest.mark.parametrize("T", [1, 2, 3, 4, 5, 6, 7])
def test_ozaki1_bits_match_restatement_and_meet_the_tier_bound(gpu_lib, T):
    A = inputs.normal(1, (200, 900))
    B = inputs.normal(2, (900, 300))
    got = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=T)
    assert gu.same_bits(got, ol.oz1(A, B, T))
    assert normwise(got, true_product(A, B)) < OZAKI_TOL[T]


def test_ozaki1_cuda_core_and_tensor_core_products_agree(gpu_lib):
    A = inputs.wide(3, (130, 1300), span=9, lo=-4)
    B = inputs.wide(4, (1300, 270), span=9, lo=-4)
    a = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=6, simt=True)
    b = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=6)
    assert gu.same_bits(a, b)


@pytest.mark.parametrize("regime", [0, 1, 2, 3])
def test_ozaki1_reference_gate(gpu_lib, regime):
    # tests/gpu/cuda_ozaki_correctness_gate.sh:99-118: T=6 normwise < 1e-9, T=4 < 1e-6 over the probe grid
    n = 1024
    A, B = fx.regime_operands(regime, n)
    rows = fx.probe_grid(n)
    ref = np.array([[fx.naive_dot(A, B, i, j) for j in rows] for i in rows])
    for T, tol in ((6, 1e-9), (4, 1e-6)):
        C = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=T)
        assert normwise(C[np.ix_(rows, rows)], ref) < tol


@pytest.mark.parametrize("n_mod", [10, 11, 12, 14, 16])
def test_fast_tier_within_published_bounds(gpu_lib, n_mod):
    A = inputs.normal(5, (96, 700))
    B = inputs.normal(6, (700, 80))
    got = gu.gemm(A, B, tier=eb.TIER_OZAKI2_FAST, param=n_mod)
    # the integer CRT is error-free: same bits as python integers on the integerised operands
    ideal, E = ol.fast_exact_reference(A, B, n_mod)
    assert gu.same_bits(got, ideal)
    # against the true product: the tier's documented accuracy (normwise; cells that
    # cancel to almost nothing have no meaningful element-wise relative error)
    assert normwise(got, true_product(A, B)) < FAST_TOL.get(n_mod, 1e-10), (n_mod, E)


@pytest.mark.parametrize("regime", [0, 1, 2, 3])
def test_fast_tier_reference_gate(gpu_lib, regime):
    # tests/gpu/ozaki_fast_test.esk:13: max rel err < 1e-7 at the default 11 moduli
    n = 512
    A, B = fx.regime_operands(regime, n)
    C = gu.gemm(A, B, tier=eb.TIER_OZAKI2_FAST, param=11)
    rows = fx.probe_grid(n)
    assert max(fx.rel_err(C[i, j], fx.naive_dot(A, B, i, j)) for i in rows for j in rows) < 1e-7


def test_native_dgemm_tier(gpu_lib):
    A = inputs.uniform(7, (150, 333))
    B = inputs.uniform(8, (333, 97))
    got = gu.gemm(A, B, tier=eb.TIER_DGEMM)
    assert np.max(np.abs(got - A @ B)) < 1e-12


def _conv_gpu(inp, ker, stride, pad, activation=0):
    return api.conv2d(inp, ker, stride, pad, activation)


@pytest.mark.parametrize("case", range(len(fx.CONV_CASES)))
def test_conv_known_answers(gpu_lib, case):
    ishape, ival, kshape, kval, stride, pad, oshape, oval = fx.CONV_CASES[case]
    ishape, kshape = fx.conv_promote(ishape, kshape)  # the 2-D form reaches the kernel as NCHW with one plane
    inp = np.array(ival, dtype=np.float64).reshape(ishape)
    ker = np.array(kval, dtype=np.float64).reshape(kshape)
    got = _conv_gpu(inp, ker, stride, pad)
    assert got.size == int(np.prod(oshape))
    assert np.allclose(got.reshape(oshape), np.array(oval, dtype=np.float64).reshape(oshape), rtol=0, atol=1e-9)


@pytest.mark.parametrize("cfg", [(2, 5, 13, 11, 7, 3, 3, 1, 1), (3, 4, 9, 9, 6, 2, 3, 2, 0), (1, 3, 8, 8, 130, 3, 3, 1, 1)])
def test_conv_bits_match_oracle_on_the_lowered_operands(gpu_lib, cfg):
    b, ic, H, W, oc, kH, kW, stride, pad = cfg
    inp = inputs.normal(1, (b, ic, H, W), scale=0.1)
    ker = inputs.normal(2, (oc, ic, kH, kW), scale=0.1)
    got = _conv_gpu(inp, ker, stride, pad, activation=1)
    col, oH, oW = fx.im2col(inp, kH, kW, stride, pad)
    low = ol.oz2_exact(ker.reshape(oc, -1), col, 52).reshape(oc, b, oH, oW).transpose(1, 0, 2, 3)
    assert gu.same_bits(got, np.where(low > 0.0, low, 0.0))
    # against the direct loop: every cell to rounding except the few that carry the
    # exact tier's own 2^-25-relative CRT rounding (its split weights sl1 round in about 0.7 % of the cells)
    direct = fx.conv2d_numpy(inp, ker, stride, pad)
    direct = np.where(direct > 0.0, direct, 0.0)
    err = np.abs(got - direct)
    assert np.median(err) < 1e-15 and np.mean(err < 1e-12) > 0.95 and err.max() < 1e-7


def test_conv_c4_whole_result_bit_exact(gpu_lib):
    """The conv2d benchmark configuration: batch 32, 64 -> 128 channels, 56 x 56, 3 x 3, stride 1,
    pad 1, inputs and weights normal(0, 0.1), fused ReLU.  The whole output, bit for bit, against
    the oracle's exact-tier product of the weight matrix with the im2col operand (the library
    itself never builds that operand: its scan and split read the NCHW tensor through the index
    map), and against the reference's direct loop to the exact tier's own error."""
    ol.set_threads(len(__import__("os").sched_getaffinity(0)))
    inp = inputs.normal(1, (32, 64, 56, 56), scale=0.1)
    ker = inputs.normal(2, (128, 64, 3, 3), scale=0.1)
    got = _conv_gpu(inp, ker, 1, 1, activation=1)
    assert got.shape == (32, 128, 56, 56)
    col, oH, oW = fx.im2col(inp, 3, 3, 1, 1)
    low = ol.oz2_exact(ker.reshape(128, -1), col, 52)
    low = np.where(low > 0.0, low, 0.0).reshape(128, 32, oH, oW).transpose(1, 0, 2, 3)
    assert gu.same_bits(got, np.ascontiguousarray(low))
    ref = ol.ref_conv2d(inp[:1], ker, 1, 1)
    if ref is not None:
        err = np.abs(got[0] - np.where(ref[0] > 0.0, ref[0], 0.0))
        assert np.mean(err < 1e-12) > 0.95 and err.max() < 1e-6


def _make_tensor(arr):
    """eshkol_tensor_t over a numpy array (kept alive by the returned tuple)"""
    from eshkol_b200.abi import EshkolTensor
    arr = np.ascontiguousarray(arr, dtype=np.float64)
    dims = (ctypes.c_uint64 * arr.ndim)(*arr.shape)
    t = EshkolTensor()
    t.dimensions = ctypes.cast(dims, ctypes.POINTER(ctypes.c_uint64))
    t.num_dimensions = arr.ndim
    t.elements = ctypes.cast(arr.ctypes.data, ctypes.POINTER(ctypes.c_int64))
    t.total_elements = arr.size
    t.dtype = 0
    return t, (arr, dims)


@pytest.mark.parametrize("case", range(len(fx.CONV_CASES)))
def test_rt_conv2d_on_tensor_structs(gpu_lib, case):
    """eshkol_rt_conv2d, the symbol generated code calls (lib/backend/tensor_conv_kernel.cpp:32-109):
    heap tensors in, a fresh tensor out whose shape follows the reference's contract -- including
    the 2-D single-plane form, which keeps its rank."""
    from eshkol_b200.abi import EshkolTensor
    ishape, ival, kshape, kval, stride, pad, oshape, oval = fx.CONV_CASES[case]
    made = []

    @ctypes.CFUNCTYPE(ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64)
    def allocate(arena, nd, total):
        t = EshkolTensor()
        dims = (ctypes.c_uint64 * max(1, nd))()
        elems = (ctypes.c_int64 * max(1, total))()
        t.dimensions = ctypes.cast(dims, ctypes.POINTER(ctypes.c_uint64))
        t.elements = ctypes.cast(elems, ctypes.POINTER(ctypes.c_int64))
        t.num_dimensions, t.total_elements, t.dtype = nd, total, 0
        made.append((t, dims, elems))
        return ctypes.addressof(t)

    gpu_lib.eshkol_b200_set_tensor_allocator(ctypes.cast(allocate, ctypes.c_void_p))
    try:
        ti, keep_i = _make_tensor(np.array(ival, dtype=np.float64).reshape(ishape))
        tk, keep_k = _make_tensor(np.array(kval, dtype=np.float64).reshape(kshape))
        arena = ctypes.c_int(0)
        out = gpu_lib.eshkol_rt_conv2d(ctypes.addressof(arena), ctypes.addressof(ti), ctypes.addressof(tk), stride, pad)
        assert out, "eshkol_rt_conv2d returned NULL"
        t = EshkolTensor.from_address(out)
        assert tuple(t.dimensions[i] for i in range(t.num_dimensions)) == tuple(oshape)
        got = np.ctypeslib.as_array(ctypes.cast(t.elements, ctypes.POINTER(ctypes.c_double)), shape=(t.total_elements,))
        assert np.allclose(got, np.array(oval, dtype=np.float64), rtol=0, atol=1e-9)
        # shape errors give NULL, as in the reference: mismatched channels, kernel larger than the input
        bad, keep_b = _make_tensor(np.zeros((1, 3, 5, 5)))
        k2, keep_k2 = _make_tensor(np.zeros((2, 2, 3, 3)))
        assert not gpu_lib.eshkol_rt_conv2d(ctypes.addressof(arena), ctypes.addressof(bad), ctypes.addressof(k2), 1, 0)
        big, keep_big = _make_tensor(np.zeros((1, 1, 9, 9)))
        assert not gpu_lib.eshkol_rt_conv2d(ctypes.addressof(arena), ctypes.addressof(ti), ctypes.addressof(big), 1, 0)
    finally:
        gpu_lib.eshkol_b200_set_tensor_allocator(None)


def test_dispatch_on_host_pointers(gpu_lib):
    gpu_lib.eshkol_gpu_set_threshold(1)  # as the reference's GPU gates do with ESHKOL_GPU_THRESHOLD=1
    try:
        assert np.array_equal(eb.matmul_dispatch([[1, 2], [3, 4]], [[5, 6], [7, 8]]), [[19, 22], [43, 50]])
        assert np.array_equal(eb.matmul_dispatch([[1, 2, 3], [4, 5, 6]], [[7, 8], [9, 10], [11, 12]]),
                              [[58, 64], [139, 154]])
        A = inputs.uniform(1, (50, 50))
        assert gu.same_bits(eb.matmul_dispatch(A, np.eye(50)), ol.oz2_exact(A, np.eye(50), 52))
        assert np.array_equal(eb.matmul_dispatch(np.arange(64.0).reshape(8, 8) - 17.0, np.eye(8)),
                              np.arange(64.0).reshape(8, 8) - 17.0)
        A = inputs.full53(3, (333, 777))[:, 1:]          # unaligned, non-contiguous source made contiguous
        B = inputs.full53(4, (776, 201))
        assert gu.same_bits(eb.matmul_dispatch(A, B), ol.oz2_exact(np.ascontiguousarray(A), B, 52))
        a = inputs.uniform(5, (3, 40, 64))
        b = inputs.uniform(6, (3, 64, 24))
        c = eb.batch_matmul_dispatch(a, b)
        for i in range(3):
            assert gu.same_bits(c[i], ol.oz2_exact(a[i], b[i], 52))
    finally:
        gpu_lib.eshkol_gpu_set_threshold(100000)


def test_buffer_api_round_trip_like_the_vm(gpu_lib):
    # lib/backend/vm_gpu_dispatch.h:62-86: wrap three host arrays, multiply, free (no explicit sync)
    A = inputs.uniform(1, (120, 256))
    B = inputs.uniform(2, (256, 140))
    C = np.zeros((120, 140))
    ba, bb, bc = eb.EshkolGPUBuffer(), eb.EshkolGPUBuffer(), eb.EshkolGPUBuffer()
    assert gpu_lib.eshkol_gpu_wrap_host(A.ctypes.data, A.nbytes, ctypes.byref(ba)) == 0
    assert gpu_lib.eshkol_gpu_wrap_host(B.ctypes.data, B.nbytes, ctypes.byref(bb)) == 0
    assert gpu_lib.eshkol_gpu_wrap_host(C.ctypes.data, C.nbytes, ctypes.byref(bc)) == 0
    assert gpu_lib.eshkol_gpu_matmul_f64(ctypes.byref(ba), ctypes.byref(bb), ctypes.byref(bc), 120, 256, 140) == 0
    for b in (ba, bb, bc):
        gpu_lib.eshkol_gpu_free(ctypes.byref(b))
    assert bc.device_ptr is None and bc.size_bytes == 0
    assert gu.same_bits(C, ol.oz2_exact(A, B, 52))
    # device buffers + elementwise ReLU (lib/backend/gpu/gpu_cuda_kernels.cu:37)
    x = eb.EshkolGPUBuffer()
    assert gpu_lib.eshkol_gpu_alloc(C.nbytes, 3, ctypes.byref(x)) == 0  # unified: host_ptr == device_ptr
    assert x.host_ptr == x.device_ptr
    v = np.ctypeslib.as_array(ctypes.cast(x.host_ptr, ctypes.POINTER(ctypes.c_double)), shape=(C.size,))
    v[:] = np.linspace(-1, 1, C.size)
    v[0] = float("nan")
    assert gpu_lib.eshkol_gpu_elementwise_f64(ctypes.byref(x), None, ctypes.byref(x), C.size, 11) == 0
    assert v[0] == 0.0 and v.min() == 0.0 and v[-1] == 1.0
    gpu_lib.eshkol_gpu_free(ctypes.byref(x))


def test_residency_chain_uploads_each_operand_once(gpu_lib):
    """(matmul (matmul A B) A), the chain of tests/gpu/matmul_correctness_test.esk:54, through
    eshkol_matmul_dispatch with residency on: A and B cross the link once each, the first result
    is found on the device as the left operand of the second product, a repeated product with
    the same right-hand operand neither uploads nor splits it again, and every result carries the
    bits of the plain path.  After eshkol_gpu_invalidate a changed operand is uploaded again."""
    lib = gpu_lib
    n = 1024
    A = inputs.uniform(71, (n, n))
    B = inputs.uniform(72, (n, n))
    C1 = np.full((n, n), np.nan)
    C2 = np.full((n, n), np.nan)
    want1 = ol.oz2_exact(A, B, 52)
    want2 = ol.oz2_exact(want1, A, 52)
    h2d, d2h = ctypes.c_uint64(), ctypes.c_uint64()

    def moved():
        lib.eshkol_b200_transfer_bytes(ctypes.byref(h2d), ctypes.byref(d2h))
        return h2d.value, d2h.value

    old = lib.eshkol_gpu_get_threshold()
    lib.eshkol_gpu_set_threshold(1)
    lib.eshkol_gpu_set_residency(1, 4096)
    try:
        up0, down0 = moved()
        lib.eshkol_matmul_dispatch(A.ctypes.data, B.ctypes.data, C1.ctypes.data, n, n, n, 0)
        up1, down1 = moved()
        assert up1 - up0 == A.nbytes + B.nbytes and down1 - down0 == C1.nbytes
        assert gu.same_bits(C1, want1)
        lib.eshkol_matmul_dispatch(C1.ctypes.data, A.ctypes.data, C2.ctypes.data, n, n, n, 0)
        up2, down2 = moved()
        assert up2 == up1, "the second product of the chain uploaded something"
        assert down2 - down1 == C2.nbytes
        assert gu.same_bits(C2, want2)
        # the same right-hand operand again: still prepared, so no upload and no new preparation
        tok = lib.eshkol_b200_prepared_b_token()
        assert tok != 0
        A2 = inputs.uniform(73, (n, n))
        C3 = np.full((n, n), np.nan)
        lib.eshkol_matmul_dispatch(A2.ctypes.data, A.ctypes.data, C3.ctypes.data, n, n, n, 0)
        up3, _ = moved()
        assert up3 - up2 == A2.nbytes
        assert lib.eshkol_b200_prepared_b_token() == tok
        assert gu.same_bits(C3, ol.oz2_exact(A2, A, 52))
        # the host changes B and says so
        B[17, 33] = 0.123
        lib.eshkol_gpu_invalidate(B.ctypes.data, 0)
        lib.eshkol_matmul_dispatch(A.ctypes.data, B.ctypes.data, C1.ctypes.data, n, n, n, 0)
        up4, _ = moved()
        assert up4 - up3 == B.nbytes
        assert gu.same_bits(C1, ol.oz2_exact(A, B, 52))
        # ... and a change it forgot to report is caught when it touches a sampled value
        A[0, 0] = 0.5
        lib.eshkol_matmul_dispatch(A.ctypes.data, B.ctypes.data, C1.ctypes.data, n, n, n, 0)
        assert gu.same_bits(C1, ol.oz2_exact(A, B, 52))
    finally:
        lib.eshkol_gpu_set_residency(0, 0)
        lib.eshkol_gpu_set_threshold(old)


def test_dispatch_on_pageable_and_pinned_host_memory_agree(gpu_lib):
    """Arena memory is pageable: the dispatcher moves it through pinned staging slots filled by a
    few copy threads.  Same bits as from pinned memory, for a shape of several row blocks and
    with sizes that are not multiples of the staging chunk."""
    import torch
    lib = gpu_lib
    M, K, N = 3000, 1100, 1300
    A = inputs.uniform(75, (M, K))
    B = inputs.uniform(76, (K, N))
    C_page = np.full((M, N), np.nan)
    pA, pB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
    pC = torch.empty((M, N), dtype=torch.float64).pin_memory()
    old = lib.eshkol_gpu_get_threshold()
    lib.eshkol_gpu_set_threshold(1)
    try:
        lib.eshkol_matmul_dispatch(A.ctypes.data, B.ctypes.data, C_page.ctypes.data, M, K, N, 0)
        lib.eshkol_matmul_dispatch(pA.data_ptr(), pB.data_ptr(), pC.data_ptr(), M, K, N, 0)
    finally:
        lib.eshkol_gpu_set_threshold(old)
    assert gu.same_bits(C_page, pC.numpy())
    assert gu.same_bits(C_page[:64], ol.oz2_exact(A[:64], B, 52))


def test_buffer_api_rejects_buffers_smaller_than_their_operands(gpu_lib):
    lib = gpu_lib
    bufs = [eb.EshkolGPUBuffer() for _ in range(3)]
    for b, nbytes in zip(bufs, (64 * 64 * 8, 64 * 64 * 8, 64 * 32 * 8)):
        assert lib.eshkol_gpu_alloc(nbytes, 2, ctypes.byref(b)) == 0  # ESHKOL_MEM_DEVICE
    a, b, c = (ctypes.byref(x) for x in bufs)
    assert lib.eshkol_gpu_matmul_f64(a, b, c, 64, 64, 64) == -1      # C holds 64 x 32
    assert lib.eshkol_gpu_matmul_f64(a, b, c, 64, 128, 32) == -1     # A and B too small for K = 128
    assert lib.eshkol_gpu_matmul_f64(a, b, c, 64, 64, 32) == 0
    assert lib.eshkol_gpu_elementwise_f64(a, b, c, 64 * 64, 0) == -1  # out holds 64 x 32
    assert lib.eshkol_gpu_elementwise_f64(a, b, c, 64 * 32, 0) == 0
    assert lib.eshkol_gpu_conv2d_backward_input_f64(a, b, c, 64, 64, 3, 3, 62, 62, 1, 1, 4, 4, 1) == -1
    assert lib.eshkol_gpu_conv2d_backward_kernel_f64(a, b, c, 64, 64, 3, 3, 62, 62, 1, 1, 4, 4, 1) == -1
    for x in bufs:
        lib.eshkol_gpu_free(ctypes.byref(x))


def test_an_allocation_failure_is_loud_and_leaves_the_library_usable(gpu_lib):
    """Host-side failure injection: the n-th device allocation of the library is made to fail, as
    an exhausted device would.  The device entry point returns -1, the void dispatcher fills C
    with NaN instead of leaving a number of unknown provenance, and the very next call works."""
    import torch
    lib = gpu_lib
    n = 700  # a shape no earlier test used, so the product has to grow the library's scratch
    A = inputs.uniform(77, (n + 3000, n))
    B = inputs.uniform(78, (n, n + 5000))
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.zeros((A.shape[0], B.shape[1]), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    lib.eshkol_gpu_residency_clear()
    lib.eshkol_b200_shutdown()           # drop every grow-only block: the next product must allocate
    assert lib.eshkol_b200_init(torch.cuda.current_device()) == 0
    lib.eshkol_b200_debug_fail_allocation(1)
    try:
        rc = lib.eshkol_b200_gemm_f64_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), A.shape[0], n, B.shape[1], None)
        assert rc == -1
    finally:
        lib.eshkol_b200_debug_fail_allocation(0)
    assert api.sync_status() == 0
    # the dispatcher: every allocation of the call fails in turn until the call gets through
    old = lib.eshkol_gpu_get_threshold()
    lib.eshkol_gpu_set_threshold(1)
    try:
        failures = 0
        A64, B96 = np.ascontiguousarray(A[:64]), np.ascontiguousarray(B[:, :96])  # alive across the calls
        want = ol.oz2_exact(A64, B96, 52)
        for nth in range(1, 8):
            C = np.zeros((64, 96))
            lib.eshkol_gpu_residency_clear()
            lib.eshkol_b200_shutdown()
            assert lib.eshkol_b200_init(torch.cuda.current_device()) == 0
            lib.eshkol_b200_debug_fail_allocation(nth)
            lib.eshkol_matmul_dispatch(A64.ctypes.data, B96.ctypes.data, C.ctypes.data, 64, n, 96, 0)
            lib.eshkol_b200_debug_fail_allocation(0)
            if np.isnan(C).all():
                failures += 1
            else:
                assert gu.same_bits(C, want)
        assert failures >= 2   # the staging block and the prepared operand; a failed first try for the scratch falls back to the exact size
    finally:
        lib.eshkol_b200_debug_fail_allocation(0)
        lib.eshkol_gpu_set_threshold(old)
    assert gu.same_bits(gu.gemm(A64, B96), want)


def test_reduced_tiers_refuse_k_beyond_their_int32_bound(gpu_lib):
    """One int8 product of the slice tier is exact only while K * 127^2 < 2^31
    (lib/backend/gpu/gpu_memory_cuda.cpp:351-361): the slice and fast tiers say so and return -1;
    the buffer API then takes the exact tier, which has no depth limit."""
    import torch
    K = 140000
    a = torch.zeros((1, K), dtype=torch.float64, device="cuda")
    b = torch.zeros((K, 1), dtype=torch.float64, device="cuda")
    c = torch.zeros((1, 1), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    for tier, param in ((eb.TIER_OZAKI1, 6), (eb.TIER_OZAKI2_FAST, 11)):
        opts = api.make_opts(tier, param)
        assert gpu_lib.eshkol_b200_gemm_f64_device(a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, K, 1, ctypes.byref(opts)) == -1
    assert api.sync_status() == 0


def _f16_reference(A, B):
    """The reference's dtype fast path restated on the CPU (lib/backend/gpu/gpu_memory_cuda.cpp:677-733):
    operands rounded f64 -> f32 -> f16, product with wide accumulation, result rounded to f16.
    Returns (half-rounded exact product, sum |a||b| of the rounded operands)."""
    a = np.asarray(A, dtype=np.float64).astype(np.float32).astype(np.float16).astype(np.float64)
    b = np.asarray(B, dtype=np.float64).astype(np.float32).astype(np.float16).astype(np.float64)
    exact = a @ b  # products of halves are exact in f64; the f64 sum is exact to 2^-53 relative
    return exact, np.abs(a) @ np.abs(b)


def _check_f16(got, exact, mag, K):
    # f32 accumulation in an unspecified order: |acc - exact| <= K * 2^-24 * sum|a||b| (first order);
    # the final rounding to f16 adds half an f16 ulp of the accumulated value: 2^-11 relative
    # (2^-25 absolute in the subnormal range)
    acc_err = K * 2.0 ** -24 * mag
    bound = acc_err + 2.0 ** -11 * (np.abs(exact) + acc_err) + 2.0 ** -25
    assert np.all(np.isfinite(got))
    assert np.all(np.abs(got - exact) <= bound)
    # every output is an f16 value
    assert np.array_equal(got, got.astype(np.float16).astype(np.float64))


@pytest.mark.parametrize("shape", [(128, 64, 256), (300, 200, 130), (1, 1, 1), (513, 1000, 77), (1024, 4096, 512)])
def test_f16_fast_path_device(gpu_lib, shape):
    import torch
    M, K, N = shape
    A = inputs.uniform(301, (M, K))
    B = inputs.uniform(302, (K, N))
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_gemm_f16_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 1, M, K, N) == 0
    assert api.sync_status() == 0
    exact, mag = _f16_reference(A, B)
    _check_f16(dC.cpu().numpy(), exact, mag, K)


def test_f16_small_integers_are_exact(gpu_lib):
    """Integers whose products and sums fit f16 / f32 exactly: the half-precision product has
    no rounding anywhere, so the result equals the integer product."""
    rng = np.random.default_rng(11)
    A = rng.integers(-4, 5, (200, 96)).astype(np.float64)
    B = rng.integers(-4, 5, (96, 144)).astype(np.float64)
    C = eb.matmul_dispatch(A, B, dtype=2)
    assert np.array_equal(C, A @ B)


def test_f16_dtype_dispatch_and_batch(gpu_lib):
    """dtype 2 / 3 on the dispatchers take the half-precision path whatever the size; the
    batched dispatcher multiplies all matrices in one launch."""
    A = inputs.uniform(303, (40, 50))
    B = inputs.uniform(304, (50, 30))
    for dtype in (2, 3):
        C = eb.matmul_dispatch(A, B, dtype=dtype)
        exact, mag = _f16_reference(A, B)
        _check_f16(C, exact, mag, 50)
    batch = 5
    a = inputs.uniform(305, (batch, 70, 90))
    b = inputs.uniform(306, (batch, 90, 33))
    launches0 = api.launch_count()
    c = eb.batch_matmul_dispatch(a, b, dtype=2)
    assert api.launch_count() - launches0 == 2 * batch + 1  # conversions per matrix, one product launch
    for i in range(batch):
        exact, mag = _f16_reference(a[i], b[i])
        _check_f16(c[i], exact, mag, 90)


def test_f32_buffers(gpu_lib):
    """eshkol_gpu_matmul_f32 on f32 device buffers: correctly rounded f32 of the exact-tier product."""
    import ctypes
    import torch
    M, K, N = 150, 333, 90
    A = inputs.uniform(307, (M, K)).astype(np.float32)
    B = inputs.uniform(308, (K, N)).astype(np.float32)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.zeros((M, N), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_gemm_f32_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, K, N) == 0
    assert api.sync_status() == 0
    want = ol.oz2_exact(A.astype(np.float64), B.astype(np.float64), 52).astype(np.float32)
    assert np.array_equal(dC.cpu().numpy(), want)
    # and within an f32 GEMM's own error of the f64 product
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert np.all(np.abs(dC.cpu().numpy() - ref) <= 2.0 ** -23 * (np.abs(A).astype(np.float64) @ np.abs(B)))


def test_copy_engine_entry_points_on_one_gpu(gpu_lib):
    """copy_async / copy2d_async / interprocess events, as far as one process can exercise them:
    the copies land, a recorded event orders a second stream, the handles have 64 bytes."""
    import torch
    lib = gpu_lib
    src = torch.arange(6 * 1024, dtype=torch.float64, device="cuda").reshape(6, 1024)
    dst = torch.zeros((6, 1024), dtype=torch.float64, device="cuda")
    pan = torch.zeros((6, 256), dtype=torch.float64, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    ev, buf = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    assert lib.eshkol_b200_ipc_event_create(ctypes.byref(ev), buf) == 0 and len(buf.raw) == 64
    assert lib.eshkol_b200_copy_async(dst.data_ptr(), src.data_ptr(), src.numel() * 8, s1.cuda_stream) == 0
    assert lib.eshkol_b200_event_record(ev, s1.cuda_stream) == 0
    assert lib.eshkol_b200_event_wait(ev, s2.cuda_stream) == 0
    # columns 512..767 of the copy, as a contiguous panel, on the stream that waited
    assert lib.eshkol_b200_copy2d_async(pan.data_ptr(), 256 * 8, dst.data_ptr() + 512 * 8, 1024 * 8,
                                        256 * 8, 6, s2.cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, src) and torch.equal(pan, src[:, 512:768])
    assert lib.eshkol_b200_event_destroy(ev) == 0
    blk = ctypes.c_void_p()
    assert lib.eshkol_b200_mem_alloc(0, 1 << 20, ctypes.byref(blk)) == 0
    hbuf = ctypes.create_string_buffer(64)
    assert lib.eshkol_b200_ipc_export_mem(blk, hbuf) == 0 and any(hbuf.raw)
    lib.eshkol_b200_mem_free(0, blk)
    assert lib.eshkol_b200_enable_peer_access(torch.cuda.current_device()) == 0  # own device: nothing to do


def _conv_backward_reference(G, X, Wt, sH, sW):
    """The loops of the reference's two backward kernels (lib/backend/gpu/gpu_cuda_kernels.cu:413-486),
    in longdouble so that the comparison measures the GPU result, not this restatement."""
    G, X, Wt = (np.asarray(t, dtype=np.longdouble) for t in (G, X, Wt))
    batch, C_out, oH, oW = G.shape
    _, C_in, H, W = X.shape
    _, _, kH, kW = Wt.shape
    gX = np.zeros((batch, C_in, H, W), dtype=np.longdouble)
    gK = np.zeros((C_out, C_in, kH, kW), dtype=np.longdouble)
    for kh in range(kH):
        for kw in range(kW):
            xs = X[:, :, kh:kh + (oH - 1) * sH + 1:sH, kw:kw + (oW - 1) * sW + 1:sW]  # b, ci, oh, ow
            gK[:, :, kh, kw] = np.einsum("bohw,bihw->oi", G, xs)
            gX[:, :, kh:kh + (oH - 1) * sH + 1:sH, kw:kw + (oW - 1) * sW + 1:sW] += np.einsum(
                "bohw,oi->bihw", G, Wt[:, :, kh, kw])
    return gX, gK


@pytest.mark.parametrize("cfg", [(2, 3, 9, 10, 4, 3, 3, 1, 1), (3, 5, 12, 11, 6, 3, 2, 2, 1), (1, 2, 8, 8, 3, 1, 1, 2, 2)])
def test_conv2d_backward_both_gradients(gpu_lib, cfg):
    import torch
    batch, C_in, H, W, C_out, kH, kW, sH, sW = cfg
    oH, oW = (H - kH) // sH + 1, (W - kW) // sW + 1
    X = inputs.uniform(401, (batch, C_in, H, W))
    Wt = inputs.uniform(402, (C_out, C_in, kH, kW))
    G = inputs.normal(403, (batch, C_out, oH, oW))
    dX, dW, dG = (torch.from_numpy(t).cuda() for t in (X, Wt, G))
    gX = torch.full_like(dX, float("nan"))
    gK = torch.full_like(dW, float("nan"))
    torch.cuda.synchronize()
    opts = api.make_opts(eb.TIER_OZAKI2, 16)
    dims = (H, W, kH, kW, oH, oW, sH, sW, C_in, C_out, batch)
    assert gpu_lib.eshkol_b200_conv2d_backward_kernel_f64_device(dG.data_ptr(), dX.data_ptr(), gK.data_ptr(),
                                                                *dims, ctypes.byref(opts)) == 0
    assert gpu_lib.eshkol_b200_conv2d_backward_input_f64_device(dG.data_ptr(), dW.data_ptr(), gX.data_ptr(),
                                                               *dims, ctypes.byref(opts)) == 0
    assert api.sync_status() == 0
    wantX, wantK = _conv_backward_reference(G, X, Wt, sH, sW)
    # the exact tier's own error: about 2^-25 of the magnitude sum (its CRT weights round); allow 2^-22
    magK = float(np.abs(G).sum()) * float(np.abs(X).max())
    magX = float(np.abs(G).max()) * float(np.abs(Wt).sum())
    assert np.all(np.abs(gK.cpu().numpy() - wantK.astype(np.float64)) <= magK * 2.0 ** -22)
    assert np.all(np.abs(gX.cpu().numpy() - wantX.astype(np.float64)) <= magX * 2.0 ** -22)
    # tight on the typical element: relative error of the whole tensors
    assert normwise(gK.cpu().numpy(), wantK.astype(np.float64)) < 1e-7
    assert normwise(gX.cpu().numpy(), wantX.astype(np.float64)) < 1e-7


@pytest.mark.parametrize("cfg", [(2, 3, 9, 10, 4, 3, 3, 1, 1), (3, 5, 12, 11, 6, 3, 2, 2, 1), (4, 8, 20, 20, 16, 3, 3, 1, 1)])
def test_conv2d_backward_against_the_reference_cuda_kernels(gpu_lib, tmp_path, cfg):
    """Both gradients against the reference's own conv2d_backward_input / _kernel kernels
    (lib/backend/gpu/gpu_cuda_kernels.cu:413-486), compiled from the reference's sources and run on
    this GPU in a process of its own.  The reference adds one product at a time in f64; the GEMMs
    here are exact-tier sums, so the two agree to the reference's own rounding: n terms of half an
    ulp of the running magnitude, plus the exact tier's 2^-25-of-magnitude bound."""
    import os
    import subprocess
    import sys
    import torch
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "oracle", "_ref", "libref_gpu_cuda.so")):
        pytest.skip("reference CUDA backend not built (oracle/Makefile target _ref/libref_gpu_cuda.so)")
    batch, C_in, H, W, C_out, kH, kW, sH, sW = cfg
    out = str(tmp_path / "ref_conv_backward.npz")
    r = subprocess.run([sys.executable, os.path.join(root, "tests", "ref_gpu_runner.py"), "conv-backward",
                        *map(str, cfg), out], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = np.load(out)
    oH, oW = (H - kH) // sH + 1, (W - kW) // sW + 1
    X = inputs.uniform(401, (batch, C_in, H, W))
    Wt = inputs.uniform(402, (C_out, C_in, kH, kW))
    G = inputs.normal(403, (batch, C_out, oH, oW))
    dX, dW, dG = (torch.from_numpy(t).cuda() for t in (X, Wt, G))
    gX = torch.full_like(dX, float("nan"))
    gK = torch.full_like(dW, float("nan"))
    torch.cuda.synchronize()
    opts = api.make_opts(eb.TIER_OZAKI2, 16)
    dims = (H, W, kH, kW, oH, oW, sH, sW, C_in, C_out, batch)
    assert gpu_lib.eshkol_b200_conv2d_backward_kernel_f64_device(dG.data_ptr(), dX.data_ptr(), gK.data_ptr(),
                                                                *dims, ctypes.byref(opts)) == 0
    assert gpu_lib.eshkol_b200_conv2d_backward_input_f64_device(dG.data_ptr(), dW.data_ptr(), gX.data_ptr(),
                                                               *dims, ctypes.byref(opts)) == 0
    assert api.sync_status() == 0
    nK, nX = batch * oH * oW, C_out * kH * kW
    magK = float(np.abs(G).sum()) * float(np.abs(X).max())
    magX = float(np.abs(G).max()) * float(np.abs(Wt).sum())
    assert np.all(np.abs(gK.cpu().numpy() - ref["grad_kernel"]) <= magK * (2.0 ** -22 + nK * 2.0 ** -53))
    assert np.all(np.abs(gX.cpu().numpy() - ref["grad_input"]) <= magX * (2.0 ** -22 + nX * 2.0 ** -53))
    assert normwise(gK.cpu().numpy(), ref["grad_kernel"]) < 1e-7
    assert normwise(gX.cpu().numpy(), ref["grad_input"]) < 1e-7


def test_feed_forward_block(gpu_lib):
    """out = gelu(x W1 + b1) W2 + b2 with the tanh-by-exp GELU of the reference's generated loops
    (lib/backend/tensor_transformer_codegen.cpp:2469-2664), two GEMMs with fused epilogues."""
    import torch
    rows, d_model, d_ff = 70, 96, 200
    x = inputs.normal(501, (rows, d_model))
    W1 = inputs.uniform(502, (d_model, d_ff)) * 0.2
    b1 = inputs.uniform(503, (d_ff,))
    W2 = inputs.uniform(504, (d_ff, d_model)) * 0.2
    b2 = inputs.uniform(505, (d_model,))
    dev = [torch.from_numpy(np.ascontiguousarray(t)).cuda() for t in (x, W1, b1, W2, b2)]
    out = torch.full((rows, d_model), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    opts = api.make_opts(eb.TIER_OZAKI2, 16)
    rc = gpu_lib.eshkol_b200_feed_forward_f64_device(*(t.data_ptr() for t in dev), out.data_ptr(), rows, d_model,
                                                     d_ff, ctypes.byref(opts))
    assert rc == 0 and api.sync_status() == 0
    ld = np.longdouble
    pre = (x.astype(ld) @ W1.astype(ld) + b1.astype(ld)).astype(np.float64)
    u = 0.7978845608028654 * (pre + 0.044715 * (pre * (pre * pre)))
    e = np.exp(2.0 * u)
    hidden = 0.5 * (pre * (1.0 + (e - 1.0) / (e + 1.0)))
    want = (hidden.astype(ld) @ W2.astype(ld) + b2.astype(ld)).astype(np.float64)
    got = out.cpu().numpy()
    assert normwise(got, want) < 1e-7
    # element by element: the exact tier's 2^-25-of-magnitude error through both products
    mag = np.abs(hidden) @ np.abs(W2) + np.abs(b2) + (np.abs(x) @ np.abs(W1)).max() * np.abs(W2).sum(axis=0)
    assert np.all(np.abs(got - want) <= mag * 2.0 ** -21)
    # the fused ReLU / GELU epilogue equals the separate elementwise pass on the same product
    plain = gu.gemm(x, W1)
    fused = gu.gemm(x, W1, activation=2, bias=b1, bias_mode=2)
    t = plain + b1
    uu = 0.7978845608028654 * (t + 0.044715 * (t * (t * t)))
    ee = np.exp(2.0 * uu)
    np.testing.assert_allclose(fused, 0.5 * (t * (1.0 + (ee - 1.0) / (ee + 1.0))), rtol=1e-13, atol=1e-15)


def _run_reference_gpu(kernel, T, M, K, N, sa, sb, tmp_path):
    """The reference's own CUDA backend in a process of its own (tests/ref_gpu_runner.py)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if not os.path.exists(os.path.join(root, "oracle", "_ref", "libref_gpu_cuda.so")):
        pytest.skip("reference CUDA backend not built (oracle/Makefile target _ref/libref_gpu_cuda.so)")
    out = str(tmp_path / f"ref_{kernel}_{T}.npy")
    r = subprocess.run([sys.executable, os.path.join(root, "tests", "ref_gpu_runner.py"), kernel, str(T), str(M),
                        str(K), str(N), str(sa), str(sb), out], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return np.load(out)


@pytest.mark.parametrize("T", [4, 6])
def test_slice_tier_against_the_reference_cuda_backend(gpu_lib, tmp_path, T):
    """The INT8 slice tier of the reference itself (cuda_matmul_ozaki_int8_f64,
    lib/backend/gpu/gpu_memory_cuda.cpp:339-452, compiled from the reference's sources and run on
    this GPU) against this library's Ozaki-I tier on the same operands: integer-exact products and
    the same reconstruction order on both sides, so the bits agree.  1024^3 is the smallest shape
    the reference sends to that tier (gpu_memory_cuda.cpp:463)."""
    M = K = N = 1024
    ref = _run_reference_gpu("ozaki-int8", T, M, K, N, 601, 602, tmp_path)
    A = inputs.uniform(601, (M, K))
    B = inputs.uniform(602, (K, N))
    got = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=T)
    assert gu.same_bits(got, ref)
    assert gu.same_bits(ol.oz1(A, B, T), ref)  # and pins the CPU restatement


def test_exact_tier_against_the_reference_cublas_dgemm(gpu_lib, tmp_path):
    """cublasDgemm through the reference's backend (its default f64 path on CUDA) against the exact
    tier: both within rounding of the true product; the exact tier's error is the smaller one on
    most elements and never beyond its 2^-25-of-magnitude bound."""
    M, K, N = 1024, 1024, 1024
    ref = _run_reference_gpu("dgemm", 0, M, K, N, 603, 604, tmp_path)
    A = inputs.uniform(603, (M, K))
    B = inputs.uniform(604, (K, N))
    got = gu.gemm(A, B)
    mag = np.abs(A) @ np.abs(B)
    assert np.all(np.abs(got - ref) <= mag * 2.0 ** -22)
    assert normwise(got, ref) < 1e-8


@pytest.mark.parametrize("T", [4, 6])
def test_slice_tier_against_committed_reference_rows(gpu_lib, T):
    """The committed rows of the reference's CUDA slice tier (tests/golden/reference_cuda_1024.npz,
    made on a B200 by tests/golden/make_golden.py): this library's tier reproduces them bit for bit,
    whether or not the reference library is present on this machine."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cuda_1024.npz"))
    n, rows = int(g["n"]), g["rows"]
    A = inputs.uniform(int(g["seed_a"]), (n, n))
    B = inputs.uniform(int(g["seed_b"]), (n, n))
    got = gu.gemm(A, B, tier=eb.TIER_OZAKI1, param=T)
    assert gu.same_bits(got[rows], g[f"slice_T{T}"])
