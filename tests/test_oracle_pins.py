"""The CPU oracle against every fixture the reference holds for this path."""
import math

import numpy as np
import pytest

import fixtures as fx
import oracle_lib as ol


def test_certificate_25_cells_equal_exact_integer_dot():
    a, b = fx.certificate_operands()
    A, B = a.astype(np.float64), b.astype(np.float64)
    E = ol.oz2_E(A, B)
    assert E == 52
    for flags in (0, ol.EXPFIELD, ol.UNFUSED):
        C = ol.oz2_exact(A, B, E, flags=flags)
        for i in fx.CERT_POINTS:
            for j in fx.CERT_POINTS:
                assert C[i, j] == float(fx.exact_dot(a, b, i, j)), (flags, i, j)


def test_certificate_rows_within_one_ulp_of_exact():
    # outside exact ties the result is the correctly rounded integer dot product
    a, b = fx.certificate_operands()
    rows = [0, 77, 511]
    C = ol.oz2_exact(a[rows].astype(np.float64), b.astype(np.float64), 52)
    for r, i in enumerate(rows):
        for j in range(0, 512, 7):
            ref = fx.exact_dot(a, b, i, j)
            assert abs(C[r, j] - float(ref)) <= math.ulp(float(ref))


@pytest.mark.parametrize("regime", [0, 1, 2, 3])
@pytest.mark.parametrize("n", [512, 1024])
def test_regimes_within_1e9_of_naive_dot(regime, n):
    A, B = fx.regime_operands(regime, n)
    E = ol.oz2_E(A, B)
    rows = fx.probe_grid(n)
    C = ol.oz2_exact(A[rows], np.ascontiguousarray(B[:, rows]), E)
    worst = 0.0
    for a_i, i in enumerate(rows):
        for b_j, j in enumerate(rows):
            worst = max(worst, fx.rel_err(C[a_i, b_j], fx.naive_dot(A, B, i, j)))
    assert worst < 1e-9


def test_ones_4096_is_exactly_4096():
    # tests/gpu/gpu_scale_correctness_test.esk: ones(4096)^2 == 4096 everywhere
    A = np.ones((3, 4096))
    B = np.ones((4096, 5))
    assert np.all(ol.oz2_exact(A, B, 52) == 4096.0)
    idx = np.arange(4, dtype=np.float64)[:, None] * np.ones((1, 4096))
    assert np.array_equal(ol.oz2_exact(idx, B, 52), np.arange(4.0)[:, None] * 4096.0 * np.ones((1, 5)))


def test_small_integer_products():
    # tests/gpu/matmul_correctness_test.esk: 2x2 and 2x3 * 3x2 integer answers, A*I = A
    assert np.array_equal(ol.oz2_exact([[1, 2], [3, 4]], [[5, 6], [7, 8]], 52), [[19, 22], [43, 50]])
    assert np.array_equal(ol.oz2_exact([[1, 2, 3], [4, 5, 6]], [[7, 8], [9, 10], [11, 12]], 52),
                          [[58, 64], [139, 154]])
    A = np.arange(64.0).reshape(8, 8) - 17.0
    assert np.array_equal(ol.oz2_exact(A, np.eye(8), 52), A)


def test_subset_rows_and_columns_reproduce_full_bits():
    rng = np.random.default_rng(5)
    A = rng.standard_normal((40, 1100))
    B = rng.standard_normal((1100, 30))
    E = ol.oz2_E(A, B)
    full = ol.oz2_exact(A, B, E)
    rows, cols = [3, 17, 39], [0, 29]
    sub = ol.oz2_exact(A[rows], np.ascontiguousarray(B[:, cols]), E)
    assert np.array_equal(sub, full[np.ix_(rows, cols)])


def test_floor_log2_model_matches_libm():
    vals = []
    for t in list(range(-1074, 1024, 37)) + [-4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 8, 16, 17, 1023]:
        p = math.ldexp(1.0, t) if t > -1074 else 5e-324
        x = p
        for _ in range(6):  # the power of two and the doubles just below / above it
            vals.append(x)
            x = np.nextafter(x, 0.0)
        x = p
        for _ in range(3):
            x = np.nextafter(x, np.inf)
            if np.isfinite(x):
                vals.append(x)
    rng = np.random.default_rng(1)
    vals += list(np.ldexp(rng.uniform(0.5, 1.0, 2000), rng.integers(-1000, 1000, 2000)))
    for x in vals:
        x = float(x)
        if x <= 0.0 or not math.isfinite(x):
            continue
        assert ol.floor_log2_model(x) == math.floor(math.log2(x)), x.hex()


def test_libm_and_model_variants_agree_on_ordinary_data():
    rng = np.random.default_rng(2)
    A = rng.standard_normal((16, 300)) * np.exp2(rng.integers(-30, 30, (16, 1)))
    B = rng.standard_normal((300, 12))
    assert np.array_equal(ol.oz2_exact(A, B, 52, flags=0), ol.oz2_exact(A, B, 52, flags=ol.EXPFIELD))


@pytest.mark.parametrize("case", range(len(fx.CONV_CASES)))
def test_conv_known_answers(case):
    ishape, ival, kshape, kval, stride, pad, oshape, oval = fx.CONV_CASES[case]
    ishape, kshape = fx.conv_promote(ishape, kshape)  # the 2-D form reaches the kernel as NCHW with one plane
    inp = np.array(ival, dtype=np.float64).reshape(ishape)
    ker = np.array(kval, dtype=np.float64).reshape(kshape)
    want = np.array(oval, dtype=np.float64).reshape(-1)
    got = fx.conv2d_numpy(inp, ker, stride, pad)
    assert got.size == int(np.prod(oshape))
    want = want.reshape(got.shape)
    assert np.allclose(got, want, rtol=0, atol=1e-9)
    ref = ol.ref_conv2d(inp, ker, stride, pad)
    if ref is not None:  # the reference's own kernel, when it was compiled here
        assert np.array_equal(ref, got)
    # the lowering: exact-tier GEMM of the kernel matrix with the im2col operand
    col, oH, oW = fx.im2col(inp, kshape[2], kshape[3], stride, pad)
    low = ol.oz2_exact(ker.reshape(kshape[0], -1), col, 52)
    low = low.reshape(kshape[0], ishape[0], oH, oW).transpose(1, 0, 2, 3)
    assert np.allclose(low, want, rtol=0, atol=1e-9)


def test_reference_cpu_matmul_agrees_with_oracle_to_rounding():
    rng = np.random.default_rng(3)
    A = rng.uniform(-1, 1, (96, 200))
    B = rng.uniform(-1, 1, (200, 80))
    ref = ol.ref_matmul(A, B)
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    got = ol.oz2_exact(A, B)
    err = np.abs(got - ref)
    # Almost every cell is the correctly rounded product of the scaled operands.  A
    # small fraction carries a relative error near 2^-25: the reference's split CRT
    # weights do not share one exponent, so its S1 accumulation can round
    # (lib/backend/gpu/gpu_memory.mm:323-333, 2637).  The oracle restates that
    # arithmetic as it is, so the same cells are off here.
    assert np.median(err) < 1e-14
    assert np.mean(err < 1e-12) > 0.98
    assert np.max(err / np.maximum(np.abs(ref), 1e-9)) < 1e-6


def test_reference_backward_is_two_products_of_transposes():
    """eshkol_matmul_backward_f64 (blas_backend.cpp:924) compiled from the reference: grad_A and
    grad_B equal G B^T and A^T G; the oracle's exact products of the transposed operands agree
    with it to the tier's accuracy.  This is what the GPU backward entry is compared with."""
    rng = np.random.default_rng(5)
    G, A, B = rng.standard_normal((37, 29)), rng.standard_normal((37, 41)), rng.standard_normal((41, 29))
    ref = ol.ref_matmul_backward(G, A, B)
    if ref is None:
        pytest.skip("reference CPU library not built")
    gA, gB = ref
    np.testing.assert_allclose(gA, G @ B.T, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(gB, A.T @ G, rtol=1e-12, atol=1e-12)
    # the exact tier's own error (its split CRT weights round in about 0.7 % of the cells, near
    # 2^-25 of the row-by-column magnitude) bounds the agreement, as for the forward product
    np.testing.assert_allclose(ol.oz2_exact(G, np.ascontiguousarray(B.T), 52), gA, rtol=1e-6, atol=5e-6)
    np.testing.assert_allclose(ol.oz2_exact(np.ascontiguousarray(A.T), G, 52), gB, rtol=1e-6, atol=5e-6)


def _golden_reference_cuda():
    import os
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_cuda_1024.npz")
    return np.load(path)


def test_slice_tier_restatement_matches_the_reference_cuda_backend_bits():
    """tests/golden/reference_cuda_1024.npz holds rows of 1024^3 products computed by the reference's
    own CUDA backend on a B200 (tests/golden/make_golden.py).  Its INT8 slice tier is integer-exact
    with a fixed reconstruction order, so the CPU restatement must reproduce those rows bit for bit."""
    from eshkol_b200 import inputs
    g = _golden_reference_cuda()
    n, rows = int(g["n"]), g["rows"]
    A = inputs.uniform(int(g["seed_a"]), (n, n))[rows]
    B = inputs.uniform(int(g["seed_b"]), (n, n))
    for T in (4, 6):
        got = ol.oz1(A, B, T)
        want = g[f"slice_T{T}"]
        assert np.array_equal(got.view(np.uint64), want.view(np.uint64))


def test_exact_tier_restatement_within_its_bound_of_the_reference_cublas_dgemm():
    """The same file's cublasDgemm rows: the exact tier's restatement agrees with them to the exact
    tier's own error (about 2^-25 of sum |a||b| in 0.7 % of the cells) plus DGEMM's rounding."""
    from eshkol_b200 import inputs
    g = _golden_reference_cuda()
    n, rows = int(g["n"]), g["rows"]
    A = inputs.uniform(int(g["seed_a"]), (n, n))[rows]
    B = inputs.uniform(int(g["seed_b"]), (n, n))
    got = ol.oz2_exact(A, B, 52)
    mag = np.abs(A) @ np.abs(B)
    assert np.all(np.abs(got - g["dgemm"]) <= mag * 2.0 ** -22)
