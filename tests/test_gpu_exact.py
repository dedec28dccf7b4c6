"""Exact tier on the GPU against the CPU oracle, stage by stage and end to end (bit-exact)."""
import numpy as np
import pytest

import eshkol_b200 as eb
from eshkol_b200 import api, inputs
import fixtures as fx
import gpu_util as gu
import oracle_lib as ol

pytestmark = pytest.mark.gpu

MODULI = (256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193)


def check_stages(A, B, simt):
    """scales, residue planes, product residues and C of one GEMM, each against the oracle"""
    M, K = A.shape
    N = B.shape[1]
    C = gu.gemm(A, B, simt=simt)
    Cref, d = ol.oz2_exact(A, B, 52, debug=True)
    mu, _ = api.debug_fetch(0)
    nu, _ = api.debug_fetch(1)
    assert np.array_equal(mu[0, :M], d["mu"])
    assert np.array_equal(nu[0, :N], d["nu"])
    # modulus 256: representative in [-128, 128] with the reference's tie rule, carried as
    # the int8 byte plus two flag bit-planes (+128, odd)
    a0, _ = api.debug_fetch(2)
    ra = d["Ares"][0].astype(np.int32)
    assert np.array_equal(gu.decode_plane0(a0, K).astype(np.int32), ((ra + 128) % 256) - 128)
    assert np.array_equal(gu.decode_flags(api.debug_fetch(8)[0], K), (ra == 128).astype(np.int32))
    assert np.array_equal(gu.decode_flags(api.debug_fetch(9)[0], K), ra & 1)
    b0, _ = api.debug_fetch(4)
    rb = d["Bres"][0].astype(np.int32).T
    assert np.array_equal(gu.decode_plane0(b0, K).astype(np.int32), ((rb + 128) % 256) - 128)
    assert np.array_equal(gu.decode_flags(api.debug_fetch(10)[0], K), (rb == 128).astype(np.int32))
    assert np.array_equal(gu.decode_flags(api.debug_fetch(11)[0], K), rb & 1)
    # odd moduli: an int8 representative of the same class as the reference's value
    # (within half a modulus plus one of zero, so that K products still fit int32)
    for l in (1, 2, 8, 15):
        p = MODULI[l]
        ap, _ = api.debug_fetch(3, l - 1)
        got = ap[:, :K].astype(np.int32)
        assert np.abs(got).max() <= (p - 1) // 2 + 1
        assert not ((got - d["Ares"][l].astype(np.int32)) % p).any()
        assert not ap[:, K:].any()
        bp, _ = api.debug_fetch(5, l - 1)
        got = bp[:, :K].astype(np.int32)
        assert np.abs(got).max() <= (p - 1) // 2 + 1
        assert not ((got - d["Bres"][l].astype(np.int32).T) % p).any()
    # residues of the products
    w0, _ = api.debug_fetch(6)
    flip, _ = api.debug_fetch(12)
    fl = ((flip.view(np.uint32)[:, np.arange(N) // 32] >> (np.arange(N) % 32).astype(np.uint32)) & 1).astype(np.int64)
    x = (w0[:M, :N].astype(np.int64) + 256 * fl[:M]) % 512
    got0 = np.where(x == 128, 128, ((x + 128) % 256) - 128)
    assert np.array_equal(got0, d["W"][0].astype(np.int64))
    for l in range(1, 16):
        wl, _ = api.debug_fetch(7, l - 1)
        assert np.array_equal(wl[:M, :N].astype(np.int32), d["W"][l].astype(np.int32)), l
    assert gu.same_bits(C, Cref)


@pytest.mark.parametrize("simt", [True, False], ids=["cuda-core-products", "tcgen05-products"])
def test_stages_small_ragged(gpu_lib, simt):
    A = inputs.uniform(1, (200, 1100))
    B = inputs.uniform(2, (1100, 300))
    check_stages(A, B, simt)


@pytest.mark.parametrize("simt", [True, False], ids=["cuda-core-products", "tcgen05-products"])
def test_stages_full53_hits_the_mod256_tie_path(gpu_lib, simt):
    A = inputs.full53(1, (256, 2100))
    B = inputs.full53(2, (2100, 256))
    d = ol.oz2_exact(A, B, 52, debug=True)[1]
    assert (np.abs(d["Ares"][0]) == 128).any() and (np.abs(d["W"][0]) == 128).any()
    check_stages(A, B, simt)


@pytest.mark.parametrize("shape", [(1, 1, 1), (1, 7, 1), (3, 1008, 5), (129, 1009, 257), (128, 2016, 256),
                                   (130, 127, 513), (257, 4000, 100)])
def test_bit_exact_odd_shapes(gpu_lib, shape):
    M, K, N = shape
    A = inputs.full53(11, (M, K))
    B = inputs.wide(12, (K, N), span=9, lo=-4)
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))


def test_c1_512_cubed_bit_exact(gpu_lib):
    A = inputs.uniform(1, (512, 512))
    B = inputs.uniform(2, (512, 512))
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))


def test_tile_n_128_variant_bit_exact(gpu_lib):
    A = inputs.full53(5, (300, 1500))
    B = inputs.full53(6, (1500, 400))
    assert gu.same_bits(gu.gemm(A, B, tile_n=128), ol.oz2_exact(A, B, 52))


def test_certificate_all_cells_match_oracle_and_25_match_exact_ints(gpu_lib):
    a, b = fx.certificate_operands()
    A, B = a.astype(np.float64), b.astype(np.float64)
    C = gu.gemm(A, B)
    for i in fx.CERT_POINTS:
        for j in fx.CERT_POINTS:
            assert C[i, j] == float(fx.exact_dot(a, b, i, j))
    assert gu.same_bits(C, ol.oz2_exact(A, B, 52))


@pytest.mark.parametrize("regime", [0, 1, 2, 3])
def test_regimes_gate_and_bits(gpu_lib, regime):
    n = 512
    A, B = fx.regime_operands(regime, n)
    C = gu.gemm(A, B)
    rows = fx.probe_grid(n)
    worst = max(fx.rel_err(C[i, j], fx.naive_dot(A, B, i, j)) for i in rows for j in rows)
    assert worst < 1e-9
    assert gu.same_bits(C, ol.oz2_exact(A, B, 52))


def test_zero_rows_columns_and_signed_zero(gpu_lib):
    A = inputs.uniform(3, (140, 300))
    B = inputs.uniform(4, (300, 270))
    A[5, :] = 0.0
    A[130, :] = -0.0
    B[:, 0] = 0.0
    B[:, 269] = 0.0
    C = gu.gemm(A, B)
    assert gu.same_bits(C, ol.oz2_exact(A, B, 52))
    assert not C[5].any() and not C[:, 0].any()


def test_fewer_moduli_follow_the_reference_exponent_rule(gpu_lib):
    A = inputs.uniform(7, (150, 700))
    B = inputs.uniform(8, (700, 260))
    for n_mod in (8, 12, 15):
        E = ol.oz2_E(A, B, n_mod)
        assert E < 52 or n_mod == 15
        assert gu.same_bits(gu.gemm(A, B, param=n_mod), ol.oz2_exact(A, B, E, n_mod=n_mod))


def test_ones_and_identity(gpu_lib):
    # tests/gpu/gpu_scale_correctness_test.esk, tests/gpu/cuda_host_sync_regression_test.esk
    n = 1024
    assert np.all(gu.gemm(np.ones((n, n)), np.ones((n, n))) == float(n))
    A = inputs.uniform(9, (50, 50))
    assert gu.same_bits(gu.gemm(A, np.eye(50)), ol.oz2_exact(A, np.eye(50), 52))


def test_fused_relu_and_bias(gpu_lib):
    A = inputs.uniform(1, (130, 400))
    B = inputs.uniform(2, (400, 300))
    ref = ol.oz2_exact(A, B, 52)
    got = gu.gemm(A, B, activation=1)
    assert gu.same_bits(got, np.where(ref > 0.0, ref, 0.0))
    bias = inputs.uniform(3, (130,))
    got = gu.gemm(A, B, activation=1, bias=bias, bias_mode=1)
    want = ref + bias[:, None]
    assert gu.same_bits(got, np.where(want > 0.0, want, 0.0))


def test_c2_4096_wide_exponent_sampled_rows_and_columns(gpu_lib):
    n = 4096
    A = inputs.wide(1, (n, n))
    B = inputs.wide(2, (n, n))
    C = gu.gemm(A, B)
    rng = np.random.default_rng(0)
    rows = np.sort(rng.choice(n, 24, replace=False))
    cols = np.sort(rng.choice(n, 24, replace=False))
    assert gu.same_bits(C[rows], ol.oz2_exact(A[rows], B, 52))
    assert gu.same_bits(C[:, cols], ol.oz2_exact(A, np.ascontiguousarray(B[:, cols]), 52))


def test_prepared_b_row_blocks_have_the_bits_of_the_one_shot_product(gpu_lib):
    import ctypes
    import torch
    A = inputs.full53(31, (700, 1300))
    B = inputs.full53(32, (1300, 520))
    want = gu.gemm(A, B)
    dA = torch.from_numpy(A).cuda()
    dB = torch.from_numpy(B).cuda()
    dC = torch.full((700, 520), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_prepare_b_f64_device(dB.data_ptr(), 1300, 520) == 0
    dB.zero_()  # the prepared planes, not B, are what the products read
    for r0, rows in ((0, 300), (300, 1), (301, 399)):
        assert gpu_lib.eshkol_b200_gemm_prepared_f64_device(dA[r0:].data_ptr(), dC[r0:].data_ptr(), rows, None) == 0
    assert api.sync_status() == 0
    assert gu.same_bits(dC.cpu().numpy(), want)
    assert gu.same_bits(want, ol.oz2_exact(A, B, 52))


def test_host_pipeline_over_several_row_blocks(gpu_lib):
    # eshkol_matmul_dispatch on host arrays: 1024-row blocks, three streams
    A = inputs.uniform(41, (2500, 640))
    B = inputs.wide(42, (640, 384), span=9, lo=-4)
    gpu_lib.eshkol_gpu_set_threshold(1)
    try:
        C = eb.matmul_dispatch(A, B)
        C2 = eb.matmul_dispatch(A, B)
    finally:
        gpu_lib.eshkol_gpu_set_threshold(100000)
    want = gu.gemm(A, B)
    assert gu.same_bits(C, want) and gu.same_bits(C2, want)
    rows = [0, 1023, 1024, 2047, 2048, 2499]
    assert gu.same_bits(C[rows], ol.oz2_exact(A[rows], B, 52))


def test_operands_at_the_top_of_the_53_bit_range(gpu_lib):
    # scaled integers close to 2^53: the quotient x/p is least accurate there and the
    # residue representatives reach their widest range
    rng = np.random.default_rng(7)
    A = np.ldexp(1.0 - rng.integers(0, 4096, (130, 900)) * 2.0 ** -53, 0) * rng.choice([-1.0, 1.0], (130, 900))
    B = np.ldexp(1.0 - rng.integers(0, 4096, (900, 270)) * 2.0 ** -53, 3) * rng.choice([-1.0, 1.0], (900, 270))
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))
    assert gu.same_bits(gu.gemm(A, B, simt=True), ol.oz2_exact(A, B, 52))


def test_prepared_a_times_column_panels_of_b(gpu_lib):
    import ctypes
    import torch
    A = inputs.full53(51, (333, 1100))
    B = inputs.full53(52, (1100, 768))
    want = gu.gemm(A, B)
    dA = torch.from_numpy(A).cuda()
    dC = torch.full((333, 768), float("nan"), dtype=torch.float64, device="cuda")
    panels = [torch.from_numpy(np.ascontiguousarray(B[:, c0:c0 + 256])).cuda() for c0 in (0, 256, 512)]
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_prepare_a_f64_device(dA.data_ptr(), 333, 1100, 256) == 0
    for p, dB in enumerate(panels):
        assert gpu_lib.eshkol_b200_prepare_b_f64_device(dB.data_ptr(), 1100, 256) == 0
        opts = api.make_opts(ldc=768)  # each panel lands in its columns of the wide C
        assert gpu_lib.eshkol_b200_multiply_prepared_f64_device(dC[:, 256 * p:].data_ptr(), ctypes.byref(opts)) == 0
    assert api.sync_status() == 0
    assert gu.same_bits(dC.cpu().numpy(), want)
    # a result wider than the room reserved with A is refused, not silently moved
    wide = torch.zeros((1100, 1024), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    assert gpu_lib.eshkol_b200_prepare_b_f64_device(wide.data_ptr(), 1100, 1024) == 0
    big = torch.zeros((333, 1024), dtype=torch.float64, device="cuda")
    rc = gpu_lib.eshkol_b200_multiply_prepared_f64_device(big.data_ptr(), None)
    assert rc in (0, -1)  # 0 only if the workspace already held enough room
    assert api.sync_status() == 0


@pytest.mark.parametrize("shape", [(256, 1024, 256), (300, 1100, 520), (1, 130, 1), (513, 4000, 300)])
def test_two_sm_products_kernel_bit_exact(gpu_lib, shape):
    M, K, N = shape
    A = inputs.full53(61, (M, K))
    B = inputs.full53(62, (K, N))
    gpu_lib.eshkol_b200_set_pair_gemm(1)
    try:
        got = gu.gemm(A, B)
    finally:
        gpu_lib.eshkol_b200_set_pair_gemm(0)
    assert gu.same_bits(got, ol.oz2_exact(A, B, 52))


@pytest.mark.parametrize("shape,band", [((700, 600, 300), 256), ((1030, 2100, 520), 512), ((512, 130, 70), 256)])
def test_row_band_pipeline_bit_exact(gpu_lib, shape, band):
    """Bands of rows on three streams (split / products / reconstruction overlapped) give the
    bits of the serial product and of the oracle, with a ragged last band."""
    M, K, N = shape
    A = inputs.full53(71, (M, K))
    B = inputs.full53(72, (K, N))
    bias = np.linspace(-1.0, 1.0, M)
    gpu_lib.eshkol_b200_set_row_bands(0)
    serial = gu.gemm(A, B)
    serial_b = gu.gemm(A, B, activation=1, bias=bias, bias_mode=1)
    gpu_lib.eshkol_b200_set_row_bands(band)
    try:
        first = gu.gemm(A, B)
        second = gu.gemm(A, B)  # the slots and events are reused
        banded_b = gu.gemm(A, B, activation=1, bias=bias, bias_mode=1)
    finally:
        gpu_lib.eshkol_b200_set_row_bands(0)
    assert gu.same_bits(first, serial) and gu.same_bits(second, serial)
    assert gu.same_bits(banded_b, serial_b)
    assert gu.same_bits(first, ol.oz2_exact(A, B, 52))


def test_row_band_pipeline_stage_times(gpu_lib):
    """Stage times under the band pipeline are per-stage sums over the bands."""
    import ctypes
    A = inputs.uniform(73, (1024, 512))
    B = inputs.uniform(74, (512, 512))
    gpu_lib.eshkol_b200_set_row_bands(256)
    gpu_lib.eshkol_b200_set_phase_timing(1)
    try:
        got = gu.gemm(A, B)
        ph = (ctypes.c_float * 8)()
        assert gpu_lib.eshkol_b200_get_phase_times(ph, 8) == 7
        assert int(ph[7]) == 4 and all(ph[i] > 0.0 for i in range(7))
        gpu_lib.eshkol_b200_set_row_bands(0)
        again = gu.gemm(A, B)
        assert gpu_lib.eshkol_b200_get_phase_times(ph, 8) == 7 and int(ph[7]) == 0
    finally:
        gpu_lib.eshkol_b200_set_phase_timing(0)
        gpu_lib.eshkol_b200_set_row_bands(0)
    assert gu.same_bits(got, again)


def _device_gemm(dA, dB):
    import torch
    M, K = dA.shape
    N = dB.shape[1]
    dC = torch.full((M, N), float("nan"), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    api.gemm_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, K, N, api.make_opts(eb.TIER_OZAKI2, 16))
    assert api.sync_status() == 0
    return dC


def test_c3_8192_cubed_normal_64_rows_and_64_columns(gpu_lib):
    """The benchmarked single-GPU configuration itself: 8192^3, standard-normal operands, exact
    tier.  64 random full rows and 64 random full columns of the result, bit for bit against the
    oracle (rows and columns of the exact tier are independent given E = 52).  The operands are
    generated on the device and the oracle gets the very same bits copied back."""
    import torch
    n = 8192
    ol.set_threads(len(__import__("os").sched_getaffinity(0)))
    dA = inputs.normal(1, (n, n), device="cuda")
    dB = inputs.normal(2, (n, n), device="cuda")
    dC = _device_gemm(dA, dB)
    g = torch.Generator().manual_seed(83)
    rows = torch.randperm(n, generator=g)[:64].sort().values.cuda()
    cols = torch.randperm(n, generator=g)[:64].sort().values.cuda()
    B_host = dB.cpu().numpy()
    want = ol.oz2_exact(dA[rows].cpu().numpy(), B_host, 52)
    assert gu.same_bits(dC[rows].cpu().numpy(), want)
    want = ol.oz2_exact(dA.cpu().numpy(), np.ascontiguousarray(B_host[:, cols.cpu().numpy()]), 52)
    assert gu.same_bits(dC[:, cols].contiguous().cpu().numpy(), want)


def test_sharded_configuration_depth_64_rows(gpu_lib):
    """K = 32768, the depth of the multi-GPU configuration (33 extraction chunks): 64 rows of A
    taken from all over the 32768-row operand of that configuration against 2048 columns, bit for
    bit against the oracle."""
    K = 32768
    ol.set_threads(len(__import__("os").sched_getaffinity(0)))
    picks = [int(x) for x in np.random.default_rng(7).choice(32768, size=64, replace=False)]
    A = np.concatenate([inputs.uniform(1, (1, K), start=r * K) for r in sorted(picks)])
    B = inputs.uniform(2, (K, 2048))
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))


@pytest.mark.parametrize("tier,param", [(eb.TIER_OZAKI2, 16), (eb.TIER_OZAKI1, 5)])
def test_sharded_driver_on_one_device(gpu_lib, tier, param):
    """The row-sharded driver with one rank on the device: several column panels through the
    prepared-operand entry points (exact tier) or whole products per panel (slice tier), every
    hand-off ordered by stream events on the library's own stream.  Same bits as one product."""
    import torch
    from eshkol_b200.sharded import ShardedGemm
    M, K, N = 384, 1500, 1024
    A = torch.from_numpy(inputs.full53(91, (M, K))).cuda()
    B = torch.from_numpy(inputs.full53(92, (K, N))).cuda()
    sg = ShardedGemm(M, K, N, torch.device("cuda", torch.cuda.current_device()), tier=tier, param=param, panels=4)
    for _ in range(2):
        C = sg.step(A, B).clone()
    want = gu.gemm(A.cpu().numpy(), B.cpu().numpy(), tier=tier, param=param)
    assert gu.same_bits(C.cpu().numpy(), want)
    sg.close()


def test_c_sharded_driver_on_one_device(gpu_lib):
    """The multi-GPU schedule as a C host drives it (include/eshkol_b200_multi.h), with one rank:
    shared-memory session, B in the session's buffer, this rank's columns of every panel split
    into the panel's plane buffer, the panel adopted and multiplied, two steps in a row.  Same
    bits as one product.  (With more ranks the same calls run in every process; the benchmark's
    multi-GPU leg goes through this entry point.)"""
    import os
    import torch
    from eshkol_b200.sharded import CShardedGemm
    M, K, N = 384, 1500, 8192  # N / 4 a multiple of 2048: the panels ramp as in the benchmark
    A = torch.from_numpy(inputs.full53(93, (M, K))).cuda()
    B = inputs.full53(94, (K, N))
    sg = CShardedGemm(M, K, N, torch.device("cuda", torch.cuda.current_device()), name=f"/eshkol-b200-test-{os.getpid()}")
    try:
        assert sg.panels > 4 and sum(w for _, w in sg.cols) == N
        buf = sg.source_buffer()
        buf.copy_(torch.from_numpy(B))
        for _ in range(2):
            C = sg.step(A, buf).clone()
        want = gu.gemm(A.cpu().numpy(), B)
        assert gu.same_bits(C.cpu().numpy(), want)
    finally:
        sg.close()


def test_sharded_configuration_depth_sampled_rows(gpu_lib):
    """K = 32768 (33 extraction chunks), the depth of the multi-GPU configuration: a few rows
    of A against 2048 columns of B, bit for bit against the oracle."""
    K = 32768
    A = inputs.uniform(1, (4, K), start=12345 * K)
    B = inputs.uniform(2, (K, 2048))
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))


@pytest.mark.parametrize("K", [131071, 131072, 140001, 262144])
def test_exact_tier_at_and_beyond_the_int32_depth(gpu_lib, K):
    """K = 131071 is the last depth whose int32 accumulation of 128^2-bounded products is exact.
    The reference's modular GEMM has no depth limit (it extracts every 1008 elements,
    lib/backend/gpu/metal_softfloat.h:3966-3969, 4054-4067); beyond that depth the odd-modulus
    accumulators are handed over in parts of 1023 k-blocks and their residues summed.  Bit for bit
    against the oracle up to the last depth whose exponent E is 52 whatever the data."""
    A = inputs.full53(81, (3, K))
    B = inputs.full53(82, (K, 40))
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, 52))


def test_exact_tier_where_the_exponent_depends_on_the_data(gpu_lib):
    """Beyond K = 262144 the exponent E of gpu_memory.mm:2510-2512 falls below 52 and depends on the
    maxima of both operands: the one-shot driver scans both before it scales either."""
    K = 400000
    A = inputs.full53(83, (2, K))
    B = inputs.full53(84, (K, 5))
    E = ol.oz2_E(A, B)
    assert E < 52
    assert gu.same_bits(gu.gemm(A, B), ol.oz2_exact(A, B, E))


def test_a_wait_that_runs_out_ends_the_kernel_and_leaves_the_library_usable(gpu_lib):
    """Every wait inside the products kernel is bounded.  With the limit set to a millisecond and
    the producer told to withhold the first stage's arrival, the kernel's waits run out: it
    returns by itself, the status word says which role gave up, eshkol_b200_sync_status reports
    it once, and the next product is bit-exact again.  Nothing faults and nothing hangs: the
    waits simply end."""
    lib = gpu_lib
    A = inputs.uniform(85, (128, 128))
    B = inputs.uniform(86, (128, 128))
    want = ol.oz2_exact(A, B, 52)
    assert gu.same_bits(gu.gemm(A, B), want)
    import torch
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.zeros((128, 128), dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    lib.eshkol_b200_debug_set_wait_limit_ns(1_000_000)
    lib.eshkol_b200_debug_withhold_arrival(1)
    try:
        api.gemm_device(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 128, 128, 128, api.make_opts(eb.TIER_OZAKI2, 16))
        st = api.sync_status()
        assert st in (1, 2, 3), st
    finally:
        lib.eshkol_b200_debug_set_wait_limit_ns(0)
        lib.eshkol_b200_debug_withhold_arrival(0)
    assert api.sync_status() == 0  # reported once, then clear
    assert gu.same_bits(gu.gemm(A, B), want)


def test_c_host_built_against_the_reference_headers(gpu_lib, tmp_path):
    """tests/c_harness, compiled against the reference's own gpu_memory.h and vm_gpu_dispatch.h
    and linked to this library: eshkol_matmul_dispatch and the VM's vm_gpu_try_matmul on operands
    that are 8- but not 16-byte aligned (arena payloads behind their header) give the oracle's bits."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = os.path.join(root, "oracle", "_ref", "c_harness")
    if not os.path.exists(exe):
        pytest.skip("the harness is built where the reference tree is present (oracle/Makefile)")
    M, K, N = 300, 1100, 200
    r = subprocess.run([exe, "run", str(M), str(K), str(N), str(tmp_path)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    A = inputs.uniform(1, (M, K))
    B = inputs.uniform(2, (K, N))
    want = ol.oz2_exact(A, B, 52)
    for name in ("dispatch.bin", "vm.bin"):
        got = np.fromfile(str(tmp_path / name), dtype=np.float64).reshape(M, N)
        assert gu.same_bits(got, want), name
    # the VM's other try-functions (softmax, transpose, add, reduce) on A through the same library
    from oracle import operators_ref as ops
    load = lambda name, shape: np.fromfile(str(tmp_path / name), dtype=np.float64).reshape(shape)
    assert np.array_equal(load("vm_transpose.bin", (K, M)), A.T)
    assert np.array_equal(load("vm_add.bin", (M, K)), A + A)
    assert np.allclose(load("vm_softmax.bin", (M, K)), ops.softmax(A), rtol=1e-13, atol=0)
    red = load("vm_reduce.bin", (4,))
    assert abs(red[0] - A.sum()) < 1e-9 and red[1] == A.min() and red[2] == A.max()
    assert abs(red[3] - A.mean()) < 1e-14


@pytest.mark.parametrize("shape", [(130, 300, 70), (257, 1100, 129), (64, 64, 64)])
def test_transposed_operands_read_in_place(gpu_lib, shape):
    """trans_a / trans_b: the exact tier reads the transposed storage directly (column scan and
    transposing split for A, row scan and plain split for B); bits of the explicit transposes."""
    M, K, N = shape
    A = inputs.full53(91, (M, K))
    B = inputs.full53(92, (K, N))
    want = ol.oz2_exact(A, B, 52)
    At = np.ascontiguousarray(A.T)
    Bt = np.ascontiguousarray(B.T)
    assert gu.same_bits(gu.gemm(At, B, trans_a=True), want)
    assert gu.same_bits(gu.gemm(A, Bt, trans_b=True), want)
    assert gu.same_bits(gu.gemm(At, Bt, trans_a=True, trans_b=True), want)


@pytest.mark.parametrize("tier,param", [(eb.TIER_OZAKI1, 4), (eb.TIER_OZAKI2_FAST, 12), (eb.TIER_DGEMM, 0),
                                        (eb.TIER_OZAKI2, 9)])
def test_transposed_operands_other_tiers(gpu_lib, tier, param):
    A = inputs.uniform(93, (100, 260))
    B = inputs.uniform(94, (260, 150))
    want = gu.gemm(A, B, tier=tier, param=param)
    got = gu.gemm(np.ascontiguousarray(A.T), np.ascontiguousarray(B.T), tier=tier, param=param,
                  trans_a=True, trans_b=True)
    assert gu.same_bits(got, want)


def test_matmul_backward_both_gradients(gpu_lib):
    """eshkol_gpu_matmul_backward_f64: grad_A = G B^T and grad_B = A^T G with the bits of the exact
    products of the explicitly transposed operands, and the reference's CPU backward to the tier's accuracy."""
    M, K, N = 300, 520, 260
    G = inputs.normal(95, (M, N))
    A = inputs.uniform(96, (M, K))
    B = inputs.wide(97, (K, N), span=9, lo=-4)
    gpu_lib.eshkol_gpu_set_threshold(1)
    try:
        gA, gB = eb.matmul_backward(G, A, B)
    finally:
        gpu_lib.eshkol_gpu_set_threshold(100000)
    assert gu.same_bits(gA, ol.oz2_exact(G, np.ascontiguousarray(B.T), 52))
    assert gu.same_bits(gB, ol.oz2_exact(np.ascontiguousarray(A.T), G, 52))
    ref = ol.ref_matmul_backward(G, A, B)
    if ref is not None:
        # the tier's own error is bounded by about 2^-25 of sum |g||b|; allow 2^-22
        assert np.all(np.abs(gA - ref[0]) <= (np.abs(G) @ np.abs(B.T)) * 2.0 ** -22)
        assert np.all(np.abs(gB - ref[1]) <= (np.abs(A.T) @ np.abs(G)) * 2.0 ** -22)
    # below the element threshold the call declines and the caller keeps its CPU branch
    with pytest.raises(RuntimeError):
        eb.matmul_backward(G[:4, :4], A[:4, :4], np.ascontiguousarray(B[:4, :4]))
