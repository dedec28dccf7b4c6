// Device-level C ABI (include/eshkol_b200_ext.h): stream and workspace ownership,
// TMA tensor maps, and the drivers that chain scan -> split -> tensor-core
// products -> reconstruction for each precision tier.
#include "../../include/eshkol_b200_ext.h"
#include "../../include/eshkol_b200_testing.h"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "b200_internal.h"
#include "b200_ozaki2.h"
#include "b200_tiers.h"

namespace b200 {

// ---------------------------------------------------------------- global state
struct State {
  bool ready = false;
  int device = -1;
  int num_sms = 0;
  int sm_limit = 0;  // > 0: SMs the persistent products kernels may occupy (the rest stay free for a communication library's kernels)
  cudaStream_t stream = nullptr;
  uint8_t* ws = nullptr;
  size_t ws_bytes = 0;
  int* d_status = nullptr;
  unsigned long long launches = 0;
  unsigned long long h2d_bytes = 0, d2h_bytes = 0;  // host <-> device bytes this library has moved
  cudaEvent_t ev_g0 = nullptr, ev_g1 = nullptr;     // around the last eshkol_b200_gemm_f64_device
  bool ev_g_valid = false;
  unsigned long long prep_token = 0;                // bumped whenever a right-hand operand is prepared
  uint8_t* aux = nullptr;  // second scratch block (conv2d im2col operand)
  size_t aux_bytes = 0;
  uint8_t* tbuf = nullptr;  // third scratch block: operands transposed for the tiers that need it
  size_t tbuf_bytes = 0;
  PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
  // optional per-stage timing of the Ozaki-II driver (CUDA events on the stream)
  bool timing = false;
  bool pair_gemm = false;  // odd-moduli products on CTA pairs (tcgen05 cta_group::2)
  // Rings of stage events, one entry per call of the stage: B side {start, scan + scales done,
  // split done}, A side likewise, multiplication {start, modulus 256 + ties done, odd moduli
  // done, reconstruction done}.  n_* count the entries recorded since timing was switched on.
  static constexpr int kEvRing = 256;
  cudaEvent_t ev_b[kEvRing][3] = {}, ev_a[kEvRing][3] = {}, ev_m[kEvRing][4] = {};
  unsigned long long n_evb = 0, n_eva = 0, n_evm = 0;
  cudaEvent_t ev_scratch = nullptr;
  bool ev_made = false, ev_valid = false;
  // prepared right-hand operand of the exact tier (its own allocation)
  uint8_t* bside = nullptr;
  size_t bside_bytes = 0;
  struct Prepared {
    bool valid = false;
    long long K = 0, N = 0, Kp = 0, K0 = 0, Np = 0;
    int n_chunks = 0, last_seg = 0, bn = 256, tiles_n = 0;
    double* bmax = nullptr; int* nu = nullptr; double* sb = nullptr; double* sbi = nullptr;
    int8_t* b0 = nullptr; int8_t* bodd = nullptr; long long bodd_stride = 0;
    uint16_t* b_hi = nullptr; uint16_t* b_odd = nullptr;  // flag bit-planes of the modulus-256 residues
    CUtensorMap mB0, mB1, mB1_half;  // mB1_half: boxes of 128 rows, for the two-SM kernel
    Oz2DeviceConsts consts;
  } prep;
  struct PreparedA {
    bool valid = false;
    long long M = 0, K = 0, Kp = 0, K0 = 0, Mp = 0, a_stride = 0;
    int n_chunks = 0, last_seg = 0, tiles_m = 0;
    size_t end = 0;  // workspace offset behind the A planes, where the product residues start
    double* amax = nullptr; int* mu = nullptr; double* sa = nullptr; double* sai = nullptr;
    GemmJob* jobs = nullptr;
    int8_t* a0 = nullptr; int8_t* aodd = nullptr;
    uint16_t* a_hi = nullptr; uint16_t* a_odd = nullptr;
    CUtensorMap mA0, mA1;
  } prepA;
  GemmJob* d_jobs16 = nullptr;  // job table of the 16 modular products, uploaded once
  // row-band pipeline of the one-shot device product: band r+1 is split while band r is
  // multiplied and band r-1 reconstructed, on three streams over two workspace slots
  bool overlap_prep = false;         // one-shot product: B prepared on a second stream beside A (measured: no gain)
  cudaEvent_t b_pending = nullptr;   // recorded behind that preparation; the multiplication waits for it
  long long band_rows = 0;  // off unless asked for: measured, the overlap slows the power-capped products as much as it hides
  bool lanes_made = false;
  cudaStream_t s_prep = nullptr, s_post = nullptr;
  cudaEvent_t eb_start = nullptr, eb_done = nullptr;
  cudaEvent_t eb_a_ready[2] = {}, eb_g0[2] = {}, eb_g1[2] = {}, eb_w_free[2] = {};
  PreparedA bandA[2];
  static constexpr int kMaxBands = 16, kBandEvents = 10;
  cudaEvent_t ev_band[kMaxBands * kBandEvents] = {};
  bool ev_band_made = false;
  int bands_timed = 0;  // > 0: the last timed product ran as this many bands
  // host pipeline: upload / download streams and their hand-off events
  bool pipe_made = false;
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t e_b_ready = nullptr, e_a_ready[2] = {}, e_a_free[2] = {}, e_c_ready[2] = {}, e_c_free[2] = {};
  // layout of the last Ozaki-II GEMM, for eshkol_b200_debug_fetch
  struct Last {
    bool valid = false;
    long long M = 0, K = 0, N = 0, Kp = 0, K0 = 0, Mp = 0, Np = 0;
    int n_mod = 0, n_chunks = 0, last_seg = 0;
    int* mu = nullptr; int* nu = nullptr;
    int8_t* a0 = nullptr; int8_t* aodd = nullptr; long long aodd_stride = 0;
    int8_t* b0 = nullptr; int8_t* bodd = nullptr; long long bodd_stride = 0;
    int16_t* w0 = nullptr; int8_t* wodd = nullptr; long long wodd_stride = 0;
    uint16_t* a_hi = nullptr; uint16_t* a_odd = nullptr; uint16_t* b_hi = nullptr; uint16_t* b_odd = nullptr;
    uint32_t* flip = nullptr;
  } last;
};
static State g;
static std::mutex g_mu;

#define B200_CHECK(call)                                                              \
  do {                                                                                \
    cudaError_t e_ = (call);                                                          \
    if (e_ != cudaSuccess) {                                                          \
      fprintf(stderr, "[eshkol-b200] %s failed: %s (%s:%d)\n", #call,                 \
              cudaGetErrorString(e_), __FILE__, __LINE__);                            \
      return -1;                                                                      \
    }                                                                                 \
  } while (0)

static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

// Bump allocator over the workspace; every block is 1024-byte aligned so TMA
// bases and swizzled tiles never need a second thought.
struct Carver {
  size_t off = 0;
  size_t take(size_t bytes) {
    const size_t o = off;
    off += (bytes + 1023) & ~static_cast<size_t>(1023);
    return o;
  }
};

static int g_dbg_fail_alloc = 0;  // tests: the n-th device allocation from now fails (0 = off)
// every device allocation of the library goes through here
static cudaError_t lib_malloc(void** p, size_t bytes) {
  if (g_dbg_fail_alloc > 0 && --g_dbg_fail_alloc == 0) {
    *p = nullptr;
    return cudaErrorMemoryAllocation;
  }
  return cudaMalloc(p, bytes);
}

static int ensure_workspace(size_t bytes) {
  if (bytes <= g.ws_bytes) return 0;
  B200_CHECK(cudaStreamSynchronize(g.stream));
  if (g.ws) B200_CHECK(cudaFree(g.ws));
  g.ws = nullptr;
  g.ws_bytes = 0;
  g.last.valid = false;
  g.prepA.valid = false;
  const size_t want = bytes + (bytes >> 4);  // a little headroom against regrowth
  cudaError_t e = lib_malloc(reinterpret_cast<void**>(&g.ws), want);
  if (e != cudaSuccess) {
    cudaGetLastError();
    e = lib_malloc(reinterpret_cast<void**>(&g.ws), bytes);
    if (e != cudaSuccess) {
      fprintf(stderr, "[eshkol-b200] workspace allocation of %zu bytes failed: %s\n", bytes,
              cudaGetErrorString(e));
      cudaGetLastError();
      return -1;
    }
    g.ws_bytes = bytes;
    return 0;
  }
  g.ws_bytes = want;
  return 0;
}

uint8_t* aux_reserve(size_t bytes) {
  if (bytes <= g.aux_bytes) return g.aux;
  if (cudaStreamSynchronize(g.stream) != cudaSuccess) return nullptr;
  if (g.aux) cudaFree(g.aux);
  g.aux = nullptr;
  g.aux_bytes = 0;
  if (lib_malloc(reinterpret_cast<void**>(&g.aux), bytes) != cudaSuccess) {
    fprintf(stderr, "[eshkol-b200] scratch allocation of %zu bytes failed\n", bytes);
    cudaGetLastError();
    return nullptr;
  }
  g.aux_bytes = bytes;
  return g.aux;
}

static uint8_t* tbuf_reserve(size_t bytes) {
  if (bytes <= g.tbuf_bytes) return g.tbuf;
  if (cudaStreamSynchronize(g.stream) != cudaSuccess) return nullptr;
  if (g.tbuf) cudaFree(g.tbuf);
  g.tbuf = nullptr;
  g.tbuf_bytes = 0;
  if (lib_malloc(reinterpret_cast<void**>(&g.tbuf), bytes) != cudaSuccess) {
    fprintf(stderr, "[eshkol-b200] scratch allocation of %zu bytes failed\n", bytes);
    cudaGetLastError();
    return nullptr;
  }
  g.tbuf_bytes = bytes;
  return g.tbuf;
}

uint8_t* workspace_reserve(size_t bytes) { return ensure_workspace(bytes) == 0 ? g.ws : nullptr; }
cudaStream_t lib_stream() { return g.stream; }
int lib_device() { return g.ready ? g.device : -1; }
static unsigned long long g_dbg_wait_ns = 0;
static int g_dbg_withhold = 0;
unsigned long long lib_wait_limit_ns() { return g_dbg_wait_ns ? g_dbg_wait_ns : 2000000000ull; }
int lib_take_withhold() { const int w = g_dbg_withhold; g_dbg_withhold = 0; return w; }
static inline int gemm_sms() {
  int n = g.num_sms;
  if (g.sm_limit > 0 && g.sm_limit < n) n = g.sm_limit;
  return n < 2 ? 2 : (n & ~1);  // whole CTA pairs
}
int lib_num_sms() { return gemm_sms(); }
int* lib_status_word() { return g.d_status; }
void count_launches(int n) { g.launches += static_cast<unsigned long long>(n); }

// rows x inner_bytes int8 planes, `planes` of them `plane_stride` bytes apart,
// tiled {128 bytes, box_rows, 1} with the 128-byte swizzle; out-of-range rows and
// bytes read as zero.
int make_plane_map(CUtensorMap* map, const void* base, long long inner_bytes, long long rows,
                   long long planes, long long plane_stride, int box_rows) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner_bytes), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(planes)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner_bytes),
                                 static_cast<cuuint64_t>(plane_stride)};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(kBK), static_cast<cuuint32_t>(box_rows), 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUresult r = g.encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims,
                              strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[eshkol-b200] cuTensorMapEncodeTiled failed (%d): inner=%lld rows=%lld planes=%lld\n",
            static_cast<int>(r), inner_bytes, rows, planes);
    return -1;
  }
  return 0;
}

static void fill_mod_job(GemmJob* j, int a_plane, int b_plane, int out_plane, unsigned p) {
  memset(j, 0, sizeof(*j));
  j->n_seg = 1;
  j->a_plane[0] = a_plane;
  j->b_plane[0] = b_plane;
  j->out_plane = out_plane;
  j->modulus = p;
  if (p) {
    j->magic = static_cast<unsigned>((1ull << 32) / p);
    const unsigned long long bound = 2147483648ull;  // > 131071 * 128 * 128
    j->offset = static_cast<unsigned>((bound + p - 1) / p * p);
  }
}

// ------------------------------------------------------- Ozaki-II CRT constants
static const int kModuli[16] = {256, 255, 253, 251, 247, 241, 239, 233,
                                229, 227, 223, 217, 211, 199, 197, 193};

static long long egcd(long long a, long long b, long long& x, long long& y) {
  if (a == 0) { x = 0; y = 1; return b; }
  long long x1, y1;
  const long long gg = egcd(b % a, a, x1, y1);
  x = y1 - (b / a) * x1;
  y = x1;
  return gg;
}
static int mod_inverse(long long a, long long m) {
  long long x, y;
  egcd(a % m, m, x, y);
  return static_cast<int>((x % m + m) % m);
}

// P, its double-double split, 1/P, and the split CRT weights s_l = (P/p_l) *
// ((P/p_l)^-1 mod p_l); the high part keeps 53 - (8 + ceil(log2 n) + 1) bits.
// Restates precompute_ozaki_constants, lib/backend/gpu/gpu_memory.mm:301-341.
void oz2_host_consts(int n_mod, Oz2DeviceConsts* c, double* log2P) {
  memset(c, 0, sizeof(*c));
  c->n_mod = n_mod;
  __int128 P = 1;
  for (int l = 0; l < n_mod; ++l) P *= kModuli[l];
  c->P1 = static_cast<double>(P);
  c->P2 = static_cast<double>(P - static_cast<__int128>(c->P1));
  c->Pinv = 1.0 / static_cast<double>(P);
  if (log2P) *log2P = log2(static_cast<double>(P));
  const int bits_to_remove = 8 + static_cast<int>(ceil(log2(static_cast<double>(n_mod))));
  for (int l = 0; l < n_mod; ++l) {
    const int p = kModuli[l];
    const __int128 Pp = P / p;
    const int q = mod_inverse(static_cast<long long>(Pp % p), p);
    const __int128 s = Pp * static_cast<__int128>(q);
    const double s_d = static_cast<double>(s);
    const double factor = static_cast<double>(1LL << (bits_to_remove + 1)) + 1.0;
    volatile double t = factor * s_d;
    volatile double u = t - s_d;
    c->sl1[l] = t - u;
    c->sl2[l] = static_cast<double>(s - static_cast<__int128>(c->sl1[l]));
    c->p_d[l] = static_cast<double>(p);
    c->p_inv[l] = 1.0 / static_cast<double>(p);
    c->p_i[l] = p;
    c->q_i[l] = q;
  }
}

// E = clamp(floor((log2 P - 1 - log2 K - fracA - fracB) / 2), 0, 52), with fracA
// the largest fractional part of log2 of a nonzero row maximum, fracB likewise
// for columns.  Restates gpu_memory.mm:403-417 and :2510-2512 on the host.
static int oz2_exponent(double log2P, long long K, const double* amax, long long M,
                        const double* bmax, long long N) {
  double fa = 0.0, fb = 0.0;
  for (long long i = 0; i < M; ++i)
    if (amax[i] > 0.0) { const double lg = log2(amax[i]); const double f = lg - floor(lg); if (f > fa) fa = f; }
  for (long long j = 0; j < N; ++j)
    if (bmax[j] > 0.0) { const double lg = log2(bmax[j]); const double f = lg - floor(lg); if (f > fb) fb = f; }
  int E = static_cast<int>(floor((log2P - 1.0 - log2(static_cast<double>(K)) - fa - fb) / 2.0));
  if (E > 52) E = 52;
  if (E < 0) E = 0;
  return E;
}

// ------------------------------------------------------------ Ozaki-II driver
struct Oz2Geom {
  long long M, K, N, Kp, K0, Mp, Np;
  int n_chunks, last_seg, tiles_m, tiles_n, bn;
};

static Oz2Geom oz2_geometry(long long M, long long K, long long N, int bn) {
  Oz2Geom q;
  q.M = M; q.K = K; q.N = N; q.bn = bn;
  q.Kp = round_up(K, kBK);
  q.n_chunks = static_cast<int>((K + kChunkK - 1) / kChunkK);
  const int last_len = static_cast<int>(K - static_cast<long long>(q.n_chunks - 1) * kChunkK);
  q.last_seg = static_cast<int>(round_up(last_len, kBK));
  q.K0 = static_cast<long long>(q.n_chunks - 1) * kChunkSeg + q.last_seg;
  q.tiles_m = static_cast<int>((M + kBM - 1) / kBM);
  q.tiles_n = static_cast<int>((N + bn - 1) / bn);
  q.Mp = round_up(M, 2 * kBM);  // whole pair tiles, for the two-SM products kernel
  q.Np = static_cast<long long>(q.tiles_n) * bn;
  return q;
}

// k-blocks of 128 an odd-modulus accumulator takes before it is handed to the epilogue:
// 1023 * 128 * 128^2 < 2^31
constexpr int kOddUnitKb = 1023;
// deepest product for which the exponent E is 52 whatever the data (gpu_memory.mm:2510-2512 with
// log2 P = 125.37 and both fractional parts below 1): beyond it E needs the maxima of both
// operands, and operands can no longer be prepared one without the other
constexpr long long kMaxPreparedK = 262144;

static int oz2_check_shape(long long M, long long K, long long N, int n_mod) {
  if (n_mod < 2 || n_mod > 16) {
    fprintf(stderr, "[eshkol-b200] Ozaki-II: moduli count %d outside [2,16]\n", n_mod);
    return -1;
  }
  // int32 accumulation of products of magnitude <= 128^2 is exact for 131071 of them; deeper
  // products hand the accumulator over every kOddUnitKb k-blocks and sum the residues
  if (K > (1LL << 24)) {
    fprintf(stderr, "[eshkol-b200] Ozaki-II: K=%lld is beyond what this library accepts (2^24)\n", K);
    return -1;
  }
  if (M > 0x7fffff00LL || N > 0x7fffff00LL) return -1;
  return 0;
}

#define B200_MARK(i) do { if (timed) B200_CHECK(cudaEventRecord(g.ev_b[g.n_evb % State::kEvRing][i], st)); } while (0)

// Right-hand operand of the exact tier, prepared once and kept: nu_j, 2^+-nu_j and
// the residue planes of B.  Rows of A can then be multiplied block by block (the
// host pipeline, the row-sharded multi-GPU driver) without touching B again.  Only
// with all 16 moduli, where the exponent E is 52 whatever the data; with fewer moduli
// E depends on the maxima of both operands and the one-shot path below is used.
// Where the pieces of a prepared right-hand operand sit behind a base address.
struct BLayout {
  size_t bmax, nu, sb, sbi, b0, bhi, boddf, bodd, pix, total;
  size_t flag_row_bytes, b_stride;
};

static BLayout oz2_b_layout(const Oz2Geom& q, size_t view_pixels) {
  const int n_odd = 15;
  BLayout L;
  Carver cv;
  L.bmax = cv.take(q.N * 8); L.nu = cv.take(q.N * 4); L.sb = cv.take(q.N * 8); L.sbi = cv.take(q.N * 8);
  L.b0 = cv.take(static_cast<size_t>(q.N) * q.K0);
  L.flag_row_bytes = static_cast<size_t>(q.n_chunks) * kChunkUnits * sizeof(uint16_t);
  L.bhi = cv.take(static_cast<size_t>(q.N) * L.flag_row_bytes);
  L.boddf = cv.take(static_cast<size_t>(q.N) * L.flag_row_bytes);
  L.b_stride = static_cast<size_t>(q.N) * q.Kp;
  L.bodd = cv.take(L.b_stride * n_odd);
  L.pix = cv.take(view_pixels * 8);
  L.total = cv.off;
  return L;
}

// g.prep <- the operand whose pieces lie behind ws (its planes written or about to be written)
static void oz2_bind_b(uint8_t* ws, const Oz2Geom& q, const BLayout& L, int bn) {
  State::Prepared& P = g.prep;
  P.K = q.K; P.N = q.N; P.Kp = q.Kp; P.K0 = q.K0; P.n_chunks = q.n_chunks; P.last_seg = q.last_seg;
  P.bn = bn; P.Np = q.Np; P.tiles_n = q.tiles_n;
  P.bmax = reinterpret_cast<double*>(ws + L.bmax);
  P.nu = reinterpret_cast<int*>(ws + L.nu);
  P.sb = reinterpret_cast<double*>(ws + L.sb);
  P.sbi = reinterpret_cast<double*>(ws + L.sbi);
  P.b0 = reinterpret_cast<int8_t*>(ws + L.b0);
  P.b_hi = reinterpret_cast<uint16_t*>(ws + L.bhi);
  P.b_odd = reinterpret_cast<uint16_t*>(ws + L.boddf);
  P.bodd = reinterpret_cast<int8_t*>(ws + L.bodd);
  P.bodd_stride = static_cast<long long>(L.b_stride);
  oz2_host_consts(16, &P.consts, nullptr);
}

static int oz2_b_maps(const Oz2Geom& q, int bn) {
  State::Prepared& P = g.prep;
  const int n_odd = 15;
  if (make_plane_map(&P.mB0, P.b0, q.K0, q.N, 1, static_cast<long long>(q.N) * q.K0, bn)) return -1;
  if (make_plane_map(&P.mB1, P.bodd, q.Kp, q.N, n_odd, P.bodd_stride, bn)) return -1;
  if (make_plane_map(&P.mB1_half, P.bodd, q.Kp, q.N, n_odd, P.bodd_stride, kBM)) return -1;
  return 0;
}

// Right-hand operand of the exact tier, prepared once and kept: nu_j, 2^+-nu_j and
// the residue planes of B.  Rows of A can then be multiplied block by block (the
// host pipeline, the row-sharded multi-GPU driver) without touching B again.  Only
// with all 16 moduli, where the exponent E is 52 whatever the data; with fewer moduli
// E depends on the maxima of both operands and the one-shot path below is used.
static int oz2_prepare_b(const double* dB, long long K, long long N, int bn, bool trans = false,
                         const Im2colView* view = nullptr, cudaStream_t on_stream = nullptr) {
  if (oz2_check_shape(1, K, N, 16)) return -1;
  if (K > kMaxPreparedK) {
    fprintf(stderr, "[eshkol-b200] an operand can be prepared on its own only for K <= %lld\n", kMaxPreparedK);
    return -1;
  }
  const Oz2Geom q = oz2_geometry(1, K, N, bn);
  const int n_odd = 15;
  const BLayout L = oz2_b_layout(q, view ? static_cast<size_t>(view->batch * view->H * view->W) : 0);
  g.prep.valid = false;
  if (L.total > g.bside_bytes) {
    B200_CHECK(cudaStreamSynchronize(g.stream));
    if (g.bside) B200_CHECK(cudaFree(g.bside));
    g.bside = nullptr; g.bside_bytes = 0;
    if (lib_malloc(reinterpret_cast<void**>(&g.bside), L.total) != cudaSuccess) {
      fprintf(stderr, "[eshkol-b200] allocation of %zu bytes for the prepared operand failed\n", L.total);
      cudaGetLastError();
      return -1;
    }
    g.bside_bytes = L.total;
  }
  uint8_t* ws = g.bside;
  oz2_bind_b(ws, q, L, bn);
  State::Prepared& P = g.prep;
  cudaStream_t st = on_stream ? on_stream : g.stream;
  const bool timed = g.timing && g.ev_made;
  g.ev_valid = false;
  B200_MARK(0);
  // trans: B is stored N x K (each column of the operand is a contiguous row), which is the
  // layout the row scan and the non-transposing split of a left-hand operand read
  if (trans) B200_CHECK(launch_scan_rows(dB, N, K, P.bmax, st));
  else if (view) B200_CHECK(launch_scan_view(*view, N, reinterpret_cast<double*>(ws + L.pix), P.bmax, st));
  else B200_CHECK(launch_scan_cols(dB, K, N, reinterpret_cast<unsigned long long*>(P.bmax), st));
  B200_CHECK(launch_scales(P.bmax, N, 52, P.nu, P.sb, P.sbi, st));
  B200_MARK(1);
  SplitPlanes pb{N, K, q.Kp, q.K0, q.n_chunks, n_odd, P.b0, P.b_hi, P.b_odd, P.bodd, P.bodd_stride};
  if (trans) B200_CHECK(launch_split_a(dB, P.sb, pb, P.consts, st));
  else B200_CHECK(launch_split_b(dB, P.sb, N, pb, P.consts, st, view));
  B200_MARK(2);
  if (timed) ++g.n_evb;
  g.launches += 3;
  if (oz2_b_maps(q, bn)) return -1;
  P.valid = true;
  ++g.prep_token;
  return 0;
}

// A block of columns [col0, col0 + ncols) of a right-hand operand of N columns, prepared into a
// caller-owned buffer laid out as oz2_b_layout lays out the whole operand: the ranks of the
// multi-GPU driver each prepare their share of a panel's columns and exchange the pieces.
// dB points at the first of those columns, rows ldb elements apart.
static int oz2_prepare_b_columns(const double* dB, long long ldb, long long K, long long N, long long col0,
                                 long long ncols, uint8_t* ws) {
  if (oz2_check_shape(1, K, N, 16) || K > kMaxPreparedK) return -1;
  if (col0 < 0 || ncols <= 0 || col0 + ncols > N || ldb < ncols) return -1;
  const Oz2Geom q = oz2_geometry(1, K, N, 256);
  const int n_odd = 15;
  const BLayout L = oz2_b_layout(q, 0);
  double* bmax = reinterpret_cast<double*>(ws + L.bmax) + col0;
  int* nu = reinterpret_cast<int*>(ws + L.nu) + col0;
  double* sb = reinterpret_cast<double*>(ws + L.sb) + col0;
  double* sbi = reinterpret_cast<double*>(ws + L.sbi) + col0;
  Oz2DeviceConsts hc;
  oz2_host_consts(16, &hc, nullptr);
  cudaStream_t st = g.stream;
  const bool timed = g.timing && g.ev_made;
  B200_MARK(0);
  B200_CHECK(launch_scan_cols(dB, K, ncols, reinterpret_cast<unsigned long long*>(bmax), st, ldb));
  B200_CHECK(launch_scales(bmax, ncols, 52, nu, sb, sbi, st));
  B200_MARK(1);
  SplitPlanes pb{ncols, K, q.Kp, q.K0, q.n_chunks, n_odd,
                 reinterpret_cast<int8_t*>(ws + L.b0) + col0 * q.K0,
                 reinterpret_cast<uint16_t*>(ws + L.bhi + static_cast<size_t>(col0) * L.flag_row_bytes),
                 reinterpret_cast<uint16_t*>(ws + L.boddf + static_cast<size_t>(col0) * L.flag_row_bytes),
                 reinterpret_cast<int8_t*>(ws + L.bodd) + col0 * q.Kp, static_cast<long long>(L.b_stride)};
  B200_CHECK(launch_split_b(dB, sb, ncols, pb, hc, st, nullptr, ldb));
  B200_MARK(2);
  if (timed) ++g.n_evb;
  g.launches += 3;
  return 0;
}

// Where the pieces of one prepared block of rows of A sit behind a base address, and how
// much room the product residues of a result n_cols wide need behind them.
struct ALayout {
  size_t amax, mu, sa, sai, a0, ahi, aoddf, aodd, end, total;
};

static ALayout oz2_a_layout(const Oz2Geom& q) {
  const int n_odd = 15;
  ALayout L;
  Carver cv;
  L.amax = cv.take(q.M * 8); L.mu = cv.take(q.M * 4); L.sa = cv.take(q.M * 8); L.sai = cv.take(q.M * 8);
  L.a0 = cv.take(static_cast<size_t>(q.M) * q.K0);
  const size_t flag_bytes = static_cast<size_t>(q.M) * q.n_chunks * kChunkUnits * sizeof(uint16_t);
  L.ahi = cv.take(flag_bytes); L.aoddf = cv.take(flag_bytes);
  L.aodd = cv.take(static_cast<size_t>(q.M) * q.Kp * n_odd);
  L.end = cv.off;
  const size_t w_stride = static_cast<size_t>(q.Mp) * q.Np;
  cv.take(w_stride * 2);
  cv.take(w_stride * n_odd);
  cv.take(1024 + w_stride / 32 * 16 * q.n_chunks);  // tie list: a cursor, then room for a record per group and chunk
  cv.take(w_stride / 32 * 4);                       // flip bits
  L.total = cv.off;
  return L;
}

// scan, scale and split one block of rows on stream st into the planes behind ws.
// tev (optional): three events recorded before the scan, after the scales, after the split.
static int oz2_prepare_a_at(State::PreparedA& A, uint8_t* ws, const Oz2Geom& q, const double* dA,
                            cudaStream_t st, cudaEvent_t* tev, bool trans = false) {
  const int n_odd = 15;
  const ALayout L = oz2_a_layout(q);
  const long long M = q.M;
  A.valid = false;
  A.M = M; A.K = q.K; A.Kp = q.Kp; A.K0 = q.K0; A.Mp = q.Mp; A.tiles_m = q.tiles_m;
  A.n_chunks = q.n_chunks; A.last_seg = q.last_seg; A.end = L.end;
  A.amax = reinterpret_cast<double*>(ws + L.amax);
  A.mu = reinterpret_cast<int*>(ws + L.mu);
  A.sa = reinterpret_cast<double*>(ws + L.sa);
  A.sai = reinterpret_cast<double*>(ws + L.sai);
  A.jobs = g.d_jobs16;
  A.a0 = reinterpret_cast<int8_t*>(ws + L.a0);
  A.a_hi = reinterpret_cast<uint16_t*>(ws + L.ahi);
  A.a_odd = reinterpret_cast<uint16_t*>(ws + L.aoddf);
  A.aodd = reinterpret_cast<int8_t*>(ws + L.aodd);
  A.a_stride = static_cast<long long>(M) * q.Kp;
  Oz2DeviceConsts hc;
  oz2_host_consts(16, &hc, nullptr);
  if (tev) B200_CHECK(cudaEventRecord(tev[0], st));
  // trans: A is stored K x M, the layout of a right-hand operand: column scan, transposing split
  if (trans) B200_CHECK(launch_scan_cols(dA, q.K, M, reinterpret_cast<unsigned long long*>(A.amax), st));
  else B200_CHECK(launch_scan_rows(dA, M, q.K, A.amax, st));
  B200_CHECK(launch_scales(A.amax, M, 52, A.mu, A.sa, A.sai, st));
  if (tev) B200_CHECK(cudaEventRecord(tev[1], st));
  SplitPlanes pa{M, q.K, q.Kp, q.K0, q.n_chunks, n_odd, A.a0, A.a_hi, A.a_odd, A.aodd, A.a_stride};
  if (trans) B200_CHECK(launch_split_b(dA, A.sa, M, pa, hc, st));
  else B200_CHECK(launch_split_a(dA, A.sa, pa, hc, st));
  if (tev) B200_CHECK(cudaEventRecord(tev[2], st));
  g.launches += 3;
  if (make_plane_map(&A.mA0, A.a0, q.K0, M, 1, static_cast<long long>(M) * q.K0, kBM)) return -1;
  if (make_plane_map(&A.mA1, A.aodd, q.Kp, M, n_odd, A.a_stride, kBM)) return -1;
  A.valid = true;
  return 0;
}

// Left-hand operand prepared once: mu_i, 2^+-mu_i and the residue planes of a block
// of rows of A, kept at the front of the workspace; room for the product residues of
// a result up to n_cols_hint columns wide is reserved behind them so that the
// following multiplications never move the planes.
static int oz2_prepare_a(const double* dA, long long M, long long K, long long n_cols_hint, int bn,
                         bool trans = false) {
  if (oz2_check_shape(M, K, n_cols_hint, 16)) return -1;
  const Oz2Geom q = oz2_geometry(M, K, n_cols_hint, bn);
  g.prepA.valid = false;
  if (ensure_workspace(oz2_a_layout(q).total) != 0) return -1;
  const bool timed = g.timing && g.ev_made;
  g.bands_timed = 0;
  const int rc = oz2_prepare_a_at(g.prepA, g.ws, q, dA, g.stream,
                                  timed ? g.ev_a[g.n_eva % State::kEvRing] : nullptr, trans);
  if (timed && rc == 0) ++g.n_eva;
  return rc;
}

// Streams of one multiplication.  Serial: all three are the library stream.  In the band
// pipeline the tie resolution and the reconstruction run on `post`, ordered behind the
// products by the two events, so that they overlap the next band's products.
struct MulLanes {
  cudaStream_t gemm, post;
  cudaEvent_t g0_done, g1_done;  // used only when post != gemm
  cudaEvent_t* tev;              // optional: gemm-stream events [0..2], post-stream events [3..6]
};

// C = (prepared A) * (prepared B): the 16 modular products on the tensor cores and
// the reconstruction.  ws / cap: the block A was prepared in.
static int oz2_multiply_at(const State::PreparedA& A, uint8_t* ws, size_t cap, double* dC,
                           const EshkolB200GemmOpts& o, const MulLanes& ln) {
  const State::Prepared& P = g.prep;
  if (!P.valid || !A.valid) {
    fprintf(stderr, "[eshkol-b200] multiply needs both operands prepared\n");
    return -1;
  }
  if (A.K != P.K) {
    fprintf(stderr, "[eshkol-b200] prepared operands disagree on K (%lld vs %lld)\n", A.K, P.K);
    return -1;
  }
  const int n_odd = 15;
  const long long M = A.M;
  if (static_cast<long long>(A.tiles_m) * P.tiles_n * 16 > 0x7fffffffLL) return -1;
  Carver cv;
  cv.off = A.end;
  const size_t w_stride = static_cast<size_t>(A.Mp) * P.Np;
  const size_t o_w0 = cv.take(w_stride * 2), o_wodd = cv.take(w_stride * n_odd);
  const size_t o_tie = cv.take(1024 + w_stride / 32 * 16 * A.n_chunks), o_flip = cv.take(w_stride / 32 * 4);
  if (cv.off > cap) {
    fprintf(stderr, "[eshkol-b200] result of %lld columns exceeds the room reserved when A was prepared\n", P.N);
    return -1;
  }
  int16_t* w0 = reinterpret_cast<int16_t*>(ws + o_w0);
  int8_t* wodd = reinterpret_cast<int8_t*>(ws + o_wodd);
  uint32_t* tie_bits = reinterpret_cast<uint32_t*>(ws + o_tie);
  uint32_t* flip_bits = reinterpret_cast<uint32_t*>(ws + o_flip);
  cudaStream_t st = ln.gemm, sp = ln.post;
  const bool lanes = sp != st;
  cudaEvent_t* tev = ln.tev;
  if (g.b_pending) {
    // the right-hand operand was prepared on the side stream
    B200_CHECK(cudaStreamWaitEvent(st, g.b_pending, 0));
    g.b_pending = nullptr;
  }

  GemmParams p0 = make_gemm_params();
  p0.tie_bits = tie_bits + 256;  // the dense table, for shapes whose fields do not fit a list record
  if (tie_list_fits(P.Np, A.n_chunks) && !o.use_simt_products) {
    p0.tie_cursor = reinterpret_cast<unsigned int*>(tie_bits);
    p0.tie_list = reinterpret_cast<uint4*>(tie_bits + 256);
  }
  p0.tiles_m = A.tiles_m; p0.tiles_n = P.tiles_n; p0.n_jobs = 1;
  p0.kb_per_seg = static_cast<int>(A.K0 / kBK);
  p0.kb_per_unit = kChunkSeg / kBK;
  p0.a_hi = A.a_hi; p0.a_odd = A.a_odd; p0.b_odd = P.b_odd; p0.b_hi = P.b_hi;
  p0.n_chunks = A.n_chunks;
  p0.group_m = 16;
  p0.jobs = A.jobs;
  p0.out = reinterpret_cast<uint8_t*>(w0);
  p0.out_plane_stride = 0;
  p0.ldo = static_cast<int>(P.Np);
  p0.status = g.d_status;
  p0.work_counter = g.d_status + 1;
  GemmParams p1 = p0;
  p1.n_jobs = n_odd;
  p1.kb_per_seg = static_cast<int>(A.Kp / kBK);
  p1.kb_per_unit = kOddUnitKb;
  p1.jobs = A.jobs + 1;
  p1.out = reinterpret_cast<uint8_t*>(wodd);
  p1.out_plane_stride = static_cast<long long>(w_stride);
  const int tiles = A.tiles_m * P.tiles_n;
  if (tev) B200_CHECK(cudaEventRecord(tev[0], st));
  if (o.use_simt_products) {
    SimtPlanes s0{A.a0, 0, static_cast<int>(A.K0), P.b0, 0, static_cast<int>(A.K0), static_cast<int>(M), static_cast<int>(P.N)};
    SimtPlanes s1{A.aodd, A.a_stride, static_cast<int>(A.Kp), P.bodd, P.bodd_stride,
                  static_cast<int>(A.Kp), static_cast<int>(M), static_cast<int>(P.N)};
    B200_CHECK(launch_modgemm_simt(kEpiMod256, s0, p0, st));
    if (lanes) { B200_CHECK(cudaEventRecord(ln.g0_done, st)); B200_CHECK(cudaStreamWaitEvent(sp, ln.g0_done, 0)); }
    if (tev) B200_CHECK(cudaEventRecord(tev[3], sp));
    B200_CHECK(cudaMemsetAsync(flip_bits, 0, w_stride / 32 * 4, sp));
    if (tev) B200_CHECK(cudaEventRecord(tev[4], sp));
    if (tev) B200_CHECK(cudaEventRecord(tev[1], st));
    B200_CHECK(launch_modgemm_simt(kEpiModI8, s1, p1, st));
  } else {
    if (p0.tie_cursor) B200_CHECK(cudaMemsetAsync(p0.tie_cursor, 0, sizeof(unsigned int), st));
    B200_CHECK(launch_modgemm(P.bn, kEpiMod256, A.mA0, P.mB0, p0, tiles, gemm_sms(), st));
    if (lanes) { B200_CHECK(cudaEventRecord(ln.g0_done, st)); B200_CHECK(cudaStreamWaitEvent(sp, ln.g0_done, 0)); }
    if (tev) B200_CHECK(cudaEventRecord(tev[3], sp));
    B200_CHECK(launch_tie_resolve(p0, flip_bits, static_cast<int>(M), static_cast<int>(P.N), sp));
    if (tev) B200_CHECK(cudaEventRecord(tev[4], sp));
    if (tev) B200_CHECK(cudaEventRecord(tev[1], st));
    if (g.pair_gemm && P.bn == 256 && p1.kb_per_seg <= kOddUnitKb) {
      B200_CHECK(launch_modgemm_pair(kEpiModI8, A.mA1, P.mB1_half, p1, static_cast<int>(A.Mp / (2 * kBM)),
                                     gemm_sms(), st));
    } else {
      B200_CHECK(launch_modgemm(P.bn, kEpiModI8, A.mA1, P.mB1, p1, tiles * n_odd, gemm_sms(), st));
    }
  }
  if (tev) B200_CHECK(cudaEventRecord(tev[2], st));
  if (lanes) { B200_CHECK(cudaEventRecord(ln.g1_done, st)); B200_CHECK(cudaStreamWaitEvent(sp, ln.g1_done, 0)); }
  CrtArgs ca;
  ca.w0 = w0; ca.flip = flip_bits; ca.w_odd = wodd; ca.w_odd_stride = static_cast<long long>(w_stride); ca.ldw = P.Np;
  ca.n_mod = 16; ca.M = M; ca.N = P.N;
  ca.inv_scale_a = A.sai; ca.inv_scale_b = P.sbi;
  ca.C = dC; ca.ldc = (o.ldc > 0) ? o.ldc : P.N;
  ca.bias_mode = o.bias ? o.bias_mode : 0; ca.bias = o.bias;
  ca.activation = o.activation;
  ca.pixels_per_image = o.pixels_per_image;
  if (tev) B200_CHECK(cudaEventRecord(tev[5], sp));
  B200_CHECK(launch_crt(ca, P.consts, sp));
  if (tev) B200_CHECK(cudaEventRecord(tev[6], sp));
  g.launches += 4;

  State::Last& L = g.last;
  L.valid = true; L.M = M; L.K = P.K; L.N = P.N; L.Kp = A.Kp; L.K0 = A.K0; L.Mp = A.Mp; L.Np = P.Np;
  L.n_mod = 16; L.n_chunks = A.n_chunks; L.last_seg = A.last_seg;
  L.mu = A.mu; L.nu = P.nu; L.a0 = A.a0; L.aodd = A.aodd; L.aodd_stride = A.a_stride;
  L.b0 = P.b0; L.bodd = P.bodd; L.bodd_stride = P.bodd_stride;
  L.w0 = w0; L.wodd = wodd; L.wodd_stride = static_cast<long long>(w_stride);
  L.a_hi = A.a_hi; L.a_odd = A.a_odd; L.b_hi = P.b_hi; L.b_odd = P.b_odd; L.flip = flip_bits;
  return 0;
}

// Serial multiplication on the library stream.  Stage events of this call's ring entry: [0] at
// its start, [1] behind the modulus-256 product and its tie resolution, [2] behind the odd
// products, [3] behind the reconstruction; the lane marks that have no serial meaning land on
// a scratch event.
static int oz2_multiply(double* dC, const EshkolB200GemmOpts& o) {
  const bool timed = g.timing && g.ev_made;
  cudaEvent_t* e = g.ev_m[g.n_evm % State::kEvRing];
  cudaEvent_t tev[7] = {e[0], e[1], e[2], g.ev_scratch, e[1], g.ev_scratch, e[3]};
  MulLanes ln{g.stream, g.stream, nullptr, nullptr, timed ? tev : nullptr};
  const int rc = oz2_multiply_at(g.prepA, g.ws, g.ws_bytes, dC, o, ln);
  if (timed && rc == 0) ++g.n_evm;
  g.ev_valid = timed && rc == 0;
  return rc;
}

static int make_band_lanes() {
  if (g.lanes_made) return 0;
  int least = 0, greatest = 0;
  B200_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  // the products run on the library stream (highest priority); the splits and the
  // reconstruction fill the issue slots the tensor-core kernel leaves idle
  B200_CHECK(cudaStreamCreateWithPriority(&g.s_prep, cudaStreamNonBlocking, least));
  B200_CHECK(cudaStreamCreateWithPriority(&g.s_post, cudaStreamNonBlocking, least));
  B200_CHECK(cudaEventCreateWithFlags(&g.eb_start, cudaEventDisableTiming));
  B200_CHECK(cudaEventCreateWithFlags(&g.eb_done, cudaEventDisableTiming));
  for (int i = 0; i < 2; ++i) {
    B200_CHECK(cudaEventCreateWithFlags(&g.eb_a_ready[i], cudaEventDisableTiming));
    B200_CHECK(cudaEventCreateWithFlags(&g.eb_g0[i], cudaEventDisableTiming));
    B200_CHECK(cudaEventCreateWithFlags(&g.eb_g1[i], cudaEventDisableTiming));
    B200_CHECK(cudaEventCreateWithFlags(&g.eb_w_free[i], cudaEventDisableTiming));
  }
  g.lanes_made = true;
  return 0;
}

// C = A * (prepared B) over bands of rows, three streams, two workspace slots:
//   prep:  scan / scale / split of band r+1
//   gemm:  the 16 modular products of band r          (the library stream)
//   post:  tie resolution and reconstruction of band r (and r-1)
// Every row's result depends on that row of A and on B only, so the bits are those of the
// serial product.  The library stream is ordered behind the last band when this returns.
static int oz2_gemm_banded(const double* dA, double* dC, long long M, long long bm,
                           const EshkolB200GemmOpts& o) {
  const State::Prepared& P = g.prep;
  const long long nb = (M + bm - 1) / bm;
  const Oz2Geom qb = oz2_geometry(bm, P.K, P.N, P.bn);
  const size_t slot = (oz2_a_layout(qb).total + 1023) & ~static_cast<size_t>(1023);
  g.prepA.valid = false;
  if (ensure_workspace(2 * slot) != 0) return -1;
  if (make_band_lanes() != 0) return -1;
  const bool timed = g.timing && g.ev_band_made && nb <= State::kMaxBands;
  const long long ldc = (o.ldc > 0) ? o.ldc : P.N;
  cudaStream_t st = g.stream;
  B200_CHECK(cudaEventRecord(g.eb_start, st));
  B200_CHECK(cudaStreamWaitEvent(g.s_prep, g.eb_start, 0));
  B200_CHECK(cudaStreamWaitEvent(g.s_post, g.eb_start, 0));
  int rc = 0;
  for (long long r = 0; r < nb; ++r) {
    const int s = static_cast<int>(r & 1);
    const long long r0 = r * bm, rows = (r0 + bm <= M) ? bm : M - r0;
    uint8_t* ws = g.ws + s * slot;
    cudaEvent_t* tev = timed ? &g.ev_band[r * State::kBandEvents] : nullptr;
    const Oz2Geom q = oz2_geometry(rows, P.K, P.N, P.bn);
    // the slot's A planes are free once band r-2 is through its odd products (residue planes)
    // and its tie resolution (flag planes); the reconstruction event covers the latter
    if (r >= 2) {
      B200_CHECK(cudaStreamWaitEvent(g.s_prep, g.eb_g1[s], 0));
      B200_CHECK(cudaStreamWaitEvent(g.s_prep, g.eb_w_free[s], 0));
    }
    rc = oz2_prepare_a_at(g.bandA[s], ws, q, dA + r0 * P.K, g.s_prep, tev);
    if (rc) break;
    B200_CHECK(cudaEventRecord(g.eb_a_ready[s], g.s_prep));
    B200_CHECK(cudaStreamWaitEvent(st, g.eb_a_ready[s], 0));
    // ... and its product residues once band r-2 is reconstructed
    if (r >= 2) B200_CHECK(cudaStreamWaitEvent(st, g.eb_w_free[s], 0));
    EshkolB200GemmOpts ob = o;
    if (ob.bias && ob.bias_mode == 1) ob.bias = o.bias + r0;
    MulLanes ln{st, g.s_post, g.eb_g0[s], g.eb_g1[s], tev ? tev + 3 : nullptr};
    rc = oz2_multiply_at(g.bandA[s], ws, slot, dC + r0 * ldc, ob, ln);
    if (rc) break;
    B200_CHECK(cudaEventRecord(g.eb_w_free[s], g.s_post));
  }
  // join: later work on the library stream sees the whole result
  B200_CHECK(cudaEventRecord(g.eb_done, g.s_post));
  B200_CHECK(cudaStreamWaitEvent(st, g.eb_done, 0));
  B200_CHECK(cudaEventRecord(g.eb_done, g.s_prep));
  B200_CHECK(cudaStreamWaitEvent(st, g.eb_done, 0));
  g.bandA[0].valid = g.bandA[1].valid = false;
  if (rc == 0 && timed) { g.bands_timed = static_cast<int>(nb); g.ev_valid = g.timing && g.ev_made; }
  return rc;
}

// C[rows] = A[rows] * (prepared B) for one block of rows.  Bit-identical to the same
// rows of a one-shot product.  allow_bands: large blocks go through the band pipeline.
static int oz2_gemm_rows(const double* dA, double* dC, long long M, const EshkolB200GemmOpts& o,
                         bool allow_bands) {
  const State::Prepared& P = g.prep;
  if (!P.valid) {
    fprintf(stderr, "[eshkol-b200] no prepared right-hand operand\n");
    return -1;
  }
  const long long bm = g.band_rows;
  if (allow_bands && bm >= 256 && M >= 2 * bm && o.pixels_per_image == 0 && !o.use_simt_products &&
      !o.trans_a) {
    // bands of whole pair tiles; at most kMaxBands of them
    long long rows = bm;
    while ((M + rows - 1) / rows > State::kMaxBands) rows *= 2;
    return oz2_gemm_banded(dA, dC, M, rows, o);
  }
  if (oz2_prepare_a(dA, M, P.K, P.N, P.bn, o.trans_a != 0)) return -1;
  const int rc = oz2_multiply(dC, o);
  g.prepA.valid = false;  // dA belongs to the caller
  return rc;
}

// One-shot product with fewer than 16 moduli: the exponent E needs the maxima of both
// operands (gpu_memory.mm:2510-2512), so the operands are scanned together.
static int ozaki2_gemm_general(const double* dA, const double* dB, double* dC, long long M,
                               long long K, long long N, int n_mod, const EshkolB200GemmOpts& o) {
  g.bands_timed = 0;
  if (oz2_check_shape(M, K, N, n_mod)) return -1;
  const int bn = (o.gemm_tile_n == 128) ? 128 : 256;
  const Oz2Geom q = oz2_geometry(M, K, N, bn);
  const int n_odd = n_mod - 1;
  if (static_cast<long long>(q.tiles_m) * q.tiles_n * n_mod > 0x7fffffffLL) return -1;
  Carver cv;
  const size_t o_amax = cv.take(M * 8), o_bmax = cv.take(N * 8);
  const size_t o_mu = cv.take(M * 4), o_nu = cv.take(N * 4);
  const size_t o_sa = cv.take(M * 8), o_sai = cv.take(M * 8);
  const size_t o_sb = cv.take(N * 8), o_sbi = cv.take(N * 8);
  const size_t o_jobs = cv.take(sizeof(GemmJob) * 16);
  const size_t o_a0 = cv.take(static_cast<size_t>(M) * q.K0), o_b0 = cv.take(static_cast<size_t>(N) * q.K0);
  const size_t fa_bytes = static_cast<size_t>(M) * q.n_chunks * kChunkUnits * sizeof(uint16_t);
  const size_t fb_bytes = static_cast<size_t>(N) * q.n_chunks * kChunkUnits * sizeof(uint16_t);
  const size_t o_ahi = cv.take(fa_bytes), o_aoddf = cv.take(fa_bytes);
  const size_t o_bhi = cv.take(fb_bytes), o_boddf = cv.take(fb_bytes);
  const size_t a_stride = static_cast<size_t>(M) * q.Kp, b_stride = static_cast<size_t>(N) * q.Kp;
  const size_t o_aodd = cv.take(a_stride * n_odd), o_bodd = cv.take(b_stride * n_odd);
  const size_t w_stride = static_cast<size_t>(q.Mp) * q.Np;
  const size_t o_w0 = cv.take(w_stride * 2), o_wodd = cv.take(w_stride * n_odd);
  const size_t o_tie = cv.take(1024 + w_stride / 32 * 16 * q.n_chunks), o_flip = cv.take(w_stride / 32 * 4);
  if (ensure_workspace(cv.off) != 0) return -1;
  uint8_t* ws = g.ws;
  uint32_t* tie_bits = reinterpret_cast<uint32_t*>(ws + o_tie);
  uint32_t* flip_bits = reinterpret_cast<uint32_t*>(ws + o_flip);
  double* amax = reinterpret_cast<double*>(ws + o_amax);
  double* bmax = reinterpret_cast<double*>(ws + o_bmax);
  int* mu = reinterpret_cast<int*>(ws + o_mu);
  int* nu = reinterpret_cast<int*>(ws + o_nu);
  double* sa = reinterpret_cast<double*>(ws + o_sa);
  double* sai = reinterpret_cast<double*>(ws + o_sai);
  double* sb = reinterpret_cast<double*>(ws + o_sb);
  double* sbi = reinterpret_cast<double*>(ws + o_sbi);
  GemmJob* d_jobs = reinterpret_cast<GemmJob*>(ws + o_jobs);
  int8_t* a0 = reinterpret_cast<int8_t*>(ws + o_a0);
  int8_t* b0 = reinterpret_cast<int8_t*>(ws + o_b0);
  int8_t* aodd = reinterpret_cast<int8_t*>(ws + o_aodd);
  int8_t* bodd = reinterpret_cast<int8_t*>(ws + o_bodd);
  uint16_t* a_hi = reinterpret_cast<uint16_t*>(ws + o_ahi);
  uint16_t* a_oddf = reinterpret_cast<uint16_t*>(ws + o_aoddf);
  uint16_t* b_hi = reinterpret_cast<uint16_t*>(ws + o_bhi);
  uint16_t* b_oddf = reinterpret_cast<uint16_t*>(ws + o_boddf);
  int16_t* w0 = reinterpret_cast<int16_t*>(ws + o_w0);
  int8_t* wodd = reinterpret_cast<int8_t*>(ws + o_wodd);
  cudaStream_t st = g.stream;
  g.ev_valid = false;

  double log2P = 0.0;
  Oz2DeviceConsts hc;
  oz2_host_consts(n_mod, &hc, &log2P);
  B200_CHECK(launch_scan_rows(dA, M, K, amax, st));
  B200_CHECK(launch_scan_cols(dB, K, N, reinterpret_cast<unsigned long long*>(bmax), st));
  std::vector<double> ha(M), hb(N);
  B200_CHECK(cudaMemcpyAsync(ha.data(), amax, M * 8, cudaMemcpyDeviceToHost, st));
  B200_CHECK(cudaMemcpyAsync(hb.data(), bmax, N * 8, cudaMemcpyDeviceToHost, st));
  B200_CHECK(cudaStreamSynchronize(st));
  const int E = oz2_exponent(log2P, K, ha.data(), M, hb.data(), N);
  B200_CHECK(launch_scales(amax, M, E, mu, sa, sai, st));
  B200_CHECK(launch_scales(bmax, N, E, nu, sb, sbi, st));
  SplitPlanes pa{M, K, q.Kp, q.K0, q.n_chunks, n_odd, a0, a_hi, a_oddf, aodd, static_cast<long long>(a_stride)};
  SplitPlanes pb{N, K, q.Kp, q.K0, q.n_chunks, n_odd, b0, b_hi, b_oddf, bodd, static_cast<long long>(b_stride)};
  B200_CHECK(launch_split_a(dA, sa, pa, hc, st));
  B200_CHECK(launch_split_b(dB, sb, N, pb, hc, st));

  GemmJob jobs[16];
  fill_mod_job(&jobs[0], 0, 0, 0, 0);
  for (int l = 1; l < n_mod; ++l) fill_mod_job(&jobs[l], l - 1, l - 1, l - 1, kModuli[l]);
  B200_CHECK(cudaMemcpyAsync(d_jobs, jobs, sizeof(GemmJob) * n_mod, cudaMemcpyHostToDevice, st));
  GemmParams p0 = make_gemm_params();
  p0.tiles_m = q.tiles_m; p0.tiles_n = q.tiles_n; p0.n_jobs = 1;
  p0.kb_per_seg = static_cast<int>(q.K0 / kBK);
  p0.kb_per_unit = kChunkSeg / kBK;
  p0.a_hi = a_hi; p0.a_odd = a_oddf; p0.b_odd = b_oddf; p0.b_hi = b_hi;
  p0.n_chunks = q.n_chunks;
  p0.tie_bits = tie_bits + 256;
  if (tie_list_fits(q.Np, q.n_chunks) && !o.use_simt_products) {
    p0.tie_cursor = reinterpret_cast<unsigned int*>(tie_bits);
    p0.tie_list = reinterpret_cast<uint4*>(tie_bits + 256);
  }
  p0.group_m = 16;
  p0.jobs = d_jobs;
  p0.out = reinterpret_cast<uint8_t*>(w0);
  p0.out_plane_stride = 0;
  p0.ldo = static_cast<int>(q.Np);
  p0.status = g.d_status;
  p0.work_counter = g.d_status + 1;
  GemmParams p1 = p0;
  p1.n_jobs = n_odd;
  p1.kb_per_seg = static_cast<int>(q.Kp / kBK);
  p1.kb_per_unit = kOddUnitKb;
  p1.jobs = d_jobs + 1;
  p1.out = reinterpret_cast<uint8_t*>(wodd);
  p1.out_plane_stride = static_cast<long long>(w_stride);
  const int tiles = q.tiles_m * q.tiles_n;
  if (o.use_simt_products) {
    SimtPlanes s0{a0, 0, static_cast<int>(q.K0), b0, 0, static_cast<int>(q.K0), static_cast<int>(M), static_cast<int>(N)};
    SimtPlanes s1{aodd, static_cast<long long>(a_stride), static_cast<int>(q.Kp), bodd,
                  static_cast<long long>(b_stride), static_cast<int>(q.Kp), static_cast<int>(M), static_cast<int>(N)};
    B200_CHECK(launch_modgemm_simt(kEpiMod256, s0, p0, st));
    B200_CHECK(cudaMemsetAsync(flip_bits, 0, w_stride / 32 * 4, st));
    B200_CHECK(launch_modgemm_simt(kEpiModI8, s1, p1, st));
  } else {
    CUtensorMap mA0, mB0, mA1, mB1;
    if (make_plane_map(&mA0, a0, q.K0, M, 1, static_cast<long long>(M) * q.K0, kBM)) return -1;
    if (make_plane_map(&mB0, b0, q.K0, N, 1, static_cast<long long>(N) * q.K0, bn)) return -1;
    if (make_plane_map(&mA1, aodd, q.Kp, M, n_odd, static_cast<long long>(a_stride), kBM)) return -1;
    if (make_plane_map(&mB1, bodd, q.Kp, N, n_odd, static_cast<long long>(b_stride), bn)) return -1;
    if (p0.tie_cursor) B200_CHECK(cudaMemsetAsync(p0.tie_cursor, 0, sizeof(unsigned int), st));
    B200_CHECK(launch_modgemm(bn, kEpiMod256, mA0, mB0, p0, tiles, gemm_sms(), st));
    B200_CHECK(launch_tie_resolve(p0, flip_bits, static_cast<int>(M), static_cast<int>(N), st));
    B200_CHECK(launch_modgemm(bn, kEpiModI8, mA1, mB1, p1, tiles * n_odd, gemm_sms(), st));
  }
  CrtArgs ca;
  ca.w0 = w0; ca.flip = flip_bits; ca.w_odd = wodd; ca.w_odd_stride = static_cast<long long>(w_stride); ca.ldw = q.Np;
  ca.n_mod = n_mod; ca.M = M; ca.N = N;
  ca.inv_scale_a = sai; ca.inv_scale_b = sbi;
  ca.C = dC; ca.ldc = (o.ldc > 0) ? o.ldc : N;
  ca.bias_mode = o.bias ? o.bias_mode : 0; ca.bias = o.bias;
  ca.activation = o.activation;
  ca.pixels_per_image = o.pixels_per_image;
  B200_CHECK(launch_crt(ca, hc, st));
  g.launches += 10;

  State::Last& L = g.last;
  L.valid = true; L.M = M; L.K = K; L.N = N; L.Kp = q.Kp; L.K0 = q.K0; L.Mp = q.Mp; L.Np = q.Np;
  L.n_mod = n_mod; L.n_chunks = q.n_chunks; L.last_seg = q.last_seg;
  L.mu = mu; L.nu = nu; L.a0 = a0; L.aodd = aodd; L.aodd_stride = static_cast<long long>(a_stride);
  L.b0 = b0; L.bodd = bodd; L.bodd_stride = static_cast<long long>(b_stride);
  L.w0 = w0; L.wodd = wodd; L.wodd_stride = static_cast<long long>(w_stride);
  L.a_hi = a_hi; L.a_odd = a_oddf; L.b_hi = b_hi; L.b_odd = b_oddf; L.flip = flip_bits;
  return 0;
}
#undef B200_MARK

static int ozaki2_gemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                       long long N, int n_mod, const EshkolB200GemmOpts& o) {
  if (n_mod != 16 || K > kMaxPreparedK) {
    if (o.trans_a || o.trans_b) {
      fprintf(stderr, "[eshkol-b200] transposed operands beyond K = %lld are not served\n", kMaxPreparedK);
      return -1;
    }
    return ozaki2_gemm_general(dA, dB, dC, M, K, N, n_mod, o);
  }
  if (oz2_check_shape(M, K, N, 16)) return -1;
  // Optionally the two operands are prepared side by side on two streams.  Measured at 8192^3
  // it does not pay (8.70 ms against 8.60 ms one after the other: the column scan beside the
  // row scan and split runs four times longer), so it is off unless ESHKOL_B200_OVERLAP_PREP=1.
  cudaStream_t side = nullptr;
  if (g.overlap_prep && g.band_rows == 0 && make_band_lanes() == 0) {
    side = g.s_prep;
    B200_CHECK(cudaEventRecord(g.eb_start, g.stream));
    B200_CHECK(cudaStreamWaitEvent(side, g.eb_start, 0));
  }
  if (oz2_prepare_b(dB, K, N, (o.gemm_tile_n == 128) ? 128 : 256, o.trans_b != 0, nullptr, side)) return -1;
  if (side) {
    B200_CHECK(cudaEventRecord(g.eb_done, side));
    g.b_pending = g.eb_done;
  }
  const int rc = oz2_gemm_rows(dA, dC, M, o, true);
  if (g.b_pending) {  // the multiplication never ran: order the stream behind the side stream all the same
    cudaStreamWaitEvent(g.stream, g.b_pending, 0);
    g.b_pending = nullptr;
  }
  g.prep.valid = false;  // dB belongs to the caller and may change before the next call
  return rc;
}

// Exact tier with the right-hand operand given as an im2col view of an NCHW tensor (conv2d):
// the view is scanned and split directly, no K x N matrix of doubles exists.
int ozaki2_exact_gemm_im2col(const double* dA, const Im2colView& view, double* dC, long long M, long long K,
                             long long N, const EshkolB200GemmOpts& o) {
  if (oz2_check_shape(M, K, N, 16)) return -1;
  if (oz2_prepare_b(nullptr, K, N, (o.gemm_tile_n == 128) ? 128 : 256, false, &view)) return -1;
  const int rc = oz2_gemm_rows(dA, dC, M, o, true);
  g.prep.valid = false;
  return rc;
}

// Host-pointer product, pipelined over row blocks of A: B is uploaded and prepared
// once; then block i+1 of A crosses PCIe while block i is multiplied and block i-1 of
// C travels back.  Three streams (upload, compute = the library stream, download) and
// double-buffered device blocks.  Pinned host memory overlaps fully; pageable memory
// is staged by the runtime and still produces the same bits.
// rs (optional): full-size device copies of the three matrices that the caller keeps across
// calls.  a_state 0: hA is uploaded into rs->dA block by block; 1: rs->dA already holds A.
// b_state 0: hB is uploaded into rs->dB and prepared; 1: rs->dB already holds B, which is
// prepared from there; 2: the library's prepared right-hand operand is this B (the caller
// compared the token), nothing is uploaded or split.  rs->dC receives the whole result, which
// is also downloaded.  The prepared operand stays valid afterwards.
struct ResidentSet {
  double* dA; int a_state;
  double* dB; int b_state;
  double* dC;
};

static int oz2_matmul_host(const double* hA, const double* hB, double* hC, long long M, long long K,
                           long long N, const EshkolB200GemmOpts& o, const ResidentSet* rs = nullptr) {
  if (oz2_check_shape(M, K, N, 16)) return -1;
  long long bm = 1024;
  if (M <= 2048) bm = M;  // too small to be worth splitting
  // Row blocks: a short ramp (256, 256, 512 rows: the first rows of C start their way back after
  // a quarter of a block's upload and products, and the download is the stream everything else
  // has to hide behind), whole blocks of bm rows, then a taper (half of what is left, rounded to
  // a tile, until at most 256 rows remain) so that what is still to do once the last byte of A
  // has crossed the link -- one block's products and its way back -- is a small block.
  long long blk_r0[280], blk_rows[280];
  int nblk = 0;
  {
    if (M / bm > 250) bm = round_up((M + 249) / 250, 256);
    long long r0 = 0;
    if (M > 4096 && bm >= 1024) {
      const long long ramp[3] = {256, 256, 512};
      for (long long w : ramp) { blk_r0[nblk] = r0; blk_rows[nblk++] = w; r0 += w; }
    }
    while (M - r0 > bm) { blk_r0[nblk] = r0; blk_rows[nblk++] = bm; r0 += bm; }
    long long left = M - r0;
    while (M > 2048 && left > 256) {
      const long long t = round_up(left / 2, kBM);
      blk_r0[nblk] = r0; blk_rows[nblk++] = t; r0 += t; left -= t;
    }
    if (left > 0) { blk_r0[nblk] = r0; blk_rows[nblk++] = left; }
  }
  const size_t bytesB = static_cast<size_t>(K) * N * 8;
  const size_t bytesA = static_cast<size_t>(bm) * K * 8, bytesC = static_cast<size_t>(bm) * N * 8;
  double* dB = nullptr;
  double* dA[2] = {nullptr, nullptr};
  double* dC[2] = {nullptr, nullptr};
  if (rs) {
    dB = rs->dB;
  } else {
    const size_t need = ((bytesB + 1023) & ~size_t(1023)) + 2 * ((bytesA + 1023) & ~size_t(1023)) +
                        2 * ((bytesC + 1023) & ~size_t(1023));
    uint8_t* base = aux_reserve(need);
    if (!base) return -1;
    dB = reinterpret_cast<double*>(base);
    size_t off = (bytesB + 1023) & ~size_t(1023);
    for (int i = 0; i < 2; ++i) { dA[i] = reinterpret_cast<double*>(base + off); off += (bytesA + 1023) & ~size_t(1023); }
    for (int i = 0; i < 2; ++i) { dC[i] = reinterpret_cast<double*>(base + off); off += (bytesC + 1023) & ~size_t(1023); }
  }
  if (!g.pipe_made) {
    B200_CHECK(cudaStreamCreateWithFlags(&g.s_in, cudaStreamNonBlocking));
    B200_CHECK(cudaStreamCreateWithFlags(&g.s_out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      B200_CHECK(cudaEventCreateWithFlags(&g.e_a_ready[i], cudaEventDisableTiming));
      B200_CHECK(cudaEventCreateWithFlags(&g.e_a_free[i], cudaEventDisableTiming));
      B200_CHECK(cudaEventCreateWithFlags(&g.e_c_ready[i], cudaEventDisableTiming));
      B200_CHECK(cudaEventCreateWithFlags(&g.e_c_free[i], cudaEventDisableTiming));
    }
    B200_CHECK(cudaEventCreateWithFlags(&g.e_b_ready, cudaEventDisableTiming));
    g.pipe_made = true;
  }
  cudaStream_t st = g.stream;
  const int b_state = rs ? rs->b_state : 0;
  const bool a_resident = rs && rs->a_state == 1;
  // earlier work on the compute stream may still read the buffers written below
  B200_CHECK(cudaEventRecord(g.e_b_ready, st));
  B200_CHECK(cudaStreamWaitEvent(g.s_in, g.e_b_ready, 0));
  B200_CHECK(cudaStreamWaitEvent(g.s_out, g.e_b_ready, 0));
  if (b_state == 0) {
    B200_CHECK(staged_upload(dB, hB, bytesB, g.s_in));
    g.h2d_bytes += bytesB;
    B200_CHECK(cudaEventRecord(g.e_b_ready, g.s_in));
    // the first block of A rides behind B on the upload stream
    B200_CHECK(cudaStreamWaitEvent(st, g.e_b_ready, 0));
  }
  if (b_state == 2) {
    if (!g.prep.valid || g.prep.K != K || g.prep.N != N) {
      fprintf(stderr, "[eshkol-b200] the prepared right-hand operand is not the one the caller expects\n");
      return -1;
    }
  } else if (oz2_prepare_b(dB, K, N, (o.gemm_tile_n == 128) ? 128 : 256)) {
    return -1;
  }
  int rc = 0;
  for (int i = 0; i < nblk && rc == 0; ++i) {
    const int s = i & 1;
    const long long r0 = blk_r0[i], rows = blk_rows[i];
    double* a_blk = rs ? rs->dA + r0 * K : dA[s];
    double* c_blk = rs ? rs->dC + r0 * N : dC[s];
    if (!a_resident) {
      if (i >= 2 && !rs) B200_CHECK(cudaStreamWaitEvent(g.s_in, g.e_a_free[s], 0));
      B200_CHECK(staged_upload(a_blk, hA + r0 * K, static_cast<size_t>(rows) * K * 8, g.s_in));
      g.h2d_bytes += static_cast<size_t>(rows) * K * 8;
      B200_CHECK(cudaEventRecord(g.e_a_ready[s], g.s_in));
      B200_CHECK(cudaStreamWaitEvent(st, g.e_a_ready[s], 0));
    }
    if (i >= 2 && !rs) B200_CHECK(cudaStreamWaitEvent(st, g.e_c_free[s], 0));
    rc = oz2_gemm_rows(a_blk, c_blk, rows, o, false);
    if (rc) break;
    B200_CHECK(cudaEventRecord(g.e_a_free[s], st));
    B200_CHECK(cudaEventRecord(g.e_c_ready[s], st));
    B200_CHECK(cudaStreamWaitEvent(g.s_out, g.e_c_ready[s], 0));
    B200_CHECK(staged_download(hC + r0 * N, c_blk, static_cast<size_t>(rows) * N * 8, g.s_out));
    g.d2h_bytes += static_cast<size_t>(rows) * N * 8;
    B200_CHECK(cudaEventRecord(g.e_c_free[s], g.s_out));
  }
  if (!rs) g.prep.valid = false;  // the staging copy of B is overwritten by the next call
  B200_CHECK(staged_finish(g.s_out));
  B200_CHECK(cudaStreamSynchronize(g.s_out));
  B200_CHECK(cudaStreamSynchronize(g.s_in));
  return rc;
}

}  // namespace b200

using namespace b200;

extern "C" {

int eshkol_b200_init(int device) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g.ready) return 0;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { cudaGetLastError(); return -1; }
  if (device < 0 || device >= count) return -1;
  B200_CHECK(cudaSetDevice(device));
  cudaDeviceProp prop;
  B200_CHECK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    fprintf(stderr, "[eshkol-b200] device %d is sm_%d%d; this library carries sm_100a code only\n",
            device, prop.major, prop.minor);
    return -1;
  }
  g.device = device;
  g.num_sms = prop.multiProcessorCount;
  {
    int least = 0, greatest = 0;
    B200_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    const char* pe = getenv("ESHKOL_B200_STREAM_PRIORITY");  // "default": do not raise the library stream
    const bool raise = !(pe && !strcmp(pe, "default"));
    B200_CHECK(cudaStreamCreateWithPriority(&g.stream, cudaStreamNonBlocking, raise ? greatest : least));
  }
  B200_CHECK(cudaEventCreate(&g.ev_g0));
  B200_CHECK(cudaEventCreate(&g.ev_g1));
  // [0] kernel status word, [1] work counter of the persistent products kernel
  B200_CHECK(cudaMalloc(&g.d_status, 2 * sizeof(int)));
  B200_CHECK(cudaMemset(g.d_status, 0, 2 * sizeof(int)));
  {
    GemmJob jobs[16];
    fill_mod_job(&jobs[0], 0, 0, 0, 0);
    for (int l = 1; l < 16; ++l) fill_mod_job(&jobs[l], l - 1, l - 1, l - 1, kModuli[l]);
    B200_CHECK(cudaMalloc(&g.d_jobs16, sizeof(jobs)));
    B200_CHECK(cudaMemcpy(g.d_jobs16, jobs, sizeof(jobs), cudaMemcpyHostToDevice));
  }
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  B200_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess) {
    fprintf(stderr, "[eshkol-b200] cuTensorMapEncodeTiled is not available from this driver\n");
    return -1;
  }
  g.encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  B200_CHECK(modgemm_set_attributes());
  B200_CHECK(modgemm2_set_attributes());
  {
    const char* e = getenv("ESHKOL_B200_PAIR_GEMM");
    g.pair_gemm = e && e[0] == '1';
    e = getenv("ESHKOL_B200_OVERLAP_PREP");
    g.overlap_prep = e && e[0] == '1';
    e = getenv("ESHKOL_B200_BAND_ROWS");
    if (e && e[0]) eshkol_b200_set_row_bands(atoll(e));
  }
  B200_CHECK(split_set_attributes());
  B200_CHECK(tiers_set_attributes());
  // the allocation-free entry point's scratch array: its module is loaded and its address
  // resolved here, so that entry point itself never causes a load or an allocation
  if (static_scratch_setup(device) != 0) return -1;
  g.ready = true;
  return 0;
}

void eshkol_b200_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g.ready) return;
  cudaStreamSynchronize(g.stream);
  staged_shutdown();
  if (g.ws) cudaFree(g.ws);
  if (g.aux) cudaFree(g.aux);
  if (g.tbuf) cudaFree(g.tbuf);
  if (g.d_status) cudaFree(g.d_status);
  if (g.ev_g0) cudaEventDestroy(g.ev_g0);
  if (g.ev_g1) cudaEventDestroy(g.ev_g1);
  if (g.ev_made) {
    for (int r = 0; r < State::kEvRing; ++r) {
      for (cudaEvent_t e : g.ev_b[r]) cudaEventDestroy(e);
      for (cudaEvent_t e : g.ev_a[r]) cudaEventDestroy(e);
      for (cudaEvent_t e : g.ev_m[r]) cudaEventDestroy(e);
    }
    cudaEventDestroy(g.ev_scratch);
  }
  if (g.ev_band_made) for (cudaEvent_t e : g.ev_band) cudaEventDestroy(e);
  if (g.d_jobs16) cudaFree(g.d_jobs16);
  if (g.lanes_made) {
    cudaStreamSynchronize(g.s_prep); cudaStreamSynchronize(g.s_post);
    cudaStreamDestroy(g.s_prep); cudaStreamDestroy(g.s_post);
    cudaEventDestroy(g.eb_start); cudaEventDestroy(g.eb_done);
    for (int i = 0; i < 2; ++i) {
      cudaEventDestroy(g.eb_a_ready[i]); cudaEventDestroy(g.eb_g0[i]);
      cudaEventDestroy(g.eb_g1[i]); cudaEventDestroy(g.eb_w_free[i]);
    }
  }
  if (g.bside) cudaFree(g.bside);
  if (g.pipe_made) {
    cudaStreamDestroy(g.s_in); cudaStreamDestroy(g.s_out); cudaEventDestroy(g.e_b_ready);
    for (int i = 0; i < 2; ++i) {
      cudaEventDestroy(g.e_a_ready[i]); cudaEventDestroy(g.e_a_free[i]);
      cudaEventDestroy(g.e_c_ready[i]); cudaEventDestroy(g.e_c_free[i]);
    }
  }
  cudaStreamDestroy(g.stream);
  g = State();
}

void* eshkol_b200_stream(void) { return g.ready ? static_cast<void*>(g.stream) : nullptr; }

int eshkol_b200_gemm_f64_device(const double* dA, const double* dB, double* dC, uint64_t M,
                                uint64_t K, uint64_t N, const EshkolB200GemmOpts* opts) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] gemm called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!dA || !dB || !dC || M == 0 || K == 0 || N == 0) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) o = *opts;
  const long long m = static_cast<long long>(M), k = static_cast<long long>(K), n = static_cast<long long>(N);
  if ((o.trans_a || o.trans_b) &&
      !(o.tier == ESHKOL_B200_TIER_OZAKI2 && (o.param == 0 || o.param == 16) && !o.use_simt_products &&
        k <= kMaxPreparedK)) {
    // only the 16-moduli exact tier reads transposed storage directly
    const size_t ba = o.trans_a ? ((static_cast<size_t>(m) * k * 8 + 1023) & ~size_t(1023)) : 0;
    const size_t bb = o.trans_b ? static_cast<size_t>(k) * n * 8 : 0;
    uint8_t* t = tbuf_reserve(ba + bb);
    if (!t) return -1;
    if (o.trans_a) {
      B200_CHECK(launch_transpose(dA, k, m, reinterpret_cast<double*>(t), g.stream));
      dA = reinterpret_cast<const double*>(t);
    }
    if (o.trans_b) {
      B200_CHECK(launch_transpose(dB, n, k, reinterpret_cast<double*>(t + ba), g.stream));
      dB = reinterpret_cast<const double*>(t + ba);
    }
    g.launches += (o.trans_a ? 1 : 0) + (o.trans_b ? 1 : 0);
    o.trans_a = o.trans_b = 0;
  }
  g.ev_g_valid = false;
  if (g.ev_g0) B200_CHECK(cudaEventRecord(g.ev_g0, g.stream));
  int rc;
  switch (o.tier) {
    case ESHKOL_B200_TIER_OZAKI2:
      rc = ozaki2_gemm(dA, dB, dC, m, k, n, o.param ? o.param : 16, o);
      break;
    case ESHKOL_B200_TIER_OZAKI1:
      rc = ozaki1_gemm(dA, dB, dC, m, k, n, o.param ? o.param : 6, o);
      break;
    case ESHKOL_B200_TIER_OZAKI2_FAST:
      rc = ozaki2_fast_gemm(dA, dB, dC, m, k, n, o.param ? o.param : 11, o);
      break;
    case ESHKOL_B200_TIER_DGEMM:
      rc = native_dgemm(dA, dB, dC, m, k, n, o);
      break;
    default:
      fprintf(stderr, "[eshkol-b200] unknown tier %d\n", o.tier);
      return -1;
  }
  if (rc == 0 && g.ev_g1) {
    B200_CHECK(cudaEventRecord(g.ev_g1, g.stream));
    g.ev_g_valid = true;
  }
  return rc;
}

double eshkol_b200_last_gemm_ms(void) {
  if (!g.ready || !g.ev_g_valid) return -1.0;
  float ms = 0.f;
  if (cudaEventSynchronize(g.ev_g1) != cudaSuccess || cudaEventElapsedTime(&ms, g.ev_g0, g.ev_g1) != cudaSuccess) {
    cudaGetLastError();
    return -1.0;
  }
  return static_cast<double>(ms);
}

int eshkol_b200_matmul_f64_host(const double* hA, const double* hB, double* hC, uint64_t M,
                                uint64_t K, uint64_t N, const EshkolB200GemmOpts* opts) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] matmul called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!hA || !hB || !hC || M == 0 || K == 0 || N == 0) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) o = *opts;
  if (o.tier != ESHKOL_B200_TIER_OZAKI2 || (o.param != 0 && o.param != 16) || K > static_cast<uint64_t>(kMaxPreparedK)) return -2;
  return oz2_matmul_host(hA, hB, hC, static_cast<long long>(M), static_cast<long long>(K),
                         static_cast<long long>(N), o);
}

int eshkol_b200_feed_forward_f64_device(const double* d_x, const double* d_w1, const double* d_b1,
                                        const double* d_w2, const double* d_b2, double* d_out,
                                        uint64_t rows, uint64_t d_model, uint64_t d_ff,
                                        const EshkolB200GemmOpts* opts) {
  if (!g.ready || !d_x || !d_w1 || !d_w2 || !d_out || rows == 0 || d_model == 0 || d_ff == 0) return -1;
  uint8_t* hid = aux_reserve(static_cast<size_t>(rows) * d_ff * 8);
  if (!hid) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) { o.tier = opts->tier; o.param = opts->param; }
  EshkolB200GemmOpts o1 = o;
  o1.activation = 2;
  o1.bias = d_b1; o1.bias_mode = d_b1 ? 2 : 0;
  if (eshkol_b200_gemm_f64_device(d_x, d_w1, reinterpret_cast<double*>(hid), rows, d_model, d_ff, &o1) != 0) return -1;
  EshkolB200GemmOpts o2 = o;
  o2.bias = d_b2; o2.bias_mode = d_b2 ? 2 : 0;
  return eshkol_b200_gemm_f64_device(reinterpret_cast<const double*>(hid), d_w2, d_out, rows, d_ff, d_model, &o2);
}

int eshkol_b200_conv2d_backward_kernel_f64_device(const double* d_grad_out, const double* d_input,
                                                  double* d_grad_kernel, uint64_t in_h, uint64_t in_w,
                                                  uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
                                                  uint64_t stride_h, uint64_t stride_w, uint64_t channels_in,
                                                  uint64_t channels_out, uint64_t batch,
                                                  const EshkolB200GemmOpts* opts) {
  if (!g.ready || !d_grad_out || !d_input || !d_grad_kernel) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) { o.tier = opts->tier; o.param = opts->param; }
  return conv2d_backward_kernel(d_grad_out, d_input, d_grad_kernel, in_h, in_w, k_h, k_w, out_h, out_w, stride_h,
                                stride_w, channels_in, channels_out, batch, o);
}

int eshkol_b200_conv2d_backward_input_f64_device(const double* d_grad_out, const double* d_weights,
                                                 double* d_grad_input, uint64_t in_h, uint64_t in_w,
                                                 uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
                                                 uint64_t stride_h, uint64_t stride_w, uint64_t channels_in,
                                                 uint64_t channels_out, uint64_t batch,
                                                 const EshkolB200GemmOpts* opts) {
  if (!g.ready || !d_grad_out || !d_weights || !d_grad_input) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) { o.tier = opts->tier; o.param = opts->param; }
  return conv2d_backward_input(d_grad_out, d_weights, d_grad_input, in_h, in_w, k_h, k_w, out_h, out_w, stride_h,
                               stride_w, channels_in, channels_out, batch, o);
}

int eshkol_b200_gemm_f16_device(const double* dA, const double* dB, double* dC, uint64_t batch,
                                uint64_t M, uint64_t K, uint64_t N) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] gemm called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!dA || !dB || !dC) return -1;
  g.last.valid = false;
  g.prepA.valid = false;
  return f16_gemm(dA, dB, dC, static_cast<long long>(batch), static_cast<long long>(M),
                  static_cast<long long>(K), static_cast<long long>(N));
}

int eshkol_b200_gemm_f32_device(const float* dA, const float* dB, float* dC, uint64_t M, uint64_t K,
                                uint64_t N) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] gemm called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!dA || !dB || !dC) return -1;
  return f32_gemm(dA, dB, dC, static_cast<long long>(M), static_cast<long long>(K), static_cast<long long>(N));
}

int eshkol_b200_matmul_backward_f64_host(const double* grad_out, const double* A, const double* B,
                                         double* grad_A, double* grad_B, uint64_t M, uint64_t K,
                                         uint64_t N, const EshkolB200GemmOpts* opts_grad_a,
                                         const EshkolB200GemmOpts* opts_grad_b) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] matmul backward called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!grad_out || !A || !B || !grad_A || !grad_B || M == 0 || K == 0 || N == 0) return -1;
  EshkolB200GemmOpts oa, ob;
  memset(&oa, 0, sizeof(oa));
  memset(&ob, 0, sizeof(ob));
  if (opts_grad_a) { oa.tier = opts_grad_a->tier; oa.param = opts_grad_a->param; }
  if (opts_grad_b) { ob.tier = opts_grad_b->tier; ob.param = opts_grad_b->param; }
  const size_t bg = (M * N * 8 + 1023) & ~size_t(1023), ba = (M * K * 8 + 1023) & ~size_t(1023),
               bb = (K * N * 8 + 1023) & ~size_t(1023);
  uint8_t* base = aux_reserve(bg + 2 * ba + 2 * bb);
  if (!base) return -1;
  double* dG = reinterpret_cast<double*>(base);
  double* dA = reinterpret_cast<double*>(base + bg);
  double* dB = reinterpret_cast<double*>(base + bg + ba);
  double* dGA = reinterpret_cast<double*>(base + bg + ba + bb);
  double* dGB = reinterpret_cast<double*>(base + bg + 2 * ba + bb);
  cudaStream_t st = g.stream;
  B200_CHECK(cudaMemcpyAsync(dG, grad_out, M * N * 8, cudaMemcpyHostToDevice, st));
  B200_CHECK(cudaMemcpyAsync(dB, B, K * N * 8, cudaMemcpyHostToDevice, st));
  // grad_A[M x K] = G[M x N] * B^T: inner dimension N, B stored (columns of the operand) x (inner)
  oa.trans_a = 0; oa.trans_b = 1;
  if (eshkol_b200_gemm_f64_device(dG, dB, dGA, M, N, K, &oa) != 0) return -1;
  B200_CHECK(cudaMemcpyAsync(grad_A, dGA, M * K * 8, cudaMemcpyDeviceToHost, st));
  B200_CHECK(cudaMemcpyAsync(dA, A, M * K * 8, cudaMemcpyHostToDevice, st));
  // grad_B[K x N] = A^T * G: inner dimension M, A stored (inner) x (rows of the operand)
  ob.trans_a = 1; ob.trans_b = 0;
  if (eshkol_b200_gemm_f64_device(dA, dG, dGB, K, M, N, &ob) != 0) return -1;
  B200_CHECK(cudaMemcpyAsync(grad_B, dGB, K * N * 8, cudaMemcpyDeviceToHost, st));
  B200_CHECK(cudaStreamSynchronize(st));
  return 0;
}

int eshkol_b200_prepare_b_f64_device(const double* dB, uint64_t K, uint64_t N) {
  if (!g.ready || !dB || K == 0 || N == 0) return -1;
  return oz2_prepare_b(dB, static_cast<long long>(K), static_cast<long long>(N), 256);
}

uint64_t eshkol_b200_prepared_b_bytes(uint64_t K, uint64_t N) {
  if (K == 0 || N == 0) return 0;
  return oz2_b_layout(oz2_geometry(1, static_cast<long long>(K), static_cast<long long>(N), 256), 0).total;
}

int eshkol_b200_prepare_b_columns_f64_device(const double* dB, uint64_t ldb, uint64_t K, uint64_t N, uint64_t col0,
                                             uint64_t ncols, void* planes) {
  if (!g.ready || !dB || !planes) return -1;
  return oz2_prepare_b_columns(dB, static_cast<long long>(ldb), static_cast<long long>(K), static_cast<long long>(N),
                               static_cast<long long>(col0), static_cast<long long>(ncols),
                               static_cast<uint8_t*>(planes));
}

int eshkol_b200_prepared_b_regions(uint64_t K_, uint64_t N_, uint64_t col0, uint64_t ncols, uint64_t out[7][4]) {
  if (!out || K_ == 0 || N_ == 0 || ncols == 0 || col0 + ncols > N_) return -1;
  const Oz2Geom q = oz2_geometry(1, static_cast<long long>(K_), static_cast<long long>(N_), 256);
  const BLayout L = oz2_b_layout(q, 0);
  const uint64_t c0 = col0, n = ncols;
  const uint64_t rows[7][4] = {
      {L.nu + c0 * 4, n * 4, 1, n * 4},
      {L.sb + c0 * 8, n * 8, 1, n * 8},
      {L.sbi + c0 * 8, n * 8, 1, n * 8},
      {L.b0 + c0 * static_cast<uint64_t>(q.K0), n * static_cast<uint64_t>(q.K0), 1, n * static_cast<uint64_t>(q.K0)},
      {L.bhi + c0 * L.flag_row_bytes, n * L.flag_row_bytes, 1, n * L.flag_row_bytes},
      {L.boddf + c0 * L.flag_row_bytes, n * L.flag_row_bytes, 1, n * L.flag_row_bytes},
      {L.bodd + c0 * static_cast<uint64_t>(q.Kp), n * static_cast<uint64_t>(q.Kp), 15, L.b_stride}};
  memcpy(out, rows, sizeof(rows));
  return 7;
}

int eshkol_b200_adopt_prepared_b(void* planes, uint64_t K, uint64_t N) {
  if (!g.ready || !planes || K == 0 || N == 0) return -1;
  const long long k = static_cast<long long>(K), n = static_cast<long long>(N);
  if (oz2_check_shape(1, k, n, 16) || k > kMaxPreparedK) return -1;
  const Oz2Geom q = oz2_geometry(1, k, n, 256);
  g.prep.valid = false;
  oz2_bind_b(static_cast<uint8_t*>(planes), q, oz2_b_layout(q, 0), 256);
  if (oz2_b_maps(q, 256)) return -1;
  g.prep.valid = true;
  ++g.prep_token;
  return 0;
}

int eshkol_b200_prepare_a_f64_device(const double* dA, uint64_t M, uint64_t K, uint64_t n_cols_hint) {
  if (!g.ready || !dA || M == 0 || K == 0 || n_cols_hint == 0) return -1;
  return oz2_prepare_a(dA, static_cast<long long>(M), static_cast<long long>(K),
                       static_cast<long long>(n_cols_hint), 256);
}

int eshkol_b200_multiply_prepared_f64_device(double* dC, const EshkolB200GemmOpts* opts) {
  if (!g.ready || !dC) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) o = *opts;
  return oz2_multiply(dC, o);
}

int eshkol_b200_gemm_prepared_f64_device(const double* dA, double* dC, uint64_t M,
                                         const EshkolB200GemmOpts* opts) {
  if (!g.ready || !dA || !dC || M == 0) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) o = *opts;
  return oz2_gemm_rows(dA, dC, static_cast<long long>(M), o, true);
}

int eshkol_b200_conv2d_f64_device(const double* d_in, int64_t batch, int64_t in_c, int64_t H,
                                  int64_t W, const double* d_ker, int64_t out_c, int64_t kH,
                                  int64_t kW, int64_t stride, int64_t pad, double* d_out,
                                  const EshkolB200GemmOpts* opts) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] conv2d called before eshkol_b200_init succeeded\n");
    return -1;
  }
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  if (opts) o = *opts;
  return conv2d_lowered(d_in, batch, in_c, H, W, d_ker, out_c, kH, kW, stride, pad, d_out, o);
}

int eshkol_b200_mem_alloc(int kind, size_t bytes, void** out_ptr) {
  if (!g.ready || !out_ptr || bytes == 0) return -1;
  cudaError_t e;
  switch (kind) {
    case 0: e = lib_malloc(out_ptr, bytes); break;
    case 1: e = cudaMallocManaged(out_ptr, bytes); break;
    case 2: e = cudaMallocHost(out_ptr, bytes); break;
    default: return -1;
  }
  if (e != cudaSuccess) { cudaGetLastError(); *out_ptr = nullptr; return -1; }
  return 0;
}

void eshkol_b200_mem_free(int kind, void* ptr) {
  if (!g.ready || !ptr) return;
  cudaStreamSynchronize(g.stream);
  if (kind == 2) cudaFreeHost(ptr); else cudaFree(ptr);
}

int eshkol_b200_copy_h2d(void* device_dst, const void* host_src, size_t bytes) {
  if (!g.ready) return -1;
  B200_CHECK(staged_upload(device_dst, host_src, bytes, g.stream));
  g.h2d_bytes += bytes;
  return 0;
}

int eshkol_b200_copy_d2h(void* host_dst, const void* device_src, size_t bytes) {
  if (!g.ready) return -1;
  B200_CHECK(staged_download(host_dst, device_src, bytes, g.stream));
  g.d2h_bytes += bytes;
  return 0;
}

void eshkol_b200_transfer_bytes(uint64_t* h2d, uint64_t* d2h) {
  if (h2d) *h2d = g.h2d_bytes;
  if (d2h) *d2h = g.d2h_bytes;
}

uint64_t eshkol_b200_prepared_b_token(void) { return (g.ready && g.prep.valid) ? g.prep_token : 0; }

int eshkol_b200_matmul_f64_host_resident(const double* hA, const double* hB, double* hC, uint64_t M,
                                         uint64_t K, uint64_t N, double* dA, int a_state, double* dB,
                                         int b_state, double* dC, uint64_t* prepared_token) {
  if (!g.ready) {
    fprintf(stderr, "[eshkol-b200] matmul called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!hC || !dA || !dB || !dC || M == 0 || K == 0 || N == 0) return -1;
  if ((a_state == 0 && !hA) || (b_state == 0 && !hB) || a_state < 0 || a_state > 1 || b_state < 0 || b_state > 2) return -1;
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  ResidentSet rs{dA, a_state, dB, b_state, dC};
  const int rc = oz2_matmul_host(hA, hB, hC, static_cast<long long>(M), static_cast<long long>(K),
                                 static_cast<long long>(N), o, &rs);
  if (prepared_token) *prepared_token = (rc == 0 && g.prep.valid) ? g.prep_token : 0;
  return rc;
}

int eshkol_b200_elementwise_f64_device(const double* a, const double* b, double* out,
                                       uint64_t n, int op) {
  if (!g.ready || !a || !out || n == 0 || op < 0 || op > 14) return -1;
  B200_CHECK(launch_elementwise(a, b, out, static_cast<long long>(n), op, g.stream));
  g.launches += 1;
  return 0;
}

int eshkol_b200_sync_status(void) {
  if (!g.ready) return -1;
  if (staged_finish(g.stream) != cudaSuccess) {
    fprintf(stderr, "[eshkol-b200] a staged download failed: %s\n", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  int h = 0;
  if (cudaMemcpyAsync(&h, g.d_status, sizeof(int), cudaMemcpyDeviceToHost, g.stream) != cudaSuccess ||
      cudaStreamSynchronize(g.stream) != cudaSuccess) {
    fprintf(stderr, "[eshkol-b200] stream failed: %s\n", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (h != 0) {
    fprintf(stderr, "[eshkol-b200] a kernel gave up a bounded wait (status %d)\n", h);
    cudaMemsetAsync(g.d_status, 0, sizeof(int), g.stream);
    cudaStreamSynchronize(g.stream);
  }
  return h;
}

void eshkol_b200_set_pair_gemm(int on) { g.pair_gemm = on != 0; }

int eshkol_b200_enable_peer_access(int peer_device) {
  if (!g.ready) return -1;
  if (peer_device == g.device) return 0;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, g.device, peer_device) != cudaSuccess || !can) { cudaGetLastError(); return -1; }
  B200_CHECK(cudaSetDevice(g.device));
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
    fprintf(stderr, "[eshkol-b200] peer access to device %d: %s\n", peer_device, cudaGetErrorString(e));
    cudaGetLastError();
    return -1;
  }
  cudaGetLastError();
  return 0;
}

int eshkol_b200_copy_async(void* dst, const void* src, size_t bytes, void* stream) {
  if (!g.ready || !dst || !src) return -1;
  if (bytes == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, st));
  return 0;
}

// ---- interprocess handles (one process per GPU): memory and events of a peer rank ----
int eshkol_b200_ipc_export_mem(void* device_ptr, unsigned char handle[64]) {
  if (!g.ready || !device_ptr || !handle) return -1;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  B200_CHECK(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle, &h, 64);
  return 0;
}

int eshkol_b200_ipc_import_mem(const unsigned char handle[64], void** device_ptr) {
  if (!g.ready || !device_ptr || !handle) return -1;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  B200_CHECK(cudaSetDevice(g.device));
  // opened in this rank's own context; peer access to the owning device is enabled on demand
  B200_CHECK(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

int eshkol_b200_ipc_close_mem(void* device_ptr) {
  if (!g.ready || !device_ptr) return -1;
  B200_CHECK(cudaIpcCloseMemHandle(device_ptr));
  return 0;
}

int eshkol_b200_ipc_event_create(void** event, unsigned char handle[64]) {
  if (!g.ready || !event || !handle) return -1;
  static_assert(sizeof(cudaIpcEventHandle_t) == 64, "handle size");
  cudaEvent_t ev = nullptr;
  B200_CHECK(cudaSetDevice(g.device));
  B200_CHECK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming | cudaEventInterprocess));
  cudaIpcEventHandle_t h;
  B200_CHECK(cudaIpcGetEventHandle(&h, ev));
  memcpy(handle, &h, 64);
  *event = ev;
  return 0;
}

int eshkol_b200_ipc_event_import(const unsigned char handle[64], void** event) {
  if (!g.ready || !event || !handle) return -1;
  cudaIpcEventHandle_t h;
  memcpy(&h, handle, 64);
  cudaEvent_t ev = nullptr;
  B200_CHECK(cudaSetDevice(g.device));
  B200_CHECK(cudaIpcOpenEventHandle(&ev, h));
  *event = ev;
  return 0;
}

int eshkol_b200_event_record(void* event, void* stream) {
  if (!g.ready || !event) return -1;
  B200_CHECK(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)));
  return 0;
}

int eshkol_b200_event_wait(void* event, void* stream) {
  if (!g.ready || !event) return -1;
  B200_CHECK(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream),
                                 static_cast<cudaEvent_t>(event), 0));
  return 0;
}

int eshkol_b200_event_destroy(void* event) {
  if (!g.ready || !event) return -1;
  B200_CHECK(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
  return 0;
}

int eshkol_b200_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                             size_t width_bytes, size_t rows, void* stream) {
  if (!g.ready || !dst || !src) return -1;
  if (width_bytes == 0 || rows == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  B200_CHECK(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault, st));
  return 0;
}

void eshkol_b200_set_sm_limit(int sms) { g.sm_limit = sms > 0 ? sms : 0; }

void eshkol_b200_set_row_bands(long long rows) {
  // whole pair tiles (256 rows); 0 switches the band pipeline off
  g.band_rows = rows <= 0 ? 0 : (rows + 255) / 256 * 256;
}

void eshkol_b200_set_phase_timing(int on) {
  if (!g.ready) return;
  if (on && !g.ev_made) {
    for (int r = 0; r < State::kEvRing; ++r) {
      for (cudaEvent_t& e : g.ev_b[r]) if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
      for (cudaEvent_t& e : g.ev_a[r]) if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
      for (cudaEvent_t& e : g.ev_m[r]) if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
    }
    if (cudaEventCreate(&g.ev_scratch) != cudaSuccess) { cudaGetLastError(); return; }
    g.ev_made = true;
  }
  if (on && !g.ev_band_made) {
    for (cudaEvent_t& e : g.ev_band)
      if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); return; }
    g.ev_band_made = true;
  }
  g.timing = on != 0;
  g.ev_valid = false;
  g.n_evb = g.n_eva = g.n_evm = 0;
}

// stage durations of ring entry `idx` of each group
static int phase_entry(unsigned long long ib, unsigned long long ia, unsigned long long im, float* ms,
                       bool with_a_and_m) {
  const cudaEvent_t* b = g.ev_b[ib % State::kEvRing];
  if (cudaEventElapsedTime(&ms[0], b[0], b[1]) != cudaSuccess || cudaEventElapsedTime(&ms[1], b[1], b[2]) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  if (!with_a_and_m) return 0;
  const cudaEvent_t* a = g.ev_a[ia % State::kEvRing];
  const cudaEvent_t* m = g.ev_m[im % State::kEvRing];
  if (cudaEventElapsedTime(&ms[2], a[0], a[1]) != cudaSuccess || cudaEventElapsedTime(&ms[3], a[1], a[2]) != cudaSuccess ||
      cudaEventElapsedTime(&ms[4], m[0], m[1]) != cudaSuccess || cudaEventElapsedTime(&ms[5], m[1], m[2]) != cudaSuccess ||
      cudaEventElapsedTime(&ms[6], m[2], m[3]) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return 0;
}

int eshkol_b200_get_phase_times(float* ms, int capacity) {
  if (!g.ready || !ms || capacity < 7 || !g.ev_valid || g.n_evb == 0) return -1;
  if (cudaStreamSynchronize(g.stream) != cudaSuccess) { cudaGetLastError(); return -1; }
  const bool banded = g.bands_timed > 0;
  if (!banded && (g.n_eva == 0 || g.n_evm == 0)) return -1;
  if (phase_entry(g.n_evb - 1, g.n_eva - 1, g.n_evm - 1, ms, !banded) != 0) return -1;
  if (banded) {
    // band pipeline: each stage is the sum over the bands of its own kernels' time on its own
    // stream; the stages overlap, so they add up to more than the product took
    for (int i = 2; i < 7; ++i) ms[i] = 0.f;
    static const int lo[6] = {0, 1, 3, 6, 4, 8}, hi[6] = {1, 2, 4, 7, 5, 9}, into[6] = {2, 3, 4, 4, 5, 6};
    for (int r = 0; r < g.bands_timed; ++r) {
      const cudaEvent_t* e = &g.ev_band[r * State::kBandEvents];
      for (int k = 0; k < 6; ++k) {
        float t = 0.f;
        if (cudaEventElapsedTime(&t, e[lo[k]], e[hi[k]]) != cudaSuccess) { cudaGetLastError(); return -1; }
        ms[into[k]] += t;
      }
    }
    if (capacity >= 8) ms[7] = static_cast<float>(g.bands_timed);
    return 7;
  }
  if (capacity >= 8) ms[7] = 0.f;
  return 7;
}

int eshkol_b200_get_phase_totals(float ms[7], int counts[3]) {
  if (!g.ready || !ms || !counts || !g.ev_made) return -1;
  if (cudaStreamSynchronize(g.stream) != cudaSuccess) { cudaGetLastError(); return -1; }
  for (int i = 0; i < 7; ++i) ms[i] = 0.f;
  const unsigned long long R = State::kEvRing;
  const unsigned long long nb = g.n_evb < R ? g.n_evb : R, na = g.n_eva < R ? g.n_eva : R,
                           nm = g.n_evm < R ? g.n_evm : R;
  float t = 0.f;
#define B200_ADD(slot, e0, e1)                                                          \
  do {                                                                                  \
    if (cudaEventElapsedTime(&t, e0, e1) != cudaSuccess) { cudaGetLastError(); return -1; } \
    ms[slot] += t;                                                                      \
  } while (0)
  for (unsigned long long i = g.n_evb - nb; i < g.n_evb; ++i) {
    const cudaEvent_t* b = g.ev_b[i % R];
    B200_ADD(0, b[0], b[1]); B200_ADD(1, b[1], b[2]);
  }
  for (unsigned long long i = g.n_eva - na; i < g.n_eva; ++i) {
    const cudaEvent_t* a = g.ev_a[i % R];
    B200_ADD(2, a[0], a[1]); B200_ADD(3, a[1], a[2]);
  }
  for (unsigned long long i = g.n_evm - nm; i < g.n_evm; ++i) {
    const cudaEvent_t* m = g.ev_m[i % R];
    B200_ADD(4, m[0], m[1]); B200_ADD(5, m[1], m[2]); B200_ADD(6, m[2], m[3]);
  }
#undef B200_ADD
  counts[0] = static_cast<int>(nb); counts[1] = static_cast<int>(na); counts[2] = static_cast<int>(nm);
  return 0;
}

void eshkol_b200_debug_set_wait_limit_ns(unsigned long long ns) { g_dbg_wait_ns = ns; }
void eshkol_b200_debug_fail_allocation(int nth) { g_dbg_fail_alloc = nth > 0 ? nth : 0; }
void eshkol_b200_debug_withhold_arrival(int on) { g_dbg_withhold = on ? 1 : 0; }

uint64_t eshkol_b200_launch_count(void) { return g.launches; }
uint64_t eshkol_b200_workspace_bytes(void) { return g.ws_bytes + g.aux_bytes + g.bside_bytes; }

int eshkol_b200_debug_fetch(int what, int index, void* host_dst, uint64_t capacity_bytes,
                            uint64_t info[6]) {
  if (!g.ready || !g.last.valid || !host_dst || !info) return -1;
  const State::Last& L = g.last;
  const void* src = nullptr;
  uint64_t rows = 0, pitch = 0, esz = 1;
  const int n_odd = L.n_mod - 1;
  switch (what) {
    case 0: src = L.mu; rows = 1; pitch = L.M; esz = 4; break;
    case 1: src = L.nu; rows = 1; pitch = L.N; esz = 4; break;
    case 2: src = L.a0; rows = L.M; pitch = L.K0; break;
    case 3: if (index < 0 || index >= n_odd) return -1;
            src = L.aodd + index * L.aodd_stride; rows = L.M; pitch = L.Kp; break;
    case 4: src = L.b0; rows = L.N; pitch = L.K0; break;
    case 5: if (index < 0 || index >= n_odd) return -1;
            src = L.bodd + index * L.bodd_stride; rows = L.N; pitch = L.Kp; break;
    case 6: src = L.w0; rows = L.Mp; pitch = L.Np; esz = 2; break;
    case 7: if (index < 0 || index >= n_odd) return -1;
            src = L.wodd + index * L.wodd_stride; rows = L.Mp; pitch = L.Np; break;
    case 8: src = L.a_hi; rows = L.M; pitch = static_cast<uint64_t>(L.n_chunks) * kChunkUnits; esz = 2; break;
    case 9: src = L.a_odd; rows = L.M; pitch = static_cast<uint64_t>(L.n_chunks) * kChunkUnits; esz = 2; break;
    case 10: src = L.b_hi; rows = L.N; pitch = static_cast<uint64_t>(L.n_chunks) * kChunkUnits; esz = 2; break;
    case 12: src = L.flip; rows = L.Mp; pitch = L.Np / 32; esz = 4; break;
    case 11: src = L.b_odd; rows = L.N; pitch = static_cast<uint64_t>(L.n_chunks) * kChunkUnits; esz = 2; break;
    default: return -1;
  }
  const uint64_t bytes = rows * pitch * esz;
  if (bytes > capacity_bytes) return -2;
  if (cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, g.stream) != cudaSuccess ||
      cudaStreamSynchronize(g.stream) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  info[0] = rows; info[1] = pitch; info[2] = esz; info[3] = L.n_chunks; info[4] = L.last_seg;
  info[5] = bytes;
  return 0;
}

}  // extern "C"
