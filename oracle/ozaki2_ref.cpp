// TEST INFRASTRUCTURE ONLY -- CPU oracle for the Ozaki-II exact f64 GEMM tier.
//
// This file restates, step by step, the arithmetic of the reference's Metal
// "Ozaki-II" exact DGEMM so that the CUDA path can be compared bit for bit
// against it.  Only tests/, the smoke check and the bench's cpu_baseline leg may
// load it; the shipped library never links or calls anything in oracle/.
//
// Reference lines restated (paths inside the reference project):
//   moduli table                    lib/backend/gpu/gpu_memory.mm:227-233
//   CRT constants (P, q_l, s_l)     lib/backend/gpu/gpu_memory.mm:301-341
//   frac bounds and exponent E      lib/backend/gpu/gpu_memory.mm:376-420, 2510-2512
//   per-row / per-column scales     lib/backend/gpu/gpu_memory.mm:2514-2532
//   integerisation trunc(a*2^mu)    lib/backend/gpu/gpu_memory.mm:2538-2547
//   residues x - p*rint(x/p)        lib/backend/gpu/gpu_memory.mm:2573-2583
//   modular GEMM, 1008-element
//   extraction, final reduce        lib/backend/gpu/metal_softfloat.h:3925-3926,
//                                   3966-3969, 4054-4099
//   CRT accumulation S1/S2          lib/backend/gpu/gpu_memory.mm:2619-2641
//   reconstruction and descaling    lib/backend/gpu/gpu_memory.mm:2644-2655
//
// Parity status: pinned by the reference's own known-answer fixture (the 512x512
// integer witness of tests/gpu/ozaki_certification_test.esk, 25 cells that must
// EQUAL the exact integer dot product) and by its tolerance fixtures
// (tests/gpu/ozaki_correctness_test.esk, 1e-9).  No reference test asserts the
// bits of the result on non-integer data; there the oracle itself is the pin.
//
// Choices made explicit here (the reference leaves them to its compiler/device):
//  * "a*b+c" in the reference's host loops is evaluated fused (its only build
//    target contracts them); flag OZ2_UNFUSED selects separate mul+add.
//  * floor(log2(max)) is evaluated with the libm call, as the reference does;
//    flag OZ2_EXPFIELD uses oz2_floor_log2_model(), an integer-only model of
//    that call, which is what the CUDA kernels use.  tests compare the two.
//  * the K-extraction interval of the modular GEMM is 63 blocks of 16 = 1008.
//  * the modular dot products are accumulated in exact integers; the reference
//    carries the same integers in f32, exact while |sum| < 2^24.
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off -fopenmp -shared).

#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#define OZ2_UNFUSED 1
#define OZ2_EXPFIELD 2

static const int OZ2_MODULI[16] = {256, 255, 253, 251, 247, 241, 239, 233,
                                   229, 227, 223, 217, 211, 199, 197, 193};
static const int OZ2_CHUNK = 1008;  // 63 K-blocks of 16

struct Oz2Crt {
  double P1, P2, Pinv, log2P;
  double sl1[16], sl2[16];
  int q[16];
  int n;
};

static int64_t egcd(int64_t a, int64_t b, int64_t& x, int64_t& y) {
  if (a == 0) { x = 0; y = 1; return b; }
  int64_t x1, y1;
  int64_t g = egcd(b % a, a, x1, y1);
  x = y1 - (b / a) * x1;
  y = x1;
  return g;
}
static int modinv(int64_t a, int64_t m) {
  int64_t x, y;
  egcd(a % m, m, x, y);
  return (int)((x % m + m) % m);
}

// gpu_memory.mm:301-341
static void oz2_precompute(int n, Oz2Crt* c) {
  c->n = n;
  __int128 P = 1;
  for (int l = 0; l < n; l++) P *= OZ2_MODULI[l];
  c->P1 = (double)P;
  __int128 P1i = (__int128)c->P1;
  c->P2 = (double)(P - P1i);
  c->Pinv = 1.0 / (double)P;
  c->log2P = std::log2((double)P);
  for (int l = 0; l < n; l++) {
    int p = OZ2_MODULI[l];
    __int128 Pp = P / p;
    c->q[l] = modinv((int64_t)(Pp % p), p);
    __int128 s = Pp * (__int128)c->q[l];
    int bits_to_remove = 8 + (int)std::ceil(std::log2((double)n));
    double s_d = (double)s;
    double factor = (double)(1LL << (bits_to_remove + 1)) + 1.0;
    volatile double t = factor * s_d;
    volatile double u = t - s_d;
    c->sl1[l] = t - u;
    __int128 sl1i = (__int128)c->sl1[l];
    c->sl2[l] = (double)(s - sl1i);
  }
}

// Integer-only model of floor(log2(x)) as a correctly rounded libm evaluates it
// for finite x > 0.  log2 of the largest doubles below a power of two 2^t rounds
// to t itself once |t| >= 3, so the libm call returns t where the exponent field
// says t-1.  x = 2^t * (1 - m*2^-53); -log2(1 - m*2^-53) = m*2^-53/ln 2 (+ O(2^-106));
// it rounds to t iff that distance is below half the spacing of doubles next to t
// on the side the value lies on.
extern "C" int oz2_floor_log2_model(double x) {
  uint64_t bits;
  std::memcpy(&bits, &x, 8);
  int ef = (int)((bits >> 52) & 0x7ff);
  uint64_t man = bits & ((1ull << 52) - 1);
  int e;
  uint64_t sig;  // 53-bit significand with leading one at bit 52
  if (ef == 0) {
    if (man == 0) return 0;  // caller never passes 0
    int lz = __builtin_clzll(man) - 11;  // shift needed to put the top bit at 52
    sig = man << lz;
    e = -1022 - lz;
  } else {
    sig = man | (1ull << 52);
    e = ef - 1023;
  }
  uint64_t m = (1ull << 53) - sig;  // deficit to the next power of two, 1..2^52
  int t = e + 1;
  if (t == 0 || m > 2048) return e;
  int a = t < 0 ? -t : t;
  int lg = 31 - __builtin_clz((unsigned)a);
  bool pow2 = (a & (a - 1)) == 0;
  // half spacing (units of 2^-53) of the doubles adjacent to t on the far-from-zero
  // side is 2^lg; on the near-zero side of a power of two it is 2^(lg-1).
  double thr = (t > 0 && pow2) ? std::ldexp(1.0, lg - 1) : std::ldexp(1.0, lg);
  return ((double)m * 1.4426950408889634 < thr) ? t : e;
}

static inline int floor_log2_of(double x, int flags) {
  if (flags & OZ2_EXPFIELD) return oz2_floor_log2_model(x);
  return (int)std::floor(std::log2(x));
}

extern "C" {

int oracle_oz2_constants(int n_mod, double* P1, double* P2, double* Pinv, double* log2P,
                         double* sl1, double* sl2, int* q) {
  if (n_mod < 2 || n_mod > 16) return -1;
  Oz2Crt c;
  oz2_precompute(n_mod, &c);
  *P1 = c.P1; *P2 = c.P2; *Pinv = c.Pinv; *log2P = c.log2P;
  for (int l = 0; l < n_mod; l++) { sl1[l] = c.sl1[l]; sl2[l] = c.sl2[l]; q[l] = c.q[l]; }
  return 0;
}

// gpu_memory.mm:376-420 and 2510-2512.  Full matrices are needed: the bound is a
// maximum over every row of A and every column of B.
int oracle_oz2_E(const double* A, const double* B, int64_t M, int64_t K, int64_t N,
                 int n_mod, double* fracA_out, double* fracB_out) {
  Oz2Crt c;
  oz2_precompute(n_mod, &c);
  double fracA = 0.0, fracB = 0.0;
  for (int64_t i = 0; i < M; i++) {
    double mx = 0.0;
    for (int64_t k = 0; k < K; k++) { double v = std::fabs(A[i * K + k]); if (v > mx) mx = v; }
    if (mx > 0.0) { double lg = std::log2(mx); double f = lg - std::floor(lg); if (f > fracA) fracA = f; }
  }
  std::vector<double> cm(N, 0.0);
  for (int64_t k = 0; k < K; k++)
    for (int64_t j = 0; j < N; j++) { double v = std::fabs(B[k * N + j]); if (v > cm[j]) cm[j] = v; }
  for (int64_t j = 0; j < N; j++)
    if (cm[j] > 0.0) { double lg = std::log2(cm[j]); double f = lg - std::floor(lg); if (f > fracB) fracB = f; }
  if (fracA_out) *fracA_out = fracA;
  if (fracB_out) *fracB_out = fracB;
  int E = (int)std::floor((c.log2P - 1.0 - std::log2((double)K) - fracA - fracB) / 2.0);
  if (E > 52) E = 52;
  if (E < 0) E = 0;
  return E;
}

// Exact-tier GEMM on a sub-problem: As is m x K (any subset of rows of A), Bs is
// K x n (any subset of columns of B, made contiguous), Cs is m x n.  Rows and
// columns are independent given E, so a subset reproduces the same bits as the
// full product.  Optional debug outputs: mu[m], nu[n], and the residues of the
// modular products W[n_mod][m][n] as floats.
int oracle_oz2_exact_sub(const double* As, const double* Bs, double* Cs,
                         int64_t m, int64_t K, int64_t n, int E, int n_mod, int flags,
                         int* mu_out, int* nu_out, float* W_out,
                         float* Ares_out, float* Bres_out) {
  if (n_mod < 2 || n_mod > 16 || m <= 0 || K <= 0 || n <= 0) return -1;
  Oz2Crt crt;
  oz2_precompute(n_mod, &crt);
  const bool unfused = (flags & OZ2_UNFUSED) != 0;

  // --- scales (gpu_memory.mm:2514-2532) ---
  std::vector<int> mu(m), nu(n);
  for (int64_t i = 0; i < m; i++) {
    double mx = 0.0;
    for (int64_t k = 0; k < K; k++) { double v = std::fabs(As[i * K + k]); if (v > mx) mx = v; }
    mu[i] = (mx == 0.0) ? 0 : E - floor_log2_of(mx, flags);
  }
  {
    std::vector<double> cm(n, 0.0);
    for (int64_t k = 0; k < K; k++)
      for (int64_t j = 0; j < n; j++) { double v = std::fabs(Bs[k * n + j]); if (v > cm[j]) cm[j] = v; }
    for (int64_t j = 0; j < n; j++) nu[j] = (cm[j] == 0.0) ? 0 : E - floor_log2_of(cm[j], flags);
  }
  if (mu_out) std::memcpy(mu_out, mu.data(), m * sizeof(int));
  if (nu_out) std::memcpy(nu_out, nu.data(), n * sizeof(int));

  // --- integerisation (gpu_memory.mm:2538-2547) ---
  std::vector<double> Ai((size_t)m * K), Bi((size_t)K * n);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; i++) {
    double scale = std::ldexp(1.0, mu[i]);
    for (int64_t k = 0; k < K; k++) Ai[i * K + k] = std::trunc(As[i * K + k] * scale);
  }
  {
    std::vector<double> sc(n);
    for (int64_t j = 0; j < n; j++) sc[j] = std::ldexp(1.0, nu[j]);
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < K; k++)
      for (int64_t j = 0; j < n; j++) Bi[k * n + j] = std::trunc(Bs[k * n + j] * sc[j]);
  }

  std::vector<double> S1((size_t)m * n, 0.0), S2((size_t)m * n, 0.0);
  std::vector<int16_t> Ar((size_t)m * K), Br((size_t)K * n);
  std::vector<float> Wl((size_t)m * n);
  const int64_t nchunk = (K + OZ2_CHUNK - 1) / OZ2_CHUNK;

  for (int l = 0; l < n_mod; l++) {
    const int p = OZ2_MODULI[l];
    const double p_d = (double)p, p_inv = 1.0 / p_d;
    // --- residues (gpu_memory.mm:2573-2583): (float)(x - p*rint(x*(1/p))) ---
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m * K; i++) {
      double x = Ai[i], r = std::rint(x * p_inv);
      float f = unfused ? (float)(x - p_d * r) : (float)std::fma(-p_d, r, x);
      Ar[i] = (int16_t)f;
      if (Ares_out) Ares_out[(size_t)l * m * K + i] = f;
    }
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < K * n; i++) {
      double x = Bi[i], r = std::rint(x * p_inv);
      float f = unfused ? (float)(x - p_d * r) : (float)std::fma(-p_d, r, x);
      Br[i] = (int16_t)f;
      if (Bres_out) Bres_out[(size_t)l * K * n + i] = f;
    }
    // --- modular GEMM (metal_softfloat.h:3966-3969, 4054-4099) ---
    const float p_f = (float)p, p_invf = 1.0f / p_f;
#pragma omp parallel
    {
      std::vector<int32_t> acc(n);
      std::vector<float> part(n);
#pragma omp for schedule(dynamic, 4)
      for (int64_t i = 0; i < m; i++) {
        std::fill(part.begin(), part.end(), 0.0f);
        for (int64_t c = 0; c < nchunk; c++) {
          std::fill(acc.begin(), acc.end(), 0);
          int64_t k0 = c * OZ2_CHUNK, k1 = k0 + OZ2_CHUNK;
          if (k1 > K) k1 = K;
          for (int64_t k = k0; k < k1; k++) {
            const int32_t a = Ar[i * K + k];
            if (a == 0) continue;
            const int16_t* brow = &Br[k * n];
            int32_t* ac = acc.data();
            for (int64_t j = 0; j < n; j++) ac[j] += a * (int32_t)brow[j];
          }
          for (int64_t j = 0; j < n; j++) {
            // the accumulator is an exact integer; in f32 it is exact below 2^24
            float v = (float)acc[j];
            volatile float qf = std::rint(v * p_invf);
            volatile float pq = p_f * qf;
            part[j] += v - pq;
          }
        }
        for (int64_t j = 0; j < n; j++) {
          float w = part[j];
          volatile float qf = std::rint(w * p_invf);
          volatile float pq = p_f * qf;
          Wl[i * n + j] = w - pq;
        }
      }
    }
    if (W_out) std::memcpy(W_out + (size_t)l * m * n, Wl.data(), (size_t)m * n * sizeof(float));
    // --- CRT accumulation (gpu_memory.mm:2632-2640) ---
    const double sl1 = crt.sl1[l], sl2 = crt.sl2[l];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m * n; i++) {
      double w = (double)Wl[i];
      if (unfused) {
        volatile double t1 = sl1 * w, t2 = sl2 * w;
        S1[i] += t1; S2[i] += t2;
      } else {
        S1[i] = std::fma(sl1, w, S1[i]);
        S2[i] = std::fma(sl2, w, S2[i]);
      }
    }
  }
  // --- reconstruction (gpu_memory.mm:2644-2655) ---
  const double P1 = crt.P1, P2 = crt.P2, Pinv = crt.Pinv;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < m; i++) {
    double mu_inv = std::ldexp(1.0, -mu[i]);
    for (int64_t j = 0; j < n; j++) {
      size_t idx = (size_t)i * n + j;
      volatile double s = S1[idx] + S2[idx];
      volatile double sp = s * Pinv;
      double Q = std::round(sp);
      volatile double c1 = std::fma(-P1, Q, S1[idx]);
      volatile double c2 = std::fma(-P2, Q, S2[idx]);
      volatile double cp = c1 + c2;
      volatile double t = cp * mu_inv;
      Cs[idx] = t * std::ldexp(1.0, -nu[j]);
    }
  }
  return 0;
}

}  // extern "C"
