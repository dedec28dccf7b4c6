// Exact-tier GEMM whose device scratch lives in a fixed array inside this library
// instead of coming from cudaMalloc.
//
// Who this is for.  Two kinds of host cannot let a matmul allocate:
//   * a runtime that hands every free byte of device memory to its own arena at
//     start-up (Eshkol's arena/region allocator is built that way on the host side;
//     a device twin would leave nothing for cudaMalloc to give, so the ordinary
//     entry point would fail in its workspace step);
//   * a caller that runs other streams next to the GEMM and cannot afford the
//     device-wide synchronisation that cudaMalloc / cudaFree imply, or that must
//     not fail for lack of memory in the middle of a computation.
// For them eshkol_b200_gemm_f64_static_scratch runs the same Ozaki-II exact tier
// (16 moduli, same kernels, same bits) with every intermediate -- row/column
// maxima, scales, residue planes of A and B, residue planes of the products, the
// job table -- carved out of `g_static_scratch` below.  The caller still owns and
// passes A, B and C.  The function calls no cudaMalloc, cudaFree or any other
// allocating routine.
//
// The price is a size limit: the scratch a shape needs (see scratch_need) must fit
// kStaticScratchBytes = 24 MiB, which admits e.g. 512 x 512 x 512 or
// 256 x 2048 x 256; anything larger is refused with a message and -1.  Every GPU
// that loads the library holds those 24 MiB until the process exits.
//
// All calls share the one array.  It keeps whatever the previous call left; the
// parts that must start from zero (the modulus-256 planes and their flag bit-planes,
// the column-maximum accumulators) are cleared inside each call.  Calls are ordered by the library's
// stream; two calls made to overlap on the GPU by other means would race on the
// array and must not be issued.
//
// Set-up: eshkol_b200_init asks the runtime for the array's device address on the
// device it selects (the array's name is only a host-side handle; it is not an
// address a kernel can use) and fails if that does not work.  The CUDA runtime
// loads this module, and with it the 24 MiB, at that moment -- so a host whose
// arena takes all remaining device memory must call eshkol_b200_init first, and
// the GEMM entry point itself never triggers a module load or an allocation.
// eshkol_b200_init should be called before any stream capture begins.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include "../../include/eshkol_b200_ext.h"
#include "b200_internal.h"
#include "b200_ozaki2.h"
#include "b200_tiers.h"

namespace b200 {

constexpr size_t kStaticScratchBytes = 24u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

constexpr int kMaxDevices = 64;
unsigned char* s_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch array on the library's device (resolved by
// static_scratch_setup at init), or null.
unsigned char* scratch_base() {
  const int dev = lib_device();
  if (dev < 0 || dev >= kMaxDevices) return nullptr;
  return s_scratch_ptr[dev];
}

__constant__ int c_moduli[16] = {256, 255, 253, 251, 247, 241, 239, 233,
                                 229, 227, 223, 217, 211, 199, 197, 193};

// Job table written on the device, so no host-to-device copy is needed: job 0 is
// the modulus-256 product, jobs 1..15 the odd moduli with their division constants.
__global__ void fill_jobs_kernel(GemmJob* jobs) {
  const int l = threadIdx.x;
  if (l >= 16) return;
  GemmJob j;
  j.n_seg = 1;
  for (int s = 0; s < kMaxSeg; ++s) { j.a_plane[s] = 0; j.b_plane[s] = 0; }
  j.a_plane[0] = (l == 0) ? 0 : l - 1;
  j.b_plane[0] = j.a_plane[0];
  j.out_plane = j.a_plane[0];
  j.modulus = 0; j.magic = 0; j.offset = 0;
  if (l > 0) {
    const unsigned p = static_cast<unsigned>(c_moduli[l]);
    j.modulus = p;
    j.magic = static_cast<unsigned>((1ull << 32) / p);
    j.offset = static_cast<unsigned>((2147483648ull + p - 1) / p * p);
  }
  jobs[l] = j;
}

struct Layout {
  long long Kp, K0, Mp, Np;
  int n_chunks, last_seg, tiles_m, tiles_n;
  size_t o_amax, o_bmax, o_mu, o_nu, o_sa, o_sai, o_sb, o_sbi, o_jobs, o_a0, o_b0, o_aodd, o_bodd,
      o_w0, o_wodd, o_ahi, o_aoddf, o_bhi, o_boddf, o_tie, o_flip, total;
  size_t a_stride, b_stride, w_stride;
};

inline size_t take(size_t& off, size_t bytes) {
  const size_t o = off;
  off += (bytes + 1023) & ~static_cast<size_t>(1023);
  return o;
}

// Scratch a shape needs: vectors of M and N, a little over 16 bytes per element of A
// and of B (padded), 17 bytes per element of the padded C.
Layout scratch_need(long long M, long long K, long long N) {
  Layout L;
  const int bn = 256;
  L.Kp = (K + kBK - 1) / kBK * kBK;
  L.n_chunks = static_cast<int>((K + kChunkK - 1) / kChunkK);
  const int last_len = static_cast<int>(K - static_cast<long long>(L.n_chunks - 1) * kChunkK);
  L.last_seg = (last_len + kBK - 1) / kBK * kBK;
  L.K0 = static_cast<long long>(L.n_chunks - 1) * kChunkSeg + L.last_seg;
  L.tiles_m = static_cast<int>((M + kBM - 1) / kBM);
  L.tiles_n = static_cast<int>((N + bn - 1) / bn);
  L.Mp = static_cast<long long>(L.tiles_m) * kBM;
  L.Np = static_cast<long long>(L.tiles_n) * bn;
  size_t off = 0;
  L.o_amax = take(off, M * 8); L.o_bmax = take(off, N * 8);
  L.o_mu = take(off, M * 4); L.o_nu = take(off, N * 4);
  L.o_sa = take(off, M * 8); L.o_sai = take(off, M * 8);
  L.o_sb = take(off, N * 8); L.o_sbi = take(off, N * 8);
  L.o_jobs = take(off, sizeof(GemmJob) * 16);
  L.o_a0 = take(off, static_cast<size_t>(M) * L.K0);
  L.o_b0 = take(off, static_cast<size_t>(N) * L.K0);
  const size_t fa = static_cast<size_t>(M) * L.n_chunks * kChunkUnits * 2;
  const size_t fb = static_cast<size_t>(N) * L.n_chunks * kChunkUnits * 2;
  L.o_ahi = take(off, fa); L.o_aoddf = take(off, fa);
  L.o_bhi = take(off, fb); L.o_boddf = take(off, fb);
  L.a_stride = static_cast<size_t>(M) * L.Kp;
  L.b_stride = static_cast<size_t>(N) * L.Kp;
  L.o_aodd = take(off, L.a_stride * 15);
  L.o_bodd = take(off, L.b_stride * 15);
  L.w_stride = static_cast<size_t>(L.Mp) * L.Np;
  L.o_w0 = take(off, L.w_stride * 2);
  L.o_wodd = take(off, L.w_stride * 15);
  L.o_tie = take(off, L.w_stride / 32 * 8 * L.n_chunks);
  L.o_flip = take(off, L.w_stride / 32 * 4);
  L.total = off;
  return L;
}

#define SS_CHECK(call)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess) {                                                            \
      fprintf(stderr, "[eshkol-b200] %s failed: %s (%s:%d)\n", #call,                   \
              cudaGetErrorString(e_), __FILE__, __LINE__);                              \
      return -1;                                                                        \
    }                                                                                   \
  } while (0)

}  // namespace

// Called by eshkol_b200_init with `device` current: resolves the array's address on that
// device once.  This is the only place the symbol is looked up.
int static_scratch_setup(int device) {
  if (device < 0 || device >= kMaxDevices) return -1;
  if (s_scratch_ptr[device]) return 0;
  unsigned char* p = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
  if (e != cudaSuccess || !p) {
    fprintf(stderr, "[eshkol-b200] cudaGetSymbolAddress(static scratch) failed: %s\n", cudaGetErrorString(e));
    cudaGetLastError();
    return -1;
  }
  s_scratch_ptr[device] = p;
  return 0;
}

}  // namespace b200

using namespace b200;

extern "C" int eshkol_b200_gemm_f64_static_scratch(const double* dA, const double* dB, double* dC,
                                                   uint64_t M_, uint64_t K_, uint64_t N_) {
  cudaStream_t st = lib_stream();
  if (!st) {
    fprintf(stderr, "[eshkol-b200] static-scratch gemm called before eshkol_b200_init succeeded\n");
    return -1;
  }
  if (!dA || !dB || !dC || M_ == 0 || K_ == 0 || N_ == 0) return -1;
  if (M_ > (1u << 20) || N_ > (1u << 20) || K_ > 131071) {
    fprintf(stderr, "[eshkol-b200] static-scratch gemm: %llu x %llu x %llu is beyond what the fixed "
                    "%zu-byte scratch can serve\n", (unsigned long long)M_, (unsigned long long)K_,
            (unsigned long long)N_, kStaticScratchBytes);
    return -1;
  }
  const long long M = static_cast<long long>(M_), K = static_cast<long long>(K_), N = static_cast<long long>(N_);
  const Layout L = scratch_need(M, K, N);
  if (L.total > kStaticScratchBytes) {
    fprintf(stderr, "[eshkol-b200] static-scratch gemm: %lld x %lld x %lld needs %zu bytes of scratch, "
                    "the fixed array holds %zu; use eshkol_b200_gemm_f64_device for this shape\n",
            M, K, N, L.total, kStaticScratchBytes);
    return -1;
  }
  unsigned char* ws = scratch_base();
  if (!ws) {
    fprintf(stderr, "[eshkol-b200] static-scratch gemm: the scratch array was not resolved at init\n");
    return -1;
  }

  double* amax = reinterpret_cast<double*>(ws + L.o_amax);
  double* bmax = reinterpret_cast<double*>(ws + L.o_bmax);
  int* mu = reinterpret_cast<int*>(ws + L.o_mu);
  int* nu = reinterpret_cast<int*>(ws + L.o_nu);
  double* sa = reinterpret_cast<double*>(ws + L.o_sa);
  double* sai = reinterpret_cast<double*>(ws + L.o_sai);
  double* sb = reinterpret_cast<double*>(ws + L.o_sb);
  double* sbi = reinterpret_cast<double*>(ws + L.o_sbi);
  GemmJob* jobs = reinterpret_cast<GemmJob*>(ws + L.o_jobs);
  int8_t* a0 = reinterpret_cast<int8_t*>(ws + L.o_a0);
  int8_t* b0 = reinterpret_cast<int8_t*>(ws + L.o_b0);
  int8_t* aodd = reinterpret_cast<int8_t*>(ws + L.o_aodd);
  int8_t* bodd = reinterpret_cast<int8_t*>(ws + L.o_bodd);
  uint16_t* a_hi = reinterpret_cast<uint16_t*>(ws + L.o_ahi);
  uint16_t* a_oddf = reinterpret_cast<uint16_t*>(ws + L.o_aoddf);
  uint16_t* b_hi = reinterpret_cast<uint16_t*>(ws + L.o_bhi);
  uint16_t* b_oddf = reinterpret_cast<uint16_t*>(ws + L.o_boddf);
  int16_t* w0 = reinterpret_cast<int16_t*>(ws + L.o_w0);
  int8_t* wodd = reinterpret_cast<int8_t*>(ws + L.o_wodd);
  uint32_t* tie_bits = reinterpret_cast<uint32_t*>(ws + L.o_tie);
  uint32_t* flip_bits = reinterpret_cast<uint32_t*>(ws + L.o_flip);

  Oz2DeviceConsts hc;
  oz2_host_consts(16, &hc, nullptr);

  SS_CHECK(launch_scan_rows(dA, M, K, amax, st));
  // clears the column accumulators before use
  SS_CHECK(launch_scan_cols(dB, K, N, reinterpret_cast<unsigned long long*>(bmax), st));
  SS_CHECK(launch_scales(amax, M, 52, mu, sa, sai, st));
  SS_CHECK(launch_scales(bmax, N, 52, nu, sb, sbi, st));
  SplitPlanes pa{M, K, L.Kp, L.K0, L.n_chunks, 15, a0, a_hi, a_oddf, aodd, static_cast<long long>(L.a_stride)};
  SplitPlanes pb{N, K, L.Kp, L.K0, L.n_chunks, 15, b0, b_hi, b_oddf, bodd, static_cast<long long>(L.b_stride)};
  // each clears its modulus-256 plane and flag bit-planes before writing into them
  SS_CHECK(launch_split_a(dA, sa, pa, hc, st));
  SS_CHECK(launch_split_b(dB, sb, N, pb, hc, st));
  fill_jobs_kernel<<<1, 32, 0, st>>>(jobs);
  SS_CHECK(cudaGetLastError());

  GemmParams p0 = make_gemm_params();
  p0.tiles_m = L.tiles_m; p0.tiles_n = L.tiles_n; p0.n_jobs = 1;
  p0.kb_per_seg = static_cast<int>(L.K0 / kBK);
  p0.kb_per_unit = kChunkSeg / kBK;
  p0.a_hi = a_hi; p0.a_odd = a_oddf; p0.b_odd = b_oddf; p0.b_hi = b_hi;
  p0.n_chunks = L.n_chunks;
  p0.tie_bits = tie_bits;
  p0.group_m = 16;
  p0.jobs = jobs;
  p0.out = reinterpret_cast<uint8_t*>(w0);
  p0.out_plane_stride = 0;
  p0.ldo = static_cast<int>(L.Np);
  p0.status = lib_status_word();
  p0.work_counter = lib_status_word() + 1;
  GemmParams p1 = p0;
  p1.n_jobs = 15;
  p1.kb_per_seg = static_cast<int>(L.Kp / kBK);
  p1.kb_per_unit = 1023;  // deeper products hand the accumulator over in parts (none fits the array anyway)
  p1.jobs = jobs + 1;
  p1.out = reinterpret_cast<uint8_t*>(wodd);
  p1.out_plane_stride = static_cast<long long>(L.w_stride);
  CUtensorMap mA0, mB0, mA1, mB1;
  if (make_plane_map(&mA0, a0, L.K0, M, 1, M * L.K0, kBM)) return -1;
  if (make_plane_map(&mB0, b0, L.K0, N, 1, N * L.K0, 256)) return -1;
  if (make_plane_map(&mA1, aodd, L.Kp, M, 15, static_cast<long long>(L.a_stride), kBM)) return -1;
  if (make_plane_map(&mB1, bodd, L.Kp, N, 15, static_cast<long long>(L.b_stride), 256)) return -1;
  SS_CHECK(launch_modgemm(256, kEpiMod256, mA0, mB0, p0, L.tiles_m * L.tiles_n, lib_num_sms(), st));
  SS_CHECK(launch_tie_resolve(p0, flip_bits, static_cast<int>(M), static_cast<int>(N), st));
  SS_CHECK(launch_modgemm(256, kEpiModI8, mA1, mB1, p1, L.tiles_m * L.tiles_n * 15, lib_num_sms(), st));

  CrtArgs ca;
  ca.w0 = w0; ca.flip = flip_bits; ca.w_odd = wodd; ca.w_odd_stride = static_cast<long long>(L.w_stride); ca.ldw = L.Np;
  ca.n_mod = 16; ca.M = M; ca.N = N;
  ca.inv_scale_a = sai; ca.inv_scale_b = sbi;
  ca.C = dC; ca.ldc = N;
  ca.bias_mode = 0; ca.bias = nullptr; ca.activation = 0; ca.pixels_per_image = 0;
  SS_CHECK(launch_crt(ca, hc, st));
  count_launches(11);
  return 0;
}
