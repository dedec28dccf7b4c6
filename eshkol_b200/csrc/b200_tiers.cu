// Reduced-precision tiers of the f64 GEMM and the conv2d lowering.
//
//  * Ozaki-I (int8 slices): restates cuda_matmul_ozaki_int8_f64 and its kernels,
//    lib/backend/gpu/gpu_memory_cuda.cpp:339-452 and
//    lib/backend/gpu/gpu_cuda_kernels.cu:664-741, with every slice pair of one
//    diagonal accumulated in a single TMEM accumulator instead of one library GEMM
//    per pair.
//  * Ozaki-II fast: restates ozaki_ii_fast_dispatch and its three shaders,
//    lib/backend/gpu/gpu_memory.mm:2816-3012 and
//    lib/backend/gpu/metal_softfloat.h:4150-4246, with the CRT carried in exact 128-bit
//    integers instead of double-float and the exact tier's moduli (int32 accumulation
//    lifts the cap the f32 GEMM imposed on them).
//  * native f64 GEMM on CUDA cores: the stand-in for the reference's cublasDgemm call.
//  * conv2d: in the exact tier the right-hand operand is the im2col index map over the NCHW
//    tensor, read in place by the column scan and the split; the other tiers materialise the
//    im2col matrix first.  NCHW scatter and optional bias / ReLU are fused into the last pass.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "b200_common.cuh"
#include "b200_internal.h"
#include "b200_residue.cuh"
#include "b200_tiers.h"

#include <cuda_fp16.h>
#include <vector>

namespace b200 {

#define TIER_CHECK(call)                                                               \
  do {                                                                                 \
    cudaError_t e_ = (call);                                                           \
    if (e_ != cudaSuccess) {                                                           \
      fprintf(stderr, "[eshkol-b200] %s failed: %s (%s:%d)\n", #call,                  \
              cudaGetErrorString(e_), __FILE__, __LINE__);                             \
      return -1;                                                                       \
    }                                                                                  \
  } while (0)

namespace {

inline long long round_up_ll(long long x, long long m) { return (x + m - 1) / m * m; }

struct Carver {
  size_t off = 0;
  size_t take(size_t bytes) {
    const size_t o = off;
    off += (bytes + 1023) & ~static_cast<size_t>(1023);
    return o;
  }
};

struct Epilogue {
  double* C;
  long long M, N, ldc;
  int bias_mode;
  const double* bias;
  int activation;
  long long pixels_per_image;
};

__device__ __forceinline__ void store_out(const Epilogue& ep, long long i, long long j, double c) {
  if (ep.bias_mode == 1) c = __dadd_rn(c, ep.bias[i]);
  else if (ep.bias_mode == 2) c = __dadd_rn(c, ep.bias[j]);
  c = apply_activation(c, ep.activation);
  long long o;
  if (ep.pixels_per_image > 0) {
    const long long img = j / ep.pixels_per_image, pix = j - img * ep.pixels_per_image;
    o = (img * ep.M + i) * ep.pixels_per_image + pix;
  } else {
    o = i * ep.ldc + j;
  }
  ep.C[o] = c;
}

Epilogue make_epilogue(double* C, long long M, long long N, const EshkolB200GemmOpts& o) {
  Epilogue ep;
  ep.C = C; ep.M = M; ep.N = N; ep.ldc = (o.ldc > 0) ? o.ldc : N;
  ep.bias_mode = o.bias ? o.bias_mode : 0;
  ep.bias = o.bias;
  ep.activation = o.activation;
  ep.pixels_per_image = o.pixels_per_image;
  return ep;
}

__device__ __forceinline__ void load4(const double* src, long long k4, long long K, double (&a)[4]) {
  if (k4 + 3 < K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const double2 v0 = __ldg(reinterpret_cast<const double2*>(src));
    const double2 v1 = __ldg(reinterpret_cast<const double2*>(src) + 1);
    a[0] = v0.x; a[1] = v0.y; a[2] = v1.x; a[3] = v1.y;
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] = (k4 + e < K) ? __ldg(src + e) : 0.0;
  }
}

// ====================================================================== Ozaki-I
__global__ void oz1_fix_max_kernel(double* v, long long n) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n && !(v[i] > 0.0)) v[i] = 1.0;  // gpu_cuda_kernels.cu:672
}

// one slice step: res *= 128; a = clamp(rint(res), +-127); res -= a   (gpu_cuda_kernels.cu:695-700)
__device__ __forceinline__ int oz1_slice(double& res) {
  res *= 128.0;
  double a = (res + kRoundMagic) - kRoundMagic;
  a = (a > 127.0) ? 127.0 : ((a < -127.0) ? -127.0 : a);
  res -= a;
  return __double2int_rn(a);
}

__global__ void __launch_bounds__(256) oz1_split_a_kernel(const double* __restrict__ A,
                                                          const double* __restrict__ rmax,
                                                          long long K, long long Kp, int s,
                                                          int8_t* __restrict__ planes,
                                                          long long plane_stride) {
  const long long row = blockIdx.x;
  const long long k4 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * 4;
  if (k4 >= Kp) return;
  double a[4];
  load4(A + row * K + k4, k4, K, a);
  const double r = rmax[row];
  double res[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) res[e] = a[e] / r;
  for (int p = 0; p < s; ++p) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) word |= (static_cast<uint32_t>(oz1_slice(res[e])) & 0xffu) << (8 * e);
    *reinterpret_cast<uint32_t*>(planes + p * plane_stride + row * Kp + k4) = word;
  }
}

constexpr int kTJ = 32, kTK = 128, kTPitch = 33;
__global__ void __launch_bounds__(256) oz1_split_b_kernel(const double* __restrict__ B,
                                                          const double* __restrict__ cmax,
                                                          long long K, long long Kp, long long N,
                                                          int s, int8_t* __restrict__ planes,
                                                          long long plane_stride) {
  extern __shared__ uint32_t sm[];  // [s][32][33]
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long j = static_cast<long long>(blockIdx.x) * kTJ + tx;
  const long long kbase = static_cast<long long>(blockIdx.y) * kTK;
  const double c = (j < N) ? cmax[j] : 1.0;
#pragma unroll 1
  for (int qd = ty; qd < kTK / 4; qd += 8) {
    const long long k = kbase + qd * 4;
    double res[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const double b = (j < N && k + e < K) ? __ldg(B + (k + e) * N + j) : 0.0;
      res[e] = b / c;
    }
    for (int p = 0; p < s; ++p) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) word |= (static_cast<uint32_t>(oz1_slice(res[e])) & 0xffu) << (8 * e);
      sm[(p * kTJ + tx) * kTPitch + qd] = word;
    }
  }
  __syncthreads();
  const int jj = threadIdx.x >> 3, gq = threadIdx.x & 7;
  const long long jo = static_cast<long long>(blockIdx.x) * kTJ + jj;
  const long long k16 = kbase + gq * 16;
  if (jo >= N || k16 >= Kp) return;
  for (int p = 0; p < s; ++p) {
    const uint32_t* w = &sm[(p * kTJ + jj) * kTPitch + gq * 4];
    *reinterpret_cast<uint4*>(planes + p * plane_stride + jo * Kp + k16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

struct Oz1Weights {
  double w[24];
  int n;
};

// C = (sum_b w_b * G_b) * r_i * c_j, buffers in order (gpu_cuda_kernels.cu:736-739)
__global__ void __launch_bounds__(256) oz1_reconstruct_kernel(const int32_t* __restrict__ G,
                                                              long long g_stride, long long ldg,
                                                              const Oz1Weights wt,
                                                              const double* __restrict__ rmax,
                                                              const double* __restrict__ cmax,
                                                              const Epilogue ep) {
  const long long i = blockIdx.x;
  const long long j4 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * 4;
  if (j4 >= ep.N) return;
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  for (int b = 0; b < wt.n; ++b) {
    const int4 gv = __ldg(reinterpret_cast<const int4*>(G + b * g_stride + i * ldg + j4));
    const double w = wt.w[b];
    acc[0] = fma(w, static_cast<double>(gv.x), acc[0]);
    acc[1] = fma(w, static_cast<double>(gv.y), acc[1]);
    acc[2] = fma(w, static_cast<double>(gv.z), acc[2]);
    acc[3] = fma(w, static_cast<double>(gv.w), acc[3]);
  }
  const double r = rmax[i];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const long long j = j4 + e;
    if (j >= ep.N) break;
    store_out(ep, i, j, __dmul_rn(__dmul_rn(acc[e], r), cmax[j]));
  }
}

// ================================================================ Ozaki-II fast
// frexp exponent of the row / column maximum, 0 for an all-zero row (gpu_memory.mm:2893, 2904)
__global__ void fast_exps_kernel(const double* __restrict__ vmax, long long n, int* __restrict__ ex) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double mx = vmax[i];
  int e = 0;
  if (mx != 0.0) frexp(mx, &e);
  ex[i] = e;
}

// metal_softfloat.h:4163-4187: the 53-bit significand shifted right by
// s = -((exp - 1075) + E - es) with round-half-up, sign re-applied; subnormals -> 0.
__device__ __forceinline__ double fast_integerise(double a, int E, int es) {
  const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(a));
  const int ex = static_cast<int>((bits >> 52) & 0x7ffu);
  if (ex == 0) return 0.0;
  unsigned long long m = (bits & ((1ull << 52) - 1)) | (1ull << 52);
  int s = -((ex - 1075) + E - es);
  if (s > 53) return 0.0;
  if (s < 0) s = 0;
  if (s >= 1) m += 1ull << (s - 1);
  m >>= s;
  const double x = static_cast<double>(static_cast<long long>(m));
  return (bits >> 63) ? -x : x;
}

__device__ __forceinline__ uint32_t fast_residue_byte(double x, uint32_t xlo, int l, const Oz2DeviceConsts& c) {
  if (c.p_i[l] == 256) return xlo & 255u;
  return static_cast<uint32_t>(residue_odd(x, xlo, c.p_inv[l], c.p_i[l])) & 0xffu;
}

__global__ void __launch_bounds__(256) fast_split_a_kernel(const double* __restrict__ A,
                                                           const int* __restrict__ erow, int E,
                                                           long long K, long long Kp,
                                                           int8_t* __restrict__ planes,
                                                           long long plane_stride,
                                                           const __grid_constant__ Oz2DeviceConsts c) {
  const long long row = blockIdx.x;
  const long long k4 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * 4;
  if (k4 >= Kp) return;
  double a[4], x[4];
  load4(A + row * K + k4, k4, K, a);
  const int es = erow[row];
  uint32_t xlo[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    x[e] = fast_integerise(a[e], E, es);
    xlo[e] = static_cast<uint32_t>(static_cast<long long>(x[e]));
  }
  for (int l = 0; l < c.n_mod; ++l) {
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) word |= fast_residue_byte(x[e], xlo[e], l, c) << (8 * e);
    *reinterpret_cast<uint32_t*>(planes + l * plane_stride + row * Kp + k4) = word;
  }
}

__global__ void __launch_bounds__(256) fast_split_b_kernel(const double* __restrict__ B,
                                                           const int* __restrict__ ecol, int E,
                                                           long long K, long long Kp, long long N,
                                                           int8_t* __restrict__ planes,
                                                           long long plane_stride,
                                                           const __grid_constant__ Oz2DeviceConsts c) {
  extern __shared__ uint32_t sm[];  // [n_mod][32][33]
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long j = static_cast<long long>(blockIdx.x) * kTJ + tx;
  const long long kbase = static_cast<long long>(blockIdx.y) * kTK;
  const int es = (j < N) ? ecol[j] : 0;
#pragma unroll 1
  for (int qd = ty; qd < kTK / 4; qd += 8) {
    const long long k = kbase + qd * 4;
    double x[4];
    uint32_t xlo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const double b = (j < N && k + e < K) ? __ldg(B + (k + e) * N + j) : 0.0;
      x[e] = fast_integerise(b, E, es);
      xlo[e] = static_cast<uint32_t>(static_cast<long long>(x[e]));
    }
    for (int l = 0; l < c.n_mod; ++l) {
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) word |= fast_residue_byte(x[e], xlo[e], l, c) << (8 * e);
      sm[(l * kTJ + tx) * kTPitch + qd] = word;
    }
  }
  __syncthreads();
  const int jj = threadIdx.x >> 3, gq = threadIdx.x & 7;
  const long long jo = static_cast<long long>(blockIdx.x) * kTJ + jj;
  const long long k16 = kbase + gq * 16;
  if (jo >= N || k16 >= Kp) return;
  for (int l = 0; l < c.n_mod; ++l) {
    const uint32_t* w = &sm[(l * kTJ + jj) * kTPitch + gq * 4];
    *reinterpret_cast<uint4*>(planes + l * plane_stride + jo * Kp + k16) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// The fractional CRT of metal_softfloat.h:4192-4245, carried out in exact 128-bit
// integer arithmetic instead of double-float: x = sum_l u_l * (P/p_l) mod P with
// u_l = (G_l mod p_l) * q_l mod p_l, centred to [-P/2, P/2), converted to f64 with one
// round-to-nearest-even, then scaled by 2^(e_i + f_j - 2E).  No rounding happens before
// the final conversion, so the tier's only error is the integerisation of the inputs.
struct FastCrtConsts {
  unsigned long long P_hi, P_lo;
  unsigned long long Pp_hi[16], Pp_lo[16];  // P / p_l
  int p[16], q[16];
  int n_mod;
};

__device__ __forceinline__ double u128_to_double_rne(unsigned __int128 v) {
  const unsigned long long hi = static_cast<unsigned long long>(v >> 64);
  const unsigned long long lo = static_cast<unsigned long long>(v);
  if (hi == 0) return __ull2double_rn(lo);
  const int lz = __clzll(static_cast<long long>(hi));
  const unsigned __int128 n = v << lz;                       // leading one at bit 127
  unsigned long long mant = static_cast<unsigned long long>(n >> 75);  // top 53 bits
  const unsigned __int128 rest = n & ((static_cast<unsigned __int128>(1) << 75) - 1);
  const unsigned __int128 half = static_cast<unsigned __int128>(1) << 74;
  if (rest > half || (rest == half && (mant & 1ull))) ++mant;
  return ldexp(static_cast<double>(mant), 75 - lz);
}

__global__ void __launch_bounds__(256) fast_crt_kernel(const int8_t* __restrict__ W,
                                                       long long w_stride, long long ldw,
                                                       const int* __restrict__ erow,
                                                       const int* __restrict__ ecol, int E,
                                                       const Epilogue ep,
                                                       const __grid_constant__ FastCrtConsts c) {
  const long long i = blockIdx.x;
  const long long j4 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * 4;
  if (j4 >= ep.N) return;
  const unsigned __int128 P = (static_cast<unsigned __int128>(c.P_hi) << 64) | c.P_lo;
  unsigned __int128 S[4] = {0, 0, 0, 0};
  for (int l = 0; l < c.n_mod; ++l) {
    const uint32_t w = __ldg(reinterpret_cast<const uint32_t*>(W + l * w_stride + i * ldw + j4));
    const int p = c.p[l], q = c.q[l];
    const unsigned __int128 Pp = (static_cast<unsigned __int128>(c.Pp_hi[l]) << 64) | c.Pp_lo[l];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      int gg = static_cast<int8_t>((w >> (8 * e)) & 0xffu);
      gg = (gg < 0) ? gg + p : gg;
      const unsigned u = static_cast<unsigned>(gg * q) % static_cast<unsigned>(p);
      unsigned __int128 t = S[e] + Pp * u;   // both < P < 2^126: no overflow
      S[e] = (t >= P) ? t - P : t;
    }
  }
  const int ei = erow[i];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const long long j = j4 + e;
    if (j >= ep.N) break;
    const unsigned __int128 rem = P - S[e];
    const bool neg = S[e] >= rem;            // 2S >= P: the centred value is S - P
    double x = u128_to_double_rne(neg ? rem : S[e]);
    x = neg ? -x : x;
    store_out(ep, i, j, ldexp(x, ei + ecol[j] - 2 * E));
  }
}

// ================================================================= native DGEMM
constexpr int kDgBM = 64, kDgBN = 64, kDgBK = 16;
__global__ void __launch_bounds__(256) dgemm_kernel(const double* __restrict__ A,
                                                    const double* __restrict__ B, long long K,
                                                    const Epilogue ep) {
  __shared__ double As[kDgBK][kDgBM + 1];
  __shared__ double Bs[kDgBK][kDgBN];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long m0 = static_cast<long long>(blockIdx.y) * kDgBM, n0 = static_cast<long long>(blockIdx.x) * kDgBN;
  double acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.0;
  for (long long k0 = 0; k0 < K; k0 += kDgBK) {
    for (int t = threadIdx.x; t < kDgBM * kDgBK; t += 256) {
      const int r = t / kDgBK, kk = t % kDgBK;
      const long long gi = m0 + r, gk = k0 + kk;
      As[kk][r] = (gi < ep.M && gk < K) ? __ldg(A + gi * K + gk) : 0.0;
    }
    for (int t = threadIdx.x; t < kDgBK * kDgBN; t += 256) {
      const int kk = t / kDgBN, cc = t % kDgBN;
      const long long gk = k0 + kk, gj = n0 + cc;
      Bs[kk][cc] = (gk < K && gj < ep.N) ? __ldg(B + gk * ep.N + gj) : 0.0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kDgBK; ++kk) {
      double av[4], bv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) av[a] = As[kk][ty * 4 + a];
#pragma unroll
      for (int b = 0; b < 4; ++b) bv[b] = Bs[kk][tx * 4 + b];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fma(av[a], bv[b], acc[a][b]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const long long i = m0 + ty * 4 + a, j = n0 + tx * 4 + b;
      if (i < ep.M && j < ep.N) store_out(ep, i, j, acc[a][b]);
    }
}

// ======================================================================= conv2d
// Bcol[kk][n], kk = (ic*kH + kh)*kW + kw, n = (b*oH + oh)*oW + ow
__global__ void __launch_bounds__(256) im2col_kernel(const double* __restrict__ in, long long batch,
                                                     long long in_c, long long H, long long W,
                                                     long long kH, long long kW, long long stride,
                                                     long long pad, long long oH, long long oW,
                                                     double* __restrict__ col) {
  const long long ncol = batch * oH * oW;
  const long long n = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long kk = blockIdx.y;
  if (n >= ncol) return;
  const long long kw = kk % kW, kh = (kk / kW) % kH, ic = kk / (kW * kH);
  const long long ow = n % oW, oh = (n / oW) % oH, b = n / (oW * oH);
  const long long ih = oh * stride + kh - pad, iw = ow * stride + kw - pad;
  double v = 0.0;
  if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = __ldg(in + ((b * in_c + ic) * H + ih) * W + iw);
  col[kk * ncol + n] = v;
}

// op numbering of EshkolElementwiseOp; a missing b acts as 0 (add, sub) or 1 (mul, div)
__global__ void __launch_bounds__(256) elementwise_kernel(const double* __restrict__ a,
                                                          const double* __restrict__ b,
                                                          double* __restrict__ out, long long n,
                                                          int op) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(blockDim.x) * gridDim.x) {
    const double x = a[i];
    double r;
    switch (op) {
      case 0: r = x + (b ? b[i] : 0.0); break;
      case 1: r = x - (b ? b[i] : 0.0); break;
      case 2: r = x * (b ? b[i] : 1.0); break;
      case 3: r = x / (b ? b[i] : 1.0); break;
      case 4: r = -x; break;
      case 5: r = fabs(x); break;
      case 6: r = exp(x); break;
      case 7: r = log(x); break;
      case 8: r = sin(x); break;
      case 9: r = cos(x); break;
      case 10: r = tanh(x); break;
      case 11: r = x > 0.0 ? x : 0.0; break;
      case 12: r = 1.0 / (1.0 + exp(-x)); break;
      case 13: r = sqrt(x); break;
      default: r = 1.0 / x; break;
    }
    out[i] = r;
  }
}

}  // namespace

// ------------------------------------------------------------ f16 tier (dtype fast path)
namespace {
// f64 -> f32 -> f16, two roundings to nearest even as the reference's host loop does
// (lib/backend/gpu/gpu_memory_cuda.cpp:691-692: __float2half((float)x))
__device__ __forceinline__ __half to_half_like_reference(double x) {
  return __float2half_rn(static_cast<float>(x));
}

// rows x K f64 row-major -> rows x Kp halves (zero padding up to the 64-element k-block)
__global__ void __launch_bounds__(256) f16_rows_kernel(const double* __restrict__ A, long long K, long long Kp,
                                                       __half* __restrict__ out) {
  const long long i = blockIdx.x;
  const long long k2 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * 2;
  if (k2 >= Kp) return;
  const double* a = A + i * K;
  const __half h0 = (k2 < K) ? to_half_like_reference(a[k2]) : __float2half_rn(0.f);
  const __half h1 = (k2 + 1 < K) ? to_half_like_reference(a[k2 + 1]) : __float2half_rn(0.f);
  *reinterpret_cast<__half2*>(out + i * Kp + k2) = __halves2half2(h0, h1);
}

// K x N f64 row-major -> N x Kp halves (transposed: the products kernel wants both operands K-major)
__global__ void __launch_bounds__(256) f16_cols_kernel(const double* __restrict__ B, long long K, long long N,
                                                       long long Kp, __half* __restrict__ out) {
  __shared__ __half tile[64][66];  // [k][j], pitch 66 halves: conflict-free column reads
  const long long j0 = static_cast<long long>(blockIdx.x) * 64, k0 = static_cast<long long>(blockIdx.y) * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const long long k = k0 + ty + 4 * r, j = j0 + tx;
    tile[ty + 4 * r][tx] = (k < K && j < N) ? to_half_like_reference(B[k * N + j]) : __float2half_rn(0.f);
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 16; ++r) {
    const long long j = j0 + ty + 4 * r, k = k0 + tx;
    if (j < N && k < Kp) out[j * Kp + k] = tile[tx][ty + 4 * r];
  }
}

__global__ void __launch_bounds__(256) widen_f32_kernel(const float* __restrict__ in, long long n, double* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i < n) out[i] = static_cast<double>(in[i]);
}
__global__ void __launch_bounds__(256) narrow_f32_kernel(const double* __restrict__ in, long long n, float* __restrict__ out) {
  const long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (i < n) out[i] = static_cast<float>(in[i]);
}
}  // namespace

// C[b] = half(A[b]) * half(B[b]) for b < batch, f32 accumulation on the tensor cores, the
// result rounded to f16 and widened: what cublasGemmEx(16F, 16F, 16F out, COMPUTE_32F) followed
// by the host widening gives in the reference (gpu_memory_cuda.cpp:677-784), up to the order
// of the f32 accumulation.  One launch covers the whole batch (one job per matrix).
int f16_gemm(const double* dA, const double* dB, double* dC, long long batch, long long M, long long K,
             long long N) {
  if (batch <= 0 || M <= 0 || K <= 0 || N <= 0) return -1;
  const int bn = 256;
  const long long Kp = round_up_ll(K, 64);  // halves; 128-byte k-blocks
  const int tiles_m = static_cast<int>((M + kBM - 1) / kBM), tiles_n = static_cast<int>((N + bn - 1) / bn);
  if (static_cast<long long>(tiles_m) * tiles_n * batch > 0x7fffffffLL || M > 0x7fffff00LL || N > 0x7fffff00LL)
    return -1;
  Carver cv;
  const size_t a_stride = static_cast<size_t>(M) * Kp * 2, b_stride = static_cast<size_t>(N) * Kp * 2;
  const size_t o_jobs = cv.take(sizeof(GemmJob) * batch);
  const size_t o_a = cv.take(a_stride * batch), o_b = cv.take(b_stride * batch);
  uint8_t* ws = workspace_reserve(cv.off);
  if (!ws) return -1;
  GemmJob* d_jobs = reinterpret_cast<GemmJob*>(ws + o_jobs);
  __half* ap = reinterpret_cast<__half*>(ws + o_a);
  __half* bp = reinterpret_cast<__half*>(ws + o_b);
  cudaStream_t st = lib_stream();
  if ((Kp / 2 + 255) / 256 > 65535 || (Kp + 63) / 64 > 65535) return -1;
  for (long long b = 0; b < batch; ++b) {
    const dim3 ga(static_cast<unsigned>(M), static_cast<unsigned>((Kp / 2 + 255) / 256));
    f16_rows_kernel<<<ga, 256, 0, st>>>(dA + b * M * K, K, Kp, ap + b * M * Kp);
    const dim3 gb(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((Kp + 63) / 64));
    f16_cols_kernel<<<gb, 256, 0, st>>>(dB + b * K * N, K, N, Kp, bp + b * N * Kp);
  }
  TIER_CHECK(cudaGetLastError());
  std::vector<GemmJob> jobs(static_cast<size_t>(batch));
  for (long long b = 0; b < batch; ++b) {
    memset(&jobs[b], 0, sizeof(GemmJob));
    jobs[b].n_seg = 1;
    jobs[b].a_plane[0] = static_cast<int>(b); jobs[b].b_plane[0] = static_cast<int>(b);
    jobs[b].out_plane = static_cast<int>(b);
  }
  TIER_CHECK(cudaMemcpyAsync(d_jobs, jobs.data(), sizeof(GemmJob) * jobs.size(), cudaMemcpyHostToDevice, st));
  TIER_CHECK(cudaStreamSynchronize(st));  // the job table above is host memory of this frame
  GemmParams prm = make_gemm_params();
  prm.tiles_m = tiles_m; prm.tiles_n = tiles_n; prm.n_jobs = static_cast<int>(batch);
  prm.kb_per_seg = static_cast<int>(Kp * 2 / kBK);
  prm.kb_per_unit = 1 << 28;
  prm.group_m = 16;
  prm.jobs = d_jobs;
  prm.out = reinterpret_cast<uint8_t*>(dC);
  prm.out_plane_stride = M * N * 8;
  prm.ldo = static_cast<int>(N);
  prm.out_rows = static_cast<int>(M); prm.out_cols = static_cast<int>(N);
  prm.status = lib_status_word();
  prm.work_counter = lib_status_word() + 1;
  CUtensorMap mA, mB;
  if (make_plane_map(&mA, ap, Kp * 2, M, batch, static_cast<long long>(a_stride), kBM)) return -1;
  if (make_plane_map(&mB, bp, Kp * 2, N, batch, static_cast<long long>(b_stride), bn)) return -1;
  TIER_CHECK(launch_modgemm(bn, kEpiF16, mA, mB, prm, static_cast<int>(tiles_m * tiles_n * batch), lib_num_sms(), st));
  count_launches(static_cast<int>(2 * batch + 1));
  return 0;
}

// f32 storage in and out (the reference runs cublasSgemm, gpu_memory_cuda.cpp:653-669): widened,
// multiplied in the exact tier, narrowed with one rounding -- at least as accurate as an f32 GEMM.
int f32_gemm(const float* dA, const float* dB, float* dC, long long M, long long K, long long N) {
  if (M <= 0 || K <= 0 || N <= 0) return -1;
  const size_t ba = (static_cast<size_t>(M) * K * 8 + 1023) & ~size_t(1023),
               bb = (static_cast<size_t>(K) * N * 8 + 1023) & ~size_t(1023);
  uint8_t* t = aux_reserve(ba + bb + static_cast<size_t>(M) * N * 8);
  if (!t) return -1;
  double* wA = reinterpret_cast<double*>(t);
  double* wB = reinterpret_cast<double*>(t + ba);
  double* wC = reinterpret_cast<double*>(t + ba + bb);
  cudaStream_t st = lib_stream();
  widen_f32_kernel<<<static_cast<unsigned>((M * K + 255) / 256), 256, 0, st>>>(dA, M * K, wA);
  widen_f32_kernel<<<static_cast<unsigned>((K * N + 255) / 256), 256, 0, st>>>(dB, K * N, wB);
  TIER_CHECK(cudaGetLastError());
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  o.tier = ESHKOL_B200_TIER_OZAKI2;
  if (eshkol_b200_gemm_f64_device(wA, wB, wC, M, K, N, &o) != 0) return -1;
  narrow_f32_kernel<<<static_cast<unsigned>((M * N + 255) / 256), 256, 0, st>>>(wC, M * N, dC);
  TIER_CHECK(cudaGetLastError());
  count_launches(3);
  return 0;
}

namespace {
// 32 x 32 tiles through padded shared memory: both sides coalesced
__global__ void __launch_bounds__(256) transpose_kernel(const double* __restrict__ src, long long rows,
                                                        long long cols, double* __restrict__ dst) {
  __shared__ double tile[32][33];
  const long long c0 = static_cast<long long>(blockIdx.x) * 32, r0 = static_cast<long long>(blockIdx.y) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const long long r = r0 + ty + 8 * k, c = c0 + tx;
    if (r < rows && c < cols) tile[ty + 8 * k][tx] = src[r * cols + c];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const long long c = c0 + ty + 8 * k, r = r0 + tx;
    if (r < rows && c < cols) dst[c * rows + r] = tile[tx][ty + 8 * k];
  }
}
}  // namespace

cudaError_t launch_transpose(const double* src, long long rows, long long cols, double* dst, cudaStream_t st) {
  if (rows <= 0 || cols <= 0) return cudaSuccess;
  const long long gx = (cols + 31) / 32, gy = (rows + 31) / 32;
  if (gy > 65535) return cudaErrorInvalidValue;
  transpose_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0, st>>>(src, rows, cols, dst);
  return cudaGetLastError();
}

cudaError_t launch_elementwise(const double* a, const double* b, double* out, long long n, int op,
                               cudaStream_t st) {
  long long blocks = (n + 255) / 256;
  const long long cap = static_cast<long long>(lib_num_sms()) * 16;
  if (blocks > cap) blocks = cap;
  elementwise_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(a, b, out, n, op);
  return cudaGetLastError();
}

cudaError_t tiers_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(fast_split_b_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       16 * kTJ * kTPitch * 4);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(oz1_split_b_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              9 * kTJ * kTPitch * 4);
}

int ozaki1_gemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                long long N, int T, const EshkolB200GemmOpts& o) {
  if (T < 1 || T > 8) {
    fprintf(stderr, "[eshkol-b200] Ozaki-I: T=%d outside [1,8]\n", T);
    return -1;
  }
  // gpu_memory_cuda.cpp:351-361: one int8 GEMM is int32-exact only while K*127^2 < 2^31
  if (K > 133000) {
    fprintf(stderr, "[eshkol-b200] Ozaki-I: K=%lld exceeds the int32-exact bound 133000\n", K);
    return -1;
  }
  const int s = T + 1;
  const int bn = (o.gemm_tile_n == 128) ? 128 : 256;
  const long long Kp = round_up_ll(K, kBK);
  const int tiles_m = static_cast<int>((M + kBM - 1) / kBM), tiles_n = static_cast<int>((N + bn - 1) / bn);
  const long long Mp = static_cast<long long>(tiles_m) * kBM, Np = static_cast<long long>(tiles_n) * bn;

  // diagonal plan (gpu_memory_cuda.cpp:364-390): pairs p+q=d share weight 2^-7(d+2);
  // a buffer holds at most `cap` pairs so its int32 sum stays exact
  long long cap = static_cast<long long>(2147483647.0 / (static_cast<double>(K) * 16129.0));
  if (cap < 1) return -1;
  if (cap > kMaxSeg) cap = kMaxSeg;
  std::vector<GemmJob> jobs;
  Oz1Weights wt;
  wt.n = 0;
  for (int d = 0; d <= T; ++d) {
    std::vector<int> ps;
    for (int p = 0; p < s; ++p) { const int q = d - p; if (q >= 0 && q < s) ps.push_back(p); }
    for (size_t off = 0; off < ps.size(); off += static_cast<size_t>(cap)) {
      GemmJob jb;
      memset(&jb, 0, sizeof(jb));
      for (size_t t = off; t < ps.size() && t < off + static_cast<size_t>(cap); ++t) {
        jb.a_plane[jb.n_seg] = ps[t];
        jb.b_plane[jb.n_seg] = d - ps[t];
        ++jb.n_seg;
      }
      jb.out_plane = wt.n;
      if (wt.n >= 24) return -1;
      wt.w[wt.n++] = pow(2.0, -7.0 * (d + 2));
      jobs.push_back(jb);
    }
  }
  const int nbuf = wt.n;

  Carver cv;
  const size_t o_r = cv.take(M * 8), o_c = cv.take(N * 8);
  const size_t o_jobs = cv.take(sizeof(GemmJob) * jobs.size());
  const size_t a_stride = static_cast<size_t>(M) * Kp, b_stride = static_cast<size_t>(N) * Kp;
  const size_t o_a = cv.take(a_stride * s), o_b = cv.take(b_stride * s);
  const size_t g_stride = static_cast<size_t>(Mp) * Np;
  const size_t o_g = cv.take(g_stride * 4 * nbuf);
  uint8_t* ws = workspace_reserve(cv.off);
  if (!ws) return -1;
  double* rmax = reinterpret_cast<double*>(ws + o_r);
  double* cmax = reinterpret_cast<double*>(ws + o_c);
  GemmJob* d_jobs = reinterpret_cast<GemmJob*>(ws + o_jobs);
  int8_t* ap = reinterpret_cast<int8_t*>(ws + o_a);
  int8_t* bp = reinterpret_cast<int8_t*>(ws + o_b);
  int32_t* G = reinterpret_cast<int32_t*>(ws + o_g);
  cudaStream_t st = lib_stream();

  TIER_CHECK(launch_scan_rows(dA, M, K, rmax, st));
  TIER_CHECK(launch_scan_cols(dB, K, N, reinterpret_cast<unsigned long long*>(cmax), st));
  oz1_fix_max_kernel<<<static_cast<unsigned>((M + 255) / 256), 256, 0, st>>>(rmax, M);
  oz1_fix_max_kernel<<<static_cast<unsigned>((N + 255) / 256), 256, 0, st>>>(cmax, N);
  TIER_CHECK(cudaGetLastError());
  {
    const dim3 grid(static_cast<unsigned>(M), static_cast<unsigned>((Kp + 1023) / 1024));
    oz1_split_a_kernel<<<grid, 256, 0, st>>>(dA, rmax, K, Kp, s, ap, static_cast<long long>(a_stride));
    TIER_CHECK(cudaGetLastError());
    const dim3 gridb(static_cast<unsigned>((N + kTJ - 1) / kTJ), static_cast<unsigned>(Kp / kTK));
    oz1_split_b_kernel<<<gridb, 256, static_cast<size_t>(s) * kTJ * kTPitch * 4, st>>>(
        dB, cmax, K, Kp, N, s, bp, static_cast<long long>(b_stride));
    TIER_CHECK(cudaGetLastError());
  }
  TIER_CHECK(cudaMemcpyAsync(d_jobs, jobs.data(), sizeof(GemmJob) * jobs.size(), cudaMemcpyHostToDevice, st));

  GemmParams prm = make_gemm_params();
  prm.tiles_m = tiles_m; prm.tiles_n = tiles_n; prm.n_jobs = nbuf;
  prm.kb_per_seg = static_cast<int>(Kp / kBK);
  prm.kb_per_unit = 1 << 28;
  prm.group_m = 16;
  prm.jobs = d_jobs;
  prm.out = reinterpret_cast<uint8_t*>(G);
  prm.out_plane_stride = static_cast<long long>(g_stride) * 4;
  prm.ldo = static_cast<int>(Np);
  prm.status = lib_status_word();
  prm.work_counter = lib_status_word() + 1;
  if (o.use_simt_products) {
    SimtPlanes sp{ap, static_cast<long long>(a_stride), static_cast<int>(Kp), bp,
                  static_cast<long long>(b_stride), static_cast<int>(Kp), static_cast<int>(M), static_cast<int>(N)};
    TIER_CHECK(launch_modgemm_simt(kEpiRawI32, sp, prm, st));
  } else {
    CUtensorMap mA, mB;
    if (make_plane_map(&mA, ap, Kp, M, s, static_cast<long long>(a_stride), kBM)) return -1;
    if (make_plane_map(&mB, bp, Kp, N, s, static_cast<long long>(b_stride), bn)) return -1;
    TIER_CHECK(launch_modgemm(bn, kEpiRawI32, mA, mB, prm, tiles_m * tiles_n * nbuf, lib_num_sms(), st));
  }
  {
    const dim3 grid(static_cast<unsigned>(M), static_cast<unsigned>((N + 1023) / 1024));
    oz1_reconstruct_kernel<<<grid, 256, 0, st>>>(G, static_cast<long long>(g_stride), Np, wt, rmax, cmax,
                                                 make_epilogue(dC, M, N, o));
    TIER_CHECK(cudaGetLastError());
  }
  count_launches(8);
  return 0;
}

int ozaki2_fast_gemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                     long long N, int n_mod, const EshkolB200GemmOpts& o) {
  if (n_mod < 2 || n_mod > 16) {
    fprintf(stderr, "[eshkol-b200] Ozaki-II fast: moduli count %d outside [2,16]\n", n_mod);
    return -1;
  }
  if (K > 131071) {
    fprintf(stderr, "[eshkol-b200] Ozaki-II fast: K=%lld exceeds the int32-exact bound 131071\n", K);
    return -1;
  }
  const int bn = (o.gemm_tile_n == 128) ? 128 : 256;
  const long long Kp = round_up_ll(K, kBK);
  const int tiles_m = static_cast<int>((M + kBM - 1) / kBM), tiles_n = static_cast<int>((N + bn - 1) / bn);
  const long long Mp = static_cast<long long>(tiles_m) * kBM, Np = static_cast<long long>(tiles_n) * bn;
  Oz2DeviceConsts hc;
  double log2P = 0.0;
  oz2_host_consts(n_mod, &hc, &log2P);
  // gpu_memory.mm:2854-2855
  int E = static_cast<int>(floor((log2P - log2(static_cast<double>(K)) - 2.0) / 2.0));
  if (E > 52) E = 52;
  if (E < 1) E = 1;

  Carver cv;
  const size_t o_amax = cv.take(M * 8), o_bmax = cv.take(N * 8);
  const size_t o_er = cv.take(M * 4), o_ec = cv.take(N * 4);
  const size_t o_jobs = cv.take(sizeof(GemmJob) * 16);
  const size_t a_stride = static_cast<size_t>(M) * Kp, b_stride = static_cast<size_t>(N) * Kp;
  const size_t o_a = cv.take(a_stride * n_mod), o_b = cv.take(b_stride * n_mod);
  const size_t w_stride = static_cast<size_t>(Mp) * Np;
  const size_t o_w = cv.take(w_stride * n_mod);
  uint8_t* ws = workspace_reserve(cv.off);
  if (!ws) return -1;
  double* amax = reinterpret_cast<double*>(ws + o_amax);
  double* bmax = reinterpret_cast<double*>(ws + o_bmax);
  int* er = reinterpret_cast<int*>(ws + o_er);
  int* ec = reinterpret_cast<int*>(ws + o_ec);
  GemmJob* d_jobs = reinterpret_cast<GemmJob*>(ws + o_jobs);
  int8_t* ap = reinterpret_cast<int8_t*>(ws + o_a);
  int8_t* bp = reinterpret_cast<int8_t*>(ws + o_b);
  int8_t* wp = reinterpret_cast<int8_t*>(ws + o_w);
  cudaStream_t st = lib_stream();

  TIER_CHECK(launch_scan_rows(dA, M, K, amax, st));
  TIER_CHECK(launch_scan_cols(dB, K, N, reinterpret_cast<unsigned long long*>(bmax), st));
  fast_exps_kernel<<<static_cast<unsigned>((M + 255) / 256), 256, 0, st>>>(amax, M, er);
  fast_exps_kernel<<<static_cast<unsigned>((N + 255) / 256), 256, 0, st>>>(bmax, N, ec);
  TIER_CHECK(cudaGetLastError());
  {
    const dim3 grid(static_cast<unsigned>(M), static_cast<unsigned>((Kp + 1023) / 1024));
    fast_split_a_kernel<<<grid, 256, 0, st>>>(dA, er, E, K, Kp, ap, static_cast<long long>(a_stride), hc);
    TIER_CHECK(cudaGetLastError());
    const dim3 gridb(static_cast<unsigned>((N + kTJ - 1) / kTJ), static_cast<unsigned>(Kp / kTK));
    fast_split_b_kernel<<<gridb, 256, static_cast<size_t>(n_mod) * kTJ * kTPitch * 4, st>>>(
        dB, ec, E, K, Kp, N, bp, static_cast<long long>(b_stride), hc);
    TIER_CHECK(cudaGetLastError());
  }
  GemmJob jobs[16];
  for (int l = 0; l < n_mod; ++l) {
    memset(&jobs[l], 0, sizeof(GemmJob));
    jobs[l].n_seg = 1;
    jobs[l].a_plane[0] = l; jobs[l].b_plane[0] = l; jobs[l].out_plane = l;
    const unsigned p = static_cast<unsigned>(hc.p_i[l]);
    jobs[l].modulus = p;
    jobs[l].magic = static_cast<unsigned>((1ull << 32) / p);
    jobs[l].offset = static_cast<unsigned>((2147483648ull + p - 1) / p * p);
  }
  TIER_CHECK(cudaMemcpyAsync(d_jobs, jobs, sizeof(GemmJob) * n_mod, cudaMemcpyHostToDevice, st));
  GemmParams prm = make_gemm_params();
  prm.tiles_m = tiles_m; prm.tiles_n = tiles_n; prm.n_jobs = n_mod;
  prm.kb_per_seg = static_cast<int>(Kp / kBK);
  prm.kb_per_unit = 1 << 28;
  prm.group_m = 16;
  prm.jobs = d_jobs;
  prm.out = reinterpret_cast<uint8_t*>(wp);
  prm.out_plane_stride = static_cast<long long>(w_stride);
  prm.ldo = static_cast<int>(Np);
  prm.status = lib_status_word();
  prm.work_counter = lib_status_word() + 1;
  if (o.use_simt_products) {
    SimtPlanes sp{ap, static_cast<long long>(a_stride), static_cast<int>(Kp), bp,
                  static_cast<long long>(b_stride), static_cast<int>(Kp), static_cast<int>(M), static_cast<int>(N)};
    TIER_CHECK(launch_modgemm_simt(kEpiModI8, sp, prm, st));
  } else {
    CUtensorMap mA, mB;
    if (make_plane_map(&mA, ap, Kp, M, n_mod, static_cast<long long>(a_stride), kBM)) return -1;
    if (make_plane_map(&mB, bp, Kp, N, n_mod, static_cast<long long>(b_stride), bn)) return -1;
    TIER_CHECK(launch_modgemm(bn, kEpiModI8, mA, mB, prm, tiles_m * tiles_n * n_mod, lib_num_sms(), st));
  }
  {
    const dim3 grid(static_cast<unsigned>(M), static_cast<unsigned>((N + 1023) / 1024));
    FastCrtConsts fc;
    memset(&fc, 0, sizeof(fc));
    unsigned __int128 P = 1;
    for (int l = 0; l < n_mod; ++l) P *= static_cast<unsigned>(hc.p_i[l]);
    fc.P_hi = static_cast<unsigned long long>(P >> 64);
    fc.P_lo = static_cast<unsigned long long>(P);
    for (int l = 0; l < n_mod; ++l) {
      const unsigned __int128 Pp = P / static_cast<unsigned>(hc.p_i[l]);
      fc.Pp_hi[l] = static_cast<unsigned long long>(Pp >> 64);
      fc.Pp_lo[l] = static_cast<unsigned long long>(Pp);
      fc.p[l] = hc.p_i[l];
      fc.q[l] = hc.q_i[l];
    }
    fc.n_mod = n_mod;
    fast_crt_kernel<<<grid, 256, 0, st>>>(wp, static_cast<long long>(w_stride), Np, er, ec, E,
                                          make_epilogue(dC, M, N, o), fc);
    TIER_CHECK(cudaGetLastError());
  }
  count_launches(8);
  return 0;
}

int native_dgemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                 long long N, const EshkolB200GemmOpts& o) {
  const dim3 grid(static_cast<unsigned>((N + kDgBN - 1) / kDgBN), static_cast<unsigned>((M + kDgBM - 1) / kDgBM));
  if (grid.y > 65535u) return -1;
  dgemm_kernel<<<grid, 256, 0, lib_stream()>>>(dA, dB, K, make_epilogue(dC, M, N, o));
  TIER_CHECK(cudaGetLastError());
  count_launches(1);
  return 0;
}

int conv2d_lowered(const double* d_in, long long batch, long long in_c, long long H, long long W,
                   const double* d_ker, long long out_c, long long kH, long long kW,
                   long long stride, long long pad, double* d_out, const EshkolB200GemmOpts& o_in) {
  if (!d_in || !d_ker || !d_out) return -1;
  if (batch <= 0 || in_c <= 0 || H <= 0 || W <= 0 || out_c <= 0 || kH <= 0 || kW <= 0) return -1;
  if (stride <= 0) stride = 1;  // tensor_conv_kernel.h:51-52, 70-71
  if (pad < 0) pad = 0;
  const long long spanH = H + 2 * pad - kH, spanW = W + 2 * pad - kW;
  if (spanH < 0 || spanW < 0) return 0;  // empty output, as the reference returns
  const long long oH = spanH / stride + 1, oW = spanW / stride + 1;
  const long long Kc = in_c * kH * kW, ncol = batch * oH * oW;
  if (o_in.tier == ESHKOL_B200_TIER_OZAKI2 && (o_in.param == 0 || o_in.param == 16) && !o_in.use_simt_products &&
      H < 0x7fffffffLL && W < 0x7fffffffLL) {
    // exact tier: the scan and the split read the NCHW tensor through the im2col index map
    const Im2colView view{d_in, batch, in_c, H, W, kH, kW, stride, pad, oH, oW};
    EshkolB200GemmOpts o = o_in;
    o.pixels_per_image = oH * oW;
    o.trans_a = o.trans_b = 0;
    return ozaki2_exact_gemm_im2col(d_ker, view, d_out, out_c, Kc, ncol, o);
  }
  if (Kc > 65535) return -1;
  double* col = reinterpret_cast<double*>(aux_reserve(static_cast<size_t>(Kc) * ncol * 8));
  if (!col) return -1;
  const dim3 grid(static_cast<unsigned>((ncol + 255) / 256), static_cast<unsigned>(Kc));
  im2col_kernel<<<grid, 256, 0, lib_stream()>>>(d_in, batch, in_c, H, W, kH, kW, stride, pad, oH, oW, col);
  TIER_CHECK(cudaGetLastError());
  count_launches(1);
  EshkolB200GemmOpts o = o_in;
  o.pixels_per_image = oH * oW;
  return eshkol_b200_gemm_f64_device(d_ker, col, d_out, static_cast<uint64_t>(out_c),
                                     static_cast<uint64_t>(Kc), static_cast<uint64_t>(ncol), &o);
}

// ------------------------------------------------------------ conv2d backward
namespace {
// G[b][c][pix] (NCHW) -> Gm[c][b*pix + pix]: rows of the GEMM operand are channels
__global__ void __launch_bounds__(256) nchw_to_channel_rows_kernel(const double* __restrict__ g, long long batch,
                                                                   long long C, long long pix,
                                                                   double* __restrict__ out) {
  const long long n = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long c = blockIdx.y;
  if (n >= batch * pix) return;
  const long long b = n / pix, p = n - b * pix;
  out[c * batch * pix + n] = __ldg(g + (b * C + c) * pix + p);
}

// col[kk][n], kk = (ci*kH + kh)*kW + kw, n = (b*oH + oh)*oW + ow; no padding, separate strides
__global__ void __launch_bounds__(256) im2col_strides_kernel(const double* __restrict__ in, long long batch,
                                                             long long C, long long H, long long W, long long kH,
                                                             long long kW, long long sH, long long sW,
                                                             long long oH, long long oW, double* __restrict__ col) {
  const long long ncol = batch * oH * oW;
  const long long n = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  const long long kk = blockIdx.y;
  if (n >= ncol) return;
  const long long kw = kk % kW, kh = (kk / kW) % kH, ci = kk / (kW * kH);
  const long long ow = n % oW, oh = (n / oW) % oH, b = n / (oW * oH);
  const long long ih = oh * sH + kh, iw = ow * sW + kw;
  col[kk * ncol + n] = (ih < H && iw < W) ? __ldg(in + ((b * C + ci) * H + ih) * W + iw) : 0.0;
}

// gX[b][ci][ih][iw] = sum over kh, kw (kh outer, as the reference's loop) of Z[(ci,kh,kw)][(b,oh,ow)]
// for the output pixels (oh, ow) = ((ih-kh)/sH, (iw-kw)/sW) that exist: a gather, no atomics
__global__ void __launch_bounds__(256) col2im_gather_kernel(const double* __restrict__ Z, long long batch,
                                                            long long C, long long H, long long W, long long kH,
                                                            long long kW, long long sH, long long sW, long long oH,
                                                            long long oW, double* __restrict__ gx) {
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (idx >= batch * C * H * W) return;
  const long long iw = idx % W, ih = (idx / W) % H, ci = (idx / (W * H)) % C, b = idx / (W * H * C);
  const long long ncol = batch * oH * oW;
  double sum = 0.0;
  for (long long kh = 0; kh < kH; ++kh) {
    const long long oh_c = ih - kh;
    if (oh_c < 0 || oh_c % sH != 0 || oh_c / sH >= oH) continue;
    for (long long kw = 0; kw < kW; ++kw) {
      const long long ow_c = iw - kw;
      if (ow_c < 0 || ow_c % sW != 0 || ow_c / sW >= oW) continue;
      sum = __dadd_rn(sum, __ldg(Z + ((ci * kH + kh) * kW + kw) * ncol + (b * oH + oh_c / sH) * oW + ow_c / sW));
    }
  }
  gx[idx] = sum;
}
}  // namespace

// grad_kernel[co][ci][kh][kw] = sum over (b, oh, ow) of G[b][co][oh][ow] * X[b][ci][oh*sH+kh][ow*sW+kw]
// (lib/backend/gpu/gpu_cuda_kernels.cu:451-486) as one GEMM: (co x b*pix) times im2col(X)^T, the
// im2col matrix read in its own (kk x b*pix) storage.
int conv2d_backward_kernel(const double* d_gout, const double* d_in, double* d_gker, long long H, long long W,
                           long long kH, long long kW, long long oH, long long oW, long long sH, long long sW,
                           long long C_in, long long C_out, long long batch, const EshkolB200GemmOpts& o_in) {
  if (H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || oH <= 0 || oW <= 0 || sH <= 0 || sW <= 0 || C_in <= 0 ||
      C_out <= 0 || batch <= 0)
    return -1;
  const long long Kc = C_in * kH * kW, ncol = batch * oH * oW;
  if (Kc > 65535 || C_out > 65535) return -1;
  const size_t bg = (static_cast<size_t>(C_out) * ncol * 8 + 1023) & ~size_t(1023);
  uint8_t* base = aux_reserve(bg + static_cast<size_t>(Kc) * ncol * 8);
  if (!base) return -1;
  double* gm = reinterpret_cast<double*>(base);
  double* col = reinterpret_cast<double*>(base + bg);
  cudaStream_t st = lib_stream();
  const unsigned gx = static_cast<unsigned>((ncol + 255) / 256);
  nchw_to_channel_rows_kernel<<<dim3(gx, static_cast<unsigned>(C_out)), 256, 0, st>>>(d_gout, batch, C_out, oH * oW, gm);
  im2col_strides_kernel<<<dim3(gx, static_cast<unsigned>(Kc)), 256, 0, st>>>(d_in, batch, C_in, H, W, kH, kW, sH, sW,
                                                                             oH, oW, col);
  TIER_CHECK(cudaGetLastError());
  count_launches(2);
  EshkolB200GemmOpts o = o_in;
  o.trans_a = 0; o.trans_b = 1;
  o.bias = nullptr; o.bias_mode = 0; o.activation = 0; o.pixels_per_image = 0; o.ldc = 0;
  return eshkol_b200_gemm_f64_device(gm, col, d_gker, static_cast<uint64_t>(C_out), static_cast<uint64_t>(ncol),
                                     static_cast<uint64_t>(Kc), &o);
}

// grad_input (gpu_cuda_kernels.cu:413-449): Z = W^T (kk x co) * G (co x b*pix) as one GEMM with W read
// in its own (co x kk) storage, then the gather above.
int conv2d_backward_input(const double* d_gout, const double* d_ker, double* d_gin, long long H, long long W,
                          long long kH, long long kW, long long oH, long long oW, long long sH, long long sW,
                          long long C_in, long long C_out, long long batch, const EshkolB200GemmOpts& o_in) {
  if (H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || oH <= 0 || oW <= 0 || sH <= 0 || sW <= 0 || C_in <= 0 ||
      C_out <= 0 || batch <= 0)
    return -1;
  const long long Kc = C_in * kH * kW, ncol = batch * oH * oW;
  if (C_out > 65535) return -1;
  const size_t bg = (static_cast<size_t>(C_out) * ncol * 8 + 1023) & ~size_t(1023);
  uint8_t* base = aux_reserve(bg + static_cast<size_t>(Kc) * ncol * 8);
  if (!base) return -1;
  double* gm = reinterpret_cast<double*>(base);
  double* Z = reinterpret_cast<double*>(base + bg);
  cudaStream_t st = lib_stream();
  nchw_to_channel_rows_kernel<<<dim3(static_cast<unsigned>((ncol + 255) / 256), static_cast<unsigned>(C_out)), 256, 0,
                                st>>>(d_gout, batch, C_out, oH * oW, gm);
  TIER_CHECK(cudaGetLastError());
  EshkolB200GemmOpts o = o_in;
  o.trans_a = 1; o.trans_b = 0;
  o.bias = nullptr; o.bias_mode = 0; o.activation = 0; o.pixels_per_image = 0; o.ldc = 0;
  if (eshkol_b200_gemm_f64_device(d_ker, gm, Z, static_cast<uint64_t>(Kc), static_cast<uint64_t>(C_out),
                                  static_cast<uint64_t>(ncol), &o) != 0)
    return -1;
  const long long total = batch * C_in * H * W;
  col2im_gather_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, st>>>(Z, batch, C_in, H, W, kH, kW, sH,
                                                                                   sW, oH, oW, d_gin);
  TIER_CHECK(cudaGetLastError());
  count_launches(2);
  return 0;
}

}  // namespace b200
