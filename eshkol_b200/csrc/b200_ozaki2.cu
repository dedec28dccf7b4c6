// Bandwidth-bound stages of the Ozaki-II exact f64 GEMM:
//   scan      per-row max|A|, per-column max|B|
//   scales    mu_i = E - floor(log2 amax_i), nu_j likewise, and the 2^(+/-mu) factors
//   split     trunc(a * 2^mu) -> residues for every modulus, int8 planes (+ two flag
//             bit-planes for modulus 256, whose representative +128 does not fit int8)
//             (A planes row-major M x Kp, B planes TRANSPOSED to N x Kp so both GEMM
//             operands are K-major), 128-bit loads, whole-word / 16-byte stores
//   crt       S1/S2 accumulation over the residue planes of the products, Q, the two
//             fma's of the reconstruction and the two exact descalings -> f64 C
//
// Arithmetic restated from the reference's host code, lib/backend/gpu/gpu_memory.mm:
// scales :2514-2532, integerisation :2538-2547, residues :2573-2583, CRT accumulation
// :2619-2641, reconstruction :2644-2655 (see the notes on each kernel).
#include "b200_common.cuh"
#include "b200_internal.h"
#include "b200_ozaki2.h"
#include <stdlib.h>
#include "b200_residue.cuh"

#include <math.h>

namespace b200 {

namespace {

__device__ __forceinline__ double dmax_ref(double mx, double v) {
  // the reference's update "if (v > mx) mx = v": a NaN never replaces the maximum
  return (v > mx) ? v : mx;
}

// ------------------------------------------------------------------- row scan
// One warp per row of A.
__global__ void __launch_bounds__(256) scan_rows_kernel(const double* __restrict__ A, long long M,
                                                        long long K, double* __restrict__ amax) {
  const long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const double* p = A + row * K;
  double mx = 0.0;
  const long long head = ((reinterpret_cast<uintptr_t>(p) & 8) && K > 0) ? 1 : 0;
  if (lane == 0 && head) mx = dmax_ref(mx, fabs(p[0]));
  const long long npair = (K - head) >> 1;
  const double2* p2 = reinterpret_cast<const double2*>(p + head);
  long long i = lane;
  for (; i + 96 < npair; i += 128) {  // four independent 16-byte loads in flight
    const double2 v0 = __ldg(p2 + i), v1 = __ldg(p2 + i + 32), v2 = __ldg(p2 + i + 64),
                  v3 = __ldg(p2 + i + 96);
    mx = dmax_ref(mx, fabs(v0.x)); mx = dmax_ref(mx, fabs(v0.y));
    mx = dmax_ref(mx, fabs(v1.x)); mx = dmax_ref(mx, fabs(v1.y));
    mx = dmax_ref(mx, fabs(v2.x)); mx = dmax_ref(mx, fabs(v2.y));
    mx = dmax_ref(mx, fabs(v3.x)); mx = dmax_ref(mx, fabs(v3.y));
  }
  for (; i < npair; i += 32) {
    const double2 v = __ldg(p2 + i);
    mx = dmax_ref(mx, fabs(v.x)); mx = dmax_ref(mx, fabs(v.y));
  }
  if (lane == 0 && ((K - head) & 1)) mx = dmax_ref(mx, fabs(p[K - 1]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = dmax_ref(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) amax[row] = mx;
}

// ------------------------------------------------- the operand as an im2col view
// Where column n of the view starts in the tensor: image base, top-left input coordinate.
// All of it in 32-bit arithmetic (the launchers refuse extents beyond int).
struct ViewColumn {
  long long base;
  int ih0, iw0;
};
__device__ __forceinline__ ViewColumn view_column(const Im2colView& v, long long n) {
  const int oW = static_cast<int>(v.oW), oH = static_cast<int>(v.oH);
  const int t = static_cast<int>(n / oW), ow = static_cast<int>(n - static_cast<long long>(t) * oW);
  const int b = t / oH, oh = t - b * oH;
  ViewColumn c;
  c.base = static_cast<long long>(b) * v.in_c * v.H * v.W;
  c.ih0 = oh * static_cast<int>(v.stride) - static_cast<int>(v.pad);
  c.iw0 = ow * static_cast<int>(v.stride) - static_cast<int>(v.pad);
  return c;
}
// kernel tap of row kk: (ic, kh, kw)
struct ViewTap {
  int ic, kh, kw;
};
__device__ __forceinline__ ViewTap view_tap(const Im2colView& v, int kk) {
  const int kW = static_cast<int>(v.kW), kH = static_cast<int>(v.kH);
  ViewTap t;
  const int q = kk / kW;
  t.kw = kk - q * kW;
  t.ic = q / kH;
  t.kh = q - t.ic * kH;
  return t;
}
__device__ __forceinline__ void view_tap_next(const Im2colView& v, ViewTap& t) {
  if (++t.kw == static_cast<int>(v.kW)) {
    t.kw = 0;
    if (++t.kh == static_cast<int>(v.kH)) { t.kh = 0; ++t.ic; }
  }
}
__device__ __forceinline__ double view_load(const Im2colView& v, const ViewColumn& c, const ViewTap& t) {
  const int ih = c.ih0 + t.kh, iw = c.iw0 + t.kw;
  const int H = static_cast<int>(v.H), W = static_cast<int>(v.W);
  if (ih < 0 || ih >= H || iw < 0 || iw >= W) return 0.0;
  return __ldg(v.in + c.base + (static_cast<long long>(t.ic) * H + ih) * W + iw);
}

// Column maxima of the view without walking it: first the maximum over the channels of every
// input pixel (the tensor is read once), then for every output pixel the maximum over its
// kH x kW window of that image.
__global__ void __launch_bounds__(256) view_channel_max_kernel(const Im2colView v, double* __restrict__ cmax) {
  const long long plane = v.H * v.W;
  const long long idx = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;  // (b, ih, iw)
  if (idx >= v.batch * plane) return;
  const long long b = idx / plane, pix = idx - b * plane;
  const double* p = v.in + b * v.in_c * plane + pix;
  double mx = 0.0;
  for (long long ic = 0; ic < v.in_c; ++ic) mx = dmax_ref(mx, fabs(__ldg(p + ic * plane)));
  cmax[idx] = mx;
}
__global__ void __launch_bounds__(256) view_window_max_kernel(const Im2colView v, const double* __restrict__ cmax,
                                                              long long N, double* __restrict__ bmax) {
  const long long n = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  if (n >= N) return;
  const ViewColumn c = view_column(v, n);
  const long long plane = v.H * v.W;
  const double* img = cmax + (c.base / (v.in_c * plane)) * plane;
  double mx = 0.0;
  for (int kh = 0; kh < static_cast<int>(v.kH); ++kh) {
    const int ih = c.ih0 + kh;
    if (ih < 0 || ih >= static_cast<int>(v.H)) continue;
    for (int kw = 0; kw < static_cast<int>(v.kW); ++kw) {
      const int iw = c.iw0 + kw;
      if (iw < 0 || iw >= static_cast<int>(v.W)) continue;
      mx = dmax_ref(mx, img[static_cast<long long>(ih) * v.W + iw]);
    }
  }
  bmax[n] = mx;
}

// ---------------------------------------------------------------- column scan
// Block = 64 columns x 4 row phases over a slab of rows; partial maxima merge
// through atomicMax on the bit pattern (order-preserving for non-negative doubles).
constexpr int kColSlab = 256;
__global__ void __launch_bounds__(256) scan_cols_kernel(const double* __restrict__ B, long long K,
                                                        long long N, long long ld,
                                                        unsigned long long* __restrict__ bmax_bits) {
  __shared__ double red[4][64];
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  const long long j = static_cast<long long>(blockIdx.x) * 64 + tx;
  const long long k0 = static_cast<long long>(blockIdx.y) * kColSlab;
  const long long k1 = (k0 + kColSlab < K) ? k0 + kColSlab : K;
  double mx = 0.0;
  if (j < N) {
    long long k = k0 + ty;
    for (; k + 12 < k1; k += 16) {
      const double v0 = __ldg(B + k * ld + j), v1 = __ldg(B + (k + 4) * ld + j),
                   v2 = __ldg(B + (k + 8) * ld + j), v3 = __ldg(B + (k + 12) * ld + j);
      mx = dmax_ref(mx, fabs(v0)); mx = dmax_ref(mx, fabs(v1));
      mx = dmax_ref(mx, fabs(v2)); mx = dmax_ref(mx, fabs(v3));
    }
    for (; k < k1; k += 4) mx = dmax_ref(mx, fabs(__ldg(B + k * ld + j)));
  }
  red[ty][tx] = mx;
  __syncthreads();
  if (ty == 0 && j < N) {
    mx = dmax_ref(mx, red[1][tx]);
    mx = dmax_ref(mx, red[2][tx]);
    mx = dmax_ref(mx, red[3][tx]);
    if (mx > 0.0) atomicMax(bmax_bits + j, static_cast<unsigned long long>(__double_as_longlong(mx)));
  }
}

// floor(log2(x)) for finite x > 0 as a correctly rounded log2 followed by floor
// returns it (the reference calls libm): equal to the exponent field except for
// the few largest doubles below 2^t with |t| >= 3, whose logarithm rounds to t.
__device__ int floor_log2_ref(double x) {
  const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(x));
  const int ef = static_cast<int>((bits >> 52) & 0x7ff);
  const unsigned long long man = bits & ((1ull << 52) - 1);
  int e;
  unsigned long long sig;
  if (ef == 0) {
    if (man == 0) return 0;
    const int lz = __clzll(static_cast<long long>(man)) - 11;
    sig = man << lz;
    e = -1022 - lz;
  } else {
    sig = man | (1ull << 52);
    e = ef - 1023;
  }
  const unsigned long long m = (1ull << 53) - sig;
  const int t = e + 1;
  if (t == 0 || m > 2048ull) return e;
  const int a = t < 0 ? -t : t;
  const int lg = 31 - __clz(a);
  const bool pow2 = (a & (a - 1)) == 0;
  const double thr = (t > 0 && pow2) ? ldexp(1.0, lg - 1) : ldexp(1.0, lg);
  return (static_cast<double>(m) * 1.4426950408889634 < thr) ? t : e;
}

// gpu_memory.mm:2523/2531: shift = (max == 0) ? 0 : E - floor(log2(max))
__global__ void scales_kernel(const double* __restrict__ vmax, long long n, int E,
                              int* __restrict__ shift, double* __restrict__ scale,
                              double* __restrict__ inv_scale) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const double mx = vmax[i];
  const int s = (mx == 0.0) ? 0 : E - floor_log2_ref(mx);
  shift[i] = s;
  scale[i] = ldexp(1.0, s);
  inv_scale[i] = ldexp(1.0, -s);
}

struct SplitGeom {
  long long rows;      // M for A, N for B
  long long K, Kp;     // logical and padded (multiple of 128) inner extent
  long long K0;        // inner extent of the modulus-256 plane (1024 per chunk of 1008)
  int n_chunks;        // ceil(K / 1008)
  int n_odd;           // number of odd-modulus planes (n_mod - 1)
  int8_t* plane0;      // rows x K0: the residue bytes modulo 256
  uint16_t* flag_hi;   // rows x n_chunks x 64 units: residue == +128
  uint16_t* flag_odd;  // rows x n_chunks x 64 units: residue odd
  int8_t* odd;         // n_odd planes of rows x Kp
  long long odd_stride;
};

// element k of a row -> column inside the modulus-256 plane and 16-bit flag unit
__device__ __forceinline__ void chunk_cols(const SplitGeom& g, long long k, long long* col,
                                           long long* unit) {
  const int c = static_cast<int>(k / kChunkK);
  const int off = static_cast<int>(k - static_cast<long long>(c) * kChunkK);
  *col = static_cast<long long>(c) * kChunkSeg + off;
  *unit = static_cast<long long>(c) * kChunkUnits + (off >> 4);
}

// A: one thread per 8 consecutive k of one row (64 bytes in flight per thread, 8-byte stores);
// grid = (rows, ceil(Kp/2048)).
constexpr int kSplitAW = 8;
__global__ void __launch_bounds__(256) split_a_kernel(const double* __restrict__ A,
                                                      const double* __restrict__ scale,
                                                      const SplitGeom g,
                                                      const __grid_constant__ Oz2DeviceConsts c) {
  const long long row = blockIdx.x;
  const long long k8 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * kSplitAW;
  if (k8 >= g.Kp) return;
  const double* src = A + row * g.K + k8;
  double a[kSplitAW];
  if (k8 + kSplitAW - 1 < g.K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const double2* s2 = reinterpret_cast<const double2*>(src);
    const double2 v0 = __ldg(s2), v1 = __ldg(s2 + 1), v2 = __ldg(s2 + 2), v3 = __ldg(s2 + 3);
    a[0] = v0.x; a[1] = v0.y; a[2] = v1.x; a[3] = v1.y; a[4] = v2.x; a[5] = v2.y; a[6] = v3.x; a[7] = v3.y;
  } else {
#pragma unroll
    for (int e = 0; e < kSplitAW; ++e) a[e] = (k8 + e < g.K) ? __ldg(src + e) : 0.0;
  }
  const double s = scale[row];
  double x[kSplitAW];
  uint32_t xlo[kSplitAW];
#pragma unroll
  for (int e = 0; e < kSplitAW; ++e) {
    x[e] = trunc(a[e] * s);  // gpu_memory.mm:2541
    xlo[e] = static_cast<uint32_t>(static_cast<long long>(x[e]));
  }

  const long long o = row * g.Kp + k8;
  // plane 0 is modulus 255, the only one whose residue can come out as +128
  int8_t* dst_odd = g.odd + o;
  {
    const double p_inv = c.p_inv[1];
    *reinterpret_cast<uint2*>(dst_odd) = make_uint2(
        pack_bytes4(residue_odd_t<true>(x[0], xlo[0], p_inv, 255), residue_odd_t<true>(x[1], xlo[1], p_inv, 255),
                    residue_odd_t<true>(x[2], xlo[2], p_inv, 255), residue_odd_t<true>(x[3], xlo[3], p_inv, 255)),
        pack_bytes4(residue_odd_t<true>(x[4], xlo[4], p_inv, 255), residue_odd_t<true>(x[5], xlo[5], p_inv, 255),
                    residue_odd_t<true>(x[6], xlo[6], p_inv, 255), residue_odd_t<true>(x[7], xlo[7], p_inv, 255)));
  }
#pragma unroll 7
  for (int l = 1; l < g.n_odd; ++l) {
    const double p_inv = c.p_inv[l + 1];
    const int pi = c.p_i[l + 1];
    dst_odd += g.odd_stride;
    *reinterpret_cast<uint2*>(dst_odd) = make_uint2(
        pack_bytes4(residue_odd_t<false>(x[0], xlo[0], p_inv, pi), residue_odd_t<false>(x[1], xlo[1], p_inv, pi),
                    residue_odd_t<false>(x[2], xlo[2], p_inv, pi), residue_odd_t<false>(x[3], xlo[3], p_inv, pi)),
        pack_bytes4(residue_odd_t<false>(x[4], xlo[4], p_inv, pi), residue_odd_t<false>(x[5], xlo[5], p_inv, pi),
                    residue_odd_t<false>(x[6], xlo[6], p_inv, pi), residue_odd_t<false>(x[7], xlo[7], p_inv, pi)));
  }
  // modulus 256: the bytes, and the two flag bits of each element gathered into 16-bit
  // units along k (2 lanes x 8 elements; chunk boundaries are multiples of 16)
  uint32_t w0 = 0, w1 = 0, b_hi = 0, b_odd = 0;
#pragma unroll
  for (int e = 0; e < kSplitAW; ++e) {
    const Res256 r = residue_256(xlo[e]);
    if (e < 4) w0 |= r.lo8 << (8 * e); else w1 |= r.lo8 << (8 * (e - 4));
    b_hi |= r.hi << e;
    b_odd |= r.odd << e;
  }
  const int sh = 8 * (threadIdx.x & 1);
  uint32_t u_hi = b_hi << sh, u_odd = b_odd << sh;
  u_hi |= __shfl_xor_sync(0xffffffffu, u_hi, 1);
  u_odd |= __shfl_xor_sync(0xffffffffu, u_odd, 1);
  if (k8 < g.K) {
    long long col, unit;
    chunk_cols(g, k8, &col, &unit);
    *reinterpret_cast<uint2*>(g.plane0 + row * g.K0 + col) = make_uint2(w0, w1);
    if ((threadIdx.x & 1) == 0) {
      const long long fo = row * g.n_chunks * kChunkUnits + unit;
      g.flag_hi[fo] = static_cast<uint16_t>(u_hi);
      g.flag_odd[fo] = static_cast<uint16_t>(u_odd);
    }
  }
}

// B (K x N row-major) -> planes N x Kp.  Block = 32 columns x 128 k; loads are
// coalesced along j, residues are packed 4-per-word along k into shared memory
// (row pitch 33 words: conflict-free both ways), then written out as 16-byte
// vectors along k.
constexpr int kSplitBJ = 32, kSplitBK = 128, kSplitBPitch = 33;
template <bool kView>
__global__ void __launch_bounds__(256) split_b_kernel(const double* __restrict__ B,
                                                      const double* __restrict__ scale,
                                                      long long N, long long ld, const SplitGeom g,
                                                      const __grid_constant__ Oz2DeviceConsts c,
                                                      const __grid_constant__ Im2colView view) {
  extern __shared__ uint32_t sm[];  // [n_odd + 2][32][33]: bytes mod 256, flag nibbles, odd moduli
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const long long j = static_cast<long long>(blockIdx.x) * kSplitBJ + tx;
  const long long kbase = static_cast<long long>(blockIdx.y) * kSplitBK;
  const double s = (j < N) ? scale[j] : 0.0;
  const int n_planes = g.n_odd + 2;
  // all 16 loads of this thread are issued before any arithmetic: two resident blocks
  // per SM then keep 64 KB of reads in flight, enough to cover HBM latency
  double bv[4][4];
  if (kView) {
    const ViewColumn vc = view_column(view, (j < N) ? j : 0);
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const long long k = kbase + (ty + 8 * t) * 4;
      ViewTap tap = view_tap(view, static_cast<int>(k));
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        bv[t][e] = (j < N && k + e < g.K) ? view_load(view, vc, tap) : 0.0;
        view_tap_next(view, tap);
      }
    }
  } else {
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const long long k = kbase + (ty + 8 * t) * 4;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        bv[t][e] = (j < N && k + e < g.K) ? __ldg(B + (k + e) * ld + j) : 0.0;
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int qd = ty + 8 * t;
    double x[4];
    uint32_t xlo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      x[e] = trunc(bv[t][e] * s);  // gpu_memory.mm:2546
      xlo[e] = static_cast<uint32_t>(static_cast<long long>(x[e]));
    }
    uint32_t w0 = 0, nib = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const Res256 r = residue_256(xlo[e]);
      w0 |= r.lo8 << (8 * e);
      nib |= (r.odd << e) | (r.hi << (8 + e));  // byte 0: odd flags, byte 1: +128 flags
    }
    sm[(0 * kSplitBJ + tx) * kSplitBPitch + qd] = w0;
    sm[(1 * kSplitBJ + tx) * kSplitBPitch + qd] = nib;
    {
      const double p_inv = c.p_inv[1];  // modulus 255: the only residue that can come out as +128
      sm[(2 * kSplitBJ + tx) * kSplitBPitch + qd] =
          pack_bytes4(residue_odd_t<true>(x[0], xlo[0], p_inv, 255), residue_odd_t<true>(x[1], xlo[1], p_inv, 255),
                      residue_odd_t<true>(x[2], xlo[2], p_inv, 255), residue_odd_t<true>(x[3], xlo[3], p_inv, 255));
    }
#pragma unroll 7
    for (int l = 1; l < g.n_odd; ++l) {
      const double p_inv = c.p_inv[l + 1];
      const int pi = c.p_i[l + 1];
      sm[((2 + l) * kSplitBJ + tx) * kSplitBPitch + qd] =
          pack_bytes4(residue_odd_t<false>(x[0], xlo[0], p_inv, pi), residue_odd_t<false>(x[1], xlo[1], p_inv, pi),
                      residue_odd_t<false>(x[2], xlo[2], p_inv, pi), residue_odd_t<false>(x[3], xlo[3], p_inv, pi));
    }
  }
  __syncthreads();
  // write-out: thread = (column jj, 16-byte group gq of the 128-k tile)
  const int jj = threadIdx.x >> 3, gq = threadIdx.x & 7;
  const long long jo = static_cast<long long>(blockIdx.x) * kSplitBJ + jj;
  if (jo >= N) return;
  const long long k16 = kbase + gq * 16;
  for (int pl = 0; pl < n_planes; ++pl) {
    const uint32_t* srcw = &sm[(pl * kSplitBJ + jj) * kSplitBPitch + gq * 4];
    if (pl >= 2) {
      if (k16 < g.Kp)
        *reinterpret_cast<uint4*>(g.odd + (pl - 2) * g.odd_stride + jo * g.Kp + k16) =
            make_uint4(srcw[0], srcw[1], srcw[2], srcw[3]);
    } else if (k16 < g.K) {
      long long col, unit;
      chunk_cols(g, k16, &col, &unit);
      if (pl == 0) {
        *reinterpret_cast<uint4*>(g.plane0 + jo * g.K0 + col) = make_uint4(srcw[0], srcw[1], srcw[2], srcw[3]);
      } else {
        // four nibbles per flag -> one 16-bit unit each
        const uint32_t f_odd = (srcw[0] & 15u) | ((srcw[1] & 15u) << 4) | ((srcw[2] & 15u) << 8) |
                               ((srcw[3] & 15u) << 12);
        const uint32_t f_hi = ((srcw[0] >> 8) & 15u) | (((srcw[1] >> 8) & 15u) << 4) |
                              (((srcw[2] >> 8) & 15u) << 8) | (((srcw[3] >> 8) & 15u) << 12);
        const long long fo = jo * g.n_chunks * kChunkUnits + unit;
        g.flag_odd[fo] = static_cast<uint16_t>(f_odd);
        g.flag_hi[fo] = static_cast<uint16_t>(f_hi);
      }
    }
  }
}

// ------------------------------------------------------------------------ CRT
// One thread per kCrtW consecutive columns of one row.  grid = (M, ceil(N / (256 * kCrtW))).
// gpu_memory.mm:2632-2640 (S1/S2 in modulus order, fused) and :2650-2653.
// The kernel is bound by instruction issue, not by HBM (17 bytes in, 8 out per element): eight
// columns per thread halve the loads and the address arithmetic per element, and the 16
// independent accumulation chains of a thread keep the FP64 pipe fed.
constexpr int kCrtW = 8;
// kMode 0: 16 moduli, no bias, no activation, row-major C (decided at launch); 1: the general
// form without GELU; 2: with it.  The general form carries the run-time switches of the epilogue
// (and, for GELU, eight inlined exponentials and divisions) through the whole kernel -- 0.78
// against 0.41 ms at 8192^2 -- so the plain product, which is what a GEMM call is, has its own
// instance.
template <int kMode>
__global__ void __launch_bounds__(256) crt_kernel(const CrtArgs a,
                                                  const __grid_constant__ Oz2DeviceConsts c) {
  constexpr bool kPlain = kMode == 0;
  const long long i = blockIdx.x;
  const long long j0 = (static_cast<long long>(blockIdx.y) * 256 + threadIdx.x) * kCrtW;
  if (j0 >= a.N) return;
  const long long wo = i * a.ldw + j0;
  const int n_mod = kPlain ? 16 : a.n_mod;
  double S1[kCrtW], S2[kCrtW];
  {
    // modulus 256: finish the reduction the products kernel left open -- apply the tie
    // corrections, then centre with the half-even rule (+128 iff the sum is 128 mod 512)
    const uint4 w = __ldg(reinterpret_cast<const uint4*>(a.w0 + wo));
    const uint32_t fl = __ldg(a.flip + i * (a.ldw >> 5) + (j0 >> 5)) >> (j0 & 31);
    const uint32_t raw[kCrtW] = {w.x & 0xffffu, w.x >> 16, w.y & 0xffffu, w.y >> 16,
                                 w.z & 0xffffu, w.z >> 16, w.w & 0xffffu, w.w >> 16};
    const double s1 = c.sl1[0], s2 = c.sl2[0];
#pragma unroll
    for (int e = 0; e < kCrtW; ++e) {
      const uint32_t x = (raw[e] + (((fl >> e) & 1u) << 8)) & 511u;
      const int v = (x == 128u) ? 128 : static_cast<int>((x + 128u) & 255u) - 128;
      const double wd = static_cast<double>(v);
      S1[e] = __dmul_rn(s1, wd);  // fma(s1, wd, 0.0): the first term of the sum
      S2[e] = __dmul_rn(s2, wd);
    }
  }
  // the planes are fetched in two groups, each group's words requested before its first use
#pragma unroll
  for (int l0 = 1; l0 < 16; l0 += 8) {
    uint2 wv[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int l = l0 + t;
      wv[t] = (l < 16 && l < n_mod)
                  ? __ldg(reinterpret_cast<const uint2*>(a.w_odd + (l - 1) * a.w_odd_stride + wo))
                  : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int l = l0 + t;
      if (l < 16 && l < n_mod) {
        const double s1 = c.sl1[l], s2 = c.sl2[l];
        // signed byte -> double through the mantissa: (2^52 + (b + 128)) - (2^52 + 128), exact,
        // on the FP64 add pipe instead of the slower integer-to-double conversion unit
        const uint32_t lo = wv[t].x ^ 0x80808080u, hi = wv[t].y ^ 0x80808080u;
#pragma unroll
        for (int e = 0; e < kCrtW; ++e) {
          const uint32_t byte = __byte_perm(e < 4 ? lo : hi, 0u, 0x4440 + (e & 3));
          const double wd = __hiloint2double(0x43300000, static_cast<int>(byte)) - 4503599627370624.0;
          S1[e] = fma(s1, wd, S1[e]);
          S2[e] = fma(s2, wd, S2[e]);
        }
      }
    }
  }
  const double mu_inv = a.inv_scale_a[i];
  const double P1 = c.P1, P2 = c.P2, Pinv = c.Pinv;
  double sb[kCrtW];
  if (j0 + kCrtW - 1 < a.N && (reinterpret_cast<uintptr_t>(a.inv_scale_b + j0) & 15) == 0) {
#pragma unroll
    for (int h = 0; h < kCrtW / 2; ++h) {
      const double2 t = __ldg(reinterpret_cast<const double2*>(a.inv_scale_b + j0) + h);
      sb[2 * h] = t.x;
      sb[2 * h + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int e = 0; e < kCrtW; ++e) sb[e] = a.inv_scale_b[(j0 + e < a.N) ? j0 + e : a.N - 1];
  }
  double out[kCrtW];
#pragma unroll
  for (int e = 0; e < kCrtW; ++e) {
    const double s = __dadd_rn(S1[e], S2[e]);
    const double q = __dmul_rn(s, Pinv);
    const double Q = round(q);  // half away from zero
    const double c1 = fma(-P1, Q, S1[e]);
    const double c2 = fma(-P2, Q, S2[e]);
    double v = __dmul_rn(__dmul_rn(__dadd_rn(c1, c2), mu_inv), sb[e]);
    if (!kPlain) {
      const long long j = (j0 + e < a.N) ? j0 + e : a.N - 1;
      if (a.bias_mode == 1) v = __dadd_rn(v, a.bias[i]);
      else if (a.bias_mode == 2) v = __dadd_rn(v, a.bias[j]);
      if (kMode == 2) v = apply_activation(v, a.activation);
      else if (a.activation == 1) v = (v > 0.0) ? v : 0.0;  // apply_activation's ReLU
    }
    out[e] = v;
  }
  if (!kPlain && a.pixels_per_image > 0) {
#pragma unroll
    for (int e = 0; e < kCrtW; ++e) {
      const long long j = j0 + e;
      if (j >= a.N) break;
      const long long img = j / a.pixels_per_image, pix = j - img * a.pixels_per_image;
      a.C[(img * a.M + i) * a.pixels_per_image + pix] = out[e];  // [image][row][pixel]
    }
    return;
  }
  double* dst = a.C + i * a.ldc + j0;
  if (j0 + kCrtW - 1 < a.N && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
    // 32-byte stores: whole sectors, a quarter of the store instructions
#pragma unroll
    for (int h = 0; h < kCrtW / 4; ++h)
      asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 4 * h),
                   "f"(__int_as_float(__double2loint(out[4 * h]))), "f"(__int_as_float(__double2hiint(out[4 * h]))),
                   "f"(__int_as_float(__double2loint(out[4 * h + 1]))), "f"(__int_as_float(__double2hiint(out[4 * h + 1]))),
                   "f"(__int_as_float(__double2loint(out[4 * h + 2]))), "f"(__int_as_float(__double2hiint(out[4 * h + 2]))),
                   "f"(__int_as_float(__double2loint(out[4 * h + 3]))), "f"(__int_as_float(__double2hiint(out[4 * h + 3])))
                   : "memory");
  } else {
#pragma unroll
    for (int e = 0; e < kCrtW; ++e)
      if (j0 + e < a.N) dst[e] = out[e];
  }
}

}  // namespace

cudaError_t launch_scan_rows(const double* A, long long M, long long K, double* amax,
                             cudaStream_t st) {
  if (M <= 0) return cudaSuccess;
  scan_rows_kernel<<<static_cast<unsigned>((M + 7) / 8), 256, 0, st>>>(A, M, K, amax);
  return cudaGetLastError();
}

cudaError_t launch_scan_cols(const double* B, long long K, long long N,
                             unsigned long long* bmax_bits, cudaStream_t st, long long ld) {
  if (ld <= 0) ld = N;
  if (N <= 0 || K <= 0) return cudaSuccess;
  cudaError_t e = cudaMemsetAsync(bmax_bits, 0, static_cast<size_t>(N) * 8, st);
  if (e != cudaSuccess) return e;
  const dim3 grid(static_cast<unsigned>((N + 63) / 64), static_cast<unsigned>((K + kColSlab - 1) / kColSlab));
  if (grid.y > 65535u) return cudaErrorInvalidValue;
  scan_cols_kernel<<<grid, 256, 0, st>>>(B, K, N, ld, bmax_bits);
  return cudaGetLastError();
}

cudaError_t launch_scan_view(const Im2colView& view, long long N, double* pixel_max, double* bmax, cudaStream_t st) {
  const long long pixels = view.batch * view.H * view.W;
  if (N <= 0 || pixels <= 0) return cudaSuccess;
  if (view.H * view.W > 0x7fffffffLL || view.in_c * view.kH * view.kW > 0x7fffffffLL ||
      N / view.oW > 0x7fffffffLL)
    return cudaErrorInvalidValue;
  view_channel_max_kernel<<<static_cast<unsigned>((pixels + 255) / 256), 256, 0, st>>>(view, pixel_max);
  view_window_max_kernel<<<static_cast<unsigned>((N + 255) / 256), 256, 0, st>>>(view, pixel_max, N, bmax);
  return cudaGetLastError();
}

cudaError_t launch_scales(const double* vmax, long long n, int E, int* shift, double* scale,
                          double* inv_scale, cudaStream_t st) {
  if (n <= 0) return cudaSuccess;
  scales_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(vmax, n, E, shift, scale,
                                                                        inv_scale);
  return cudaGetLastError();
}

// the padding inside the modulus-256 plane and the unused flag units must read as zero
static cudaError_t clear_plane0(const SplitPlanes& p, cudaStream_t st) {
  const size_t fbytes = static_cast<size_t>(p.rows) * p.n_chunks * kChunkUnits * sizeof(uint16_t);
  const uint8_t* b0 = reinterpret_cast<const uint8_t*>(p.plane0);
  const uint8_t* f1 = reinterpret_cast<const uint8_t*>(p.flag_hi);
  const uint8_t* f2 = reinterpret_cast<const uint8_t*>(p.flag_odd);
  // the drivers carve the three pieces one behind the other: one fill then covers them all
  if (b0 < f1 && f1 < f2 && static_cast<size_t>(f1 - b0) < static_cast<size_t>(p.rows) * p.K0 + 1024 &&
      static_cast<size_t>(f2 - f1) < fbytes + 1024)
    return cudaMemsetAsync(p.plane0, 0, static_cast<size_t>(f2 - b0) + fbytes, st);
  cudaError_t e = cudaMemsetAsync(p.plane0, 0, static_cast<size_t>(p.rows) * p.K0, st);
  if (e != cudaSuccess) return e;
  const size_t fb = static_cast<size_t>(p.rows) * p.n_chunks * kChunkUnits * sizeof(uint16_t);
  e = cudaMemsetAsync(p.flag_hi, 0, fb, st);
  if (e != cudaSuccess) return e;
  return cudaMemsetAsync(p.flag_odd, 0, fb, st);
}

static SplitGeom make_geom(const SplitPlanes& p) {
  SplitGeom g;
  g.rows = p.rows; g.K = p.K; g.Kp = p.Kp; g.K0 = p.K0;
  g.n_chunks = p.n_chunks; g.n_odd = p.n_odd;
  g.plane0 = p.plane0; g.flag_hi = p.flag_hi; g.flag_odd = p.flag_odd;
  g.odd = p.odd; g.odd_stride = p.odd_stride;
  return g;
}

cudaError_t launch_split_a(const double* A, const double* scale, const SplitPlanes& p,
                           const Oz2DeviceConsts& c, cudaStream_t st) {
  cudaError_t e = clear_plane0(p, st);
  if (e != cudaSuccess) return e;
  const dim3 grid(static_cast<unsigned>(p.rows), static_cast<unsigned>((p.Kp + 256 * kSplitAW - 1) / (256 * kSplitAW)));
  if (grid.y > 65535u) return cudaErrorInvalidValue;
  split_a_kernel<<<grid, 256, 0, st>>>(A, scale, make_geom(p), c);
  return cudaGetLastError();
}

size_t split_b_smem_bytes(int n_odd) {
  return static_cast<size_t>(n_odd + 2) * kSplitBJ * kSplitBPitch * sizeof(uint32_t);
}

cudaError_t split_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(split_b_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(split_b_smem_bytes(15)));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(split_b_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(split_b_smem_bytes(15)));
}

cudaError_t launch_split_b(const double* B, const double* scale, long long N, const SplitPlanes& p,
                           const Oz2DeviceConsts& c, cudaStream_t st, const Im2colView* view, long long ld) {
  if (ld <= 0) ld = N;
  cudaError_t e = clear_plane0(p, st);
  if (e != cudaSuccess) return e;
  const dim3 grid(static_cast<unsigned>((N + kSplitBJ - 1) / kSplitBJ),
                  static_cast<unsigned>(p.Kp / kSplitBK));
  if (grid.y > 65535u) return cudaErrorInvalidValue;
  if (view) split_b_kernel<true><<<grid, 256, split_b_smem_bytes(p.n_odd), st>>>(nullptr, scale, N, ld, make_geom(p), c, *view);
  else split_b_kernel<false><<<grid, 256, split_b_smem_bytes(p.n_odd), st>>>(B, scale, N, ld, make_geom(p), c, Im2colView{});
  return cudaGetLastError();
}

cudaError_t launch_crt(const CrtArgs& a, const Oz2DeviceConsts& c, cudaStream_t st) {
  if (a.M <= 0 || a.N <= 0) return cudaSuccess;
  const dim3 grid(static_cast<unsigned>(a.M), static_cast<unsigned>((a.N + 256 * kCrtW - 1) / (256 * kCrtW)));
  if (grid.y > 65535u) return cudaErrorInvalidValue;
  if (a.n_mod == 16 && a.bias_mode == 0 && a.activation == 0 && a.pixels_per_image == 0)
    crt_kernel<0><<<grid, 256, 0, st>>>(a, c);
  else if (a.activation == 0 || a.activation == 1)
    crt_kernel<1><<<grid, 256, 0, st>>>(a, c);
  else
    crt_kernel<2><<<grid, 256, 0, st>>>(a, c);
  return cudaGetLastError();
}

}  // namespace b200
