// Tensor operators of the backend ABI beside the matrix product: full and per-axis reductions,
// transpose, softmax, layer normalisation and the two normalisation gradients.  They restate the
// arithmetic of the reference's CUDA kernels (lib/backend/gpu/gpu_cuda_kernels.cu:76-213, 319-389,
// 489-555) but not their shape: the reference gives a slice, a feature or a sample to ONE thread
// and walks it serially, which leaves all but a few SMs idle for the shapes its callers use; here
// a warp or a block shares each slice, sums are combined in a fixed order (so a result does not
// depend on timing), and every access is coalesced.  All kernels are HBM-bound streaming passes.
//
// Sums are therefore associated differently from the reference's serial loops: results agree
// with it to rounding (a few ulp times the condition of the sum), not bit for bit.  min, max and
// transpose are exact.
#include <math.h>
#include <stdio.h>

#include "b200_tiers.h"

namespace b200 {
namespace {

enum { kSum = 0, kProd = 1, kMin = 2, kMax = 3, kMean = 4 };  // EshkolReduceOp, gpu_memory.h:302-308

__device__ __forceinline__ double red_identity(int op) {
  return op == kProd ? 1.0 : op == kMin ? INFINITY : op == kMax ? -INFINITY : 0.0;
}
__device__ __forceinline__ double red_combine(int op, double a, double b) {
  switch (op) {
    case kProd: return a * b;
    case kMin: return fmin(a, b);  // NaN-ignoring, as the reference's fmin / fmax
    case kMax: return fmax(a, b);
    default: return a + b;
  }
}

// every lane gets the combination of the 32 lanes' values (butterfly: the same tree on every lane)
__device__ __forceinline__ double warp_all(int op, double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = red_combine(op, v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// every thread of a group of kThreads (32: a warp, else the whole block) gets the combination
template <int kThreads>
__device__ __forceinline__ double group_all(int op, double v, double* sm) {
  v = warp_all(op, v);
  if (kThreads == 32) return v;
  const int w = threadIdx.x >> 5;
  __syncthreads();  // the previous use of sm is over
  if ((threadIdx.x & 31) == 0) sm[w] = v;
  __syncthreads();
  double r = sm[0];
#pragma unroll
  for (int i = 1; i < kThreads / 32; ++i) r = red_combine(op, r, sm[i]);
  return r;
}

// ------------------------------------------------------------------ full reduce
constexpr int kMaxPartials = 2048;
__device__ double g_partials[kMaxPartials];

__global__ void __launch_bounds__(256) reduce_partial_kernel(const double* __restrict__ in, long long n, int op) {
  __shared__ double sm[8];
  const long long stride = static_cast<long long>(gridDim.x) * 256;
  long long i = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
  double a0 = red_identity(op), a1 = a0, a2 = a0, a3 = a0;  // four chains in flight per thread
  for (; i + 3 * stride < n; i += 4 * stride) {
    a0 = red_combine(op, a0, __ldg(in + i));
    a1 = red_combine(op, a1, __ldg(in + i + stride));
    a2 = red_combine(op, a2, __ldg(in + i + 2 * stride));
    a3 = red_combine(op, a3, __ldg(in + i + 3 * stride));
  }
  for (; i < n; i += stride) a0 = red_combine(op, a0, __ldg(in + i));
  const double v = group_all<256>(op, red_combine(op, red_combine(op, a0, a1), red_combine(op, a2, a3)), sm);
  if (threadIdx.x == 0) g_partials[blockIdx.x] = v;
}

__global__ void __launch_bounds__(256) reduce_final_kernel(int n_partials, long long n, int op, double* out) {
  __shared__ double sm[8];
  double a = red_identity(op);
  for (int i = threadIdx.x; i < n_partials; i += 256) a = red_combine(op, a, g_partials[i]);
  a = group_all<256>(op, a, sm);
  if (threadIdx.x == 0) out[0] = (op == kMean) ? a / static_cast<double>(n) : a;
}

// ------------------------------------------------------------------ reduce along one axis
// in is [outer][axis_len][inner]; out is [outer][inner].
// inner > 1: a thread column per output, kLanes threads sharing the axis (lane t takes k = t,
// t + kLanes, ...), combined in lane order through shared memory.  Neighbouring threads read
// neighbouring `inner`, so every load is coalesced.
template <int kLanes>
__global__ void __launch_bounds__(256) reduce_axis_strided_kernel(const double* __restrict__ in, double* __restrict__ out,
                                                                  long long outer, long long axis_len, long long inner,
                                                                  int op) {
  __shared__ double sm[256];
  constexpr int kCols = 256 / kLanes;
  const int col = threadIdx.x % kCols, lane = threadIdx.x / kCols;
  const long long total = outer * inner;
  for (long long base = static_cast<long long>(blockIdx.x) * kCols; base < total;
       base += static_cast<long long>(gridDim.x) * kCols) {
    const long long idx = base + col;
    double acc = red_identity(op);
    if (idx < total) {
      const long long o = idx / inner, r = idx - o * inner;
      const double* p = in + o * axis_len * inner + r;
      for (long long k = lane; k < axis_len; k += kLanes) acc = red_combine(op, acc, __ldg(p + k * inner));
    }
    if (kLanes > 1) {
      __syncthreads();
      sm[threadIdx.x] = acc;
      __syncthreads();
      if (lane == 0) {
#pragma unroll
        for (int t = 1; t < kLanes; ++t) acc = red_combine(op, acc, sm[t * kCols + col]);
      }
    }
    if (lane == 0 && idx < total) out[idx] = (op == kMean) ? acc / static_cast<double>(axis_len) : acc;
  }
}

// inner == 1: the axis is contiguous; a warp (short axes) or a block per output row
template <int kThreads>
__global__ void __launch_bounds__(256) reduce_rows_kernel(const double* __restrict__ in, double* __restrict__ out,
                                                          long long rows, long long len, int op) {
  __shared__ double sm[8];
  constexpr int kGroups = 256 / kThreads;
  const int t = threadIdx.x % kThreads, grp = threadIdx.x / kThreads;
  // whole blocks iterate together: group_all<256> has a barrier inside
  for (long long base = static_cast<long long>(blockIdx.x) * kGroups; base < rows;
       base += static_cast<long long>(gridDim.x) * kGroups) {
    const long long row = base + grp;
    double acc = red_identity(op);
    if (row < rows)
      for (long long k = t; k < len; k += kThreads) acc = red_combine(op, acc, __ldg(in + row * len + k));
    acc = group_all<kThreads>(op, acc, sm);
    if (t == 0 && row < rows) out[row] = (op == kMean) ? acc / static_cast<double>(len) : acc;
  }
}

// ------------------------------------------------------------------ transpose
// 32 x 32 tiles through shared memory (pitch 33: the column reads hit 32 banks); tiles are
// numbered along one grid axis so neither extent meets the 65535 limit of grid.y.
__global__ void __launch_bounds__(256) transpose_kernel(const double* __restrict__ in, double* __restrict__ out,
                                                        long long rows, long long cols, long long tiles_x) {
  __shared__ double tile[32][33];
  const long long ty = blockIdx.x / tiles_x, tx = blockIdx.x - ty * tiles_x;
  const int x = threadIdx.x & 31, y0 = threadIdx.x >> 5;
#pragma unroll
  for (int y = y0; y < 32; y += 8) {
    const long long r = ty * 32 + y, c = tx * 32 + x;
    if (r < rows && c < cols) tile[y][x] = __ldg(in + r * cols + c);
  }
  __syncthreads();
#pragma unroll
  for (int y = y0; y < 32; y += 8) {
    const long long r = tx * 32 + y, c = ty * 32 + x;  // row / column of the output
    if (r < cols && c < rows) out[r * rows + c] = tile[x][y];
  }
}

// ------------------------------------------------------------------ softmax, layer norm
// One group of kThreads per slice; the block's groups walk the slices together.
template <int kThreads>
__global__ void __launch_bounds__(256) softmax_kernel(const double* in, double* out,  // may be the same array
                                                      long long slices, long long len) {
  __shared__ double sm[8];
  constexpr int kGroups = 256 / kThreads;
  const int t = threadIdx.x % kThreads, grp = threadIdx.x / kThreads;
  for (long long base = static_cast<long long>(blockIdx.x) * kGroups; base < slices;
       base += static_cast<long long>(gridDim.x) * kGroups) {
    const long long s = base + grp;
    const bool live = s < slices;
    const double* x = in + s * len;
    double* y = out + s * len;
    double m = -INFINITY;
    if (live) for (long long k = t; k < len; k += kThreads) m = fmax(m, x[k]);
    m = group_all<kThreads>(kMax, m, sm);
    double sum = 0.0;
    if (live)
      for (long long k = t; k < len; k += kThreads) {
        const double e = exp(x[k] - m);
        y[k] = e;  // re-read below by this same thread
        sum += e;
      }
    sum = group_all<kThreads>(kSum, sum, sm);
    if (sum == 0.0) sum = 1.0;  // gpu_cuda_kernels.cu:340
    if (live) for (long long k = t; k < len; k += kThreads) y[k] /= sum;
  }
}

template <int kThreads>
__global__ void __launch_bounds__(256) normalize_kernel(const double* in, double* out,  // may be the same array
                                                        long long slices, long long len, double gamma, double beta,
                                                        double epsilon) {
  __shared__ double sm[8];
  constexpr int kGroups = 256 / kThreads;
  const int t = threadIdx.x % kThreads, grp = threadIdx.x / kThreads;
  const double n = static_cast<double>(len);
  for (long long base = static_cast<long long>(blockIdx.x) * kGroups; base < slices;
       base += static_cast<long long>(gridDim.x) * kGroups) {
    const long long s = base + grp;
    const bool live = s < slices;
    const double* x = in + s * len;
    double sum = 0.0;
    if (live) for (long long k = t; k < len; k += kThreads) sum += x[k];
    const double mean = group_all<kThreads>(kSum, sum, sm) / n;
    double var = 0.0;
    if (live)
      for (long long k = t; k < len; k += kThreads) {
        const double d = x[k] - mean;
        var += d * d;
      }
    const double inv_std = rsqrt(group_all<kThreads>(kSum, var, sm) / n + epsilon);  // gpu_cuda_kernels.cu:383
    if (live)
      for (long long k = t; k < len; k += kThreads) out[s * len + k] = gamma * (x[k] - mean) * inv_std + beta;
  }
}

// gradient of layer normalisation wrt its input, one group per sample (gpu_cuda_kernels.cu:524-555)
template <int kThreads>
__global__ void __launch_bounds__(256) layernorm_backward_kernel(
    const double* __restrict__ grad_out, const double* __restrict__ x, const double* __restrict__ mean,
    const double* __restrict__ inv_std, const double* __restrict__ gamma, double* __restrict__ grad_in,
    long long samples, long long features) {
  __shared__ double sm[8];
  constexpr int kGroups = 256 / kThreads;
  const int t = threadIdx.x % kThreads, grp = threadIdx.x / kThreads;
  const double D = static_cast<double>(features);
  for (long long base = static_cast<long long>(blockIdx.x) * kGroups; base < samples;
       base += static_cast<long long>(gridDim.x) * kGroups) {
    const long long s = base + grp;
    const bool live = s < samples;
    const double mu = live ? mean[s] : 0.0, is = live ? inv_std[s] : 0.0;
    double sg = 0.0, sgn = 0.0;
    if (live)
      for (long long f = t; f < features; f += kThreads) {
        const double g = grad_out[s * features + f] * __ldg(gamma + f);
        sg += g;
        sgn += g * ((x[s * features + f] - mu) * is);
      }
    sg = group_all<kThreads>(kSum, sg, sm);
    sgn = group_all<kThreads>(kSum, sgn, sm);
    const double inv_D = is / D;
    if (live)
      for (long long f = t; f < features; f += kThreads) {
        const double g = grad_out[s * features + f] * __ldg(gamma + f);
        const double nz = (x[s * features + f] - mu) * is;
        grad_in[s * features + f] = inv_D * (D * g - sg - nz * sgn);
      }
  }
}

// gradient of batch normalisation (gpu_cuda_kernels.cu:489-521): 32 features per block, the
// batch shared by 8 lanes per feature and combined in lane order
__global__ void __launch_bounds__(256) batchnorm_backward_kernel(
    const double* __restrict__ grad_out, const double* __restrict__ x, const double* __restrict__ mean,
    const double* __restrict__ inv_std, const double* __restrict__ gamma, double* __restrict__ grad_in,
    double* __restrict__ grad_gamma, double* __restrict__ grad_beta, long long batch, long long features) {
  __shared__ double sm_g[8][32], sm_gn[8][32];
  const int col = threadIdx.x & 31, lane = threadIdx.x >> 5;
  const long long f = static_cast<long long>(blockIdx.x) * 32 + col;
  const bool live = f < features;
  const double mu = live ? mean[f] : 0.0, is = live ? inv_std[f] : 0.0;
  double sg = 0.0, sgn = 0.0;
  if (live)
    for (long long b = lane; b < batch; b += 8) {
      const double g = grad_out[b * features + f];
      sg += g;
      sgn += g * ((x[b * features + f] - mu) * is);
    }
  sm_g[lane][col] = sg;
  sm_gn[lane][col] = sgn;
  __syncthreads();
  sg = sm_g[0][col];
  sgn = sm_gn[0][col];
#pragma unroll
  for (int t = 1; t < 8; ++t) {
    sg += sm_g[t][col];
    sgn += sm_gn[t][col];
  }
  if (!live) return;
  if (lane == 0) {
    grad_beta[f] = sg;
    grad_gamma[f] = sgn;
  }
  const double N = static_cast<double>(batch);
  const double coeff = gamma[f] * is / N;
  for (long long b = lane; b < batch; b += 8) {
    const double g = grad_out[b * features + f];
    const double nz = (x[b * features + f] - mu) * is;
    grad_in[b * features + f] = coeff * (N * g - sg - nz * sgn);
  }
}

unsigned grid_for(long long units, int per_block) {
  const long long want = (units + per_block - 1) / per_block;
  const long long cap = static_cast<long long>(lib_num_sms()) * 8;  // 8 blocks of 256 threads fill an SM
  return static_cast<unsigned>(want < 1 ? 1 : (want < cap ? want : cap));
}

int finish(int launches) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[eshkol-b200] operator launch failed: %s\n", cudaGetErrorString(e));
    return -1;
  }
  count_launches(launches);
  return 0;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

int eshkol_b200_reduce_f64_device(const double* in, double* out, uint64_t n, int op) {
  if (lib_device() < 0 || !in || !out || n == 0 || op < 0 || op > 4 || n > (1ull << 62)) return -1;
  // at least 16 elements per thread, at most eight blocks per SM and one partial per block
  unsigned blocks = grid_for(static_cast<long long>(n), 4096);
  if (blocks > static_cast<unsigned>(kMaxPartials)) blocks = kMaxPartials;
  reduce_partial_kernel<<<blocks, 256, 0, lib_stream()>>>(in, static_cast<long long>(n), op);
  reduce_final_kernel<<<1, 256, 0, lib_stream()>>>(static_cast<int>(blocks), static_cast<long long>(n), op, out);
  return finish(2);
}

int eshkol_b200_reduce_axis_f64_device(const double* in, double* out, uint64_t outer, uint64_t axis_len,
                                       uint64_t inner, int op) {
  if (lib_device() < 0 || !in || !out || outer == 0 || axis_len == 0 || inner == 0 || op < 0 || op > 4) return -1;
  if (outer > (1ull << 40) || axis_len > (1ull << 40) || inner > (1ull << 40)) return -1;
  const long long o = static_cast<long long>(outer), l = static_cast<long long>(axis_len),
                  r = static_cast<long long>(inner);
  cudaStream_t st = lib_stream();
  if (r == 1) {
    if (l <= 1024) reduce_rows_kernel<32><<<grid_for(o, 8), 256, 0, st>>>(in, out, o, l, op);
    else reduce_rows_kernel<256><<<grid_for(o, 1), 256, 0, st>>>(in, out, o, l, op);
  } else if (o * r >= static_cast<long long>(lib_num_sms()) * 2048 || l < 64) {
    reduce_axis_strided_kernel<1><<<grid_for(o * r, 256), 256, 0, st>>>(in, out, o, l, r, op);
  } else {
    // few outputs, long axis: eight threads share each output's axis
    reduce_axis_strided_kernel<8><<<grid_for(o * r, 32), 256, 0, st>>>(in, out, o, l, r, op);
  }
  return finish(1);
}

int eshkol_b200_transpose_f64_device(const double* in, double* out, uint64_t rows, uint64_t cols) {
  if (lib_device() < 0 || !in || !out || rows == 0 || cols == 0 || in == out) return -1;
  const uint64_t tx = (cols + 31) / 32, ty = (rows + 31) / 32;
  if (rows > (1ull << 40) || cols > (1ull << 40) || tx * ty > 0x7fffffffull) return -1;
  transpose_kernel<<<static_cast<unsigned>(tx * ty), 256, 0, lib_stream()>>>(
      in, out, static_cast<long long>(rows), static_cast<long long>(cols), static_cast<long long>(tx));
  return finish(1);
}

int eshkol_b200_softmax_f64_device(const double* in, double* out, uint64_t num_slices, uint64_t slice_len) {
  if (lib_device() < 0 || !in || !out || num_slices == 0 || slice_len == 0) return -1;
  if (num_slices > (1ull << 40) || slice_len > (1ull << 40)) return -1;
  const long long s = static_cast<long long>(num_slices), l = static_cast<long long>(slice_len);
  if (l <= 1024) softmax_kernel<32><<<grid_for(s, 8), 256, 0, lib_stream()>>>(in, out, s, l);
  else softmax_kernel<256><<<grid_for(s, 1), 256, 0, lib_stream()>>>(in, out, s, l);
  return finish(1);
}

int eshkol_b200_normalize_f64_device(const double* in, double* out, uint64_t num_slices, uint64_t slice_len,
                                     double gamma, double beta, double epsilon) {
  if (lib_device() < 0 || !in || !out || num_slices == 0 || slice_len == 0) return -1;
  if (num_slices > (1ull << 40) || slice_len > (1ull << 40)) return -1;
  const long long s = static_cast<long long>(num_slices), l = static_cast<long long>(slice_len);
  if (l <= 1024) normalize_kernel<32><<<grid_for(s, 8), 256, 0, lib_stream()>>>(in, out, s, l, gamma, beta, epsilon);
  else normalize_kernel<256><<<grid_for(s, 1), 256, 0, lib_stream()>>>(in, out, s, l, gamma, beta, epsilon);
  return finish(1);
}

int eshkol_b200_batchnorm_backward_f64_device(const double* grad_out, const double* saved_input,
                                              const double* saved_mean, const double* saved_inv_std,
                                              const double* saved_gamma, double* grad_input, double* grad_gamma,
                                              double* grad_beta, uint64_t batch, uint64_t features) {
  if (lib_device() < 0 || !grad_out || !saved_input || !saved_mean || !saved_inv_std || !saved_gamma ||
      !grad_input || !grad_gamma || !grad_beta || batch == 0 || features == 0)
    return -1;
  if (batch > (1ull << 40) || features > (1ull << 35)) return -1;
  batchnorm_backward_kernel<<<static_cast<unsigned>((features + 31) / 32), 256, 0, lib_stream()>>>(
      grad_out, saved_input, saved_mean, saved_inv_std, saved_gamma, grad_input, grad_gamma, grad_beta,
      static_cast<long long>(batch), static_cast<long long>(features));
  return finish(1);
}

int eshkol_b200_layernorm_backward_f64_device(const double* grad_out, const double* saved_input,
                                              const double* saved_mean, const double* saved_inv_std,
                                              const double* saved_gamma, double* grad_input, uint64_t samples,
                                              uint64_t features) {
  if (lib_device() < 0 || !grad_out || !saved_input || !saved_mean || !saved_inv_std || !saved_gamma ||
      !grad_input || samples == 0 || features == 0)
    return -1;
  if (samples > (1ull << 40) || features > (1ull << 40)) return -1;
  const long long s = static_cast<long long>(samples), f = static_cast<long long>(features);
  if (f <= 1024)
    layernorm_backward_kernel<32><<<grid_for(s, 8), 256, 0, lib_stream()>>>(grad_out, saved_input, saved_mean,
                                                                              saved_inv_std, saved_gamma, grad_input, s, f);
  else
    layernorm_backward_kernel<256><<<grid_for(s, 1), 256, 0, lib_stream()>>>(grad_out, saved_input, saved_mean,
                                                                               saved_inv_std, saved_gamma, grad_input, s, f);
  return finish(1);
}

}  // extern "C"
