// Drivers of the reduced-precision tiers and of conv2d, plus the few services of
// the shim they build on.  Internal to the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/eshkol_b200_ext.h"
#include "b200_ozaki2.h"

namespace b200 {

// services implemented in b200_shim.cu
uint8_t* workspace_reserve(size_t bytes);  // grow-only scratch, nullptr on failure
uint8_t* aux_reserve(size_t bytes);        // second grow-only block (outlives a nested GEMM)
cudaStream_t lib_stream();
int lib_device();  // the device eshkol_b200_init selected, -1 before init
int lib_num_sms();
int* lib_status_word();
void count_launches(int n);
int make_plane_map(CUtensorMap* map, const void* base, long long inner_bytes, long long rows,
                   long long planes, long long plane_stride, int box_rows);
void oz2_host_consts(int n_mod, Oz2DeviceConsts* c, double* log2P);
int ozaki2_exact_gemm_im2col(const double* dA, const Im2colView& view, double* dC, long long M, long long K,
                             long long N, const EshkolB200GemmOpts& o);

// b200_tiers.cu
int ozaki1_gemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                long long N, int T, const EshkolB200GemmOpts& o);
int ozaki2_fast_gemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                     long long N, int n_mod, const EshkolB200GemmOpts& o);
int native_dgemm(const double* dA, const double* dB, double* dC, long long M, long long K,
                 long long N, const EshkolB200GemmOpts& o);
int conv2d_lowered(const double* d_in, long long batch, long long in_c, long long H, long long W,
                   const double* d_ker, long long out_c, long long kH, long long kW,
                   long long stride, long long pad, double* d_out, const EshkolB200GemmOpts& o);
int conv2d_backward_kernel(const double* d_gout, const double* d_in, double* d_gker, long long H, long long W,
                           long long kH, long long kW, long long oH, long long oW, long long sH, long long sW,
                           long long C_in, long long C_out, long long batch, const EshkolB200GemmOpts& o);
int conv2d_backward_input(const double* d_gout, const double* d_ker, double* d_gin, long long H, long long W,
                          long long kH, long long kW, long long oH, long long oW, long long sH, long long sW,
                          long long C_in, long long C_out, long long batch, const EshkolB200GemmOpts& o);
int f16_gemm(const double* dA, const double* dB, double* dC, long long batch, long long M, long long K,
             long long N);
int f32_gemm(const float* dA, const float* dB, float* dC, long long M, long long K, long long N);
cudaError_t tiers_set_attributes();
// b200_static_scratch.cu: resolve the fixed scratch array's address on `device` (current)
int static_scratch_setup(int device);
// dst[cols x rows] = transpose of src[rows x cols] (row-major f64)
cudaError_t launch_transpose(const double* src, long long rows, long long cols, double* dst, cudaStream_t st);
cudaError_t launch_elementwise(const double* a, const double* b, double* out, long long n, int op,
                               cudaStream_t st);

}  // namespace b200
