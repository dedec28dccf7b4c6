// Host-visible declarations of the scan / split / CRT stages (b200_ozaki2.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

struct Oz2DeviceConsts {
  double P1, P2, Pinv;
  double sl1[16], sl2[16];
  double p_d[16], p_inv[16];
  int p_i[16];
  int q_i[16];  // (P/p_l)^-1 mod p_l
  int n_mod;
};

// Residue planes of one operand.
struct SplitPlanes {
  long long rows;       // M (A) or N (B)
  long long K, Kp, K0;  // logical, padded-to-128, and modulus-256-plane inner extents
  int n_chunks, n_odd;
  int8_t* plane0;       // rows x K0 (1024 bytes per 1008-element chunk)
  uint16_t* flag_hi;    // rows x n_chunks x 64 units of 16 bits along k: residue == +128
  uint16_t* flag_odd;   // same shape: residue odd
  int8_t* odd;          // n_odd planes, each rows x Kp
  long long odd_stride; // bytes between odd planes
};

struct CrtArgs {
  const int16_t* w0;     // modulus 256: sum of the chunk residues mod 512, ties taken as +128; M_pad x ldw
  const uint32_t* flip;  // one bit per element of w0: add 256 (a tie was -128); M_pad x ldw/32 words
  const int8_t* w_odd;   // odd-modulus residues, (n_mod-1) planes of M_pad x ldw
  long long w_odd_stride;
  long long ldw;
  int n_mod;
  long long M, N;
  const double* inv_scale_a;  // 2^-mu_i
  const double* inv_scale_b;  // 2^-nu_j
  double* C;
  long long ldc;
  int bias_mode;              // 0 none, 1 per row, 2 per column
  const double* bias;
  int activation;             // 0 none, 1 ReLU, 2 tanh-form GELU
  long long pixels_per_image; // > 0: scatter columns to [image][row][pixel] (conv2d NCHW)
};

// A right-hand operand that is never materialised: the im2col view of an NCHW tensor.
// Element (kk, n), kk = (ic*kH + kh)*kW + kw, n = (b*oH + oh)*oW + ow, is
// in[b][ic][oh*stride + kh - pad][ow*stride + kw - pad], or 0 outside the image (the loop
// bounds of eshkol_conv2d_kernel, lib/backend/tensor_conv_kernel.h:66-105).  The column scan
// and the split read the tensor through this map, so HBM sees the tensor once per kernel tap
// that L2 does not serve instead of a kH*kW times larger f64 matrix written and read back.
struct Im2colView {
  const double* in;
  long long batch, in_c, H, W, kH, kW, stride, pad, oH, oW;
};

cudaError_t launch_scan_rows(const double* A, long long M, long long K, double* amax, cudaStream_t st);
// ld: elements between rows of B (0 = N): B may be a block of columns of a wider matrix
cudaError_t launch_scan_cols(const double* B, long long K, long long N,
                             unsigned long long* bmax_bits, cudaStream_t st, long long ld = 0);
// column maxima of an im2col view: the maximum over the channels of every input pixel (into
// pixel_max, batch * H * W doubles of scratch), then the window maximum per output pixel
cudaError_t launch_scan_view(const Im2colView& view, long long N, double* pixel_max, double* bmax, cudaStream_t st);
cudaError_t launch_scales(const double* vmax, long long n, int E, int* shift, double* scale,
                          double* inv_scale, cudaStream_t st);
cudaError_t launch_split_a(const double* A, const double* scale, const SplitPlanes& p,
                           const Oz2DeviceConsts& c, cudaStream_t st);
cudaError_t launch_split_b(const double* B, const double* scale, long long N, const SplitPlanes& p,
                           const Oz2DeviceConsts& c, cudaStream_t st, const Im2colView* view = nullptr,
                           long long ld = 0);
cudaError_t split_set_attributes();
cudaError_t launch_crt(const CrtArgs& a, const Oz2DeviceConsts& c, cudaStream_t st);

}  // namespace b200
