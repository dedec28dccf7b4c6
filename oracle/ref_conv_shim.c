/* TEST INFRASTRUCTURE ONLY.  Exports the reference's header-only direct conv2d
 * (lib/backend/tensor_conv_kernel.h:49-105 in the reference project) as a
 * shared-object symbol so tests and the CPU-baseline leg can call it.  The
 * header is included from where the reference lies; nothing is copied. */
#include "tensor_conv_kernel.h"

int64_t ref_conv_out_dim(int64_t in_dim, int64_t k_dim, int64_t stride, int64_t pad) {
  return eshkol_conv_out_dim(in_dim, k_dim, stride, pad);
}

void ref_conv2d(const double* in, int64_t batch, int64_t in_c, int64_t H, int64_t W,
                const double* ker, int64_t out_c, int64_t kH, int64_t kW,
                int64_t stride, int64_t pad, double* out) {
  eshkol_conv2d_kernel(in, batch, in_c, H, W, ker, out_c, kH, kW, stride, pad, out);
}
