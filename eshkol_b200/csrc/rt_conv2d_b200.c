/*
 * eshkol_rt_conv2d on the GPU: adapts the heap-tensor representation to the flat NCHW entry
 * point eshkol_gpu_conv2d_f64 and works out the output shape, as the reference's runtime
 * entry point does around its CPU kernel (lib/backend/tensor_conv_kernel.cpp:32-109).
 */
#include "../../include/eshkol_tensor_b200.h"
#include "../../include/eshkol_gpu_memory_b200.h"

#include <stdio.h>

/* the runtime's allocator; present when this object is linked into Eshkol */
extern eshkol_tensor_t* arena_allocate_tensor_full(void* arena, uint64_t num_dims, uint64_t total_elements)
    __attribute__((weak));

static eshkol_b200_tensor_allocator g_alloc = NULL;

void eshkol_b200_set_tensor_allocator(eshkol_b200_tensor_allocator fn) { g_alloc = fn; }

/* eshkol_conv_out_dim, lib/backend/tensor_conv_kernel.h:49-56 */
static int64_t out_dim(int64_t in, int64_t k, int64_t stride, int64_t pad) {
  const int64_t span = in + 2 * pad - k;
  return span < 0 ? 0 : span / stride + 1;
}

eshkol_tensor_t* eshkol_rt_conv2d(void* arena, const eshkol_tensor_t* input, const eshkol_tensor_t* kernel,
                                  int64_t stride, int64_t pad) {
  if (!input || !kernel || !arena) return NULL;
  if (stride <= 0) stride = 1;
  if (pad < 0) pad = 0;
  const int64_t in_nd = (int64_t)input->num_dimensions, k_nd = (int64_t)kernel->num_dimensions;
  if (in_nd < 2 || k_nd < 2) return NULL;
  const uint64_t* ind = input->dimensions;
  const uint64_t* kd = kernel->dimensions;
  if (!ind || !kd || !input->elements || !kernel->elements) return NULL;
  const int64_t H = (int64_t)ind[in_nd - 2], W = (int64_t)ind[in_nd - 1];
  const int64_t kH = (int64_t)kd[k_nd - 2], kW = (int64_t)kd[k_nd - 1];
  const int64_t oH = out_dim(H, kH, stride, pad), oW = out_dim(W, kW, stride, pad);
  if (oH <= 0 || oW <= 0) return NULL;

  int64_t batch = 1, in_c, out_c, out_nd, lead;
  if (k_nd >= 4) {
    /* kernel [out_c, in_c, kH, kW], input [..., in_c, H, W] */
    out_c = (int64_t)kd[0];
    in_c = (int64_t)kd[1];
    const int64_t in_channels = (in_nd >= 3) ? (int64_t)ind[in_nd - 3] : 1;
    if (in_channels != in_c) return NULL;
    lead = in_nd - 3;
    if (lead < 0) lead = 0;
    for (int64_t i = 0; i < in_nd - 3; ++i) batch *= (int64_t)ind[i];
    out_nd = lead + 3;
  } else {
    /* a rank-2 (or rank-3) kernel is one plane: every leading input dimension is a plane of its own */
    out_c = 1;
    in_c = 1;
    lead = in_nd - 2;
    for (int64_t i = 0; i < in_nd - 2; ++i) batch *= (int64_t)ind[i];
    out_nd = in_nd;
  }
  const int64_t out_total = batch * out_c * oH * oW;
  if (out_total <= 0) return NULL;

  eshkol_tensor_t* out = NULL;
  if (g_alloc) out = g_alloc(arena, (uint64_t)out_nd, (uint64_t)out_total);
  else if (arena_allocate_tensor_full) out = arena_allocate_tensor_full(arena, (uint64_t)out_nd, (uint64_t)out_total);
  else fprintf(stderr, "[GPU] eshkol_rt_conv2d: no tensor allocator (arena_allocate_tensor_full is not linked in)\n");
  if (!out || !out->dimensions || !out->elements) return NULL;

  if (k_nd >= 4) {
    for (int64_t i = 0; i < lead; ++i) out->dimensions[i] = ind[i];
    out->dimensions[lead] = (uint64_t)out_c;
    out->dimensions[lead + 1] = (uint64_t)oH;
    out->dimensions[lead + 2] = (uint64_t)oW;
  } else {
    for (int64_t i = 0; i < in_nd - 2; ++i) out->dimensions[i] = ind[i];
    out->dimensions[in_nd - 2] = (uint64_t)oH;
    out->dimensions[in_nd - 1] = (uint64_t)oW;
  }
  /* elements are doubles stored as int64 bit patterns: a double view is bit-identical */
  if (eshkol_gpu_conv2d_f64((const double*)input->elements, batch, in_c, H, W, (const double*)kernel->elements,
                            out_c, kH, kW, stride, pad, (double*)out->elements, 0) != 0) {
    fprintf(stderr, "[GPU] eshkol_rt_conv2d: the B200 path FAILED; no result\n");
    return NULL;
  }
  return out;
}
