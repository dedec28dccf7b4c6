/*
 * TEST INFRASTRUCTURE.  lib/backend/vm_gpu_dispatch.h of the reference project compiled the way
 * the VM compiles it (ESHKOL_GPU_ENABLED, its hand-written mirror of EshkolGPUBuffer and its
 * void* prototypes of the buffer API), with the few VM types the header uses stood in for.
 * The tensor stand-in keeps the leading fields of the VM's own VmTensor
 * (lib/backend/vm_tensor.c:48-58); the region stack is opaque here.
 */
#include <stdint.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
  int n_dims;
  int64_t* shape;
  int64_t* strides;
  double* data;
  int64_t total;
  int owns_data;
  int dtype;
  int64_t inline_shape[4];
  int64_t inline_strides[4];
} VmTensor;
typedef struct VmRegionStack VmRegionStack;

static VmTensor* vm_tensor_zeros(VmRegionStack* rs, const int64_t* shape, int n_dims) {
  (void)rs;
  VmTensor* t = (VmTensor*)calloc(1, sizeof(VmTensor));
  if (!t || n_dims > 4) return NULL;
  t->n_dims = n_dims;
  t->shape = t->inline_shape;
  t->strides = t->inline_strides;
  t->total = 1;
  for (int i = 0; i < n_dims; ++i) { t->shape[i] = shape[i]; t->total *= shape[i]; }
  /* 8 bytes past a 16-byte boundary, like an arena payload behind its header */
  char* p = NULL;
  if (posix_memalign((void**)&p, 64, (size_t)t->total * sizeof(double) + 64) != 0) return NULL;
  memset(p, 0, (size_t)t->total * sizeof(double) + 64);
  t->data = (double*)(p + 8);
  t->owns_data = 1;
  return t;
}

#define ESHKOL_GPU_ENABLED 1
#include "backend/vm_gpu_dispatch.h"

int harness_vm_matmul(const double* a, const double* b, double* c, long M, long K, long N) {
  VmTensor ta, tb;
  memset(&ta, 0, sizeof(ta));
  memset(&tb, 0, sizeof(tb));
  ta.n_dims = tb.n_dims = 2;
  ta.shape = ta.inline_shape; tb.shape = tb.inline_shape;
  ta.shape[0] = M; ta.shape[1] = K; tb.shape[0] = K; tb.shape[1] = N;
  ta.total = (int64_t)M * K; tb.total = (int64_t)K * N;
  ta.data = (double*)a; tb.data = (double*)b;
  g_vm_gpu.threshold = 1;
  VmTensor* out = vm_gpu_try_matmul(NULL, &ta, &tb);
  if (!out) return -1;
  memcpy(c, out->data, (size_t)M * N * sizeof(double));
  return 0;
}

static void as_matrix(VmTensor* t, const double* data, long rows, long cols) {
  memset(t, 0, sizeof(*t));
  t->n_dims = 2;
  t->shape = t->inline_shape;
  t->shape[0] = rows; t->shape[1] = cols;
  t->total = (int64_t)rows * cols;
  t->data = (double*)data;
}

/* the VM's other try-functions on one rows x cols matrix: softmax over the last axis, transpose,
 * a + a, and the four reductions the VM asks for (sum 0, min 2, max 3, mean 4) */
int harness_vm_operators(const double* a, long rows, long cols, double* softmax_out, double* transpose_out,
                         double* sum_out, double reduced[4]) {
  VmTensor t;
  as_matrix(&t, a, rows, cols);
  g_vm_gpu.threshold = 1;
  VmTensor* s = vm_gpu_try_softmax(NULL, &t);
  VmTensor* tr = vm_gpu_try_transpose(NULL, &t);
  VmTensor* add = vm_gpu_try_binary(NULL, &t, &t, 0);
  if (!s || !tr || !add) return -1;
  if (tr->shape[0] != cols || tr->shape[1] != rows) return -2;
  memcpy(softmax_out, s->data, (size_t)t.total * sizeof(double));
  memcpy(transpose_out, tr->data, (size_t)t.total * sizeof(double));
  memcpy(sum_out, add->data, (size_t)t.total * sizeof(double));
  static const int ops[4] = {0, 2, 3, 4};
  for (int i = 0; i < 4; ++i) {
    reduced[i] = vm_gpu_try_reduce(&t, ops[i]);
    if (isnan(reduced[i])) return -3;
  }
  return 0;
}
