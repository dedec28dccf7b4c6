/*
 * TEST INFRASTRUCTURE.  A C translation unit compiled against the REFERENCE's own header
 * (inc/eshkol/backend/gpu/gpu_memory.h of the reference project) and linked to
 * libeshkol_gpu_b200.so: what a maintainer's build does when the library replaces the
 * reference's GPU runtime object.  Built by oracle/Makefile into oracle/_ref/c_harness.
 *
 *   c_harness link                     take the address of every function of the header
 *   c_harness run M K N out_dir        eshkol_matmul_dispatch and the VM's vm_gpu_try_matmul on
 *                                      arena-like operands that are 8- but not 16-byte aligned;
 *                                      results go to out_dir/dispatch.bin and out_dir/vm.bin;
 *                                      the VM's softmax, transpose, add and reductions of A go to
 *                                      out_dir/vm_softmax.bin, vm_transpose.bin, vm_add.bin, vm_reduce.bin
 */
#include <eshkol/backend/gpu/gpu_memory.h>

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

/* harness_vm.c: lib/backend/vm_gpu_dispatch.h compiled as the VM compiles it */
int harness_vm_matmul(const double* a, const double* b, double* c, long M, long K, long N);
int harness_vm_operators(const double* a, long rows, long cols, double* softmax_out, double* transpose_out,
                         double* sum_out, double reduced[4]);

/* the runtime's 48-bit generator (lib/core/prng.cpp:45-58, 76-80), entries 2u - 1 */
static void fill_uniform(double* dst, size_t n, unsigned long long seed) {
  unsigned long long x = ((seed << 16) | 0x330EULL) & 0xFFFFFFFFFFFFULL;
  for (size_t i = 0; i < n; ++i) {
    x = (x * 0x5DEECE66DULL + 0xBULL) & 0xFFFFFFFFFFFFULL;
    dst[i] = 2.0 * ((double)x * (1.0 / 281474976710656.0)) - 1.0;
  }
}

/* a block whose payload starts 8 bytes past a 16-byte boundary, as arena objects behind an
 * 8-byte header do */
static double* arena_like(size_t n, void** base) {
  char* p = NULL;
  if (posix_memalign((void**)&p, 64, n * sizeof(double) + 64) != 0) return NULL;
  *base = p;
  return (double*)(p + 8);
}

static int write_file(const char* dir, const char* name, const double* v, size_t n) {
  char path[4096];
  snprintf(path, sizeof(path), "%s/%s", dir, name);
  FILE* f = fopen(path, "wb");
  if (!f) return -1;
  const size_t w = fwrite(v, sizeof(double), n, f);
  fclose(f);
  return w == n ? 0 : -1;
}

static int link_check(void) {
  /* every function the header declares; the build fails if the library lacks one */
  void* fns[] = {(void*)eshkol_gpu_init, (void*)eshkol_gpu_shutdown, (void*)eshkol_gpu_get_backend,
                 (void*)eshkol_gpu_backend_name, (void*)eshkol_gpu_backend_available, (void*)eshkol_gpu_supports_f64,
                 (void*)eshkol_gpu_has_fp64, (void*)eshkol_gpu_alloc, (void*)eshkol_gpu_alloc_aligned,
                 (void*)eshkol_gpu_free, (void*)eshkol_gpu_wrap_host, (void*)eshkol_gpu_sync,
                 (void*)eshkol_gpu_sync_async, (void*)eshkol_gpu_wait, (void*)eshkol_gpu_matmul_f64,
                 (void*)eshkol_gpu_matmul_f32, (void*)eshkol_gpu_set_threshold, (void*)eshkol_gpu_get_threshold,
                 (void*)eshkol_gpu_should_use, (void*)eshkol_gpu_elementwise_f64, (void*)eshkol_gpu_reduce_f64,
                 (void*)eshkol_gpu_reduce_axis_f64, (void*)eshkol_gpu_transpose_f64, (void*)eshkol_gpu_softmax_f64,
                 (void*)eshkol_gpu_normalize_f64, (void*)eshkol_gpu_conv2d_backward_input_f64,
                 (void*)eshkol_gpu_conv2d_backward_kernel_f64, (void*)eshkol_gpu_batchnorm_backward_f64,
                 (void*)eshkol_gpu_layernorm_backward_f64, (void*)eshkol_matmul_dispatch,
                 (void*)eshkol_batch_matmul_dispatch};
  int n = 0;
  for (size_t i = 0; i < sizeof(fns) / sizeof(fns[0]); ++i) n += fns[i] != NULL;
  printf("linked %d functions, sizeof(EshkolGPUBuffer) = %zu, g_gpu_threshold = %zu\n", n, sizeof(EshkolGPUBuffer),
         g_gpu_threshold);
  return (n == (int)(sizeof(fns) / sizeof(fns[0])) && sizeof(EshkolGPUBuffer) == 48) ? 0 : 1;
}

int main(int argc, char** argv) {
  if (argc >= 2 && !strcmp(argv[1], "link")) return link_check();
  if (argc < 6 || strcmp(argv[1], "run")) {
    fprintf(stderr, "usage: c_harness link | run M K N out_dir\n");
    return 2;
  }
  const long M = atol(argv[2]), K = atol(argv[3]), N = atol(argv[4]);
  const char* dir = argv[5];
  if (eshkol_gpu_init() != 1) {
    fprintf(stderr, "eshkol_gpu_init found no device\n");
    return 3;
  }
  eshkol_gpu_set_threshold(1); /* as the reference's GPU gates do with ESHKOL_GPU_THRESHOLD=1 */
  void *ba, *bb, *bc;
  double* A = arena_like((size_t)M * K, &ba);
  double* B = arena_like((size_t)K * N, &bb);
  double* C = arena_like((size_t)M * N, &bc);
  if (!A || !B || !C) return 4;
  fill_uniform(A, (size_t)M * K, 1);
  fill_uniform(B, (size_t)K * N, 2);
  for (size_t i = 0; i < (size_t)M * N; ++i) C[i] = -7.0; /* the result tensor is not zero-filled for us */
  eshkol_matmul_dispatch(A, B, C, (uint64_t)M, (uint64_t)K, (uint64_t)N, 0);
  if (write_file(dir, "dispatch.bin", C, (size_t)M * N)) return 5;
  for (size_t i = 0; i < (size_t)M * N; ++i) C[i] = -7.0;
  if (harness_vm_matmul(A, B, C, M, K, N) != 0) {
    fprintf(stderr, "vm_gpu_try_matmul declined or failed\n");
    return 6;
  }
  if (write_file(dir, "vm.bin", C, (size_t)M * N)) return 7;
  {
    /* the VM's softmax / transpose / add / reduce try-functions on A */
    const size_t n = (size_t)M * K;
    double* out = (double*)malloc(3 * n * sizeof(double));
    double reduced[4];
    if (!out) return 4;
    const int rc = harness_vm_operators(A, M, K, out, out + n, out + 2 * n, reduced);
    if (rc != 0) {
      fprintf(stderr, "a vm_gpu_try_* operator declined or failed (%d)\n", rc);
      return 8;
    }
    if (write_file(dir, "vm_softmax.bin", out, n) || write_file(dir, "vm_transpose.bin", out + n, n) ||
        write_file(dir, "vm_add.bin", out + 2 * n, n) || write_file(dir, "vm_reduce.bin", reduced, 4))
      return 9;
    free(out);
  }
  eshkol_gpu_shutdown();
  free(ba); free(bb); free(bc);
  printf("ok\n");
  return 0;
}
