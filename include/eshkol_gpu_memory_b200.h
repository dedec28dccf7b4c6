/*
 * Drop-in boundary of libeshkol_gpu_b200.so: the C ABI of Eshkol's GPU backend.
 *
 * Every symbol below has the name, argument order and return convention of the
 * declaration it replaces in the reference's inc/eshkol/backend/gpu/gpu_memory.h
 * (cited per symbol as gpu_memory.h:LINE), so generated code, the VM and .esk
 * programs that bind these names link against this library unchanged.  Types are
 * laid out identically; EshkolGPUBuffer in particular is mirrored by hand inside
 * the reference's VM (lib/backend/vm_gpu_dispatch.h:60) and must not be reordered.
 *
 * Conventions (gpu_memory.h:79-88): eshkol_gpu_init returns 1 when a GPU backend
 * is active and 0 otherwise; every other int function returns 0 on success and
 * -1 on failure; the two dispatchers return void and leave a complete C.
 */
#ifndef ESHKOL_GPU_MEMORY_B200_H
#define ESHKOL_GPU_MEMORY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* gpu_memory.h:33-38 */
typedef enum {
  ESHKOL_GPU_NONE = 0,
  ESHKOL_GPU_METAL = 1,
  ESHKOL_GPU_CUDA = 2,
  ESHKOL_GPU_VULKAN = 3
} EshkolGPUBackend;

/* gpu_memory.h:40-45 */
typedef enum {
  ESHKOL_MEM_HOST = 0,
  ESHKOL_MEM_HOST_PINNED = 1,
  ESHKOL_MEM_DEVICE = 2,
  ESHKOL_MEM_UNIFIED = 3
} EshkolMemoryType;

/* gpu_memory.h:47-52 */
typedef enum {
  ESHKOL_SYNC_NONE = 0,
  ESHKOL_SYNC_HOST_TO_DEVICE,
  ESHKOL_SYNC_DEVICE_TO_HOST,
  ESHKOL_SYNC_BIDIRECTIONAL
} EshkolSyncDirection;

/* gpu_memory.h:60-68 -- 48 bytes on LP64 */
typedef struct EshkolGPUBuffer {
  void* host_ptr;
  void* device_ptr;
  size_t size_bytes;
  EshkolMemoryType mem_type;
  EshkolGPUBackend backend;
  uint32_t flags;       /* bit 0: wraps caller memory (never freed here); bit 1: copy back on sync/free */
  void* backend_data;   /* for a wrapped buffer: the caller's host pointer */
} EshkolGPUBuffer;

/* ---- device management ---- */
int eshkol_gpu_init(void);                                        /* gpu_memory.h:90 */
void eshkol_gpu_shutdown(void);                                   /* gpu_memory.h:95 */
EshkolGPUBackend eshkol_gpu_get_backend(void);                    /* gpu_memory.h:101 */
const char* eshkol_gpu_backend_name(EshkolGPUBackend backend);    /* gpu_memory.h:108 */
int eshkol_gpu_backend_available(EshkolGPUBackend backend);       /* gpu_memory.h:115 */
int eshkol_gpu_supports_f64(void);                                /* gpu_memory.h:133 */
int eshkol_gpu_has_fp64(void);                                    /* gpu_memory.h:149 */

/* ---- memory ---- */
int eshkol_gpu_alloc(size_t size_bytes, EshkolMemoryType mem_type,
                     EshkolGPUBuffer* out_buffer);                /* gpu_memory.h:164 */
int eshkol_gpu_alloc_aligned(size_t size_bytes, size_t alignment, EshkolMemoryType mem_type,
                             EshkolGPUBuffer* out_buffer);        /* gpu_memory.h:175 */
void eshkol_gpu_free(EshkolGPUBuffer* buffer);                    /* gpu_memory.h:183 */
int eshkol_gpu_wrap_host(void* host_ptr, size_t size_bytes,
                         EshkolGPUBuffer* out_buffer);            /* gpu_memory.h:195 */
int eshkol_gpu_sync(EshkolGPUBuffer* buffer, EshkolSyncDirection direction);   /* gpu_memory.h:208 */
int eshkol_gpu_sync_async(EshkolGPUBuffer* buffer, EshkolSyncDirection direction,
                          void* stream_handle);                   /* gpu_memory.h:217 */
void eshkol_gpu_wait(EshkolGPUBuffer* buffer);                    /* gpu_memory.h:224 */

/* ---- matrix products ---- */
/* C = A*B, row-major f64; the tier is chosen from the environment exactly as the
 * reference's backends read it.  gpu_memory.h:242 */
int eshkol_gpu_matmul_f64(EshkolGPUBuffer* A, EshkolGPUBuffer* B, EshkolGPUBuffer* C,
                          uint64_t M, uint64_t K, uint64_t N);
/* f32 buffers.  gpu_memory.h:250 */
int eshkol_gpu_matmul_f32(EshkolGPUBuffer* A, EshkolGPUBuffer* B, EshkolGPUBuffer* C,
                          uint64_t M, uint64_t K, uint64_t N);

/* ---- dispatch threshold ---- */
extern size_t g_gpu_threshold;                                    /* gpu_memory.h:261 */
void eshkol_gpu_set_threshold(size_t threshold);                  /* gpu_memory.h:267 */
size_t eshkol_gpu_get_threshold(void);                            /* gpu_memory.h:273 */
int eshkol_gpu_should_use(size_t num_elements);                   /* gpu_memory.h:280 */

/* ---- elementwise / reductions ---- */
/* gpu_memory.h:284-300 */
typedef enum {
  ESHKOL_ELEMWISE_ADD = 0, ESHKOL_ELEMWISE_SUB = 1, ESHKOL_ELEMWISE_MUL = 2,
  ESHKOL_ELEMWISE_DIV = 3, ESHKOL_ELEMWISE_NEG = 4, ESHKOL_ELEMWISE_ABS = 5,
  ESHKOL_ELEMWISE_EXP = 6, ESHKOL_ELEMWISE_LOG = 7, ESHKOL_ELEMWISE_SIN = 8,
  ESHKOL_ELEMWISE_COS = 9, ESHKOL_ELEMWISE_TANH = 10, ESHKOL_ELEMWISE_RELU = 11,
  ESHKOL_ELEMWISE_SIGMOID = 12, ESHKOL_ELEMWISE_SQRT = 13, ESHKOL_ELEMWISE_RECIPROCAL = 14
} EshkolElementwiseOp;

/* gpu_memory.h:302-308 */
typedef enum {
  ESHKOL_REDUCE_SUM = 0, ESHKOL_REDUCE_PROD = 1, ESHKOL_REDUCE_MIN = 2,
  ESHKOL_REDUCE_MAX = 3, ESHKOL_REDUCE_MEAN = 4
} EshkolReduceOp;

int eshkol_gpu_elementwise_f64(EshkolGPUBuffer* a, EshkolGPUBuffer* b, EshkolGPUBuffer* out,
                               uint64_t n, EshkolElementwiseOp op);          /* gpu_memory.h:322 */

/* The backend's other tensor operators.  They run on device buffers (every buffer needs a
 * device_ptr and room for its tensor) as the CUDA branch of the reference does
 * (lib/backend/gpu/gpu_memory_cuda.cpp:1229-1560); anything else returns -1, which every
 * caller in the reference treats as "run the CPU version".  Sums are shared by the threads of
 * a warp or block, so results agree with the reference's serial kernels to rounding. */
int eshkol_gpu_reduce_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t n,
                          EshkolReduceOp op);                                /* gpu_memory.h:335 */
int eshkol_gpu_reduce_axis_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t rank,
                               const uint64_t* shape, uint64_t axis,
                               EshkolReduceOp op);                           /* gpu_memory.h:351 */
int eshkol_gpu_transpose_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t rows,
                             uint64_t cols);                                 /* gpu_memory.h:364 */
int eshkol_gpu_softmax_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t num_slices,
                           uint64_t slice_len);                              /* gpu_memory.h:379 */
int eshkol_gpu_normalize_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t num_slices,
                             uint64_t slice_len, double gamma, double beta,
                             double epsilon);                                /* gpu_memory.h:395 */
int eshkol_gpu_conv2d_backward_input_f64(                                    /* gpu_memory.h:404 */
    EshkolGPUBuffer* grad_out, EshkolGPUBuffer* kernel_weights, EshkolGPUBuffer* grad_input,
    uint64_t in_h, uint64_t in_w, uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
    uint64_t stride_h, uint64_t stride_w, uint64_t channels_in, uint64_t channels_out,
    uint64_t batch_size);
int eshkol_gpu_conv2d_backward_kernel_f64(                                   /* gpu_memory.h:415 */
    EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input, EshkolGPUBuffer* grad_kernel,
    uint64_t in_h, uint64_t in_w, uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
    uint64_t stride_h, uint64_t stride_w, uint64_t channels_in, uint64_t channels_out,
    uint64_t batch_size);
int eshkol_gpu_batchnorm_backward_f64(                                       /* gpu_memory.h:426 */
    EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input, EshkolGPUBuffer* saved_mean,
    EshkolGPUBuffer* saved_inv_std, EshkolGPUBuffer* saved_gamma, EshkolGPUBuffer* grad_input,
    EshkolGPUBuffer* grad_gamma, EshkolGPUBuffer* grad_beta, uint64_t batch_size,
    uint64_t feature_size);
int eshkol_gpu_layernorm_backward_f64(                                       /* gpu_memory.h:437 */
    EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input, EshkolGPUBuffer* saved_mean,
    EshkolGPUBuffer* saved_inv_std, EshkolGPUBuffer* saved_gamma, EshkolGPUBuffer* grad_input,
    uint64_t num_samples, uint64_t feature_size);

/* ---- runtime integration: what generated code and the VM call ---- */
/* Host pointers owned by the caller, any alignment, valid for the call only.
 * dtype follows eshkol_tensor_dtype_t (lib/core/arena_memory.h:749-762); 2 and 3
 * (f16 / bf16) select the loosest tier.  gpu_memory.h:466 */
void eshkol_matmul_dispatch(const double* A, const double* B, double* C, uint64_t M, uint64_t K,
                            uint64_t N, int32_t dtype);
/* gpu_memory.h:472 */
void eshkol_batch_matmul_dispatch(const double* a, const double* b, double* c, int64_t batch,
                                  int64_t M, int64_t K, int64_t N, int32_t dtype);

/* conv2d forward on host arrays, the GPU twin of the loop the reference runs inside
 * eshkol_rt_conv2d (lib/backend/tensor_conv_kernel.cpp:32-109 calls
 * eshkol_conv2d_kernel, lib/backend/tensor_conv_kernel.h:66-105); same argument
 * order as that kernel plus a fused activation (0 none, 1 ReLU).  Returns 0 / -1. */
int eshkol_gpu_conv2d_f64(const double* in, int64_t batch, int64_t in_c, int64_t H, int64_t W,
                          const double* ker, int64_t out_c, int64_t kH, int64_t kW,
                          int64_t stride, int64_t pad, double* out, int32_t activation);

/* Both gradients of C = A * B on host arrays: grad_A[M x K] = grad_out * B^T and
 * grad_B[K x N] = A^T * grad_out.  The GPU branch of eshkol_matmul_backward_f64
 * (lib/backend/blas_backend.cpp:955-1012) in one call: that branch transposes A and B on the
 * host and wraps six buffers around two eshkol_gpu_matmul_f64 calls; here the operands are
 * uploaded once and read transposed on the device.  Each gradient carries the bits the
 * reference's two calls would produce in the same tier.  The tier follows the environment as
 * for the forward product, with each gradient's own shape.  Returns 0, or -1 when the GPU path
 * is unavailable or failed (the caller then takes its BLAS branch, as it does today); below the
 * element threshold of eshkol_gpu_should_use it returns -1 without touching the GPU. */
int eshkol_gpu_matmul_backward_f64(const double* grad_out, const double* A, const double* B,
                                   double* grad_A, double* grad_B, uint64_t M, uint64_t K, uint64_t N);

/* ---- residency of operands across eshkol_matmul_dispatch calls (no counterpart in the
 * reference, whose dispatcher wraps and unwraps host memory on every call,
 * lib/backend/gpu/gpu_memory_cuda.cpp:1136-1145) ----
 * Off unless ESHKOL_B200_RESIDENCY=1 or eshkol_gpu_set_residency(1, ...).  When on, the exact-tier
 * dispatcher keeps a device copy of every operand and result, keyed on (host pointer, bytes);
 * a later call that passes the same host range finds the copy and skips the upload, and a
 * right-hand operand that is still the library's prepared one also skips its split.  The
 * result of one call is found as an operand of the next, so a chain such as
 * (matmul (matmul A B) A) (tests/gpu/matmul_correctness_test.esk:54) uploads each distinct
 * operand once.  Results are still written to host memory on every call.
 * The host must call eshkol_gpu_invalidate after writing to a range it has passed before
 * (tensor-set!, an arena reset that reuses the address): the library cannot see host writes.
 * As a guard against a forgotten call, 256 values of the range, evenly spaced, are compared
 * with the ones seen at upload; a mismatch drops the copy.  Copies are evicted least recently
 * used first once they exceed limit_mb (ESHKOL_B200_RESIDENCY_MB, default 65536). */
void eshkol_gpu_set_residency(int on, size_t limit_mb);
/* Forget the device copy of any cached range that overlaps [host_ptr, host_ptr + bytes);
 * bytes = 0 means every range that contains host_ptr. */
void eshkol_gpu_invalidate(const void* host_ptr, size_t bytes);
/* Forget every cached range and free the device copies. */
void eshkol_gpu_residency_clear(void);

#ifdef __cplusplus
}
#endif

#endif /* ESHKOL_GPU_MEMORY_B200_H */
