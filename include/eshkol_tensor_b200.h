/*
 * The tensor-struct side of the conv2d path: the heap tensor as generated code lays it out,
 * and the runtime entry point that code calls for (conv2d input kernel stride [pad]).
 *
 * Reference: eshkol_tensor_t, lib/core/arena_memory.h:768-780 (40 bytes, five 8-byte fields,
 * elements are doubles stored as int64 bit patterns; static assert at :781-785);
 * eshkol_rt_conv2d, lib/backend/tensor_conv_kernel.cpp:32-109.
 */
#ifndef ESHKOL_TENSOR_B200_H
#define ESHKOL_TENSOR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* A translation unit that also includes the reference's own arena_memory.h already has this
 * type and defines ESHKOL_ARENA_MEMORY_H. */
#ifndef ESHKOL_ARENA_MEMORY_H
typedef struct eshkol_tensor {
  uint64_t* dimensions;     /* dimension sizes */
  uint64_t num_dimensions;  /* rank */
  int64_t* elements;        /* doubles as int64 bit patterns */
  uint64_t total_elements;  /* product of the dimensions */
  uint64_t dtype;           /* 0 f64, 1 f32, 2 f16, 3 bf16, 4 i8 (arena_memory.h:749-765) */
} eshkol_tensor_t;
#endif

/* conv2d(input, kernel) into a fresh arena tensor, on the GPU: NCHW cross-correlation lowered
 * to the exact-tier GEMM.  Shape contract of tensor_conv_kernel.cpp:32-109: the last two
 * dimensions of both tensors are the spatial ones; a rank >= 4 kernel is [out_c, in_c, kH, kW]
 * and the input [..., in_c, H, W] with every leading dimension a batch index; a rank-2 kernel is
 * a single plane applied to every leading plane of the input (in_c = out_c = 1), the output
 * keeping the input's rank.  stride <= 0 is taken as 1, pad < 0 as 0.  Returns NULL on a shape
 * error, when the arena cannot allocate, or when the GPU path fails (it then says so on
 * stderr): there is no CPU result.  The output tensor comes from the runtime's
 * arena_allocate_tensor_full (lib/core/arena_memory.h:793), resolved when this library is
 * linked into Eshkol, or from the allocator given to eshkol_b200_set_tensor_allocator. */
eshkol_tensor_t* eshkol_rt_conv2d(void* arena, const eshkol_tensor_t* input, const eshkol_tensor_t* kernel,
                                  int64_t stride, int64_t pad);

/* A host that is not Eshkol's runtime (a test, an embedding) supplies the allocator of result
 * tensors: same contract as arena_allocate_tensor_full -- a tensor whose dimensions and elements
 * arrays exist, num_dimensions and total_elements set.  NULL restores the runtime's symbol.
 * No counterpart in the reference. */
typedef eshkol_tensor_t* (*eshkol_b200_tensor_allocator)(void* arena, uint64_t num_dims, uint64_t total_elements);
void eshkol_b200_set_tensor_allocator(eshkol_b200_tensor_allocator fn);

#ifdef __cplusplus
}
#endif

#endif /* ESHKOL_TENSOR_B200_H */
