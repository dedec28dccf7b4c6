/*
 * B200 extension entry points of libeshkol_gpu_b200.so.
 *
 * The drop-in boundary is include/eshkol_gpu_memory_b200.h (the reference's own
 * ABI).  The functions here sit one level below it: they take DEVICE pointers and
 * an explicit tier, so a host runtime that keeps tensors resident (and the tests
 * and the benchmark) can call the GEMM without the wrap/sync round trip that
 * eshkol_matmul_dispatch performs on every call
 * (reference: lib/backend/gpu/gpu_memory_cuda.cpp:1134-1147).
 *
 * All functions use plain C types.  Unless stated otherwise they return 0 on
 * success and a negative value on failure, and they enqueue work on the
 * library's stream without waiting for it.
 */
#ifndef ESHKOL_B200_EXT_H
#define ESHKOL_B200_EXT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Precision tiers of the f64 GEMM. */
typedef enum {
  /* Ozaki-II, CRT over the first `param` moduli (2..16; 0 means 16), residues of
   * the products combined exactly as the reference's exact tier does.
   * Reference: ozaki_ii_dispatch, lib/backend/gpu/gpu_memory.mm:2474-2771. */
  ESHKOL_B200_TIER_OZAKI2 = 0,
  /* Ozaki-I, int8 slices, slice pairs with p+q <= T kept, T = `param` (1..8; 0
   * means 6).  Reference: cuda_matmul_ozaki_int8_f64,
   * lib/backend/gpu/gpu_memory_cuda.cpp:339-452. */
  ESHKOL_B200_TIER_OZAKI1 = 1,
  /* Ozaki-II "fast" tier: frexp exponents, round-half-up significand shift, CRT in
   * exact 128-bit integers, `param` moduli (2..16; 0 means 11).
   * Reference: ozaki_ii_fast_dispatch, lib/backend/gpu/gpu_memory.mm:2816-3012. */
  ESHKOL_B200_TIER_OZAKI2_FAST = 2,
  /* Native f64 FMA GEMM on the CUDA cores (the stand-in for cublasDgemm,
   * lib/backend/gpu/gpu_memory_cuda.cpp:633-640). */
  ESHKOL_B200_TIER_DGEMM = 3
} EshkolB200Tier;

typedef struct EshkolB200GemmOpts {
  int32_t tier;             /* EshkolB200Tier */
  int32_t param;            /* tier parameter, 0 = tier default */
  int32_t activation;       /* fused into the last pass: 0 none, 1 ReLU (x > 0 ? x : 0), 2 the tanh-form GELU of
                               the reference's feed-forward (tensor_transformer_codegen.cpp:2469-2577) */
  int32_t bias_mode;        /* 0 none, 1 bias[row], 2 bias[column], added before the activation */
  const double* bias;       /* device pointer, M or N doubles */
  int64_t pixels_per_image; /* > 0: C is written as [N/pixels][M][pixels] (conv2d NCHW) */
  int32_t use_simt_products;/* tests only: integer products on CUDA cores instead of tcgen05 */
  int32_t gemm_tile_n;      /* 0 = default (256), or 128 */
  int64_t ldc;              /* elements between rows of C; 0 = N (C may be a column panel of a wider matrix) */
  int32_t trans_a;          /* 1: A is stored K x M row-major (the product uses its transpose) */
  int32_t trans_b;          /* 1: B is stored N x K row-major (the product uses its transpose) */
} EshkolB200GemmOpts;

/* Selects `device`, creates the stream and queries the SM count.  Idempotent.
 * Returns 0, or -1 when no sm_100 device is usable. */
int eshkol_b200_init(int device);
void eshkol_b200_shutdown(void);

/* The CUDA stream (cudaStream_t) every call of this library enqueues on. */
void* eshkol_b200_stream(void);

/* C[M x N] = op(A)[M x K] * op(B)[K x N], row-major f64, all three in device memory.
 * Asynchronous.  opts may be NULL (exact tier, no epilogue, no transposes).  With
 * opts->trans_a / trans_b an operand is read in its transposed storage: the exact tier
 * (16 moduli) reads it directly -- a transposed A goes through the column scan and the
 * transposing split that B normally takes, a transposed B through the row scan and split
 * of A -- and the result carries the bits of the product of the explicitly transposed
 * matrices; the other tiers transpose into library scratch first.  This is what the
 * gradients of a product need (grad_A = G * B^T, grad_B = A^T * G) without the host-side
 * transposes of lib/backend/blas_backend.cpp:969-977. */
int eshkol_b200_gemm_f64_device(const double* dA, const double* dB, double* dC,
                                uint64_t M, uint64_t K, uint64_t N,
                                const EshkolB200GemmOpts* opts);

/* Device time in milliseconds of the last eshkol_b200_gemm_f64_device call (two events on the
 * library stream around everything it enqueued); waits for that call.  -1 when there is none.
 * The C host layer feeds it to the time model of its accuracy-budget selector, as the reference
 * feeds its wall-clock time (lib/backend/gpu/gpu_memory_cuda.cpp:605-614). */
double eshkol_b200_last_gemm_ms(void);

/* feed-forward block on device tensors, the arithmetic of the loops the reference generates inline
 * for (feed-forward x W1 b1 W2 b2) (lib/backend/tensor_transformer_codegen.cpp:2557-2664):
 *   out[rows x d_model] = gelu(x[rows x d_model] * W1[d_model x d_ff] + b1) * W2[d_ff x d_model] + b2
 * as two GEMMs of the tier opts selects with bias and activation fused into their last pass; the
 * hidden activations stay in library scratch.  The GEMMs are exact-tier sums where the generated
 * loops add one product at a time, and exp is the device's: agreement is to rounding, not bits.
 * Asynchronous; 0 / -1. */
int eshkol_b200_feed_forward_f64_device(const double* d_x, const double* d_w1, const double* d_b1,
                                        const double* d_w2, const double* d_b2, double* d_out,
                                        uint64_t rows, uint64_t d_model, uint64_t d_ff,
                                        const EshkolB200GemmOpts* opts);

/* conv2d backward on device tensors (NCHW, no padding, strides sH / sW), the two kernels of
 * lib/backend/gpu/gpu_cuda_kernels.cu:413-486 as GEMMs in the tier opts selects:
 *   grad_kernel[co][ci][kh][kw] = (grad_out as co x batch*pixels) * im2col(input)^T
 *   grad_input = gather over (kh, kw) of  weights^T (ci*kh*kw x co) * (grad_out as co x batch*pixels)
 * Both transposed operands are read in place.  In the exact tier every GEMM element is the
 * exact-tier sum where the reference adds products one by one in f64, so results agree to the
 * reference's own rounding error, not bit for bit.  Asynchronous; 0 / -1. */
int eshkol_b200_conv2d_backward_kernel_f64_device(const double* d_grad_out, const double* d_input,
                                                  double* d_grad_kernel, uint64_t in_h, uint64_t in_w,
                                                  uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
                                                  uint64_t stride_h, uint64_t stride_w, uint64_t channels_in,
                                                  uint64_t channels_out, uint64_t batch,
                                                  const EshkolB200GemmOpts* opts);
int eshkol_b200_conv2d_backward_input_f64_device(const double* d_grad_out, const double* d_weights,
                                                 double* d_grad_input, uint64_t in_h, uint64_t in_w,
                                                 uint64_t k_h, uint64_t k_w, uint64_t out_h, uint64_t out_w,
                                                 uint64_t stride_h, uint64_t stride_w, uint64_t channels_in,
                                                 uint64_t channels_out, uint64_t batch,
                                                 const EshkolB200GemmOpts* opts);

/* The dtype fast path (f16 / bf16-tagged tensors keep f64 storage): for b < batch,
 * C[b][M x N] = f16(A[b]) * f16(B[b]) with f32 accumulation on the tensor cores
 * (tcgen05.mma kind::f16), the result rounded to f16 and widened back to f64 -- the arithmetic of
 * cuda_matmul_f16_from_f64 / cuda_batch_matmul_f16_from_f64
 * (lib/backend/gpu/gpu_memory_cuda.cpp:677-784) up to the order of the f32 accumulation, with
 * the f64 -> f32 -> f16 conversion (two roundings, as the reference's host loop) done on the
 * device.  Matrices of a batch are contiguous; one kernel launch multiplies the whole batch.
 * Device pointers; asynchronous.  Returns 0 / -1. */
int eshkol_b200_gemm_f16_device(const double* dA, const double* dB, double* dC, uint64_t batch,
                                uint64_t M, uint64_t K, uint64_t N);

/* C = A * B on f32 matrices in device memory (the role of cuda_matmul_f32,
 * gpu_memory_cuda.cpp:653-669): widened to f64, multiplied in the exact tier, narrowed with one
 * rounding, so every element is the correctly rounded f32 of the exact-tier product.
 * Asynchronous.  Returns 0 / -1. */
int eshkol_b200_gemm_f32_device(const float* dA, const float* dB, float* dC, uint64_t M, uint64_t K,
                                uint64_t N);

/* Both gradients of C = A * B from host memory (the GPU branch of
 * eshkol_matmul_backward_f64, lib/backend/blas_backend.cpp:924-1012, without its host
 * transposes): grad_A[M x K] = grad_out[M x N] * B^T, grad_B[K x N] = A^T * grad_out, each
 * with the bits of eshkol_b200_gemm_f64_device on the explicitly transposed operand.
 * Synchronous; returns 0 or -1.  opts_grad_a / opts_grad_b select the tier of each product as
 * for the forward one (NULL = exact tier); only their tier and param are used. */
int eshkol_b200_matmul_backward_f64_host(const double* grad_out, const double* A, const double* B,
                                         double* grad_A, double* grad_B, uint64_t M, uint64_t K,
                                         uint64_t N, const EshkolB200GemmOpts* opts_grad_a,
                                         const EshkolB200GemmOpts* opts_grad_b);

/* Exact tier (16 moduli) with the right-hand operand prepared once: prepare_b scans
 * and splits B (K x N, device memory) into library-owned residue planes; each
 * gemm_prepared call then multiplies a block of rows, C[M x N] = A[M x K] * B, with
 * the bits of the same rows of a one-shot product (rows are independent).  The
 * prepared operand stays valid until the next prepare_b, any other GEMM of this
 * library, or shutdown; B itself is not read again.  This is what lets a caller
 * reuse one B (weights) across many products, pipeline row blocks against PCIe, or
 * shard rows across GPUs.  The reference re-uploads and re-splits both operands on
 * every call (lib/backend/gpu/gpu_memory.mm:2538-2583).  Asynchronous. */
int eshkol_b200_prepare_b_f64_device(const double* dB, uint64_t K, uint64_t N);
int eshkol_b200_gemm_prepared_f64_device(const double* dA, double* dC, uint64_t M,
                                         const EshkolB200GemmOpts* opts);
/* The left-hand twin: prepare_a scans and splits a block of rows of A once (room for
 * results up to n_cols_hint columns wide is reserved with it); multiply_prepared then
 * forms C = A * B from the two prepared operands, e.g. once per column panel of B as
 * the panels arrive from another GPU.  opts->ldc lets C be a column panel of a wider
 * matrix.  The prepared A stays valid until another GEMM of this library needs more
 * workspace than is held, or prepare_a is called again.  Asynchronous. */
int eshkol_b200_prepare_a_f64_device(const double* dA, uint64_t M, uint64_t K, uint64_t n_cols_hint);
int eshkol_b200_multiply_prepared_f64_device(double* dC, const EshkolB200GemmOpts* opts);

/* A right-hand operand prepared in pieces, by several GPUs (no counterpart in the reference,
 * which is single-device).  Preparing B -- the column scan and the split into 16 residue
 * planes -- is the same work on every GPU that multiplies its own rows of A by that B; these
 * entry points let each of G ranks prepare 1/G of a panel's columns and fetch the other ranks'
 * pieces with the copy engines instead (16.3 bytes per element where the f64 panel is 8, but
 * none of it on the SMs).
 *   prepared_b_bytes      size of the buffer that holds a whole prepared K x N operand; the
 *                         caller allocates it (eshkol_b200_mem_alloc, so that peers can open it)
 *   prepare_b_columns     scans and splits columns [col0, col0 + ncols) of that operand into
 *                         their places in `planes`; dB points at the first of those columns,
 *                         consecutive rows ldb elements apart.  Asynchronous
 *   prepared_b_regions    the seven pieces of those columns inside the buffer, each as
 *                         {byte offset, bytes per row, rows, pitch}: shifts and both scale
 *                         vectors, the modulus-256 plane, its two flag planes, and the 15 odd
 *                         planes as one pitched region -- what a peer copies (copy2d_async)
 *   adopt_prepared_b      declares that `planes` now holds the complete operand: it becomes the
 *                         library's prepared right-hand operand (multiply_prepared uses it).
 *                         The buffer stays the caller's and must outlive its use.
 * All return 0 / -1 (regions: the number of regions). */
uint64_t eshkol_b200_prepared_b_bytes(uint64_t K, uint64_t N);
int eshkol_b200_prepare_b_columns_f64_device(const double* dB, uint64_t ldb, uint64_t K, uint64_t N, uint64_t col0,
                                             uint64_t ncols, void* planes);
int eshkol_b200_prepared_b_regions(uint64_t K, uint64_t N, uint64_t col0, uint64_t ncols, uint64_t out[7][4]);
int eshkol_b200_adopt_prepared_b(void* planes, uint64_t K, uint64_t N);

/* Exact tier on HOST arrays (what eshkol_matmul_dispatch runs for large shapes): B is
 * uploaded and prepared once, then 1024-row blocks of A are uploaded, multiplied and
 * their rows of C downloaded on three streams so PCIe and the tensor cores overlap.
 * Returns when C is complete in host memory: 0, -1 on failure, -2 when opts ask for a
 * tier this path does not serve (the caller then uses the buffer API).  Pinned host
 * memory is read and written by DMA directly; pageable memory (what an arena hands out)
 * moves in chunks through pinned staging slots filled by a few copy threads
 * (ESHKOL_B200_COPY_THREADS, default 8) -- same bits, about half the rate. */
int eshkol_b200_matmul_f64_host(const double* hA, const double* hB, double* hC, uint64_t M,
                                uint64_t K, uint64_t N, const EshkolB200GemmOpts* opts);

/* The host pipeline with device copies the CALLER keeps between calls (the mechanism under the
 * residency cache of eshkol_matmul_dispatch; the reference wraps and unwraps host memory on
 * every call, lib/backend/gpu/gpu_memory_cuda.cpp:1136-1145).  dA, dB, dC are device buffers of
 * M*K, K*N and M*N doubles.  a_state 0: hA is uploaded into dA block by block, overlapped with
 * the products; 1: dA already holds A (hA is not read).  b_state 0: hB is uploaded into dB and
 * prepared; 1: dB already holds B and is prepared from there; 2: the library's prepared
 * right-hand operand is still this B -- the caller checks that eshkol_b200_prepared_b_token()
 * equals the token this function wrote when it prepared that B -- and nothing is uploaded or
 * split.  C is written to dC and downloaded to hC.  Returns when hC is complete; 0 / -1.
 * *prepared_token receives the token of the operand now prepared (0 if none). */
int eshkol_b200_matmul_f64_host_resident(const double* hA, const double* hB, double* hC, uint64_t M,
                                         uint64_t K, uint64_t N, double* dA, int a_state, double* dB,
                                         int b_state, double* dC, uint64_t* prepared_token);
/* Token of the currently prepared right-hand operand: changes whenever one is prepared, 0 when
 * none is valid (any one-shot GEMM invalidates it). */
uint64_t eshkol_b200_prepared_b_token(void);
/* Bytes this library has copied host -> device and device -> host since init. */
void eshkol_b200_transfer_bytes(uint64_t* h2d, uint64_t* d2h);

/* The same exact-tier product (16 moduli, identical bits) for callers that must not
 * allocate: a host whose own arena already owns all device memory, so that
 * cudaMalloc would fail, or one that cannot take the device-wide synchronisation
 * and possible out-of-memory failure of cudaMalloc / cudaFree next to its other
 * streams.  Every intermediate lives in a fixed 24 MiB array inside the library
 * (held by each GPU that loads it, until exit); no allocating routine is called.
 * A, B and C are device pointers owned by the caller.  Shapes whose scratch need
 * exceeds the array (roughly 16*(M+N)*K + 17*M*N bytes after padding; 512x512x512
 * and 256x2048x256 fit) are refused with a message and -1.  Calls share the array:
 * they are ordered on the library stream and must not be made to overlap on the GPU.
 * eshkol_b200_init resolves the array's address on its device (that is when the CUDA
 * runtime loads the array's module and takes the 24 MiB), so a host that hands the
 * rest of device memory to its own arena must call eshkol_b200_init before it does,
 * and before any stream capture.  Asynchronous.  This entry point has no counterpart
 * in the reference. */
int eshkol_b200_gemm_f64_static_scratch(const double* dA, const double* dB, double* dC,
                                        uint64_t M, uint64_t K, uint64_t N);

/* conv2d forward, NCHW cross-correlation with zero padding, lowered to the same
 * GEMM: out[b][oc][oh][ow] = sum_{ic,kh,kw} in[b][ic][oh*s+kh-p][ow*s+kw-p] * ker[oc][ic][kh][kw].
 * Device pointers; out is [batch][out_c][oH][oW].  Asynchronous.
 * Reference semantics: eshkol_conv2d_kernel, lib/backend/tensor_conv_kernel.h:66-105. */
int eshkol_b200_conv2d_f64_device(const double* d_in, int64_t batch, int64_t in_c, int64_t H,
                                  int64_t W, const double* d_ker, int64_t out_c, int64_t kH,
                                  int64_t kW, int64_t stride, int64_t pad, double* d_out,
                                  const EshkolB200GemmOpts* opts);

/* Memory services for the C host layer.  kind: 0 device (cudaMalloc), 1 managed,
 * 2 pinned host.  Copies are asynchronous on the library stream; a pageable host
 * range is staged by the CUDA runtime, a pinned one is read by DMA directly. */
int eshkol_b200_mem_alloc(int kind, size_t bytes, void** out_ptr);
void eshkol_b200_mem_free(int kind, void* ptr);
int eshkol_b200_copy_h2d(void* device_dst, const void* host_src, size_t bytes);
int eshkol_b200_copy_d2h(void* host_dst, const void* device_src, size_t bytes);

/* out[i] = op(a[i], b[i]) over n device-resident doubles; op numbering and the
 * meaning of a missing b follow elementwise_f64_kernel,
 * lib/backend/gpu/gpu_cuda_kernels.cu:21-43 (ReLU is x > 0 ? x : 0).  Asynchronous. */
int eshkol_b200_elementwise_f64_device(const double* a, const double* b, double* out,
                                       uint64_t n, int op);

/* The backend's other tensor operators on device-resident doubles (asynchronous on the library
 * stream; -1 on bad arguments).  Arithmetic follows the reference's kernels in
 * lib/backend/gpu/gpu_cuda_kernels.cu -- reduce :76-141 (op: 0 sum, 1 product, 2 min, 3 max,
 * 4 mean; min / max ignore NaN), axis reduce :147-180 (the tensor seen as
 * [outer][axis_len][inner]), transpose :189-213, softmax :319-343 (a zero sum divides by 1),
 * normalize :364-389 (population variance, rsqrt), batchnorm / layernorm backward :489-555 --
 * with sums shared by the threads of a warp or block, so they agree with the reference's serial
 * sums to rounding, not bit for bit.  softmax and normalize may run in place. */
int eshkol_b200_reduce_f64_device(const double* in, double* out, uint64_t n, int op);
int eshkol_b200_reduce_axis_f64_device(const double* in, double* out, uint64_t outer, uint64_t axis_len,
                                       uint64_t inner, int op);
int eshkol_b200_transpose_f64_device(const double* in, double* out, uint64_t rows, uint64_t cols);
int eshkol_b200_softmax_f64_device(const double* in, double* out, uint64_t num_slices, uint64_t slice_len);
int eshkol_b200_normalize_f64_device(const double* in, double* out, uint64_t num_slices, uint64_t slice_len,
                                     double gamma, double beta, double epsilon);
int eshkol_b200_batchnorm_backward_f64_device(const double* grad_out, const double* saved_input,
                                              const double* saved_mean, const double* saved_inv_std,
                                              const double* saved_gamma, double* grad_input, double* grad_gamma,
                                              double* grad_beta, uint64_t batch, uint64_t features);
int eshkol_b200_layernorm_backward_f64_device(const double* grad_out, const double* saved_input,
                                              const double* saved_mean, const double* saved_inv_std,
                                              const double* saved_gamma, double* grad_input, uint64_t samples,
                                              uint64_t features);

/* Waits for the stream, then returns 0 if every kernel since the previous call
 * completed normally, a positive kernel status code if a bounded wait inside a
 * kernel ran out, or -1 on a CUDA error. */
int eshkol_b200_sync_status(void);

/* Selects the products kernel of the exact tier's odd moduli: 0 = one CTA per 128 x 256
 * tile, 1 = CTA pairs on 256 x 256 tiles (tcgen05 cta_group::2, each SM loads half of the B
 * tile).  Same results either way.  Initial value: environment ESHKOL_B200_PAIR_GEMM. */
void eshkol_b200_set_pair_gemm(int on);

/* Copy-engine transfers for the multi-GPU driver (no counterpart in the reference, which is
 * single-device).  enable_peer_access lets the library's device read and write peer_device's
 * memory directly over NVLink (0 = enabled or already so, -1 = no peer path).  copy_async
 * enqueues one cudaMemcpyAsync of `bytes` bytes on `stream` (a cudaStream_t exactly as CUDA
 * reads it: NULL is the legacy default stream, eshkol_b200_stream() the library's); dst and src are device pointers of this process, either of which may
 * live on a peer device (e.g. another rank's buffer opened through CUDA IPC).  The copy
 * engines move the data, no SM is used: measured on a B200, a 1 GiB device-to-device copy on a
 * second stream finishes in 4.7 ms beside a running exact-tier product, while kernels of other
 * streams (a collective's, an elementwise copy) wait for the gaps between the products
 * kernels, whose CTAs hold every SM in the maximum shared-memory configuration. */
int eshkol_b200_enable_peer_access(int peer_device);
int eshkol_b200_copy_async(void* dst, const void* src, size_t bytes, void* stream);
/* The same for `rows` rows of width_bytes bytes with pitches (cudaMemcpy2DAsync): a column
 * panel of a row-major matrix moves in one call. */
int eshkol_b200_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                             size_t width_bytes, size_t rows, void* stream);

/* Interprocess handles for the one-process-per-GPU driver (no counterpart in the reference).
 * export_mem writes the 64-byte CUDA IPC handle of an allocation made with
 * eshkol_b200_mem_alloc(0, ...) (device_ptr must be the pointer that call returned);
 * import_mem opens a peer rank's handle in this rank's own context, with peer access to the
 * owning device enabled on demand, and returns a device pointer valid for copy_async /
 * copy2d_async.  event_create makes an interprocess event (no timing) and writes its 64-byte
 * handle; event_import opens a peer's.  record / wait enqueue cudaEventRecord /
 * cudaStreamWaitEvent on `stream` (a cudaStream_t as CUDA reads it, NULL = legacy default).  A wait on an imported event
 * waits for the most recent record the owner has *called*, so the ranks must agree on the
 * host (a barrier) that the record was called before a peer calls wait.  All return 0 / -1. */
int eshkol_b200_ipc_export_mem(void* device_ptr, unsigned char handle[64]);
int eshkol_b200_ipc_import_mem(const unsigned char handle[64], void** device_ptr);
int eshkol_b200_ipc_close_mem(void* device_ptr);
int eshkol_b200_ipc_event_create(void** event, unsigned char handle[64]);
int eshkol_b200_ipc_event_import(const unsigned char handle[64], void** event);
int eshkol_b200_event_record(void* event, void* stream);
int eshkol_b200_event_wait(void* event, void* stream);
int eshkol_b200_event_destroy(void* event);

/* Number of SMs the persistent tensor-core products kernels occupy (one CTA each); 0 = all.
 * The multi-GPU driver leaves a few SMs free so that the communication library's kernels,
 * which cannot share an SM with a products CTA (shared memory), run beside the products
 * instead of waiting for the gaps between them.  Odd values are rounded down. */
void eshkol_b200_set_sm_limit(int sms);

/* Row-band pipeline of the one-shot exact-tier product (eshkol_b200_gemm_f64_device and
 * eshkol_b200_gemm_prepared_f64_device): with at least two bands of `rows` rows of A, band
 * r+1 is scanned and split while band r is multiplied and band r-1 is reconstructed, on
 * three streams over two workspace slots.  Rows of the result depend on their own row of A
 * and on B only, so the bits do not change.  rows is rounded up to a multiple of 256;
 * 0 switches the pipeline off.  Initial value 0 (off), or environment ESHKOL_B200_BAND_ROWS:
 * on a power-capped B200 the overlapped kernels slow the tensor-core products by about as
 * much as they hide (8192^3: 7.85 ms serial, 7.78 ms in 4 bands; 16384^3: 59.6 vs 62.8 ms).
 * The library stream is ordered behind the last band when the call returns. */
void eshkol_b200_set_row_bands(long long rows);

/* Per-stage timing of the Ozaki-II driver, the counterpart of the reference's
 * ESHKOL_OZAKI_PROFILE line (lib/backend/gpu/gpu_memory.mm:2479, 2658-2664).  When
 * switched on, CUDA events on the library stream bracket each stage of every
 * Ozaki-II GEMM.  get_phase_times waits for the stream and writes the durations
 * of the LAST 16-moduli GEMM in milliseconds: [0] column scan + scales of B,
 * [1] split B, [2] row scan + scales of A, [3] split A, [4] products modulo 256,
 * [5] products modulo the odd moduli, [6] reconstruction.  When the product ran through
 * the row-band pipeline, each of [2]..[6] is the sum over the bands of that stage's kernels
 * on their own stream (the stages overlap, so they add up to more than the product took)
 * and, if capacity >= 8, [7] is the number of bands (0 for a serial product).  Returns 7,
 * or -1 when nothing was timed. */
void eshkol_b200_set_phase_timing(int on);
int eshkol_b200_get_phase_times(float* ms, int capacity);
/* The same seven stages summed over every stage call made since timing was switched on
 * (at most the last 256 calls of each group are kept): counts[0] = right-hand operands
 * prepared, counts[1] = left-hand operands prepared, counts[2] = multiplications.  The
 * multi-GPU driver prepares A once and B once per column panel, so the three counts differ
 * there.  Waits for the stream.  Returns 0, or -1 when timing was never switched on. */
int eshkol_b200_get_phase_totals(float ms[7], int counts[3]);

/* Number of kernels this library has launched since init (monotonic). */
uint64_t eshkol_b200_launch_count(void);

/* Bytes of device scratch currently held by the library's workspace. */
uint64_t eshkol_b200_workspace_bytes(void);

#ifdef __cplusplus
}
#endif

#endif /* ESHKOL_B200_EXT_H */
