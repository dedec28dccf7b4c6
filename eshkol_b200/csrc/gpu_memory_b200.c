/*
 * Host side of the drop-in backend, in C: buffer handles, the dispatch policy and
 * the environment switches of the reference's GPU backends, on top of the thin
 * device-level shim (include/eshkol_b200_ext.h).
 *
 * What each function mirrors in the reference:
 *   init / shutdown / queries      lib/backend/gpu/gpu_memory_cuda.cpp:839-920
 *   alloc / free / wrap / sync     lib/backend/gpu/gpu_memory_cuda.cpp:168-285, 793-821, 924-1027
 *   tier selection for f64 matmul  lib/backend/gpu/gpu_memory_cuda.cpp:310-326, 527-566, 577-650
 *                                  lib/backend/gpu/gpu_memory.mm:1309-1343, 3028-3051
 *   eshkol_matmul_dispatch         lib/backend/gpu/gpu_memory_cuda.cpp:1107-1157
 *   eshkol_batch_matmul_dispatch   lib/backend/gpu/gpu_memory_cuda.cpp:1165-1175
 *
 * Differences that are deliberate:
 *   - a wrapped host buffer is staged into device memory (one DMA in, one out)
 *     instead of being mapped: the GEMM reads each operand many times and must
 *     not do so across PCIe;
 *   - there is no silent CPU result.  Below the element threshold the call is
 *     handed to the runtime's eshkol_matmul_f64 when that symbol is linked in
 *     (dispatch policy, unchanged); a failure of the GPU path is reported on
 *     stderr and by the return value, and the void dispatchers then fill C with
 *     NaN rather than a number of unknown provenance.
 */
#include "../../include/eshkol_gpu_memory_b200.h"
#include "../../include/eshkol_b200_ext.h"
#include "../../include/eshkol_b200_testing.h"

#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

size_t g_gpu_threshold = 100000; /* gpu_memory_cuda.cpp:107 */

static EshkolGPUBackend g_backend = ESHKOL_GPU_NONE;
static int g_initialized = 0;
static pthread_mutex_t g_init_mutex = PTHREAD_MUTEX_INITIALIZER;

/* bit 0 and 1 as in the reference (gpu_memory_cuda.cpp:123-124); bit 2 marks a wrapped
 * buffer whose device copy was written by an operator and not yet copied back */
enum { FLAG_WRAPPED = 1u << 0, FLAG_COPY_BACK = 1u << 1, FLAG_DIRTY = 1u << 2 };

/* CPU entry points of the host runtime; present when this object is linked into
 * Eshkol, absent when the library is used on its own. */
extern void eshkol_matmul_f64(const double*, const double*, double*, uint64_t, uint64_t, uint64_t)
    __attribute__((weak));
extern void eshkol_batch_matmul_f64(const double*, const double*, double*, int64_t, int64_t,
                                    int64_t, int64_t) __attribute__((weak));

static int gpu_verbose(void) {
  static int checked = 0, verbose = 0;
  if (!checked) { verbose = getenv("ESHKOL_GPU_VERBOSE") != NULL; checked = 1; }
  return verbose;
}
#define GPU_LOG(...) do { if (gpu_verbose()) { fprintf(stderr, "[GPU] " __VA_ARGS__); fputc('\n', stderr); } } while (0)

/* ------------------------------------------------------------------ init ---- */
int eshkol_gpu_init(void) {
  if (__atomic_load_n(&g_initialized, __ATOMIC_ACQUIRE)) return g_backend != ESHKOL_GPU_NONE;
  pthread_mutex_lock(&g_init_mutex);
  if (!g_initialized) {
    const char* env = getenv("ESHKOL_GPU_THRESHOLD");
    if (env) {
      long v = atol(env);
      if (v > 0) g_gpu_threshold = (size_t)v;
    }
    int dev = 0;
    const char* denv = getenv("ESHKOL_B200_DEVICE");
    if (denv) dev = atoi(denv);
    g_backend = (eshkol_b200_init(dev) == 0) ? ESHKOL_GPU_CUDA : ESHKOL_GPU_NONE;
    __atomic_store_n(&g_initialized, 1, __ATOMIC_RELEASE);
  }
  pthread_mutex_unlock(&g_init_mutex);
  return g_backend != ESHKOL_GPU_NONE;
}

void eshkol_gpu_residency_clear(void);

void eshkol_gpu_shutdown(void) {
  pthread_mutex_lock(&g_init_mutex);
  if (g_backend == ESHKOL_GPU_CUDA) {
    eshkol_gpu_residency_clear();
    eshkol_b200_shutdown();
  }
  g_backend = ESHKOL_GPU_NONE;
  __atomic_store_n(&g_initialized, 0, __ATOMIC_RELEASE);
  pthread_mutex_unlock(&g_init_mutex);
}

EshkolGPUBackend eshkol_gpu_get_backend(void) { return g_backend; }

const char* eshkol_gpu_backend_name(EshkolGPUBackend backend) {
  switch (backend) {
    case ESHKOL_GPU_NONE: return "CPU (no GPU)";
    case ESHKOL_GPU_METAL: return "Apple Metal (not available on Linux)";
    case ESHKOL_GPU_CUDA: return "NVIDIA CUDA";
    case ESHKOL_GPU_VULKAN: return "Vulkan";
  }
  return "Unknown";
}

int eshkol_gpu_backend_available(EshkolGPUBackend backend) { return g_backend == backend; }
int eshkol_gpu_supports_f64(void) { return g_backend == ESHKOL_GPU_CUDA; }
int eshkol_gpu_has_fp64(void) { return eshkol_gpu_supports_f64(); }

/* ---------------------------------------------------------------- memory ---- */
int eshkol_gpu_alloc(size_t size_bytes, EshkolMemoryType mem_type, EshkolGPUBuffer* out) {
  if (!out || size_bytes == 0) return -1;
  memset(out, 0, sizeof(*out));
  if (g_backend != ESHKOL_GPU_CUDA) {
    out->host_ptr = malloc(size_bytes);
    if (!out->host_ptr) return -1;
    out->device_ptr = out->host_ptr;
    out->size_bytes = size_bytes;
    out->mem_type = ESHKOL_MEM_HOST;
    out->backend = ESHKOL_GPU_NONE;
    return 0;
  }
  void* p = NULL;
  switch (mem_type) {
    case ESHKOL_MEM_DEVICE:
      if (eshkol_b200_mem_alloc(0, size_bytes, &p)) return -1;
      out->device_ptr = p;
      break;
    case ESHKOL_MEM_HOST_PINNED:
      if (eshkol_b200_mem_alloc(2, size_bytes, &p)) return -1;
      out->host_ptr = p;
      break;
    default: /* unified, and anything else, as the reference does */
      if (eshkol_b200_mem_alloc(1, size_bytes, &p)) return -1;
      out->host_ptr = p;
      out->device_ptr = p;
      mem_type = (mem_type == ESHKOL_MEM_UNIFIED) ? ESHKOL_MEM_UNIFIED : mem_type;
      break;
  }
  out->size_bytes = size_bytes;
  out->mem_type = mem_type;
  out->backend = ESHKOL_GPU_CUDA;
  return 0;
}

int eshkol_gpu_alloc_aligned(size_t size_bytes, size_t alignment, EshkolMemoryType mem_type,
                             EshkolGPUBuffer* out) {
  if (alignment == 0) alignment = 1;
  const size_t aligned = (size_bytes + alignment - 1) & ~(alignment - 1);
  return eshkol_gpu_alloc(aligned, mem_type, out);
}

static int copy_back(EshkolGPUBuffer* b) {
  if (!(b->flags & FLAG_COPY_BACK) || !b->backend_data || !b->device_ptr) return 0;
  if (eshkol_b200_copy_d2h(b->backend_data, b->device_ptr, b->size_bytes)) return -1;
  b->flags &= ~(uint32_t)FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}

void eshkol_gpu_free(EshkolGPUBuffer* b) {
  if (!b) return;
  if (b->backend == ESHKOL_GPU_CUDA) {
    if (b->flags & FLAG_WRAPPED) {
      /* the device copy is ours, the host memory is the caller's.  A caller that
       * frees without syncing (lib/backend/vm_gpu_dispatch.h:78-83) still gets its
       * result: an operator's output is copied back here, as cuda_free does for its
       * staged buffers (gpu_memory_cuda.cpp:214-219). */
      if (b->flags & FLAG_DIRTY) (void)copy_back(b);
      if (b->device_ptr) eshkol_b200_mem_free(0, b->device_ptr);
    } else if (b->mem_type == ESHKOL_MEM_HOST_PINNED) {
      if (b->host_ptr) eshkol_b200_mem_free(2, b->host_ptr);
    } else if (b->device_ptr) {
      eshkol_b200_mem_free(0, b->device_ptr);
    }
  } else if (b->host_ptr && !(b->flags & FLAG_WRAPPED)) {
    free(b->host_ptr);
  }
  memset(b, 0, sizeof(*b));
}

int eshkol_gpu_wrap_host(void* host_ptr, size_t size_bytes, EshkolGPUBuffer* out) {
  if (!host_ptr || !out || size_bytes == 0) return -1;
  memset(out, 0, sizeof(*out));
  if (g_backend != ESHKOL_GPU_CUDA) {
    out->host_ptr = host_ptr;
    out->device_ptr = host_ptr;
    out->size_bytes = size_bytes;
    out->mem_type = ESHKOL_MEM_HOST;
    out->backend = ESHKOL_GPU_NONE;
    out->flags = FLAG_WRAPPED;
    return 0;
  }
  void* d = NULL;
  if (eshkol_b200_mem_alloc(0, size_bytes, &d)) return -1;
  if (eshkol_b200_copy_h2d(d, host_ptr, size_bytes)) { eshkol_b200_mem_free(0, d); return -1; }
  out->host_ptr = host_ptr;
  out->device_ptr = d;
  out->size_bytes = size_bytes;
  out->mem_type = ESHKOL_MEM_DEVICE;
  out->backend = ESHKOL_GPU_CUDA;
  out->flags = FLAG_WRAPPED | FLAG_COPY_BACK;
  out->backend_data = host_ptr;
  return 0;
}

int eshkol_gpu_sync(EshkolGPUBuffer* b, EshkolSyncDirection direction) {
  if (!b) return -1;
  if (b->backend != ESHKOL_GPU_CUDA) return 0;
  if (b->flags & FLAG_WRAPPED) {
    if (direction == ESHKOL_SYNC_HOST_TO_DEVICE || direction == ESHKOL_SYNC_BIDIRECTIONAL)
      if (eshkol_b200_copy_h2d(b->device_ptr, b->backend_data, b->size_bytes)) return -1;
    if (direction == ESHKOL_SYNC_DEVICE_TO_HOST || direction == ESHKOL_SYNC_BIDIRECTIONAL)
      return copy_back(b);
  }
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}

int eshkol_gpu_sync_async(EshkolGPUBuffer* b, EshkolSyncDirection direction, void* stream) {
  (void)stream; /* one stream, as in the reference (gpu_memory_cuda.cpp:1012-1015) */
  return eshkol_gpu_sync(b, direction);
}

void eshkol_gpu_wait(EshkolGPUBuffer* b) {
  (void)b;
  if (g_backend == ESHKOL_GPU_CUDA) (void)eshkol_b200_sync_status();
}

/* ------------------------------------------------------- tier selection ---- */
typedef struct { int tier, param; const char* why; } TierChoice;

/* guaranteed relative error of Ozaki-I at T = 1..8 (gpu_memory_cuda.cpp:485-487) */
static const double OZAKI_TOL[9] = {1.0, 1e-3, 1e-5, 1e-7, 1e-9, 1e-11, 1e-13, 1e-14, 1e-14};

static int env_int_clamped(const char* name, int lo, int hi, int dflt, int clamp_to_edge) {
  const char* e = getenv(name);
  if (!e) return dflt;
  const int v = atoi(e);
  if (v >= lo && v <= hi) return v;
  const int used = clamp_to_edge ? (v < lo ? lo : hi) : dflt;
  fprintf(stderr, "[GPU] %s=%d out of range [%d,%d]; using %d\n", name, v, lo, hi, used);
  return used;
}

/* Self-calibrated time model per kernel, t_ns = overhead_ns + work / peak_gflops with
 * work = 2*M*K*N (gpu_memory_cuda.cpp:499-522).  Index 0 is the full-precision kernel -- the
 * reference's cublasDgemm, here the Ozaki-II exact tier -- and 1..8 are the slice tiers.  The
 * seeds are this library's own rates on a B200 at 8192^3 under sustained load (f64-equivalent
 * GFLOP/s) and the fixed cost of its launches on a small shape; peak_gflops then follows the
 * best rate each kernel has actually shown (cuda_gemm_calibrate, :515-522). */
typedef struct { double overhead_ns, peak_gflops; } GemmModel;
static GemmModel g_gemm_model[9] = {
    /* exact  */ {90000.0, 123000.0},
    /* T = 1  */ {60000.0, 510000.0},
    /* T = 2  */ {60000.0, 328000.0},
    /* T = 3  */ {65000.0, 224000.0},
    /* T = 4  */ {65000.0, 156000.0},
    /* T = 5  */ {70000.0, 114000.0},
    /* T = 6  */ {70000.0, 86600.0},
    /* T = 7  */ {75000.0, 66400.0},
    /* T = 8  */ {80000.0, 52000.0}};
/* Ozaki must be predicted this much faster before the full-precision kernel is left
 * (gpu_memory_cuda.cpp:549-552) */
static const double OZAKI_SAFETY = 1.15;

static double gemm_predict_ns(int idx, double work) {
  return g_gemm_model[idx].overhead_ns + work / g_gemm_model[idx].peak_gflops;
}

static void gemm_calibrate(int idx, double work, double measured_ns) {
  if (idx < 0 || idx > 8) return;
  const double compute_ns = measured_ns - g_gemm_model[idx].overhead_ns;
  if (compute_ns <= 0.0) return; /* overhead-dominated: no throughput signal */
  const double achieved = work / compute_ns;
  if (achieved > g_gemm_model[idx].peak_gflops) g_gemm_model[idx].peak_gflops = achieved;
}

/* the crude size guard of the slice tiers (gpu_memory_cuda.cpp:462-464) */
static int ozaki_worthwhile(uint64_t M, uint64_t K, uint64_t N) { return M >= 1024 && N >= 1024 && K >= 1024; }

/* cuda_select_f64 (gpu_memory_cuda.cpp:560-575): the smallest T whose guaranteed error meets
 * the budget, taken only if the model predicts it clearly faster than the full-precision kernel */
static int select_slice_tier(uint64_t M, uint64_t K, uint64_t N, double budget, double* speedup) {
  const double work = 2.0 * (double)M * (double)K * (double)N;
  *speedup = 1.0;
  if (K > 133000 || !ozaki_worthwhile(M, K, N)) return 0;
  int Treq = 0;
  for (int T = 1; T <= 7; ++T)
    if (OZAKI_TOL[T] <= budget) { Treq = T; break; }
  if (!Treq) return 0;
  const double t_full = gemm_predict_ns(0, work), t_oz = gemm_predict_ns(Treq, work);
  if (t_oz * OZAKI_SAFETY < t_full) { *speedup = t_full / t_oz; return Treq; }
  return 0;
}

static TierChoice choose_tier(uint64_t M, uint64_t K, uint64_t N) {
  TierChoice c = {ESHKOL_B200_TIER_OZAKI2, 16, "default: Ozaki-II exact"};
  const char* k;
  if ((k = getenv("ESHKOL_B200_TIER")) != NULL) {
    if (!strncmp(k, "ozaki1", 6)) { c.tier = ESHKOL_B200_TIER_OZAKI1; c.param = k[6] == ':' ? atoi(k + 7) : 6; c.why = "ESHKOL_B200_TIER"; return c; }
    if (!strncmp(k, "fast", 4)) { c.tier = ESHKOL_B200_TIER_OZAKI2_FAST; c.param = k[4] == ':' ? atoi(k + 5) : 11; c.why = "ESHKOL_B200_TIER"; return c; }
    if (!strncmp(k, "exact", 5)) { c.param = k[5] == ':' ? atoi(k + 6) : 16; c.why = "ESHKOL_B200_TIER"; return c; }
    if (!strcmp(k, "dgemm")) { c.tier = ESHKOL_B200_TIER_DGEMM; c.param = 0; c.why = "ESHKOL_B200_TIER"; return c; }
    fprintf(stderr, "[GPU] ESHKOL_B200_TIER=%s not understood; ignoring\n", k);
  }
  /* CUDA backend's explicit switch: fixed T when every dimension is >= 1024 */
  if ((k = getenv("ESHKOL_CUDA_F64_KERNEL")) != NULL && !strcmp(k, "ozaki-int8")) {
    const int T = env_int_clamped("ESHKOL_OZAKI_CUDA_T", 1, 8, 6, 0);
    if (ozaki_worthwhile(M, K, N)) {
      c.tier = ESHKOL_B200_TIER_OZAKI1; c.param = T; c.why = "ESHKOL_CUDA_F64_KERNEL override";
      return c;
    }
  }
  /* CUDA backend's accuracy budget: the cheapest kernel that meets it.  "exact" / "full" and any
   * budget no slice tier guarantees stay on the full-precision kernel, which here is the
   * Ozaki-II exact tier */
  if ((k = getenv("ESHKOL_MATMUL_ACCURACY")) != NULL && *k) {
    double budget, speedup;
    if (!strcmp(k, "fast")) budget = 1e-2;
    else if (!strcmp(k, "exact") || !strcmp(k, "full")) budget = 1e-15;
    else { budget = atof(k); if (!(budget > 0.0)) budget = 1e-15; }
    const int T = select_slice_tier(M, K, N, budget, &speedup);
    if (T) { c.tier = ESHKOL_B200_TIER_OZAKI1; c.param = T; c.why = "accuracy-budget selector"; return c; }
    c.why = "budget met cheapest by the full-precision kernel: Ozaki-II exact";
    return c;
  }
  /* Metal backend's switches */
  int fast = 0;
  if ((k = getenv("ESHKOL_OZAKI_FAST")) != NULL && strcmp(k, "0") != 0) fast = 1;
  if ((k = getenv("ESHKOL_SF64_KERNEL")) != NULL && !strcmp(k, "ozaki-fast")) fast = 1;
  if (fast) {
    c.tier = ESHKOL_B200_TIER_OZAKI2_FAST;
    c.param = env_int_clamped("ESHKOL_OZAKI_FAST_MODULI", 2, 16, 11, 1);
    c.why = "Ozaki-II fast tier";
    return c;
  }
  c.param = env_int_clamped("ESHKOL_OZAKI_NUM_MODULI", 2, 16, 16, 0);
  return c;
}

/* model slot of a choice: 0 the full-precision kernel, T for a slice tier, -1 for the others */
static int model_index(const TierChoice* c) {
  if (c->tier == ESHKOL_B200_TIER_OZAKI2 && c->param == 16) return 0;
  if (c->tier == ESHKOL_B200_TIER_OZAKI1 && c->param >= 1 && c->param <= 8) return c->param;
  return -1;
}

/* tests: the tier the environment selects for a shape, without touching a GPU */
void eshkol_b200_debug_choose_tier(uint64_t M, uint64_t K, uint64_t N, int* tier, int* param) {
  const TierChoice c = choose_tier(M, K, N);
  if (tier) *tier = c.tier;
  if (param) *param = c.param;
}

/* tests: read one slot of the time model, or feed it one measurement */
void eshkol_b200_debug_gemm_model(int idx, double* overhead_ns, double* peak_gflops) {
  if (idx < 0 || idx > 8) return;
  if (overhead_ns) *overhead_ns = g_gemm_model[idx].overhead_ns;
  if (peak_gflops) *peak_gflops = g_gemm_model[idx].peak_gflops;
}
void eshkol_b200_debug_gemm_calibrate(int idx, double work, double measured_ns) {
  gemm_calibrate(idx, work, measured_ns);
}

int eshkol_gpu_matmul_f64(EshkolGPUBuffer* A, EshkolGPUBuffer* B, EshkolGPUBuffer* C,
                          uint64_t M, uint64_t K, uint64_t N) {
  if (!A || !B || !C) return -1;
  if (g_backend != ESHKOL_GPU_CUDA) {
    fprintf(stderr, "[GPU] eshkol_gpu_matmul_f64: no B200 backend is active\n");
    return -1;
  }
  if (!A->device_ptr || !B->device_ptr || !C->device_ptr) return -1;
  if (M == 0 || K == 0 || N == 0 || A->size_bytes / 8 / K < M || B->size_bytes / 8 / N < K ||
      C->size_bytes / 8 / N < M) {
    fprintf(stderr, "[GPU] eshkol_gpu_matmul_f64: a buffer is smaller than its %llux%llux%llu operand\n",
            (unsigned long long)M, (unsigned long long)K, (unsigned long long)N);
    return -1;
  }
  TierChoice c = choose_tier(M, K, N);
  if (c.tier != ESHKOL_B200_TIER_DGEMM && !(c.tier == ESHKOL_B200_TIER_OZAKI2 && c.param == 16) && K > 131071) {
    c.tier = ESHKOL_B200_TIER_OZAKI2; c.param = 16; c.why = "K beyond the reduced tiers' int32-exact bound: Ozaki-II exact";
  }
  GPU_LOG("matmul %llux%llu @ %llux%llu -> tier %d param %d (%s)", (unsigned long long)M,
          (unsigned long long)K, (unsigned long long)K, (unsigned long long)N, c.tier, c.param, c.why);
  EshkolB200GemmOpts o;
  memset(&o, 0, sizeof(o));
  o.tier = c.tier;
  o.param = c.param;
  if (eshkol_b200_gemm_f64_device((const double*)A->device_ptr, (const double*)B->device_ptr,
                                  (double*)C->device_ptr, M, K, N, &o))
    return -1;
  if (C->flags & FLAG_WRAPPED) C->flags |= FLAG_DIRTY;
  /* every operator returns only after the device finished (gpu_memory_cuda.cpp:611, 642) */
  if (eshkol_b200_sync_status() != 0) return -1;
  /* every real GEMM calibrates the model of the kernel that ran (:611-614), here from the
   * device time between two events on the library stream */
  const double ms = eshkol_b200_last_gemm_ms();
  if (ms > 0.0) gemm_calibrate(model_index(&c), 2.0 * (double)M * (double)K * (double)N, ms * 1e6);
  return 0;
}

int eshkol_gpu_matmul_f32(EshkolGPUBuffer* A, EshkolGPUBuffer* B, EshkolGPUBuffer* C,
                          uint64_t M, uint64_t K, uint64_t N) {
  /* gpu_memory_cuda.cpp:653-669 (cublasSgemm on f32 buffers) */
  if (!A || !B || !C) return -1;
  if (g_backend != ESHKOL_GPU_CUDA) {
    fprintf(stderr, "[GPU] eshkol_gpu_matmul_f32: no B200 backend is active\n");
    return -1;
  }
  if (!A->device_ptr || !B->device_ptr || !C->device_ptr) return -1;
  if (A->size_bytes < M * K * 4 || B->size_bytes < K * N * 4 || C->size_bytes < M * N * 4) return -1;
  if (eshkol_b200_gemm_f32_device((const float*)A->device_ptr, (const float*)B->device_ptr,
                                  (float*)C->device_ptr, M, K, N))
    return -1;
  if (C->flags & FLAG_WRAPPED) C->flags |= FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}

/* f16 / bf16-tagged operands (dtype 2 / 3, f64 storage): the tensor-core half-precision product,
 * whatever the size (gpu_memory_cuda.cpp:1122-1131, :1170-1175).  0 on success. */
static int gpu_matmul_f16_host(const double* a, const double* b, double* c, uint64_t batch, uint64_t M,
                               uint64_t K, uint64_t N) {
  const size_t ab = (size_t)(batch * M * K) * 8, bb = (size_t)(batch * K * N) * 8, cb = (size_t)(batch * M * N) * 8;
  void *da = NULL, *db = NULL, *dc = NULL;
  int rc = -1;
  if (eshkol_b200_mem_alloc(0, ab, &da) == 0 && eshkol_b200_mem_alloc(0, bb, &db) == 0 &&
      eshkol_b200_mem_alloc(0, cb, &dc) == 0 && eshkol_b200_copy_h2d(da, a, ab) == 0 &&
      eshkol_b200_copy_h2d(db, b, bb) == 0 &&
      eshkol_b200_gemm_f16_device((const double*)da, (const double*)db, (double*)dc, batch, M, K, N) == 0 &&
      eshkol_b200_copy_d2h(c, dc, cb) == 0 && eshkol_b200_sync_status() == 0)
    rc = 0;
  if (da) eshkol_b200_mem_free(0, da);
  if (db) eshkol_b200_mem_free(0, db);
  if (dc) eshkol_b200_mem_free(0, dc);
  return rc;
}

void eshkol_gpu_set_threshold(size_t threshold) { g_gpu_threshold = threshold; }
size_t eshkol_gpu_get_threshold(void) { return g_gpu_threshold; }
int eshkol_gpu_should_use(size_t n) { return g_backend != ESHKOL_GPU_NONE && n >= g_gpu_threshold; }

/* ----------------------------------------------------------- elementwise ---- */
int eshkol_gpu_elementwise_f64(EshkolGPUBuffer* a, EshkolGPUBuffer* b, EshkolGPUBuffer* out,
                               uint64_t n, EshkolElementwiseOp op) {
  if (!a || !out || n == 0) return -1;
  if (g_backend != ESHKOL_GPU_CUDA || !a->device_ptr || !out->device_ptr) return -1;
  if (a->size_bytes / 8 < n || out->size_bytes / 8 < n || (b && b->device_ptr && b->size_bytes / 8 < n)) {
    fprintf(stderr, "[GPU] eshkol_gpu_elementwise_f64: a buffer holds fewer than %llu doubles\n", (unsigned long long)n);
    return -1;
  }
  const double* bp = (b && b->device_ptr) ? (const double*)b->device_ptr : NULL;
  if (eshkol_b200_elementwise_f64_device((const double*)a->device_ptr, bp, (double*)out->device_ptr,
                                         n, (int)op))
    return -1;
  if (out->flags & FLAG_WRAPPED) out->flags |= FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}

/* ------------------------------------------------ the other operators ---- */
/* Device buffers only, like the reference's CUDA branch (gpu_memory_cuda.cpp:1229-1560); where
 * the reference then falls back to a CPU loop on host_ptr, these return -1 and the caller's own
 * CPU path runs (vm_gpu_dispatch.h treats any non-zero result that way). */
static int on_device(const EshkolGPUBuffer* b, uint64_t doubles, const char* who) {
  if (!b || !b->device_ptr || g_backend != ESHKOL_GPU_CUDA) return 0;
  if (b->size_bytes / 8 < doubles) {
    fprintf(stderr, "[GPU] %s: a buffer holds fewer than %llu doubles\n", who, (unsigned long long)doubles);
    return 0;
  }
  return 1;
}
static int operator_done(EshkolGPUBuffer* out) {
  if (out->flags & FLAG_WRAPPED) out->flags |= FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}

int eshkol_gpu_reduce_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t n, EshkolReduceOp op) {
  if (!in || !out || n == 0) return -1;
  if (!on_device(in, n, "eshkol_gpu_reduce_f64") || !on_device(out, 1, "eshkol_gpu_reduce_f64")) return -1;
  if (eshkol_b200_reduce_f64_device((const double*)in->device_ptr, (double*)out->device_ptr, n, (int)op)) return -1;
  return operator_done(out);
}
int eshkol_gpu_reduce_axis_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t rank,
                               const uint64_t* shape, uint64_t axis, EshkolReduceOp op) {
  if (!in || !out || !shape || rank == 0 || axis >= rank) return -1;
  uint64_t outer = 1, inner = 1;
  for (uint64_t i = 0; i < axis; ++i) outer *= shape[i];
  for (uint64_t i = axis + 1; i < rank; ++i) inner *= shape[i];
  const uint64_t len = shape[axis];
  if (outer == 0 || inner == 0 || len == 0) return -1;
  if (!on_device(in, outer * len * inner, "eshkol_gpu_reduce_axis_f64") ||
      !on_device(out, outer * inner, "eshkol_gpu_reduce_axis_f64"))
    return -1;
  if (eshkol_b200_reduce_axis_f64_device((const double*)in->device_ptr, (double*)out->device_ptr, outer, len,
                                         inner, (int)op))
    return -1;
  return operator_done(out);
}
int eshkol_gpu_transpose_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t rows, uint64_t cols) {
  if (!in || !out || rows == 0 || cols == 0) return -1;
  if (!on_device(in, rows * cols, "eshkol_gpu_transpose_f64") || !on_device(out, rows * cols, "eshkol_gpu_transpose_f64"))
    return -1;
  if (eshkol_b200_transpose_f64_device((const double*)in->device_ptr, (double*)out->device_ptr, rows, cols)) return -1;
  return operator_done(out);
}
int eshkol_gpu_softmax_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t num_slices,
                           uint64_t slice_len) {
  if (!in || !out || num_slices == 0 || slice_len == 0) return -1;
  if (!on_device(in, num_slices * slice_len, "eshkol_gpu_softmax_f64") ||
      !on_device(out, num_slices * slice_len, "eshkol_gpu_softmax_f64"))
    return -1;
  if (eshkol_b200_softmax_f64_device((const double*)in->device_ptr, (double*)out->device_ptr, num_slices, slice_len))
    return -1;
  return operator_done(out);
}
int eshkol_gpu_normalize_f64(EshkolGPUBuffer* in, EshkolGPUBuffer* out, uint64_t num_slices,
                             uint64_t slice_len, double gamma, double beta, double epsilon) {
  if (!in || !out || num_slices == 0 || slice_len == 0) return -1;
  if (!on_device(in, num_slices * slice_len, "eshkol_gpu_normalize_f64") ||
      !on_device(out, num_slices * slice_len, "eshkol_gpu_normalize_f64"))
    return -1;
  if (eshkol_b200_normalize_f64_device((const double*)in->device_ptr, (double*)out->device_ptr, num_slices,
                                       slice_len, gamma, beta, epsilon))
    return -1;
  return operator_done(out);
}
/* tier of one GEMM of a conv2d gradient: what the forward product of that shape would get */
static void conv_grad_opts(uint64_t M, uint64_t K, uint64_t N, EshkolB200GemmOpts* o) {
  TierChoice c = choose_tier(M, K, N);
  if (c.tier != ESHKOL_B200_TIER_DGEMM && !(c.tier == ESHKOL_B200_TIER_OZAKI2 && c.param == 16) && K > 131071) {
    c.tier = ESHKOL_B200_TIER_OZAKI2; c.param = 16;
  }
  memset(o, 0, sizeof(*o));
  o->tier = c.tier; o->param = c.param;
}

int eshkol_gpu_conv2d_backward_input_f64(EshkolGPUBuffer* grad_out, EshkolGPUBuffer* kernel_weights,
    EshkolGPUBuffer* grad_input, uint64_t in_h, uint64_t in_w, uint64_t k_h, uint64_t k_w, uint64_t out_h,
    uint64_t out_w, uint64_t stride_h, uint64_t stride_w, uint64_t channels_in, uint64_t channels_out,
    uint64_t batch_size) {
  /* gpu_memory.h:404; kernel lib/backend/gpu/gpu_cuda_kernels.cu:413-449 */
  if (!grad_out || !kernel_weights || !grad_input || g_backend != ESHKOL_GPU_CUDA) return -1;
  if (!grad_out->device_ptr || !kernel_weights->device_ptr || !grad_input->device_ptr) return -1;
  if (grad_out->size_bytes / 8 < batch_size * channels_out * out_h * out_w ||
      kernel_weights->size_bytes / 8 < channels_out * channels_in * k_h * k_w ||
      grad_input->size_bytes / 8 < batch_size * channels_in * in_h * in_w) {
    fprintf(stderr, "[GPU] eshkol_gpu_conv2d_backward_input_f64: a buffer is smaller than its tensor\n");
    return -1;
  }
  EshkolB200GemmOpts o;
  conv_grad_opts(channels_in * k_h * k_w, channels_out, batch_size * out_h * out_w, &o);
  if (eshkol_b200_conv2d_backward_input_f64_device((const double*)grad_out->device_ptr,
          (const double*)kernel_weights->device_ptr, (double*)grad_input->device_ptr, in_h, in_w, k_h, k_w,
          out_h, out_w, stride_h, stride_w, channels_in, channels_out, batch_size, &o))
    return -1;
  if (grad_input->flags & FLAG_WRAPPED) grad_input->flags |= FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}
int eshkol_gpu_conv2d_backward_kernel_f64(EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input,
    EshkolGPUBuffer* grad_kernel, uint64_t in_h, uint64_t in_w, uint64_t k_h, uint64_t k_w, uint64_t out_h,
    uint64_t out_w, uint64_t stride_h, uint64_t stride_w, uint64_t channels_in, uint64_t channels_out,
    uint64_t batch_size) {
  /* gpu_memory.h:415; kernel lib/backend/gpu/gpu_cuda_kernels.cu:451-486 */
  if (!grad_out || !saved_input || !grad_kernel || g_backend != ESHKOL_GPU_CUDA) return -1;
  if (!grad_out->device_ptr || !saved_input->device_ptr || !grad_kernel->device_ptr) return -1;
  if (grad_out->size_bytes / 8 < batch_size * channels_out * out_h * out_w ||
      saved_input->size_bytes / 8 < batch_size * channels_in * in_h * in_w ||
      grad_kernel->size_bytes / 8 < channels_out * channels_in * k_h * k_w) {
    fprintf(stderr, "[GPU] eshkol_gpu_conv2d_backward_kernel_f64: a buffer is smaller than its tensor\n");
    return -1;
  }
  EshkolB200GemmOpts o;
  conv_grad_opts(channels_out, batch_size * out_h * out_w, channels_in * k_h * k_w, &o);
  if (eshkol_b200_conv2d_backward_kernel_f64_device((const double*)grad_out->device_ptr,
          (const double*)saved_input->device_ptr, (double*)grad_kernel->device_ptr, in_h, in_w, k_h, k_w,
          out_h, out_w, stride_h, stride_w, channels_in, channels_out, batch_size, &o))
    return -1;
  if (grad_kernel->flags & FLAG_WRAPPED) grad_kernel->flags |= FLAG_DIRTY;
  return eshkol_b200_sync_status() == 0 ? 0 : -1;
}
int eshkol_gpu_batchnorm_backward_f64(EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input,
    EshkolGPUBuffer* saved_mean, EshkolGPUBuffer* saved_inv_std, EshkolGPUBuffer* saved_gamma,
    EshkolGPUBuffer* grad_input, EshkolGPUBuffer* grad_gamma, EshkolGPUBuffer* grad_beta,
    uint64_t batch_size, uint64_t feature_size) {
  /* gpu_memory.h:426; kernel lib/backend/gpu/gpu_cuda_kernels.cu:489-521 */
  static const char* who = "eshkol_gpu_batchnorm_backward_f64";
  if (!grad_out || !saved_input || !saved_mean || !saved_inv_std || !saved_gamma || !grad_input || !grad_gamma ||
      !grad_beta || batch_size == 0 || feature_size == 0)
    return -1;
  const uint64_t all = batch_size * feature_size;
  if (!on_device(grad_out, all, who) || !on_device(saved_input, all, who) || !on_device(saved_mean, feature_size, who) ||
      !on_device(saved_inv_std, feature_size, who) || !on_device(saved_gamma, feature_size, who) ||
      !on_device(grad_input, all, who) || !on_device(grad_gamma, feature_size, who) ||
      !on_device(grad_beta, feature_size, who))
    return -1;
  if (eshkol_b200_batchnorm_backward_f64_device((const double*)grad_out->device_ptr,
          (const double*)saved_input->device_ptr, (const double*)saved_mean->device_ptr,
          (const double*)saved_inv_std->device_ptr, (const double*)saved_gamma->device_ptr,
          (double*)grad_input->device_ptr, (double*)grad_gamma->device_ptr, (double*)grad_beta->device_ptr,
          batch_size, feature_size))
    return -1;
  if (grad_gamma->flags & FLAG_WRAPPED) grad_gamma->flags |= FLAG_DIRTY;
  if (grad_beta->flags & FLAG_WRAPPED) grad_beta->flags |= FLAG_DIRTY;
  return operator_done(grad_input);
}
int eshkol_gpu_layernorm_backward_f64(EshkolGPUBuffer* grad_out, EshkolGPUBuffer* saved_input,
    EshkolGPUBuffer* saved_mean, EshkolGPUBuffer* saved_inv_std, EshkolGPUBuffer* saved_gamma,
    EshkolGPUBuffer* grad_input, uint64_t num_samples, uint64_t feature_size) {
  /* gpu_memory.h:437; kernel lib/backend/gpu/gpu_cuda_kernels.cu:524-555 */
  static const char* who = "eshkol_gpu_layernorm_backward_f64";
  if (!grad_out || !saved_input || !saved_mean || !saved_inv_std || !saved_gamma || !grad_input ||
      num_samples == 0 || feature_size == 0)
    return -1;
  const uint64_t all = num_samples * feature_size;
  if (!on_device(grad_out, all, who) || !on_device(saved_input, all, who) || !on_device(saved_mean, num_samples, who) ||
      !on_device(saved_inv_std, num_samples, who) || !on_device(saved_gamma, feature_size, who) ||
      !on_device(grad_input, all, who))
    return -1;
  if (eshkol_b200_layernorm_backward_f64_device((const double*)grad_out->device_ptr,
          (const double*)saved_input->device_ptr, (const double*)saved_mean->device_ptr,
          (const double*)saved_inv_std->device_ptr, (const double*)saved_gamma->device_ptr,
          (double*)grad_input->device_ptr, num_samples, feature_size))
    return -1;
  return operator_done(grad_input);
}

/* ------------------------------------------------- residency of operands ---- */
typedef struct {
  const char* host;      /* NULL: free slot */
  size_t bytes;
  void* dev;
  uint64_t finger;       /* sampled contents of the host range when the copy was made */
  uint64_t last_use;
  uint64_t prep_token;   /* token of the prepared right-hand operand made from this copy, or 0 */
  int pinned;            /* in use by the call in progress: not evictable */
  int stale;             /* the host range was written since: the buffer is kept, its contents are not */
} ResEntry;
enum { RES_SLOTS = 64 };
static ResEntry g_res[RES_SLOTS];
static size_t g_res_bytes = 0, g_res_limit = 0;
static uint64_t g_res_clock = 0;
static int g_res_on = -1; /* -1: read the environment on first use */

static int res_enabled(void) {
  if (g_res_on < 0) {
    const char* e = getenv("ESHKOL_B200_RESIDENCY");
    g_res_on = (e && e[0] == '1') ? 1 : 0;
    const char* m = getenv("ESHKOL_B200_RESIDENCY_MB");
    const long mb = m ? atol(m) : 0;
    g_res_limit = (size_t)(mb > 0 ? mb : 65536) << 20;
  }
  return g_res_on;
}

/* 256 evenly spaced 8-byte words of the range and its length, FNV-1a */
static uint64_t res_fingerprint(const void* p, size_t bytes) {
  const uint64_t* w = (const uint64_t*)p;
  const size_t n = bytes / 8;
  uint64_t h = 1469598103934665603ull ^ (uint64_t)bytes;
  const size_t samples = n < 256 ? n : 256;
  for (size_t i = 0; i < samples; ++i) {
    uint64_t v;
    memcpy(&v, w + (samples > 1 ? i * (n - 1) / (samples - 1) : 0), 8);
    h = (h ^ v) * 1099511628211ull;
  }
  return h;
}

static void res_drop(ResEntry* e) {
  if (!e->host) return;
  if (e->dev) eshkol_b200_mem_free(0, e->dev);
  g_res_bytes -= e->bytes;
  memset(e, 0, sizeof(*e));
}

/* every cached range that overlaps [host, host + bytes): the one that is exactly this range keeps
 * its device buffer and is only marked stale (a host that rewrites a tensor in place, or a result
 * written to the same place call after call, would otherwise free and allocate the same buffer
 * every time, and cudaFree synchronises the device); the others are dropped */
static void res_invalidate_overlapping(const void* host, size_t bytes) {
  const char* lo = (const char*)host;
  const char* hi = lo + (bytes ? bytes : 1);
  for (int i = 0; i < RES_SLOTS; ++i) {
    ResEntry* e = &g_res[i];
    if (!e->host || !(e->host < hi && lo < e->host + e->bytes)) continue;
    if (e->host == lo && (bytes == 0 || e->bytes == bytes)) { e->stale = 1; e->finger = 0; e->prep_token = 0; }
    else res_drop(e);
  }
}

/* the cached copy of exactly this range, if its sampled contents are still what was uploaded */
static ResEntry* res_find(const void* host, size_t bytes) {
  for (int i = 0; i < RES_SLOTS; ++i) {
    ResEntry* e = &g_res[i];
    if (e->host == (const char*)host && e->bytes == bytes) {
      if (e->stale) return NULL;
      if (e->finger != res_fingerprint(host, bytes)) {
        GPU_LOG("residency: host range %p changed since it was uploaded; its device copy is stale", host);
        e->stale = 1; e->finger = 0; e->prep_token = 0;
        return NULL;
      }
      e->last_use = ++g_res_clock;
      return e;
    }
  }
  return NULL;
}

/* a new entry with a device buffer of `bytes`; evicts least recently used copies to stay under
 * the limit; NULL when there is no room (every candidate pinned, or the allocation fails) */
static ResEntry* res_insert(const void* host, size_t bytes) {
  res_invalidate_overlapping(host, bytes);
  for (int i = 0; i < RES_SLOTS; ++i) {
    ResEntry* e = &g_res[i];
    if (e->host == (const char*)host && e->bytes == bytes) {  /* the stale entry of this very range: reuse its buffer */
      e->stale = 0; e->finger = 0; e->prep_token = 0; e->pinned = 1;
      e->last_use = ++g_res_clock;
      return e;
    }
  }
  for (;;) {
    ResEntry* slot = NULL;
    ResEntry* lru = NULL;
    for (int i = 0; i < RES_SLOTS; ++i) {
      ResEntry* e = &g_res[i];
      if (!e->host) { if (!slot) slot = e; continue; }
      if (!e->pinned && (!lru || e->last_use < lru->last_use)) lru = e;
    }
    if (slot && g_res_bytes + bytes <= g_res_limit) {
      void* d = NULL;
      if (eshkol_b200_mem_alloc(0, bytes, &d) == 0) {
        slot->host = (const char*)host; slot->bytes = bytes; slot->dev = d;
        slot->finger = 0; slot->prep_token = 0; slot->pinned = 1; slot->stale = 0;
        slot->last_use = ++g_res_clock;
        g_res_bytes += bytes;
        return slot;
      }
    }
    if (!lru) return NULL;
    res_drop(lru);
  }
}

void eshkol_gpu_set_residency(int on, size_t limit_mb) {
  (void)res_enabled();
  g_res_on = on ? 1 : 0;
  if (limit_mb) g_res_limit = limit_mb << 20;
  if (!on) eshkol_gpu_residency_clear();
}

void eshkol_gpu_invalidate(const void* host_ptr, size_t bytes) {
  if (host_ptr) res_invalidate_overlapping(host_ptr, bytes);
}

void eshkol_gpu_residency_clear(void) {
  for (int i = 0; i < RES_SLOTS; ++i) res_drop(&g_res[i]);
}

/* exact-tier product with cached device copies; 0 done, -1 failed, -2 not served this way */
static int matmul_resident(const double* A, const double* B, double* C, uint64_t M, uint64_t K, uint64_t N) {
  const size_t ab = (size_t)(M * K) * 8, bb = (size_t)(K * N) * 8, cb = (size_t)(M * N) * 8;
  const char *a0 = (const char*)A, *b0 = (const char*)B, *c0 = (const char*)C;
  /* a result that overlaps an operand is not a case the reference's callers produce */
  if ((c0 < a0 + ab && a0 < c0 + cb) || (c0 < b0 + bb && b0 < c0 + cb)) return -2;
  for (int i = 0; i < RES_SLOTS; ++i) g_res[i].pinned = 0;
  ResEntry* ea = res_find(A, ab);
  int a_state = ea ? 1 : 0;
  if (ea) ea->pinned = 1; else ea = res_insert(A, ab);
  if (!ea) return -2;
  ResEntry* eb = ((const void*)A == (const void*)B && ab == bb) ? ea : res_find(B, bb);
  int b_state = 0;
  if (eb == ea) b_state = a_state;  /* A * A: one copy serves both; uploaded (if at all) as the right-hand operand */
  else if (eb) b_state = 1;
  if (eb) eb->pinned = 1; else eb = res_insert(B, bb);
  if (!eb) { if (!a_state) res_drop(ea); return -2; }
  if (eb == ea && !a_state) a_state = 1;  /* the upload of B fills the shared copy before any block of A is read */
  if (b_state == 1 && eb->prep_token && eb->prep_token == eshkol_b200_prepared_b_token()) b_state = 2;
  ResEntry* ec = res_insert(C, cb);
  if (!ec) {
    if (!ea->finger) res_drop(ea);
    if (eb != ea && !eb->finger) res_drop(eb);
    return -2;
  }
  uint64_t token = 0;
  GPU_LOG("matmul %llux%llu @ %llux%llu -> Ozaki-II exact, resident operands (A %s, B %s)", (unsigned long long)M,
          (unsigned long long)K, (unsigned long long)K, (unsigned long long)N, a_state ? "on device" : "uploaded",
          b_state == 2 ? "prepared" : (b_state == 1 ? "on device" : "uploaded"));
  int rc = eshkol_b200_matmul_f64_host_resident(A, B, C, M, K, N, (double*)ea->dev, a_state, (double*)eb->dev,
                                                b_state, (double*)ec->dev, &token);
  if (rc == 0 && eshkol_b200_sync_status() != 0) rc = -1;
  if (rc != 0) {
    res_drop(ec);
    if (!ea->finger) res_drop(ea);
    if (eb != ea && !eb->finger) res_drop(eb);
    return -1;
  }
  if (!ea->finger) ea->finger = res_fingerprint(A, ab);
  if (!eb->finger) eb->finger = res_fingerprint(B, bb);
  ec->finger = res_fingerprint(C, cb);
  /* only one right-hand operand is prepared at a time */
  for (int i = 0; i < RES_SLOTS; ++i) g_res[i].prep_token = 0;
  eb->prep_token = token;
  for (int i = 0; i < RES_SLOTS; ++i) g_res[i].pinned = 0;
  return 0;
}

/* ------------------------------------------------------------ dispatchers ---- */
static void fill_nan(double* c, uint64_t n) {
  for (uint64_t i = 0; i < n; ++i) c[i] = NAN;
}

/* one GEMM on host arrays through the buffer API; 0 on success */
static int gpu_matmul_host(const double* A, const double* B, double* C, uint64_t M, uint64_t K,
                           uint64_t N) {
  EshkolGPUBuffer a, b, c;
  memset(&a, 0, sizeof(a)); memset(&b, 0, sizeof(b)); memset(&c, 0, sizeof(c));
  int rc = -1;
  /* C is output only: give it device memory without the upload a wrap would do */
  void* dc = NULL;
  if (eshkol_gpu_wrap_host((void*)A, M * K * sizeof(double), &a) == 0 &&
      eshkol_gpu_wrap_host((void*)B, K * N * sizeof(double), &b) == 0 &&
      eshkol_b200_mem_alloc(0, M * N * sizeof(double), &dc) == 0) {
    c.host_ptr = C; c.device_ptr = dc; c.size_bytes = M * N * sizeof(double);
    c.mem_type = ESHKOL_MEM_DEVICE; c.backend = ESHKOL_GPU_CUDA;
    c.flags = FLAG_WRAPPED | FLAG_COPY_BACK; c.backend_data = C;
    if (eshkol_gpu_matmul_f64(&a, &b, &c, M, K, N) == 0 &&
        eshkol_gpu_sync(&c, ESHKOL_SYNC_DEVICE_TO_HOST) == 0)
      rc = 0;
  }
  a.flags &= ~FLAG_COPY_BACK; b.flags &= ~FLAG_COPY_BACK;
  if (a.device_ptr) eshkol_gpu_free(&a);
  if (b.device_ptr) eshkol_gpu_free(&b);
  if (c.device_ptr) eshkol_gpu_free(&c);
  else if (dc) eshkol_b200_mem_free(0, dc);
  return rc;
}

void eshkol_matmul_dispatch(const double* A, const double* B, double* C, uint64_t M, uint64_t K,
                            uint64_t N, int32_t dtype) {
  if (!A || !B || !C || M == 0 || K == 0 || N == 0) return;
  if (g_backend == ESHKOL_GPU_NONE) eshkol_gpu_init(); /* gpu_memory_cuda.cpp:1117-1119 */
  if ((dtype == 2 || dtype == 3) && g_backend == ESHKOL_GPU_CUDA) {
    /* the half-precision fast path bypasses the element threshold (gpu_memory_cuda.cpp:1122-1131);
     * if it fails the f64 path below still produces C, as in the reference */
    GPU_LOG("matmul %llux%llu @ %llux%llu -> f16 tensor-core path (dtype %d)", (unsigned long long)M,
            (unsigned long long)K, (unsigned long long)K, (unsigned long long)N, (int)dtype);
    if (gpu_matmul_f16_host(A, B, C, 1, M, K, N) == 0) return;
    fprintf(stderr, "[GPU] eshkol_matmul_dispatch: the f16 path failed; continuing in f64\n");
  }
  const size_t n_out = (size_t)(M * N);
  if (!eshkol_gpu_should_use(n_out) && eshkol_matmul_f64) {
    eshkol_matmul_f64(A, B, C, M, K, N); /* small shapes stay on the CPU: policy, not a fallback */
    return;
  }
  if (g_backend == ESHKOL_GPU_CUDA) {
    /* exact tier: upload, products and download pipelined over row blocks of A */
    const TierChoice c = choose_tier(M, K, N);
    int rc = -2;
    if (c.tier == ESHKOL_B200_TIER_OZAKI2 && c.param == 16 && K <= 262144) {
      EshkolB200GemmOpts o;
      memset(&o, 0, sizeof(o));
      o.tier = c.tier; o.param = c.param;
      if (res_enabled()) {
        rc = matmul_resident(A, B, C, M, K, N);
        if (rc == 0) return;
      }
      if (rc == -2) {
        GPU_LOG("matmul %llux%llu @ %llux%llu -> Ozaki-II exact, host pipeline (%s)", (unsigned long long)M,
                (unsigned long long)K, (unsigned long long)K, (unsigned long long)N, c.why);
        rc = eshkol_b200_matmul_f64_host(A, B, C, M, K, N, &o);
      }
      if (rc == 0 && eshkol_b200_sync_status() != 0) rc = -1;
      if (rc == 0) return;
    }
    /* other tiers: the buffer API, as the reference's dispatcher does */
    if (rc == -2 && gpu_matmul_host(A, B, C, M, K, N) == 0) return;
  }
  fprintf(stderr, "[GPU] eshkol_matmul_dispatch: the B200 path FAILED for %llux%llux%llu; "
                  "C is filled with NaN\n", (unsigned long long)M, (unsigned long long)K,
          (unsigned long long)N);
  fill_nan(C, M * N);
}

void eshkol_batch_matmul_dispatch(const double* a, const double* b, double* c, int64_t batch,
                                  int64_t M, int64_t K, int64_t N, int32_t dtype) {
  if (!a || !b || !c || batch <= 0 || M <= 0 || K <= 0 || N <= 0) return;
  if (g_backend == ESHKOL_GPU_NONE) eshkol_gpu_init();
  if ((dtype == 2 || dtype == 3) && g_backend == ESHKOL_GPU_CUDA) {
    /* one launch for the whole batch (gpu_memory_cuda.cpp:1170-1175) */
    if (gpu_matmul_f16_host(a, b, c, (uint64_t)batch, (uint64_t)M, (uint64_t)K, (uint64_t)N) == 0) return;
    fprintf(stderr, "[GPU] eshkol_batch_matmul_dispatch: the f16 path failed; continuing in f64\n");
    dtype = 0;
  }
  if (!eshkol_gpu_should_use((size_t)(M * N)) && eshkol_batch_matmul_f64) {
    eshkol_batch_matmul_f64(a, b, c, batch, M, K, N);
    return;
  }
  for (int64_t i = 0; i < batch; ++i)
    eshkol_matmul_dispatch(a + i * M * K, b + i * K * N, c + i * M * N, (uint64_t)M, (uint64_t)K,
                           (uint64_t)N, dtype);
}

int eshkol_gpu_conv2d_f64(const double* in, int64_t batch, int64_t in_c, int64_t H, int64_t W,
                          const double* ker, int64_t out_c, int64_t kH, int64_t kW,
                          int64_t stride, int64_t pad, double* out, int32_t activation) {
  if (!in || !ker || !out) return -1;
  if (g_backend == ESHKOL_GPU_NONE) eshkol_gpu_init();
  if (g_backend != ESHKOL_GPU_CUDA) return -1;
  if (stride <= 0) stride = 1;
  if (pad < 0) pad = 0;
  const int64_t spanH = H + 2 * pad - kH, spanW = W + 2 * pad - kW;
  if (spanH < 0 || spanW < 0) return 0;
  const int64_t oH = spanH / stride + 1, oW = spanW / stride + 1;
  const size_t in_b = (size_t)(batch * in_c * H * W) * 8, k_b = (size_t)(out_c * in_c * kH * kW) * 8,
               o_b = (size_t)(batch * out_c * oH * oW) * 8;
  void *d_in = NULL, *d_k = NULL, *d_o = NULL;
  int rc = -1;
  if (eshkol_b200_mem_alloc(0, in_b, &d_in) == 0 && eshkol_b200_mem_alloc(0, k_b, &d_k) == 0 &&
      eshkol_b200_mem_alloc(0, o_b, &d_o) == 0 && eshkol_b200_copy_h2d(d_in, in, in_b) == 0 &&
      eshkol_b200_copy_h2d(d_k, ker, k_b) == 0) {
    TierChoice c = choose_tier((uint64_t)out_c, (uint64_t)(in_c * kH * kW), (uint64_t)(batch * oH * oW));
    EshkolB200GemmOpts o;
    memset(&o, 0, sizeof(o));
    o.tier = c.tier; o.param = c.param; o.activation = activation;
    if (eshkol_b200_conv2d_f64_device((const double*)d_in, batch, in_c, H, W, (const double*)d_k,
                                      out_c, kH, kW, stride, pad, (double*)d_o, &o) == 0 &&
        eshkol_b200_copy_d2h(out, d_o, o_b) == 0 && eshkol_b200_sync_status() == 0)
      rc = 0;
  }
  if (d_in) eshkol_b200_mem_free(0, d_in);
  if (d_k) eshkol_b200_mem_free(0, d_k);
  if (d_o) eshkol_b200_mem_free(0, d_o);
  if (rc) fprintf(stderr, "[GPU] eshkol_gpu_conv2d_f64: the B200 path FAILED\n");
  return rc;
}

int eshkol_gpu_matmul_backward_f64(const double* grad_out, const double* A, const double* B,
                                   double* grad_A, double* grad_B, uint64_t M, uint64_t K, uint64_t N) {
  if (!grad_out || !A || !B || !grad_A || !grad_B || M == 0 || K == 0 || N == 0) return -1;
  if (g_backend == ESHKOL_GPU_NONE) eshkol_gpu_init();
  if (g_backend != ESHKOL_GPU_CUDA) return -1;
  const size_t out_a = (size_t)(M * K), out_b = (size_t)(K * N);
  if (!eshkol_gpu_should_use(out_a > out_b ? out_a : out_b)) return -1; /* blas_backend.cpp:957-958 */
  /* each gradient is a product of its own shape and gets the tier that shape would get */
  const TierChoice ca = choose_tier(M, N, K), cb = choose_tier(K, M, N);
  EshkolB200GemmOpts oa, ob;
  memset(&oa, 0, sizeof(oa));
  memset(&ob, 0, sizeof(ob));
  oa.tier = ca.tier; oa.param = ca.param;
  ob.tier = cb.tier; ob.param = cb.param;
  GPU_LOG("matmul backward M=%llu K=%llu N=%llu -> grad_A tier %d:%d, grad_B tier %d:%d (%s)",
          (unsigned long long)M, (unsigned long long)K, (unsigned long long)N, ca.tier, ca.param,
          cb.tier, cb.param, ca.why);
  if (eshkol_b200_matmul_backward_f64_host(grad_out, A, B, grad_A, grad_B, M, K, N, &oa, &ob) != 0 ||
      eshkol_b200_sync_status() != 0) {
    fprintf(stderr, "[GPU] eshkol_gpu_matmul_backward_f64: the B200 path FAILED\n");
    return -1;
  }
  return 0;
}
