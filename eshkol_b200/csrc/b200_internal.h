// Internal (non-exported) declarations shared by the .cu translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kBM = 128;       // output tile rows (UMMA M, one TMEM lane per row)
constexpr int kBK = 128;       // int8 elements per k-block = one 128-byte swizzle row
constexpr int kMaxSeg = 8;     // operand-plane pairs accumulated into one tile
constexpr int kChunkK = 1008;  // modulus-256 extraction interval of the reference
constexpr int kChunkSeg = 1024;   // a chunk inside the modulus-256 plane, padded to whole k-blocks
constexpr int kChunkUnits = 64;   // 16-bit flag units per chunk and row (63 used: 1008 = 63 * 16)

enum GemmEpilogue : int {
  kEpiModI8 = 0,     // centred residue mod an odd modulus -> int8 plane
  kEpiRawI32 = 1,    // raw int32 accumulator -> int32 plane
  kEpiMod256 = 2,    // per-chunk reduction mod 256 with the reference's tie rule -> int16 plane
  kEpiF16 = 3,       // f16 operands, f32 accumulator; rounded to f16 and widened -> f64 matrix
};

// One accumulation: sum over segments of A_plane[seg] * B_plane[seg]^T.
struct GemmJob {
  int n_seg;
  int a_plane[kMaxSeg];
  int b_plane[kMaxSeg];
  int out_plane;
  unsigned modulus;  // kEpiModI8 only
  unsigned magic;    // floor(2^32 / modulus)
  unsigned offset;   // multiple of modulus, >= the largest |accumulator|
};

struct GemmParams {
  int tiles_m, tiles_n, n_jobs;
  int kb_per_seg;    // k-blocks in one segment
  int kb_per_unit;   // k-blocks per accumulator hand-off (whole job unless chunked)
  int group_m;       // m-tiles per raster group
  const GemmJob* jobs;
  uint8_t* out;
  long long out_plane_stride;  // bytes
  int ldo;                     // elements per output row
  int* status;
  int* work_counter;  // zero at launch; hands out work items beyond the first gridDim.x
  // kEpiMod256 only: per row / column and chunk, 64 16-bit units of flags along k
  const uint16_t* a_hi;   // A residue == +128
  const uint16_t* a_odd;  // A residue odd
  const uint16_t* b_odd;  // B residue odd
  const uint16_t* b_hi;   // B residue == +128
  int n_chunks;
  // kEpiMod256: per chunk, row and 32 columns, (tie mask, bit-8 mask) of the byte sums
  uint32_t* tie_bits;
  // kEpiMod256, when tie_list is set: instead of that dense table, only the groups that hold a
  // tie are recorded, appended through tie_cursor as {row, column word | chunk << 17, tie mask,
  // bit-8 mask}; the list has room for every group, so nothing can overflow
  uint4* tie_list;
  unsigned int* tie_cursor;
  // kEpiF16: the output is the caller's matrix, not a padded plane: rows / columns that exist
  int out_rows, out_cols;
  // set by the launchers: how long a bounded wait may last, and (tests only) whether the
  // producer withholds its first arrival so that the waits of this launch run out
  unsigned long long wait_ns;
  int withhold;
};

// Launchers (b200_modgemm.cu).  bn is 128 or 256.
cudaError_t launch_modgemm(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB,
                           const GemmParams& prm, int total_work, int num_sms,
                           cudaStream_t stream);
cudaError_t modgemm_set_attributes();
// After a kEpiMod256 launch: flip_bits[row][word] = which elements' sums need 256 added.
// The CUDA-core checker resolves its ties itself; its flip bits must be cleared instead.
cudaError_t launch_tie_resolve(const GemmParams& prm, uint32_t* flip_bits, int M, int N,
                               cudaStream_t stream);
// whether a result of this geometry can use the tie list (its packed fields have room)
inline bool tie_list_fits(long long Np, int n_chunks) { return Np / 32 < (1LL << 17) && n_chunks < (1 << 15); }

// Two-SM variant (b200_modgemm2.cu): pairs of CTAs on 256 x 256 tiles; tmB_half is tiled in
// boxes of 128 rows.  kEpiModI8 and kEpiRawI32 only.
cudaError_t launch_modgemm_pair(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB_half,
                                const GemmParams& prm, int tiles_m2, int num_sms, cudaStream_t stream);
cudaError_t modgemm2_set_attributes();

// Plain CUDA-core version of the same job table, used by tests to localise a
// fault to the tensor-core kernel; never on the product path.
struct SimtPlanes {
  const int8_t* a_base; long long a_plane_stride; int lda;
  const int8_t* b_base; long long b_plane_stride; int ldb;
  int M, N;
};

// Zero-initialised parameter block (flag pointers null unless the caller sets them).
inline GemmParams make_gemm_params() {
  GemmParams p;
  p.tiles_m = p.tiles_n = p.n_jobs = 0;
  p.kb_per_seg = 0; p.kb_per_unit = 1 << 28; p.group_m = 16;
  p.jobs = nullptr; p.out = nullptr; p.out_plane_stride = 0; p.ldo = 0;
  p.status = nullptr; p.work_counter = nullptr;
  p.a_hi = p.a_odd = p.b_odd = p.b_hi = nullptr;
  p.n_chunks = 0;
  p.tie_bits = nullptr;
  p.tie_list = nullptr;
  p.tie_cursor = nullptr;
  p.out_rows = p.out_cols = 0;
  p.wait_ns = 2000000000ull;
  p.withhold = 0;
  return p;
}
cudaError_t launch_modgemm_simt(int epi, const SimtPlanes& pl, const GemmParams& prm,
                                cudaStream_t stream);

// Test hooks kept by the shim: the wait limit the launchers hand to the kernels, and a
// one-shot request to withhold a producer arrival (cleared by the call that reads it).
unsigned long long lib_wait_limit_ns();
int lib_take_withhold();

// Host <-> device copies on stream st (b200_staging.cu).  Pinned or registered host memory:
// one cudaMemcpyAsync.  Pageable host memory: chunks through rings of pinned slots, the host
// side of each chunk copied by a small thread pool; a download's last hop into the caller's
// memory happens lazily, at the latest in staged_finish.
cudaError_t staged_upload(void* dst_dev, const void* src_host, size_t bytes, cudaStream_t st);
cudaError_t staged_download(void* dst_host, const void* src_dev, size_t bytes, cudaStream_t st);
cudaError_t staged_finish(cudaStream_t st);
void staged_shutdown();

}  // namespace b200
