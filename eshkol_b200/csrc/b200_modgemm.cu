// int8 x int8 -> int32 tile GEMM on the 5th-generation tensor cores (tcgen05),
// persistent and warp-specialised:
//   warp 0      one lane issues TMA loads of the A / B operand tiles into a
//               multi-stage shared-memory ring (128-byte swizzle, K-major)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=32)
//               into one of two TMEM accumulators and commits to mbarriers
//   warps 2-5   drain a finished accumulator with tcgen05.ld and run the epilogue
//               (residue mod p -> int8, raw int32, or the chunked mod-256 rule)
// Work items are (job, output tile); a job is a sum of plane-pair products, so a
// whole diagonal of slice products or one modulus accumulates without leaving TMEM.
//
// Replaces, on the reference's side, the per-modulus Metal GEMM
// (lib/backend/gpu/metal_softfloat.h:3907-4100) and the per-pair cublasGemmEx
// calls (lib/backend/gpu/gpu_memory_cuda.cpp:413-436).
#include "b200_common.cuh"
#include "b200_internal.h"

namespace b200 {

namespace {

constexpr int kNumThreads = 192;
constexpr int kUmmaK = 32;

struct WorkItem {
  int job, tm, tn;
};

__device__ __forceinline__ WorkItem decode_work(int w, const GemmParams& prm) {
  const int tiles_total = prm.tiles_m * prm.tiles_n;
  WorkItem it;
  it.job = w / tiles_total;
  const int t = w - it.job * tiles_total;
  const int per_group = prm.group_m * prm.tiles_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m0 = g * prm.group_m;
  const int gm = min(prm.group_m, prm.tiles_m - m0);
  it.tn = r / gm;
  it.tm = m0 + (r - it.tn * gm);
  return it;
}

// centred residue of x (given modulo 512) for modulus 256, ties as round-half-even
// on x/256 decides them: +128 when x = 128 (mod 512), -128 when x = 384 (mod 512)
__device__ __forceinline__ int center256(uint32_t x512) {
  int r = static_cast<int>((x512 + 128u) & 255u) - 128;
  return (x512 == 128u) ? 128 : r;
}

template <int BN, int EPI>
__global__ void __launch_bounds__(kNumThreads, 1)
modgemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmParams prm, const int total_work) {
  constexpr int kStages = (BN == 256) ? 4 : 6;
  constexpr uint32_t kABytes = kBM * kBK;
  constexpr uint32_t kBBytes = BN * kBK;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulators; 256 or 512, a power of two

  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[kStages];
  __shared__ uint64_t empty_bar[kStages];
  __shared__ uint64_t acc_full[2];
  __shared__ uint64_t acc_empty[2];
  __shared__ uint64_t sched_full[2];
  __shared__ uint64_t sched_empty[2];
  __shared__ int sched_work[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t dyn_addr = smem_u32(smem_dyn);
  const uint32_t tile_base = (dyn_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* tiles = smem_dyn + (tile_base - dyn_addr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 128);
      mbar_init(&sched_full[b], 1);
      mbar_init(&sched_empty[b], 129);  // the MMA lane and the 128 epilogue threads
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0, last_parity = 0;
      bool ok = true;
      // Work items are handed out by a global counter, so a CTA that starts late (its
      // SM was busy with another kernel) simply takes fewer tiles.  This lane claims
      // the items and publishes each id to the other roles through a 2-slot ring.
      int w = blockIdx.x;
      for (uint32_t item = 0; ok; ++item) {
        const uint32_t slot = item & 1u, sphase = (item >> 1) & 1u;
        if (!mbar_wait<false>(&sched_empty[slot], sphase ^ 1u, &abort_flag)) {
          atomicCAS(prm.status, kStatusOk, kStatusProducerTimeout);
          abort_flag = 1;
          break;
        }
        sched_work[slot] = (w < total_work) ? w : -1;
        mbar_arrive(&sched_full[slot]);
        if (w >= total_work) break;
        const WorkItem it = decode_work(w, prm);
        const GemmJob* job = &prm.jobs[it.job];
        const int nseg = job->n_seg;
        for (int seg = 0; seg < nseg && ok; ++seg) {
          const int ap = job->a_plane[seg], bp = job->b_plane[seg];
          for (int kb = 0; kb < prm.kb_per_seg; ++kb) {
            if (!mbar_wait<false>(&empty_bar[stage], phase ^ 1u, &abort_flag)) {
              atomicCAS(prm.status, kStatusOk, kStatusProducerTimeout);
              abort_flag = 1;
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&full_bar[stage], kABytes + kBBytes);
            tma_load_3d(tiles + stage * kABytes, &tmA, &full_bar[stage], kb * kBK, it.tm * kBM, ap);
            tma_load_3d(tiles + kStages * kABytes + stage * kBBytes, &tmB, &full_bar[stage],
                        kb * kBK, it.tn * BN, bp);
            issued |= 1u << stage;
            last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
        }
        w = atomicAdd(prm.work_counter, 1) + static_cast<int>(gridDim.x);
      }
      if (!ok || abort_flag) {
        // leaving early: let every copy this thread started land before the CTA exits
        int none = 0;
        for (int s = 0; s < kStages; ++s)
          if (issued & (1u << s)) mbar_wait<true>(&full_bar[s], (last_parity >> s) & 1u, &none);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_s8(kBM, BN);
      int stage = 0;
      uint32_t phase = 0, unit = 0;
      bool ok = true;
      for (uint32_t item = 0; ok; ++item) {
        const uint32_t slot = item & 1u, sphase = (item >> 1) & 1u;
        if (!mbar_wait<false>(&sched_full[slot], sphase, &abort_flag)) {
          atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
          abort_flag = 1;
          break;
        }
        const int w = sched_work[slot];
        mbar_arrive(&sched_empty[slot]);
        if (w < 0) break;
        const WorkItem it = decode_work(w, prm);
        const int kb_total = prm.jobs[it.job].n_seg * prm.kb_per_seg;
        for (int kb0 = 0; kb0 < kb_total && ok; kb0 += prm.kb_per_unit) {
          const int kb1 = min(kb0 + prm.kb_per_unit, kb_total);
          const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
          if (!mbar_wait<false>(&acc_empty[buf], aphase ^ 1u, &abort_flag)) {
            atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait<false>(&full_bar[stage], phase, &abort_flag)) {
              atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
              abort_flag = 1;
              ok = false;
              break;
            }
            tc_fence_after();
            const uint64_t da = umma_desc_k128(tile_base + stage * kABytes);
            const uint64_t db = umma_desc_k128(tile_base + kStages * kABytes + stage * kBBytes);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              // +32 bytes along K inside the swizzle atom = +2 in the encoded address
              umma_i8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
          }
          if (ok) umma_commit(&acc_full[buf]);
          ++unit;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. 32*quarter+31 belong to this warp
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t unit = 0;
    bool ok = true;
    for (uint32_t item = 0; ok; ++item) {
      const uint32_t slot = item & 1u, sphase = (item >> 1) & 1u;
      if (!mbar_wait<true>(&sched_full[slot], sphase, &abort_flag)) {
        atomicCAS(prm.status, kStatusOk, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      const int w = sched_work[slot];
      mbar_arrive(&sched_empty[slot]);
      if (w < 0) break;
      const WorkItem it = decode_work(w, prm);
      const GemmJob* job = &prm.jobs[it.job];
      const long long row = static_cast<long long>(it.tm) * kBM + row_in_tile;
      uint8_t* out_plane = prm.out + static_cast<long long>(job->out_plane) * prm.out_plane_stride;
      const long long elem0 = row * prm.ldo + static_cast<long long>(it.tn) * BN;

      if (EPI == kEpiMod256) {
        const int kb_total = job->n_seg * prm.kb_per_seg;
        uint32_t wsum[BN / 2];  // running sum of chunk residues, two 16-bit lanes per word
#pragma unroll
        for (int i = 0; i < BN / 2; ++i) wsum[i] = 0u;
        for (int kb0 = 0; kb0 < kb_total && ok; kb0 += prm.kb_per_unit) {
          const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
          if (!mbar_wait<true>(&acc_full[buf], aphase, &abort_flag)) {
            atomicCAS(prm.status, kStatusOk, kStatusEpilogueTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < BN / 32; ++cc) {
            uint32_t v[32];
            tmem_ld32(tmem_base + lane_addr + buf * BN + cc * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const int r0 = center256(v[e] & 511u);
              const int r1 = center256(v[e + 1] & 511u);
              const uint32_t packed = (static_cast<uint32_t>(r0) & 0xffffu) |
                                      (static_cast<uint32_t>(r1) << 16);
              wsum[cc * 16 + e / 2] = __vadd2(wsum[cc * 16 + e / 2], packed);
            }
          }
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
          ++unit;
        }
        if (ok) {
          int16_t* dst = reinterpret_cast<int16_t*>(out_plane) + elem0;
#pragma unroll
          for (int i = 0; i < BN / 2; i += 4) {
            uint32_t o[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              const uint32_t ws = wsum[i + t];
              const int w0 = center256(ws & 511u);
              const int w1 = center256((ws >> 16) & 511u);
              o[t] = (static_cast<uint32_t>(w0) & 0xffffu) | (static_cast<uint32_t>(w1) << 16);
            }
            *reinterpret_cast<uint4*>(dst + 2 * i) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      } else {
        const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
        if (!mbar_wait<true>(&acc_full[buf], aphase, &abort_flag)) {
          atomicCAS(prm.status, kStatusOk, kStatusEpilogueTimeout);
          abort_flag = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t p = job->modulus, magic = job->magic, offs = job->offset;
        const int half = static_cast<int>(p >> 1);  // (p-1)/2 for odd p
#pragma unroll
        for (int cc = 0; cc < BN / 32; ++cc) {
          uint32_t v[32];
          tmem_ld32(tmem_base + lane_addr + buf * BN + cc * 32, v);
          tmem_ld_wait();
          if (EPI == kEpiModI8) {
            uint32_t o[8];
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              uint32_t word = 0;
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const uint32_t u = v[g * 4 + b] + offs;   // non-negative, same class mod p
                const uint32_t q = __umulhi(u, magic);    // floor(u/p) or one less
                uint32_t r = u - q * p;
                r = (r >= p) ? r - p : r;
                const int c = (static_cast<int>(r) > half) ? static_cast<int>(r) - static_cast<int>(p)
                                                           : static_cast<int>(r);
                word |= (static_cast<uint32_t>(c) & 0xffu) << (8 * b);
              }
              o[g] = word;
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int8_t*>(out_plane) + elem0 + cc * 32);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          } else {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int32_t*>(out_plane) + elem0 + cc * 32);
#pragma unroll
            for (int g = 0; g < 8; ++g)
              dst[g] = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
        ++unit;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int BN>
constexpr size_t smem_bytes() {
  return static_cast<size_t>((BN == 256) ? 4 : 6) * (kBM * kBK + BN * kBK) + 1024;
}

template <int BN, int EPI>
cudaError_t launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& prm,
                       int total_work, int num_sms, cudaStream_t stream) {
  const int grid = total_work < num_sms ? total_work : num_sms;
  if (grid <= 0) return cudaSuccess;
  const cudaError_t e = cudaMemsetAsync(prm.work_counter, 0, sizeof(int), stream);
  if (e != cudaSuccess) return e;
  modgemm_kernel<BN, EPI><<<grid, kNumThreads, smem_bytes<BN>(), stream>>>(tmA, tmB, prm, total_work);
  return cudaGetLastError();
}

// ------------------------------------------------------------------ SIMT check
__global__ void modgemm_simt_kernel(int epi, SimtPlanes pl, GemmParams prm, int K_per_seg) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long per_job = static_cast<long long>(pl.M) * pl.N;
  if (idx >= per_job * prm.n_jobs) return;
  const int jb = static_cast<int>(idx / per_job);
  const long long rem = idx - jb * per_job;
  const int i = static_cast<int>(rem / pl.N), j = static_cast<int>(rem % pl.N);
  const GemmJob* job = &prm.jobs[jb];
  uint8_t* out_plane = prm.out + static_cast<long long>(job->out_plane) * prm.out_plane_stride;
  const long long o = static_cast<long long>(i) * prm.ldo + j;
  if (epi == kEpiMod256) {
    const int8_t* a = pl.a_base + static_cast<long long>(job->a_plane[0]) * pl.a_plane_stride +
                      static_cast<long long>(i) * pl.lda;
    const int8_t* b = pl.b_base + static_cast<long long>(job->b_plane[0]) * pl.b_plane_stride +
                      static_cast<long long>(j) * pl.ldb;
    const int unit_k = prm.kb_per_unit * kBK;
    int w = 0;
    for (int k0 = 0; k0 < K_per_seg; k0 += unit_k) {
      int acc = 0;
      const int k1 = min(k0 + unit_k, K_per_seg);
      for (int k = k0; k < k1; ++k) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
      w += center256(static_cast<uint32_t>(acc) & 511u);
    }
    reinterpret_cast<int16_t*>(out_plane)[o] =
        static_cast<int16_t>(center256(static_cast<uint32_t>(w) & 511u));
    return;
  }
  int acc = 0;
  for (int s = 0; s < job->n_seg; ++s) {
    const int8_t* a = pl.a_base + static_cast<long long>(job->a_plane[s]) * pl.a_plane_stride +
                      static_cast<long long>(i) * pl.lda;
    const int8_t* b = pl.b_base + static_cast<long long>(job->b_plane[s]) * pl.b_plane_stride +
                      static_cast<long long>(j) * pl.ldb;
    for (int k = 0; k < K_per_seg; ++k) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
  }
  if (epi == kEpiRawI32) {
    reinterpret_cast<int32_t*>(out_plane)[o] = acc;
  } else {
    const int p = static_cast<int>(job->modulus);
    int r = acc % p;
    if (r < 0) r += p;
    if (r > (p >> 1)) r -= p;
    reinterpret_cast<int8_t*>(out_plane)[o] = static_cast<int8_t>(r);
  }
}

}  // namespace

cudaError_t modgemm_set_attributes() {
  cudaError_t e;
#define B200_SET(BN, EPI)                                                                     \
  e = cudaFuncSetAttribute(modgemm_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           static_cast<int>(smem_bytes<BN>()));                               \
  if (e != cudaSuccess) return e;
  B200_SET(256, kEpiModI8)
  B200_SET(256, kEpiRawI32)
  B200_SET(256, kEpiMod256)
  B200_SET(128, kEpiModI8)
  B200_SET(128, kEpiRawI32)
  B200_SET(128, kEpiMod256)
#undef B200_SET
  return cudaSuccess;
}

cudaError_t launch_modgemm(int bn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB,
                           const GemmParams& prm, int total_work, int num_sms,
                           cudaStream_t stream) {
  if (bn == 256) {
    if (epi == kEpiModI8) return launch_one<256, kEpiModI8>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiRawI32) return launch_one<256, kEpiRawI32>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiMod256) return launch_one<256, kEpiMod256>(tmA, tmB, prm, total_work, num_sms, stream);
  } else if (bn == 128) {
    if (epi == kEpiModI8) return launch_one<128, kEpiModI8>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiRawI32) return launch_one<128, kEpiRawI32>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiMod256) return launch_one<128, kEpiMod256>(tmA, tmB, prm, total_work, num_sms, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_modgemm_simt(int epi, const SimtPlanes& pl, const GemmParams& prm,
                                cudaStream_t stream) {
  const long long total = static_cast<long long>(pl.M) * pl.N * prm.n_jobs;
  const int bs = 256;
  const long long grid = (total + bs - 1) / bs;
  if (grid <= 0 || grid > 0x7fffffffLL) return cudaErrorInvalidValue;
  modgemm_simt_kernel<<<static_cast<unsigned>(grid), bs, 0, stream>>>(epi, pl, prm,
                                                                      prm.kb_per_seg * kBK);
  return cudaGetLastError();
}

}  // namespace b200
