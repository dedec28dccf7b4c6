// Two-SM variant of the int8 products kernel: a cluster of two CTAs computes one
// 256 x 256 output tile with tcgen05.mma.cta_group::2 (M = 256 across the pair, N = 256).
// Each CTA loads its own 128 rows of A and only HALF of the B tile (128 of the 256
// columns); the tensor cores of both SMs read the two halves from both shared memories.
// Per SM and k-block that is 32 KB arriving from L2 instead of 48 KB, which is what
// bounds the one-SM kernel.  No multicast load is used: every CTA issues its own TMA
// loads; only their completion is counted on the leader CTA's barrier, and
// tcgen05.commit signals the barriers of both CTAs.
//
// Roles per CTA (192 threads): warp 0 lane 0 issues TMA loads; warp 1 allocates TMEM
// (both CTAs, cta_group::2) and, in the leader CTA only, one lane issues the MMAs;
// warps 2-5 drain the CTA's own 128 x 256 accumulator.  Work items are (job, pair
// tile), statically strided over the clusters.  Every wait is bounded like in the
// one-SM kernel; both CTAs meet at a cluster barrier before TMEM is freed.
#include "b200_common.cuh"
#include "b200_internal.h"

namespace b200 {

namespace {

constexpr int kThreads2 = 192;
constexpr int kUmmaK = 32;
constexpr int kBN2 = 256;                       // pair tile columns
constexpr int kStages2 = 6;
constexpr uint32_t kABytes2 = kBM * kBK;        // 16 KB: this CTA's 128 rows of A
constexpr uint32_t kBBytes2 = (kBN2 / 2) * kBK;  // 16 KB: this CTA's half of the B tile
constexpr uint32_t kTmemCols2 = 2 * kBN2;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.aligned;\n\tbarrier.cluster.wait.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// load into THIS CTA's shared memory; completion bytes are counted on the barrier at
// `bar_cluster_addr`, which lives in the leader CTA
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(c0),
        "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs once the MMAs issued so
// far have completed
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smem_u32(bar)),
      "h"(mask)
      : "memory");
}

struct PairWork {
  int job, tm, tn;
};
__device__ __forceinline__ PairWork decode_pair(int w, int tiles_m2, const GemmParams& prm) {
  const int tiles_total = tiles_m2 * prm.tiles_n;
  PairWork it;
  it.job = w / tiles_total;
  const int t = w - it.job * tiles_total;
  const int gmx = max(prm.group_m / 2, 1);
  const int per_group = gmx * prm.tiles_n;
  const int g = t / per_group;
  const int r = t - g * per_group;
  const int m0 = g * gmx;
  const int gm = min(gmx, tiles_m2 - m0);
  it.tn = r / gm;
  it.tm = m0 + (r - it.tn * gm);
  return it;
}

template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads2, 1)
modgemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                const GemmParams prm, const int tiles_m2, const int total_work) {
  extern __shared__ uint8_t smem_dyn[];
  __shared__ uint64_t full_bar[kStages2];   // used in the leader: both CTAs' loads of a stage landed
  __shared__ uint64_t empty_bar[kStages2];  // per CTA: the MMAs reading this stage completed
  __shared__ uint64_t acc_full[2];          // per CTA: an accumulator is complete
  __shared__ uint64_t acc_empty[2];         // used in the leader: both CTAs drained an accumulator
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const uint32_t dyn_addr = smem_u32(smem_dyn);
  const uint32_t tile_base = (dyn_addr + 1023u) & ~1023u;
  uint8_t* tiles = smem_dyn + (tile_base - dyn_addr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 256);
    }
    abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc2(&tmem_slot, kTmemCols2);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled on them
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
      for (int w = pair; w < total_work && ok; w += npairs) {
        const PairWork it = decode_pair(w, tiles_m2, prm);
        const GemmJob* job = &prm.jobs[it.job];
        const int nseg = job->n_seg;
        for (int seg = 0; seg < nseg && ok; ++seg) {
          const int ap = job->a_plane[seg], bp = job->b_plane[seg];
          for (int kb = 0; kb < prm.kb_per_seg; ++kb) {
            if (!mbar_wait<false>(&empty_bar[stage], phase ^ 1u, &abort_flag, prm.wait_ns)) {
              atomicCAS(prm.status, kStatusOk, kStatusProducerTimeout);
              abort_flag = 1;
              ok = false;
              break;
            }
            const uint32_t leader_full = mapa_u32(smem_u32(&full_bar[stage]), 0);
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2u * (kABytes2 + kBBytes2));
            tma_load_3d_pair(tiles + stage * kABytes2, &tmA, leader_full, kb * kBK,
                             it.tm * 256 + static_cast<int>(rank) * kBM, ap);
            tma_load_3d_pair(tiles + kStages2 * kABytes2 + stage * kBBytes2, &tmB, leader_full, kb * kBK,
                             it.tn * kBN2 + static_cast<int>(rank) * (kBN2 / 2), bp);
            issued |= 1u << stage;
            last_parity = (last_parity & ~(1u << stage)) | (phase << stage);
            if (++stage == kStages2) { stage = 0; phase ^= 1u; }
          }
        }
      }
      if ((!ok || abort_flag) && rank == 0) {
        // leaving early: both CTAs' copies of a stage complete on the leader's barrier, so the
        // leader waits (bounded) for every stage it armed; the peer cannot leave before the
        // leader does (the cluster barrier at the end of the kernel), and its own copies, which
        // take microseconds, have long landed by then
        int none = 0;
        for (int s = 0; s < kStages2; ++s)
          if (issued & (1u << s)) mbar_wait<true>(&full_bar[s], (last_parity >> s) & 1u, &none, prm.wait_ns);
      }
    }
  } else if (warp == 1) {
    // --------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_s8(256, kBN2);
      int stage = 0;
      uint32_t phase = 0, unit = 0;
      bool ok = true;
      for (int w = pair; w < total_work && ok; w += npairs) {
        const PairWork it = decode_pair(w, tiles_m2, prm);
        const int kb_total = prm.jobs[it.job].n_seg * prm.kb_per_seg;
        const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
        if (!mbar_wait<false>(&acc_empty[buf], aphase ^ 1u, &abort_flag, prm.wait_ns)) {
          atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
          abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kBN2;
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait<false>(&full_bar[stage], phase, &abort_flag, prm.wait_ns)) {
            atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = umma_desc_k128(tile_base + stage * kABytes2);
          const uint64_t db = umma_desc_k128(tile_base + kStages2 * kABytes2 + stage * kBBytes2);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_i8_pair(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(&acc_full[buf]);
        ++unit;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    uint32_t unit = 0;
    for (int w = pair; w < total_work; w += npairs) {
      const PairWork it = decode_pair(w, tiles_m2, prm);
      const GemmJob* job = &prm.jobs[it.job];
      const long long row = static_cast<long long>(it.tm) * 256 + static_cast<long long>(rank) * kBM + row_in_tile;
      uint8_t* out_plane = prm.out + static_cast<long long>(job->out_plane) * prm.out_plane_stride;
      const long long elem0 = row * prm.ldo + static_cast<long long>(it.tn) * kBN2;
      const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
      if (!mbar_wait<true>(&acc_full[buf], aphase, &abort_flag, prm.wait_ns)) {
        atomicCAS(prm.status, kStatusOk, kStatusEpilogueTimeout);
        abort_flag = 1;
        break;
      }
      tc_fence_after();
      const uint32_t p = job->modulus, magic = job->magic, offs = job->offset;
      const int half = static_cast<int>(p >> 1);
#pragma unroll
      for (int cc = 0; cc < kBN2 / 32; ++cc) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_addr + buf * kBN2 + cc * 32, v);
        tmem_ld_wait();
        if (EPI == kEpiModI8) {
          uint32_t o[8];
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t u = v[g * 4 + b] + offs;
              const uint32_t q = __umulhi(u, magic);
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
      // the leader's MMA lane reuses the accumulator once all 256 epilogue threads of the pair arrived
      mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty[buf]), 0));
      ++unit;
    }
  }

  tc_fence_before();
  __syncwarp();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols2);
  }
}

constexpr size_t kSmem2 = static_cast<size_t>(kStages2) * (kABytes2 + kBBytes2) + 1024;

template <int EPI>
cudaError_t launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& prm,
                        int tiles_m2, int total_work, int num_sms, cudaStream_t stream) {
  int grid = (num_sms / 2) * 2;
  if (2 * total_work < grid) grid = 2 * total_work;
  if (grid <= 0) return cudaSuccess;
  GemmParams p = prm;
  p.wait_ns = lib_wait_limit_ns();
  p.withhold = 0;
  modgemm2_kernel<EPI><<<grid, kThreads2, kSmem2, stream>>>(tmA, tmB, p, tiles_m2, total_work);
  return cudaGetLastError();
}

}  // namespace

cudaError_t modgemm2_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(modgemm2_kernel<kEpiModI8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmem2));
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(modgemm2_kernel<kEpiRawI32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(kSmem2));
}

// tmB must be tiled in boxes of 128 rows (half of the pair tile's columns).
cudaError_t launch_modgemm_pair(int epi, const CUtensorMap& tmA, const CUtensorMap& tmB_half,
                                const GemmParams& prm, int tiles_m2, int num_sms, cudaStream_t stream) {
  const int total = prm.n_jobs * tiles_m2 * prm.tiles_n;
  if (epi == kEpiModI8) return launch_pair<kEpiModI8>(tmA, tmB_half, prm, tiles_m2, total, num_sms, stream);
  if (epi == kEpiRawI32) return launch_pair<kEpiRawI32>(tmA, tmB_half, prm, tiles_m2, total, num_sms, stream);
  return cudaErrorInvalidValue;
}

}  // namespace b200
