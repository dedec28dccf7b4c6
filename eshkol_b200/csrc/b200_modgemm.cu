// int8 x int8 -> int32 tile GEMM on the 5th-generation tensor cores (tcgen05),
// persistent and warp-specialised:
//   warp 0      one lane issues TMA loads of the A / B operand tiles into a
//               multi-stage shared-memory ring (128-byte swizzle, K-major)
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=32)
//               into one of two TMEM accumulators and commits to mbarriers
//   warps 2-5   drain a finished accumulator with tcgen05.ld and run the epilogue
//               (residue mod p -> int8, raw int32, or the chunked mod-256 rule with its
//               tie look-up in the operands' flag bit-planes)
// Work items are (job, output tile); a job is a sum of plane-pair products, so a
// whole diagonal of slice products or one modulus accumulates without leaving TMEM.
//
// Replaces, on the reference's side, the per-modulus Metal GEMM
// (lib/backend/gpu/metal_softfloat.h:3907-4100) and the per-pair cublasGemmEx
// calls (lib/backend/gpu/gpu_memory_cuda.cpp:413-436).
#include <cuda_fp16.h>

#include "b200_common.cuh"
#include "b200_internal.h"
#include "b200_residue.cuh"

namespace b200 {

namespace {

// warps 0 and 1 load and issue; 4 epilogue warps, or 8 for the chunked modulus-256 mode whose
// epilogue runs once per 8 k-blocks instead of once per tile
template <int EPI> struct EpiShape {
  static constexpr int kWarps = (EPI == kEpiMod256) ? 8 : 4;
  static constexpr int kThreads = 64 + 32 * kWarps;
};
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
__global__ void __launch_bounds__(EpiShape<EPI>::kThreads, 1)
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
      mbar_init(&acc_empty[b], 32 * EpiShape<EPI>::kWarps);
      mbar_init(&sched_full[b], 1);
      mbar_init(&sched_empty[b], 1 + 32 * EpiShape<EPI>::kWarps);  // the MMA lane and the epilogue threads
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
        if (!mbar_wait<false>(&sched_empty[slot], sphase ^ 1u, &abort_flag, prm.wait_ns)) {
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
            if (!mbar_wait<false>(&empty_bar[stage], phase ^ 1u, &abort_flag, prm.wait_ns)) {
              atomicCAS(prm.status, kStatusOk, kStatusProducerTimeout);
              abort_flag = 1;
              ok = false;
              break;
            }
            if (prm.withhold && item == 0 && seg == 0 && kb == 0) {
              // tests: this stage is never filled, so the MMA lane's wait for it runs out
              if (++stage == kStages) { stage = 0; phase ^= 1u; }
              continue;
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
          if (issued & (1u << s)) mbar_wait<true>(&full_bar[s], (last_parity >> s) & 1u, &none, prm.wait_ns);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = (EPI == kEpiF16) ? umma_idesc_f16(kBM, BN) : umma_idesc_s8(kBM, BN);
      int stage = 0;
      uint32_t phase = 0, unit = 0;
      bool ok = true;
      for (uint32_t item = 0; ok; ++item) {
        const uint32_t slot = item & 1u, sphase = (item >> 1) & 1u;
        if (!mbar_wait<false>(&sched_full[slot], sphase, &abort_flag, prm.wait_ns)) {
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
          if (!mbar_wait<false>(&acc_empty[buf], aphase ^ 1u, &abort_flag, prm.wait_ns)) {
            atomicCAS(prm.status, kStatusOk, kStatusMmaTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait<false>(&full_bar[stage], phase, &abort_flag, prm.wait_ns)) {
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
              // +32 bytes along K inside the swizzle atom = +2 in the encoded address (32 int8
              // or 16 f16 elements: one instruction's K either way)
              if (EPI == kEpiF16) umma_f16(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
              else umma_i8(d_tmem, da + 2u * k, db + 2u * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
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
      if (!mbar_wait<true>(&sched_full[slot], sphase, &abort_flag, prm.wait_ns)) {
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
        // Eight warps: warps w and w+4 read the same 32 TMEM lanes and take half of the
        // columns each.  The accumulator holds the chunk sum formed with the int8 bytes:
        // the true sum modulo 256, and modulo 512 up to the parity of the +128 / odd flag
        // products.  Bit 8 only matters when the sum is 128 modulo 256 (it then decides
        // +128 against -128), so those elements are only marked here, for a parity look-up
        // by tie_resolve_kernel.  Arithmetic runs on two 16-bit lanes per register:
        //   t = sum & 255;  residue mod 512 = t + 256*[t > 128]  (a tie counts as +128).
        constexpr int kHalfCc = BN / 64;  // 32-column groups per warp
        const int half = (warp - 2) >> 2;
        const int kb_total = job->n_seg * prm.kb_per_seg;
        uint32_t wsum[BN / 4];
#pragma unroll
        for (int i = 0; i < BN / 4; ++i) wsum[i] = 0u;
        int chunk = 0;
        for (int kb0 = 0; kb0 < kb_total && ok; kb0 += prm.kb_per_unit, ++chunk) {
          const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
          if (!mbar_wait<true>(&acc_full[buf], aphase, &abort_flag, prm.wait_ns)) {
            atomicCAS(prm.status, kStatusOk, kStatusEpilogueTimeout);
            abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          uint32_t tie_g[kHalfCc], bit8_g[kHalfCc];
#pragma unroll
          for (int c2 = 0; c2 < kHalfCc; ++c2) {
            const int cc = half * kHalfCc + c2;
            uint32_t v[32];
            tmem_ld32(tmem_base + lane_addr + buf * BN + cc * 32, v);
            tmem_ld_wait();
            uint32_t tie = 0, bit8 = 0;  // bit p: element 2p, bit 16+p: element 2p+1
#pragma unroll
            for (int p2 = 0; p2 < 16; ++p2) {
              const uint32_t pr = __byte_perm(v[2 * p2], v[2 * p2 + 1], 0x5410);  // low halves
              const uint32_t t = pr & 0x00ff00ffu;
              const uint32_t gt = (t + 0x007f007fu) & 0x01000100u;   // 256 where t > 128
              wsum[c2 * 16 + p2] += t + gt;                          // lanes stay below 2^16 (masked below)
              const uint32_t x = t ^ 0x00800080u;                    // zero lane <=> t == 128
              const uint32_t z = (x - 0x00010001u) & ~x & 0x80008000u;
              tie |= __funnelshift_r(z, z, (15 - p2) & 31);
              const uint32_t b8 = pr & 0x01000100u;
              bit8 |= __funnelshift_r(b8, b8, (8 - p2) & 31);
            }
            tie_g[c2] = tie;
            bit8_g[c2] = bit8;
            if (prm.tie_list == nullptr) {
              uint2* rec = reinterpret_cast<uint2*>(prm.tie_bits) +
                           ((static_cast<long long>(chunk) * prm.tiles_m * kBM + row) * (prm.ldo / 32) +
                            static_cast<long long>(it.tn) * (BN / 32) + cc);
              *rec = make_uint2(tie, bit8);
            }
          }
          tc_fence_before();
          mbar_arrive(&acc_empty[buf]);
          ++unit;
          if (prm.tie_list != nullptr) {
            // ties are 1 in 256 sums: only the groups of 32 columns that hold one are recorded,
            // one reservation per warp and chunk
            uint32_t has[kHalfCc];
            uint32_t count = 0;
#pragma unroll
            for (int c2 = 0; c2 < kHalfCc; ++c2) {
              has[c2] = __ballot_sync(0xffffffffu, tie_g[c2] != 0u);
              count += __popc(has[c2]);
            }
            if (count != 0u) {
              uint32_t base = 0;
              if (lane == 0) base = atomicAdd(prm.tie_cursor, count);
              base = __shfl_sync(0xffffffffu, base, 0);
#pragma unroll
              for (int c2 = 0; c2 < kHalfCc; ++c2) {
                if (tie_g[c2] != 0u) {
                  const uint32_t slot = base + __popc(has[c2] & ((1u << lane) - 1u));
                  const uint32_t cw = static_cast<uint32_t>(it.tn * (BN / 32) + half * kHalfCc + c2);
                  prm.tie_list[slot] = make_uint4(static_cast<uint32_t>(row), cw | (static_cast<uint32_t>(chunk) << 17),
                                                  tie_g[c2], bit8_g[c2]);
                }
                base += __popc(has[c2]);
              }
            }
          }
          if ((chunk & 63) == 63) {
            // only the sums modulo 512 are wanted: fold before a 16-bit lane can carry into its
            // neighbour (64 chunks add at most 64 * 511 to a lane below 512)
#pragma unroll
            for (int i = 0; i < BN / 4; ++i) wsum[i] &= 0x01ff01ffu;
          }
        }
        if (ok) {
          // sum of the chunk residues modulo 512, ties counted as +128; the reconstruction
          // adds 256 per tie that was really -128 and centres
          // 32-byte stores: a thread's row segment is contiguous, its lanes' rows are not, so
          // every store instruction of a warp touches 32 sectors; whole sectors halve their
          // number and spare L2 the merging of halves.  The warp's next barrier operation waits
          // behind these stores (cycle stamps: 7500 cycles between the last chunk of a tile and
          // the first of the next with 16-byte stores, 3700 with these).
          int16_t* dst = reinterpret_cast<int16_t*>(out_plane) + elem0 + half * (BN / 2);
#pragma unroll
          for (int i = 0; i < BN / 4; i += 8)
            asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + 2 * i),
                         "r"(wsum[i] & 0x01ff01ffu), "r"(wsum[i + 1] & 0x01ff01ffu), "r"(wsum[i + 2] & 0x01ff01ffu),
                         "r"(wsum[i + 3] & 0x01ff01ffu), "r"(wsum[i + 4] & 0x01ff01ffu), "r"(wsum[i + 5] & 0x01ff01ffu),
                         "r"(wsum[i + 6] & 0x01ff01ffu), "r"(wsum[i + 7] & 0x01ff01ffu)
                         : "memory");
        }
      } else {
       // One accumulator hand-off per tile, except for a residue product deeper than the int32
       // accumulator is exact for: it is handed over every kb_per_unit k-blocks (the reference
       // extracts every 1008 elements and sums the residues, metal_softfloat.h:4054-4067; for an
       // odd modulus only the class of the sum matters, so any interval will do) and each later
       // part is reduced together with the residue already stored.
       const int kb_total_i = job->n_seg * prm.kb_per_seg;
       for (int kb0 = 0; kb0 < kb_total_i && ok; kb0 += prm.kb_per_unit) {
        const bool later_part = (EPI == kEpiModI8) && kb0 > 0;
        const uint32_t buf = unit & 1u, aphase = (unit >> 1) & 1u;
        if (!mbar_wait<true>(&acc_full[buf], aphase, &abort_flag, prm.wait_ns)) {
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
          if (EPI == kEpiF16) {
            // f32 accumulator -> f16 (round to nearest even) -> f64, as a GEMM with f16 output
            // widened by the caller would give; the matrix is the caller's: guard its edges
            double* dst = reinterpret_cast<double*>(out_plane) + elem0 + cc * 32;
            const int col0 = it.tn * BN + cc * 32;
            if (row < prm.out_rows) {
              if (col0 + 32 <= prm.out_cols && (reinterpret_cast<uintptr_t>(dst) & 31) == 0) {
                // whole 32-byte sectors: four doubles per store
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                  double d[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    d[e] = static_cast<double>(__half2float(__float2half_rn(__uint_as_float(v[g * 4 + e]))));
                  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(dst + g * 4),
                               "f"(__int_as_float(__double2loint(d[0]))), "f"(__int_as_float(__double2hiint(d[0]))),
                               "f"(__int_as_float(__double2loint(d[1]))), "f"(__int_as_float(__double2hiint(d[1]))),
                               "f"(__int_as_float(__double2loint(d[2]))), "f"(__int_as_float(__double2hiint(d[2]))),
                               "f"(__int_as_float(__double2loint(d[3]))), "f"(__int_as_float(__double2hiint(d[3])))
                               : "memory");
                }
              } else {
#pragma unroll
                for (int e = 0; e < 32; ++e)
                  if (col0 + e < prm.out_cols)
                    dst[e] = static_cast<double>(__half2float(__float2half_rn(__uint_as_float(v[e]))));
              }
            }
          } else if (EPI == kEpiModI8) {
            uint32_t o[8];
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<int8_t*>(out_plane) + elem0 + cc * 32);
            if (later_part) {
              // add the residue of the parts before (|r| <= 127, the sum stays inside int32)
              const uint4 p0 = dst[0], p1 = dst[1];
              const uint32_t prev[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
              for (int g = 0; g < 8; ++g)
#pragma unroll
                for (int b = 0; b < 4; ++b)
                  v[g * 4 + b] += static_cast<uint32_t>(static_cast<int>(static_cast<int8_t>((prev[g] >> (8 * b)) & 0xffu)));
            }
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
  GemmParams p = prm;
  p.wait_ns = lib_wait_limit_ns();
  p.withhold = lib_take_withhold();
  modgemm_kernel<BN, EPI><<<grid, EpiShape<EPI>::kThreads, smem_bytes<BN>(), stream>>>(tmA, tmB, p, total_work);
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
    int w = 0, chunk = 0;
    for (int k0 = 0; k0 < K_per_seg; k0 += unit_k, ++chunk) {
      int acc = 0;
      const int k1 = min(k0 + unit_k, K_per_seg);
      for (int k = k0; k < k1; ++k) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
      uint32_t x = static_cast<uint32_t>(acc) & 511u;
      if ((x & 255u) == 128u) {
        const long long fa = (static_cast<long long>(i) * prm.n_chunks + chunk) * kChunkUnits;
        const long long fb = (static_cast<long long>(j) * prm.n_chunks + chunk) * kChunkUnits;
        x ^= chunk_flag_parity(prm.a_hi + fa, prm.a_odd + fa, prm.b_odd + fb, prm.b_hi + fb) << 8;
      }
      w += center256(x);
    }
    // ties are resolved here, so the value is final: the flip bits of this element stay clear
    reinterpret_cast<int16_t*>(out_plane)[o] = static_cast<int16_t>(static_cast<uint32_t>(w) & 511u);
    return;
  }
  long long acc = 0;  // a residue product may be deeper than int32 holds
  for (int s = 0; s < job->n_seg; ++s) {
    const int8_t* a = pl.a_base + static_cast<long long>(job->a_plane[s]) * pl.a_plane_stride +
                      static_cast<long long>(i) * pl.lda;
    const int8_t* b = pl.b_base + static_cast<long long>(job->b_plane[s]) * pl.b_plane_stride +
                      static_cast<long long>(j) * pl.ldb;
    for (int k = 0; k < K_per_seg; ++k) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
  }
  if (epi == kEpiRawI32) {
    reinterpret_cast<int32_t*>(out_plane)[o] = static_cast<int32_t>(acc);
  } else {
    const int p = static_cast<int>(job->modulus);
    int r = static_cast<int>(acc % p);
    if (r < 0) r += p;
    if (r > (p >> 1)) r -= p;
    reinterpret_cast<int8_t*>(out_plane)[o] = static_cast<int8_t>(r);
  }
}

// One warp per (row, 32 words of 32 columns).  The products kernel marked the elements
// whose byte sum was 128 modulo 256 in some chunk; for each of them the warp forms the
// parity of the flag products sum_k hi_a*odd_b + odd_a*hi_b over that chunk -- lane l holds
// 32-bit word l of the row's two flag vectors and loads word l of the column's -- and
// compares it with bit 8 of the byte sum: if they differ the true sum was 384 modulo 512,
// the residue -128 rather than +128, and 256 has to be added to the element's total.  The
// XOR of those corrections over the chunks is the element's flip bit.
__global__ void __launch_bounds__(256) tie_resolve_kernel(const uint2* __restrict__ tie_bits,
                                                          uint32_t* __restrict__ flip_bits,
                                                          GemmParams prm, int M, int N) {
  const int lane = threadIdx.x & 31;
  const int words = prm.ldo / 32;
  const int groups = (words + 31) / 32;
  const long long rows_p = static_cast<long long>(prm.tiles_m) * kBM;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (gw >= rows_p * groups) return;
  const long long row = gw / groups;
  const int cw = static_cast<int>(gw - row * groups) * 32 + lane;
  const bool valid = cw < words;
  const uint32_t* a_hi = reinterpret_cast<const uint32_t*>(prm.a_hi);
  const uint32_t* a_odd = reinterpret_cast<const uint32_t*>(prm.a_odd);
  const uint32_t* b_hi = reinterpret_cast<const uint32_t*>(prm.b_hi);
  const uint32_t* b_odd = reinterpret_cast<const uint32_t*>(prm.b_odd);
  constexpr int kWordsPerChunk = kChunkUnits / 2;  // 32
  uint32_t flip = 0;
  if (row < M) {
    for (int chunk = 0; chunk < prm.n_chunks; ++chunk) {
      uint2 rec = make_uint2(0u, 0u);
      if (valid) rec = __ldg(tie_bits + (static_cast<long long>(chunk) * rows_p + row) * words + cw);
      uint32_t tie = rec.x;
      uint32_t bal = __ballot_sync(0xffffffffu, tie != 0u);
      if (bal == 0u) continue;
      const long long fa = (row * prm.n_chunks + chunk) * kWordsPerChunk + lane;
      const uint32_t ahi = __ldg(a_hi + fa), aodd = __ldg(a_odd + fa);
      while (bal != 0u) {
        const int src = __ffs(bal) - 1;
        const int b = __shfl_sync(0xffffffffu, __ffs(tie) - 1, src);  // mask bit p: element 2p, 16+p: 2p+1
        const int scw = __shfl_sync(0xffffffffu, cw, src);
        const int e = (b < 16) ? 2 * b : 2 * (b - 16) + 1;
        const long long col = static_cast<long long>(scw) * 32 + e;
        if (col < N) {
          const long long fb = (col * prm.n_chunks + chunk) * kWordsPerChunk + lane;
          uint32_t x = __popc(ahi & __ldg(b_odd + fb)) ^ __popc(aodd & __ldg(b_hi + fb));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) x ^= __shfl_xor_sync(0xffffffffu, x, o);
          if (lane == src) flip ^= (((rec.y >> b) & 1u) ^ (x & 1u)) << e;
        }
        if (lane == src) tie &= tie - 1u;
        bal = __ballot_sync(0xffffffffu, tie != 0u);
      }
    }
  }
  if (valid) flip_bits[row * words + cw] = flip;
}

// The same resolution driven by the list of recorded groups: eight lanes per record, four
// records per warp at a time (the pass is bound by the latency of its dependent loads -- the
// record, then the row's flags, then each tied column's flags -- so what counts is how many
// records are in flight).  A lane holds 16 bytes of each 128-byte flag row.  The flip words
// start at zero; records of different chunks may meet in one word, hence the atomic.
__global__ void __launch_bounds__(256) tie_resolve_list_kernel(const uint4* __restrict__ list,
                                                               const unsigned int* __restrict__ cursor,
                                                               uint32_t* __restrict__ flip_bits,
                                                               GemmParams prm, int M, int N) {
  const int lane = threadIdx.x & 31, sub = lane & 7;
  const int words = prm.ldo / 32;
  const unsigned int n = *cursor;
  const unsigned int ngroups = (gridDim.x * blockDim.x) >> 3;
  const uint4* a_hi = reinterpret_cast<const uint4*>(prm.a_hi);
  const uint4* a_odd = reinterpret_cast<const uint4*>(prm.a_odd);
  const uint4* b_hi = reinterpret_cast<const uint4*>(prm.b_hi);
  const uint4* b_odd = reinterpret_cast<const uint4*>(prm.b_odd);
  constexpr int kVecPerChunk = kChunkUnits * 2 / 16;  // 8 vectors of 16 bytes per flag row
  const unsigned int g0 = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  // every group of the warp runs the same number of rounds (the shuffles below are warp-wide)
  const unsigned int rounds = (n + ngroups - 1) / ngroups;
  for (unsigned int it = 0; it < rounds; ++it) {
    const unsigned int r = g0 + it * ngroups;
    uint4 rec = make_uint4(0u, 0u, 0u, 0u);
    if (r < n) rec = __ldg(list + r);
    const long long row = rec.x;
    const int cw = static_cast<int>(rec.y & 0x1ffffu), chunk = static_cast<int>(rec.y >> 17);
    uint32_t tie = (r < n && row < M) ? rec.z : 0u;
    uint4 ahi = make_uint4(0u, 0u, 0u, 0u), aodd = ahi;
    if (tie != 0u) {
      const long long fa = (row * prm.n_chunks + chunk) * kVecPerChunk + sub;
      ahi = __ldg(a_hi + fa);
      aodd = __ldg(a_odd + fa);
    }
    uint32_t flip = 0;
    while (__any_sync(0xffffffffu, tie != 0u)) {
      uint32_t x = 0;
      int b = 0, e = 0;
      bool live = false;
      if (tie != 0u) {
        b = __ffs(tie) - 1;  // mask bit p: element 2p, 16+p: 2p+1
        tie &= tie - 1u;
        e = (b < 16) ? 2 * b : 2 * (b - 16) + 1;
        const long long col = static_cast<long long>(cw) * 32 + e;
        if (col < N) {
          live = true;
          const long long fb = (col * prm.n_chunks + chunk) * kVecPerChunk + sub;
          const uint4 bo = __ldg(b_odd + fb), bh = __ldg(b_hi + fb);
          x = __popc(ahi.x & bo.x) ^ __popc(ahi.y & bo.y) ^ __popc(ahi.z & bo.z) ^ __popc(ahi.w & bo.w) ^
              __popc(aodd.x & bh.x) ^ __popc(aodd.y & bh.y) ^ __popc(aodd.z & bh.z) ^ __popc(aodd.w & bh.w);
        }
      }
      x ^= __shfl_xor_sync(0xffffffffu, x, 1);
      x ^= __shfl_xor_sync(0xffffffffu, x, 2);
      x ^= __shfl_xor_sync(0xffffffffu, x, 4);
      if (live) flip ^= (((rec.w >> b) & 1u) ^ (x & 1u)) << e;
    }
    if (sub == 0 && flip != 0u) atomicXor(flip_bits + row * words + cw, flip);
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
  B200_SET(256, kEpiF16)
  B200_SET(128, kEpiF16)
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
    if (epi == kEpiF16) return launch_one<256, kEpiF16>(tmA, tmB, prm, total_work, num_sms, stream);
  } else if (bn == 128) {
    if (epi == kEpiF16) return launch_one<128, kEpiF16>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiModI8) return launch_one<128, kEpiModI8>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiRawI32) return launch_one<128, kEpiRawI32>(tmA, tmB, prm, total_work, num_sms, stream);
    if (epi == kEpiMod256) return launch_one<128, kEpiMod256>(tmA, tmB, prm, total_work, num_sms, stream);
  }
  return cudaErrorInvalidValue;
}

cudaError_t launch_tie_resolve(const GemmParams& prm, uint32_t* flip_bits, int M, int N,
                               cudaStream_t stream) {
  if (prm.tie_list != nullptr) {
    const size_t flip_bytes = static_cast<size_t>(prm.tiles_m) * kBM * (prm.ldo / 32) * sizeof(uint32_t);
    const cudaError_t e = cudaMemsetAsync(flip_bits, 0, flip_bytes, stream);
    if (e != cudaSuccess) return e;
    tie_resolve_list_kernel<<<148 * 8, 256, 0, stream>>>(prm.tie_list, prm.tie_cursor, flip_bits, prm, M, N);
    return cudaGetLastError();
  }
  const int words = prm.ldo / 32;
  const long long warps = static_cast<long long>(prm.tiles_m) * kBM * ((words + 31) / 32);
  if (warps <= 0) return cudaSuccess;
  tie_resolve_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint2*>(prm.tie_bits), flip_bits, prm, M, N);
  return cudaGetLastError();
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
