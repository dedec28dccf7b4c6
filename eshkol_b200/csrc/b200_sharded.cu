// Row-sharded exact-tier GEMM over the GPUs of one box, driven from C
// (include/eshkol_b200_multi.h): one process per GPU, the ranks meeting in a POSIX
// shared-memory segment that carries the CUDA IPC handles and the host barriers.
//
// The schedule per rank and step:
//   * B stays on the source rank.  For every column panel this rank pulls its 1/world of the
//     panel's columns (one pitched copy), scans and splits them into its place of the panel's
//     plane buffer, and pulls the other ranks' pieces out of their buffers -- B is split once,
//     not once per rank;
//   * A is prepared once; a panel is multiplied as soon as its planes are complete, the
//     products writing their block of C in place; every other rank pulls that block into the
//     same place of its own C while later panels are multiplied;
//   * panels are narrow at both ends, because the first panel's way to the ranks and the last
//     block's way back are the two transfers no products hide.
// Only copy engines move data between the GPUs (cudaMemcpy2DAsync on mapped peer memory):
// beside the persistent tensor-core kernels a copy runs at full rate, a kernel of another
// stream does not run at all.  The reference is single-device and has no counterpart.
#include "../../include/eshkol_b200_multi.h"

#include <cuda_runtime.h>
#include <fcntl.h>
#include <sched.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <new>

#include "../../include/eshkol_b200_ext.h"
#include "../../include/eshkol_b200_testing.h"

namespace {

constexpr int kMaxRanks = 16, kMaxPanels = 24, kSlots = 3, kPool = 8;
constexpr uint32_t kMagic = 0xE5B20001u;

struct Ctl {  // the shared-memory segment
  std::atomic<uint32_t> magic, arrived, generation;
  std::atomic<int32_t> failed;
  struct Rank {
    cudaIpcMemHandle_t b, c, planes[kMaxPanels];
    cudaIpcEventHandle_t planes_ev[kMaxPanels], block_ev[kMaxPanels];
  } rank[kMaxRanks];
};

double now_s() {
  timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return static_cast<double>(t.tv_sec) + 1e-9 * static_cast<double>(t.tv_nsec);
}

}  // namespace

struct EshkolB200Sharded {
  char name[128];
  int rank, world, src, P;
  long long M, K, N;
  Ctl* ctl;
  double timeout_s;
  long long col0[kMaxPanels], width[kMaxPanels];
  long long row0[kMaxRanks], rows[kMaxRanks];
  long long part0[kMaxPanels][kMaxRanks], partn[kMaxPanels][kMaxRanks];  // this panel's columns per rank
  uint64_t regions[kMaxPanels][kMaxRanks][7][4];
  void *blk_b, *blk_c, *blk_p[kMaxPanels];
  char *addr_b, *addr_c[kMaxRanks], *addr_p[kMaxRanks][kMaxPanels];
  cudaEvent_t ev_planes[kMaxRanks][kMaxPanels], ev_block[kMaxRanks][kMaxPanels];
  double* bcol[kSlots];
  cudaEvent_t bcol_free[kSlots];
  bool bcol_used[kSlots];
  cudaStream_t x1, x2, pool[kPool], gpool[kPool];
  int npool;
  int ahead;  // panels of B whose planes are on their way while one is multiplied
  cudaEvent_t ev_got[kMaxPanels], ev_arrived[kMaxPanels], ev_tmp[kPool];
};

namespace {

#define SH_CHECK(call)                                                                  \
  do {                                                                                  \
    cudaError_t e_ = (call);                                                            \
    if (e_ != cudaSuccess) {                                                            \
      fprintf(stderr, "[eshkol-b200] rank %d: %s failed: %s (%s:%d)\n", s->rank, #call, \
              cudaGetErrorString(e_), __FILE__, __LINE__);                              \
      s->ctl->failed.store(1);                                                          \
      return -1;                                                                        \
    }                                                                                   \
  } while (0)

int fail(EshkolB200Sharded* s, const char* what) {
  fprintf(stderr, "[eshkol-b200] rank %d: %s\n", s->rank, what);
  if (s->ctl) s->ctl->failed.store(1);
  return -1;
}

// Sense-reversing barrier in the shared segment; gives up when a rank has failed or after the
// timeout (a rank that never arrives must not hold the others for ever).
int barrier(EshkolB200Sharded* s) {
  Ctl* c = s->ctl;
  const uint32_t gen = c->generation.load();
  if (c->arrived.fetch_add(1) + 1 == static_cast<uint32_t>(s->world)) {
    c->arrived.store(0);
    c->generation.fetch_add(1);
    return c->failed.load() ? -1 : 0;
  }
  const double t0 = now_s();
  unsigned spins = 0;
  while (c->generation.load() == gen) {
    if (c->failed.load()) return -1;
    if ((++spins & 1023u) == 0u) {
      if (now_s() - t0 > s->timeout_s) return fail(s, "a barrier of the sharded step timed out");
      sched_yield();
    }
  }
  return c->failed.load() ? -1 : 0;
}

// The shared segment: rank 0 creates it afresh, the others wait for it to appear and to be
// initialised.  0 / -1.
int join_segment(EshkolB200Sharded* s) {
  const char* name = s->name;
  const int rank = s->rank;
  int fd = -1;
  const double t0 = now_s();
  if (rank == 0) {
    shm_unlink(name);
    fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0 || ftruncate(fd, sizeof(Ctl)) != 0) {
      fprintf(stderr, "[eshkol-b200] rank 0: cannot create the session segment %s\n", name);
      if (fd >= 0) close(fd);
      return -1;
    }
  } else {
    for (;;) {
      fd = shm_open(name, O_RDWR, 0600);
      struct stat sb;
      if (fd >= 0 && fstat(fd, &sb) == 0 && static_cast<size_t>(sb.st_size) >= sizeof(Ctl)) break;
      if (fd >= 0) close(fd);
      fd = -1;
      if (now_s() - t0 > s->timeout_s) {
        fprintf(stderr, "[eshkol-b200] rank %d: the session segment %s never appeared\n", rank, name);
        return -1;
      }
      usleep(1000);
    }
  }
  void* map = mmap(nullptr, sizeof(Ctl), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (map == MAP_FAILED) return -1;
  s->ctl = static_cast<Ctl*>(map);
  if (rank == 0) {
    s->ctl->arrived.store(0); s->ctl->generation.store(0); s->ctl->failed.store(0);
    s->ctl->magic.store(kMagic);
  } else {
    while (s->ctl->magic.load() != kMagic) {
      if (now_s() - t0 > s->timeout_s) {
        fail(s, "the session segment was never initialised");
        munmap(map, sizeof(Ctl));
        s->ctl = nullptr;
        return -1;
      }
      usleep(1000);
    }
  }
  return 0;
}

// (first, count) of part r when n items are cut into `world` contiguous parts
void partition(long long n, int world, int r, long long* first, long long* count) {
  const long long base = n / world, extra = n % world;
  *first = r * base + (r < extra ? r : extra);
  *count = base + (r < extra ? 1 : 0);
}

// A panel's columns cut into one contiguous share per rank, in rank order.  The source rank
// also sends every other rank its f64 columns, so its link carries more than the others';
// its share (and with it the planes it serves to every peer) is src_weight of theirs.
void column_shares(long long wd, int world, int src, double src_weight, long long* first, long long* count) {
  if (world == 1) { first[0] = 0; count[0] = wd; return; }
  long long n0 = static_cast<long long>(static_cast<double>(wd) * src_weight / (world - 1 + src_weight));
  if (n0 < 0) n0 = 0;
  if (n0 > wd) n0 = wd;
  const long long rest = wd - n0, base = rest / (world - 1), extra = rest % (world - 1);
  long long c = 0;
  int k = 0;
  for (int r = 0; r < world; ++r) {
    count[r] = (r == src) ? n0 : base + (k++ < extra ? 1 : 0);
    first[r] = c;
    c += count[r];
  }
}

// Column panels: widths grow by half from w/8 (w = N/4), stay near w, halve down to w/8.  A
// panel of residue planes is twice the bytes of its f64 columns, so its exchange hides behind
// the products of the panel before it only up to a ratio of about 1.5.
int make_panels(long long N, long long* col0, long long* width) {
  const long long w = N / 4;
  int P = 0;
  if (N % 4 != 0 || w % 2048 != 0) {  // shapes that do not allow multiples of the 256-column tile
    const int parts = (N % 4 == 0 && w > 0) ? 4 : 1;
    for (int p = 0; p < parts; ++p) { col0[p] = p * (N / parts); width[p] = N / parts; }
    return parts;
  }
  long long up[kMaxPanels];
  int n_up = 0;
  for (long long x = w / 8; x < w * 3 / 4; x = (x * 3 / 2 + 255) / 256 * 256) up[n_up++] = x;
  const long long down[3] = {w / 2, w / 4, w / 8};
  long long sum_up = 0;
  for (int i = 0; i < n_up; ++i) sum_up += up[i];
  const long long mid_total = N - sum_up - (down[0] + down[1] + down[2]);
  const long long n_mid = (mid_total + w - 1) / w > 0 ? (mid_total + w - 1) / w : 1;
  const long long mid = (mid_total / n_mid) / 256 * 256;
  long long c = 0;
  for (int i = 0; i < n_up; ++i) { col0[P] = c; width[P++] = up[i]; c += up[i]; }
  for (long long i = 0; i < n_mid; ++i) {
    const long long wd = (i + 1 < n_mid) ? mid : mid_total - mid * (n_mid - 1);
    col0[P] = c; width[P++] = wd; c += wd;
  }
  for (int i = 0; i < 3; ++i) { col0[P] = c; width[P++] = down[i]; c += down[i]; }
  return P;
}

int copy2d(EshkolB200Sharded* s, void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t rows,
           cudaStream_t st) {
  if (width == 0 || rows == 0) return 0;
  SH_CHECK(cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, rows, cudaMemcpyDefault, st));
  return 0;
}

// this rank's share of panel p: fetch its columns of B (the source reads its own B in place),
// scan and split them into the panel's plane buffer, and say so to the peers
int stage_prep(EshkolB200Sharded* s, int p) {
  cudaStream_t lib = static_cast<cudaStream_t>(eshkol_b200_stream());
  const int R = s->rank;
  const long long c0 = s->part0[p][R], n = s->partn[p][R], wd = s->width[p];
  if (n > 0) {
    const double* src_ptr;
    long long ldb;
    if (R == s->src) {
      src_ptr = reinterpret_cast<const double*>(s->blk_b) + s->col0[p] + c0;
      ldb = s->N;
    } else {
      const int slot = p % kSlots;
      if (s->bcol_used[slot]) SH_CHECK(cudaStreamWaitEvent(s->x1, s->bcol_free[slot], 0));
      if (copy2d(s, s->bcol[slot], static_cast<size_t>(n) * 8, s->addr_b + (s->col0[p] + c0) * 8,
                 static_cast<size_t>(s->N) * 8, static_cast<size_t>(n) * 8, static_cast<size_t>(s->K), s->x1))
        return -1;
      SH_CHECK(cudaEventRecord(s->ev_got[p], s->x1));
      SH_CHECK(cudaStreamWaitEvent(lib, s->ev_got[p], 0));
      src_ptr = s->bcol[slot];
      ldb = n;
    }
    if (eshkol_b200_prepare_b_columns_f64_device(src_ptr, static_cast<uint64_t>(ldb), static_cast<uint64_t>(s->K),
                                                 static_cast<uint64_t>(wd), static_cast<uint64_t>(c0),
                                                 static_cast<uint64_t>(n), s->blk_p[p]) != 0)
      return fail(s, "prepare_b_columns failed");
    if (R != s->src) {
      SH_CHECK(cudaEventRecord(s->bcol_free[p % kSlots], lib));
      s->bcol_used[p % kSlots] = true;
    }
  }
  SH_CHECK(cudaEventRecord(s->ev_planes[R][p], lib));
  return 0;
}

// pull the other ranks' shares of panel p's planes into their places; ev_arrived[p] follows them
int pull_planes(EshkolB200Sharded* s, int p) {
  const int R = s->rank, W = s->world;
  for (int i = 1; i < W; ++i) {
    const int q = (R + i) % W;
    if (s->partn[p][q] == 0) continue;
    cudaStream_t st = s->pool[i % s->npool];
    SH_CHECK(cudaStreamWaitEvent(st, s->ev_planes[q][p], 0));
    for (int g = 0; g < 7; ++g) {
      const uint64_t* rg = s->regions[p][q][g];
      if (copy2d(s, static_cast<char*>(s->blk_p[p]) + rg[0], rg[3], s->addr_p[q][p] + rg[0], rg[3], rg[1], rg[2], st))
        return -1;
    }
  }
  for (int i = 0; i < s->npool; ++i) {
    SH_CHECK(cudaEventRecord(s->ev_tmp[i], s->pool[i]));
    SH_CHECK(cudaStreamWaitEvent(s->x2, s->ev_tmp[i], 0));
  }
  SH_CHECK(cudaEventRecord(s->ev_arrived[p], s->x2));
  return 0;
}

// pull every other rank's block of panel p of C into its place, once it is computed
int gather_panel(EshkolB200Sharded* s, int p) {
  const int R = s->rank, W = s->world;
  for (int i = 1; i < W; ++i) {
    const int q = (R + i) % W;
    if (s->rows[q] == 0) continue;
    cudaStream_t st = s->gpool[i % s->npool];
    SH_CHECK(cudaStreamWaitEvent(st, s->ev_block[q][p], 0));
    const size_t off = static_cast<size_t>(s->row0[q] * s->N + s->col0[p]) * 8;
    if (copy2d(s, static_cast<char*>(s->blk_c) + off, static_cast<size_t>(s->N) * 8, s->addr_c[q] + off,
               static_cast<size_t>(s->N) * 8, static_cast<size_t>(s->width[p]) * 8, static_cast<size_t>(s->rows[q]), st))
      return -1;
  }
  return 0;
}

}  // namespace

extern "C" {

int eshkol_b200_sharded_open(const char* name, int rank, int world, uint64_t M_, uint64_t K_, uint64_t N_,
                             int src_rank, EshkolB200Sharded** out) {
  if (!name || !out || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || src_rank < 0 ||
      src_rank >= world || M_ == 0 || K_ == 0 || N_ == 0 || K_ > 262144 || strlen(name) >= sizeof(EshkolB200Sharded::name))
    return -1;
  if (!eshkol_b200_stream()) {
    fprintf(stderr, "[eshkol-b200] sharded_open called before eshkol_b200_init succeeded\n");
    return -1;
  }
  EshkolB200Sharded* s = new (std::nothrow) EshkolB200Sharded();
  if (!s) return -1;
  memset(static_cast<void*>(s), 0, sizeof(*s));
  snprintf(s->name, sizeof(s->name), "%s", name);
  s->rank = rank; s->world = world; s->src = src_rank;
  s->M = static_cast<long long>(M_); s->K = static_cast<long long>(K_); s->N = static_cast<long long>(N_);
  const char* te = getenv("ESHKOL_B200_BARRIER_TIMEOUT_S");
  s->timeout_s = (te && atof(te) > 0.0) ? atof(te) : 60.0;

  if (join_segment(s) != 0) { delete s; return -1; }

  // ---- geometry ----
  s->P = make_panels(s->N, s->col0, s->width);
  for (int r = 0; r < world; ++r) partition(s->M, world, r, &s->row0[r], &s->rows[r]);
  double src_weight = 0.5;
  if (const char* e = getenv("ESHKOL_B200_SRC_SHARE")) {
    if (e[0]) src_weight = atof(e);
    if (!(src_weight >= 0.0)) src_weight = 0.0;
    if (src_weight > 1.0) src_weight = 1.0;
  }
  for (int p = 0; p < s->P; ++p)
    column_shares(s->width[p], world, src_rank, src_weight, s->part0[p], s->partn[p]);
  for (int p = 0; p < s->P; ++p)
    for (int r = 0; r < world; ++r) {
      if (s->partn[p][r] > 0 &&
          eshkol_b200_prepared_b_regions(K_, static_cast<uint64_t>(s->width[p]), static_cast<uint64_t>(s->part0[p][r]),
                                         static_cast<uint64_t>(s->partn[p][r]), s->regions[p][r]) != 7) {
        fail(s, "prepared_b_regions failed");
        return -1;
      }
    }

  // ---- this rank's buffers, events and streams ----
  Ctl::Rank& mine = s->ctl->rank[rank];
  if (rank == src_rank) {
    if (eshkol_b200_mem_alloc(0, static_cast<size_t>(s->K) * s->N * 8, &s->blk_b) != 0) return fail(s, "allocation of B failed");
    SH_CHECK(cudaIpcGetMemHandle(&mine.b, s->blk_b));
  }
  if (eshkol_b200_mem_alloc(0, static_cast<size_t>(s->M) * s->N * 8, &s->blk_c) != 0) return fail(s, "allocation of C failed");
  SH_CHECK(cudaIpcGetMemHandle(&mine.c, s->blk_c));
  long long ncmax = 1;
  for (int p = 0; p < s->P; ++p) {
    if (eshkol_b200_mem_alloc(0, eshkol_b200_prepared_b_bytes(K_, static_cast<uint64_t>(s->width[p])), &s->blk_p[p]) != 0)
      return fail(s, "allocation of a plane buffer failed");
    SH_CHECK(cudaIpcGetMemHandle(&mine.planes[p], s->blk_p[p]));
    SH_CHECK(cudaEventCreateWithFlags(&s->ev_planes[rank][p], cudaEventDisableTiming | cudaEventInterprocess));
    SH_CHECK(cudaEventCreateWithFlags(&s->ev_block[rank][p], cudaEventDisableTiming | cudaEventInterprocess));
    SH_CHECK(cudaIpcGetEventHandle(&mine.planes_ev[p], s->ev_planes[rank][p]));
    SH_CHECK(cudaIpcGetEventHandle(&mine.block_ev[p], s->ev_block[rank][p]));
    SH_CHECK(cudaEventCreateWithFlags(&s->ev_got[p], cudaEventDisableTiming));
    SH_CHECK(cudaEventCreateWithFlags(&s->ev_arrived[p], cudaEventDisableTiming));
    for (int r = 0; r < world; ++r) if (s->partn[p][r] > ncmax) ncmax = s->partn[p][r];
  }
  if (rank != src_rank)
    for (int i = 0; i < kSlots; ++i) {
      void* d = nullptr;
      if (eshkol_b200_mem_alloc(0, static_cast<size_t>(s->K) * ncmax * 8, &d) != 0) return fail(s, "allocation of a column buffer failed");
      s->bcol[i] = static_cast<double*>(d);
      SH_CHECK(cudaEventCreateWithFlags(&s->bcol_free[i], cudaEventDisableTiming));
    }
  {
    // streams the pulls of one panel are spread over (each peer's copies stay on one stream)
    const char* e = getenv("ESHKOL_B200_POOL");
    int want = (e && e[0]) ? atoi(e) : 4;
    if (want < 1) want = 1;
    if (want > kPool) want = kPool;
    s->npool = world - 1 < want ? (world - 1 > 0 ? world - 1 : 1) : want;
  }
  SH_CHECK(cudaStreamCreateWithFlags(&s->x1, cudaStreamNonBlocking));
  SH_CHECK(cudaStreamCreateWithFlags(&s->x2, cudaStreamNonBlocking));
  for (int i = 0; i < s->npool; ++i) {
    SH_CHECK(cudaStreamCreateWithFlags(&s->pool[i], cudaStreamNonBlocking));
    SH_CHECK(cudaStreamCreateWithFlags(&s->gpool[i], cudaStreamNonBlocking));
    SH_CHECK(cudaEventCreateWithFlags(&s->ev_tmp[i], cudaEventDisableTiming));
  }
  {
    const char* e = getenv("ESHKOL_B200_AHEAD");
    s->ahead = (e && e[0]) ? atoi(e) : 2;
    if (s->ahead < 2) s->ahead = 2;
    if (s->ahead > kMaxPanels) s->ahead = kMaxPanels;
  }

  // ---- exchange: every rank has published its handles, then opens the peers' ----
  if (barrier(s) != 0) return -1;
  for (int q = 0; q < world; ++q) {
    if (q == rank) {
      s->addr_c[q] = static_cast<char*>(s->blk_c);
      for (int p = 0; p < s->P; ++p) s->addr_p[q][p] = static_cast<char*>(s->blk_p[p]);
      if (q == src_rank) s->addr_b = static_cast<char*>(s->blk_b);
      continue;
    }
    const Ctl::Rank& peer = s->ctl->rank[q];
    void* ptr = nullptr;
    if (q == src_rank) {
      SH_CHECK(cudaIpcOpenMemHandle(&ptr, peer.b, cudaIpcMemLazyEnablePeerAccess));
      s->addr_b = static_cast<char*>(ptr);
    }
    SH_CHECK(cudaIpcOpenMemHandle(&ptr, peer.c, cudaIpcMemLazyEnablePeerAccess));
    s->addr_c[q] = static_cast<char*>(ptr);
    for (int p = 0; p < s->P; ++p) {
      SH_CHECK(cudaIpcOpenMemHandle(&ptr, peer.planes[p], cudaIpcMemLazyEnablePeerAccess));
      s->addr_p[q][p] = static_cast<char*>(ptr);
      SH_CHECK(cudaIpcOpenEventHandle(&s->ev_planes[q][p], peer.planes_ev[p]));
      SH_CHECK(cudaIpcOpenEventHandle(&s->ev_block[q][p], peer.block_ev[p]));
    }
  }
  SH_CHECK(cudaDeviceSynchronize());
  if (barrier(s) != 0) return -1;
  *out = s;
  return 0;
}

// Tests only: the rendezvous and the barriers of a session without any GPU work.  Runs
// `barriers` barriers; a rank given fail_at = k marks the session failed instead of entering
// barrier k and leaves (what a rank does whose step hit an error), leave_at = k makes it leave
// without a word.  Returns 0, or -1 as soon as a barrier gives up.
int eshkol_b200_debug_rendezvous(const char* name, int rank, int world, int barriers, int fail_at, int leave_at,
                                 double timeout_s) {
  if (!name || world < 1 || world > kMaxRanks || rank < 0 || rank >= world || strlen(name) >= sizeof(EshkolB200Sharded::name))
    return -1;
  EshkolB200Sharded* s = new (std::nothrow) EshkolB200Sharded();
  if (!s) return -1;
  memset(static_cast<void*>(s), 0, sizeof(*s));
  snprintf(s->name, sizeof(s->name), "%s", name);
  s->rank = rank; s->world = world;
  s->timeout_s = timeout_s > 0.0 ? timeout_s : 60.0;
  if (join_segment(s) != 0) { delete s; return -1; }
  int rc = 0;
  for (int k = 0; k < barriers && rc == 0; ++k) {
    if (k == leave_at) break;
    if (k == fail_at) { fail(s, "told to fail"); rc = -1; break; }
    rc = barrier(s);
  }
  munmap(s->ctl, sizeof(Ctl));
  delete s;
  return rc;
}

// Tests only, no GPU: the plan a session of this shape would follow -- the column panels
// (first column and width of each, at most `capacity`) and, per panel, every rank's share of
// its columns (first[p * world + r], count[p * world + r]).  Returns the number of panels.
int eshkol_b200_debug_sharded_plan(uint64_t N, int world, int src, double src_weight, int capacity,
                                   uint64_t* col0, uint64_t* width, uint64_t* first, uint64_t* count) {
  if (!col0 || !width || !first || !count || world < 1 || world > kMaxRanks || src < 0 || src >= world || N == 0)
    return -1;
  long long c0[kMaxPanels], wd[kMaxPanels], f[kMaxRanks], n[kMaxRanks];
  const int P = make_panels(static_cast<long long>(N), c0, wd);
  if (P > capacity) return -1;
  for (int p = 0; p < P; ++p) {
    col0[p] = static_cast<uint64_t>(c0[p]);
    width[p] = static_cast<uint64_t>(wd[p]);
    column_shares(wd[p], world, src, src_weight, f, n);
    for (int r = 0; r < world; ++r) {
      first[p * world + r] = static_cast<uint64_t>(f[r]);
      count[p * world + r] = static_cast<uint64_t>(n[r]);
    }
  }
  return P;
}

int eshkol_b200_sharded_rows(const EshkolB200Sharded* s, uint64_t* row0, uint64_t* rows) {
  if (!s) return -1;
  if (row0) *row0 = static_cast<uint64_t>(s->row0[s->rank]);
  if (rows) *rows = static_cast<uint64_t>(s->rows[s->rank]);
  return 0;
}

double* eshkol_b200_sharded_b_buffer(EshkolB200Sharded* s) {
  return (s && s->rank == s->src) ? static_cast<double*>(s->blk_b) : nullptr;
}

double* eshkol_b200_sharded_c_buffer(EshkolB200Sharded* s) { return s ? static_cast<double*>(s->blk_c) : nullptr; }

int eshkol_b200_sharded_step(EshkolB200Sharded* s, const double* dA_rows) {
  if (!s) return -1;
  const int R = s->rank, P = s->P;
  const long long my_rows = s->rows[R];
  if (my_rows > 0 && !dA_rows) return fail(s, "no rows of A were passed");
  cudaStream_t lib = static_cast<cudaStream_t>(eshkol_b200_stream());
  for (int i = 0; i < kSlots; ++i) s->bcol_used[i] = false;
  // every rank is in the step: B on the source rank is complete, nobody reads last step's buffers
  if (barrier(s) != 0) return -1;
  const int ahead = s->ahead;
  // the first two panels' shares are split before this rank's rows of A are: their exchange
  // then runs beside the preparation of A instead of behind it
  int prepared = 0, pulled = 0;
  while (prepared < 2 && prepared < P)
    if (stage_prep(s, prepared++)) return -1;
  long long wmax = 0;
  for (int p = 0; p < P; ++p) if (s->width[p] > wmax) wmax = s->width[p];
  if (my_rows > 0 &&
      eshkol_b200_prepare_a_f64_device(dA_rows, static_cast<uint64_t>(my_rows), static_cast<uint64_t>(s->K),
                                       static_cast<uint64_t>(wmax)) != 0)
    return fail(s, "prepare_a failed");
  for (int p = 0; p < P; ++p) {
    // An imported event's wait sees the most recent record the owner has CALLED, so this
    // barrier stands between every rank's calls of the records so far (the planes of the
    // panels staged up to here, the block of panel p - 1) and the peers' calls of their waits.
    if (barrier(s) != 0) return -1;
    // The planes of every panel staged so far are on their way: `ahead` panels beyond the one
    // being multiplied.  Two is the measured optimum on 8 GPUs (with three or four in flight
    // the step was slower there).
    while (pulled < prepared)
      if (pull_planes(s, pulled++)) return -1;
    if (my_rows > 0) {
      SH_CHECK(cudaStreamWaitEvent(lib, s->ev_arrived[p], 0));
      if (eshkol_b200_adopt_prepared_b(s->blk_p[p], static_cast<uint64_t>(s->K), static_cast<uint64_t>(s->width[p])) != 0)
        return fail(s, "adopt_prepared_b failed");
      EshkolB200GemmOpts o;
      memset(&o, 0, sizeof(o));
      o.ldc = s->N;
      double* c = static_cast<double*>(s->blk_c) + s->row0[R] * s->N + s->col0[p];
      if (eshkol_b200_multiply_prepared_f64_device(c, &o) != 0) return fail(s, "multiply failed");
    }
    SH_CHECK(cudaEventRecord(s->ev_block[R][p], lib));
    // behind the products of panel p: the shares of the panels up to p + ahead
    while (prepared < P && prepared <= p + ahead)
      if (stage_prep(s, prepared++)) return -1;
    // the blocks of the panel before this one, on streams of their own
    if (p >= 1 && gather_panel(s, p - 1)) return -1;
  }
  if (barrier(s) != 0) return -1;
  if (gather_panel(s, P - 1)) return -1;
  for (int i = 0; i < s->npool; ++i) {
    SH_CHECK(cudaStreamSynchronize(s->pool[i]));
    SH_CHECK(cudaStreamSynchronize(s->gpool[i]));
  }
  SH_CHECK(cudaStreamSynchronize(s->x1));
  SH_CHECK(cudaStreamSynchronize(s->x2));
  if (eshkol_b200_sync_status() != 0) return fail(s, "a kernel of the step reported a failure");
  // nobody overwrites a buffer a peer may still be reading
  return barrier(s);
}

int eshkol_b200_sharded_close(EshkolB200Sharded* s) {
  if (!s) return -1;
  cudaDeviceSynchronize();
  int rc = barrier(s);  // no peer still reads this rank's buffers
  for (int q = 0; q < s->world; ++q) {
    if (q == s->rank) continue;
    if (q == s->src && s->addr_b) cudaIpcCloseMemHandle(s->addr_b);
    if (s->addr_c[q]) cudaIpcCloseMemHandle(s->addr_c[q]);
    for (int p = 0; p < s->P; ++p) {
      if (s->addr_p[q][p]) cudaIpcCloseMemHandle(s->addr_p[q][p]);
      if (s->ev_planes[q][p]) cudaEventDestroy(s->ev_planes[q][p]);
      if (s->ev_block[q][p]) cudaEventDestroy(s->ev_block[q][p]);
    }
  }
  if (barrier(s) != 0) rc = -1;  // every mapping is closed before its owner frees the memory
  for (int p = 0; p < s->P; ++p) {
    if (s->blk_p[p]) eshkol_b200_mem_free(0, s->blk_p[p]);
    if (s->ev_planes[s->rank][p]) cudaEventDestroy(s->ev_planes[s->rank][p]);
    if (s->ev_block[s->rank][p]) cudaEventDestroy(s->ev_block[s->rank][p]);
    if (s->ev_got[p]) cudaEventDestroy(s->ev_got[p]);
    if (s->ev_arrived[p]) cudaEventDestroy(s->ev_arrived[p]);
  }
  if (s->blk_b) eshkol_b200_mem_free(0, s->blk_b);
  if (s->blk_c) eshkol_b200_mem_free(0, s->blk_c);
  for (int i = 0; i < kSlots; ++i) {
    if (s->bcol[i]) eshkol_b200_mem_free(0, s->bcol[i]);
    if (s->bcol_free[i]) cudaEventDestroy(s->bcol_free[i]);
  }
  if (s->x1) cudaStreamDestroy(s->x1);
  if (s->x2) cudaStreamDestroy(s->x2);
  for (int i = 0; i < s->npool; ++i) {
    if (s->pool[i]) cudaStreamDestroy(s->pool[i]);
    if (s->gpool[i]) cudaStreamDestroy(s->gpool[i]);
    if (s->ev_tmp[i]) cudaEventDestroy(s->ev_tmp[i]);
  }
  if (s->rank == 0) shm_unlink(s->name);
  munmap(s->ctl, sizeof(Ctl));
  delete s;
  cudaGetLastError();
  return rc;
}

}  // extern "C"
