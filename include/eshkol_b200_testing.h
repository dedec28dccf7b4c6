/*
 * Test hooks of libeshkol_gpu_b200.so.  Not part of the installed interface: a host
 * runtime includes eshkol_gpu_memory_b200.h (and eshkol_b200_ext.h if it keeps tensors on
 * the device); only the test suite includes this file.
 */
#ifndef ESHKOL_B200_TESTING_H
#define ESHKOL_B200_TESTING_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Tests only: copy one intermediate of the LAST Ozaki-II GEMM to host memory.
 * what: 0 mu (int32[M])          1 nu (int32[N])
 *       2 A residues, modulus 256 plane   3 A residues, odd plane `index` (0-based)
 *       4 B residues, modulus 256 plane   5 B residues, odd plane `index`
 *       6 products mod 256: sum of chunk residues mod 512, ties as +128 (int16); 12 its flip bits
 *       7 product residues, odd plane `index` (int8)
 *       8 / 9 A flags (+128, odd)   10 / 11 B flags (+128, odd): uint16 units, 64 per chunk
 * info[0..5] receive rows, row pitch (elements), element size, n_chunks, last
 * segment length, bytes copied.  Synchronises the stream. */
int eshkol_b200_debug_fetch(int what, int index, void* host_dst, uint64_t capacity_bytes,
                            uint64_t info[6]);

/* Tests only: the tier and parameter eshkol_gpu_matmul_f64 would select for this
 * shape from the current environment.  Touches no GPU. */
void eshkol_b200_debug_choose_tier(uint64_t M, uint64_t K, uint64_t N, int* tier, int* param);

/* Tests only: one slot of the selector's time model (0 = the full-precision kernel, 1..8 = the
 * slice tiers), and one measurement fed to it as a finished GEMM would feed it. */
void eshkol_b200_debug_gemm_model(int idx, double* overhead_ns, double* peak_gflops);
void eshkol_b200_debug_gemm_calibrate(int idx, double work_flop, double measured_ns);

/* Tests only: the wait limit of every bounded wait inside the kernels, in nanoseconds
 * (0 restores the default of two seconds), and a switch that makes the next products launch
 * withhold one producer arrival so that its waits run out.  The kernel then returns by itself
 * with a status code, which eshkol_b200_sync_status reports once and clears. */
void eshkol_b200_debug_set_wait_limit_ns(unsigned long long ns);
void eshkol_b200_debug_withhold_arrival(int on);

/* Tests only: the nth device allocation the library makes from now on fails as if the device
 * were out of memory (0 switches the hook off).  The call that needed it must fail loudly --
 * -1, or NaN from a void dispatcher -- and the library must stay usable. */
void eshkol_b200_debug_fail_allocation(int nth);

/* Tests only, no GPU: the plan a multi-GPU session of N columns would follow -- its column
 * panels (first column, width; at most `capacity` of them) and every rank's share of each
 * panel's columns (first[p * world + r], count[p * world + r]) when the source rank's share is
 * src_weight of the others'.  Returns the number of panels, -1 on bad arguments. */
int eshkol_b200_debug_sharded_plan(uint64_t N, int world, int src, double src_weight, int capacity,
                                   uint64_t* col0, uint64_t* width, uint64_t* first, uint64_t* count);

/* Tests only: the rendezvous and the host barriers of a multi-GPU session
 * (eshkol_b200_multi.h) without any GPU work.  Every rank runs `barriers` barriers; a rank given
 * fail_at = k marks the session failed instead of entering barrier k, a rank given leave_at = k
 * leaves silently before it.  Returns 0, or -1 as soon as one of this rank's barriers gives up
 * (a failed peer: at once; a missing peer: after timeout_s). */
int eshkol_b200_debug_rendezvous(const char* name, int rank, int world, int barriers, int fail_at, int leave_at,
                                 double timeout_s);

#ifdef __cplusplus
}
#endif

#endif /* ESHKOL_B200_TESTING_H */
