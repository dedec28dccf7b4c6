// TEST INFRASTRUCTURE ONLY.  The reference's CUDA backend (lib/backend/gpu/gpu_memory_cuda.cpp
// in the reference project) imports eshkol_batch_matmul_f64 from the runtime
// (lib/core/runtime_tensor_math.cpp:796), a file that needs the whole tensor runtime.  This
// stand-in supplies the symbol so the backend links on its own: matrix by matrix through the
// reference's own eshkol_matmul_f64, which is compiled into the same library.
#include <cstdint>

extern "C" void eshkol_matmul_f64(const double*, const double*, double*, uint64_t, uint64_t, uint64_t);

extern "C" void eshkol_batch_matmul_f64(const double* a, const double* b, double* c, int64_t batch, int64_t M,
                                        int64_t K, int64_t N) {
  for (int64_t i = 0; i < batch; ++i)
    eshkol_matmul_f64(a + i * M * K, b + i * K * N, c + i * M * N, (uint64_t)M, (uint64_t)K, (uint64_t)N);
}
