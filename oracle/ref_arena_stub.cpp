// TEST INFRASTRUCTURE ONLY.  Three-function stand-in for the reference runtime's
// arena so that its CPU matmul translation unit (lib/backend/blas_backend.cpp in
// the reference project) links on its own.  Only the symbols that file imports
// are provided; plain malloc backs them and nothing is ever freed (the matmul
// path itself never allocates; only its backward / tensor-helper code does).
#include <cstdint>
#include <cstdlib>

struct ref_stub_tensor {
  uint64_t* dimensions;
  uint64_t num_dimensions;
  int64_t* elements;
  uint64_t total_elements;
  int32_t dtype;
};

extern "C" {
void* get_global_arena(void) { static int token; return &token; }
void* arena_allocate(void* arena, size_t size) { (void)arena; return std::malloc(size ? size : 1); }
void* arena_allocate_tensor_full(void* arena, uint64_t num_dims, uint64_t total_elements) {
  (void)arena;
  ref_stub_tensor* t = (ref_stub_tensor*)std::calloc(1, sizeof(ref_stub_tensor));
  if (!t) return nullptr;
  t->dimensions = (uint64_t*)std::calloc(num_dims ? num_dims : 1, sizeof(uint64_t));
  t->elements = (int64_t*)std::calloc(total_elements ? total_elements : 1, sizeof(int64_t));
  t->num_dimensions = num_dims;
  t->total_elements = total_elements;
  return t;
}
}
