// Residue helpers shared by the split kernels of every Ozaki tier.
#pragma once
#include <stdint.h>

namespace b200 {

constexpr double kRoundMagic = 6755399441055744.0;  // 1.5 * 2^52

// Residue of an integer-valued double |x| < 2^53 modulo odd p <= 255, as a value in
// [-128, 127] of the right class; xlo is x modulo 2^32.  The reference evaluates
// x - p*rint(x*(1/p)) in f64 (lib/backend/gpu/gpu_memory.mm:2580); for odd p only the
// residue CLASS reaches the result (the product's final reduction has no ties), so
// any representative that fits int8 serves.  q = x/p rounded to an integer comes out
// of one fused multiply-add against 1.5*2^52 (its low mantissa word is q modulo 2^32;
// q is off from the true nearest integer by at most 0.0052 because |x|/p * 2^-53 is),
// and r = x - p*q is formed modulo 2^32 in one integer multiply-add.  |r| <= 0.5052*p,
// i.e. within +-127 for p <= 253 and within +-128 for p = 255, where +128 is folded
// to -127.
template <bool kMay128>
__device__ __forceinline__ int residue_odd_t(double x, uint32_t xlo, double p_inv, int pi) {
  const uint32_t qlo = static_cast<uint32_t>(__double2loint(fma(x, p_inv, kRoundMagic)));
  int ri = static_cast<int>(xlo - static_cast<uint32_t>(pi) * qlo);
  if (kMay128) ri = (ri == 128) ? 128 - pi : ri;  // only p = 255 can reach +128
  return ri;
}
__device__ __forceinline__ int residue_odd(double x, uint32_t xlo, double p_inv, int pi) {
  return (pi == 255) ? residue_odd_t<true>(x, xlo, p_inv, pi) : residue_odd_t<false>(x, xlo, p_inv, pi);
}

// low bytes of four values -> one word (three byte-permutes instead of shifts and masks)
__device__ __forceinline__ uint32_t pack_bytes4(int r0, int r1, int r2, int r3) {
  const uint32_t lo = __byte_perm(static_cast<uint32_t>(r0), static_cast<uint32_t>(r1), 0x0040);
  const uint32_t hi = __byte_perm(static_cast<uint32_t>(r2), static_cast<uint32_t>(r3), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

struct Res256 {
  uint32_t lo8, hi, odd;  // a (mod 256) as a byte, [a == +128], [a odd]
};
// Modulus 256: the reference's x - 256*rint(x/256) is exact; its value is the
// centred residue with the half-even tie rule, +128 iff x = 128 (mod 512).  +128
// does not fit int8: it is carried as the byte -128 plus a flag bit.
__device__ __forceinline__ Res256 residue_256(uint32_t xlo) {
  const uint32_t x512 = xlo & 511u;
  Res256 r;
  r.lo8 = x512 & 255u;
  r.hi = (x512 == 128u) ? 1u : 0u;
  r.odd = x512 & 1u;
  return r;
}

// Parity of sum_k hi_a[k]*odd_b[k] + odd_a[k]*hi_b[k] over one chunk, from the 128-byte
// flag rows of the two operands.  This is bit 8 of the true chunk sum minus bit 8 of
// the sum formed with the int8 bytes alone: a = a8 + 256*[a = +128] gives
// a*b = a8*b8 + 256*([a=+128]*b + a8*[b=+128]) (mod 512), and 256*x depends on x mod 2.
__device__ __forceinline__ uint32_t chunk_flag_parity(const uint16_t* a_hi, const uint16_t* a_odd,
                                                      const uint16_t* b_odd, const uint16_t* b_hi) {
  const uint4* ah = reinterpret_cast<const uint4*>(a_hi);
  const uint4* ao = reinterpret_cast<const uint4*>(a_odd);
  const uint4* bo = reinterpret_cast<const uint4*>(b_odd);
  const uint4* bh = reinterpret_cast<const uint4*>(b_hi);
  uint32_t acc = 0;
#pragma unroll 2
  for (int w = 0; w < 8; ++w) {
    const uint4 x = __ldg(ah + w), y = __ldg(bo + w), z = __ldg(ao + w), t = __ldg(bh + w);
    acc ^= __popc(x.x & y.x) ^ __popc(x.y & y.y) ^ __popc(x.z & y.z) ^ __popc(x.w & y.w);
    acc ^= __popc(z.x & t.x) ^ __popc(z.y & t.y) ^ __popc(z.z & t.z) ^ __popc(z.w & t.w);
  }
  return acc & 1u;
}

// Epilogue activations: 0 none, 1 ReLU (x > 0 ? x : 0, lib/backend/gpu/gpu_cuda_kernels.cu:37),
// 2 the tanh-form GELU of the reference's feed-forward, written as its generated code computes
// it (lib/backend/tensor_transformer_codegen.cpp:2469-2577): tanh through exp(2u), each
// operation rounded on its own.  Like that code it returns NaN once exp(2u) overflows (u > 354).
__device__ __forceinline__ double apply_activation(double x, int activation) {
  if (activation == 1) return (x > 0.0) ? x : 0.0;
  if (activation == 2) {
    const double x3 = __dmul_rn(x, __dmul_rn(x, x));
    const double u = __dmul_rn(0.7978845608028654, __dadd_rn(x, __dmul_rn(0.044715, x3)));
    const double e = exp(__dmul_rn(2.0, u));
    const double t = __ddiv_rn(__dsub_rn(e, 1.0), __dadd_rn(e, 1.0));
    return __dmul_rn(0.5, __dmul_rn(x, __dadd_rn(1.0, t)));
  }
  return x;
}

}  // namespace b200
