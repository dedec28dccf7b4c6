// Residue helpers shared by the split kernels of every Ozaki tier.
#pragma once
#include <stdint.h>

namespace b200 {

constexpr double kRoundMagic = 6755399441055744.0;  // 1.5 * 2^52

// Centred residue of an integer-valued double |x| < 2^53 modulo odd p, in
// [-(p-1)/2, (p-1)/2].  The reference evaluates x - p*rint(x*(1/p)) in f64
// (lib/backend/gpu/gpu_memory.mm:2580); for odd p only the residue class reaches
// the result, so the canonical representative (which always fits int8) is used.
__device__ __forceinline__ int residue_odd(double x, double p, double p_inv, int pi) {
  const double t = fma(x, p_inv, kRoundMagic);
  const double q = t - kRoundMagic;          // x/p rounded to an integer, off by at most 1
  const double r = fma(-p, q, x);            // exact, |r| <= p/2 + 1
  int ri = __double2loint(r + kRoundMagic);  // low mantissa word = r in two's complement
  const int h = pi >> 1;
  ri = (ri > h) ? ri - pi : ri;
  ri = (ri < -h) ? ri + pi : ri;
  return ri;
}

struct Res256 {
  uint32_t lo8, hi, odd;  // a (mod 256) as a byte, 16*[a == +128], 16*[a odd]
};
// Modulus 256: the reference's x - 256*rint(x/256) is exact; its value is the
// centred residue with the half-even tie rule, +128 iff x = 128 (mod 512).  +128
// does not fit int8: it is carried as the byte -128 plus a flag (times 16).
__device__ __forceinline__ Res256 residue_256(double x) {
  const long long xi = static_cast<long long>(x);
  const uint32_t x512 = static_cast<uint32_t>(xi) & 511u;
  Res256 r;
  r.lo8 = x512 & 255u;
  r.hi = (x512 == 128u) ? 16u : 0u;
  r.odd = (x512 & 1u) ? 16u : 0u;
  return r;
}

}  // namespace b200
