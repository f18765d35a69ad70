// Device math that rounds like the CPU program's libm calls, for GPTOSS_EXACT.
#pragma once

#include <stdint.h>

namespace gptoss {

// T[i] = bits(2^(i/32) as a double) - (i << 47), i = 0..31: the table of the published
// algorithm (Arm Optimized Routines / glibc exp2f_data, N = 32).  tests/test_abi_and_host.py
// recomputes every entry from 2^(i/32) at 60 decimal digits; the GPU tests hold the function
// built on it to the C library's expf on a dense sweep.
__device__ static const unsigned long long kExp2Tab32[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};

// expf as glibc 2.39 computes it on x86-64 CPUs that have FMA (the published
// algorithm of Arm Optimized Routines' expf, glibc
// sysdeps/ieee754/flt-32/e_expf.c): with N = 32,
//   z = x * N/ln2;  k = round(z);  r = z - k;
//   2^(k/N) from a 32-entry table plus an exponent shift;
//   2^(r/N) ~ 1 + c2 r + (c1 + c0 r) r^2   (cubic, coefficients pre-divided by N^j);
// all in double, rounded to float once.  The reference's GPU engine relies on
// the same restatement (kernels/exact_math.hpp:8-52) for its bit-exact path.
//
// The inputs with a result of their own: |x| >= 88, infinities, NaN.
__device__ __forceinline__ bool glibc_expf_special(float x, float *result) {
  const uint32_t bits = __float_as_uint(x);
  const uint32_t top = (bits >> 20) & 0x7ffu;
  if (top < (0x42b00000u >> 20))
    return false;
  if (bits == 0xff800000u) {
    *result = 0.0f; // exp(-inf)
    return true;
  }
  if (top >= (0x7f800000u >> 20)) {
    *result = x + x; // +inf or NaN
    return true;
  }
  if (x > 0x1.62e42ep6f) {
    *result = __int_as_float(0x7f800000); // overflow
    return true;
  }
  if (x < -0x1.9fe368p6f) {
    *result = 0.0f; // underflow
    return true;
  }
  return false;
}

// entry_of(i) returns table entry i (0..31).  With kSpecialsLast it is called exactly once by
// every thread, before any branch on x, so it may be a warp shuffle of entries that the lanes
// hold; the special inputs then replace the polynomial's result afterwards.  Otherwise they
// leave early, as in the C library.
template <bool kSpecialsLast, class Lookup>
__device__ __forceinline__ float glibc_expf_with(float x, Lookup entry_of) {
  const double kScale = 0x1.71547652b82fep+0 * 32.0; // N / ln 2
  const double kRound = 0x1.8p+52;                   // adding it rounds to an integer
  const double c0 = 0x1.c6af84b912394p-5 / 32768.0;
  const double c1 = 0x1.ebfce50fac4f3p-3 / 1024.0;
  const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;

  float special;
  if constexpr (!kSpecialsLast)
    if (glibc_expf_special(x, &special))
      return special;
  const double z = __dmul_rn(kScale, (double)x);
  double kd = __dadd_rn(z, kRound);
  // k sits in the low bits of kd's mantissa.  Table entry + (k << 47) only ever changes the
  // high word (the low 32 bits of k << 47 are zero, so nothing carries), and only k's low 17
  // bits survive the shift: the 64-bit add is a 32-bit add of k << 15 to the high word.
  const uint32_t k_lo = (uint32_t)__double2loint(kd);
  kd = __dsub_rn(kd, kRound);
  const double r = __dsub_rn(z, kd);
  const unsigned long long entry = entry_of(k_lo & 31u);
  const double s = __hiloint2double((int)((uint32_t)(entry >> 32) + (k_lo << 15)), (int)(uint32_t)entry);
  const double hi = __fma_rn(c0, r, c1);
  double y = __fma_rn(c2, r, 1.0);
  y = __fma_rn(hi, __dmul_rn(r, r), y);
  const float out = (float)__dmul_rn(y, s);
  if constexpr (kSpecialsLast)
    if (glibc_expf_special(x, &special))
      return special;
  return out;
}

__device__ __forceinline__ float glibc_expf(float x) {
  return glibc_expf_with<false>(x, [](uint32_t i) { return kExp2Tab32[i]; });
}

} // namespace gptoss
