/*
 * Exact fp32 division by a divisor shared across many elements.
 *
 * The quantize kernels divide every element by a scale that is constant over a row, a
 * tensor or a 16-element block.  IEEE division per element costs ~10 instructions; the
 * quantize kernels are HBM-bound only if the per-element instruction count stays low.
 * With y = RN(1/d) computed once per divisor, the quotient is recovered as
 *     q0 = RN(a * y);  r = fma(d, q0, -a)  (exact);  q = fma(-r, y, q0)
 * which equals RN(a / d) whenever no intermediate under/overflows (Markstein's
 * correction step).  `b200q_div_fast_ok` states the divisor range where that holds for
 * every quotient that can influence an E4M3 / E2M1 code (|q| >= 2^-10); outside it the
 * callers fall back to a true division.
 *
 * The header compiles as plain C for the host-side check that compares this sequence
 * with `a / d` on hundreds of millions of operand pairs, and as CUDA for the kernels.
 */
#ifndef B200Q_EXACT_DIV_H_
#define B200Q_EXACT_DIV_H_

#include <stdint.h>

#if defined(__CUDACC__)
#define B200Q_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#include <string.h>
#define B200Q_HD static inline
#endif

B200Q_HD uint32_t b200q_f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}

/* Biased exponent of d in [37, 227]: 1/d is normal, and for any numerator whose
 * quotient is >= 2^-10 the residual a - d*q0 is exactly representable. */
B200Q_HD int b200q_div_fast_ok(float d) {
  uint32_t e = (b200q_f32_bits(d) >> 23) & 0xffu;
  return e >= 37u && e <= 227u;
}

B200Q_HD float b200q_rcp_rn(float d) {
#if defined(__CUDA_ARCH__)
  return __frcp_rn(d);
#else
  return 1.0f / d;
#endif
}

/* a finite (either sign, zeros included), d > 0 with b200q_div_fast_ok(d), y = b200q_rcp_rn(d),
 * |a / d| < 2^127.  The residual is formed as r = d*q0 - a and subtracted again, which is the
 * same arithmetic as the textbook a - d*q0 but keeps the sign of a zero numerator:
 * a = -0 gives q0 = -0, r = +0, q = (-0)*y + (-0) = -0. */
B200Q_HD float b200q_div_by_shared(float a, float d, float y) {
#if defined(__CUDA_ARCH__)
  float q0 = __fmul_rn(a, y);
  float r = __fmaf_rn(d, q0, -a);
  return __fmaf_rn(-r, y, q0);
#else
  float q0 = a * y;
  volatile float r = fmaf(d, q0, -a); /* volatile: keeps the host compiler from folding the
                                         negation below into the fma above, which would lose
                                         the sign of a zero numerator */
  return fmaf(-r, y, q0);
#endif
}

#endif /* B200Q_EXACT_DIV_H_ */
