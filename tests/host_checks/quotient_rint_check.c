/* Host check of the division-free quantisation quotient used by the device glue (quotient_rint / dynq_byte in
 * oxionnx_b200/csrc/kernels_glue.cu): q = x*r corrected once with the exact remainder, rounded with the
 * 1.5 * 2^23 addend, and redone with the IEEE division whenever q is within 2^-13 of a tie or |q| >= 1024.
 * The result must equal rintf(x / s) for every operand pair; the operands are concentrated on ties, their
 * neighbours, exact integers, tiny values and the ends of the supported scale range.
 * Usage: quotient_rint_check SCALES PER_SCALE  -> prints "total N bad M slow K", exit status 1 when M > 0. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static uint64_t state = 88172645463325252ull;
static uint64_t rnd(void) {
  state ^= state << 13;
  state ^= state >> 7;
  state ^= state << 17;
  return state;
}
static float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static long slow = 0;

static float quotient_rint(float x, float s, float r) {
  const float q0 = x * r;
  const float q = fmaf(fmaf(-s, q0, x), r, q0);
  if (fabsf(q) < 1024.0f) {
    volatile float t = q + 12582912.0f;
    const float ri = t - 12582912.0f;
    if (fabsf(q - ri) <= 0.49987793f) return ri;
  }
  slow++;
  return rintf(x / s);
}

int main(int argc, char** argv) {
  const long scales = argc > 1 ? atol(argv[1]) : 2000, per = argc > 2 ? atol(argv[2]) : 2000;
  long bad = 0, total = 0;
  for (long si = 0; si < scales; ++si) {
    const int e = (int)(rnd() % 201) - 100; /* 2^-100 .. 2^100 */
    const float s = ldexpf(1.0f + (float)(rnd() & 0x7fffff) / 8388608.0f, e);
    const float r = 1.0f / s; /* correctly rounded, as __frcp_rn and the host division give */
    for (long t = 0; t < per; ++t) {
      float x;
      const int mode = (int)(t & 3);
      if (mode == 0) { /* around a tie */
        const int k = (int)(rnd() % 2200) - 1100;
        x = ((float)k + 0.5f) * s;
        x = u2f(f2u(x) + (uint32_t)((int)(rnd() % 9) - 4));
      } else if (mode == 1) { /* uniform quotient */
        x = ((float)(rnd() % 1000000) / 1000000.0f * 2400.f - 1200.f) * s;
      } else if (mode == 2) { /* tiny */
        x = ldexpf((float)(rnd() & 0xffff), e - 40 - (int)(rnd() % 40));
        if (rnd() & 1) x = -x;
      } else { /* exact integers and their neighbours */
        const int k = (int)(rnd() % 2200) - 1100;
        x = (float)k * s;
        x = u2f(f2u(x) + (uint32_t)((int)(rnd() % 5) - 2));
      }
      total++;
      const float want = rintf(x / s);
      const float got = quotient_rint(x, s, r);
      if (!(got == want) && !(got != got && want != want)) { /* both NaN (an overflowed operand) counts as equal */
        if (bad < 10) printf("mismatch x=%a s=%a got=%g want=%g\n", x, s, got, want);
        bad++;
      }
    }
  }
  printf("total %ld bad %ld slow %ld\n", total, bad, slow);
  return bad != 0;
}
