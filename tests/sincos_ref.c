/* CPU restatement of the branch-free sine / cosine of the Tiled broadcast kernel (cutile.jl_b200/csrc/tiled.cu,
 * sincos_reduced): the same sequence of f32 operations, every fmaf one rounding.  Test infrastructure: the tests
 * build it with the constants read from the kernel source (-DP1=... and so on), measure its distance from the exact
 * value over strided sweeps of all arguments, and compare the GPU's results with it bit for bit.
 * Build: gcc -O2 -mfma -ffp-contract=off -shared -fPIC (the fused multiply-add must be a real one). */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float asf(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t asu(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float sincos_reduced(float x, int want_cos) {
  const float ax = fabsf(x);
  float jf = fmaf(ax, TWO_OVER_PI, MAGIC);
  uint32_t q = asu(jf);
  jf -= MAGIC;
  float r = fmaf(jf, -(P1), ax);
  r = fmaf(jf, -(P2), r);
  r = fmaf(jf, -(P3), r);
  if (want_cos) q += 1;
  const float s = r * r;
  const int odd = q & 1;
  float p = fmaf(s, odd ? C2 : S2, odd ? C1 : S1);
  p = fmaf(s, p, odd ? C0 : S0);
  const float pp = odd ? fmaf(s, p, -0.5f) : p;
  const float u = odd ? s : s * r, v = odd ? 1.0f : r;
  const float res = fmaf(u, pp, v);
  uint32_t sign = (q & 2) << 30;
  if (!want_cos) sign ^= asu(x) & 0x80000000u;
  return asf(asu(res) ^ sign);
}

void sincos_ref(const float* x, float* y, long n, int want_cos) {
  for (long i = 0; i < n; ++i) y[i] = sincos_reduced(x[i], want_cos);
}

/* Largest error in units of the last place of the exact value over the f32 bit patterns first, first + step, ...
 * up to last (non-negative arguments; the scheme is symmetric). */
double sincos_max_ulp(uint32_t first, uint32_t last, uint32_t step, int want_cos) {
  double worst = 0;
  for (uint64_t u = first; u <= last; u += step) {
    const float x = asf((uint32_t)u);
    const long double exact = want_cos ? cosl((long double)x) : sinl((long double)x);
    const float got = sincos_reduced(x, want_cos), exf = (float)exact;
    double ulp;
    if (exf == 0.0f) {
      ulp = got == exf ? 0 : 1e9;
    } else {
      int e;
      frexp((double)exf, &e);
      double one = ldexp(1.0, e - 24);
      if (one < 0x1p-149) one = 0x1p-149;
      ulp = fabs((double)got - (double)exact) / one;
    }
    if (ulp > worst) worst = ulp;
  }
  return worst;
}
