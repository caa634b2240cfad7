// Arithmetic shared by the sampling kernels and by their host-side unit tests.
//
// The reference sampler (extension/llm/sampler/sampler.cpp) is sequential scalar code, so
// its result is defined by the exact IEEE-754 value of every intermediate: expf() of each
// shifted logit (sampler.cpp:201), the float sum accumulated in index order
// (sampler.cpp:199-203), the float cumulative probabilities accumulated in sorted order
// (sampler.cpp:151-170). The kernels reproduce those values bit for bit with the two
// building blocks in this file:
//
//  * expf_ref(): the float exponential as glibc computes it (table of 2^(i/32) in double,
//    cubic polynomial in double, one final rounding to float). Restated from the published
//    algorithm (S. Nagy, "new single precision math functions", glibc >= 2.27); checked
//    exhaustively on the host against libm for every float in [-104.5, -0.0].
//  * the seqsum_* functions: a data-parallel way to get the exact result of
//    `float s = 0; for (i...) s += v[i];` for non-negative v.
//
// Everything here compiles both as CUDA device code and as plain host C++.
#pragma once

#include <stdint.h>
#include <string.h>

#include <cmath>

#if defined(__CUDACC__)
#define ETB_HD __host__ __device__ __forceinline__
#else
#define ETB_HD inline
#endif

namespace etb200 {

ETB_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
#endif
}

ETB_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  memcpy(&f, &u, 4);
  return f;
#endif
}

// ---------------------------------------------------------------------------------------
// expf as the reference's libm computes it.
//
// exp(x) = 2^(k/32) * 2^(r/32) with k = round(x * 32/ln2), r = x*32/ln2 - k in
// [-1/2, 1/2]; 2^(k/32) comes from a 32-entry table (exponent folded in with integer
// arithmetic), 2^(r/32) from a cubic. The products that glibc's x86-64 build fuses into
// FMAs are fused here too (that choice is what makes the result bit-identical).
// ---------------------------------------------------------------------------------------
constexpr int kExpTableBits = 5;
constexpr int kExpTableSize = 1 << kExpTableBits;

// 2^(i/32) as IEEE double bits with i << 47 subtracted from the bit pattern, so that
// adding (k << 47) installs the exponent floor(k/32) and leaves the mantissa of 2^((k%32)/32).
// Filled by make_exp_table(); the kernels keep a copy in shared memory.
struct ExpTable {
  uint64_t t[kExpTableSize];
};

// Host only.
inline void make_exp_table(ExpTable* out) {
  for (int i = 0; i < kExpTableSize; ++i) {
    // exp2l on long double is accurate far beyond double's 53 bits, so the cast to double
    // is the correctly rounded value of 2^(i/32).
    long double v = exp2l((long double)i / (long double)kExpTableSize);
    double d = (double)v;
    uint64_t u;
    memcpy(&u, &d, 8);
    out->t[i] = u - ((uint64_t)i << (52 - kExpTableBits));
  }
}

// Polynomial for 2^(r/32) - 1 on |r| <= 1/2, and 32/ln2. Hexadecimal literals of the
// published coefficient set, pre-divided by 32^3, 32^2, 32.
#define ETB_EXP_C0 0x1.c6af84b912394p-20
#define ETB_EXP_C1 0x1.ebfce50fac4f3p-13
#define ETB_EXP_C2 0x1.62e42ff0c52d6p-6
#define ETB_EXP_INVLN2N 0x1.71547652b82fep+5
#define ETB_EXP_SHIFT 0x1.8p+52

// x must be <= 0 (or NaN): the sampler only ever evaluates exp(logit - max).
ETB_HD float expf_ref(float x, const uint64_t* __restrict__ table) {
  // below this bound the float result underflows to +0 (libm returns 0 there)
  if (x < -0x1.9fe368p6f) return 0.0f;
#if defined(__CUDA_ARCH__)
  const double xd = (double)x;
  const double z = __dmul_rn(ETB_EXP_INVLN2N, xd);
  double kd = __dadd_rn(z, ETB_EXP_SHIFT);
  const uint64_t ki = (uint64_t)__double_as_longlong(kd);
  kd = __dadd_rn(kd, -ETB_EXP_SHIFT);
  const double r = __fma_rn(ETB_EXP_INVLN2N, xd, -kd);
  const uint64_t tb = table[ki & (kExpTableSize - 1)] + (ki << (52 - kExpTableBits));
  const double s = __longlong_as_double((long long)tb);
  const double p = __fma_rn(ETB_EXP_C0, r, ETB_EXP_C1);
  const double r2 = __dmul_rn(r, r);
  double y = __fma_rn(ETB_EXP_C2, r, 1.0);
  y = __fma_rn(p, r2, y);
  y = __dmul_rn(y, s);
  return __double2float_rn(y);
#else
  const double xd = (double)x;
  const double z = ETB_EXP_INVLN2N * xd;
  double kd = z + ETB_EXP_SHIFT;
  uint64_t ki;
  memcpy(&ki, &kd, 8);
  kd -= ETB_EXP_SHIFT;
  const double r = fma(ETB_EXP_INVLN2N, xd, -kd);
  const uint64_t tb = table[ki & (kExpTableSize - 1)] + (ki << (52 - kExpTableBits));
  double s;
  memcpy(&s, &tb, 8);
  const double p = fma(ETB_EXP_C0, r, ETB_EXP_C1);
  const double r2 = r * r;
  double y = fma(ETB_EXP_C2, r, 1.0);
  y = fma(p, r2, y);
  y = y * s;
  return (float)y;
#endif
}

// ---------------------------------------------------------------------------------------
// Exact emulation of a sequential float sum of non-negative terms.
//
// While the running sum s stays inside one binade, s = N * u with u = ulp(s) and N an
// integer below 2^24, and `s += v` is N += round_half_even(v / u), where the only
// dependence on N is the parity that breaks an exact half-way tie. A run of terms is
// therefore summarised by two integers (the increment of N for an even and for an odd
// start); summaries compose associatively, so a block-wide scan yields the exact N in
// front of every thread's chunk. The first chunk in which N would reach 2^24 (the sum
// leaves the binade, so the rounding unit changes) is re-done with real float additions
// by its owning thread; everything after it is re-summarised in the new binade.
//
// "Binade" index used here: kb = max(biased exponent of s, 1), so zero, subnormals and
// the first normal binade share u = 2^-149, and N is the 24-bit significand.
// ---------------------------------------------------------------------------------------
constexpr int kSeqSat = 1 << 26;   // saturated increment: any value >= 2^24 means "left the binade"
constexpr int kSeqLimit = 1 << 24; // N must stay below this

struct SeqSummary {
  int a0;  // increment of N when the chunk is entered with N even
  int a1;  // increment of N when the chunk is entered with N odd
};

ETB_HD int seq_kb(float s) {
  int e = (int)((f32_bits(s) >> 23) & 0xFF);
  return e == 0 ? 1 : e;
}

ETB_HD int seq_n(float s) {
  uint32_t b = f32_bits(s);
  uint32_t m = b & 0x7FFFFFu;
  return (int)(((b >> 23) & 0xFF) ? (m | 0x800000u) : m);
}

// Inverse of (seq_kb, seq_n) for n < 2^24.
ETB_HD float seq_value(int kb, int n) {
  if (n < 0x800000) {
    // only the lowest binade holds values without the implicit bit; elsewhere a running sum
    // never drops below 2^23 units, so this is kb == 1 (or a zero sum)
    return bits_f32((uint32_t)n);
  }
  return bits_f32(((uint32_t)kb << 23) | ((uint32_t)n & 0x7FFFFFu));
}

// v >= 0 finite. Splits v / u into floor q (saturated) and the position of the remainder
// relative to one half: cls 0 below, 1 exactly half, 2 above.
ETB_HD void seq_quantize(float v, int kb, int* q, int* cls) {
  const uint32_t b = f32_bits(v);
  int e = (int)(b >> 23);
  uint32_t m = b & 0x7FFFFFu;
  if (e == 0) {
    e = 1;
  } else {
    m |= 0x800000u;
  }
  // v = m * 2^(e-150), u = 2^(kb-150)  =>  v/u = m * 2^(e-kb)
  const int sh = e - kb;
  if (sh >= 0) {
    *cls = 0;
    if (m == 0) {
      *q = 0;
    } else if (sh >= 3) {
      *q = kSeqSat;
    } else {
      *q = (int)(m << sh);  // < 2^27
      if (*q > kSeqSat) *q = kSeqSat;
    }
  } else {
    const int rs = -sh;
    if (rs >= 25) {
      *q = 0;
      *cls = 0;
    } else {
      *q = (int)(m >> rs);
      const uint32_t rem = m & ((1u << rs) - 1u);
      const uint32_t half = 1u << (rs - 1);
      *cls = rem > half ? 2 : (rem == half ? 1 : 0);
    }
  }
}

ETB_HD void seq_identity(SeqSummary* s) {
  s->a0 = 0;
  s->a1 = 0;
}

// Appends one term to a chunk summary.
ETB_HD void seq_push(SeqSummary* s, float v, int kb) {
  int q, cls;
  seq_quantize(v, kb, &q, &cls);
  if (cls != 1) {
    const int inc = q + (cls >> 1);
    s->a0 += inc;
    s->a1 += inc;
  } else {
    // exact tie: round to even, which depends on the parity of N + q
    s->a0 += q;
    s->a0 += (s->a0 & 1);
    s->a1 += q;
    s->a1 += ((s->a1 + 1) & 1);
  }
  if (s->a0 > kSeqSat) s->a0 = kSeqSat;
  if (s->a1 > kSeqSat) s->a1 = kSeqSat;
}

// Fast variant for the common case kb >= 27 (s >= 2^-100) and v <= 2: the quotient is formed
// with one exact float multiply by a power of two. Same result as seq_push.
ETB_HD void seq_push_scaled(SeqSummary* s, float v, float inv_u) {
  float t = v * inv_u;  // exact unless it underflows, where it is far below 1/2 anyway
  t = t < 67108864.0f ? t : 67108864.0f;  // 2^26 == kSeqSat
#if defined(__CUDA_ARCH__)
  const float m = rintf(t);
#else
  const float m = nearbyintf(t);
#endif
  const float d = t - m;
  const int mi = (int)m;
  if (d != 0.5f && d != -0.5f) {
    s->a0 += mi;
    s->a1 += mi;
  } else {
    const int q = (d > 0.0f) ? mi : mi - 1;  // floor(t)
    s->a0 += q;
    s->a0 += (s->a0 & 1);
    s->a1 += q;
    s->a1 += ((s->a1 + 1) & 1);
  }
  if (s->a0 > kSeqSat) s->a0 = kSeqSat;
  if (s->a1 > kSeqSat) s->a1 = kSeqSat;
}

// Tie-free fast variant of seq_push_scaled: adds round_half_even(v / u) to *acc and
// multiplies *tie_prod by (|rounding error| - 1/2), which is exactly zero when v / u lies
// half-way between two integers (then the caller must redo the chunk with the two-parity
// functions, because the result depends on the parity of N). A product that underflows to
// zero without a real tie only costs that redo. v / u is clamped to 2^24; any chunk
// containing a term of 2^23 or more leaves the binade anyway, so its sum only has to stay
// at or above 2^24, which float addition of non-negative terms guarantees; below 2^24 every
// partial sum is an integer that a float holds exactly. `inv_u24` is 2^-24 / u.
//
// Seven float multiplies and adds and nothing else: on the GPU the integer/compare pipe is
// the scarce one, so neither the sum nor the tie test touches it. (The scaling by 2^24
// folds into the two fused multiply-adds, whose product is exact.)
ETB_HD void seq_push_fast(float* acc, float* tie_prod, float v, float inv_u24) {
#if defined(__CUDA_ARCH__)
  const float c = __saturatef(__fmul_rn(v, inv_u24));
  const float tm = __fmaf_rn(c, 16777216.0f, 8388608.0f);  // 2^23: rounds c * 2^24 to an integer
  const float r = __fsub_rn(tm, 8388608.0f);
  const float d = __fmaf_rn(c, 16777216.0f, -r);
  *acc = __fadd_rn(*acc, r);
  *tie_prod = __fmul_rn(*tie_prod, __fsub_rn(fabsf(d), 0.5f));
#else
  float c = v * inv_u24;
  c = c < 0.0f ? 0.0f : (c > 1.0f ? 1.0f : c);
  if (!(c == c)) c = 0.0f;  // the device's saturating multiply turns NaN into 0
  const float t = c * 16777216.0f;
  const float tm = t + 8388608.0f;
  const float r = tm - 8388608.0f;
  const float d = t - r;
  *acc = *acc + r;
  *tie_prod = *tie_prod * (fabsf(d) - 0.5f);
#endif
}

// 2^(126 - kb): 2^-24 / u as a float, representable for kb in [27, 252].
ETB_HD float seq_inv_u24(int kb) {
  return bits_f32((uint32_t)(126 - kb + 127) << 23);
}

// 2^(150 - kb) as a float when representable as a normal number (kb in [24, 150+126]); the
// caller uses seq_push_scaled only for kb >= 27.
ETB_HD float seq_inv_u(int kb) {
  return bits_f32((uint32_t)(150 - kb + 127) << 23);
}

// Summary of "a, then b".
ETB_HD SeqSummary seq_compose(SeqSummary a, SeqSummary b) {
  SeqSummary c;
  c.a0 = a.a0 + ((a.a0 & 1) ? b.a1 : b.a0);
  c.a1 = a.a1 + (((a.a1 + 1) & 1) ? b.a1 : b.a0);
  if (c.a0 > kSeqSat) c.a0 = kSeqSat;
  if (c.a1 > kSeqSat) c.a1 = kSeqSat;
  return c;
}

// N after a run summarised by s, entered with N = n.
ETB_HD int seq_apply(int n, SeqSummary s) {
  const int inc = (n & 1) ? s.a1 : s.a0;
  const int r = n + inc;
  return r > kSeqSat ? kSeqSat : r;
}

}  // namespace etb200
