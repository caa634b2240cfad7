// Exact float running sums over runs of EQUAL terms, for the value-class tail of top-p sampling.
//
// For 16-bit logits the probability is a function of the logit's bit pattern, so the sorted
// candidate list of sample_topp (extension/llm/sampler/sampler.cpp:136-170) is a sequence of
// runs: `count` copies of one float p per value class, classes in descending order. The
// reference adds them one by one (`cumulative_prob += probindex[i].prob`, sampler.cpp:151 and
// `cdf += ...`, :165). With the running sum written as N * ulp inside a binade (exact_math.cuh),
// a run of equal terms advances N by a constant per copy -- except that an exact half-way
// term rounds by the parity of N on its FIRST copy only, since a tie always leaves N even.
// So a run has a closed-form two-parity summary, and the copy at which N reaches a limit is a
// division.
//
// Everything here compiles both as CUDA device code and as plain host C++.
#pragma once

#include "exact_math.cuh"

namespace etb200 {

// Per-copy increments of N for `p` in binade kb: *first is the increment of the first copy for
// an even (index 0) and an odd (index 1) N in front of the run, *rest the increment of every
// later copy. Saturated at kSeqSat.
ETB_HD void rep_increments(float p, int kb, int first[2], int* rest) {
  if (kb >= 27 && kb <= 252) {
    // p / ulp by one exact multiplication with a power of two (as seq_push_scaled)
    float t = p * seq_inv_u(kb);
    t = t < 67108864.0f ? t : 67108864.0f;  // 2^26 == kSeqSat
#if defined(__CUDA_ARCH__)
    const float m = rintf(t);
#else
    const float m = nearbyintf(t);
#endif
    const float d = t - m;
    const int mi = (int)m;
    if (d != 0.5f && d != -0.5f) {
      first[0] = first[1] = mi;
      *rest = mi;
    } else {
      const int q = d > 0.0f ? mi : mi - 1;  // floor(t)
      first[0] = q + (q & 1);
      first[1] = q + ((q + 1) & 1);
      *rest = q + (q & 1);
    }
    return;
  }
  int q, cls;
  seq_quantize(p, kb, &q, &cls);
  if (cls != 1) {
    const int c = q >= kSeqSat ? kSeqSat : q + (cls >> 1);
    first[0] = first[1] = c;
    *rest = c;
  } else {
    // exact tie: round half to even. N even: N + q is odd iff q is odd. N odd: iff q is even.
    first[0] = q + (q & 1);
    first[1] = q + ((q + 1) & 1);
    *rest = q + (q & 1);  // N is even after a tie
  }
}

ETB_HD int rep_clamp(long long v) { return v > (long long)kSeqSat ? kSeqSat : (int)v; }

// Summary of `count` copies of p appended to a sum in binade kb.
ETB_HD SeqSummary rep_summary(float p, int count, int kb) {
  SeqSummary s;
  seq_identity(&s);
  if (count <= 0) return s;
  int first[2], rest;
  rep_increments(p, kb, first, &rest);
  const long long tail = (long long)rest * (long long)(count - 1);
  s.a0 = rep_clamp((long long)first[0] + tail);
  s.a1 = rep_clamp((long long)first[1] + tail);
  return s;
}

// The smallest N at which a sum in binade kb exceeds thr, clipped to [0, 2^24]: 0 when thr lies
// below the binade, 2^24 when no value of the binade exceeds it.
ETB_HD int thr_limit(float thr, int kb) {
  if (!(thr >= 0.0f)) return 0;  // negative (or NaN) threshold: any sum exceeds it (or none; see caller)
  const int kt = seq_kb(thr);
  if (kt < kb) return 0;
  if (kt > kb) return kSeqLimit;
  return seq_n(thr) + 1;  // at most 2^24
}

// The first copy j (1-based, j <= count) after which N >= limit, given N = n in front of the run;
// 0 when no copy of the run gets there. *n_before is N in front of that copy.
ETB_HD int rep_locate(int n, float p, int count, int kb, int limit, int* n_before) {
  *n_before = n;
  if (count <= 0) return 0;
  int first[2], rest;
  rep_increments(p, kb, first, &rest);
  const long long n1 = (long long)n + (long long)first[n & 1];
  if (n1 >= (long long)limit) return 1;
  if (rest <= 0 || count < 2) return 0;
  // 0 < limit - n1 <= 2^24 and rest <= 2^26: 32-bit arithmetic holds all of it
  const unsigned need = (unsigned)((long long)limit - n1);
  const unsigned more = (need + (unsigned)rest - 1u) / (unsigned)rest;  // copies after the first
  if (more > (unsigned)(count - 1)) return 0;
  *n_before = (int)n1 + (int)(more - 1u) * rest;  // < limit <= 2^24
  return (int)(1u + more);
}

struct WalkState {
  int kb;  // binade of the running sum
  int n;   // its significand: sum = seq_value(kb, n)
};

// Consumes copies of p up to and including the first one after which N >= thr_limit(thr, kb)
// or N leaves the binade; that copy is added with a real float addition, so the state after it
// is exact whichever happened. The caller has established (seq_apply on rep_summary) that such
// a copy exists among `count`. Returns the number of copies consumed; *found says whether the
// sum then exceeds thr, *cum is the sum.
ETB_HD int class_hit_step(WalkState* st, float p, int count, float thr, bool* found, float* cum) {
  const int limit = thr_limit(thr, st->kb);
  int n_before;
  int j = rep_locate(st->n, p, count, st->kb, limit, &n_before);
  if (j == 0) {
    // the caller's premise does not hold: the whole run stays below the limit. Consume all of
    // it; the last copy is still added for real, so the state stays exact.
    j = count;
    n_before = seq_apply(st->n, rep_summary(p, count - 1, st->kb));
  }
  const float before = seq_value(st->kb, n_before);
#if defined(__CUDA_ARCH__)
  const float after = __fadd_rn(before, p);
#else
  const float after = before + p;
#endif
  *cum = after;
  *found = after > thr;
  st->kb = seq_kb(after);
  st->n = seq_n(after);
  return j;
}

// Order-preserving 16-bit key of an IEEE half or bfloat16 pattern: larger value, larger key
// (-0 directly below +0; NaN patterns beyond the infinities).
ETB_HD uint32_t key_of_pattern16(uint32_t b) {
  return (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
}
ETB_HD uint32_t pattern_of_key16(uint32_t k) {
  return (k & 0x8000u) ? (k & 0x7FFFu) : (~k & 0xFFFFu);
}

}  // namespace etb200
