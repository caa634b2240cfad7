// Arithmetic of the cluster-per-row sampling kernel that is shared with its host-side
// unit test: how one thread summarises its 32 consecutive terms of a row before the exact
// running sum in front of them is known, and how one thread afterwards replays the row's
// exact sequential float sum (sampler.cpp:199-203) from those summaries.
//
// The sum `float s = 0; for (i) s += e[i];` is order dependent, but while s stays inside one
// binade each addition is an integer increment of its significand (exact_math.cuh). A cheap,
// slightly inaccurate prefix sum tells every chunk of 32 terms in which binade the running sum
// will be when the chunk is reached -- to within a relative margin (binade_margin) -- so every
// chunk can be turned into integer increments for that binade (or for the two binades that
// the margin leaves open) by its own thread, all chunks at once. What remains sequential is a
// walk over the few "event" chunks: those with two candidate binades (one of them holds the
// addition that leaves the binade and is redone with real float additions), those whose own
// terms span more than two binades (the start of a row), and those that hold an exact
// half-way term (their increment depends on the parity of the running significand). The walk
// applies only exact operations and checks every assumption it uses, so its result is either
// the reference's sum bit for bit or "not decided" (the caller then takes another route);
// the estimate only decides how often the latter happens.
//
// Everything here compiles both as CUDA device code and as plain host C++.
#pragma once

#include "exact_math.cuh"

namespace etb200 {

constexpr int kCTerms = 32;  // consecutive terms per chunk (one thread's share of a slice)
#ifndef ETB_MARGIN_PER_TERM
#define ETB_MARGIN_PER_TERM 1.4901161e-8f  // 2^-26
#endif
constexpr float kMarginPerTerm = ETB_MARGIN_PER_TERM;

// Relative margin around the estimated running sum inside which the true (sequentially
// rounded) running sum is assumed to lie when `terms` terms have been added. Every addition
// is off by at most half a unit of the last place of a sum that only grows, i.e. by at most
// 2^-24 of the current sum, so terms * 2^-24 bounds the deviation from the exact sum; the
// margin used is a quarter of that bound (softmax rows stay below a tenth of it: their
// deviation is mostly the terms that are too small to move the sum at all), plus a constant
// for the error of the estimate itself (approximate exponentials, a float prefix sum). A row
// that breaks the assumption is noticed by the walk and left undecided, never mis-summed.
ETB_HD float binade_margin(long long terms) {
  return (float)(terms + 64) * kMarginPerTerm + 2.0e-5f;
}

constexpr unsigned kEvTail = 1u;  // closes the list of one slice: carries only the prefix behind it
constexpr unsigned kEvLo = 2u;    // (a0lo, a1lo) summarise the chunk in binade klo
constexpr unsigned kEvHi = 4u;    // (a0hi, a1hi) summarise the chunk in binade klo + 1
constexpr unsigned kEvZero = 8u;  // every term of the chunk is zero: it changes no sum
// The chunk holds an exact half-way term for binade klo / klo + 1: its increment depends on the
// parity of the running significand. The chunk is staged, and resolve_tie_event() forms the
// two-parity summary from the staged terms before the walk (many such chunks side by side).
constexpr unsigned kEvTieLo = 16u;
constexpr unsigned kEvTieHi = 32u;

// One event chunk as the walk sees it. `xbefore` is the sum of the integer increments of the
// non-event chunks of the same slice in front of this chunk (event chunks contribute 0), so
// the difference of two consecutive events' xbefore is the increment of the run of ordinary
// chunks between them; that run is summarised in the binade klo of the event in front of it
// (a chunk whose binade differs from its predecessor's is always an event). `pool` is the slot
// in which the chunk's 32 terms are staged for the walk (chunks that may have to be added term
// by term, or whose summary is still pending), or -1.
struct alignas(16) ChunkEvent {
  int a0lo, a1lo, a0hi, a1hi;
  unsigned long long xbefore;
  short klo;
  short pool;
  unsigned short flags;
  unsigned short pad;
};

// Candidate binades of the running sum across a chunk, from the estimated sums in front of
// and behind it.
ETB_HD void chunk_binades(float p_in, float p_out, float margin, int* klo, int* khi) {
  *klo = seq_kb(p_in * (1.0f - margin));
  *khi = seq_kb(p_out * (1.0f + margin));
}

// A chunk can be summarised when at most two binades are open and the scaling 2^(150-k) is a
// normal float (exact_math.cuh); otherwise ("wild") its terms are staged and added one by one.
ETB_HD bool chunk_summarisable(int klo, int khi) { return khi - klo <= 1 && klo >= 27 && khi <= 252; }

// Increment of the significand for a chunk entered in binade k, assuming no exact half-way
// term: sum of round_half_even(e / u). *half is set when some term sits exactly half-way
// (then the caller must use chunk_summary_exact). Terms must be below 2^25 units, which holds
// for any chunk whose open binades include k or k - 1 (a term never exceeds the chunk's sum).
template <typename Arr>
ETB_HD int chunk_increment_fast(const Arr& e, int k, bool* half) {
  const float inv_u = seq_inv_u(k);
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  float md = 0.0f;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int j = 0; j < kCTerms; ++j) {
#if defined(__CUDA_ARCH__)
    const float t = __fmaf_rn(e[j], inv_u, 8388608.0f);  // 2^23 + round(e / u)
    const float q = __fsub_rn(t, 8388608.0f);
    const float d = __fmaf_rn(e[j], inv_u, -q);  // e / u - q, exact
    acc[j & 3] = __fadd_rn(acc[j & 3], q);
    md = fmaxf(md, fabsf(d));
#else
    const float t = fmaf(e[j], inv_u, 8388608.0f);
    const float q = t - 8388608.0f;
    const float d = fmaf(e[j], inv_u, -q);
    acc[j & 3] = acc[j & 3] + q;
    md = md > fabsf(d) ? md : fabsf(d);
#endif
  }
  // the partial sums are integers, exact below 2^24; a total at or beyond 2^24 only has to
  // stay there, which float addition of non-negative terms guarantees
  const float tot = (acc[0] + acc[1]) + (acc[2] + acc[3]);
  *half = !(md < 0.5f);  // also true for NaN
  return (int)(tot < 33554432.0f ? tot : 33554432.0f);
}

// The general two-parity summary of a chunk in binade k (27 <= k <= 252), term by term in row
// order.
ETB_HD SeqSummary chunk_summary_exact(const float* terms, int k) {
  SeqSummary s;
  seq_identity(&s);
  const float inv_u = seq_inv_u(k);
  for (int j = 0; j < kCTerms; ++j) seq_push_scaled(&s, terms[j], inv_u);
  return s;
}

// What one thread decides about its chunk from the tie-free increments: the flags of the
// chunk's record. `half_lo` / `half_hi`: chunk_increment_fast met an exact half-way term.
ETB_HD unsigned chunk_flags(int klo, int khi, bool half_lo, bool half_hi) {
  if (!chunk_summarisable(klo, khi)) return 0u;
  unsigned f = half_lo ? kEvTieLo : kEvLo;
  if (khi != klo) f |= half_hi ? kEvTieHi : kEvHi;
  return f;
}

// A chunk is an ordinary one (its increment simply adds to the run it is in) when it has one
// open binade and a tie-free summary for it; everything else is staged.
ETB_HD bool chunk_is_staged(unsigned flags) { return (flags & kEvZero) == 0u && flags != kEvLo; }

// Replaces the pending (kEvTieLo / kEvTieHi) summaries of one event by the exact two-parity
// summaries formed from its staged terms (row order). One thread per event.
ETB_HD void resolve_tie_event(ChunkEvent* ev, const float* terms) {
  unsigned f = ev->flags;
  if (f & kEvTieLo) {
    const SeqSummary s = chunk_summary_exact(terms, ev->klo);
    ev->a0lo = s.a0;
    ev->a1lo = s.a1;
    f = (f & ~kEvTieLo) | kEvLo;
  }
  if (f & kEvTieHi) {
    const SeqSummary s = chunk_summary_exact(terms, ev->klo + 1);
    ev->a0hi = s.a0;
    ev->a1hi = s.a1;
    f = (f & ~kEvTieHi) | kEvHi;
  }
  ev->flags = (unsigned short)f;
}

// The sequential replay. `events` holds the records of all slices; slice sl owns the
// n_events[sl] records from first_event[sl] on, in chunk order, the last of them a kEvTail
// record. `terms(slot, j)` returns term j of the chunk staged in pool slot `slot` (called for
// j = 0..31 in order, only for chunks that must be added term by term). Returns true with the exact sum in *sum, or
// false when some assumption did not hold (nothing is decided then).
template <typename Terms>
ETB_HD bool walk_events(const ChunkEvent* events, const int* first_event, const int* n_events,
                        int n_slices, int capacity, Terms terms, float* sum) {
  int k = 1, n = 0;  // the running sum, as (binade, significand): zero
  int run_k = -1;    // binade in which the ordinary chunks behind the previous event are summarised
  for (int sl = 0; sl < n_slices; ++sl) {
    unsigned long long x_prev = 0ull;
    const int ne = n_events[sl], e0 = first_event[sl];
    if (ne < 1 || e0 < 0 || e0 + ne > capacity) return false;
    const ChunkEvent* ev = events + e0;
    for (int i = 0; i < ne; ++i) {
      const ChunkEvent r = ev[i];
      const unsigned long long gap = r.xbefore - x_prev;
      x_prev = r.xbefore;
      if (gap != 0ull) {
        // a run of ordinary chunks, summarised in binade run_k: valid only if the sum is in that
        // binade now and still is behind the run
        if (run_k != k || gap >= (unsigned long long)kSeqLimit) return false;
        n += (int)gap;
        if (n >= kSeqLimit) return false;
      }
      if (r.flags & kEvTail) continue;
      run_k = r.klo;
      if (r.flags & kEvZero) continue;
      SeqSummary sm;
      bool have = false;
      if ((r.flags & kEvLo) && k == r.klo) {
        sm.a0 = r.a0lo;
        sm.a1 = r.a1lo;
        have = true;
      } else if ((r.flags & kEvHi) && k == r.klo + 1) {
        sm.a0 = r.a0hi;
        sm.a1 = r.a1hi;
        have = true;
      }
      if (have) {
        const int n2 = seq_apply(n, sm);
        if (n2 < kSeqLimit) {
          n = n2;
          continue;
        }
      }
      // the chunk leaves the binade (or was never summarised for it): real float additions
      if (r.pool < 0) return false;
      float s = seq_value(k, n);
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
      for (int j = 0; j < kCTerms; ++j) {
        const float t = terms((int)r.pool, j);
#if defined(__CUDA_ARCH__)
        s = __fadd_rn(s, t);
#else
        s = s + t;
#endif
      }
      if (!(s < 3.0e38f)) return false;  // overflow or NaN: not a sum this walk can carry
      k = seq_kb(s);
      n = seq_n(s);
    }
  }
  *sum = seq_value(k, n);
  return true;
}

}  // namespace etb200
