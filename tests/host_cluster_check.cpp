// Host model of the cluster-per-row kernel's exact sum
// (executorch_b200/csrc/cluster_math.cuh): the row is cut into slices (one per thread block of
// a cluster), every slice into chunks of 32 terms (one per thread); chunks are classified from
// an inexact prefix sum and summarised independently of each other, exactly as the kernel's
// threads do, the event records are laid out as the kernel lays them out, and the same
// walk_events() the kernel runs replays the sum. Compiled by tests/test_cluster_math.py with
// g++ and compared with a plain sequential float loop. No GPU involved.
#include <cstdint>
#include <cstring>
#include <vector>

#include "../executorch_b200/csrc/cluster_math.cuh"

using namespace etb200;

extern "C" {

// stats[0] events in all, [1] staged chunks in all, [2] largest event count of a slice,
// [3] largest staged count of a slice, [4] chunks with an exact half-way term.
// Returns 1 when the walk decided the sum (then *sum is it), 0 when it did not, -1 when the
// event list overflowed (the kernel takes the other route in both of the latter cases).
int hc_cluster_sum(const float* e, long n, int n_slices, int ev_cap, float perturb, float* sum,
                   long* stats) {
  const long slice_len = ((n + (long)n_slices * kCTerms - 1) / ((long)n_slices * kCTerms)) * kCTerms;
  std::vector<ChunkEvent> events(ev_cap);
  std::vector<int> n_events(n_slices, 0), first_event(n_slices, 0);
  std::vector<float> pool;  // staged chunks, kCTerms floats each
  int total = 0;  // records handed out so far (the kernel: one atomic add per slice)
  bool overflow = false;
  double prefix = 0.0;  // the estimate: a plain double sum, optionally perturbed
  for (int i = 0; i < 5; ++i) stats[i] = 0;
  for (int sl = 0; sl < n_slices; ++sl) {
    const long base = (long)sl * slice_len;
    const long len = base >= n ? 0 : (n - base < slice_len ? n - base : slice_len);
    const int chunks = (int)((len + kCTerms - 1) / kCTerms);
    unsigned long long x = 0ull;
    int ne = 0, np = 0;
    int prev_klo = -1;
    first_event[sl] = total;
    for (int c = 0; c < chunks; ++c) {
      float t[kCTerms];
      double csum = 0.0;
      for (int j = 0; j < kCTerms; ++j) {
        const long i = base + (long)c * kCTerms + j;
        t[j] = i < n ? e[i] : 0.0f;
        csum += t[j];
      }
      const float p_in = (float)(prefix * (1.0 + perturb));
      prefix += csum;
      const float p_out = (float)(prefix * (1.0 + perturb));
      int klo, khi;
      chunk_binades(p_in, p_out, binade_margin(base + (long)(c + 1) * kCTerms), &klo, &khi);
      // as a thread of the kernel: tie-free increments for the open binade(s), then the flags
      bool half_lo = false, half_hi = false;
      int inc_lo = 0, inc_hi = 0;
      if (chunk_summarisable(klo, khi)) {
        inc_lo = chunk_increment_fast(t, klo, &half_lo);
        if (khi != klo) inc_hi = chunk_increment_fast(t, khi, &half_hi);
      }
      unsigned flags = chunk_flags(klo, khi, half_lo, half_hi);
      const bool zero = csum == 0.0;
      if (zero) flags = kEvLo | kEvHi | kEvZero;
      const bool staged = chunk_is_staged(flags);
      const bool event = c == 0 || klo != prev_klo || staged;
      prev_klo = klo;
      if (flags & (kEvTieLo | kEvTieHi)) ++stats[4];
      if (!event) {
        x += (unsigned long long)inc_lo;
        continue;
      }
      ChunkEvent r;
      memset(&r, 0, sizeof(r));
      r.a0lo = r.a1lo = inc_lo;
      r.a0hi = r.a1hi = inc_hi;
      r.xbefore = x;
      r.klo = (short)klo;
      r.pool = -1;
      r.flags = (unsigned short)flags;
      if (staged) {
        r.pool = (short)(pool.size() / kCTerms);
        pool.insert(pool.end(), t, t + kCTerms);
        ++np;
      }
      if (total + ne < ev_cap) events[total + ne] = r; else overflow = true;
      ++ne;
    }
    ChunkEvent tail;
    memset(&tail, 0, sizeof(tail));
    tail.xbefore = x;
    tail.pool = -1;
    tail.flags = (unsigned short)kEvTail;
    if (total + ne < ev_cap) events[total + ne] = tail; else overflow = true;
    ++ne;
    n_events[sl] = ne;
    total += ne;
    stats[0] += ne;
    stats[1] += np;
    if (ne > stats[2]) stats[2] = ne;
    if (np > stats[3]) stats[3] = np;
  }
  if (overflow) return -1;
  if (pool.size() / kCTerms > 32767) return -1;
  // the pending two-parity summaries (in the kernel: one thread per event, side by side)
  for (int i = 0; i < total; ++i) {
    ChunkEvent& r = events[i];
    if (r.flags & (kEvTieLo | kEvTieHi)) resolve_tie_event(&r, &pool[(size_t)r.pool * kCTerms]);
  }
  auto terms = [&](int slot, int j) { return pool[(size_t)slot * kCTerms + j]; };
  return walk_events(events.data(), first_event.data(), n_events.data(), n_slices, ev_cap, terms, sum) ? 1 : 0;
}

// e[i] = expf_ref(x[i] * inv_t - max) for a row of float logits (the row's terms as the
// sampler forms them), so that the test can feed realistic rows.
void hc_row_terms(const float* x, long n, float inv_t, float* e) {
  ExpTable tab;
  make_exp_table(&tab);
  float mx = -INFINITY;
  for (long i = 0; i < n; ++i) {
    const float v = x[i] * inv_t;
    if (v > mx) mx = v;
  }
  for (long i = 0; i < n; ++i) e[i] = expf_ref(x[i] * inv_t - mx, tab.t);
}

}  // extern "C"
