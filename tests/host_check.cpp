// Host build of the arithmetic shared with the CUDA kernels
// (executorch_b200/csrc/exact_math.cuh), arranged exactly as the kernels arrange it:
// `threads` simulated threads, each owning `chunk` consecutive terms per tile, chunk
// summaries composed in thread order, the first chunk that leaves the binade redone with
// real float additions. Compiled by tests/test_exact_math.py with g++ and compared with a
// plain sequential float loop. No GPU involved.
#include <cstdint>
#include <vector>

#include "../executorch_b200/csrc/exact_math.cuh"

using namespace etb200;

namespace {

// One tile, as seqsum_tile in sampler_kernels.cu. Returns true on a search hit.
bool tile(const float* v, int threads, int chunk, float& s, bool search, float thr, int pos0,
          int limit, int* hit_pos, float* hit_sum, long* iterations, bool force_generic) {
  int consumed = 0;
  std::vector<SeqSummary> mine(threads), pre(threads);
  while (true) {
    ++*iterations;
    const int kb = seq_kb(s);
    const int n_s = seq_n(s);
    for (int t = 0; t < threads; ++t) {
      seq_identity(&mine[t]);
      if (t >= consumed) {
        if (kb >= 27 && kb <= 252 && !force_generic) {
          // as the kernel: tie-free fast path first, two-parity redo of the chunk on a tie
          const float inv_u24 = seq_inv_u24(kb);
          float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, t4[4] = {1.0f, 1.0f, 1.0f, 1.0f};
          for (int j = 0; j < chunk; ++j) seq_push_fast(&a4[j & 3], &t4[j & 3], v[t * chunk + j], inv_u24);
          const float accf = (a4[0] + a4[1]) + (a4[2] + a4[3]);
          const float tie_prod = (t4[0] * t4[1]) * (t4[2] * t4[3]);
          const int acc = (int)(accf < 33554432.0f ? accf : 33554432.0f);
          mine[t].a0 = mine[t].a1 = acc;
          if (!(tie_prod != 0.0f)) {
            const float inv_u = seq_inv_u(kb);
            seq_identity(&mine[t]);
            for (int j = 0; j < chunk; ++j) seq_push_scaled(&mine[t], v[t * chunk + j], inv_u);
          }
        } else {
          for (int j = 0; j < chunk; ++j) seq_push(&mine[t], v[t * chunk + j], kb);
        }
        if (mine[t].a0 > (1 << 25)) mine[t].a0 = 1 << 25;
        if (mine[t].a1 > (1 << 25)) mine[t].a1 = 1 << 25;
      }
    }
    SeqSummary run;
    seq_identity(&run);
    for (int t = 0; t < threads; ++t) {
      pre[t] = run;
      run = seq_compose(run, mine[t]);
    }
    int first = threads;
    int first_n_in = 0;
    for (int t = consumed; t < threads; ++t) {
      const int n_in = seq_apply(n_s, pre[t]);
      const int n_out = seq_apply(n_in, mine[t]);
      bool flag = n_out >= kSeqLimit;
      if (search && n_out < kSeqLimit && seq_value(kb, n_out) > thr) flag = true;
      if (flag) {
        first = t;
        first_n_in = n_in;
        break;
      }
    }
    if (first == threads) {
      s = seq_value(kb, seq_apply(n_s, run));
      return false;
    }
    float acc = seq_value(kb, first_n_in);
    bool found = false;
    for (int j = 0; j < chunk; ++j) {
      acc = acc + v[first * chunk + j];
      const int pos = pos0 + first * chunk + j;
      if (search && !found && acc > thr && pos < limit) {
        found = true;
        *hit_pos = pos;
        *hit_sum = acc;
      }
    }
    s = acc;
    if (found) return true;
    consumed = first + 1;
    if (consumed >= threads) return false;
  }
}

}  // namespace

extern "C" {

void hc_expf(const float* x, float* y, long n) {
  ExpTable tab;
  make_exp_table(&tab);
  for (long i = 0; i < n; ++i) y[i] = expf_ref(x[i], tab.t);
}

// The host libm's expf, vectorised for tests that compare the device function with it.
void hc_libm_expf(const float* x, float* y, long n) {
  for (long i = 0; i < n; ++i) y[i] = expf(x[i]);
}

// Number of floats with bit patterns lo, lo+step, ... <= hi (negative floats: larger pattern =
// more negative) whose expf_ref differs from the host libm's expf.
long hc_expf_mismatches(uint32_t lo, uint32_t hi, uint32_t step) {
  ExpTable tab;
  make_exp_table(&tab);
  long bad = 0;
  for (uint64_t b = lo; b <= hi; b += step) {
    const float x = bits_f32((uint32_t)b);
    const float a = expf(x), m = expf_ref(x, tab.t);
    if (f32_bits(a) != f32_bits(m)) ++bad;
  }
  return bad;
}

// Sum of v[0..n) in the block arrangement. iterations counts scan rounds over all tiles.
float hc_seqsum(const float* v, long n, int threads, int chunk, int force_generic, long* iterations) {
  const int tile_elems = threads * chunk;
  std::vector<float> buf(tile_elems);
  float s = 0.0f;
  long it = 0;
  // the kernels add the first terms sequentially (head), then go tile by tile
  const long head = force_generic == 2 ? 0 : (n < 256 ? n : 256);
  for (long i = 0; i < head; ++i) s = s + v[i];
  for (long base = head; base < n; base += tile_elems) {
    for (int i = 0; i < tile_elems; ++i) buf[i] = (base + i < n) ? v[base + i] : 0.0f;
    int hp;
    float hs;
    tile(buf.data(), threads, chunk, s, false, 0.0f, (int)base, (int)n, &hp, &hs, &it, force_generic != 0);
  }
  if (iterations) *iterations = it;
  return s;
}

// First position (< limit) after which the running sum exceeds thr; -1 if none, then *sum is
// the total of the terms below the limit.
long hc_search(const float* v, long n, long limit, float thr, int threads, int chunk, float* sum) {
  const int tile_elems = threads * chunk;
  std::vector<float> buf(tile_elems);
  float s = 0.0f;
  long it = 0;
  for (long base = 0; base < n; base += tile_elems) {
    for (int i = 0; i < tile_elems; ++i)
      buf[i] = (base + i < n && base + i < limit) ? v[base + i] : 0.0f;
    int hp;
    float hs;
    if (tile(buf.data(), threads, chunk, s, true, thr, (int)base, (int)limit, &hp, &hs, &it, false)) {
      *sum = hs;
      return hp;
    }
    if (base + tile_elems >= limit) break;
  }
  *sum = s;
  return -1;
}

}  // extern "C"
