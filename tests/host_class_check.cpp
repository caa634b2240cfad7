// Host model of the value-class tail's walk (class_math.cuh): runs of equal terms, summarised
// per run, composed per group of runs as the kernel's threads do, searched for the first copy
// at which the running float sum exceeds a threshold. Checked against the plain loop.
#include <stdint.h>

#include <vector>

#include "../executorch_b200/csrc/class_math.cuh"

using namespace etb200;

extern "C" {

// the reference's loop: cum += p, stop at the first cum > thr. Returns 1 when it stopped.
int hcc_brute(const float* p, const int* count, int n_classes, float thr, float* cum, long* pos) {
  volatile float c = 0.0f;
  long k = 0;
  for (int i = 0; i < n_classes; ++i) {
    for (int j = 0; j < count[i]; ++j) {
      c = c + p[i];
      if (c > thr) {
        *cum = c;
        *pos = k;
        return 1;
      }
      ++k;
    }
  }
  *cum = c;
  *pos = k;
  return 0;
}

// the kernel's scheme: tiles of `threads * per_thread` classes; rounds inside a tile
int hcc_walk(const float* p, const int* count_in, int n_classes, float thr, int threads, int per_thread,
             float* cum, long* pos, long* rounds) {
  std::vector<int> count(count_in, count_in + n_classes);
  WalkState st;
  st.kb = 1;
  st.n = 0;
  long consumed = 0;
  *rounds = 0;
  const int tile = threads * per_thread;
  for (int t0 = 0; t0 < n_classes; t0 += tile) {
    for (;;) {
      ++*rounds;
      // per thread: composed summary of its classes
      std::vector<SeqSummary> mine(threads);
      std::vector<long> cnt(threads);
      for (int t = 0; t < threads; ++t) {
        seq_identity(&mine[t]);
        cnt[t] = 0;
        for (int j = 0; j < per_thread; ++j) {
          const int b = t0 + t * per_thread + j;
          if (b >= n_classes) break;
          mine[t] = seq_compose(mine[t], rep_summary(p[b], count[b], st.kb));
          cnt[t] += count[b];
        }
      }
      const int limit = thr_limit(thr, st.kb);
      SeqSummary pre;
      seq_identity(&pre);
      long pre_cnt = 0;
      int hit_t = -1, hit_b = -1, n_at = 0;
      long cnt_at = 0;
      for (int t = 0; t < threads && hit_t < 0; ++t) {
        int n_cur = seq_apply(st.n, pre);
        long before = pre_cnt;
        for (int j = 0; j < per_thread; ++j) {
          const int b = t0 + t * per_thread + j;
          if (b >= n_classes) break;
          if (count[b] <= 0) continue;
          const int n_after = seq_apply(n_cur, rep_summary(p[b], count[b], st.kb));
          if (n_after >= limit) {
            hit_t = t;
            hit_b = b;
            n_at = n_cur;
            cnt_at = before;
            break;
          }
          n_cur = n_after;
          before += count[b];
        }
        pre = seq_compose(pre, mine[t]);
        pre_cnt += cnt[t];
      }
      if (hit_t < 0) {
        st.n = seq_apply(st.n, pre);
        consumed += pre_cnt;
        break;
      }
      WalkState s2;
      s2.kb = st.kb;
      s2.n = n_at;
      bool found;
      float c;
      int j = class_hit_step(&s2, p[hit_b], count[hit_b], thr, &found, &c);
      while (!found && j < count[hit_b]) {  // the same run through further binades, as the kernel does
        const int rest = count[hit_b] - j;
        if (seq_apply(s2.n, rep_summary(p[hit_b], rest, s2.kb)) < thr_limit(thr, s2.kb)) break;
        j += class_hit_step(&s2, p[hit_b], rest, thr, &found, &c);
      }
      const long hit_pos = consumed + cnt_at + j - 1;
      if (found) {
        *cum = c;
        *pos = hit_pos;
        return 1;
      }
      st = s2;
      consumed = hit_pos + 1;
      for (int b = t0; b < hit_b; ++b) count[b] = 0;
      count[hit_b] -= j;
    }
  }
  *cum = seq_value(st.kb, st.n);
  *pos = consumed;
  return 0;
}

uint32_t hcc_key(uint32_t pattern) { return key_of_pattern16(pattern); }
uint32_t hcc_pattern(uint32_t key) { return pattern_of_key16(key); }

}  // extern "C"
