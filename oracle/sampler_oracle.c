/*
 * TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C restatement of the algorithm of ExecuTorch's LLM token sampler,
 * extension/llm/sampler/sampler.cpp (v1.5.0), instantiated for T = float. Only tests,
 * the smoke check and the CPU-baseline leg of the benchmark may load it; the product
 * never calls into it.
 *
 * Pinning: this file is checked (a) against tokens produced by the reference's own,
 * unmodified sampler.cpp compiled in oracle/_ref (tests/golden holds such tokens with
 * the script that made them) and (b) against the argmax fixtures of the reference's own
 * tests (extension/llm/sampler/test/test_sampler.cpp:19-43,
 * extension/llm/runner/test/test_text_decoder_runner.cpp:83-140).
 *
 * Two deliberate choices, both documented where they apply:
 *  - 16-bit logits (Half, BFloat16) are upcast exactly to fp32 and sampled with the
 *    float algorithm, which is what the reference's newer runners do
 *    (examples/models/gemma4/runner/gemma4_runner.cpp:166-182,308).
 *  - The order of equal probabilities after the sort at sampler.cpp:148 is unspecified
 *    in the reference (std::sort). This file pins it to "probability descending, then
 *    token index ascending", i.e. what std::stable_sort does to the index-ascending
 *    candidate array of sampler.cpp:137-143.
 *
 * Build: gcc -std=c11 -O2 -ffp-contract=off (no fused multiply-add: the reference is
 * built for baseline x86-64, where every float operation rounds separately).
 * Third-party arithmetic underneath: libm expf (glibc 2.39 here), as in the reference
 * (sampler.cpp:201).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* ScalarType numbering, runtime/core/portable_type/scalar_type.h */
enum { ORACLE_HALF = 5, ORACLE_FLOAT = 6, ORACLE_BFLOAT16 = 15, ORACLE_UINT16 = 27 };

/* ---- xorshift64* coin: sampler.cpp:210-220 ---------------------------------------- */
uint32_t oracle_random_u32(uint64_t* state) {
  *state ^= *state >> 12;
  *state ^= *state << 25;
  *state ^= *state >> 27;
  return (uint32_t)((*state * 0x2545F4914F6CDD1Dull) >> 32);
}

float oracle_random_f32(uint64_t* state) {
  return (float)(oracle_random_u32(state) >> 8) / 16777216.0f;
}

/* ---- exact upcasts ---------------------------------------------------------------- */
float oracle_bf16_to_f32(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else { /* subnormal half: renormalise */
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while ((man & 0x400u) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7F800000u | (man << 13);
  } else {
    u = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* ---- sample_argmax: sampler.cpp:44-56 --------------------------------------------- */
/* Strict '>' keeps the lowest index among equal maxima; a NaN never replaces the
 * running maximum and a NaN at index 0 is never replaced. */
int32_t oracle_argmax_f32(const float* p, int32_t n) {
  int32_t max_i = 0;
  float max_p = p[0];
  for (int32_t i = 1; i < n; i++) {
    if (p[i] > max_p) {
      max_i = i;
      max_p = p[i];
    }
  }
  return max_i;
}

/* sample<uint16_t> with temperature 0 compares the raw 16-bit integers. */
int32_t oracle_argmax_u16(const uint16_t* p, int32_t n) {
  int32_t max_i = 0;
  uint16_t max_p = p[0];
  for (int32_t i = 1; i < n; i++) {
    if (p[i] > max_p) {
      max_i = i;
      max_p = p[i];
    }
  }
  return max_i;
}

/* ---- softmax: sampler.cpp:189-208 -------------------------------------------------- */
/* The sum is a float accumulated sequentially in index order; that rounding is part
 * of the reference's result and is reproduced on purpose. */
void oracle_softmax_f32(float* x, int32_t n) {
  float max_val = x[0];
  for (int32_t i = 1; i < n; i++) {
    if (x[i] > max_val) max_val = x[i];
  }
  float sum = 0;
  for (int32_t i = 0; i < n; i++) {
    x[i] = expf(x[i] - max_val);
    sum += x[i];
  }
  for (int32_t i = 0; i < n; i++) {
    x[i] /= sum;
  }
}

/* ---- sample_mult: sampler.cpp:58-70 ------------------------------------------------ */
int32_t oracle_sample_mult_f32(const float* p, int32_t n, float coin) {
  float cdf = 0.0f;
  for (int32_t i = 0; i < n; i++) {
    cdf += p[i];
    if (coin < cdf) return i;
  }
  return n - 1;
}

typedef struct {
  float prob;
  int32_t index;
} prob_index_t; /* ProbIndex<float>, sampler.h:31-35 */

static int cmp_desc_then_index(const void* a, const void* b) {
  const prob_index_t* x = (const prob_index_t*)a;
  const prob_index_t* y = (const prob_index_t*)b;
  if (x->prob > y->prob) return -1;
  if (x->prob < y->prob) return 1;
  return (x->index > y->index) - (x->index < y->index);
}

/* ---- sample_topp: sampler.cpp:122-171 ---------------------------------------------- */
/* Optional outputs describe the nucleus for diagnostics: n0 (candidates after the
 * cutoff crop), last_idx, and the fp32 cumulative probability at last_idx. */
int32_t oracle_sample_topp_f32(
    const float* p, int32_t n, float topp, float coin, int32_t* out_n0,
    int32_t* out_last_idx, float* out_cum) {
  prob_index_t* pi = (prob_index_t*)malloc(sizeof(prob_index_t) * (size_t)n);
  int32_t n0 = 0;
  const float cutoff = (1.0f - topp) / (float)(n - 1);
  for (int32_t i = 0; i < n; i++) {
    if (p[i] >= cutoff) {
      pi[n0].index = i;
      pi[n0].prob = p[i];
      n0++;
    }
  }
  qsort(pi, (size_t)n0, sizeof(prob_index_t), cmp_desc_then_index);
  float cumulative_prob = 0;
  int32_t last_idx = n0 - 1;
  for (int32_t i = 0; i < n0; i++) {
    cumulative_prob += pi[i].prob;
    if (cumulative_prob > topp) {
      last_idx = i;
      break;
    }
  }
  if (out_n0) *out_n0 = n0;
  if (out_last_idx) *out_last_idx = last_idx;
  if (out_cum) *out_cum = cumulative_prob;
  const float r = coin * cumulative_prob;
  float cdf = 0;
  int32_t result = -1;
  for (int32_t i = 0; i <= last_idx; i++) {
    cdf += pi[i].prob;
    if (r < cdf) {
      result = pi[i].index;
      break;
    }
  }
  if (result < 0) result = pi[last_idx].index; /* n0 == 0 is undefined in the reference too */
  free(pi);
  return result;
}

/* ---- sample_topk: sampler.cpp:72-120 ----------------------------------------------- */
/* std::partial_sort leaves ties unspecified as well; pinned like top-p. The sums are
 * float, accumulated over the k kept entries in sorted order. */
int32_t oracle_sample_topk_f32(const float* p, int32_t n, int32_t topk, float coin) {
  int32_t k = topk < n ? topk : n;
  if (k <= 0) return 0;
  prob_index_t* pi = (prob_index_t*)malloc(sizeof(prob_index_t) * (size_t)n);
  for (int32_t i = 0; i < n; i++) {
    pi[i].index = i;
    pi[i].prob = p[i];
  }
  qsort(pi, (size_t)n, sizeof(prob_index_t), cmp_desc_then_index);
  float topk_sum = 0.0f;
  for (int32_t i = 0; i < k; i++) topk_sum += pi[i].prob;
  const float r = coin * topk_sum;
  float cdf = 0.0f;
  int32_t result = pi[k - 1].index;
  for (int32_t i = 0; i < k; i++) {
    cdf += pi[i].prob;
    if (r < cdf) {
      result = pi[i].index;
      break;
    }
  }
  free(pi);
  return result;
}

/* ---- Sampler state and Sampler::sample<float>: sampler.cpp:173-187, 222-251 -------- */
typedef struct {
  int32_t vocab_size;
  float inv_temperature;
  float topp;
  int32_t topk;
  uint64_t rng_state;
} oracle_sampler_t;

void oracle_sampler_init(
    oracle_sampler_t* s, int32_t vocab_size, float temperature, float topp,
    uint64_t rng_seed) {
  s->vocab_size = vocab_size;
  /* static_cast<bool>(temperature) ? 1.0f / temperature : 0 — no clamping in the ctor */
  s->inv_temperature = (temperature != 0.0f) ? 1.0f / temperature : 0.0f;
  s->topp = topp;
  s->topk = 0;
  s->rng_state = rng_seed;
}

/* set_temperature, sampler.h:48-53: negative values are reset to 0 */
void oracle_sampler_set_temperature(oracle_sampler_t* s, float temperature) {
  if (temperature < 0.0f) temperature = 0.0f;
  s->inv_temperature = (temperature != 0.0f) ? 1.0f / temperature : 0.0f;
}

/* Mutates logits exactly like the reference (scaled, then probabilities). */
int32_t oracle_sampler_sample_f32(oracle_sampler_t* s, float* logits) {
  const int32_t n = s->vocab_size;
  if (s->inv_temperature == 0.0f) {
    return oracle_argmax_f32(logits, n);
  }
  for (int32_t q = 0; q < n; q++) logits[q] *= s->inv_temperature;
  oracle_softmax_f32(logits, n);
  float coin = oracle_random_f32(&s->rng_state);
  if (s->topk > 0 && s->topk < n) {
    return oracle_sample_topk_f32(logits, n, s->topk, coin);
  } else if (s->topp <= 0 || s->topp >= 1) {
    return oracle_sample_mult_f32(logits, n, coin);
  }
  return oracle_sample_topp_f32(logits, n, s->topp, coin, 0, 0, 0);
}

/* ---- batched driver: one fresh sampler per row, rows striped over threads ---------- */
typedef struct {
  const void* logits;
  int dtype;
  int64_t rows;
  int32_t vocab;
  int64_t stride;
  float temperature, topp;
  int32_t topk;
  uint64_t* states; /* in: seed per row; out: state after the draw */
  int32_t* out;
  int tid, nthreads;
  double seconds; /* time spent in sample() only */
} job_t;

static double now_s(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

static void* job_main(void* arg) {
  job_t* j = (job_t*)arg;
  float* buf = (float*)malloc(sizeof(float) * (size_t)j->vocab);
  for (int64_t r = j->tid; r < j->rows; r += j->nthreads) {
    oracle_sampler_t s;
    oracle_sampler_init(&s, j->vocab, j->temperature, j->topp, j->states[r]);
    s.topk = j->topk;
    if (j->dtype == ORACLE_UINT16) {
      /* sample<uint16_t>: only the temperature-0 comparison of raw integers is meaningful */
      const uint16_t* p = (const uint16_t*)j->logits + j->stride * r;
      j->out[r] = oracle_argmax_u16(p, j->vocab);
      continue;
    }
    if (j->dtype == ORACLE_FLOAT) {
      memcpy(buf, (const float*)j->logits + j->stride * r, sizeof(float) * (size_t)j->vocab);
    } else {
      const uint16_t* p = (const uint16_t*)j->logits + j->stride * r;
      if (j->dtype == ORACLE_BFLOAT16) {
        for (int32_t i = 0; i < j->vocab; i++) buf[i] = oracle_bf16_to_f32(p[i]);
      } else {
        for (int32_t i = 0; i < j->vocab; i++) buf[i] = oracle_f16_to_f32(p[i]);
      }
    }
    double t0 = now_s();
    j->out[r] = oracle_sampler_sample_f32(&s, buf);
    j->seconds += now_s() - t0;
    j->states[r] = s.rng_state;
  }
  free(buf);
  return 0;
}

/* Returns the time spent inside the sample() calls summed over threads; *wall gets the
 * elapsed time of the whole call. states[r] is the seed on entry, the advanced state on
 * return. */
double oracle_sample_rows(
    const void* logits, int dtype, int64_t rows, int32_t vocab, int64_t row_stride_elems,
    float temperature, float topp, int32_t topk, uint64_t* states, int32_t* out_tokens,
    int nthreads, double* wall) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads > 256) nthreads = 256;
  job_t jobs[256];
  pthread_t th[256];
  double w0 = now_s();
  for (int t = 0; t < nthreads; t++) {
    job_t j = {logits, dtype, rows, vocab, row_stride_elems, temperature, topp,
               topk, states, out_tokens, t, nthreads, 0.0};
    jobs[t] = j;
  }
  if (nthreads == 1) {
    job_main(&jobs[0]);
  } else {
    for (int t = 0; t < nthreads; t++) pthread_create(&th[t], 0, job_main, &jobs[t]);
    for (int t = 0; t < nthreads; t++) pthread_join(th[t], 0);
  }
  if (wall) *wall = now_s() - w0;
  double total = 0;
  for (int t = 0; t < nthreads; t++) total += jobs[t].seconds;
  return total;
}

/* One sampler whose state evolves across ndraws draws from the same row
 * (the decode loop of extension/llm/runner/text_token_generator.h:134-184). */
void oracle_sample_sequence_f32(
    const float* row, int32_t vocab, float temperature, float topp, uint64_t seed,
    int64_t ndraws, int32_t* out_tokens) {
  oracle_sampler_t s;
  oracle_sampler_init(&s, vocab, temperature, topp, seed);
  float* buf = (float*)malloc(sizeof(float) * (size_t)vocab);
  for (int64_t d = 0; d < ndraws; d++) {
    memcpy(buf, row, sizeof(float) * (size_t)vocab);
    out_tokens[d] = oracle_sampler_sample_f32(&s, buf);
  }
  free(buf);
}

/* Diagnostics used by the tolerance classification of the parity tests: the fp32
 * probabilities of one row, the coin of its first draw, and the nucleus description. */
void oracle_row_details_f32(
    const float* row, int32_t vocab, float temperature, float topp, uint64_t seed,
    float* out_probs, float* out_coin, int32_t* out_n0, int32_t* out_last_idx,
    float* out_cum, int32_t* out_token) {
  oracle_sampler_t s;
  oracle_sampler_init(&s, vocab, temperature, topp, seed);
  memcpy(out_probs, row, sizeof(float) * (size_t)vocab);
  for (int32_t q = 0; q < vocab; q++) out_probs[q] *= s.inv_temperature;
  oracle_softmax_f32(out_probs, vocab);
  float coin = oracle_random_f32(&s.rng_state);
  *out_coin = coin;
  if (topp <= 0 || topp >= 1) {
    *out_token = oracle_sample_mult_f32(out_probs, vocab, coin);
    *out_n0 = vocab;
    *out_last_idx = vocab - 1;
    *out_cum = 1.0f;
  } else {
    *out_token = oracle_sample_topp_f32(out_probs, vocab, topp, coin, out_n0, out_last_idx, out_cum);
  }
}
