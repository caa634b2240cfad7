/*
 * TEST INFRASTRUCTURE, not product code. A thin extern "C" driver around the
 * reference's own executorch::extension::llm::Sampler
 * (extension/llm/sampler/sampler.h:37-83, sampler.cpp:173-258). It is compiled
 * together with the reference's unmodified sampler.cpp (see the Makefile beside this
 * file) into oracle/_ref/; only tests, the smoke check and the CPU-baseline leg of the
 * benchmark may load it.
 *
 * Every entry point runs one fresh Sampler(vocab, temperature, topp, seed) per row on a
 * private copy of the row, because Sampler::sample() overwrites its input with
 * probabilities (sampler.cpp:231-235).
 */
#include <executorch/extension/llm/sampler/sampler.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

using executorch::extension::llm::Sampler;

namespace {

inline float bf16_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

inline float f16_to_f32(uint16_t h) {
  c10::Half v;
  std::memcpy(&v, &h, 2);
  return static_cast<float>(v);
}

// dtype codes follow ScalarType numbering (runtime/core/portable_type/scalar_type.h):
// Half=5, Float=6, BFloat16=15.
enum { kHalf = 5, kFloat = 6, kBFloat16 = 15 };

// mode 0: upcast 16-bit rows to fp32 and call sample<float>; mode 1: call the
// reference's native sample<Half>/sample<BFloat16> on the 16-bit row itself.
template <typename F>
void for_rows(int64_t rows, int nthreads, F&& body) {
  if (nthreads < 1) nthreads = 1;
  if (nthreads == 1 || rows < 2) {
    for (int64_t r = 0; r < rows; ++r) body(r);
    return;
  }
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t) {
    pool.emplace_back([&, t]() {
      for (int64_t r = t; r < rows; r += nthreads) body(r);
    });
  }
  for (auto& th : pool) th.join();
}

int32_t sample_one(
    const void* row, int dtype, int mode, int32_t vocab, float temperature,
    float topp, int32_t topk, unsigned long long seed, double* seconds,
    std::vector<float>& f32buf, std::vector<uint16_t>& u16buf) {
  Sampler s(vocab, temperature, topp, seed);
  if (topk > 0) s.set_topk(topk);
  int32_t tok;
  if (dtype == kFloat || mode == 0) {
    f32buf.resize(vocab);
    if (dtype == kFloat) {
      std::memcpy(f32buf.data(), row, sizeof(float) * vocab);
    } else if (dtype == kBFloat16) {
      const uint16_t* p = static_cast<const uint16_t*>(row);
      for (int32_t i = 0; i < vocab; ++i) f32buf[i] = bf16_to_f32(p[i]);
    } else {
      const uint16_t* p = static_cast<const uint16_t*>(row);
      for (int32_t i = 0; i < vocab; ++i) f32buf[i] = f16_to_f32(p[i]);
    }
    auto a = std::chrono::steady_clock::now();
    tok = s.sample(f32buf.data());
    auto b = std::chrono::steady_clock::now();
    if (seconds) *seconds += std::chrono::duration<double>(b - a).count();
  } else {
    u16buf.resize(vocab);
    std::memcpy(u16buf.data(), row, 2 * static_cast<size_t>(vocab));
    auto a = std::chrono::steady_clock::now();
    if (dtype == kBFloat16) {
      tok = s.sample(reinterpret_cast<c10::BFloat16*>(u16buf.data()));
    } else {
      tok = s.sample(reinterpret_cast<c10::Half*>(u16buf.data()));
    }
    auto b = std::chrono::steady_clock::now();
    if (seconds) *seconds += std::chrono::duration<double>(b - a).count();
  }
  return tok;
}

} // namespace

extern "C" {

// Samples every row with a fresh Sampler seeded by seeds[r]. Returns the summed time
// spent inside Sampler::sample() over all rows (seconds, CPU time across threads);
// wall_seconds receives the elapsed wall-clock time of the whole call.
double ref_sample_rows(
    const void* logits, int dtype, int mode, int64_t rows, int32_t vocab,
    int64_t row_stride_elems, float temperature, float topp, int32_t topk,
    const uint64_t* seeds, int32_t* out_tokens, int nthreads,
    double* wall_seconds) {
  const size_t esz = (dtype == kFloat) ? 4 : 2;
  std::vector<double> per_thread(nthreads > 0 ? nthreads : 1, 0.0);
  auto w0 = std::chrono::steady_clock::now();
  if (nthreads < 1) nthreads = 1;
  std::vector<std::thread> pool;
  auto work = [&](int t) {
    std::vector<float> f32buf;
    std::vector<uint16_t> u16buf;
    for (int64_t r = t; r < rows; r += nthreads) {
      const char* row =
          static_cast<const char*>(logits) + esz * row_stride_elems * r;
      out_tokens[r] = sample_one(
          row, dtype, mode, vocab, temperature, topp, topk, seeds[r],
          &per_thread[t], f32buf, u16buf);
    }
  };
  if (nthreads == 1) {
    work(0);
  } else {
    for (int t = 0; t < nthreads; ++t) pool.emplace_back(work, t);
    for (auto& th : pool) th.join();
  }
  auto w1 = std::chrono::steady_clock::now();
  if (wall_seconds)
    *wall_seconds = std::chrono::duration<double>(w1 - w0).count();
  double total = 0;
  for (double v : per_thread) total += v;
  return total;
}

// One Sampler whose state evolves over ndraws calls on (copies of) the same row: the
// decode-loop usage of extension/llm/runner/text_token_generator.h:134-184.
void ref_sample_sequence(
    const void* row, int dtype, int mode, int32_t vocab, float temperature,
    float topp, unsigned long long seed, int64_t ndraws, int32_t* out_tokens) {
  Sampler s(vocab, temperature, topp, seed);
  std::vector<float> base(vocab), buf(vocab);
  if (dtype == kFloat) {
    std::memcpy(base.data(), row, sizeof(float) * vocab);
  } else {
    const uint16_t* p = static_cast<const uint16_t*>(row);
    for (int32_t i = 0; i < vocab; ++i)
      base[i] = (dtype == kBFloat16) ? bf16_to_f32(p[i]) : f16_to_f32(p[i]);
  }
  (void)mode;
  for (int64_t d = 0; d < ndraws; ++d) {
    buf = base;
    out_tokens[d] = s.sample(buf.data());
  }
}

// Applies the reference's temperature scaling and softmax to an fp32 row and returns
// the probabilities the sampler would draw from (the row buffer after sample()).
int32_t ref_probs_f32(
    const float* row, int32_t vocab, float temperature, float topp,
    unsigned long long seed, float* out_probs) {
  Sampler s(vocab, temperature, topp, seed);
  std::memcpy(out_probs, row, sizeof(float) * vocab);
  return s.sample(out_probs);
}

} // extern "C"
