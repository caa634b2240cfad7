// C++ face of the B200 token sampler: the reference's Sampler class
// (extension/llm/sampler/sampler.h:37-83) re-declared over the C ABI of etb200_sampler.h.
// Header-only; link with -letb200_sampler.
//
// Same constructors and methods as the reference class, with these differences:
//  - `logits` pointers are DEVICE pointers (the reference samples host memory);
//  - a `device` ordinal and a `stream` can be given (defaults: device 0, the legacy stream);
//  - `sample_rows` is the batched extension (one launch for rows x vocab logits);
//  - logits are not modified.
// Error handling follows the reference's style: sample() cannot report failure through its
// int32_t result, so like ET_CHECK_MSG it prints the reason and aborts; everything that can
// return a code returns executorch_b200::Error, whose values are those of
// executorch::runtime::Error (runtime/core/error.h:29-100).
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <utility>

#include "etb200_sampler.h"

namespace executorch_b200 {

enum class Error : uint32_t {
  Ok = ETB200_OK,
  Internal = ETB200_INTERNAL,
  InvalidState = ETB200_INVALID_STATE,
  NotSupported = ETB200_NOT_SUPPORTED,
  InvalidArgument = ETB200_INVALID_ARGUMENT,
  MemoryAllocationFailed = ETB200_MEMORY_ALLOCATION_FAILED,
};

// ScalarType codes of the four logits types sample_from_logits dispatches on
// (extension/llm/sampler/util.h:36-53, runtime/core/portable_type/scalar_type.h:98-125).
enum class ScalarType : int32_t {
  Half = ETB200_DTYPE_HALF,
  Float = ETB200_DTYPE_FLOAT,
  BFloat16 = ETB200_DTYPE_BFLOAT16,
  UInt16 = ETB200_DTYPE_UINT16,
};

// Two-byte tags for callers that do not include the CUDA half/bfloat16 headers.
struct Half {
  uint16_t bits;
};
struct BFloat16 {
  uint16_t bits;
};

template <typename T>
struct ScalarTypeOf;
template <>
struct ScalarTypeOf<float> {
  static constexpr ScalarType value = ScalarType::Float;
};
template <>
struct ScalarTypeOf<uint16_t> {
  static constexpr ScalarType value = ScalarType::UInt16;
};
template <>
struct ScalarTypeOf<Half> {
  static constexpr ScalarType value = ScalarType::Half;
};
template <>
struct ScalarTypeOf<BFloat16> {
  static constexpr ScalarType value = ScalarType::BFloat16;
};
#if defined(__CUDA_FP16_TYPES_EXIST__)
template <>
struct ScalarTypeOf<__half> {
  static constexpr ScalarType value = ScalarType::Half;
};
#endif
#if defined(__CUDA_BF16_TYPES_EXIST__)
template <>
struct ScalarTypeOf<__nv_bfloat16> {
  static constexpr ScalarType value = ScalarType::BFloat16;
};
#endif

namespace extension {
namespace llm {

inline constexpr float kTopp = 0.9f;  // sampler.h:29

class Sampler {
 public:
  // sampler.cpp:173-181
  Sampler(int32_t vocab_size, float temperature, float topp, unsigned long long rng_seed,
          int32_t device = 0)
      : vocab_size_(vocab_size) {
    status_ = static_cast<Error>(
        etb200_sampler_create(vocab_size, temperature, topp, rng_seed, device, &handle_));
  }

  // sampler.cpp:183-187: top-p 0.9, wall-clock seed
  Sampler(int32_t vocab_size, float temperature, int32_t device = 0) : vocab_size_(vocab_size) {
    status_ = static_cast<Error>(
        etb200_sampler_create_default(vocab_size, temperature, device, &handle_));
  }

  ~Sampler() { etb200_sampler_destroy(handle_); }
  Sampler(const Sampler&) = delete;
  Sampler& operator=(const Sampler&) = delete;
  Sampler(Sampler&& o) noexcept
      : handle_(std::exchange(o.handle_, nullptr)), vocab_size_(o.vocab_size_), status_(o.status_) {}
  Sampler& operator=(Sampler&& o) noexcept {
    if (this != &o) {
      etb200_sampler_destroy(handle_);
      handle_ = std::exchange(o.handle_, nullptr);
      vocab_size_ = o.vocab_size_;
      status_ = o.status_;
    }
    return *this;
  }

  // Ok unless construction failed (no CUDA device, bad arguments, out of memory).
  Error status() const { return status_; }
  static const char* last_error_message() { return etb200_last_error_message(); }
  int32_t vocab_size() const { return vocab_size_; }

  // sampler.h:48-53: negative values are reset to 0
  void set_temperature(float temperature) { etb200_sampler_set_temperature(handle_, temperature); }
  // sampler.h:58-60
  void set_topk(int32_t topk) { etb200_sampler_set_topk(handle_, topk); }

  // sampler.cpp:222-251 on one row of vocab_size logits in device memory. Uses and advances
  // the sampler's own RNG state; synchronises `stream`.
  template <typename T>
  int32_t sample(T* logits, void* stream = nullptr) {
    int32_t token = 0;
    const uint32_t err = etb200_sampler_sample(
        handle_, logits, static_cast<int32_t>(ScalarTypeOf<T>::value), stream, &token);
    if (err != ETB200_OK) {
      std::fprintf(stderr, "Sampler::sample failed (0x%02x): %s\n", err, etb200_last_error_message());
      std::abort();
    }
    return token;
  }

  // Batched extension: every row r of `rows` (at logits + r * row_stride_elems) is sampled
  // with its own xorshift64* state rng_states[r] (device memory, advanced in place; may be
  // null at temperature 0) and the int64 token goes to out_ids[r] (device memory).
  // Asynchronous on `stream`.
  Error sample_rows(const void* logits, ScalarType dtype, int64_t rows, int64_t row_stride_elems,
                    uint64_t* rng_states, int64_t* out_ids, void* stream = nullptr) {
    return static_cast<Error>(etb200_sampler_sample_rows(
        handle_, logits, static_cast<int32_t>(dtype), rows, row_stride_elems, rng_states, out_ids,
        stream));
  }

  // The same for logits, states and ids in HOST memory (copies in and out, synchronises).
  Error sample_rows_host(const void* logits, ScalarType dtype, int64_t rows,
                         int64_t row_stride_elems, uint64_t* rng_states, int64_t* out_ids,
                         void* stream = nullptr) {
    return static_cast<Error>(etb200_sampler_sample_rows_host(
        handle_, logits, static_cast<int32_t>(dtype), rows, row_stride_elems, rng_states, out_ids,
        stream));
  }

  // Multi-GPU forms (no counterpart in the reference): the id of row r goes to index
  // dest_offset + r of every buffer in dest_buffers (this GPU's and its peers'); the second form
  // also synchronises the ranks inside the launch (see etb200_sampler_sample_rows_exchange).
  Error sample_rows_scatter(const void* logits, ScalarType dtype, int64_t rows, int64_t row_stride_elems,
                            uint64_t* rng_states, int64_t* const* dest_buffers, int32_t n_dest,
                            int64_t dest_offset, void* stream = nullptr) {
    return static_cast<Error>(etb200_sampler_sample_rows_scatter(
        handle_, logits, static_cast<int32_t>(dtype), rows, row_stride_elems, rng_states, dest_buffers,
        n_dest, dest_offset, stream));
  }
  Error sample_rows_exchange(const void* logits, ScalarType dtype, int64_t rows, int64_t row_stride_elems,
                             uint64_t* rng_states, int64_t* const* dest_buffers,
                             uint64_t* const* arrive_marks, int32_t n_dest, int32_t my_rank,
                             int64_t dest_offset, uint64_t epoch, void* stream = nullptr) {
    return static_cast<Error>(etb200_sampler_sample_rows_exchange(
        handle_, logits, static_cast<int32_t>(dtype), rows, row_stride_elems, rng_states, dest_buffers,
        arrive_marks, n_dest, my_rank, dest_offset, epoch, stream));
  }
  // Reads and clears the device status word: 0, or 2 after an arrival wait ran out.
  int32_t device_status() {
    int32_t v = 0;
    etb200_sampler_get_status(handle_, &v);
    return v;
  }

  // Sampler::rng_state_ (sampler.h:82), for checkpoint and resume.
  unsigned long long rng_state() const {
    uint64_t s = 0;
    etb200_sampler_get_rng_state(handle_, &s);
    return s;
  }
  void set_rng_state(unsigned long long s) { etb200_sampler_set_rng_state(handle_, s); }

 private:
  etb200_sampler_t* handle_ = nullptr;
  int32_t vocab_size_ = 0;
  Error status_ = Error::Ok;
};

}  // namespace llm
}  // namespace extension
}  // namespace executorch_b200
