// Drop-in replacement of extension/llm/sampler/sampler.cpp for a B200 host: defines the
// out-of-line members of the reference's OWN class executorch::extension::llm::Sampler
// (extension/llm/sampler/sampler.h:37-83, header unmodified) on top of the C ABI of
// include/etb200_sampler.h. Compiled inside the ExecuTorch tree (its headers on the include
// path) and linked with libetb200_sampler.so; util.h, TextDecoderRunner::logits_to_token
// (text_decoder_runner.h:84-94) and create_text_llm_runner (llm_runner_helper.cpp:273-275) then
// work unchanged, with `logits` pointing to device memory.
//
// The reference class has no spare member and no destructor, so the C-ABI handle lives in the
// one member that this implementation does not need on the host: `rng_state_` (sampler.h:82)
// holds the handle's address; the xorshift64* state itself is on the device, seeded by the
// constructor and advanced by every non-greedy sample(), exactly as the reference advances
// rng_state_ (sampler.cpp:210-220,237). `inv_temperature_`, `topp_` and `topk_` keep their
// meaning (the inline setters of sampler.h:48-60 write them) and are handed to the handle at
// every call. Consequences of the unmodified declaration: a Sampler is never torn down by the
// class itself (call b200_release() before dropping one that will not be reused; the runner
// keeps its sampler for its whole life), and copies of a Sampler share one RNG stream.
#include <executorch/extension/llm/sampler/sampler.h>
#include <executorch/runtime/core/exec_aten/exec_aten.h>
#include <executorch/runtime/platform/assert.h>

#include <ctime>

#include "../../include/etb200_executorch_dropin.h"
#include "../../include/etb200_sampler.h"

namespace executorch {
namespace extension {
namespace llm {

namespace {

inline etb200_sampler_t* as_handle(unsigned long long word) {
  return reinterpret_cast<etb200_sampler_t*>(static_cast<uintptr_t>(word));
}

template <typename T>
struct DtypeCode;
template <>
struct DtypeCode<float> {
  static constexpr int32_t value = ETB200_DTYPE_FLOAT;
};
template <>
struct DtypeCode<uint16_t> {
  static constexpr int32_t value = ETB200_DTYPE_UINT16;
};
template <>
struct DtypeCode<executorch::aten::Half> {
  static constexpr int32_t value = ETB200_DTYPE_HALF;
};
template <>
struct DtypeCode<executorch::aten::BFloat16> {
  static constexpr int32_t value = ETB200_DTYPE_BFLOAT16;
};

unsigned long long make_handle(int32_t vocab_size, float temperature, float topp, unsigned long long seed) {
  etb200_sampler_t* h = nullptr;
  const etb200_error_t err = etb200_sampler_create(vocab_size, temperature, topp, seed, /*device=*/-1, &h);
  ET_CHECK_MSG(err == ETB200_OK, "B200 sampler: %s", etb200_last_error_message());
  return static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(h));
}

}  // namespace

// sampler.cpp:173-181
Sampler::Sampler(int32_t vocab_size, float temperature, float topp, unsigned long long rng_seed)
    : vocab_size_(vocab_size),
      inv_temperature_((temperature != 0.0f) ? (1.0f / temperature) : 0.0f),
      topp_(topp),
      rng_state_(make_handle(vocab_size, temperature, topp, rng_seed)) {}

// sampler.cpp:183-187
Sampler::Sampler(int32_t vocab_size, float temperature)
    : vocab_size_(vocab_size),
      inv_temperature_((temperature != 0.0f) ? (1.0f / temperature) : 0.0f),
      topp_(kTopp),
      rng_state_(make_handle(vocab_size, temperature, kTopp, static_cast<unsigned long long>(std::time(nullptr)))) {}

// sampler.cpp:222-251; `logits` is a device pointer, the token comes back on the host
template <typename T>
int32_t Sampler::sample(T* logits) {
  etb200_sampler_t* h = as_handle(rng_state_);
  etb200_sampler_set_inv_temperature(h, inv_temperature_);
  etb200_sampler_set_topk(h, topk_);
  int32_t token = 0;
  const etb200_error_t err = etb200_sampler_sample(h, logits, DtypeCode<T>::value, /*stream=*/nullptr, &token);
  ET_CHECK_MSG(err == ETB200_OK, "B200 sampler: %s", etb200_last_error_message());
  return token;
}

// the instantiations of sampler.cpp:253-258
template int32_t Sampler::sample<float>(float* logits);
template int32_t Sampler::sample<uint16_t>(uint16_t* logits);
template int32_t Sampler::sample<executorch::aten::Half>(executorch::aten::Half* logits);
template int32_t Sampler::sample<executorch::aten::BFloat16>(executorch::aten::BFloat16* logits);

namespace {
// The reference keeps its members private; the first instantiated sample() above reads
// rng_state_ legitimately, and so does this member-pointer accessor (explicit instantiation
// may name private members).
template <unsigned long long Sampler::*Member>
struct StateAccess {
  friend unsigned long long& state_word(Sampler& s) { return s.*Member; }
};
unsigned long long& state_word(Sampler& s);
template struct StateAccess<&Sampler::rng_state_>;
template <float Sampler::*Member>
struct InvTAccess {
  friend float& inv_t_word(Sampler& s) { return s.*Member; }
};
float& inv_t_word(Sampler& s);
template struct InvTAccess<&Sampler::inv_temperature_>;
template <int32_t Sampler::*Member>
struct TopkAccess {
  friend int32_t& topk_word(Sampler& s) { return s.*Member; }
};
int32_t& topk_word(Sampler& s);
template struct TopkAccess<&Sampler::topk_>;
}  // namespace

::etb200_sampler* b200_handle(Sampler& sampler) { return as_handle(state_word(sampler)); }

::executorch::runtime::Error sample_rows_from_logits(
    const ::executorch::aten::Tensor& logits_tensor, Sampler& sampler, uint64_t* rng_states_device,
    int64_t* out_ids_device, void* stream) {
  using ::executorch::aten::ScalarType;
  using ::executorch::runtime::Error;
  etb200_sampler_t* h = as_handle(state_word(sampler));
  int32_t dtype;
  size_t esz = 2;
  switch (logits_tensor.scalar_type()) {
    case ScalarType::Float:
      dtype = ETB200_DTYPE_FLOAT;
      esz = 4;
      break;
    case ScalarType::Half:
      dtype = ETB200_DTYPE_HALF;
      break;
    case ScalarType::BFloat16:
      dtype = ETB200_DTYPE_BFLOAT16;
      break;
    case ScalarType::UInt16:
      dtype = ETB200_DTYPE_UINT16;
      break;
    default:
      return Error::NotSupported;  // sample_from_logits aborts here (util.h:30-34)
  }
  const auto dim = logits_tensor.dim();
  if (dim != 2 && dim != 3) return Error::InvalidArgument;
  const int64_t vocab = logits_tensor.size(dim - 1);
  const int64_t batch = logits_tensor.size(0);
  const char* base = static_cast<const char*>(logits_tensor.const_data_ptr());
  int64_t row_stride = vocab;
  if (dim == 3) {
    // the last sequence position of every batch entry (util.h:48-51 does this for entry 0)
    const int64_t tokens = logits_tensor.size(1);
    base += static_cast<size_t>((tokens - 1) * vocab) * esz;
    row_stride = tokens * vocab;
  }
  etb200_sampler_set_inv_temperature(h, inv_t_word(sampler));
  etb200_sampler_set_topk(h, topk_word(sampler));
  return static_cast<Error>(etb200_sampler_sample_rows(h, base, dtype, batch, row_stride, rng_states_device,
                                                       out_ids_device, stream));
}

}  // namespace llm
}  // namespace extension
}  // namespace executorch
