/* Tensor-level entry points for a build INSIDE the ExecuTorch tree (needs the reference's own
 * headers on the include path): the counterpart of sample_from_logits
 * (extension/llm/sampler/util.h:25-55) for logits that stay on the GPU.
 *
 * Together with executorch_b200/csrc/reference_sampler_dropin.cpp -- which defines the members
 * of the reference's own executorch::extension::llm::Sampler (extension/llm/sampler/sampler.h:
 * 37-83) on top of the C ABI, and replaces extension/llm/sampler/sampler.cpp in such a build --
 * the reference's unmodified util.h, TextDecoderRunner (text_decoder_runner.h:84-94) and
 * llm_runner_helper.cpp:273-275 compile and run unchanged, with `logits` a CUDA-resident
 * tensor. */
#ifndef ETB200_EXECUTORCH_DROPIN_H_
#define ETB200_EXECUTORCH_DROPIN_H_

#include <executorch/extension/llm/sampler/sampler.h>
#include <executorch/runtime/core/error.h>
#include <executorch/runtime/core/exec_aten/exec_aten.h>

#include <cstdint>

struct etb200_sampler; /* the handle type of include/etb200_sampler.h */

namespace executorch {
namespace extension {
namespace llm {

/* The C-ABI handle behind a reference Sampler built with the drop-in translation unit. */
::etb200_sampler* b200_handle(Sampler& sampler);

/* sample_from_logits (util.h:25-55) for EVERY batch row of a CUDA-resident logits tensor
 * ([B, V], or [B, S, V]: last sequence position of each batch entry; the reference reads batch
 * entry 0 only). rng_states_device: B xorshift64* states, advanced in place (ignored at
 * temperature 0); out_ids_device: B int64 ids. Asynchronous on `stream` (a cudaStream_t).
 * Errors are those of the C ABI, as executorch::runtime::Error values. */
::executorch::runtime::Error sample_rows_from_logits(
    const ::executorch::aten::Tensor& logits_tensor, Sampler& sampler, uint64_t* rng_states_device,
    int64_t* out_ids_device, void* stream);

}  // namespace llm
}  // namespace extension
}  // namespace executorch

#endif /* ETB200_EXECUTORCH_DROPIN_H_ */
