// TEST INFRASTRUCTURE. A small program that is built INSIDE the reference's own header tree:
// the reference's unmodified sampler.h and util.h (sample_from_logits, logits_to_token), its
// portable Tensor, and executorch_b200/csrc/reference_sampler_dropin.cpp in place of the
// reference's sampler.cpp. It replays the reference tests' fixtures with the logits in GPU
// memory:
//   argmax 396 of 32000, float and Half      extension/llm/sampler/test/test_sampler.cpp:19-43
//   {0.1, 0.2, 0.8, 0.4} -> 2, three dtypes  extension/llm/runner/test/test_text_decoder_runner.cpp:83-140
//   rank 3: last sequence position           extension/llm/runner/test/test_text_decoder_runner.cpp:95-116
//   temperature 1: token in range            extension/llm/runner/test/test_text_decoder_runner.cpp:143-153
//   injected sampler, set_temperature        extension/llm/runner/test/test_text_decoder_runner.cpp:156-193
// and the batched tensor entry point. Prints one line per check and exits non-zero on a failure.
// Built by oracle/Makefile (target `dropin`) where the reference checkout is present; the binary
// travels with the tree and is run by tests/test_gpu_dropin.py on a GPU box.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include <executorch/extension/llm/sampler/sampler.h>
#include <executorch/runtime/core/exec_aten/exec_aten.h>
#include <executorch/runtime/core/exec_aten/util/scalar_type_util.h>
// util.h uses ET_SWITCH_FOUR_TYPES without including its header: the include above comes first
#include <executorch/extension/llm/sampler/util.h>
#include <executorch/runtime/platform/runtime.h>

#include "../include/etb200_executorch_dropin.h"

using executorch::aten::BFloat16;
using executorch::aten::Half;
using executorch::aten::ScalarType;
using executorch::aten::Tensor;
using executorch::aten::TensorImpl;
using executorch::extension::llm::Sampler;
using executorch::runtime::etensor::DeviceType;

static int failures = 0;

static void check(bool ok, const char* what, long got, long want) {
  std::printf("%s %s: got %ld, want %ld\n", ok ? "PASS" : "FAIL", what, got, want);
  if (!ok) ++failures;
}

// A reference Tensor over device memory holding a copy of `host`.
template <typename T>
struct DeviceTensor {
  void* dev = nullptr;
  std::vector<TensorImpl::SizesType> sizes;
  std::vector<TensorImpl::DimOrderType> order;
  std::vector<TensorImpl::StridesType> strides;
  TensorImpl* impl = nullptr;
  DeviceTensor(ScalarType st, std::vector<int> shape, const std::vector<T>& host) {
    cudaMalloc(&dev, host.size() * sizeof(T));
    cudaMemcpy(dev, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice);
    int stride = 1;
    strides.resize(shape.size());
    for (int i = (int)shape.size() - 1; i >= 0; --i) {
      strides[i] = stride;
      stride *= shape[i];
    }
    for (size_t i = 0; i < shape.size(); ++i) {
      sizes.push_back(shape[i]);
      order.push_back((TensorImpl::DimOrderType)i);
    }
    impl = new TensorImpl(st, (ssize_t)shape.size(), sizes.data(), dev, order.data(), strides.data(),
                          executorch::aten::TensorShapeDynamism::STATIC, DeviceType::CUDA, 0);
  }
  Tensor tensor() { return Tensor(impl); }
};

int main() {
  executorch::runtime::runtime_init();
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    std::printf("SKIP no CUDA device\n");
    return 77;
  }
  // --- test_sampler.cpp:19-43
  {
    const int vocab = 32000;
    std::vector<float> x(vocab);
    srand(7);
    for (auto& v : x) v = 0.999f * (float)rand() / (float)RAND_MAX;
    x[396] = 1.0f;
    DeviceTensor<float> t(ScalarType::Float, {1, vocab}, x);
    Sampler sampler(vocab, 0.0f, 0.9f, 0ull);
    float* p = t.tensor().mutable_data_ptr<float>();
    check(sampler.sample(p) == 396, "TestArgMax float", sampler.sample(p), 396);
    std::vector<Half> xh(vocab);
    for (int i = 0; i < vocab; ++i) xh[i] = Half(x[i] > 0.998f && i != 396 ? 0.99f : x[i]);
    DeviceTensor<Half> th(ScalarType::Half, {1, 1, vocab}, xh);
    const int32_t tok = executorch::extension::llm::sample_from_logits(th.tensor(), sampler);
    check(tok == 396, "TestArgMaxWithFP16 via sample_from_logits, rank 3", tok, 396);
  }
  // --- test_text_decoder_runner.cpp:83-140, :95-116
  {
    const std::vector<float> f = {0.1f, 0.2f, 0.8f, 0.4f};
    DeviceTensor<float> tf(ScalarType::Float, {1, 4}, f);
    check(executorch::extension::llm::logits_to_token(tf.tensor(), 0.0f) == 2, "logits_to_token float",
          executorch::extension::llm::logits_to_token(tf.tensor(), 0.0f), 2);
    std::vector<Half> h(f.begin(), f.end());
    DeviceTensor<Half> thh(ScalarType::Half, {1, 4}, h);
    check(executorch::extension::llm::logits_to_token(thh.tensor(), 0.0f) == 2, "logits_to_token Half",
          executorch::extension::llm::logits_to_token(thh.tensor(), 0.0f), 2);
    std::vector<BFloat16> b(f.begin(), f.end());
    DeviceTensor<BFloat16> tb(ScalarType::BFloat16, {1, 4}, b);
    check(executorch::extension::llm::logits_to_token(tb.tensor(), 0.0f) == 2, "logits_to_token BFloat16",
          executorch::extension::llm::logits_to_token(tb.tensor(), 0.0f), 2);
    const std::vector<float> f3 = {0.9f, 0.1f, 0.1f, 0.1f, 0.1f, 0.2f, 0.8f, 0.4f};
    DeviceTensor<float> t3(ScalarType::Float, {1, 2, 4}, f3);
    check(executorch::extension::llm::logits_to_token(t3.tensor(), 0.0f) == 2, "rank 3: last position",
          executorch::extension::llm::logits_to_token(t3.tensor(), 0.0f), 2);
    const int32_t tk = executorch::extension::llm::logits_to_token(tf.tensor(), 1.0f);  // :143-153
    check(tk >= 0 && tk < 4, "temperature 1: token in range", tk, tk);
    // :156-193 -- an injected sampler whose temperature is switched between calls
    Sampler injected(4, 1.0f, 0.9f, 42ull);
    injected.set_temperature(0.0f);
    check(executorch::extension::llm::sample_from_logits(tf.tensor(), injected) == 2, "injected sampler, T -> 0",
          executorch::extension::llm::sample_from_logits(tf.tensor(), injected), 2);
    injected.set_temperature(1.0f);
    const int32_t ti = executorch::extension::llm::sample_from_logits(tf.tensor(), injected);
    check(ti >= 0 && ti < 4, "injected sampler, T -> 1", ti, ti);
    injected.set_topk(1);  // only the most probable token survives (sampler.cpp:72-120)
    check(executorch::extension::llm::sample_from_logits(tf.tensor(), injected) == 2, "injected sampler, top-k 1",
          executorch::extension::llm::sample_from_logits(tf.tensor(), injected), 2);
  }
  // --- every batch row of a [B, S, V] tensor, ids left on the device
  {
    const int B = 3, S = 2, V = 5;
    std::vector<float> x(B * S * V, 0.0f);
    const int want[B] = {4, 0, 2};
    for (int b = 0; b < B; ++b) {
      x[(b * S + 0) * V + 1] = 9.0f;         // first position: never read
      x[(b * S + 1) * V + want[b]] = 5.0f;   // last position: the answer
    }
    DeviceTensor<float> t(ScalarType::Float, {B, S, V}, x);
    Sampler sampler(V, 0.0f, 0.9f, 1ull);
    int64_t* ids = nullptr;
    cudaMalloc(&ids, B * sizeof(int64_t));
    const auto err = executorch::extension::llm::sample_rows_from_logits(t.tensor(), sampler, nullptr, ids, nullptr);
    cudaDeviceSynchronize();
    int64_t got[B];
    cudaMemcpy(got, ids, sizeof(got), cudaMemcpyDeviceToHost);
    check(err == executorch::runtime::Error::Ok, "sample_rows_from_logits status", (long)err, 0);
    for (int b = 0; b < B; ++b) check(got[b] == want[b], "sample_rows_from_logits row", got[b], want[b]);
  }
  std::printf("%s\n", failures == 0 ? "ALL PASS" : "FAILED");
  return failures == 0 ? 0 : 1;
}
