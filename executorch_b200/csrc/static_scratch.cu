// An entry point for callers that must not allocate device memory.
//
// Who that is: code running inside somebody else's memory plan -- an inference runtime
// whose arena was sized ahead of time and that treats any later cudaMalloc as a bug, a
// process that shares its GPU and has been given a fixed budget, or a real-time loop that
// cannot afford the implicit device synchronisation and the unbounded latency of
// cudaMalloc / cudaFree. The handle-based interface in c_api.cu does not suit them:
// creating a handle allocates, and so does its first top-p call.
//
// This file gives them the same sampling kernel with its candidate lists placed in a
// fixed array that is part of the library image, so nothing is ever allocated or freed:
// not here, not in a CUDA library routine, not through torch.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "../../include/etb200_sampler.h"
#include "sampler_kernels.cuh"

using namespace etb200;

namespace {

// The whole scratch budget of this entry point: 64 MiB per GPU that loads the library,
// held until the process exits. The sampling kernel needs 16 bytes per vocabulary entry
// per thread block, so this is 32 blocks' worth at a 131072-entry vocabulary.
constexpr size_t kStaticScratchBytes = size_t(64) << 20;
constexpr size_t kBytesPerVocabEntryPerBlock = 16;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a stand-in for the symbol, not an address the
// GPU can use. The real device address is looked up once per device and cached here.
constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};
int g_sm_count[kMaxDevices] = {};
int g_blocks_per_sm[kMaxDevices][3] = {};  // occupancy of the sampling kernel per dtype, queried once
bool g_table_ready = false;
ExpTable g_table;  // host-side constants of the kernels' exponential, built once per process

thread_local char g_static_err[256] = "";

etb200_error_t fail(etb200_error_t code, const char* msg) {
  snprintf(g_static_err, sizeof(g_static_err), "%s", msg);
  return code;
}

// Looks up the array's address on the CURRENT device (first call per device only).
etb200_error_t setup_current_device(int* device_out, void** ptr_out, int* sm_count_out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ETB200_INTERNAL, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(ETB200_NOT_SUPPORTED, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      return fail(ETB200_INTERNAL, e != cudaSuccess ? cudaGetErrorString(e)
                                                   : "cudaGetSymbolAddress returned a null address");
    }
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return fail(ETB200_INTERNAL, cudaGetErrorString(e));
    if (major < 10) return fail(ETB200_NOT_SUPPORTED, "this library is built for sm_100a only");
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms < 1) return fail(ETB200_INTERNAL, "cannot read the SM count");
    g_sm_count[dev] = sms;
    g_scratch_ptr[dev] = p;
  }
  if (!g_table_ready) {
    make_exp_table(&g_table);
    g_table_ready = true;
  }
  *device_out = dev;
  *ptr_out = g_scratch_ptr[dev];
  *sm_count_out = g_sm_count[dev];
  return ETB200_OK;
}

// Resident blocks per SM of the sampling kernel for a dtype on a device (cached; the query
// also opts the kernel in to its shared-memory size, which is needed once per device).
int blocks_per_sm_cached(int dev, int dtype) {
  const int slot = dtype == kDtypeFloat ? 0 : (dtype == kDtypeHalf ? 1 : 2);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_blocks_per_sm[dev][slot] == 0) g_blocks_per_sm[dev][slot] = sample_kernel_max_blocks_per_sm(dtype);
  return g_blocks_per_sm[dev][slot];
}

}  // namespace

extern "C" {

etb200_error_t etb200_sample_rows_static(
    int32_t vocab_size, float temperature, float topp, const void* logits_device, int32_t dtype,
    int64_t rows, int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* out_ids_device,
    void* stream) {
  if (vocab_size < 1) return fail(ETB200_INVALID_ARGUMENT, "vocab_size must be >= 1");
  if (rows < 0) return fail(ETB200_INVALID_ARGUMENT, "rows must be >= 0");
  if (rows == 0) return ETB200_OK;
  if (logits_device == nullptr || out_ids_device == nullptr)
    return fail(ETB200_INVALID_ARGUMENT, "logits or output pointer is null");
  if (dtype != kDtypeFloat && dtype != kDtypeHalf && dtype != kDtypeBFloat16 && dtype != kDtypeUInt16)
    return fail(ETB200_NOT_SUPPORTED, "unsupported logits dtype (Half 5, Float 6, BFloat16 15, UInt16 27)");
  if (!(rows == 1 || row_stride_elems == 0 || row_stride_elems >= vocab_size))
    return fail(ETB200_INVALID_ARGUMENT, "row_stride_elems is smaller than vocab_size and not 0");
  // the one hard limit of this entry point: at least one block's lists must fit the array.
  // Only top-p uses the lists; argmax and multinomial calls are not limited.
  const bool uses_lists = temperature != 0.0f && topp > 0.0f && topp < 1.0f;
  const size_t per_block = kBytesPerVocabEntryPerBlock * (size_t)vocab_size;
  if (uses_lists && per_block > kStaticScratchBytes) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "vocab_size %d needs %zu bytes of scratch per block, more than the %zu-byte static array "
             "(limit: vocab_size <= %zu); use etb200_sampler_sample_rows instead",
             vocab_size, per_block, kStaticScratchBytes, kStaticScratchBytes / kBytesPerVocabEntryPerBlock);
    return fail(ETB200_INVALID_ARGUMENT, msg);
  }
  int dev = 0, sms = 0;
  void* scratch = nullptr;
  etb200_error_t err = setup_current_device(&dev, &scratch, &sms);
  if (err != ETB200_OK) return err;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const float inv_t = (temperature != 0.0f) ? 1.0f / temperature : 0.0f;  // sampler.cpp:179
  cudaError_t e;
  if (inv_t == 0.0f) {
    const int64_t cap = (int64_t)sms * 4;
    e = launch_argmax_rows(dtype, logits_device, rows, vocab_size, row_stride_elems, out_ids_device,
                           PeerOut{}, (int)(rows < cap ? rows : cap), nullptr, st);
  } else {
    if (dtype == kDtypeUInt16)
      return fail(ETB200_NOT_SUPPORTED, "UInt16 logits can only be sampled at temperature 0");
    if (rng_states_device == nullptr)
      return fail(ETB200_INVALID_ARGUMENT, "rng_states_device is null (there is no handle to own a state)");
    int64_t blocks = (int64_t)sms * blocks_per_sm_cached(dev, dtype);
    if (uses_lists) {
      const int64_t fit = (int64_t)(kStaticScratchBytes / per_block);
      if (blocks > fit) blocks = fit;
    }
    if (blocks > rows) blocks = rows;
    e = launch_sample_rows(dtype, logits_device, rows, vocab_size, row_stride_elems, inv_t, topp,
                           /*topk=*/0, reinterpret_cast<unsigned long long*>(rng_states_device), out_ids_device,
                           PeerOut{}, scratch, (int)blocks, g_table, nullptr, st);
  }
  if (e != cudaSuccess) return fail(ETB200_INTERNAL, cudaGetErrorString(e));
  return ETB200_OK;
}

const char* etb200_static_last_error_message(void) { return g_static_err; }

}  // extern "C"
