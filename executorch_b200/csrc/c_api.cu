// extern "C" surface of the B200 token sampler (declared in include/etb200_sampler.h).
// Mirrors the conventions of the reference's CUDA shims
// (backends/cuda/runtime/shims/rand.cu:175-237): argument checks return InvalidArgument,
// unsupported dtypes NotSupported, CUDA failures Internal; nothing throws.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <ctime>
#include <new>

#include "../../include/etb200_sampler.h"
#include "sampler_kernels.cuh"

using namespace etb200;

struct etb200_sampler {
  int device = 0;
  int vocab = 0;
  float inv_temperature = 0.0f;  // reciprocal of temperature, 0 for greedy (sampler.h:78)
  float topp = 0.9f;
  int topk = 0;
  unsigned long long* d_state = nullptr;  // the handle's own xorshift64* state
  int64_t* h_token = nullptr;             // pinned, device-mapped host slot: the single-row call's
  int64_t* h_token_dev = nullptr;         // kernel stores the token straight into it (no copy)
  int* d_status = nullptr;       // [0]: set by a kernel whose bounded wait ran out
  int* d_blocks_done = nullptr;  // block counter of the arrival barrier, zero between launches
  void* scratch = nullptr;
  size_t scratch_bytes = 0;
  int sm_count = 0;
  // staging for the host-buffer entry point
  void* d_stage = nullptr;
  size_t stage_bytes = 0;
  unsigned long long* d_stage_states = nullptr;
  int64_t* d_stage_ids = nullptr;
  int64_t stage_rows = 0;
  // the host-buffer entry point copies in slices on its own stream while earlier slices are
  // being sampled on the caller's stream
  static constexpr int kMaxSlices = 8;
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t slice_ready[kMaxSlices] = {};
  cudaEvent_t entry_event = nullptr;
  uint64_t launches = 0;
  int blocks_per_sm[3] = {0, 0, 0};  // occupancy of the sampling kernel per dtype, queried once
  ExpTable table;
  // Rows that the cluster kernel leaves undecided: [0], [1] are the counters of alternating
  // launches (each launch clears the other one), [2...] the row numbers.
  int* d_retry = nullptr;
  int64_t retry_cap = 0;
  void* cluster_scratch = nullptr;  // per-row record lists of the cluster kernel, one batch of rows
  size_t cluster_scratch_bytes = 0;
  unsigned retry_parity = 0;
  unsigned long long wait_ns = 1000000000ull;  // limit of the in-kernel wait for the other ranks
  // 0: automatic; 1: the one-block-per-row kernel; 2: the cluster-per-row kernels where they
  // apply; 3: the one-block-per-row kernel with the estimate-guided sum for 16-bit logits
  int kernel_choice = 0;
  int guided_blocks_per_sm[2] = {0, 0};
};

namespace {

thread_local char g_err[512] = "";

etb200_error_t fail(etb200_error_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define ETB_CHECK_ARG(cond, ...) \
  do {                           \
    if (!(cond)) return fail(ETB200_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

#define ETB_CUDA(expr)                                                              \
  do {                                                                              \
    cudaError_t e_ = (expr);                                                        \
    if (e_ != cudaSuccess)                                                          \
      return fail(ETB200_INTERNAL, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
  } while (0)

// Makes the handle's device current for the duration of a call.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      switched = (err == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

size_t dtype_size(int dtype) {
  switch (dtype) {
    case kDtypeFloat:
      return 4;
    case kDtypeHalf:
    case kDtypeBFloat16:
    case kDtypeUInt16:
      return 2;
    default:
      return 0;
  }
}

float inv_temperature_of(float temperature) {
  // static_cast<bool>(temperature) ? 1.0f / temperature : 0  (sampler.cpp:179)
  return (temperature != 0.0f) ? 1.0f / temperature : 0.0f;
}

etb200_error_t create_impl(
    int32_t vocab, float temperature, float topp, uint64_t seed, int32_t device,
    etb200_sampler_t** out) {
  ETB_CHECK_ARG(out != nullptr, "out_handle is null");
  *out = nullptr;
  ETB_CHECK_ARG(vocab >= 1, "vocab_size must be >= 1, got %d", vocab);
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0) {
    return fail(ETB200_INTERNAL, "no CUDA device available (%s); this library has no CPU path",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  if (device == -1) {  // the calling thread's current device
    e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(ETB200_INTERNAL, "cudaGetDevice failed: %s", cudaGetErrorString(e));
  }
  ETB_CHECK_ARG(device >= 0 && device < ndev, "device %d out of range [0, %d)", device, ndev);
  DeviceGuard guard(device);
  if (guard.err != cudaSuccess)
    return fail(ETB200_INTERNAL, "cudaSetDevice(%d) failed: %s", device, cudaGetErrorString(guard.err));
  etb200_sampler* h = new (std::nothrow) etb200_sampler();
  if (!h) return fail(ETB200_MEMORY_ALLOCATION_FAILED, "out of host memory");
  h->device = device;
  h->vocab = vocab;
  h->inv_temperature = inv_temperature_of(temperature);
  h->topp = topp;
  make_exp_table(&h->table);
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) {
    delete h;
    return fail(ETB200_INTERNAL, "cudaGetDeviceProperties failed: %s", cudaGetErrorString(e));
  }
  if (prop.major < 10) {
    delete h;
    return fail(ETB200_NOT_SUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                device, prop.major, prop.minor);
  }
  h->sm_count = prop.multiProcessorCount;
  e = cudaMalloc(&h->d_state, sizeof(unsigned long long));
  if (e == cudaSuccess) e = cudaHostAlloc(&h->h_token, sizeof(int64_t), cudaHostAllocMapped);
  if (e == cudaSuccess) e = cudaHostGetDevicePointer(&h->h_token_dev, h->h_token, 0);
  if (e == cudaSuccess) e = cudaMalloc(&h->d_status, 2 * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(h->d_status, 0, 2 * sizeof(int));
  if (e == cudaSuccess) h->d_blocks_done = h->d_status + 1;
  unsigned long long s = seed;
  if (e == cudaSuccess) e = cudaMemcpy(h->d_state, &s, sizeof(s), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(h->d_state);
    cudaFree(h->d_status);
    cudaFreeHost(h->h_token);
    delete h;
    return fail(ETB200_MEMORY_ALLOCATION_FAILED, "device allocation failed: %s", cudaGetErrorString(e));
  }
  *out = h;
  return ETB200_OK;
}

int grid_blocks(etb200_sampler* h, int dtype, int64_t rows) {
  const int slot = dtype == kDtypeFloat ? 0 : (dtype == kDtypeHalf ? 1 : 2);
  if (h->blocks_per_sm[slot] == 0) h->blocks_per_sm[slot] = sample_kernel_max_blocks_per_sm(dtype);
  const int64_t resident = (int64_t)h->sm_count * h->blocks_per_sm[slot];
  return (int)(rows < resident ? rows : resident);
}

etb200_error_t ensure_retry_list(etb200_sampler* h, int64_t rows) {
  if (rows <= h->retry_cap) return ETB200_OK;
  if (h->d_retry) {
    ETB_CUDA(cudaDeviceSynchronize());
    ETB_CUDA(cudaFree(h->d_retry));
    h->d_retry = nullptr;
    h->retry_cap = 0;
  }
  const size_t bytes = sizeof(int) * (size_t)(rows + 2);
  cudaError_t e = cudaMalloc(&h->d_retry, bytes);
  if (e != cudaSuccess)
    return fail(ETB200_MEMORY_ALLOCATION_FAILED, "cudaMalloc of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
  ETB_CUDA(cudaMemset(h->d_retry, 0, 2 * sizeof(int)));
  h->retry_cap = rows;
  return ETB200_OK;
}

// Rows per launch of the cluster kernel pair: bounds the record scratch (about 110 KB per row
// at a 128k vocabulary).
constexpr int64_t kClusterBatchRows = 1024;

etb200_error_t ensure_cluster_scratch(etb200_sampler* h, int64_t batch_rows) {
  const size_t need = topp_cluster_scratch_bytes(h->vocab, batch_rows);
  if (need <= h->cluster_scratch_bytes) return ETB200_OK;
  if (h->cluster_scratch) {
    ETB_CUDA(cudaDeviceSynchronize());
    ETB_CUDA(cudaFree(h->cluster_scratch));
    h->cluster_scratch = nullptr;
    h->cluster_scratch_bytes = 0;
  }
  cudaError_t e = cudaMalloc(&h->cluster_scratch, need);
  if (e != cudaSuccess)
    return fail(ETB200_MEMORY_ALLOCATION_FAILED, "cudaMalloc of %zu scratch bytes failed: %s", need,
                cudaGetErrorString(e));
  h->cluster_scratch_bytes = need;
  return ETB200_OK;
}

etb200_error_t ensure_scratch(etb200_sampler* h, int blocks) {
  const size_t need = sampler_scratch_bytes(h->vocab, blocks);
  if (need <= h->scratch_bytes) return ETB200_OK;
  if (h->scratch) {
    ETB_CUDA(cudaDeviceSynchronize());
    ETB_CUDA(cudaFree(h->scratch));
    h->scratch = nullptr;
    h->scratch_bytes = 0;
  }
  cudaError_t e = cudaMalloc(&h->scratch, need);
  if (e != cudaSuccess)
    return fail(ETB200_MEMORY_ALLOCATION_FAILED, "cudaMalloc of %zu scratch bytes failed: %s", need,
                cudaGetErrorString(e));
  h->scratch_bytes = need;
  return ETB200_OK;
}

// Shared by the device- and host-buffer entry points. All pointers are device pointers.
etb200_error_t sample_rows_device(
    etb200_sampler* h, const void* logits, int dtype, int64_t rows, int64_t row_stride,
    unsigned long long* rng_states, int64_t* out_ids, cudaStream_t stream,
    const PeerOut& peers = PeerOut{}) {
  // a rank without rows still takes part in the arrival barrier: one block that only arrives
  if (rows == 0 && peers.epoch == 0ull) return ETB200_OK;
  if (h->inv_temperature == 0.0f || rows == 0) {
    // greedy: no coin is drawn and the RNG state does not move (sampler.cpp:226-228)
    int blocks = (int)(rows < (int64_t)h->sm_count * 4 ? rows : (int64_t)h->sm_count * 4);
    if (blocks < 1) blocks = 1;
    ETB_CUDA(launch_argmax_rows(rows == 0 ? kDtypeFloat : dtype, logits, rows, h->vocab, row_stride, out_ids, peers,
                                blocks, h->d_status, stream));
    h->launches += 1;
    return ETB200_OK;
  }
  if (dtype == kDtypeUInt16) {
    return fail(ETB200_NOT_SUPPORTED,
                "UInt16 logits are raw integers: only temperature 0 (argmax) is meaningful for them");
  }
  if (rng_states == nullptr) {
    ETB_CHECK_ARG(rows == 1, "rng_states may be NULL only for a single row (rows = %lld)", (long long)rows);
    rng_states = h->d_state;
  }
  // top-k when 0 < k < vocab, and then top-p is ignored (sampler.cpp:239-241)
  const int topk = (h->topk > 0 && h->topk < h->vocab) ? h->topk : 0;
  const bool use_topp = !(h->topp <= 0.0f || h->topp >= 1.0f);
  const int blocks = grid_blocks(h, dtype, rows);
  if (use_topp || topk > 0) {
    etb200_error_t err = ensure_scratch(h, blocks);
    if (err != ETB200_OK) return err;
  }
  // Automatic choice, from measurements on B200: the cluster pair is the quickest way to one
  // token from one long row (batch-1 decode); from a handful of rows on, one block per row
  // keeps more rows in flight and wins.
  const bool cluster_ok = topp_cluster_supported(dtype, logits, rows, h->vocab, row_stride, h->inv_temperature,
                                                 h->topp, topk);
  const bool want_cluster =
      cluster_ok && (h->kernel_choice == 2 || (h->kernel_choice == 0 && rows == 1 && h->vocab >= 65536));
  const bool want_guided = !want_cluster && h->kernel_choice == 3 && guided_supported(dtype);
  if (want_cluster || want_guided) {
    // Two launches: the fast kernel(s) take every row; the rows they leave undecided (rare) are
    // then sampled by the plain one-block-per-row kernel, which also carries the arrival
    // barrier of the multi-GPU forms.
    etb200_error_t err = ensure_retry_list(h, rows);
    if (err != ETB200_OK) return err;
    int* count = h->d_retry + (h->retry_parity & 1u);
    int* count_next = h->d_retry + ((h->retry_parity + 1u) & 1u);
    h->retry_parity += 1u;
    PeerOut no_barrier = peers;
    no_barrier.epoch = 0ull;
    if (want_cluster) {
      const int64_t batch = rows < kClusterBatchRows ? rows : kClusterBatchRows;
      err = ensure_cluster_scratch(h, batch);
      if (err != ETB200_OK) return err;
      ETB_CUDA(launch_topp_cluster(logits, rows, h->vocab, row_stride, h->inv_temperature, h->topp, rng_states,
                                   out_ids, no_barrier, h->table, h->cluster_scratch, batch, h->d_retry + 2,
                                   count, count_next, stream));
      h->launches += 2 * (uint64_t)((rows + batch - 1) / batch);
    } else {
      const int slot = dtype == kDtypeHalf ? 0 : 1;
      if (h->guided_blocks_per_sm[slot] == 0) h->guided_blocks_per_sm[slot] = guided_kernel_max_blocks_per_sm(dtype);
      const int64_t resident = (int64_t)h->sm_count * h->guided_blocks_per_sm[slot];
      const int gblocks = (int)(rows < resident ? rows : resident);
      if (gblocks > blocks) {
        err = ensure_scratch(h, gblocks);
        if (err != ETB200_OK) return err;
      }
      ETB_CUDA(launch_sample_rows_guided(dtype, logits, rows, h->vocab, row_stride, h->inv_temperature, h->topp,
                                         topk, rng_states, out_ids, no_barrier, h->scratch, gblocks, h->table,
                                         h->d_status, h->d_retry + 2, count, count_next, stream));
      h->launches += 1;
    }
    ETB_CUDA(launch_sample_rows(
        dtype, logits, rows, h->vocab, row_stride, h->inv_temperature, h->topp, topk, rng_states,
        out_ids, peers, h->scratch, blocks, h->table, h->d_status, stream, h->d_retry + 2, count));
    h->launches += 1;
    return ETB200_OK;
  }
  ETB_CUDA(launch_sample_rows(
      dtype, logits, rows, h->vocab, row_stride, h->inv_temperature, h->topp, topk, rng_states,
      out_ids, peers, h->scratch, blocks, h->table, h->d_status, stream));
  h->launches += 1;
  return ETB200_OK;
}

etb200_error_t check_common(
    etb200_sampler* h, const void* logits, int dtype, int64_t rows, int64_t row_stride,
    const void* out_ids) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  ETB_CHECK_ARG(rows >= 0, "rows must be >= 0, got %lld", (long long)rows);
  if (rows == 0) return ETB200_OK;
  ETB_CHECK_ARG(logits != nullptr, "logits is null");
  ETB_CHECK_ARG(out_ids != nullptr, "output pointer is null");
  if (dtype_size(dtype) == 0) {
    // sample_from_logits aborts on other dtypes (util.h:30-34); here it is an error code
    return fail(ETB200_NOT_SUPPORTED, "unsupported logits dtype code %d (Half 5, Float 6, BFloat16 15, UInt16 27)", dtype);
  }
  ETB_CHECK_ARG(rows == 1 || row_stride == 0 || row_stride >= h->vocab,
                "row_stride_elems (%lld) is smaller than vocab_size (%d) and not 0", (long long)row_stride, h->vocab);
  return ETB200_OK;
}

}  // namespace

extern "C" {

etb200_error_t etb200_sampler_create(
    int32_t vocab_size, float temperature, float topp, uint64_t rng_seed, int32_t device,
    etb200_sampler_t** out_handle) {
  return create_impl(vocab_size, temperature, topp, rng_seed, device, out_handle);
}

etb200_error_t etb200_sampler_create_default(
    int32_t vocab_size, float temperature, int32_t device, etb200_sampler_t** out_handle) {
  return create_impl(vocab_size, temperature, 0.9f, (uint64_t)std::time(nullptr), device, out_handle);
}

etb200_error_t etb200_sampler_destroy(etb200_sampler_t* h) {
  if (!h) return ETB200_OK;
  DeviceGuard guard(h->device);
  cudaDeviceSynchronize();
  cudaFree(h->d_state);
  cudaFreeHost(h->h_token);
  cudaFree(h->d_status);
  cudaFree(h->scratch);
  cudaFree(h->d_retry);
  cudaFree(h->cluster_scratch);
  cudaFree(h->d_stage);
  cudaFree(h->d_stage_states);
  cudaFree(h->d_stage_ids);
  if (h->copy_stream) cudaStreamDestroy(h->copy_stream);
  for (cudaEvent_t ev : h->slice_ready)
    if (ev) cudaEventDestroy(ev);
  if (h->entry_event) cudaEventDestroy(h->entry_event);
  delete h;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_temperature(etb200_sampler_t* h, float temperature) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  if (temperature < 0.0f) temperature = 0.0f;
  h->inv_temperature = inv_temperature_of(temperature);
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_inv_temperature(etb200_sampler_t* h, float inv_temperature) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  h->inv_temperature = inv_temperature;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_topk(etb200_sampler_t* h, int32_t topk) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  h->topk = topk;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_wait_limit_ns(etb200_sampler_t* h, uint64_t nanoseconds) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  ETB_CHECK_ARG(nanoseconds >= 1000ull && nanoseconds <= 60000000000ull,
                "the wait limit must be between 1 microsecond and 60 seconds");
  h->wait_ns = nanoseconds;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_kernel_choice(etb200_sampler_t* h, int32_t choice) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  ETB_CHECK_ARG(choice >= 0 && choice <= 3, "choice must be 0, 1, 2 or 3, got %d", choice);
  h->kernel_choice = choice;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_last_retry_count(etb200_sampler_t* h, int32_t* out_count) {
  ETB_CHECK_ARG(h != nullptr && out_count != nullptr, "null argument");
  *out_count = 0;
  if (h->d_retry == nullptr || h->retry_parity == 0u) return ETB200_OK;
  DeviceGuard guard(h->device);
  int v = 0;
  ETB_CUDA(cudaMemcpy(&v, h->d_retry + ((h->retry_parity - 1u) & 1u), sizeof(int), cudaMemcpyDeviceToHost));
  *out_count = v;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_get_rng_state(etb200_sampler_t* h, uint64_t* out_state) {
  ETB_CHECK_ARG(h != nullptr && out_state != nullptr, "null argument");
  DeviceGuard guard(h->device);
  unsigned long long s = 0;
  ETB_CUDA(cudaMemcpy(&s, h->d_state, sizeof(s), cudaMemcpyDeviceToHost));
  *out_state = s;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_set_rng_state(etb200_sampler_t* h, uint64_t state) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  DeviceGuard guard(h->device);
  unsigned long long s = state;
  ETB_CUDA(cudaMemcpy(h->d_state, &s, sizeof(s), cudaMemcpyHostToDevice));
  return ETB200_OK;
}

etb200_error_t etb200_sampler_sample(
    etb200_sampler_t* h, const void* logits_device, int32_t dtype, void* stream,
    int32_t* out_token) {
  etb200_error_t err = check_common(h, logits_device, dtype, 1, 0, out_token);
  if (err != ETB200_OK) return err;
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // the kernel's last store goes to mapped host memory: the read-back needs no copy of its own
  err = sample_rows_device(h, logits_device, dtype, 1, h->vocab, nullptr, h->h_token_dev, st);
  if (err != ETB200_OK) return err;
  ETB_CUDA(cudaStreamSynchronize(st));
  *out_token = (int32_t)*h->h_token;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_sample_rows(
    etb200_sampler_t* h, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* out_ids_device, void* stream) {
  etb200_error_t err = check_common(h, logits_device, dtype, rows, row_stride_elems, out_ids_device);
  if (err != ETB200_OK) return err;
  DeviceGuard guard(h->device);
  return sample_rows_device(
      h, logits_device, dtype, rows, row_stride_elems,
      reinterpret_cast<unsigned long long*>(rng_states_device), out_ids_device,
      static_cast<cudaStream_t>(stream));
}

etb200_error_t etb200_sampler_sample_rows_ex(
    etb200_sampler_t* h, void* logits_device, int32_t dtype, int64_t rows, int64_t row_stride_elems,
    uint64_t* rng_states_device, int64_t* out_ids_device, const etb200_row_options_t* opt, void* stream) {
  etb200_error_t err = check_common(h, logits_device, dtype, rows, row_stride_elems, out_ids_device);
  if (err != ETB200_OK) return err;
  if (rows == 0) return ETB200_OK;
  etb200_row_options_t none = {};
  none.scale = 1.0f;
  if (opt == nullptr) opt = &none;
  ETB_CHECK_ARG(opt->scale > 0.0f && opt->scale < 3.0e38f, "scale must be a positive finite number, got %g",
                (double)opt->scale);
  ETB_CHECK_ARG(opt->n_edits >= 0, "n_edits must be >= 0");
  ETB_CHECK_ARG(opt->n_edits == 0 || (opt->edit_ids_device != nullptr && opt->edit_bias_device != nullptr),
                "edit_ids_device / edit_bias_device are null but n_edits is %lld", (long long)opt->n_edits);
  ETB_CHECK_ARG(opt->n_edits == 0 || row_stride_elems >= h->vocab || rows == 1,
                "edits need rows that do not share memory (row_stride_elems >= vocab_size)");
  if (dtype == kDtypeUInt16)
    return fail(ETB200_NOT_SUPPORTED, "UInt16 logits are raw integers: only etb200_sampler_sample_rows at temperature 0");
  DeviceGuard guard(h->device);
  unsigned long long* states = reinterpret_cast<unsigned long long*>(rng_states_device);
  const bool all_greedy = h->inv_temperature == 0.0f && opt->temperature_device == nullptr;
  if (states == nullptr && !all_greedy) {
    ETB_CHECK_ARG(rows == 1, "rng_states may be NULL only for a single row (rows = %lld)", (long long)rows);
    states = h->d_state;
  }
  const int blocks = grid_blocks(h, dtype, rows);
  err = ensure_scratch(h, blocks);  // a row may use top-p or top-k whatever the handle says
  if (err != ETB200_OK) return err;
  RowSettings rs;
  rs.temperature = opt->temperature_device;
  rs.topp = opt->topp_device;
  rs.topk = opt->topk_device;
  rs.scale = opt->scale;
  RowEdits ed;
  ed.offsets = reinterpret_cast<const long long*>(opt->edit_offsets_device);
  ed.ids = opt->n_edits > 0 ? opt->edit_ids_device : nullptr;
  ed.bias = opt->edit_bias_device;
  ed.n_shared = opt->n_edits;
  const int topk = (h->topk > 0 && h->topk < h->vocab) ? h->topk : 0;
  ETB_CUDA(launch_sample_rows_ext(dtype, logits_device, rows, h->vocab, row_stride_elems, h->inv_temperature,
                                  h->topp, topk, rs, ed, states, out_ids_device, h->scratch, blocks, h->table,
                                  h->d_status, static_cast<cudaStream_t>(stream)));
  h->launches += opt->n_edits > 0 ? 2 : 1;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_sample_rows_scatter(
    etb200_sampler_t* h, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* const* dest_buffers,
    int32_t n_dest, int64_t dest_offset, void* stream) {
  ETB_CHECK_ARG(dest_buffers != nullptr, "dest_buffers is null");
  ETB_CHECK_ARG(n_dest >= 1 && n_dest <= kMaxPeers, "n_dest must be in [1, %d], got %d", kMaxPeers, n_dest);
  ETB_CHECK_ARG(dest_offset >= 0, "dest_offset must be >= 0");
  PeerOut peers{};
  for (int i = 0; i < n_dest; ++i) {
    ETB_CHECK_ARG(dest_buffers[i] != nullptr, "dest_buffers[%d] is null", i);
    peers.ptr[i] = dest_buffers[i];
  }
  peers.n = n_dest;
  peers.offset = dest_offset;
  etb200_error_t err = check_common(h, logits_device, dtype, rows, row_stride_elems, dest_buffers[0]);
  if (err != ETB200_OK) return err;
  DeviceGuard guard(h->device);
  return sample_rows_device(
      h, logits_device, dtype, rows, row_stride_elems,
      reinterpret_cast<unsigned long long*>(rng_states_device), nullptr,
      static_cast<cudaStream_t>(stream), peers);
}

etb200_error_t etb200_sampler_sample_rows_exchange(
    etb200_sampler_t* h, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* const* dest_buffers,
    uint64_t* const* arrive_marks, int32_t n_dest, int32_t my_rank, int64_t dest_offset,
    uint64_t epoch, void* stream) {
  ETB_CHECK_ARG(h != nullptr, "handle is null");
  ETB_CHECK_ARG(dest_buffers != nullptr && arrive_marks != nullptr, "dest_buffers or arrive_marks is null");
  ETB_CHECK_ARG(n_dest >= 1 && n_dest <= kMaxPeers, "n_dest must be in [1, %d], got %d", kMaxPeers, n_dest);
  ETB_CHECK_ARG(my_rank >= 0 && my_rank < n_dest, "my_rank %d is outside [0, %d)", my_rank, n_dest);
  ETB_CHECK_ARG(dest_offset >= 0, "dest_offset must be >= 0");
  ETB_CHECK_ARG(epoch != 0, "epoch must not be 0");
  ETB_CHECK_ARG(rows >= 0, "rows must be >= 0");
  PeerOut peers{};
  for (int i = 0; i < n_dest; ++i) {
    ETB_CHECK_ARG(dest_buffers[i] != nullptr && arrive_marks[i] != nullptr,
                  "dest_buffers[%d] or arrive_marks[%d] is null", i, i);
    peers.ptr[i] = dest_buffers[i];
    peers.arrive[i] = reinterpret_cast<unsigned long long*>(arrive_marks[i]);
  }
  peers.n = n_dest;
  peers.offset = dest_offset;
  peers.epoch = epoch;
  peers.rank = my_rank;
  peers.blocks_done = h->d_blocks_done;
  peers.wait_ns = h->wait_ns;
  if (rows > 0) {
    etb200_error_t err = check_common(h, logits_device, dtype, rows, row_stride_elems, dest_buffers[0]);
    if (err != ETB200_OK) return err;
  }
  DeviceGuard guard(h->device);
  return sample_rows_device(
      h, logits_device, dtype, rows, row_stride_elems,
      reinterpret_cast<unsigned long long*>(rng_states_device), nullptr,
      static_cast<cudaStream_t>(stream), peers);
}

etb200_error_t etb200_sampler_get_status(etb200_sampler_t* h, int32_t* out_status) {
  ETB_CHECK_ARG(h != nullptr && out_status != nullptr, "null argument");
  DeviceGuard guard(h->device);
  int v = 0;
  ETB_CUDA(cudaMemcpy(&v, h->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    const int zero = 0;
    ETB_CUDA(cudaMemcpy(h->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice));
  }
  *out_status = v;
  return ETB200_OK;
}

etb200_error_t etb200_sampler_sample_rows_host(
    etb200_sampler_t* h, const void* logits_host, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_host, int64_t* out_ids_host, void* stream) {
  etb200_error_t err = check_common(h, logits_host, dtype, rows, row_stride_elems, out_ids_host);
  if (err != ETB200_OK) return err;
  if (rows == 0) return ETB200_OK;
  const bool greedy = (h->inv_temperature == 0.0f);
  ETB_CHECK_ARG(greedy || rng_states_host != nullptr, "rng_states_host is null");
  DeviceGuard guard(h->device);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t esz = dtype_size(dtype);
  const size_t bytes = ((size_t)(rows - 1) * (size_t)row_stride_elems + (size_t)h->vocab) * esz;
  if (bytes > h->stage_bytes) {
    ETB_CUDA(cudaDeviceSynchronize());
    cudaFree(h->d_stage);
    h->d_stage = nullptr;
    h->stage_bytes = 0;
    cudaError_t e = cudaMalloc(&h->d_stage, bytes);
    if (e != cudaSuccess)
      return fail(ETB200_MEMORY_ALLOCATION_FAILED, "cudaMalloc of %zu staging bytes failed: %s", bytes,
                  cudaGetErrorString(e));
    h->stage_bytes = bytes;
  }
  if (rows > h->stage_rows) {
    ETB_CUDA(cudaDeviceSynchronize());
    cudaFree(h->d_stage_states);
    cudaFree(h->d_stage_ids);
    h->d_stage_states = nullptr;
    h->d_stage_ids = nullptr;
    h->stage_rows = 0;
    cudaError_t e = cudaMalloc(&h->d_stage_states, sizeof(unsigned long long) * (size_t)rows);
    if (e == cudaSuccess) e = cudaMalloc(&h->d_stage_ids, sizeof(int64_t) * (size_t)rows);
    if (e != cudaSuccess)
      return fail(ETB200_MEMORY_ALLOCATION_FAILED, "cudaMalloc of staging ids/states failed: %s",
                  cudaGetErrorString(e));
    h->stage_rows = rows;
  }
  if (!greedy) {
    ETB_CUDA(cudaMemcpyAsync(h->d_stage_states, rng_states_host, sizeof(uint64_t) * (size_t)rows,
                             cudaMemcpyHostToDevice, st));
  }
  // Large batches go in slices of whole rows: slice k+1 crosses PCIe on the handle's copy
  // stream while slice k is sampled on the caller's stream, so that only the last slice's
  // kernel is not hidden behind the copy. Slices stay above 32 rows and 4 MB each.
  int slices = 1;
  if (row_stride_elems >= h->vocab) {
    const int64_t by_rows = rows / 32;
    const int64_t by_bytes = (int64_t)(bytes >> 22);
    int64_t n = by_rows < by_bytes ? by_rows : by_bytes;
    if (n > etb200_sampler::kMaxSlices) n = etb200_sampler::kMaxSlices;
    if (n > 1) slices = (int)n;
  }
  if (slices == 1) {
    ETB_CUDA(cudaMemcpyAsync(h->d_stage, logits_host, bytes, cudaMemcpyHostToDevice, st));
    err = sample_rows_device(h, h->d_stage, dtype, rows, row_stride_elems, h->d_stage_states,
                             h->d_stage_ids, st);
    if (err != ETB200_OK) return err;
  } else {
    if (!h->copy_stream) {
      ETB_CUDA(cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking));
      ETB_CUDA(cudaEventCreateWithFlags(&h->entry_event, cudaEventDisableTiming));
      for (cudaEvent_t& ev : h->slice_ready) ETB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    }
    // the copies must not overtake work already queued on the caller's stream
    ETB_CUDA(cudaEventRecord(h->entry_event, st));
    ETB_CUDA(cudaStreamWaitEvent(h->copy_stream, h->entry_event, 0));
    const int64_t per = (rows + slices - 1) / slices;
    const char* src = static_cast<const char*>(logits_host);
    char* dst = static_cast<char*>(h->d_stage);
    for (int k = 0; k < slices; ++k) {
      const int64_t r0 = k * per;
      const int64_t n = (r0 + per <= rows) ? per : rows - r0;
      if (n <= 0) break;
      const size_t off = (size_t)r0 * (size_t)row_stride_elems * esz;
      const size_t len = ((size_t)(n - 1) * (size_t)row_stride_elems + (size_t)h->vocab) * esz;
      ETB_CUDA(cudaMemcpyAsync(dst + off, src + off, len, cudaMemcpyHostToDevice, h->copy_stream));
      ETB_CUDA(cudaEventRecord(h->slice_ready[k], h->copy_stream));
      ETB_CUDA(cudaStreamWaitEvent(st, h->slice_ready[k], 0));
      err = sample_rows_device(h, dst + off, dtype, n, row_stride_elems, h->d_stage_states + r0,
                               h->d_stage_ids + r0, st);
      if (err != ETB200_OK) {
        cudaStreamSynchronize(h->copy_stream);
        return err;
      }
    }
  }
  ETB_CUDA(cudaMemcpyAsync(out_ids_host, h->d_stage_ids, sizeof(int64_t) * (size_t)rows,
                           cudaMemcpyDeviceToHost, st));
  if (!greedy) {
    ETB_CUDA(cudaMemcpyAsync(rng_states_host, h->d_stage_states, sizeof(uint64_t) * (size_t)rows,
                             cudaMemcpyDeviceToHost, st));
  }
  ETB_CUDA(cudaStreamSynchronize(st));
  return ETB200_OK;
}

etb200_error_t etb200_sampler_launch_count(etb200_sampler_t* h, uint64_t* out_count) {
  ETB_CHECK_ARG(h != nullptr && out_count != nullptr, "null argument");
  *out_count = h->launches;
  return ETB200_OK;
}

etb200_error_t etb200_selftest_expf(
    const float* x_device, float* y_device, int64_t n, void* stream) {
  ETB_CHECK_ARG(n >= 0, "n must be >= 0");
  if (n == 0) return ETB200_OK;
  ETB_CHECK_ARG(x_device != nullptr && y_device != nullptr, "null argument");
  ExpTable table;
  make_exp_table(&table);
  ETB_CUDA(launch_expf_selftest(x_device, y_device, n, table, static_cast<cudaStream_t>(stream)));
  return ETB200_OK;
}

const char* etb200_last_error_message(void) { return g_err; }

uint32_t etb200_sampler_abi_version(void) { return 1; }

}  // extern "C"
