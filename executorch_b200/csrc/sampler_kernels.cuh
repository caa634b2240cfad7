// Launch interface of the sampling kernels (sampler_kernels.cu). Host-only declarations;
// the C ABI in c_api.cu is the only caller.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "exact_math.cuh"

namespace etb200 {

// dtype codes = the reference's ScalarType numbering
// (runtime/core/portable_type/scalar_type.h:98-125)
constexpr int kDtypeHalf = 5;
constexpr int kDtypeFloat = 6;
constexpr int kDtypeBFloat16 = 15;
constexpr int kDtypeUInt16 = 27;

// Optional destinations of the sampled ids: up to kMaxPeers int64 buffers (this GPU's and its
// peers' -- pointers obtained from symmetric / peer-mapped memory), each written at
// [offset + row]. n == 0 means "write out_ids[row] only".
constexpr int kMaxPeers = 16;
struct PeerOut {
  int64_t* ptr[kMaxPeers];
  int n;
  long long offset;
  // Optional arrival barrier at the end of the launch (epoch != 0): arrive[p] is rank p's
  // array of kMaxPeers 64-bit arrival marks. When the last block of this launch is done it
  // writes `epoch` into arrive[p][rank] of every rank p and then waits, at most wait_ns, until
  // arrive[rank][q] >= epoch for every q: when the launch completes, this GPU's buffer holds
  // the ids of all ranks. blocks_done is a counter of this GPU that is zero between launches.
  unsigned long long* arrive[kMaxPeers];
  unsigned long long epoch;
  int rank;
  int* blocks_done;
  unsigned long long wait_ns;  // limit of that wait, in nanoseconds of the GPU's global timer
};

// Per-row settings of the extended entry point (device arrays of `rows` entries, or null for
// "the handle's value"), and the scalar that multiplies every logit (1 = none).
struct RowSettings {
  const float* temperature;
  const float* topp;
  const int* topk;
  float scale;
};

// Sparse in-place edits of the logits before sampling (mask / bias logit processors): entry j
// adds bias[j] to logit ids[j] of its row (-inf masks the token; ids outside [0, vocab) are
// ignored). Row r owns entries [offsets[r], offsets[r + 1]) and n_shared is the total number of
// entries; with offsets == null the n_shared entries apply to every row. All pointers are
// device pointers; ids == null means "no edits".
struct RowEdits {
  const long long* offsets;
  const int* ids;
  const float* bias;
  long long n_shared;
};

// Bytes of candidate-list scratch the sampling kernel needs when launched with `blocks`
// thread blocks on rows of `vocab` logits.
size_t sampler_scratch_bytes(int vocab, int blocks);

// Resident thread blocks per SM of the sampling kernel for a dtype (occupancy query).
int sample_kernel_max_blocks_per_sm(int dtype);

int sampler_threads();

// temperature != 0: top-k (0 < topk < vocab), else multinomial (topp outside (0,1)) or top-p
// sampling of every row. rng_states[r] is advanced once per row; out_ids[r] receives the
// token. Top-k and top-p need `scratch` (sampler_scratch_bytes). With row_list, only the
// *row_count rows it names are sampled (both are device pointers).
cudaError_t launch_sample_rows(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t,
    float topp, int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers,
    void* scratch, int blocks, const ExpTable& table, int* status, cudaStream_t stream,
    const int* row_list = nullptr, const int* row_count = nullptr);

// launch_sample_rows for 16-bit logits with the estimate-guided exact sum (the default path):
// every row is sampled unless the kernel cannot decide it, in which case the row -- rng state
// and output untouched -- is appended to retry_rows (count in *retry_count, which must be zero
// at launch) and the caller runs launch_sample_rows with that list on the same stream.
bool guided_supported(int dtype);
int guided_kernel_max_blocks_per_sm(int dtype);
cudaError_t launch_sample_rows_guided(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t,
    float topp, int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers,
    void* scratch, int blocks, const ExpTable& table, int* status, int* retry_rows, int* retry_count,
    int* retry_count_next, cudaStream_t stream);

// Top-p sampling of bf16 rows with one thread-block cluster per row (an alternative
// decomposition, selectable per handle): per batch of at most batch_rows rows, one kernel that turns every row into a short list of
// records in `scratch` (topp_cluster_scratch_bytes) and one that replays them and draws the
// token. Rows that cannot be decided this way are appended to retry_rows (their count in
// *retry_count) with their rng state and output untouched; the caller then runs
// launch_sample_rows with that list on the same stream. *retry_count must be zero when the
// first kernel starts; *retry_count_next is cleared for the call after this one.
constexpr int kClusterMinVocab = 256;
bool topp_cluster_supported(int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride,
                            float inv_t, float topp, int topk);
size_t topp_cluster_scratch_bytes(int vocab, int64_t batch_rows);
cudaError_t launch_topp_cluster(
    const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers, const ExpTable& table,
    void* scratch, int64_t batch_rows, int* retry_rows, int* retry_count, int* retry_count_next,
    cudaStream_t stream);

// The extended form of launch_sample_rows: first the edits are applied to the logits in
// place (one thread per edit), then every row is sampled with its own settings; a row whose
// temperature is 0 takes the argmax. `logits` is written only at the edited positions.
cudaError_t launch_sample_rows_ext(
    int dtype, void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    int topk, const RowSettings& settings, const RowEdits& edits, unsigned long long* rng_states,
    int64_t* out_ids, void* scratch, int blocks, const ExpTable& table, int* status, cudaStream_t stream);

// temperature == 0: greedy argmax of every row.
cudaError_t launch_argmax_rows(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, int64_t* out_ids,
    const PeerOut& peers, int blocks, int* status, cudaStream_t stream);

// Value stored into `status` when the arrival barrier of PeerOut gave up waiting for a rank.
constexpr int kStatusPeerTimeout = 2;
constexpr int kStatusTailInconsistent = 3;  // the long-nucleus tail's final lookup found its counts inconsistent

// y[i] = expf_ref(x[i]) on the device, for x <= 0: lets a test compare the device
// exponential with the host libm.
cudaError_t launch_expf_selftest(const float* x, float* y, int64_t n, const ExpTable& table,
                                 cudaStream_t stream);

}  // namespace etb200
