/*
 * C ABI of the B200 token sampler: a drop-in for the sampling step of ExecuTorch's LLM
 * runner, i.e. executorch::extension::llm::Sampler (extension/llm/sampler/sampler.h:37-83)
 * as called through sample_from_logits / logits_to_token (extension/llm/sampler/util.h:25-71)
 * by TextDecoderRunner::logits_to_token (extension/llm/runner/text_decoder_runner.h:84-94).
 *
 * Conventions (the ones of the reference's CUDA shims, backends/cuda/runtime/shims/rand.h:
 * extern "C", error code returned, results through out-pointers, no exceptions, no C++
 * types):
 *  - every function returns an etb200_error_t whose values are the reference's
 *    executorch::runtime::Error codes (runtime/core/error.h:29-100);
 *  - dtype arguments use the reference's ScalarType numbering
 *    (runtime/core/portable_type/scalar_type.h:98-125): Half 5, Float 6, BFloat16 15,
 *    UInt16 27;
 *  - `stream` is a cudaStream_t passed as void* (the caller's stream, as in
 *    extension/cuda/caller_stream.h); work is enqueued on it and, unless stated otherwise,
 *    NOT synchronised;
 *  - logits are read in place and never modified (the reference overwrites them with
 *    probabilities, sampler.cpp:231-235; its callers never read them again);
 *  - 16-bit logits are sampled with the reference's float arithmetic on their exact fp32
 *    upcast (what the reference's newer runners do,
 *    examples/models/gemma4/runner/gemma4_runner.cpp:166-182,308);
 *  - a sampler handle, like the reference's Sampler, is not thread-safe: callers serialise
 *    calls on one handle (text_decoder_runner.h:81-82); distinct handles are independent.
 *
 * There is no CPU fallback: without a CUDA device every call fails with an error code.
 */
#ifndef ETB200_SAMPLER_H_
#define ETB200_SAMPLER_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define ETB200_EXPORT __attribute__((visibility("default")))
#else
#define ETB200_EXPORT
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef uint32_t etb200_error_t;

/* executorch::runtime::Error values used by this library (runtime/core/error.h:29-100) */
enum {
  ETB200_OK = 0x00,
  ETB200_INTERNAL = 0x01,
  ETB200_INVALID_STATE = 0x02,
  ETB200_NOT_SUPPORTED = 0x10,
  ETB200_INVALID_ARGUMENT = 0x12,
  ETB200_MEMORY_ALLOCATION_FAILED = 0x21
};

/* ScalarType codes accepted for logits (scalar_type.h:98-125); the same four types that
 * sample_from_logits dispatches on (util.h:36-53). */
enum {
  ETB200_DTYPE_HALF = 5,
  ETB200_DTYPE_FLOAT = 6,
  ETB200_DTYPE_BFLOAT16 = 15,
  ETB200_DTYPE_UINT16 = 27
};

typedef struct etb200_sampler etb200_sampler_t;

/* Sampler::Sampler(vocab_size, temperature, topp, rng_seed), sampler.cpp:173-181.
 * temperature 0 selects greedy argmax; it is not clamped here (a negative value keeps
 * 1/temperature, as in the reference). `device` is the CUDA device ordinal that owns the
 * handle's state and scratch memory; -1 means the calling thread's current device. */
ETB200_EXPORT etb200_error_t etb200_sampler_create(
    int32_t vocab_size, float temperature, float topp, uint64_t rng_seed, int32_t device,
    etb200_sampler_t** out_handle);

/* Sampler::Sampler(vocab_size, temperature), sampler.cpp:183-187: topp = 0.9 (kTopp,
 * sampler.h:29) and the seed is the wall-clock time in seconds. */
ETB200_EXPORT etb200_error_t etb200_sampler_create_default(
    int32_t vocab_size, float temperature, int32_t device, etb200_sampler_t** out_handle);

/* ~Sampler: frees the handle's device memory (synchronises the device). */
ETB200_EXPORT etb200_error_t etb200_sampler_destroy(etb200_sampler_t* handle);

/* Sampler::set_temperature, sampler.h:48-53: negative values are reset to 0. */
ETB200_EXPORT etb200_error_t etb200_sampler_set_temperature(
    etb200_sampler_t* handle, float temperature);

/* Sets Sampler::inv_temperature_ (sampler.h:78) directly: for a binding that keeps the
 * reference's own member and must hand its exact value on (1 / (1 / T) is not always T). */
ETB200_EXPORT etb200_error_t etb200_sampler_set_inv_temperature(
    etb200_sampler_t* handle, float inv_temperature);

/* Sampler::set_topk, sampler.h:58-60. k <= 0 or k >= vocab_size disables top-k; an active
 * top-k takes precedence over top-p (sampler.cpp:239-241). */
ETB200_EXPORT etb200_error_t etb200_sampler_set_topk(etb200_sampler_t* handle, int32_t topk);

/* Reads back / replaces the handle's own xorshift64* state (Sampler::rng_state_,
 * sampler.h:82), so that a caller can checkpoint and resume a decode loop. Synchronises. */
ETB200_EXPORT etb200_error_t etb200_sampler_get_rng_state(
    etb200_sampler_t* handle, uint64_t* out_state);
ETB200_EXPORT etb200_error_t etb200_sampler_set_rng_state(
    etb200_sampler_t* handle, uint64_t state);

/* int32_t Sampler::sample<T>(T* logits), sampler.cpp:222-251, for ONE row of vocab_size
 * logits in device memory. Uses and advances the handle's own RNG state. Synchronises the
 * stream and returns the token through out_token (host memory). */
ETB200_EXPORT etb200_error_t etb200_sampler_sample(
    etb200_sampler_t* handle, const void* logits_device, int32_t dtype, void* stream,
    int32_t* out_token);

/* Batched extension of Sampler::sample: samples `rows` independent rows
 * (row r starts at logits + r * row_stride_elems elements; a stride of 0 samples the same
 * row `rows` times, once per RNG state) with one launch.
 *   rng_states: device array of `rows` xorshift64* states, one per row, read and advanced
 *               once per row exactly like Sampler::rng_state_ (sampler.cpp:210-220,237);
 *               initialise it with the per-row seeds. Not touched when temperature == 0.
 *               May be NULL only when rows == 1 (the handle's own state is used).
 *   out_ids:    device array of `rows` int64 token ids.
 * The first top-p call on a handle (and any later call that needs more) allocates the
 * handle's candidate-list scratch memory with cudaMalloc. */
ETB200_EXPORT etb200_error_t etb200_sampler_sample_rows(
    etb200_sampler_t* handle, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* out_ids_device,
    void* stream);

/* Per-row settings and logit edits for etb200_sampler_sample_rows_ex. Every pointer is a device
 * pointer and may be NULL ("not used"). */
typedef struct {
  /* SamplingConfig{temperature, top_p, top_k} per request (extension/llm/runner/llm_session.h:
   * 29-34; the seed is the row's RNG state): arrays of `rows` entries that replace the handle's
   * setting for each row. A temperature <= 0 makes that row greedy (its state is not advanced);
   * top_k outside (0, vocab_size) means "no top-k"; top_p outside (0, 1) means multinomial. */
  const float* temperature_device;
  const float* topp_device;
  const int32_t* topk_device;
  /* A "multiply" logit processor (logit_processor.h:34-40) folded into the kernel's reads: every
   * logit is seen as T(logit * scale), T the logits' dtype. Must be > 0; 1 = none. */
  float scale;
  /* Mask / bias logit processors: entry j adds edit_bias[j] to logit edit_ids[j] of its row, in
   * place, rounded to the logits' dtype (-inf masks the token; ids outside [0, vocab_size) are
   * ignored, as the reference's processors ignore them). With edit_offsets (rows + 1 entries,
   * ascending, edit_offsets[rows] == n_edits) row r owns entries [edit_offsets[r],
   * edit_offsets[r + 1]); without, all n_edits entries apply to every row. Edits are applied
   * before the multiply, and before sampling; only the edited logits are written. */
  const int64_t* edit_offsets_device;
  const int32_t* edit_ids_device;
  const float* edit_bias_device;
  int64_t n_edits;
} etb200_row_options_t;

/* etb200_sampler_sample_rows for a serving batch whose rows carry their own settings, with the
 * usual logit processors applied on the device: what apply_logit_processors + logits_to_token do
 * per request in the decode loop (extension/llm/runner/text_token_generator.h:143-148), for all
 * rows in one launch (two when there are edits: they are scattered into the logits first, one
 * thread per edit, so no processor costs a pass over the logits). `logits_device` is therefore
 * not const; `options` may be NULL. No multi-GPU form. */
ETB200_EXPORT etb200_error_t etb200_sampler_sample_rows_ex(
    etb200_sampler_t* handle, void* logits_device, int32_t dtype, int64_t rows, int64_t row_stride_elems,
    uint64_t* rng_states_device, int64_t* out_ids_device, const etb200_row_options_t* options, void* stream);

/* Multi-GPU form of etb200_sampler_sample_rows (no counterpart in the reference, which is
 * single-device): instead of one out_ids array, the kernel's epilogue stores the id of row r
 * into EVERY buffer dest_buffers[0..n_dest) at index dest_offset + r. The buffers are int64
 * device arrays that this process can address: its own and its peers' (symmetric / peer-mapped
 * memory of the GPUs of one node), so that after a barrier among the ranks every GPU holds
 * all ids without a separate all-gather. dest_buffers is a HOST array of n_dest (<= 16) device
 * pointers. Asynchronous on `stream`; the caller provides the cross-GPU barrier. */
ETB200_EXPORT etb200_error_t etb200_sampler_sample_rows_scatter(
    etb200_sampler_t* handle, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* const* dest_buffers,
    int32_t n_dest, int64_t dest_offset, void* stream);

/* etb200_sampler_sample_rows_scatter with the cross-GPU synchronisation inside the same
 * launch (no counterpart in the reference). arrive_marks is a HOST array of n_dest device
 * pointers: arrive_marks[p] is an array of at least n_dest uint64 in rank p's memory that
 * every rank can address (symmetric / peer-mapped memory), zero before the first call. When
 * the last thread block of this launch has stored its ids, it writes `epoch` into
 * arrive_marks[p][my_rank] for every p and then waits until arrive_marks[my_rank][q] >= epoch
 * for every q: once the launch has completed on `stream`, this rank's buffer holds the ids
 * of all ranks for this epoch. Every rank must make the call with the same epoch, which must
 * grow from call to call (1, 2, 3, ...); a rank with rows == 0 still calls. The wait is
 * limited (one second of the GPU's global timer unless etb200_sampler_set_wait_limit_ns says
 * otherwise); if it runs out the launch ends normally, etb200_sampler_get_status reports 2 and
 * the ids of the missing ranks are stale: check the status before trusting a buffer. Ranks
 * must be distinct GPUs: two such launches never wait for each other on one GPU. A handle's
 * exchange launches must not overlap each other (they share one block counter). */
ETB200_EXPORT etb200_error_t etb200_sampler_sample_rows_exchange(
    etb200_sampler_t* handle, const void* logits_device, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* const* dest_buffers,
    uint64_t* const* arrive_marks, int32_t n_dest, int32_t my_rank, int64_t dest_offset,
    uint64_t epoch, void* stream);

/* Limit of the in-kernel wait of etb200_sampler_sample_rows_exchange, in nanoseconds
 * (1 microsecond to 60 seconds; default one second). */
ETB200_EXPORT etb200_error_t etb200_sampler_set_wait_limit_ns(etb200_sampler_t* handle, uint64_t nanoseconds);

/* Reads and clears the handle's device status word (synchronises): 0 = nothing to report,
 * 2 = the arrival wait of etb200_sampler_sample_rows_exchange ran out for some rank,
 * 3 = an internal consistency check of the long-nucleus top-p tail failed for some row since
 * the last read (that row's id is 0 and not to be trusted; not expected to happen). */
ETB200_EXPORT etb200_error_t etb200_sampler_get_status(etb200_sampler_t* handle, int32_t* out_status);

/* Same as etb200_sampler_sample_rows for callers whose logits live in HOST memory (what
 * sample_from_logits receives from a CPU tensor, util.h:25-55): copies the rows to the
 * device, samples, copies ids and advanced states back, and synchronises the stream.
 * rng_states_host must hold `rows` states (ignored when temperature == 0). */
ETB200_EXPORT etb200_error_t etb200_sampler_sample_rows_host(
    etb200_sampler_t* handle, const void* logits_host, int32_t dtype, int64_t rows,
    int64_t row_stride_elems, uint64_t* rng_states_host, int64_t* out_ids_host, void* stream);

/* No counterpart in the reference. For callers that may not allocate device memory: a
 * runtime living inside a pre-planned arena, a tenant with a fixed memory budget on a
 * shared GPU, a latency-critical loop that cannot take the implicit synchronisation of
 * cudaMalloc/cudaFree.
 * Same sampling as etb200_sampler_sample_rows (temperature, top-p / multinomial / argmax,
 * per-row xorshift64* states advanced in place, int64 ids out) but without a handle and
 * without any allocation: the kernel's candidate lists live in a fixed 64 MiB array inside
 * the library image (every GPU that loads the library holds those 64 MiB until exit).
 *   - Runs on the CURRENT CUDA device; enqueues on `stream`; does not synchronise.
 *   - Limit (top-p calls, the only ones that use the array): 16 * vocab_size bytes must fit
 *     it, i.e. vocab_size <= 4194304; larger sizes are refused with ETB200_INVALID_ARGUMENT.
 *     Fewer thread blocks run at once than with a handle (32 at a 131072-entry vocabulary), so
 *     large top-p batches are slower. Argmax and multinomial calls are not limited.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before starting any stream capture.
 *   - All calls share the one array. Nothing in it has to start at zero (each call writes
 *     its lists before reading them), and its contents after a call are meaningless. Two
 *     calls whose kernels overlap on the same GPU (different streams, threads or
 *     processes' contexts sharing the library image) race on it: serialise them.
 *   - No top-k; rng_states_device is required whenever temperature != 0.
 * Errors of this function are described by etb200_static_last_error_message(). */
ETB200_EXPORT etb200_error_t etb200_sample_rows_static(
    int32_t vocab_size, float temperature, float topp, const void* logits_device, int32_t dtype,
    int64_t rows, int64_t row_stride_elems, uint64_t* rng_states_device, int64_t* out_ids_device,
    void* stream);
ETB200_EXPORT const char* etb200_static_last_error_message(void);

/* Diagnostic: y[i] = the library's device expf(x[i]) for n floats x <= 0 in device memory.
 * The sampler's results depend on expf matching the host libm that the reference calls
 * (sampler.cpp:201) bit for bit; this lets a test verify that on the machine at hand. */
ETB200_EXPORT etb200_error_t etb200_selftest_expf(
    const float* x_device, float* y_device, int64_t n, void* stream);

/* Which sampling kernel a handle uses for temperature != 0 (a tuning and testing knob; no
 * counterpart in the reference). All choices return the same tokens.
 *   0 (default): automatic -- kernel 2 for a single bf16 row of 65536 logits or more (batch-1
 *      decode, where it is the quickest), kernel 1 otherwise.
 *   1: one thread block per row.
 *   2: a thread-block cluster per row plus a finishing kernel (top-p on bf16 rows whose starts
 *      are 16-byte aligned, 256 <= vocab_size <= 262144, temperature > 0, no top-k); other
 *      cases, and rows it cannot decide, fall to kernel 1.
 *   3: kernel 1 with the exact softmax sum formed from estimate-guided integer increments
 *      (16-bit logits); rows it cannot decide fall to kernel 1. */
ETB200_EXPORT etb200_error_t etb200_sampler_set_kernel_choice(etb200_sampler_t* handle, int32_t choice);

/* Diagnostic (synchronises the device): how many rows of the handle's most recent top-p call
 * the fast kernel left undecided and handed to the plain one-block-per-row kernel. */
ETB200_EXPORT etb200_error_t etb200_sampler_last_retry_count(etb200_sampler_t* handle, int32_t* out_count);

/* Number of kernels this library has launched through `handle` so far. */
ETB200_EXPORT etb200_error_t etb200_sampler_launch_count(
    etb200_sampler_t* handle, uint64_t* out_count);

/* Text of the last error raised on the calling thread ("" if none). */
ETB200_EXPORT const char* etb200_last_error_message(void);

/* ABI revision of this header. */
ETB200_EXPORT uint32_t etb200_sampler_abi_version(void);

#ifdef __cplusplus
}
#endif

#endif /* ETB200_SAMPLER_H_ */
