// Token-sampling kernels for sm_100a: greedy argmax, multinomial and top-p (nucleus)
// sampling of rows x vocab logits, reproducing ExecuTorch's CPU sampler
// (extension/llm/sampler/sampler.cpp) bit for bit on the fp32 upcast of the logits.
//
// Work decomposition: one thread block per row (blocks stride over the rows of a batch).
// Logits are read in place (bf16 / fp16 / fp32, 128-bit loads when the row is 16-byte
// aligned) and never written. A sampled row makes these passes:
//
//   1. max of the temperature-scaled logits                      (HBM read of the row)
//   2. e_i = expf(x_i - max), exact sequential-order float sum S (row re-read, L2 resident);
//      top-p also appends (e_i, i) of every possible nucleus member to a per-block list.
//      For bf16 logits e_i comes from a per-row table in shared memory indexed by the
//      logit's bit pattern (a bf16 row has few distinct values), so expf runs once per
//      table entry instead of once per logit.
//   3a. multinomial: exact running cdf of e_i / S in index order until it exceeds the coin
//   3b. top-p: pick a value threshold from a histogram of the list, compact the survivors
//       with p_i = e_i / S >= cutoff, LSD-radix sort them (probability descending, stable =
//       index ascending), replay the reference's cumulative sums exactly, draw.
//
// The candidate lists of 3b live in global scratch memory owned by the caller of the launch
// functions (two buffers of vocab entries per resident block).
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <type_traits>

#include "class_math.cuh"
#include "cluster_math.cuh"
#include "exact_math.cuh"
#include "sampler_kernels.cuh"

namespace etb200 {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kChunk = 16;                  // consecutive logits per thread per tile
constexpr int kTile = kThreads * kChunk;    // logits per tile
constexpr int kHead = 256;                  // leading terms of a sum that one thread adds sequentially
// Candidate values are binned by their float bits >> 21 (exponent + 2 mantissa bits). Bin
// kBins-1 holds 1.0; bin 0 also collects everything below the covered range (e < ~2.4e-10).
// Per bin two integers are kept: the count, and the sum of the 13 mantissa bits below the
// bin bits, which together give the bin's mass to about 2^-15 relative (always rounded
// down) without floating-point atomics.
constexpr int kBinShift = 21;
constexpr int kBins = 128;
constexpr int kBinTop = 0x3F800000 >> kBinShift;  // bin index of 1.0 before rebasing
constexpr int kBinBase = kBinTop - (kBins - 1);
constexpr int kRadixBits = 8;
constexpr int kRadix = 1 << kRadixBits;
constexpr int kFastSat = 1 << 25;           // per-thread clamp of chunk summaries
constexpr int kCompactSteps = 224;          // list entries compacted per segment = 448 * kThreads
constexpr float kGuessFloor = 1.0f / 8192.0f;  // first guess of a floor under the values that matter
constexpr int kListBatch = 8;               // list entries a thread loads before using any of them
constexpr int kRankSortMax = 512;           // survivor lists up to this size are rank-sorted in shared memory

// bf16 table of e by logit bit pattern: both signs, |logit| in [2^-16, 2^16). Anything else
// (zero, tiny, huge, infinite, NaN) is handled outside the table.
// Addressing is pure bit-field work so that it can run on both halves of a packed pair:
// adding kLutBias to a pattern moves the 32 covered exponents to 128..159, i.e. bits 14..12
// of the biased pattern are 100 exactly for covered values, and the slot is its low 12 bits
// (5 exponent bits, 7 mantissa bits) plus the sign as bit 12.
constexpr uint32_t kLutBias = (128u - (127u - 16u)) << 7;  // 0x0880
constexpr int kLutSize = 8192;
// A thread's kChunk staged terms are followed by 4 floats of padding: 128-bit reads of
// consecutive runs by consecutive lanes then fall into distinct banks.
constexpr int kStagePitch = kChunk + 4;

struct Entry {
  uint32_t key;  // float bits of e_i (list A) or p_i (sorted lists); positive floats order like integers
  int32_t idx;   // token index
};

// Shared state of the estimate-guided sum (guided_sum.cuh), present only in the kernel
// variant that uses it.
constexpr int kGTile = kThreads * kCTerms;  // logits per tile: one chunk of 32 per thread
constexpr int kGMaxTiles = 16;
constexpr int kGEventCap = 256;
constexpr int kGPoolCap = 112;

struct GuidedShared {
  unsigned long long mbar;  // completion barrier of the tile copies; phases alternate
  int ok;
  float sum;
  int ev_first[1];
  int ev_count[1];
  double wtot[2][kWarps];
  unsigned long long wx[2][kWarps];
  int wev[2][kWarps];
  int wst[2][kWarps];
  int wcand[2][kWarps];
  int wklo[2][kWarps];
  ChunkEvent events[kGEventCap];
  float pool[kGPoolCap][kCTerms];
  unsigned short kb[8][kThreads];  // per chunk of tiles 0..7: lower open binade | (open binades - 1) << 8
};
struct NoGuidedShared {};
static_assert(kGEventCap <= kThreads, "one thread per event resolves the pending summaries");

// Shared state of the value-class tail (value_class_tail.cuh): a window of class counts, later
// reused for per-(tile, thread) member counts, and the block's walk record.
constexpr int kVcBins = 16384;                 // 32-bit class counters of a window (or twice as many 16-bit ones)
constexpr int kVcPer = 4;                      // classes per thread in one round of the walk
constexpr int kVcTile = kThreads * kVcPer;
constexpr int kVcSelTile = kThreads * 32;      // logits per tile of the final lookup
constexpr int kVcSelTiles = kVcBins / kThreads;
constexpr int kVcListCap = 32768;              // a 16-bit top-p row with more listed candidates takes the class tail
constexpr int kVcListProbe = 2048;             // from this many on, the count so far is extrapolated to the whole row
constexpr int kVcMinNucleus = 4096;            // ... and so does one whose list is short of this many, at least
constexpr int kVcPendCap = 8;                  // deferred tails a block collects before it runs them
constexpr int kVcCheckpoints = 6;              // window starts of one row (65536 keys / kVcBins, and one)
static_assert(kVcPer == 4, "a thread reads its four class counts as one 128-bit (or 64-bit) word");

struct VcHist {
  alignas(16) unsigned hist[kVcBins];
};
struct NoVcHist {};
struct VcControl {
  SeqSummary wsum[kWarps], wpre[kWarps], tot;
  int wcnt[kWarps], wpre_cnt[kWarps], tot_cnt;
  int hit_tid, found, kb, n, hit_b, hit_j, hit_pos;
  float cum, p;
  int ended;
  unsigned last_key;
  int loaded_hi, n_ck;
  int ck_hi[kVcCheckpoints], ck_kb[kVcCheckpoints], ck_n[kVcCheckpoints], ck_pos[kVcCheckpoints];
  int g_lo, g_hi, token;
  int tile_tot[kVcSelTiles];
  // rows whose tail is deferred until the block has left its row loop (see sample_rows_kernel)
  int n_pend;      // rows recorded in pend[]
  int class_ok;    // the current row may take the class tail
  float raw_max;   // the current row's largest logit
  struct Pending {
    long long row;
    float inv_t, mx, sum, cutoff, topp, coin, raw_max;
  } pend[kVcPendCap];
};

template <bool kLut, bool kGuided = false, bool kExtended = false>
struct __align__(16) Shared {
  static constexpr bool kHasClassTail = !kGuided;  // the guided variant keeps its shared memory for itself
  VcControl vcc;
  // (members read with vector loads carry their own alignas)
  static constexpr bool kHasLut = kLut;
  static constexpr bool kExt = kExtended;  // per-row settings and the fused scalar multiply
  typename std::conditional<kGuided, GuidedShared, NoGuidedShared>::type g;
  uint64_t exp_tab[kExpTableSize];
  alignas(16) float head[kHead];  // read as float4
  SeqSummary wsum[3][kWarps];  // slots used by successive scan rounds in rotation (see seqsum_tile)
  int first[2];
  int wcnt[2][kWarps];
  float redf[kWarps];
  int redi[kWarps];
  unsigned hcnt[kBins];
  float hmass[kBins];
  float s_bcast;
  int hit_found;
  int hit_idx;
  float hit_val;
  int misc_i[4];
  float misc_f[4];
  // The table sits directly in front of the union: the value-class tail, which needs neither,
  // lays its window of class counts over both (vc_hist()).
  alignas(16) float lut[kLut ? kLutSize : 4];
  union alignas(16) {
    // terms of the row's first tile, one padded run per thread, for the one-warp start of the sum
    alignas(16) float stage[kThreads * kStagePitch];
    unsigned wbins[kWarps / 2][kBins][2];  // per warp pair and value bin: count, sum of mantissa offsets
    struct {
      unsigned short cnt[kCompactSteps][kWarps];  // survivors per (step, warp), then exclusive in step
      unsigned base[kCompactSteps];               // survivors in front of each step
    } compact;
    struct {
      unsigned long long ck[kRankSortMax];
      int rank[kRankSortMax];
    } rsort;
    struct {  // the whole tail of a row with a short nucleus, in shared memory (small_tail)
      unsigned long long ck[kRankSortMax];
      alignas(16) float p[kRankSortMax + 8];  // read four at a time, one group ahead
      int idx[kRankSortMax];
      alignas(16) float prefix[kRankSortMax + 4];
      int cnt;
      int first_above;
      int last;
      float cum;
    } small;
    struct {
      unsigned wofs[kWarps][kRadix];  // per warp and digit: count, then running output offset
      unsigned above[kRadix];
    } radix;
    typename std::conditional<(kGuided || kLut), NoVcHist, VcHist>::type vc;
  } u;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename S>
__device__ __forceinline__ float block_max(S& sm, float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sm.redf[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = sm.redf[0];
#pragma unroll
  for (int w = 1; w < kWarps; ++w) r = fmaxf(r, sm.redf[w]);
  return r;
}

// Exclusive block-wide prefix count of a per-thread count; *total gets the block sum.
template <typename S>
__device__ __forceinline__ int block_excl_count(S& sm, int cnt, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inc = cnt;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int o = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += o;
  }
  __syncthreads();
  if (lane == 31) sm.redi[warp] = inc;
  __syncthreads();
  int pre = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int c = sm.redi[w];
    if (w < warp) pre += c;
    tot += c;
  }
  *total = tot;
  return pre + inc - cnt;
}

// Summary of one thread's chunk in the binade kb of the running sum: the tie-free fast path
// first, the two-parity functions when the chunk holds an exact half-way term (or for sums
// outside the fast path's range).
__device__ __forceinline__ SeqSummary chunk_summary(const float (&v)[kChunk], int kb) {
  SeqSummary mine;
  seq_identity(&mine);
  if (kb >= 27 && kb <= 252) {
    // v / u by an exact power-of-two scaling; adding 2^23 rounds it to an integer (half to
    // even). Four interleaved accumulator pairs: short dependency chains (the partial sums
    // are integers below 2^24, hence exact, whenever the total is; otherwise the total
    // stays at or above 2^24, which is all that matters then).
    const float inv_u24 = seq_inv_u24(kb);
    float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f}, t4[4] = {1.0f, 1.0f, 1.0f, 1.0f};
#pragma unroll
    for (int j = 0; j < kChunk; ++j) seq_push_fast(&a4[j & 3], &t4[j & 3], v[j], inv_u24);
    const float accf = __fadd_rn(__fadd_rn(a4[0], a4[1]), __fadd_rn(a4[2], a4[3]));
    const float tie_prod = __fmul_rn(__fmul_rn(t4[0], t4[1]), __fmul_rn(t4[2], t4[3]));
    const int acc = (int)fminf(accf, (float)kFastSat);
    mine.a0 = acc;
    mine.a1 = acc;
    if (!(tie_prod != 0.0f)) {  // zero (a tie, or an underflowed product) or NaN
      const float inv_u = seq_inv_u(kb);
      seq_identity(&mine);
#pragma unroll
      for (int j = 0; j < kChunk; ++j) seq_push_scaled(&mine, v[j], inv_u);
    }
  } else {
#pragma unroll
    for (int j = 0; j < kChunk; ++j) seq_push(&mine, v[j], kb);
  }
  if (mine.a0 > kFastSat) mine.a0 = kFastSat;
  if (mine.a1 > kFastSat) mine.a1 = kFastSat;
  return mine;
}

// ---------------------------------------------------------------------------------------
// The same exact sequential sum at warp scope: lane l holds the kChunk terms that follow
// those of lanes 0..l-1; `s` is warp-uniform. No shared memory and no block barrier, so a
// round costs one warp's instructions instead of the whole block's. Used where the running
// sum leaves its binade every few hundred terms (the start of a row). Same contract as
// seqsum_tile otherwise (pos0 = position of lane 0's first term).
// ---------------------------------------------------------------------------------------
template <bool kSearch>
__device__ __forceinline__ bool seqsum_warp(
    const float (&v)[kChunk], float& s, float thr, int pos0, int limit, int* hit_pos,
    float* hit_sum) {
  const int lane = threadIdx.x & 31;
  int consumed = 0;
  while (true) {
    const int kb = seq_kb(s);
    const int n_s = seq_n(s);
    SeqSummary mine;
    seq_identity(&mine);
    const bool active = lane >= consumed;
    if (active) mine = chunk_summary(v, kb);
    const bool two_parity = __any_sync(0xffffffffu, mine.a0 != mine.a1);
    if (!two_parity) {
      const int n_end = n_s + __reduce_add_sync(0xffffffffu, mine.a0);  // <= 2^24 + 32 * kFastSat
      bool more = n_end >= kSeqLimit;
      if (kSearch) {
        if (!more && seq_value(kb, n_end) > thr) more = true;
      }
      if (!more) {
        s = seq_value(kb, n_end);
        return false;
      }
    }
    int n_in, n_out;  // N in front of / behind this lane's chunk
    if (!two_parity) {
      int inc = mine.a0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      n_in = n_s + (inc - mine.a0);
      n_out = n_s + inc;
    } else {
      SeqSummary sc = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        SeqSummary o;
        o.a0 = __shfl_up_sync(0xffffffffu, sc.a0, d);
        o.a1 = __shfl_up_sync(0xffffffffu, sc.a1, d);
        if (lane >= d) sc = seq_compose(o, sc);
      }
      SeqSummary excl;
      excl.a0 = __shfl_up_sync(0xffffffffu, sc.a0, 1);
      excl.a1 = __shfl_up_sync(0xffffffffu, sc.a1, 1);
      if (lane == 0) seq_identity(&excl);
      n_in = seq_apply(n_s, excl);
      n_out = seq_apply(n_in, mine);
    }
    // the first chunk whose end value left the binade or, when searching, exceeds thr
    bool flag = active && n_out >= kSeqLimit;
    if (kSearch) {
      if (active && n_out < kSeqLimit && seq_value(kb, n_out) > thr) flag = true;
    }
    const unsigned lb = __ballot_sync(0xffffffffu, flag);
    if (lb == 0) {
      s = seq_value(kb, __shfl_sync(0xffffffffu, n_out, 31));
      return false;
    }
    const int first = __ffs(lb) - 1;
    float acc = 0.0f, hval = 0.0f;
    int found = 0, hpos = 0;
    if (lane == first) {
      // the sum in front of this chunk is exact: redo the chunk with real float additions
      acc = seq_value(kb, n_in);
#pragma unroll
      for (int j = 0; j < kChunk; ++j) {
        acc = __fadd_rn(acc, v[j]);
        if (kSearch) {
          const int pos = pos0 + lane * kChunk + j;
          if (!found && acc > thr && pos < limit) {
            found = 1;
            hpos = pos;
            hval = acc;
          }
        }
      }
    }
    s = __shfl_sync(0xffffffffu, acc, first);
    if (kSearch) {
      if (__shfl_sync(0xffffffffu, found, first)) {
        *hit_pos = __shfl_sync(0xffffffffu, hpos, first);
        *hit_sum = __shfl_sync(0xffffffffu, hval, first);
        return true;
      }
    }
    consumed = first + 1;
    if (consumed >= 32) return false;
  }
}

// ---------------------------------------------------------------------------------------
// One tile of the exact sequential float sum. Thread t holds the kChunk consecutive terms
// v[] that follow the terms of threads 0..t-1. `s` is the running sum in front of the
// tile on entry and behind it on return (block-uniform).
//
// Each round summarises every thread's chunk in the binade of s, and every warp its 32
// chunks: one integer (a warp reduction) when none of them holds an exact half-way term,
// else the two-parity summary of exact_math.cuh composed along the lanes. After ONE barrier
// every warp reads the kWarps summaries and decides, redundantly and identically, whether
// the value behind the tile is still inside the binade (and not beyond thr); then the tile
// total, a reduction or a composition of kWarps summaries, is all that is needed. Otherwise
// prefix sums down to the thread name the first chunk that leaves the binade (or holds the
// searched position); its thread redoes it with real float additions and publishes the new
// sum behind a second barrier, and the threads behind it go into the next round.
//
// Rounds rotate through three sets of shared slots (`rp`, block-uniform, carried by the
// caller across tiles), so a round needs no barrier to protect its slots from the previous
// round.
//
// With kSearch, also looks for the first term after which the running sum exceeds `thr`
// (terms at position >= limit, counted from pos0 of thread 0's first term, must be zero
// padding); on a match returns true with the position in *hit_pos and the sum reached
// there in *hit_sum (block-uniform), and `s` is then not meaningful.
// ---------------------------------------------------------------------------------------
template <bool kSearch, typename S>
__device__ __forceinline__ bool seqsum_tile(
    S& sm, const float (&v)[kChunk], float& s, int& rp, float thr, int pos0, int limit,
    int* hit_pos, float* hit_sum) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int consumed = 0;
  while (true) {
    const int kb = seq_kb(s);
    const int n_s = seq_n(s);
    SeqSummary mine;
    seq_identity(&mine);
    const bool active = tid >= consumed;
    if (active) mine = chunk_summary(v, kb);
    // Warp summary: one integer when none of the warp's chunks holds an exact half-way term
    // (a reduction), else the two-parity summary composed along the lanes (rare).
    SeqSummary lane_excl;  // two-parity summary of the lanes in front of this one (tie warps only)
    seq_identity(&lane_excl);
    SeqSummary wsum;
    const bool warp_tie = __any_sync(0xffffffffu, mine.a0 != mine.a1);
    if (!warp_tie) {
      const int wtot = __reduce_add_sync(0xffffffffu, mine.a0);  // <= 32 * kFastSat
      wsum.a0 = wsum.a1 = wtot < kFastSat ? wtot : kFastSat;
    } else {
      SeqSummary sc = mine;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        SeqSummary o;
        o.a0 = __shfl_up_sync(0xffffffffu, sc.a0, d);
        o.a1 = __shfl_up_sync(0xffffffffu, sc.a1, d);
        if (lane >= d) sc = seq_compose(o, sc);
      }
      lane_excl.a0 = __shfl_up_sync(0xffffffffu, sc.a0, 1);
      lane_excl.a1 = __shfl_up_sync(0xffffffffu, sc.a1, 1);
      if (lane == 0) seq_identity(&lane_excl);
      wsum.a0 = __shfl_sync(0xffffffffu, sc.a0, 31);
      wsum.a1 = __shfl_sync(0xffffffffu, sc.a1, 31);
    }
    if (lane == 0) sm.wsum[rp][warp] = wsum;
    __syncthreads();  // ---- barrier 1: the warp summaries are visible
    SeqSummary wt;
    seq_identity(&wt);
    if (lane < kWarps) wt = sm.wsum[rp][lane];
    const int next_rp = rp == 2 ? 0 : rp + 1;
    const bool two_parity = __any_sync(0xffffffffu, wt.a0 != wt.a1);
    int n_wend;  // N behind the warp `lane` (lanes < kWarps), for the warp-level decision
    if (!two_parity) {
      // The common round: N only grows along the tile, so if the value behind the whole tile
      // is still inside the binade (and not beyond thr), nothing in between left it: the
      // tile total is all that is needed, one reduction and no prefix sums.
      const int n_end = n_s + __reduce_add_sync(0xffffffffu, wt.a0);
      bool more = n_end >= kSeqLimit;
      if (kSearch) {
        if (!more && seq_value(kb, n_end) > thr) more = true;
      }
      if (!more) {
        s = seq_value(kb, n_end);
        rp = next_rp;
        return false;
      }
      n_wend = 0;
    } else {
      // a tie somewhere: compose the kWarps summaries; exact as long as N stays in the binade
#pragma unroll
      for (int d = 1; d < kWarps; d <<= 1) {
        SeqSummary o;
        o.a0 = __shfl_up_sync(0xffffffffu, wt.a0, d);
        o.a1 = __shfl_up_sync(0xffffffffu, wt.a1, d);
        if (lane >= d) wt = seq_compose(o, wt);
      }
      n_wend = seq_apply(n_s, wt);
      const int n_end = __shfl_sync(0xffffffffu, n_wend, kWarps - 1);
      bool more = n_end >= kSeqLimit;
      if (kSearch) {
        if (!more && seq_value(kb, n_end) > thr) more = true;
      }
      if (!more) {
        s = seq_value(kb, n_end);
        rp = next_rp;
        return false;
      }
    }
    // Some chunk leaves the binade (or holds the searched position): prefix sums per thread
    int n_in, n_out;  // N in front of / behind this thread's chunk
    if (!two_parity) {
      int inc = mine.a0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += o;
      }
      int wi = wt.a0;
#pragma unroll
      for (int d = 1; d < kWarps; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, wi, d);
        if (lane >= d) wi += o;
      }
      int pre = __shfl_sync(0xffffffffu, wi, warp > 0 ? warp - 1 : 0);
      if (warp == 0) pre = 0;
      n_wend = n_s + wi;
      n_in = n_s + pre + (inc - mine.a0);
      n_out = n_in + mine.a0;
    } else {
      // wt holds the inclusive composition over the warps; tie-free warps have not formed
      // their lanes' prefix yet
      if (!warp_tie) {
        int inc = mine.a0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += o;
        }
        lane_excl.a0 = lane_excl.a1 = inc - mine.a0;
      }
      SeqSummary pre;
      pre.a0 = __shfl_sync(0xffffffffu, wt.a0, warp > 0 ? warp - 1 : 0);
      pre.a1 = __shfl_sync(0xffffffffu, wt.a1, warp > 0 ? warp - 1 : 0);
      if (warp == 0) seq_identity(&pre);
      pre = seq_compose(pre, lane_excl);
      n_in = seq_apply(n_s, pre);
      n_out = seq_apply(n_in, mine);
    }
    // Which warp holds the first chunk to redo: the first whose end value left the binade
    // (N >= 2^24) or, when searching, exceeds thr. N only grows along the tile, so this is
    // decided from the warp-end values alone, identically by every warp.
    bool wflag = lane < kWarps && n_wend >= kSeqLimit;
    if (kSearch) {
      if (lane < kWarps && n_wend < kSeqLimit && seq_value(kb, n_wend) > thr) wflag = true;
    }
    const unsigned wb = __ballot_sync(0xffffffffu, wflag);
    rp = next_rp;
    if (wb == 0) {
      // nothing left the binade: the whole tile is summarised exactly
      s = seq_value(kb, __shfl_sync(0xffffffffu, n_wend, kWarps - 1));
      return false;
    }
    const int redo_warp = __ffs(wb) - 1;
    if (warp == redo_warp) {
      bool flag = active && (n_out >= kSeqLimit);
      if (kSearch) {
        if (active && n_out < kSeqLimit && seq_value(kb, n_out) > thr) flag = true;
      }
      const unsigned lb = __ballot_sync(0xffffffffu, flag);
      const int first_lane = __ffs(lb) - 1;  // exists: this warp's end value is flagged
      if (lane == first_lane) {
        // The sum in front of this chunk is exact; redo the chunk with real float additions
        // (it leaves the binade here, or it contains the searched position).
        float acc = seq_value(kb, n_in);
        int found = 0;
#pragma unroll
        for (int j = 0; j < kChunk; ++j) {
          acc = __fadd_rn(acc, v[j]);
          if (kSearch) {
            const int pos = pos0 + tid * kChunk + j;
            if (!found && acc > thr && pos < limit) {
              found = 1;
              sm.hit_idx = pos;
              sm.hit_val = acc;
            }
          }
        }
        sm.hit_found = found;
        sm.s_bcast = acc;
        sm.first[0] = tid;
      }
    }
    __syncthreads();  // ---- barrier 2 (only in rounds that redo a chunk)
    s = sm.s_bcast;
    const int first = sm.first[0];
    const bool hit = kSearch && sm.hit_found;
    if (hit) {
      *hit_pos = sm.hit_idx;
      *hit_sum = sm.hit_val;
    }
    consumed = first + 1;
    if (hit || consumed >= kThreads) {
      __syncthreads();  // the result slots may be rewritten by the caller's next step
      return hit;
    }
    // the next round's barrier 1 orders these reads before the next writes of the slots
  }
}

// The tile behind the sequential head is where the running sum still leaves its binade every
// few hundred terms, and every such round of seqsum_tile occupies the whole block. Instead the
// tile's terms are staged in shared memory (stage_first_tile, which ends with a barrier) and
// one warp sums them 512 at a time (sum_staged_tile, block-uniform result behind a barrier)
// while the other warps wait or, between the two calls, do other work.
template <typename S>
__device__ __forceinline__ void stage_first_tile(S& sm, const float (&e)[kChunk]) {
  float4* st4 = reinterpret_cast<float4*>(sm.u.stage + threadIdx.x * kStagePitch);
#pragma unroll
  for (int q = 0; q < kChunk / 4; ++q) st4[q] = make_float4(e[4 * q], e[4 * q + 1], e[4 * q + 2], e[4 * q + 3]);
  __syncthreads();
}

template <bool kSearch, typename S>
__device__ __forceinline__ bool sum_staged_tile(
    S& sm, float& s, float thr, int vocab, int* hit_pos, float* hit_sum) {
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    const int span = (vocab - kHead) < kTile ? (vocab - kHead) : kTile;
    const int n_sub = (span + 32 * kChunk - 1) / (32 * kChunk);
    float sw = s, hs = 0.0f;
    int hp = 0;
    bool hit = false;
    for (int t = 0; t < n_sub && !hit; ++t) {
      float v[kChunk];
      const float4* p4 = reinterpret_cast<const float4*>(sm.u.stage + (t * 32 + lane) * kStagePitch);
#pragma unroll
      for (int q = 0; q < kChunk / 4; ++q) {
        const float4 x = p4[q];
        v[4 * q] = x.x;
        v[4 * q + 1] = x.y;
        v[4 * q + 2] = x.z;
        v[4 * q + 3] = x.w;
      }
      hit = seqsum_warp<kSearch>(v, sw, thr, kHead + t * 32 * kChunk, vocab, &hp, &hs);
    }
    if (lane == 0) {
      sm.s_bcast = sw;
      sm.hit_found = hit ? 1 : 0;
      sm.hit_idx = hp;
      sm.hit_val = hs;
    }
  }
  __syncthreads();  // the result; the staging buffer is free again
  s = sm.s_bcast;
  const bool hit = kSearch && sm.hit_found;
  if (hit) {
    *hit_pos = sm.hit_idx;
    *hit_sum = sm.hit_val;
  }
  return hit;
}

// The first terms of a sum leave a binade every few additions, which would cost one block
// round each; instead one thread adds the `count` terms staged in sm.head with real float
// additions. Same contract as seqsum_tile. Callers fill sm.head before the call and need no
// barrier in between: this function synchronises on entry and on exit.
template <bool kSearch, typename S>
__device__ __forceinline__ bool head_sum(
    S& sm, int count, float& s, float thr, int pos0, int* hit_pos, float* hit_sum) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // sm.head is zero-padded to a multiple of 4, and the terms are non-negative, so the
    // partial sums only grow: test four additions at a time
    float acc = s;
    int found = 0;
    const float4* h4 = reinterpret_cast<const float4*>(sm.head);
    for (int i = 0; i < count; i += 4) {
      const float4 q = h4[i >> 2];
      const float a1 = __fadd_rn(acc, q.x);
      const float a2 = __fadd_rn(a1, q.y);
      const float a3 = __fadd_rn(a2, q.z);
      const float a4 = __fadd_rn(a3, q.w);
      if (kSearch && a4 > thr) {
        int k = 3;
        float hv = a4;
        if (a3 > thr) { k = 2; hv = a3; }
        if (a2 > thr) { k = 1; hv = a2; }
        if (a1 > thr) { k = 0; hv = a1; }
        if (i + k < count) {
          found = 1;
          sm.hit_idx = pos0 + i + k;
          sm.hit_val = hv;
        }
        acc = a4;
        break;
      }
      acc = a4;
    }
    sm.hit_found = found;
    sm.s_bcast = acc;
  }
  __syncthreads();
  s = sm.s_bcast;
  bool hit = false;
  if (kSearch && sm.hit_found) {
    *hit_pos = sm.hit_idx;
    *hit_sum = sm.hit_val;
    hit = true;
  }
  __syncthreads();  // the head buffer and the result slots may be reused after this
  return hit;
}

// Writes the token of row r: to out_ids[r], or -- when peer buffers are given -- straight into
// every listed buffer at [offset + r] (each may live on another GPU of the node: plain
// stores over NVLink, one thread per destination). Block-uniform `token`.
__device__ __forceinline__ void store_token(
    int64_t* __restrict__ out_ids, const PeerOut& peers, int64_t r, int token) {
  if (peers.n == 0) {
    if (threadIdx.x == 0) out_ids[r] = (int64_t)token;
  } else if ((int)threadIdx.x < peers.n) {
    peers.ptr[threadIdx.x][peers.offset + r] = (int64_t)token;
  }
}

// Arrival barrier among the GPUs of a node at the end of a launch (see PeerOut). Every thread
// of every block calls it once, after its last store_token. No kernel of one GPU waits for
// another kernel of the same GPU; the wait for the other GPUs is limited to peers.wait_ns
// nanoseconds of the GPU's global timer, after which the launch records kStatusPeerTimeout in
// *status and ends (the context stays usable; the ids of the missing ranks are stale).
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void peer_arrival_barrier(const PeerOut& peers, int* status) {
  if (peers.epoch == 0ull) return;  // launch-uniform
  __shared__ int is_last;
  __threadfence_system();  // this thread's id stores are ordered before the block's arrival
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(peers.blocks_done, 1);
    is_last = (prev == (int)gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!is_last) return;  // block-uniform
  __threadfence_system();  // every block's ids before this rank's arrival marks
  if (threadIdx.x == 0) *peers.blocks_done = 0;
  if ((int)threadIdx.x < peers.n) {
    volatile unsigned long long* theirs = peers.arrive[threadIdx.x] + peers.rank;
    *theirs = peers.epoch;  // tell rank threadIdx.x that this rank's ids are in its buffer
    volatile unsigned long long* mine = peers.arrive[peers.rank] + threadIdx.x;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (*mine < peers.epoch) {  // until rank threadIdx.x has told this rank
      // the timer is read every 64 polls; the poll count is a second, independent bound
      if ((++spins & 63u) == 0u && (global_timer_ns() - t0 > peers.wait_ns || spins > (1u << 30))) {
        atomicExch(status, kStatusPeerTimeout);
        break;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
}

// xorshift64* step and 24-bit coin of the reference (sampler.cpp:210-220).
__device__ __forceinline__ float next_coin(unsigned long long* state) {
  unsigned long long s = *state;
  s ^= s >> 12;
  s ^= s << 25;
  s ^= s >> 27;
  *state = s;
  const unsigned u = (unsigned)((s * 0x2545F4914F6CDD1Dull) >> 32);
  return (float)(u >> 8) / 16777216.0f;
}

// ---------------------------------------------------------------------------------------
// Per-row element math: e = expf(logit * inv_t - mx) (sampler.cpp:231-233 and :201), or
// e / S once the sum is known (sampler.cpp:205-207) when `probs` is set.
// ---------------------------------------------------------------------------------------
template <typename T, typename S>
struct RowMath {
  const T* row;
  int vocab;
  bool vec_ok;
  float inv_t;
  float mx;
  float sum;   // divisor when probs is set
  bool probs;
  float scale = 1.0f;  // extended entry point only: every logit is first multiplied by this, in T

  // The logit as the sampler sees it: a "multiply" logit processor folded into the load
  // (logit_processor.h:34-40 works in place on T, so the product is rounded to T).
  __device__ __forceinline__ float xform(float logit) const {
    if constexpr (S::kExt) {
      const float y = __fmul_rn(logit, scale);
      if constexpr (std::is_same<T, __nv_bfloat16>::value) return __bfloat162float(__float2bfloat16_rn(y));
      if constexpr (std::is_same<T, __half>::value) return __half2float(__float2half_rn(y));
      return y;
    } else {
      return logit;
    }
  }

  __device__ __forceinline__ float direct(float logit, const S& sm) const {
    const float e = expf_ref(__fsub_rn(__fmul_rn(xform(logit), inv_t), mx), sm.exp_tab);
    return probs ? __fdiv_rn(e, sum) : e;
  }

  // bf16 bit pattern -> table slot, or -1 when the value is outside the table
  static __device__ __forceinline__ int lut_slot(uint32_t h) {
    const uint32_t hb = h + kLutBias;
    const int slot = (int)((hb & 0x0FFFu) | ((hb >> 3) & 0x1000u));
    return (hb & 0x7000u) == 0x4000u ? slot : -1;
  }

  static __device__ __forceinline__ uint32_t lut_pattern(int slot) {
    const uint32_t hb = 0x4000u | ((uint32_t)slot & 0x0FFFu);
    return ((hb - kLutBias) & 0x7FFFu) | (((uint32_t)slot & 0x1000u) << 3);
  }

  // Fills the table for this row (bf16 only): slot -> e, or e / S when probs is set.
  __device__ __forceinline__ void build_lut(S& sm) const {
    for (int k = threadIdx.x; k < kLutSize; k += kThreads) {
      sm.lut[k] = direct(bits_f32(lut_pattern(k) << 16), sm);
    }
  }

  __device__ __forceinline__ float from_pattern(uint32_t h, const S& sm) const {
    const int slot = lut_slot(h);
    if (slot >= 0) return sm.lut[slot];
    return direct(bits_f32(h << 16), sm);
  }

  // One element (used for the sequential head and for ragged edges). 0 beyond the row.
  __device__ __forceinline__ float at(int i, const S& sm) const {
    if (i >= vocab) return 0.0f;
    if constexpr (S::kHasLut) {
      return from_pattern((uint32_t) reinterpret_cast<const unsigned short*>(row)[i], sm);
    } else {
      return direct(to_f32(row[i]), sm);
    }
  }

  // The 128-bit loads of a full, aligned chunk, separated from their use so that the next
  // tile's loads can be in flight while this tile is processed.
  static constexpr int kRawVecs = kChunk * sizeof(T) / 16;
  struct Raw {
    uint4 q[kRawVecs];
  };
  __device__ __forceinline__ bool full(int i0) const { return vec_ok && i0 + kChunk <= vocab; }
  __device__ __forceinline__ void load_raw(int i0, Raw* r) const {
#pragma unroll
    for (int q = 0; q < kRawVecs; ++q) r->q[q] = __ldg(reinterpret_cast<const uint4*>(row + i0) + q);
  }
  __device__ __forceinline__ void eval_raw(const Raw& r, const S& sm, float (&e)[kChunk]) const {
    constexpr int kPerVec = 16 / sizeof(T);
    uint32_t bad = 0u;  // bits 14..12 of a biased half that differ from 100, over the chunk
    (void)bad;
#pragma unroll
    for (int q = 0; q < kRawVecs; ++q) {
      if constexpr (S::kHasLut) {
        const uint32_t w[4] = {r.q[q].x, r.q[q].y, r.q[q].z, r.q[q].w};
        const char* lut_bytes = reinterpret_cast<const char*>(sm.lut);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // both halves at once. A carry out of the low half only happens for a low pattern
          // that is outside the table anyway, and then the whole chunk is redone below.
          const uint32_t wb = w[j] + (kLutBias | (kLutBias << 16));
          bad |= wb ^ 0x40004000u;
          const uint32_t off0 = ((wb << 2) & 0x3FFCu) | ((wb >> 1) & 0x4000u);
          const uint32_t off1 = ((wb >> 14) & 0x3FFCu) | ((wb >> 17) & 0x4000u);
          e[q * 8 + 2 * j] = *reinterpret_cast<const float*>(lut_bytes + off0);
          e[q * 8 + 2 * j + 1] = *reinterpret_cast<const float*>(lut_bytes + off1);
        }
      } else {
        const T* p = reinterpret_cast<const T*>(&r.q[q]);
#pragma unroll
        for (int j = 0; j < kPerVec; ++j) e[q * kPerVec + j] = direct(to_f32(p[j]), sm);
      }
    }
    if constexpr (S::kHasLut) {
      // every pattern is inside the table iff bits 14..12 of every biased half are 100
      if ((bad & 0x70007000u) != 0u) {
        // rare: a zero, tiny, huge or non-finite logit in this chunk; redo the chunk element by
        // element (table where possible, direct evaluation otherwise)
#pragma unroll
        for (int q = 0; q < kRawVecs; ++q) {
          const uint32_t w[4] = {r.q[q].x, r.q[q].y, r.q[q].z, r.q[q].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            e[q * 8 + 2 * j] = from_pattern(w[j] & 0xFFFFu, sm);
            e[q * 8 + 2 * j + 1] = from_pattern(w[j] >> 16, sm);
          }
        }
      }
    }
  }

  // kChunk consecutive elements starting at i0.
  __device__ __forceinline__ void chunk(int i0, const S& sm, float (&e)[kChunk]) const {
    if (vec_ok && i0 + kChunk <= vocab) {
      constexpr int kPerVec = 16 / sizeof(T);
#pragma unroll
      for (int q = 0; q < kChunk / kPerVec; ++q) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row + i0) + q);
        if constexpr (S::kHasLut) {
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            e[q * 8 + 2 * j] = from_pattern(w[j] & 0xFFFFu, sm);
            e[q * 8 + 2 * j + 1] = from_pattern(w[j] >> 16, sm);
          }
        } else {
          const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int j = 0; j < kPerVec; ++j) e[q * kPerVec + j] = direct(to_f32(p[j]), sm);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < kChunk; ++j) e[j] = at(i0 + j, sm);
    }
  }
};

__device__ __forceinline__ __half2 neg_inf2(__half) {
  const __half v = __ushort_as_half((unsigned short)0xFC00);
  return __halves2half2(v, v);
}
__device__ __forceinline__ __nv_bfloat162 neg_inf2(__nv_bfloat16) {
  const __nv_bfloat16 v = __ushort_as_bfloat16((unsigned short)0xFF80);
  return __halves2bfloat162(v, v);
}

// Max over the row of logit * inv_t (softmax, sampler.cpp:191-196).
template <typename T, typename S>
__device__ __forceinline__ float row_max_scaled(
    S& sm, const RowMath<T, S>& rm, const T* __restrict__ row, int vocab, bool vec_ok, float inv_t,
    float* raw_max = nullptr) {
  const int tid = threadIdx.x;
  if (raw_max != nullptr) *raw_max = NAN;  // known only on the 16-bit path below
  if constexpr (sizeof(T) == 2) {
    if (inv_t > 0.0f) {
      // x -> fl(x * inv_t) is monotone for inv_t > 0, so the max can be taken on the raw
      // 16-bit values, two per instruction, and scaled once
      using T2 = decltype(neg_inf2(T()));
      const int nvec = vec_ok ? vocab / 8 : 0;
      T2 acc = neg_inf2(T());
      // this pass is the row's HBM read: four 128-bit loads in flight per thread
      int q = tid;
      for (; q + 3 * kThreads < nvec; q += 4 * kThreads) {
        uint4 raw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) raw[k] = __ldg(reinterpret_cast<const uint4*>(row) + q + k * kThreads);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const T2* p = reinterpret_cast<const T2*>(&raw[k]);
          acc = __hmax2(acc, __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3])));
        }
      }
      for (; q < nvec; q += kThreads) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row) + q);
        const T2* p = reinterpret_cast<const T2*>(&raw);
        acc = __hmax2(acc, __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3])));
      }
      float m = fmaxf(to_f32(acc.x), to_f32(acc.y));
      for (int i = nvec * 8 + tid; i < vocab; i += kThreads) m = fmaxf(m, to_f32(row[i]));
      m = block_max(sm, m);
      if (raw_max != nullptr) *raw_max = m;
      return __fmul_rn(rm.xform(m), inv_t);  // the multiply is by a positive factor: monotone too
    }
  }
  float mx = -INFINITY;
  for (int i = tid; i < vocab; i += kThreads) mx = fmaxf(mx, __fmul_rn(rm.xform(to_f32(row[i])), inv_t));
  return block_max(sm, mx);
}

// ---------------------------------------------------------------------------------------
// Stable LSD radix sort pass over a list of n entries, descending in the 8-bit digit at
// `shift`. One block; src and dst are distinct global buffers.
//
// Every warp owns a contiguous slice of the list. (1) Each warp counts the digits of its
// slice into its own 256 counters. (2) One block-wide prefix turns the counters into start
// offsets: digits in descending order, and within a digit the warps in order, which is the
// list order. (3) Each warp scatters its slice in steps of 32 entries, ranking the lanes of
// a step with a warp match and advancing its private offsets; no block barrier is needed
// inside the scatter.
// ---------------------------------------------------------------------------------------
template <typename S>
__device__ void radix_pass_desc(S& sm, const Entry* src, Entry* dst, int n, int shift) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned (*wofs)[kRadix] = sm.u.radix.wofs;
  const int per_warp = ((n + kWarps - 1) / kWarps + 31) & ~31;  // slice length, a multiple of 32
  const int lo = warp * per_warp < n ? warp * per_warp : n;
  const int hi = lo + per_warp < n ? lo + per_warp : n;
  __syncthreads();  // earlier users of the union are done
  for (int d = lane; d < kRadix; d += 32) wofs[warp][d] = 0;
  __syncwarp();
  for (int i0 = lo; i0 < hi; i0 += 32 * kListBatch) {
    uint32_t k[kListBatch];
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {  // independent loads first, so they overlap
      const int i = i0 + u * 32 + lane;
      k[u] = i < hi ? src[i].key : 0u;
    }
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {
      if (i0 + u * 32 + lane < hi) atomicAdd(&wofs[warp][(k[u] >> shift) & (kRadix - 1)], 1u);
    }
  }
  __syncthreads();
  // thread d (< 256) walks digit d over the warps; the digit totals are then prefixed in
  // descending digit order
  unsigned digit_total = 0;
  if (tid < kRadix) {
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned c = wofs[w][tid];
      wofs[w][tid] = digit_total;  // entries of this digit in earlier warps
      digit_total += c;
    }
    // suffix sums over the 256 digits: 8 warps of 32 digits each
    unsigned incl = digit_total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_down_sync(0xffffffffu, incl, d);
      if (lane + d < 32) incl += o;
    }
    sm.u.radix.above[tid] = incl - digit_total;  // larger digits inside this group of 32
    if (lane == 0) sm.redi[warp] = (int)incl;
  }
  __syncthreads();
  if (tid < kRadix) {
    unsigned above = sm.u.radix.above[tid];
    for (int w = warp + 1; w < kRadix / 32; ++w) above += (unsigned)sm.redi[w];
#pragma unroll
    for (int w = 0; w < kWarps; ++w) wofs[w][tid] += above;
  }
  __syncthreads();
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const int i = i0 + lane;
    const bool valid = i < hi;
    Entry e;
    e.key = 0;
    e.idx = 0;
    if (valid) e = src[i];
    const unsigned dg = valid ? ((e.key >> shift) & (kRadix - 1)) : 0xFFFFFFFFu;
    // rank among the lanes of this step that hold the same digit, in lane (= list) order
    const unsigned peers = __match_any_sync(0xffffffffu, dg);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    unsigned base = 0;
    if (valid) base = wofs[warp][dg];
    __syncwarp();
    if (valid) {
      dst[base + rank] = e;
      if (rank == 0) wofs[warp][dg] = base + __popc(peers);
    }
    __syncwarp();
  }
  __syncthreads();
}

// Exact cumulative sum over the key floats of a sorted list, looking for the first
// position (below `limit`) where it exceeds thr. Returns true with position and sum, else
// false with the total in *total. Short lists are summed sequentially through the head
// buffer; long ones continue with block-wide tiles.
template <typename S>
__device__ bool list_search(
    S& sm, const Entry* list, int n, int limit, float thr, int& rp, int* pos, float* sum,
    float* total) {
  const int lim = n < limit ? n : limit;
  float s = 0.0f;
  const int seq_end = lim <= 4 * kHead ? lim : kHead;
  int base = 0;
  for (; base < seq_end; base += kHead) {
    const int cnt = (seq_end - base) < kHead ? (seq_end - base) : kHead;
    __syncthreads();
    if (threadIdx.x < kHead) {
      const int i = base + threadIdx.x;
      sm.head[threadIdx.x] = (i < lim) ? bits_f32(list[i].key) : 0.0f;
    }
    if (head_sum<true>(sm, cnt, s, thr, base, pos, sum)) return true;
  }
  for (; base < lim; base += kTile) {
    float v[kChunk];
#pragma unroll
    for (int j = 0; j < kChunk; ++j) {
      const int i = base + threadIdx.x * kChunk + j;
      v[j] = (i < lim) ? bits_f32(list[i].key) : 0.0f;
    }
    if (seqsum_tile<true>(sm, v, s, rp, thr, base, lim, pos, sum)) return true;
  }
  *total = s;
  return false;
}

// ---------------------------------------------------------------------------------------
// Pieces of the top-p / top-k tail. All are block-wide and return block-uniform results.
// ---------------------------------------------------------------------------------------

// Bins the values of list A and picks the lowest value bin to keep: the largest bin b such
// that the bins >= b surely hold more than topp of the mass (top-p; the margin covers the
// rounding of the reference's own running sum) or at least topk entries (top-k). Returns
// false when even all listed entries do not suffice. *bin_out is 0 ("keep everything
// listed") in that case. *cnt_out = entries in the kept bins.
template <typename S>
__device__ bool pick_value_threshold(
    S& sm, const Entry* listA, int n_a, float sum, float topp, int topk, bool use_topk,
    int* bin_out, int* cnt_out) {
  const int tid = threadIdx.x, warp = tid >> 5;
  __syncthreads();  // earlier users of the union are done
  // per-warp integer counters, filled by one coalesced pass over the list
  for (int b = tid; b < (kWarps / 2) * kBins * 2; b += kThreads) (&sm.u.wbins[0][0][0])[b] = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n_a; i0 += kListBatch * kThreads) {
    uint32_t k[kListBatch];
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {  // independent loads first, so they overlap
      const int i = i0 + u * kThreads + tid;
      k[u] = i < n_a ? listA[i].key : 0u;
    }
#pragma unroll
    for (int u = 0; u < kListBatch; ++u) {
      if (i0 + u * kThreads + tid < n_a) {
        int bin = (int)(k[u] >> kBinShift) - kBinBase;
        bin = bin < 0 ? 0 : (bin < kBins ? bin : kBins - 1);
        atomicAdd(&sm.u.wbins[warp >> 1][bin][0], 1u);
        atomicAdd(&sm.u.wbins[warp >> 1][bin][1], (k[u] >> 8) & 0x1FFFu);
      }
    }
  }
  __syncthreads();
  // Per-bin counts and the mass they hold, slightly rounded down: a value whose bits are
  // (bin << 21 | off) equals edge(bin) + off * 2^(exponent - 23), and off was accumulated with
  // its top 13 bits only. Bin 0 also holds everything below the covered range, so its mass
  // counts as 0.
  if (tid < kBins) {
    unsigned c = 0, o = 0;
#pragma unroll
    for (int w = 0; w < kWarps / 2; ++w) {
      c += sm.u.wbins[w][tid][0];
      o += sm.u.wbins[w][tid][1];
    }
    const uint32_t edge_bits = (uint32_t)(tid + kBinBase) << kBinShift;
    const float edge = bits_f32(edge_bits);
    // one unit of the 13-bit offset is 2^8 units of the last place of the bin's binade
    const float unit = bits_f32(edge_bits & 0x7F800000u) * (256.0f / 8388608.0f);
    sm.hcnt[tid] = c;
    sm.hmass[tid] = tid == 0 ? 0.0f : (float)c * edge + (float)o * unit;
  }
  __syncthreads();
  if (tid < 32) {
    float acc = 0.0f;
    unsigned cacc = 0;
    int chosen = 0, chosen_cnt = n_a;
    bool done = false;
    for (int hi = kBins - 1; hi >= 0 && !done; hi -= 32) {
      const int b = hi - tid;
      float m = (b >= 0) ? sm.hmass[b] : 0.0f;
      unsigned c = (b >= 0) ? sm.hcnt[b] : 0u;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float om = __shfl_up_sync(0xffffffffu, m, d);
        const unsigned oc = __shfl_up_sync(0xffffffffu, c, d);
        if (tid >= d) {
          m += om;
          c += oc;
        }
      }
      const float mass_above = acc + m;
      const float cnt_above = (float)(cacc + c);
      const float need = sum * (topp * 1.002f + 0.001f + cnt_above * 4.8e-7f);
      // bin 0 is unbounded below, so it never counts as "above" anything
      const bool enough = b > 0 && (use_topk ? (cacc + c >= (unsigned)topk) : (mass_above >= need));
      const unsigned ok = __ballot_sync(0xffffffffu, enough);
      if (ok) {
        const int sel = __ffs(ok) - 1;
        chosen = hi - sel;
        chosen_cnt = (int)(cacc + __shfl_sync(0xffffffffu, c, sel));
        done = true;
      }
      acc += __shfl_sync(0xffffffffu, m, 31);
      cacc += __shfl_sync(0xffffffffu, c, 31);
    }
    if (tid == 0) {
      sm.misc_i[1] = chosen;
      sm.misc_i[2] = done ? 1 : 0;
      sm.misc_i[3] = chosen_cnt;
      sm.misc_f[1] = acc;  // mass of the bins looked at (all of them when the list was not enough)
    }
  }
  __syncthreads();
  *bin_out = sm.misc_i[1];
  *cnt_out = sm.misc_i[3];
  return sm.misc_i[2] != 0;
}

// Lists every entry of the row with e >= floor into list A, in index order. Returns the count.
template <typename T, typename S>
__device__ int gather_candidates(const RowMath<T, S>& rm, S& sm, Entry* listA, float floor) {
  const int tid = threadIdx.x;
  int n_a = 0;
  for (int base = 0; base < rm.vocab; base += kTile) {
    const int i0 = base + tid * kChunk;
    float e[kChunk];
    rm.chunk(i0, sm, e);  // 0 beyond the row, and floor > 0
    int cnt = 0;
#pragma unroll
    for (int j = 0; j < kChunk; ++j) cnt += (e[j] >= floor) ? 1 : 0;
    int tot;
    int off = n_a + block_excl_count(sm, cnt, &tot);
#pragma unroll
    for (int j = 0; j < kChunk; ++j) {
      if (e[j] >= floor) {
        Entry en;
        en.key = f32_bits(e[j]);
        en.idx = i0 + j;
        listA[off++] = en;
      }
    }
    n_a += tot;
  }
  __threadfence_block();
  __syncthreads();
  return n_a;
}

// Compacts list A into list B, in list order: entries with key >= key_lo whose probability
// e / sum passes the cutoff crop (sampler.cpp:136-143; no crop for top-k). List B holds the
// probabilities' bits. Two coalesced passes over list A per segment of kCompactSteps *
// kThreads entries: count the survivors of every (step, warp), prefix those counts, then
// write the survivors. Returns the number of survivors.
template <typename S>
__device__ int compact_candidates(
    S& sm, const Entry* listA, int n_a, Entry* listB, uint32_t key_lo, float sum, float cutoff,
    bool use_topk) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int n_b = 0;
  for (int seg0 = 0; seg0 < n_a; seg0 += kCompactSteps * kThreads) {
    const int seg_n = (n_a - seg0) < kCompactSteps * kThreads ? (n_a - seg0) : kCompactSteps * kThreads;
    const int steps = (seg_n + kThreads - 1) / kThreads;
    __syncthreads();  // earlier users of the union are done
    for (int st0 = 0; st0 < steps; st0 += kListBatch) {
      uint32_t k[kListBatch];
#pragma unroll
      for (int u = 0; u < kListBatch; ++u) {
        const int i = seg0 + (st0 + u) * kThreads + tid;
        k[u] = (st0 + u < steps && i < n_a) ? listA[i].key : 0u;
      }
#pragma unroll
      for (int u = 0; u < kListBatch; ++u) {
        if (st0 + u < steps) {  // block-uniform
          const int i = seg0 + (st0 + u) * kThreads + tid;
          const bool keep = i < n_a && k[u] >= key_lo &&
                            (use_topk || __fdiv_rn(bits_f32(k[u]), sum) >= cutoff);
          const unsigned kbal = __ballot_sync(0xffffffffu, keep);
          if (lane == 0) sm.u.compact.cnt[st0 + u][warp] = (unsigned short)__popc(kbal);
        }
      }
    }
    __syncthreads();
    // thread t owns step t: exclusive prefix inside the step, and the step total
    int step_total = 0;
    if (tid < steps) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int c = sm.u.compact.cnt[tid][w];
        sm.u.compact.cnt[tid][w] = (unsigned short)step_total;
        step_total += c;
      }
    }
    int seg_total;
    const int step_base = block_excl_count(sm, step_total, &seg_total);
    if (tid < steps) sm.u.compact.base[tid] = (unsigned)(n_b + step_base);
    __syncthreads();
    for (int st0 = 0; st0 < steps; st0 += kListBatch) {
      Entry en[kListBatch];
#pragma unroll
      for (int u = 0; u < kListBatch; ++u) {
        const int i = seg0 + (st0 + u) * kThreads + tid;
        en[u].key = 0;
        en[u].idx = 0;
        if (st0 + u < steps && i < n_a) en[u] = listA[i];
      }
#pragma unroll
      for (int u = 0; u < kListBatch; ++u) {
        if (st0 + u < steps) {  // block-uniform
          const int i = seg0 + (st0 + u) * kThreads + tid;
          bool keep = false;
          if (i < n_a && en[u].key >= key_lo) {
            const float p = __fdiv_rn(bits_f32(en[u].key), sum);
            keep = use_topk || p >= cutoff;
            en[u].key = f32_bits(p);
          }
          const unsigned kbal = __ballot_sync(0xffffffffu, keep);
          if (keep) {
            listB[sm.u.compact.base[st0 + u] + sm.u.compact.cnt[st0 + u][warp] +
                  __popc(kbal & ((1u << lane) - 1u))] = en[u];
          }
        }
      }
    }
    n_b += seg_total;
  }
  __threadfence_block();
  __syncthreads();
  return n_b;
}

// Sorts list B by probability, descending; equal probabilities end up in index order. Small
// lists are rank-sorted in shared memory; larger ones take four stable LSD radix passes that
// ping-pong between list B and `spare` (after an even number of passes the result is back in
// list B).
template <typename S>
__device__ void sort_candidates(S& sm, Entry* listB, int n_b, Entry* spare) {
  const int tid = threadIdx.x;
  if (n_b <= kRankSortMax) {
    // Composite key = (probability bits, inverted index): larger means earlier in the sorted
    // order. kThreads / kRankSortMax threads share an entry, each scanning a part of the list.
    const int ent = tid & (kRankSortMax - 1), part = tid / kRankSortMax;
    Entry en;
    en.key = 0;
    en.idx = 0;
    if (tid < n_b) {
      en = listB[tid];
      sm.u.rsort.ck[tid] = ((unsigned long long)en.key << 32) | (uint32_t)(0x7FFFFFFF - en.idx);
      sm.u.rsort.rank[tid] = 0;
    }
    __syncthreads();
    if (ent < n_b) {
      const unsigned long long mine = sm.u.rsort.ck[ent];
      constexpr int kParts = kThreads / kRankSortMax;
      const int per = (n_b + kParts - 1) / kParts;
      const int j0 = part * per, j1 = (j0 + per) < n_b ? (j0 + per) : n_b;
      int rank = 0;
#pragma unroll 8
      for (int j = j0; j < j1; ++j) rank += sm.u.rsort.ck[j] > mine ? 1 : 0;
      atomicAdd(&sm.u.rsort.rank[ent], rank);
    }
    __syncthreads();
    if (tid < n_b) listB[sm.u.rsort.rank[tid]] = en;
    __threadfence_block();
  } else {
    Entry* ping = listB;
    Entry* pong = spare;
    for (int pass = 0; pass < 32 / kRadixBits; ++pass) {
      radix_pass_desc(sm, ping, pong, n_b, pass * kRadixBits);
      __threadfence_block();
      Entry* t = ping;
      ping = pong;
      pong = t;
    }
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------
// The rest of sample_topp / sample_topk for a row whose survivors (list entries at or above
// the value threshold key_lo that pass the cutoff crop) number at most kRankSortMax, entirely
// in shared memory: unordered compaction (the sort key carries the index, so the list order
// does not matter), rank sort by (probability descending, index ascending), then one thread
// replays the reference's cumulative sum (sampler.cpp:146-156, or the top-k sum of
// sampler.cpp:105-108) and keeps every partial sum; the second loop of the reference
// (sampler.cpp:162-169) adds the same numbers in the same order, so its cdf values are those
// partial sums and the draw is a parallel lookup. Returns false, with nothing decided, when
// the survivors do not fit or do not suffice (the caller then takes the general path).
// `all_listed`: the list holds every entry that passes the crop and the threshold keeps all.
// ---------------------------------------------------------------------------------------
template <typename S>
__device__ bool small_tail(
    S& sm, const Entry* listA, int n_a, uint32_t key_lo, float sum, float cutoff, float topp,
    int topk, bool use_topk, bool all_listed, float coin, int* token) {
  const int tid = threadIdx.x, lane = tid & 31;
  __syncthreads();  // earlier users of the union are done
  if (tid == 0) {
    sm.u.small.cnt = 0;
    sm.u.small.first_above = 0x7fffffff;
    sm.u.small.last = -1;
  }
  __syncthreads();
  for (int i0 = 0; i0 < n_a; i0 += kThreads) {
    const int i = i0 + tid;
    bool keep = false;
    unsigned long long ck = 0ull;
    if (i < n_a) {
      const Entry en = listA[i];
      if (en.key >= key_lo) {
        const float p = __fdiv_rn(bits_f32(en.key), sum);
        keep = use_topk || p >= cutoff;
        ck = ((unsigned long long)f32_bits(p) << 32) | (uint32_t)(0x7FFFFFFF - en.idx);
      }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, keep);
    if (bal != 0u) {
      int base = 0;
      if (lane == 0) base = atomicAdd(&sm.u.small.cnt, __popc(bal));
      base = __shfl_sync(0xffffffffu, base, 0);
      const int slot = base + __popc(bal & ((1u << lane) - 1u));
      if (keep && slot < kRankSortMax) sm.u.small.ck[slot] = ck;
    }
  }
  __syncthreads();
  const int n_b = sm.u.small.cnt;
  if (n_b <= 0 || n_b > kRankSortMax) return false;
  if (use_topk && n_b < topk && !all_listed) return false;
  if (tid < n_b) {
    const unsigned long long mine = sm.u.small.ck[tid];
    int rank = 0;
#pragma unroll 8
    for (int j = 0; j < n_b; ++j) rank += sm.u.small.ck[j] > mine ? 1 : 0;
    sm.u.small.p[rank] = bits_f32((uint32_t)(mine >> 32));
    sm.u.small.idx[rank] = (int)(0x7FFFFFFFu - (uint32_t)(mine & 0xFFFFFFFFull));
  }
  __syncthreads();
  // the terms beyond the ones that count read as zero (adding zero changes no partial sum)
  const int lim = use_topk ? (topk < n_b ? topk : n_b) : n_b;
  if (tid < 8) sm.u.small.p[lim + tid] = 0.0f;
  __syncthreads();
  if (tid == 0) {
    const float4* p4 = reinterpret_cast<const float4*>(sm.u.small.p);
    float4* pre4 = reinterpret_cast<float4*>(sm.u.small.prefix);
    float acc = 0.0f;
    int last = -1;
    float4 q = p4[0];
    for (int i = 0; i < lim; i += 4) {
      const float4 nq = p4[(i >> 2) + 1];  // next group, ahead of the additions
      const float a1 = __fadd_rn(acc, q.x);
      const float a2 = __fadd_rn(a1, q.y);
      const float a3 = __fadd_rn(a2, q.z);
      const float a4 = __fadd_rn(a3, q.w);
      pre4[i >> 2] = make_float4(a1, a2, a3, a4);
      if (!use_topk && a4 > topp) {  // the partial sums only grow: the first one above topp
        int k = 3;
        float hv = a4;
        if (a3 > topp) { k = 2; hv = a3; }
        if (a2 > topp) { k = 1; hv = a2; }
        if (a1 > topp) { k = 0; hv = a1; }
        last = i + k;
        acc = hv;
        break;
      }
      acc = a4;
      q = nq;
    }
    // top-k keeps its k entries; top-p keeps everything when the sum never exceeds topp
    // (the "in case of rounding errors" branch, sampler.cpp:152), which is only known to be
    // everything when all candidates were listed
    if (use_topk || (last < 0 && all_listed)) last = lim - 1;
    sm.u.small.last = last;
    sm.u.small.cum = acc;
  }
  __syncthreads();
  const int last = sm.u.small.last;
  if (last < 0) return false;
  const float r = __fmul_rn(coin, sm.u.small.cum);  // sampler.cpp:162
  {
    const bool above = tid <= last && sm.u.small.prefix[tid] > r;
    const unsigned bal = __ballot_sync(0xffffffffu, above);
    if (bal != 0u && lane == 0) atomicMin(&sm.u.small.first_above, (tid & ~31) + __ffs(bal) - 1);
  }
  __syncthreads();
  const int fa = sm.u.small.first_above;
  *token = sm.u.small.idx[fa <= last ? fa : last];
  __syncthreads();  // the union may be reused by the caller
  return true;
}

// Greedy choice for one row inside the sampling kernel (extended entry point): strict '>' in
// index order on the values the sampler sees, as sample_argmax (sampler.cpp:44-56) -- the
// lowest index among equal maxima, a NaN never replaces the running maximum, a NaN in
// element 0 is never replaced. Block-uniform result.
template <typename T, typename S>
__device__ int block_argmax(S& sm, const RowMath<T, S>& rm, int vocab) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = tid; i < vocab; i += kThreads) {
    const float x = rm.xform(to_f32(rm.row[i]));
    if (x > best) {
      best = x;
      besti = i;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, d);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, d);
    if (ov > best || (ov == best && oi < besti)) {
      best = ov;
      besti = oi;
    }
  }
  __syncthreads();
  if (lane == 0) {
    sm.redf[warp] = best;
    sm.redi[warp] = besti;
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kWarps; ++w) {
      if (sm.redf[w] > best || (sm.redf[w] == best && sm.redi[w] < besti)) {
        best = sm.redf[w];
        besti = sm.redi[w];
      }
    }
    const float first = rm.xform(to_f32(rm.row[0]));
    sm.misc_i[0] = (first != first || besti == 0x7fffffff) ? 0 : besti;
  }
  __syncthreads();
  const int token = sm.misc_i[0];
  __syncthreads();
  return token;
}

#include "guided_sum.cuh"
#include "value_class_tail.cuh"

// ---------------------------------------------------------------------------------------
// The sampling kernel (temperature != 0): multinomial when topp is outside (0, 1), top-p
// otherwise. Follows Sampler::sample<float> (sampler.cpp:222-251).
// ---------------------------------------------------------------------------------------
template <typename T, bool kLut, bool kGuided, bool kExt = false>
__global__ void __launch_bounds__(kThreads, 2) sample_rows_kernel(
    const T* __restrict__ logits, int64_t rows, int vocab, int64_t row_stride, float inv_t0,
    float topp0, int topk0, unsigned long long* __restrict__ rng_states,
    int64_t* __restrict__ out_ids, PeerOut peers, Entry* scratch, ExpTable table,
    int* __restrict__ status, const int* __restrict__ row_list, const int* __restrict__ row_count,
    int* __restrict__ retry_rows, int* __restrict__ retry_count, int* __restrict__ retry_count_next,
    RowSettings ext) {
  using S = Shared<kLut, kGuided, kExt>;
  // the block's shared state exceeds the 48 KB static limit: dynamic shared memory, sized
  // sizeof(S) by the launcher
  extern __shared__ __align__(16) unsigned char smem_raw[];
  S& sm = *reinterpret_cast<S*>(smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < kExpTableSize) sm.exp_tab[tid] = table.t[tid];
  int rp = 0;  // which set of scan-round slots the next round uses (see seqsum_tile)
  // Guessed floor under the values that matter (nucleus members / the k largest). Pass 2 lists
  // only e >= guess; if that turns out to be too high for a row, the row is regathered with
  // its exact floor and the guess is lowered for the block's later rows.
  float guess = kGuessFloor;
  uint32_t copy_parity = 0u;  // phase of the tile-copy barrier (guided variant)
  if constexpr (kGuided) {
    if (tid == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&sm.g.mbar)), "r"(1u));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      // the retry counter that the NEXT call will use is cleared here (calls are ordered)
      if (blockIdx.x == 0 && retry_count_next != nullptr) *retry_count_next = 0;
    }
  }
  __syncthreads();
  Entry* listA = scratch + (size_t)blockIdx.x * 2 * (size_t)vocab;
  Entry* listB = listA + vocab;

  // with a row list (rows that the cluster kernel left undecided) only those rows are sampled;
  // that launch may have become resident before the kernel that writes the list has ended
  if (row_list != nullptr) {
    grid_dependency_wait();
    ETB_GSTAMP(15);
  }
  const int64_t n_todo = row_list != nullptr ? (int64_t)*row_count : rows;
  // Rows that finish in the value-class tail are only recorded inside the row loop; the block runs
  // those tails in batches outside it. (A call inside the loop costs every row: the state that
  // lives across it no longer fits the registers.)
  // (The bookkeeping of this lives in shared memory: the row loop has no register to spare.)
  if (tid == 0) sm.vcc.n_pend = 0;
  __syncthreads();
  int64_t it = blockIdx.x;
  for (;;) {
  for (; it < n_todo && sm.vcc.n_pend < kVcPendCap; it += gridDim.x) {
    const int64_t r = row_list != nullptr ? (int64_t)row_list[it] : it;
    // the row's settings: the handle's, or -- extended entry point -- its own
    // (LLMSession's SamplingConfig{temperature, top_p, top_k, seed}, llm_session.h:29-34)
    float inv_t = inv_t0, topp = topp0;
    int topk = topk0;
    if constexpr (kExt) {
      if (ext.temperature != nullptr) {
        const float t = ext.temperature[r];
        inv_t = t > 0.0f ? 1.0f / t : 0.0f;  // as Sampler::set_temperature: negative counts as 0
      }
      if (ext.topp != nullptr) topp = ext.topp[r];
      if (ext.topk != nullptr) topk = ext.topk[r];
    }
    // mode selection of Sampler::sample (sampler.cpp:239-248): top-k wins over top-p
    const bool use_topk = topk > 0 && topk < vocab;
    const bool use_topp = !use_topk && !(topp <= 0.0f || topp >= 1.0f);
    const bool use_list = use_topk || use_topp;  // modes that collect candidates during pass 2
    RowMath<T, S> rm;
    rm.row = logits + r * row_stride;
    rm.vocab = vocab;
    rm.vec_ok = (reinterpret_cast<uintptr_t>(rm.row) & 15u) == 0;
    rm.inv_t = inv_t;
    rm.sum = 1.0f;
    rm.probs = false;
    if constexpr (kExt) {
      rm.scale = ext.scale;
      if (inv_t == 0.0f) {
        // a greedy row among sampled ones (sampler.cpp:226-228): no coin, the state stays
        const int token = block_argmax(sm, rm, vocab);
        store_token(out_ids, peers, r, token);
        __syncthreads();
        continue;
      }
    }

    ETB_STAMP(0);
    // ---- pass 1: max of the scaled logits
    {
      float raw_max;
      rm.mx = row_max_scaled<T>(sm, rm, rm.row, vocab, rm.vec_ok, inv_t, &raw_max);
      if constexpr (sizeof(T) == 2 && S::kHasClassTail) {
        if (tid == 0) {
          // a 16-bit top-p row with finite logits can finish in the value-class tail
          const bool topp_row = !(topk > 0 && topk < vocab) && !(topp <= 0.0f || topp >= 1.0f);
          sm.vcc.raw_max = raw_max;
          sm.vcc.class_ok = (topp_row && fabsf(raw_max) < INFINITY && fabsf(rm.mx) < INFINITY &&
                             vocab <= kVcSelTiles * kVcSelTile) ? 1 : 0;
        }
      }
    }

    // the coin is drawn once per sampled row (sampler.cpp:237); the guided variant stores the
    // advanced state only once it knows that it decides the row
    unsigned long long st_next = 0ull;
    if (tid == 0) {
      st_next = rng_states[r];
      sm.misc_f[0] = next_coin(&st_next);
      if constexpr (!kGuided) rng_states[r] = st_next;
    }
    ETB_STAMP(1);
    if constexpr (kLut) {
      rm.build_lut(sm);  // the previous row's readers are behind the barriers of block_max
    }

    // ---- pass 2: e_i = expf(x_i - max) and their float sum in index order
    // (sampler.cpp:198-203). Top-p also lists every entry that can pass the cutoff crop of
    // sampler.cpp:136-143: p_i >= cutoff needs e_i >= cutoff * S and S >= 1 (the maximum
    // contributes exactly 1), so e_i >= cutoff * (1 - 1e-6) is necessary.
    const float cutoff = __fdiv_rn(__fsub_rn(1.0f, topp), (float)(vocab - 1));
    // Top-k has no crop: its exact floor is "e > 0". Both modes list only e >= max(exact
    // floor, guess) here and verify afterwards that this was enough.
    const float exact_floor0 = use_topp ? cutoff * 0.999999f : 1.4e-45f;
    const float e_floor = use_list ? fmaxf(exact_floor0, guess) : 0.0f;
    // A 16-bit top-p row whose list outgrows kVcListCap has a long nucleus: listing stops there
    // and the row is finished from its value classes instead (value_class_tail.cuh).
    bool listing = use_list;  // block-uniform
    float s = 0.0f;
    int n_a = 0;
    if constexpr (kGuided) {
      // estimate-guided sum (guided_sum.cuh); a row it does not take or cannot decide goes to the
      // retry list, untouched, for the variant without it
      __syncthreads();  // the table is complete
      bool ok = false;
      if constexpr (sizeof(T) == 2) {
        if (rm.vec_ok && vocab <= kGMaxTiles * kGTile) {
          ok = guided_sum_pass(sm, rm, copy_parity, use_list, e_floor, listA, &n_a, &s);
        }
      }
      if (!ok) {
        if (tid == 0) retry_rows[atomicAdd(retry_count, 1)] = (int)r;
        __syncthreads();
        continue;
      }
      if (tid == 0) rng_states[r] = st_next;
    }
    if constexpr (!kGuided) {
    {
      // head: the first kHead terms are added by one thread (a sum changes binade every few
      // additions at its start); their candidates are listed by all threads meanwhile
      __syncthreads();  // the table is complete
      const int cnt = vocab < kHead ? vocab : kHead;
      float e_mine = 0.0f;
      if (tid < kHead) {
        e_mine = rm.at(tid, sm);
        sm.head[tid] = e_mine;
      }
      const bool cand = use_list && tid < cnt && e_mine >= e_floor;
      const unsigned cb = __ballot_sync(0xffffffffu, cand);
      if (lane == 0) sm.wcnt[0][warp] = __popc(cb);
      __syncthreads();
      if (tid == 0) {
        float acc = 0.0f;
        const float4* h4 = reinterpret_cast<const float4*>(sm.head);
        for (int i = 0; i < cnt; i += 4) {
          const float4 q = h4[i >> 2];  // zero beyond the row
          acc = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(acc, q.x), q.y), q.z), q.w);
        }
        sm.s_bcast = acc;
      }
      int pre = 0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const int c = sm.wcnt[0][w];
        if (w < warp) pre += c;
        n_a += c;
      }
      if (cand) {
        Entry en;
        en.key = f32_bits(e_mine);
        en.idx = tid;
        listA[pre + __popc(cb & ((1u << lane) - 1u))] = en;
      }
      __syncthreads();
      s = sm.s_bcast;
    }
    int buf = 0;
    constexpr bool kPrefetch = sizeof(T) == 2;  // 8 registers; fp32 chunks would need 16
    typename RowMath<T, S>::Raw raw_next;
    if (kPrefetch && kHead < vocab && rm.full(kHead + tid * kChunk)) rm.load_raw(kHead + tid * kChunk, &raw_next);
    for (int base = kHead; base < vocab; base += kTile) {
      const int i0 = base + tid * kChunk;
      float e[kChunk];
      if (kPrefetch) {
        if (rm.full(i0)) {
          const typename RowMath<T, S>::Raw raw = raw_next;
          const int inext = i0 + kTile;
          if (inext < vocab && rm.full(inext)) rm.load_raw(inext, &raw_next);
          rm.eval_raw(raw, sm, e);
        } else {
#pragma unroll
          for (int j = 0; j < kChunk; ++j) e[j] = rm.at(i0 + j, sm);
        }
      } else {
        rm.chunk(i0, sm, e);
      }
      // p_i >= cutoff needs e_i >= cutoff * S, and S is at least the running sum so far
      const float floor_now = use_topp ? fmaxf(e_floor, cutoff * s * 0.999999f) : e_floor;
      (void)exact_floor0;
      int cnt = 0, inc = 0;
      unsigned cmask = 0;  // bit j: e[j] is a candidate
      if (listing) {
        // entries beyond the row are 0 and the floor is > 0, so they never count.
        // e >= floor is e > f for the float f just below the floor; with B = 1 / ulp(f) the
        // fused e * B - f * B is >= 1 in the first case and <= 0 otherwise, so its saturation
        // is the indicator, and the indicators weighted by 2^j add up to the mask exactly:
        // float multiply-adds only, none of the scarce compare/logic instructions.
        const uint32_t fbits = f32_bits(floor_now) - 1u;  // floor_now >= 2^-100
        const float big = bits_f32((277u - (fbits >> 23)) << 23);
        const float neg_c = -__fmul_rn(bits_f32(fbits), big);
        float m4[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // interleaved: short dependency chains
#pragma unroll
        for (int j = 0; j < kChunk; ++j) {
          const float ind = __saturatef(__fmaf_rn(e[j], big, neg_c));
          m4[j & 3] = __fmaf_rn(ind, (float)(1u << j), m4[j & 3]);
        }
        cmask = (unsigned)((m4[0] + m4[1]) + (m4[2] + m4[3]));
        cnt = __popc(cmask);
        inc = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int o = __shfl_up_sync(0xffffffffu, inc, d);
          if (lane >= d) inc += o;
        }
        if (lane == 31) sm.wcnt[buf][warp] = inc;  // published by the barriers of seqsum_tile
      }
      int hp;
      float hs;
      const bool first_tile = base == kHead;  // block-uniform
      if (first_tile) {
        // The running sum leaves its binade every few hundred terms here, and every such
        // round would occupy the whole block: stage the tile's terms in shared memory and
        // let one warp sum them, 512 at a time, while the others list their candidates.
        stage_first_tile(sm, e);  // its barrier also publishes the candidate counts
      } else {
        seqsum_tile<false>(sm, e, s, rp, 0.0f, base, vocab, &hp, &hs);
      }
      if (listing) {
        // candidates of the warps in front of this one, and of the whole tile
        const int wc = lane < kWarps ? sm.wcnt[buf][lane] : 0;
        const int pre = __reduce_add_sync(0xffffffffu, lane < warp ? wc : 0);
        const int tot = __reduce_add_sync(0xffffffffu, wc);
        int off = n_a + pre + inc - cnt;
        // Candidates are rare (well under 1 % of the logits): visit only the groups of four
        // positions in which some lane of the warp has one.
        const unsigned any = __reduce_or_sync(0xffffffffu, cmask);
#pragma unroll
        for (int g = 0; g < kChunk; g += 4) {
          if (any & (0xFu << g)) {  // warp-uniform
#pragma unroll
            for (int j = g; j < g + 4; ++j) {
              if (cmask & (1u << j)) {
                Entry en;
                en.key = f32_bits(e[j]);
                en.idx = i0 + j;
                listA[off++] = en;
              }
            }
          }
        }
        n_a += tot;
        buf ^= 1;
        if constexpr (sizeof(T) == 2 && S::kHasClassTail) {
          // n_a is the same in every thread; the flag was published by the barriers since pass 1
          // (sorting is the faster finish up to about kVcListCap candidates; candidates are
          // spread over the row, so a dense start tells early that there will be far more)
          const long long seen = (long long)base + kTile;
          if (n_a > kVcListProbe && (long long)n_a * vocab > (long long)kVcListCap * seen &&
              sm.vcc.class_ok != 0) {
            listing = false;
          }
        }
      }
      if (first_tile) sum_staged_tile<false>(sm, s, 0.0f, vocab, &hp, &hs);
    }
    }  // !kGuided
    const float sum = s;
    ETB_STAMP(2);
    __syncthreads();
    const float coin = sm.misc_f[0];
    int token;
    bool deferred = false;  // the row finishes in the value-class tail, after the row loop

    if (!use_list) {
      // ---- pass 3a: sample_mult (sampler.cpp:58-70): running float cdf of p_i = e_i / S
      token = vocab - 1;
      rm.sum = sum;
      rm.probs = true;
      if constexpr (kLut) {
        rm.build_lut(sm);  // the table now holds probabilities
      }
      float cdf = 0.0f;
      int hp;
      float hs;
      __syncthreads();
      const int cnt = vocab < kHead ? vocab : kHead;
      if (tid < kHead) sm.head[tid] = rm.at(tid, sm);
      bool hit = head_sum<true>(sm, cnt, cdf, coin, 0, &hp, &hs);
      for (int base = kHead; base < vocab && !hit; base += kTile) {
        float p[kChunk];
        rm.chunk(base + tid * kChunk, sm, p);
        if (base == kHead) {
          stage_first_tile(sm, p);
          hit = sum_staged_tile<true>(sm, cdf, coin, vocab, &hp, &hs);
        } else {
          hit = seqsum_tile<true>(sm, p, cdf, rp, coin, base, vocab, &hp, &hs);
        }
      }
      if (hit) token = hp;
    } else {
      // ---- pass 3b: sample_topp (sampler.cpp:122-171) or sample_topk (sampler.cpp:72-120)
      __threadfence_block();
      __syncthreads();
      // List A holds every entry with e >= max(exact floor, guess) ("complete" when the guess
      // was not above the exact floor). Each round: pick a value threshold from the bins,
      // compact, sort, and replay the reference's cumulative sums; a round that cannot
      // succeed first completes the list (regather with the exact floor, now that S is known)
      // and then widens the threshold to everything listed.
      const float exact_floor = use_topp ? cutoff * sum * 0.999999f : 1.4e-45f;
      bool complete = e_floor <= exact_floor;
      bool take_all = false;
      int n_b = 0, last_idx = 0;
      float cum = 0.0f;
      bool have = false, token_ready = false;
      token = 0;
      if constexpr (sizeof(T) == 2 && S::kHasClassTail) {
        if (!listing) {
          // the list was abandoned: a long nucleus, finished without list or sort
          deferred = true;
          have = true;  // skips the rounds below
        }
      }
      for (int round = 0; round < 4 && !have; ++round) {
        int bin_lo = 0, kept = n_a;
        bool enough = true;
        if (!take_all) enough = pick_value_threshold(sm, listA, n_a, sum, topp, topk, use_topk, &bin_lo, &kept);
        if constexpr (sizeof(T) == 2 && S::kHasClassTail) {
          if (!enough && !complete && sm.vcc.class_ok != 0) {
            // Every token that is not listed has e < e_floor, so the nucleus needs at least
            // (missing mass) / e_floor more of them: a long nucleus takes the class tail at once.
            const float missing = topp * sum - sm.misc_f[1];
            if ((float)n_a + missing / e_floor > (float)kVcMinNucleus) {
              deferred = true;
              break;
            }
          }
        }
        if (!enough && !complete) {
          guess = fmaxf(guess * 0.0625f, 1e-30f);  // later rows of this block start lower
          n_a = gather_candidates(rm, sm, listA, exact_floor);
          complete = true;
          continue;
        }
        if (!take_all && kept <= kRankSortMax) {
          // short nucleus (the usual case): finish in shared memory
          const uint32_t klo = bin_lo > 0 ? (uint32_t)(bin_lo + kBinBase) << kBinShift : 0u;
          int tk;
          if (small_tail(sm, listA, n_a, klo, sum, cutoff, topp, topk, use_topk, bin_lo == 0 && complete,
                         coin, &tk)) {
            token_ready = true;
            token = tk;
            break;
          }
        }
        // The radix sort ping-pongs into the free space behind list A. If the survivors may
        // not fit there, list A itself is the spare buffer, which is only allowed when list A
        // will not be needed again: make this the final round by taking everything listed
        // from a complete list.
        bool spare_is_list_a = false;
        if (n_a + kept > vocab) {
          if (!complete) {
            n_a = gather_candidates(rm, sm, listA, exact_floor);
            complete = true;
            continue;
          }
          if (!use_topk) bin_lo = 0;  // top-k's count threshold is exact: no later round either way
          spare_is_list_a = true;
        }
        const uint32_t key_lo = bin_lo > 0 ? (uint32_t)(bin_lo + kBinBase) << kBinShift : 0u;
        n_b = compact_candidates(sm, listA, n_a, listB, key_lo, sum, cutoff, use_topk);
        sort_candidates(sm, listB, n_b, spare_is_list_a ? listA : listA + n_a);
        int pos;
        float hs, total;
        if (use_topk) {
          // the k most probable entries (fewer if fewer have e > 0); their float sum in
          // sorted order is topk_sum (sampler.cpp:105-108)
          if (n_b >= topk || complete) {
            const int kk = topk < n_b ? topk : n_b;
            list_search(sm, listB, n_b, kk, INFINITY, rp, &pos, &hs, &total);
            have = true;
            last_idx = kk - 1;
            cum = total;
          } else {
            n_a = gather_candidates(rm, sm, listA, exact_floor);
            complete = true;
          }
        } else if (list_search(sm, listB, n_b, n_b, topp, rp, &pos, &hs, &total)) {
          have = true;
          last_idx = pos;
          cum = hs;
        } else if (bin_lo == 0 && complete) {
          // every candidate is in and the sum never exceeded topp: keep everything
          // (the "in case of rounding errors" branch, sampler.cpp:152)
          have = true;
          last_idx = n_b - 1;
          cum = total;
        } else if (!complete) {
          n_a = gather_candidates(rm, sm, listA, exact_floor);
          complete = true;
        } else {
          take_all = true;  // the value threshold was too optimistic: take all candidates
        }
      }
      if (deferred) {
        if (tid == 0) {
          VcControl::Pending pd;
          pd.row = (long long)r;
          pd.inv_t = inv_t;
          pd.mx = rm.mx;
          pd.sum = sum;
          pd.cutoff = cutoff;
          pd.topp = topp;
          pd.coin = coin;
          pd.raw_max = sm.vcc.raw_max;
          sm.vcc.pend[sm.vcc.n_pend] = pd;
          sm.vcc.n_pend += 1;  // read again behind the barrier that ends the row
        }
      } else if (token_ready) {
        // decided by small_tail
      } else if (n_b <= 0 || !have) {
        token = 0;  // no candidate at all (NaN rows): undefined in the reference
      } else {
        const float rr = __fmul_rn(coin, cum);  // sampler.cpp:162
        int pos;
        float hs, total;
        int j = last_idx;
        if (list_search(sm, listB, n_b, last_idx + 1, rr, rp, &pos, &hs, &total)) j = pos;
        token = listB[j].idx;
      }
    }
    ETB_STAMP(6);
    if (!deferred) store_token(out_ids, peers, r, token);
    __syncthreads();
  }
  if constexpr (sizeof(T) == 2 && S::kHasClassTail) {
    // ---- the deferred value-class tails
    const int n_pend = sm.vcc.n_pend;
    for (int k = 0; k < n_pend; ++k) {
      __syncthreads();
      const VcControl::Pending pd = sm.vcc.pend[k];
      RowMath<T, S> rm;
      rm.row = logits + pd.row * row_stride;
      rm.vocab = vocab;
      rm.vec_ok = (reinterpret_cast<uintptr_t>(rm.row) & 15u) == 0;
      rm.inv_t = pd.inv_t;
      rm.mx = pd.mx;
      rm.sum = 1.0f;
      rm.probs = false;
      if constexpr (kExt) rm.scale = ext.scale;
      int token = value_class_tail(sm, rm, pd.sum, pd.cutoff, pd.topp, pd.coin, pd.raw_max);
      if (token < 0) {
        // -1: no candidate at all, undefined in the reference (token 0 like the sorted path);
        // -2: counts that do not add up, which the host can read from the status word
        if (token == -2 && tid == 0 && status != nullptr) atomicMax(status, kStatusTailInconsistent);
        token = 0;
      }
      ETB_STAMP(6);
      store_token(out_ids, peers, pd.row, token);
    }
    __syncthreads();
  }
  if (tid == 0) sm.vcc.n_pend = 0;
  __syncthreads();
  if (it >= n_todo) break;
  }
  peer_arrival_barrier(peers, status);
}

// ---------------------------------------------------------------------------------------
// Greedy kernel (temperature == 0): sample_argmax (sampler.cpp:44-56). Strict '>' in
// index order: the lowest index among equal maxima wins, -0 equals +0, a NaN never
// replaces the running maximum, and a NaN in element 0 is never replaced.
// ---------------------------------------------------------------------------------------
// Each thread keeps eight 128-bit loads in flight per iteration, each of them contiguous
// across the warp: with one block per row and fewer than two blocks per SM at batch 256, the
// bytes in flight decide the bandwidth.
constexpr int kArgVecs = 8;

template <typename T, bool kRawU16>
__global__ void __launch_bounds__(kThreads, 2) argmax_rows_kernel(
    const T* __restrict__ logits, int64_t rows, int vocab, int64_t row_stride,
    int64_t* __restrict__ out_ids, PeerOut peers, int* __restrict__ status) {
  constexpr int kPerVec = 16 / sizeof(T);
  __shared__ float sv[kWarps];
  __shared__ int si[kWarps];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* row = logits + r * row_stride;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const uint4* row4 = reinterpret_cast<const uint4*>(row);
    const int nvec = vec_ok ? vocab / kPerVec : 0;
    float best = -INFINITY;
    int besti = 0x7fffffff;  // "nothing better than -inf seen": resolved to the first index below
    // A thread visits its elements in increasing index order (vector q * kThreads + tid of
    // each group, then the ragged tail), so strict '>' keeps its lowest index of a maximum.
    for (int v0 = 0; v0 < nvec; v0 += kThreads * kArgVecs) {
      uint4 raw[kArgVecs];
#pragma unroll
      for (int q = 0; q < kArgVecs; ++q) {
        const int v = v0 + q * kThreads + tid;
        if (v < nvec) raw[q] = __ldg(row4 + v);
      }
#pragma unroll
      for (int q = 0; q < kArgVecs; ++q) {
        const int v = v0 + q * kThreads + tid;
        if (v < nvec) {
          const T* p = reinterpret_cast<const T*>(&raw[q]);
#pragma unroll
          for (int j = 0; j < kPerVec; ++j) {
            float x;
            if constexpr (kRawU16) {
              x = (float)p[j];  // sample<uint16_t> compares the raw integers
            } else {
              x = to_f32(p[j]);
            }
            if (x > best) {
              best = x;
              besti = v * kPerVec + j;
            }
          }
        }
      }
    }
    for (int i = nvec * kPerVec + tid; i < vocab; i += kThreads) {
      float x;
      if constexpr (kRawU16) {
        x = (float)row[i];
      } else {
        x = to_f32(row[i]);
      }
      if (x > best) {
        best = x;
        besti = i;
      }
    }
    // combine: larger value wins, equal values keep the lower index
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, d);
      const int oi = __shfl_xor_sync(0xffffffffu, besti, d);
      if (ov > best || (ov == best && oi < besti)) {
        best = ov;
        besti = oi;
      }
    }
    __syncthreads();
    if (lane == 0) {
      sv[warp] = best;
      si[warp] = besti;
    }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < kWarps; ++w) {
        if (sv[w] > best || (sv[w] == best && si[w] < besti)) {
          best = sv[w];
          besti = si[w];
        }
      }
      // Sequential semantics at the edges: the scan starts from element 0, so if nothing
      // compares greater than it (all -inf, or element 0 is NaN) the answer is 0. A running
      // maximum of -inf is only replaced by something greater, so "all -inf" also yields 0.
      int ans = besti;
      float first;
      if constexpr (kRawU16) {
        first = (float)row[0];
      } else {
        first = to_f32(row[0]);
      }
      if (first != first) {
        ans = 0;  // NaN at index 0 is never replaced
      } else if (besti == 0x7fffffff) {
        ans = 0;
      }
      sv[0] = __int_as_float(ans);
    }
    __syncthreads();
    store_token(out_ids, peers, r, __float_as_int(sv[0]));
  }
  peer_arrival_barrier(peers, status);
}

#include "cluster_topp.cuh"

__global__ void expf_selftest_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n,
                                     ExpTable table) {
  __shared__ uint64_t tab[kExpTableSize];
  if (threadIdx.x < kExpTableSize) tab[threadIdx.x] = table.t[threadIdx.x];
  __syncthreads();
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    y[i] = expf_ref(x[i], tab);
  }
}

}  // namespace

cudaError_t launch_expf_selftest(const float* x, float* y, int64_t n, const ExpTable& table,
                                 cudaStream_t stream) {
  if (n <= 0) return cudaSuccess;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  expf_selftest_kernel<<<(int)blocks, 256, 0, stream>>>(x, y, n, table);
  return cudaGetLastError();
}

// cudaFuncSetAttribute is needed once per function and device, not once per launch (the batch-1
// decode loop launches three kernels per token: the host side of a launch matters there).
struct OncePerDevice {
  std::atomic<unsigned long long> mask{0ull};
};
static cudaError_t func_attr_once(OncePerDevice& once, const void* func, cudaFuncAttribute attr, int value) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  const unsigned long long bit = dev < 64 ? 1ull << dev : 0ull;
  if (bit != 0ull && (once.mask.load(std::memory_order_acquire) & bit) != 0ull) return cudaSuccess;
  e = cudaFuncSetAttribute(func, attr, value);
  if (e == cudaSuccess && bit != 0ull) once.mask.fetch_or(bit, std::memory_order_release);
  return e;
}

// Launch attribute of a kernel that may become resident while its predecessor in the stream
// still runs; such a kernel calls grid_dependency_wait() before it touches anything the
// predecessor writes.
static void programmatic_launch(cudaLaunchAttribute* attr) {
  attr->id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr->val.programmaticStreamSerializationAllowed = 1;
}

size_t sampler_scratch_bytes(int vocab, int blocks) {
  return (size_t)blocks * 2 * (size_t)vocab * sizeof(Entry);
}

int sampler_threads() { return kThreads; }

// Opts the kernel in to its dynamic shared-memory size (once per device would do; the call is
// cheap and idempotent).
template <typename T, bool kLut, bool kGuided = false>
static cudaError_t prepare_sample_kernel() {
  static OncePerDevice once;
  return func_attr_once(once, reinterpret_cast<const void*>(sample_rows_kernel<T, kLut, kGuided>),
                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared<kLut, kGuided>));
}

template <typename T, bool kLut>
static cudaError_t launch_sample_t(
    const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers, void* scratch,
    int blocks, const ExpTable& table, int* status, const int* row_list, const int* row_count,
    cudaStream_t stream) {
  const cudaError_t attr = prepare_sample_kernel<T, kLut>();
  if (attr != cudaSuccess) return attr;
  if (row_list != nullptr) {
    // the pass over the rows that a fast kernel left undecided: resident early, waits for its
    // predecessor before it reads the list
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = sizeof(Shared<kLut>);
    cfg.stream = stream;
    cudaLaunchAttribute la[1];
    programmatic_launch(&la[0]);
    cfg.attrs = la;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sample_rows_kernel<T, kLut, false>, static_cast<const T*>(logits), rows, vocab,
                              row_stride, inv_t, topp, topk, rng_states, out_ids, peers,
                              static_cast<Entry*>(scratch), table, status, row_list, row_count,
                              static_cast<int*>(nullptr), static_cast<int*>(nullptr), static_cast<int*>(nullptr),
                              RowSettings{nullptr, nullptr, nullptr, 1.0f});
  }
  sample_rows_kernel<T, kLut, false><<<blocks, kThreads, sizeof(Shared<kLut>), stream>>>(
      static_cast<const T*>(logits), rows, vocab, row_stride, inv_t, topp, topk, rng_states, out_ids,
      peers,
      static_cast<Entry*>(scratch), table, status, row_list, row_count, nullptr, nullptr, nullptr,
      RowSettings{nullptr, nullptr, nullptr, 1.0f});
  return cudaGetLastError();
}

template <typename T, bool kLut>
static cudaError_t launch_guided_t(
    const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers, void* scratch,
    int blocks, const ExpTable& table, int* status, int* retry_rows, int* retry_count,
    int* retry_count_next, cudaStream_t stream) {
  const cudaError_t attr = prepare_sample_kernel<T, kLut, true>();
  if (attr != cudaSuccess) return attr;
  sample_rows_kernel<T, kLut, true><<<blocks, kThreads, sizeof(Shared<kLut, true>), stream>>>(
      static_cast<const T*>(logits), rows, vocab, row_stride, inv_t, topp, topk, rng_states, out_ids,
      peers, static_cast<Entry*>(scratch), table, status, nullptr, nullptr, retry_rows, retry_count,
      retry_count_next, RowSettings{nullptr, nullptr, nullptr, 1.0f});
  return cudaGetLastError();
}

cudaError_t launch_sample_rows(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t,
    float topp, int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers,
    void* scratch, int blocks, const ExpTable& table, int* status, cudaStream_t stream,
    const int* row_list, const int* row_count) {
  switch (dtype) {
    case kDtypeFloat:
      return launch_sample_t<float, false>(logits, rows, vocab, row_stride, inv_t, topp, topk,
                                           rng_states, out_ids, peers, scratch, blocks, table, status,
                                           row_list, row_count, stream);
    case kDtypeHalf:
      return launch_sample_t<__half, false>(logits, rows, vocab, row_stride, inv_t, topp, topk,
                                            rng_states, out_ids, peers, scratch, blocks, table, status,
                                            row_list, row_count, stream);
    case kDtypeBFloat16:
      return launch_sample_t<__nv_bfloat16, true>(logits, rows, vocab, row_stride, inv_t, topp, topk,
                                                  rng_states, out_ids, peers, scratch, blocks, table,
                                                  status, row_list, row_count, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

namespace {

// One thread per edit: logits[row][id] = T(float(logits[row][id]) + bias), what a mask or bias
// logit processor does in place (logit_processor.h:34-40).
template <typename T>
__global__ void apply_row_edits_kernel(T* logits, int64_t rows, int vocab, int64_t row_stride, RowEdits ed,
                                       long long total) {
  const long long j = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (j >= total) return;
  int64_t row;
  long long e;
  if (ed.offsets == nullptr) {
    row = j / ed.n_shared;
    e = j % ed.n_shared;
  } else {
    // the row that owns entry j: the last row whose first entry is not behind j
    int64_t lo = 0, hi = rows - 1;
    while (lo < hi) {
      const int64_t mid = (lo + hi + 1) / 2;
      if (ed.offsets[mid] <= j) lo = mid; else hi = mid - 1;
    }
    row = lo;
    e = j;
  }
  const int id = ed.ids[e];
  if (id < 0 || id >= vocab) return;  // out of range: no-op, as the reference's processors
  T* p = logits + row * row_stride + id;
  const float v = to_f32(*p) + ed.bias[e];
  if constexpr (std::is_same<T, float>::value) {
    *p = v;
  } else if constexpr (std::is_same<T, __half>::value) {
    *p = __float2half_rn(v);
  } else {
    *p = __float2bfloat16_rn(v);
  }
}

template <typename T, bool kLut>
cudaError_t launch_ext_t(
    void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp, int topk,
    const RowSettings& settings, const RowEdits& edits, long long n_edits, unsigned long long* rng_states,
    int64_t* out_ids, void* scratch, int blocks, const ExpTable& table, int* status, cudaStream_t stream) {
  if (n_edits > 0) {
    const long long grid = (n_edits + 255) / 256;
    apply_row_edits_kernel<T><<<(unsigned)grid, 256, 0, stream>>>(static_cast<T*>(logits), rows, vocab, row_stride,
                                                                  edits, n_edits);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  cudaError_t attr = cudaFuncSetAttribute(sample_rows_kernel<T, kLut, false, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)sizeof(Shared<kLut, false, true>));
  if (attr != cudaSuccess) return attr;
  sample_rows_kernel<T, kLut, false, true><<<blocks, kThreads, sizeof(Shared<kLut, false, true>), stream>>>(
      static_cast<const T*>(logits), rows, vocab, row_stride, inv_t, topp, topk, rng_states, out_ids, PeerOut{},
      static_cast<Entry*>(scratch), table, status, nullptr, nullptr, nullptr, nullptr, nullptr, settings);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_sample_rows_ext(
    int dtype, void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    int topk, const RowSettings& settings, const RowEdits& edits, unsigned long long* rng_states,
    int64_t* out_ids, void* scratch, int blocks, const ExpTable& table, int* status, cudaStream_t stream) {
  // how many edits there are is known on the host: shared lists directly, per-row lists by
  // their last offset, which the caller passes in n_shared as well
  const long long n_edits = edits.ids == nullptr ? 0 : (edits.offsets == nullptr ? edits.n_shared * rows : edits.n_shared);
  switch (dtype) {
    case kDtypeFloat:
      return launch_ext_t<float, false>(logits, rows, vocab, row_stride, inv_t, topp, topk, settings, edits,
                                        n_edits, rng_states, out_ids, scratch, blocks, table, status, stream);
    case kDtypeHalf:
      return launch_ext_t<__half, false>(logits, rows, vocab, row_stride, inv_t, topp, topk, settings, edits,
                                         n_edits, rng_states, out_ids, scratch, blocks, table, status, stream);
    case kDtypeBFloat16:
      return launch_ext_t<__nv_bfloat16, true>(logits, rows, vocab, row_stride, inv_t, topp, topk, settings, edits,
                                               n_edits, rng_states, out_ids, scratch, blocks, table, status, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

bool guided_supported(int dtype) { return dtype == kDtypeBFloat16 || dtype == kDtypeHalf; }

cudaError_t launch_sample_rows_guided(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t,
    float topp, int topk, unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers,
    void* scratch, int blocks, const ExpTable& table, int* status, int* retry_rows, int* retry_count,
    int* retry_count_next, cudaStream_t stream) {
  switch (dtype) {
    case kDtypeHalf:
      return launch_guided_t<__half, false>(logits, rows, vocab, row_stride, inv_t, topp, topk, rng_states,
                                            out_ids, peers, scratch, blocks, table, status, retry_rows,
                                            retry_count, retry_count_next, stream);
    case kDtypeBFloat16:
      return launch_guided_t<__nv_bfloat16, true>(logits, rows, vocab, row_stride, inv_t, topp, topk,
                                                  rng_states, out_ids, peers, scratch, blocks, table, status,
                                                  retry_rows, retry_count, retry_count_next, stream);
    default:
      return cudaErrorInvalidValue;
  }
}

int guided_kernel_max_blocks_per_sm(int dtype) {
  int n = 0;
  cudaError_t e;
  if (dtype == kDtypeHalf) {
    e = prepare_sample_kernel<__half, false, true>();
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sample_rows_kernel<__half, false, true>, kThreads,
                                                        sizeof(Shared<false, true>));
  } else {
    e = prepare_sample_kernel<__nv_bfloat16, true, true>();
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sample_rows_kernel<__nv_bfloat16, true, true>,
                                                        kThreads, sizeof(Shared<true, true>));
  }
  if (e != cudaSuccess || n < 1) n = 1;
  return n;
}

bool topp_cluster_supported(int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride,
                            float inv_t, float topp, int topk) {
  if (dtype != kDtypeBFloat16 || !(inv_t > 0.0f) || topk > 0) return false;
  if (!(topp > 0.0f && topp < 1.0f)) return false;
  if (vocab < kClusterMinVocab || vocab > kCMaxCluster * kCSliceMax) return false;
  if (rows < 1 || rows > (int64_t)0x7fffffff) return false;
  // every row must start on a 16-byte boundary (bulk copies)
  if ((reinterpret_cast<uintptr_t>(logits) & 15u) != 0) return false;
  if (rows > 1 && ((row_stride * 2) & 15) != 0) return false;
  return true;
}

// Blocks per row: as few as hold the row. (Twice as many for a single row was measured and is no
// quicker: the cluster kernel's chain of barriers does not get shorter, and the finishing kernel
// gets twice the slices to join.)
static int cluster_size_for(int vocab) {
  int csize = 1;
  while (csize * kCSliceMax < vocab) csize *= 2;
  return csize;
}

size_t topp_cluster_scratch_bytes(int vocab, int64_t batch_rows) {
  return (size_t)batch_rows * (size_t)cluster_size_for(vocab) * sizeof(SliceScratch);
}

cudaError_t launch_topp_cluster(
    const void* logits, int64_t rows, int vocab, int64_t row_stride, float inv_t, float topp,
    unsigned long long* rng_states, int64_t* out_ids, const PeerOut& peers, const ExpTable& table,
    void* scratch, int64_t batch_rows, int* retry_rows, int* retry_count, int* retry_count_next,
    cudaStream_t stream) {
  const int csize = cluster_size_for(vocab);
  const int slice_len = ((vocab + csize * kCTerms - 1) / (csize * kCTerms)) * kCTerms;
  static OncePerDevice once_a, once_b, once_np;
  cudaError_t e = func_attr_once(once_a, reinterpret_cast<const void*>(topp_cluster_kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ClusterShared));
  if (e != cudaSuccess) return e;
  e = func_attr_once(once_b, reinterpret_cast<const void*>(topp_finish_kernel),
                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FinishShared));
  if (e != cudaSuccess) return e;
  if (csize > 8) {
    e = func_attr_once(once_np, reinterpret_cast<const void*>(topp_cluster_kernel),
                       cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return e;
  }
  const unsigned short* base = static_cast<const unsigned short*>(logits);
  for (int64_t row0 = 0; row0 < rows; row0 += batch_rows) {
    const int64_t n = rows - row0 < batch_rows ? rows - row0 : batch_rows;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n * csize), 1, 1);
    cfg.blockDim = dim3(kCThreads, 1, 1);
    cfg.dynamicSmemBytes = sizeof(ClusterShared);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, topp_cluster_kernel, base + row0 * row_stride, vocab, row_stride, slice_len,
                           inv_t, topp, table, static_cast<SliceScratch*>(scratch));
    if (e != cudaSuccess) return e;
    // the finishing kernel may become resident while the cluster kernel runs (it waits for it)
    cudaLaunchConfig_t fcfg = {};
    fcfg.gridDim = dim3((unsigned)n, 1, 1);
    fcfg.blockDim = dim3(kFThreads, 1, 1);
    fcfg.dynamicSmemBytes = sizeof(FinishShared);
    fcfg.stream = stream;
    cudaLaunchAttribute fattr[1];
    programmatic_launch(&fattr[0]);
    fcfg.attrs = fattr;
    fcfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&fcfg, topp_finish_kernel, static_cast<const SliceScratch*>(scratch), row0, rows, vocab,
                           csize, topp, rng_states, out_ids, peers, retry_rows, retry_count,
                           row0 == 0 ? retry_count_next : static_cast<int*>(nullptr));
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

#if defined(ETB200_PHASE_CLOCKS)
extern "C" __attribute__((visibility("default"))) int etb200_debug_phase_clocks(long long* out16) {
  return (int)cudaMemcpyFromSymbol(out16, g_phase_clock, sizeof(long long) * 16);
}
extern "C" __attribute__((visibility("default"))) int etb200_debug_phase_clocks_reset() {
  const long long zero[16] = {0};
  return (int)cudaMemcpyToSymbol(g_phase_clock, zero, sizeof(zero));
}
#endif

cudaError_t launch_argmax_rows(
    int dtype, const void* logits, int64_t rows, int vocab, int64_t row_stride, int64_t* out_ids,
    const PeerOut& peers, int blocks, int* status, cudaStream_t stream) {
  switch (dtype) {
    case kDtypeFloat:
      argmax_rows_kernel<float, false><<<blocks, kThreads, 0, stream>>>(
          static_cast<const float*>(logits), rows, vocab, row_stride, out_ids, peers, status);
      break;
    case kDtypeHalf:
      argmax_rows_kernel<__half, false><<<blocks, kThreads, 0, stream>>>(
          static_cast<const __half*>(logits), rows, vocab, row_stride, out_ids, peers, status);
      break;
    case kDtypeBFloat16:
      argmax_rows_kernel<__nv_bfloat16, false><<<blocks, kThreads, 0, stream>>>(
          static_cast<const __nv_bfloat16*>(logits), rows, vocab, row_stride, out_ids, peers, status);
      break;
    case kDtypeUInt16:
      argmax_rows_kernel<unsigned short, true><<<blocks, kThreads, 0, stream>>>(
          static_cast<const unsigned short*>(logits), rows, vocab, row_stride, out_ids, peers, status);
      break;
    default:
      return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

int sample_kernel_max_blocks_per_sm(int dtype) {
  int n = 0;
  cudaError_t e;
  switch (dtype) {
    case kDtypeFloat:
      e = prepare_sample_kernel<float, false>();
      if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sample_rows_kernel<float, false, false>, kThreads,
                                                          sizeof(Shared<false>));
      break;
    case kDtypeHalf:
      e = prepare_sample_kernel<__half, false>();
      if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sample_rows_kernel<__half, false, false>, kThreads,
                                                          sizeof(Shared<false>));
      break;
    default:
      e = prepare_sample_kernel<__nv_bfloat16, true>();
      if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, sample_rows_kernel<__nv_bfloat16, true, false>,
                                                          kThreads, sizeof(Shared<true>));
      break;
  }
  if (e != cudaSuccess || n < 1) n = 1;
  return n;
}

}  // namespace etb200
