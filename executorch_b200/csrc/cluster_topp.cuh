// Top-p sampling of bf16 rows with one thread-block CLUSTER per row (sm_100a), in two kernels.
// Included by sampler_kernels.cu inside its unnamed namespace (uses its helpers).
//
// Why a cluster: a 128 256-entry bf16 row is 250 KB -- it does not fit the shared memory of
// one SM, and one block walking it tile by tile is bound by the latency of its per-tile
// rounds. Here the row is cut into slices of up to 16 384 logits, one per block of the
// cluster (8 blocks for V = 128 256, 16 for V = 256 000); every thread owns ONE chunk of 32
// consecutive logits, so the whole row is on chip at once and every phase is a single
// parallel sweep.
//
// topp_cluster_kernel (one cluster per row, every block does the same):
//   0. each block pulls its slice into shared memory with one bulk asynchronous copy
//      (cp.async.bulk, completion on an mbarrier) -- the row's only trip from HBM;
//   1. row maximum: packed bf16 max per thread, block reduction, exchange of the block maxima
//      through distributed shared memory (every block writes its value into every block);
//   2. two things that only need the maximum, side by side: the table  bit pattern ->
//      e = expf(x / T - max)  is built ONCE per row (each block evaluates 8192 / cluster_size
//      entries and stores them into all blocks' tables), and every thread sums approximate
//      exponentials (ex2.approx) of its 32 logits; a block scan plus the exchange of the
//      block totals -- the same cluster barrier as the table's -- gives every chunk an
//      estimate of the running sum in front of it;
//   3. every thread looks up its 32 exact terms, lists the few large ones, and turns the
//      chunk into integer increments for the binade(s) the estimate allows (cluster_math.cuh);
//      the few "event" chunks write a 32-byte record (and, where the replay may have to add
//      them one by one, their 32 terms) to the row's scratch area in global memory.
// topp_finish_kernel (one small block per row): replays the exact sequential sum from the
//   records (cluster_math.cuh: walk_events) and finishes sample_topp on the listed candidates.
//   Splitting it off keeps every block of the first kernel short-lived and alike, and lets
//   the sequential part of all rows run side by side.
//
// Nothing here waits on a flag: the only waits are hardware cluster barriers and the
// mbarrier of the bulk copy (whose wait is bounded). A row that cannot be decided this way
// (the replay met an assumption that did not hold, or a list overflowed) is appended to
// `retry_rows` and left untouched; the caller runs those rows through sample_rows_kernel.
//
// No multicast loads are used anywhere: each block copies its own slice.

namespace cg = cooperative_groups;

constexpr int kCThreads = 512;
constexpr int kCWarps = kCThreads / 32;
constexpr int kCSliceMax = kCThreads * kCTerms;  // logits per block
constexpr int kCMaxCluster = 16;
// per slice, in the row's scratch area
constexpr int kCSliceEvents = 96;   // event records (the last one closes the slice)
constexpr int kCSliceCand = 192;    // candidate entries
// per row, in the finishing kernel's shared memory
constexpr int kFThreads = 256;
constexpr int kFEventCap = 448;
constexpr int kFPoolCap = 192;
constexpr int kFCandCap = 1024;
constexpr int kFSerialWalk = 256;   // lists up to this many records are replayed record by record

struct __align__(16) SliceHeader {
  int n_events;  // records written, including the closing one; 0 = the slice gave up
  int n_cand;
  int n_staged;  // staged chunks: their terms are terms[0 .. n_staged), in event order
  int pad;
  unsigned long long x_total;  // the closing record's xbefore: increments of the slice's ordinary chunks
  unsigned long long pad2;
};

// Scratch of one slice in global memory. A staged event's record holds the row of `terms` with
// its 32 terms in `pool`.
struct SliceScratch {
  SliceHeader hdr;
  ChunkEvent events[kCSliceEvents];
  Entry cand[kCSliceCand];
  float terms[kCSliceEvents][kCTerms];
};

struct __align__(128) ClusterShared {
  unsigned short slice[kCSliceMax];  // this block's logits (bf16 bit patterns), row order
  float lut[kLutSize];               // bit pattern -> e, identical in every block of the cluster
  uint64_t exp_tab[kExpTableSize];
  unsigned long long mbar;  // completion barrier of the bulk copy
  // written by the peers through distributed shared memory
  float cmax[kCMaxCluster];   // block maxima
  double ctot[kCMaxCluster];  // block totals of the estimate
  // block-level reductions and scans
  float redf[kCWarps];
  double wtot[kCWarps];
  unsigned long long wx[kCWarps];
  int wev[kCWarps];
  int wst[kCWarps];
  int wklo[kCWarps];
  int lcand_count;
  Entry lcand[kCSliceCand];  // this slice's candidates, before they go to global memory
};

// The hardware barrier of the cluster, split so that work can sit between arrival and wait.
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// e for one bf16 bit pattern: table where covered, direct evaluation otherwise.
__device__ __forceinline__ float cluster_term(const ClusterShared& sm, uint32_t h, float inv_t, float mx) {
  const uint32_t hb = h + kLutBias;
  if ((hb & 0x7000u) == 0x4000u) return sm.lut[(hb & 0x0FFFu) | ((hb >> 3) & 0x1000u)];
  return expf_ref(__fsub_rn(__fmul_rn(bits_f32(h << 16), inv_t), mx), sm.exp_tab);
}

// The eight terms of one 128-bit group of logits.
__device__ __forceinline__ void cluster_terms8(const ClusterShared& sm, const uint4& raw, float inv_t, float mx,
                                               float (&e)[8]) {
  const char* lut_bytes = reinterpret_cast<const char*>(sm.lut);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  uint32_t bad = 0u;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // both halves of the word at once (see RowMath::eval_raw)
    const uint32_t wb = w[j] + (kLutBias | (kLutBias << 16));
    bad |= wb ^ 0x40004000u;
    const uint32_t off0 = ((wb << 2) & 0x3FFCu) | ((wb >> 1) & 0x4000u);
    const uint32_t off1 = ((wb >> 14) & 0x3FFCu) | ((wb >> 17) & 0x4000u);
    e[2 * j] = *reinterpret_cast<const float*>(lut_bytes + off0);
    e[2 * j + 1] = *reinterpret_cast<const float*>(lut_bytes + off1);
  }
  if ((bad & 0x70007000u) != 0u) {
    // rare: a zero, tiny, huge or non-finite logit (or padding) in this group
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[2 * j] = cluster_term(sm, w[j] & 0xFFFFu, inv_t, mx);
      e[2 * j + 1] = cluster_term(sm, w[j] >> 16, inv_t, mx);
    }
  }
}

__global__ void __launch_bounds__(kCThreads, 2) topp_cluster_kernel(
    const unsigned short* __restrict__ logits, int vocab, int64_t row_stride, int slice_len, float inv_t,
    float topp, ExpTable table, SliceScratch* __restrict__ scratch) {
  extern __shared__ __align__(128) unsigned char cluster_smem_raw[];
  ClusterShared& sm = *reinterpret_cast<ClusterShared*>(cluster_smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t r = (int64_t)(blockIdx.x / csize);  // row inside this launch
  const unsigned short* row = logits + r * row_stride;
  SliceScratch& out = scratch[r * csize + rank];

  const int i0 = rank * slice_len;
  const int len = vocab - i0 < 0 ? 0 : (vocab - i0 < slice_len ? vocab - i0 : slice_len);
  const int n_chunks = (len + kCTerms - 1) / kCTerms;
  const int len16 = len & ~7;  // whole 16-byte units go by the bulk copy

  ETB_STAMP(0);
  ETB_GSTAMP(13);
  grid_launch_dependents();  // the finishing kernel may take its place; it waits for this grid
  // ---- phase 0: the slice comes in; everything that does not need it meanwhile
  if (tid < kExpTableSize) sm.exp_tab[tid] = table.t[tid];
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&sm.mbar)), "r"(1u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    sm.lcand_count = 0;
  }
  // the ragged end of the slice and the padding up to a whole chunk (-inf: e = 0)
  for (int i = len16 + tid; i < n_chunks * kCTerms; i += kCThreads) {
    sm.slice[i] = i < len ? row[i0 + i] : (unsigned short)0xFF80u;
  }
  __syncthreads();
  if (tid == 0 && len16 > 0) {
    const uint32_t bytes = (uint32_t)len16 * 2u;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&sm.mbar)), "r"(bytes)
                 : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_addr(sm.slice)),
        "l"(row + i0), "r"(bytes), "r"(smem_addr(&sm.mbar))
        : "memory");
  }
  // barrier 0 ("every block of the cluster is running"): its latency hides behind the copy
  cluster_arrive();
  bool copy_ok = true;
  if (len16 > 0) copy_ok = wait_bulk_copy(&sm.mbar, 0u);

  ETB_STAMP(1);
  // ---- phase 1: this thread's chunk (four 128-bit reads, rotated per thread pair so that a
  // warp's reads fall into distinct banks) and the row maximum
  const bool active = tid < n_chunks;
  const int sw = (tid >> 1) & 3;  // register group q holds the chunk's logits (q ^ sw) * 8 ...
  uint4 raw[4];
  float gmax[4];  // maximum of each group of eight logits, for the candidate filter
  {
    const uint4* mine4 = reinterpret_cast<const uint4*>(sm.slice) + tid * 4;
    __nv_bfloat162 acc = neg_inf2(__nv_bfloat16());
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      raw[q] = active ? mine4[q ^ sw] : make_uint4(0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u, 0xFF80FF80u);
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
      const __nv_bfloat162 g = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
      gmax[q] = fmaxf(__bfloat162float(g.x), __bfloat162float(g.y));
      acc = __hmax2(acc, g);
    }
    float m = fmaxf(__bfloat162float(acc.x), __bfloat162float(acc.y));
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
    if (lane == 0) sm.redf[warp] = m;
    __syncthreads();
    cluster_wait();  // barrier 0: the peers' shared memory may be written from here on
    if (tid < csize) {
      float b = sm.redf[0];
#pragma unroll
      for (int w = 1; w < kCWarps; ++w) b = fmaxf(b, sm.redf[w]);
      cluster.map_shared_rank(&sm, tid)->cmax[rank] = b;
    }
  }
  cluster_arrive();
  cluster_wait();  // barrier 1: the block maxima are everywhere
  float mx;
  {
    float b = sm.cmax[0];
    for (int c = 1; c < csize; ++c) b = fmaxf(b, sm.cmax[c]);
    mx = __fmul_rn(b, inv_t);  // x -> fl(x * inv_t) is monotone for inv_t > 0
  }

  ETB_STAMP(2);
  // ---- phase 2: this block's share of the table (stored into every block), and the estimate
  {
    const int per_block = kLutSize / csize;
    for (int k = tid; k < per_block; k += kCThreads) {
      const int slot = rank * per_block + k;
      const uint32_t hb = 0x4000u | ((uint32_t)slot & 0x0FFFu);
      const uint32_t pat = ((hb - kLutBias) & 0x7FFFu) | (((uint32_t)slot & 0x1000u) << 3);
      const float e = expf_ref(__fsub_rn(__fmul_rn(bits_f32(pat << 16), inv_t), mx), sm.exp_tab);
      for (int c = 0; c < csize; ++c) cluster.map_shared_rank(&sm, c)->lut[slot] = e;
    }
  }
  float est = 0.0f;
  if (active) {
    // sum of 2^((x * inv_t - mx) * log2 e) with the hardware's approximate exponential: good to
    // about 1e-6, which is all the binade guess needs (binade_margin allows for it)
    const float c1 = inv_t * 1.4426950408889634f;
    const float c2 = -mx * 1.4426950408889634f;
    float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a4[j] += ex2_approx(fmaf(__uint_as_float(w[j] << 16), c1, c2));
        a4[j] += ex2_approx(fmaf(__uint_as_float(w[j] & 0xFFFF0000u), c1, c2));
      }
    }
    est = (a4[0] + a4[1]) + (a4[2] + a4[3]);
  }
  // block scan of the estimates (float inside a warp, double across warps and blocks)
  float est_incl = est;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, est_incl, d);
    if (lane >= d) est_incl += o;
  }
  if (lane == 31) sm.wtot[warp] = (double)est_incl;
  __syncthreads();
  float p_in, p_out;
  {
    double warp_pre = 0.0, block_tot = 0.0;
#pragma unroll
    for (int w = 0; w < kCWarps; ++w) {
      const double t = sm.wtot[w];
      if (w < warp) warp_pre += t;
      block_tot += t;
    }
    if (tid < csize) cluster.map_shared_rank(&sm, tid)->ctot[rank] = block_tot;
    cluster_arrive();
    cluster_wait();  // barrier 2: the table and the block totals are everywhere
    double row_pre = 0.0;
    for (int c = 0; c < rank; ++c) row_pre += sm.ctot[c];
    p_out = (float)(row_pre + warp_pre + (double)est_incl);
    p_in = (float)(row_pre + warp_pre + (double)(est_incl - est));
  }

  ETB_STAMP(3);
  // ---- phase 3: the exact terms, eight at a time: candidates and integer increments
  const float cutoff = __fdiv_rn(__fsub_rn(1.0f, topp), (float)(vocab - 1));
  const float e_floor = fmaxf(cutoff * 0.999999f, kGuessFloor);
  int klo = 1, khi = 1;
  int inc_lo = 0, inc_hi = 0;
  unsigned flags = 0u;
  if (active) chunk_binades(p_in, p_out, binade_margin((long long)i0 + (long long)(tid + 1) * kCTerms), &klo, &khi);
  const bool can_sum = active && chunk_summarisable(klo, khi);
  const bool two = can_sum && khi != klo;
  // the second binade is summed by the whole warp whenever one of its chunks needs it
  const bool warp_two = __any_sync(0xffffffffu, two);
  if (active) {
    // Candidates: e >= e_floor. e is monotone in the logit, so a group of eight can only hold
    // one if its largest logit reaches a (generously low) bound; the exact test is on e.
    const float x_bound = (__logf(e_floor) + mx) / inv_t;
    const float x_low = x_bound - 0.03f * fabsf(x_bound) - 0.0625f;
    const float inv_lo = seq_inv_u(can_sum ? klo : 127), inv_hi = seq_inv_u(can_sum ? khi : 127);
    float acc_lo[2] = {0.0f, 0.0f}, acc_hi[2] = {0.0f, 0.0f};
    float md_lo = 0.0f, md_hi = 0.0f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float e[8];
      cluster_terms8(sm, raw[q], inv_t, mx, e);
      if (gmax[q] >= x_low) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (e[j] >= e_floor) {
            const int slot = atomicAdd(&sm.lcand_count, 1);
            if (slot < kCSliceCand) {
              Entry en;
              en.key = f32_bits(e[j]);
              en.idx = i0 + tid * kCTerms + ((q ^ sw) << 3) + j;
              sm.lcand[slot] = en;
            }
          }
        }
      }
      inc8(e, inv_lo, acc_lo, md_lo);  // sums of integers: the order does not matter
      if (warp_two) inc8(e, inv_hi, acc_hi, md_hi);
    }
    // a chunk whose largest logit already gives e = 0 holds nothing but zeros
    const float top = fmaxf(fmaxf(gmax[0], gmax[1]), fmaxf(gmax[2], gmax[3]));
    if (__fsub_rn(__fmul_rn(top, inv_t), mx) < -0x1.9fe368p6f) {
      flags = kEvLo | kEvHi | kEvZero;
    } else {
      const float tlo = acc_lo[0] + acc_lo[1], thi = acc_hi[0] + acc_hi[1];
      inc_lo = (int)(tlo < 33554432.0f ? tlo : 33554432.0f);
      inc_hi = two ? (int)(thi < 33554432.0f ? thi : 33554432.0f) : 0;
      // a chunk with an exact half-way term is staged; the finishing kernel forms its summary
      flags = chunk_flags(klo, khi, !(md_lo < 0.5f), two && !(md_hi < 0.5f));
    }
  }
  ETB_STAMP(4);
  const bool staged = active && chunk_is_staged(flags);
  // a chunk whose binade differs from its predecessor's is an event; so is the first of a slice
  int prev_klo = __shfl_up_sync(0xffffffffu, klo, 1);
  if (lane == 31) sm.wklo[warp] = klo;
  __syncthreads();  // also: every candidate of this slice is in sm.lcand
  if (lane == 0) prev_klo = warp > 0 ? sm.wklo[warp - 1] : -1;
  const bool event = active && (tid == 0 || klo != prev_klo || staged);
  // exclusive scans over the block: increments of the ordinary chunks, and event slots
  const unsigned inc_mine = (active && !event) ? (unsigned)inc_lo : 0u;  // < 2^24 for a valid run
  unsigned inc_incl = inc_mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned o = __shfl_up_sync(0xffffffffu, inc_incl, d);
    if (lane >= d) inc_incl += o;
  }
  const unsigned evb = __ballot_sync(0xffffffffu, event);
  const unsigned stb = __ballot_sync(0xffffffffu, event && staged);
  if (lane == 31) {
    sm.wx[warp] = (unsigned long long)inc_incl;
    sm.wev[warp] = __popc(evb);
    sm.wst[warp] = __popc(stb);
  }
  __syncthreads();
  unsigned long long x_pre = 0ull, x_tot = 0ull;
  int ev_pre = 0, ev_tot = 0, st_pre = 0, st_tot = 0;
#pragma unroll
  for (int w = 0; w < kCWarps; ++w) {
    const unsigned long long xv = sm.wx[w];
    const int c = sm.wev[w];
    const int sc = sm.wst[w];
    if (w < warp) {
      x_pre += xv;
      ev_pre += c;
      st_pre += sc;
    }
    x_tot += xv;
    ev_tot += c;
    st_tot += sc;
  }
  const int n_lc = sm.lcand_count;
  const bool fits = ev_tot + 1 <= kCSliceEvents && n_lc <= kCSliceCand && copy_ok;
  if (tid == 0) {
    SliceHeader h;
    h.n_events = fits ? ev_tot + 1 : 0;
    h.n_cand = fits ? n_lc : 0;
    h.n_staged = fits ? st_tot : 0;
    h.pad = 0;
    h.x_total = x_tot;
    h.pad2 = 0ull;
    out.hdr = h;
  }
  if (fits) {
    if (event) {
      const int slot = ev_pre + __popc(evb & ((1u << lane) - 1u));
      const int st_slot = st_pre + __popc(stb & ((1u << lane) - 1u));
      if (staged) {
        float4* dst = reinterpret_cast<float4*>(out.terms[st_slot]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float e[8];
          cluster_terms8(sm, raw[q], inv_t, mx, e);
          dst[(q ^ sw) * 2] = make_float4(e[0], e[1], e[2], e[3]);
          dst[(q ^ sw) * 2 + 1] = make_float4(e[4], e[5], e[6], e[7]);
        }
      }
      ChunkEvent rec;
      rec.a0lo = rec.a1lo = inc_lo;
      rec.a0hi = rec.a1hi = inc_hi;
      rec.xbefore = x_pre + (unsigned long long)(inc_incl - inc_mine);
      rec.klo = (short)klo;
      rec.pool = (short)(staged ? st_slot : -1);
      rec.flags = (unsigned short)flags;
      rec.pad = 0;
      out.events[slot] = rec;
    }
    if (tid == 0) {
      ChunkEvent rec;
      rec.a0lo = rec.a1lo = rec.a0hi = rec.a1hi = 0;
      rec.xbefore = x_tot;
      rec.klo = 0;
      rec.pool = -1;
      rec.flags = (unsigned short)kEvTail;
      rec.pad = 0;
      out.events[ev_tot] = rec;
    }
    for (int i = tid; i < n_lc; i += kCThreads) out.cand[i] = sm.lcand[i];
  }
  ETB_STAMP(5);
}

// ---------------------------------------------------------------------------------------
// One block per row: gathers the row's records, replays the exact sum, finishes sample_topp.
// ---------------------------------------------------------------------------------------
struct FinishTail {
  unsigned long long ck[kFCandCap];
  alignas(16) float p[kFCandCap + 8];
  int idx[kFCandCap];
  alignas(16) float prefix[kFCandCap + 4];
};

struct __align__(16) FinishShared {
  union {
    struct {
      ChunkEvent events[kFEventCap];
      float pool[kFPoolCap][kCTerms];
    } w;              // the replay
    FinishTail tail;  // after it
  };
  Entry cand[kFCandCap];
  int ev_first[kCMaxCluster + 1];    // slot of each slice's first record; [csize] = all records
  int cand_first[kCMaxCluster + 1];
  int st_first[kCMaxCluster + 1];    // the same for staged chunks
  unsigned long long xbase[kCMaxCluster];  // increments of the ordinary chunks in front of each slice
  int ok;
  float sum;
  float coin;
  int n_kept;
  int last;
  float cum;
  int first_above;
};

__global__ void __launch_bounds__(kFThreads) topp_finish_kernel(
    const SliceScratch* __restrict__ scratch, int64_t row0, int64_t rows, int vocab, int csize, float topp,
    unsigned long long* __restrict__ rng_states, int64_t* __restrict__ out_ids, PeerOut peers,
    int* __restrict__ retry_rows, int* __restrict__ retry_count, int* __restrict__ retry_count_next) {
  extern __shared__ __align__(16) unsigned char finish_smem_raw[];
  FinishShared& sm = *reinterpret_cast<FinishShared*>(finish_smem_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t rl = blockIdx.x;    // row inside this launch
  const int64_t r = row0 + rl;      // row of the batch
  const SliceScratch* sl0 = scratch + rl * csize;
  // the counter the NEXT call will use is cleared here (calls of a handle are ordered)
  grid_launch_dependents();  // the pass over undecided rows may take its place
  grid_dependency_wait();    // the cluster kernel's records are complete and visible from here on
  ETB_GSTAMP(14);
  ETB_STAMP(6);
  if (blockIdx.x == 0 && tid == 0 && retry_count_next != nullptr) *retry_count_next = 0;

  // ---- the slices' headers, all at once: where each slice's records, candidates and staged
  // terms go, and the increments in front of each slice
  if (warp == 0) {
    SliceHeader h;
    h.n_events = h.n_cand = h.n_staged = 0;
    h.x_total = 0ull;
    if (lane < csize) {
      const uint4* hp = reinterpret_cast<const uint4*>(&sl0[lane].hdr);
      const uint4 a = __ldg(hp), b = __ldg(hp + 1);
      h.n_events = (int)a.x;
      h.n_cand = (int)a.y;
      h.n_staged = (int)a.z;
      h.x_total = (unsigned long long)b.x | ((unsigned long long)b.y << 32);
    }
    const bool bad = lane < csize && (h.n_events < 1 || h.n_events > kCSliceEvents || h.n_cand < 0 ||
                                      h.n_cand > kCSliceCand || h.n_staged < 0 || h.n_staged > h.n_events);
    bool ok = !__any_sync(0xffffffffu, bad);
    int e = h.n_events, c = h.n_cand, st = h.n_staged;
    unsigned long long x = h.x_total;
#pragma unroll
    for (int d = 1; d < kCMaxCluster; d <<= 1) {
      const int oe = __shfl_up_sync(0xffffffffu, e, d), oc = __shfl_up_sync(0xffffffffu, c, d);
      const int os = __shfl_up_sync(0xffffffffu, st, d);
      const unsigned long long ox = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) {
        e += oe;
        c += oc;
        st += os;
        x += ox;
      }
    }
    // inclusive sums -> the slot behind each slice; slot 0 is 0
    if (lane < csize) {
      sm.ev_first[lane + 1] = e;
      sm.cand_first[lane + 1] = c;
      sm.st_first[lane + 1] = st;
      sm.xbase[lane] = x - h.x_total;
    }
    if (lane == csize - 1 && (e > kFEventCap || c > kFCandCap)) ok = false;
    ok = !__any_sync(0xffffffffu, !ok);
    if (lane == 0) {
      sm.ev_first[0] = sm.cand_first[0] = sm.st_first[0] = 0;
      sm.ok = ok ? 1 : 0;
      sm.n_kept = 0;
      sm.first_above = 0x7fffffff;
      unsigned long long rs = rng_states[r];
      sm.coin = next_coin(&rs);  // the state is stored only when the row is decided
    }
  }
  __syncthreads();
  bool decided = sm.ok != 0;
  int n_c = 0;
  if (decided) {
    // ---- records, candidates and the staged terms into shared memory, every load in flight at
    // once. A record's `xbefore` runs on over the slices (a slice's closing record carries the
    // increments of its trailing run, so every closing record but the last becomes an empty
    // record of the run it closes); its `pool` becomes the row-wide slot of its staged terms.
    const int n_ev = sm.ev_first[csize];
    n_c = sm.cand_first[csize];
    const int n_st = sm.st_first[csize] < kFPoolCap ? sm.st_first[csize] : kFPoolCap;
    auto slice_of = [&](const int* first, int i) {
      int sl = 0;
      while (sl + 1 < csize && i >= first[sl + 1]) ++sl;
      return sl;
    };
    for (int i = tid; i < n_ev; i += kFThreads) {
      const int sl = slice_of(sm.ev_first, i);
      const uint4* src = reinterpret_cast<const uint4*>(&sl0[sl].events[i - sm.ev_first[sl]]);
      union {
        uint4 q[2];
        ChunkEvent ev;
      } u;
      u.q[0] = __ldg(src);
      u.q[1] = __ldg(src + 1);
      u.ev.xbefore += sm.xbase[sl];
      if (u.ev.pool >= 0) {
        const int slot = sm.st_first[sl] + (int)u.ev.pool;
        u.ev.pool = (short)(slot < kFPoolCap ? slot : -1);  // no room: the replay gives up if it needs them
      }
      sm.w.events[i] = u.ev;
    }
    for (int i = tid; i < n_c; i += kFThreads) {
      const int sl = slice_of(sm.cand_first, i);
      sm.cand[i] = sl0[sl].cand[i - sm.cand_first[sl]];
    }
    for (int q = tid; q < n_st * 8; q += kFThreads) {
      const int k = q >> 3;
      const int sl = slice_of(sm.st_first, k);
      const float4* src = reinterpret_cast<const float4*>(sl0[sl].terms[k - sm.st_first[sl]]);
      reinterpret_cast<float4*>(sm.w.pool[k])[q & 7] = __ldg(src + (q & 7));
    }
    __syncthreads();
    ETB_STAMP(7);
    // ---- pending two-parity summaries: one thread per event, side by side
    for (int i = tid; i < n_ev; i += kFThreads) {
      ChunkEvent* e = &sm.w.events[i];
      if ((e->flags & (kEvTieLo | kEvTieHi)) != 0u && e->pool >= 0) resolve_tie_event(e, sm.w.pool[e->pool]);
    }
    __syncthreads();
    // ---- the exact sequential sum, replayed by one warp
    if (warp == 0) {
      float s = 0.0f;
      bool ok;
      if (n_ev <= kFSerialWalk) {
        // a short list (the usual case): record by record costs less than the scans of the warp
        // form, whose every stop at a chunk that needs real additions is a whole scan round
        const int first = 0;
        ok = walk_events(sm.w.events, &first, &n_ev, 1, kFEventCap,
                         [&](int slot, int j) { return sm.w.pool[slot][j]; }, &s);
      } else {
        ok = walk_events_warp(sm.w.events, n_ev, sm.w.pool, kFPoolCap, &s);
      }
      if (lane == 0) {
        sm.sum = s;
        sm.ok = ok ? 1 : 0;
      }
    }
    __syncthreads();
    decided = sm.ok != 0;
  }
  ETB_STAMP(8);
  const float sum = sm.sum;
  const float coin = sm.coin;
  const float cutoff = __fdiv_rn(__fsub_rn(1.0f, topp), (float)(vocab - 1));
  const float e_floor = fmaxf(cutoff * 0.999999f, kGuessFloor);

  // ---- sample_topp (sampler.cpp:122-171) on the candidate list
  int token = 0;
  if (decided) {
    // crop (sampler.cpp:136-143) and sort key: probability descending, index ascending
    for (int ib = 0; ib < n_c; ib += kFThreads) {
      const int i = ib + tid;
      bool keep = false;
      unsigned long long ck = 0ull;
      if (i < n_c) {
        const Entry en = sm.cand[i];
        const float p = __fdiv_rn(bits_f32(en.key), sum);
        keep = p >= cutoff;
        ck = ((unsigned long long)f32_bits(p) << 32) | (uint32_t)(0x7FFFFFFF - en.idx);
      }
      const unsigned bal = __ballot_sync(0xffffffffu, keep);
      if (bal != 0u) {
        int base = 0;
        if (lane == 0) base = atomicAdd(&sm.n_kept, __popc(bal));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (keep) sm.tail.ck[base + __popc(bal & ((1u << lane) - 1u))] = ck;
      }
    }
    __syncthreads();
    const int n_b = sm.n_kept;
    if (n_b > 0) {
      for (int i = tid; i < n_b; i += kFThreads) {
        const unsigned long long mine = sm.tail.ck[i];
        int rank_i = 0;
#pragma unroll 8
        for (int j = 0; j < n_b; ++j) rank_i += sm.tail.ck[j] > mine ? 1 : 0;
        sm.tail.p[rank_i] = bits_f32((uint32_t)(mine >> 32));
        sm.tail.idx[rank_i] = (int)(0x7FFFFFFFu - (uint32_t)(mine & 0xFFFFFFFFull));
      }
      if (tid < 8) sm.tail.p[n_b + tid] = 0.0f;  // written by nobody else: ranks are below n_b
    }
    __syncthreads();
    if (tid == 0) {
      // replay of the cumulative sum (sampler.cpp:151-159), keeping every partial sum: the draw
      // loop of sampler.cpp:162-169 adds the same numbers in the same order
      int last = -1;
      float acc = 0.0f;
      if (n_b > 0) {
        const float4* p4 = reinterpret_cast<const float4*>(sm.tail.p);
        float4* pre4 = reinterpret_cast<float4*>(sm.tail.prefix);
        float4 q = p4[0];
        for (int i = 0; i < n_b; i += 4) {
          const float4 nq = p4[(i >> 2) + 1];
          const float a1 = __fadd_rn(acc, q.x);
          const float a2 = __fadd_rn(a1, q.y);
          const float a3 = __fadd_rn(a2, q.z);
          const float a4 = __fadd_rn(a3, q.w);
          pre4[i >> 2] = make_float4(a1, a2, a3, a4);
          if (a4 > topp) {
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
        // the sum never exceeded topp: everything is kept (sampler.cpp:152), which is only
        // known to be everything when the list holds every entry that passes the crop
        const bool all_listed = e_floor <= cutoff * sum * 0.999999f;
        if (last < 0 && all_listed) last = n_b - 1;
      }
      sm.last = last;
      sm.cum = acc;
    }
    __syncthreads();
    const int last = sm.last;
    if (last < 0) {
      decided = false;
    } else {
      const float rr = __fmul_rn(coin, sm.cum);  // sampler.cpp:162
      for (int i0b = 0; i0b <= last; i0b += kFThreads) {
        const int i = i0b + tid;
        const bool above = i <= last && sm.tail.prefix[i] > rr;
        const unsigned bal = __ballot_sync(0xffffffffu, above);
        if (bal != 0u && lane == 0) atomicMin(&sm.first_above, (i & ~31) + __ffs(bal) - 1);
      }
      __syncthreads();
      const int fa = sm.first_above;
      token = sm.tail.idx[fa <= last ? fa : last];
    }
  }
  ETB_STAMP(9);
  if (decided) {
    store_token(out_ids, peers, r, token);
    if (tid == 0) {
      unsigned long long st = rng_states[r];
      next_coin(&st);
      rng_states[r] = st;
    }
  } else if (tid == 0) {
    retry_rows[atomicAdd(retry_count, 1)] = (int)r;
  }
}
