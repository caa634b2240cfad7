// Top-p sampling of bf16 rows with one thread-block CLUSTER per row (sm_100a).
// Included by sampler_kernels.cu inside its unnamed namespace (uses its helpers).
//
// Why a cluster: a 128 256-entry bf16 row is 250 KB -- it does not fit the shared memory of
// one SM, and one block walking it tile by tile is bound by the latency of its per-tile
// rounds. Here the row is cut into slices of up to 16 384 logits, one per block of the
// cluster (8 blocks for V = 128 256, 16 for V = 256 000); every thread owns ONE chunk of 32
// consecutive logits, so the whole row is in registers at once and every phase is a single
// parallel sweep:
//
//   0. each block pulls its slice into shared memory with one bulk asynchronous copy
//      (cp.async.bulk, completion on an mbarrier) -- the row's only trip from HBM;
//   1. row maximum: packed bf16 max per thread, block reduction, exchange of the block maxima
//      through distributed shared memory (every block writes its value into every block);
//   2. the table  bit pattern -> e = expf(x / T - max)  is built ONCE per row: each block
//      evaluates 8192 / cluster_size entries and stores them into all blocks' tables;
//   3. every thread looks up its 32 terms, sums them (inexactly) and lists the few large
//      ones in the leader block's candidate list; a block scan plus an exchange of block
//      totals gives every chunk an estimate of the running sum in front of it;
//   4. every chunk is turned into integer increments for the binade(s) that estimate allows
//      (cluster_math.cuh); the few "event" chunks send a 32-byte record to the leader;
//   5. the leader block (rank 0) replays the exact sequential sum from the records (one warp),
//      then finishes sample_topp on the candidate list in its shared memory.
//
// The other blocks of the cluster are done after phase 4 and leave. Nothing here waits on a
// flag: the only waits are hardware cluster barriers and the mbarrier of the bulk copy (whose
// wait is bounded). A row that this kernel cannot decide (the walk met an assumption that did
// not hold, or a list overflowed) is appended to `retry_rows` and left untouched; the caller
// runs those rows through sample_rows_kernel afterwards.
//
// No multicast loads are used anywhere: each block copies its own slice.

namespace cg = cooperative_groups;

constexpr int kCThreads = 512;
constexpr int kCWarps = kCThreads / 32;
constexpr int kCSliceMax = kCThreads * kCTerms;  // logits per block
constexpr int kCMaxCluster = 16;
constexpr int kCEventCap = 512;   // event records per row (all slices together)
constexpr int kCCandCap = 1024;   // candidate entries per row

// The leader's work arrays for the end of sample_topp; they reuse the slice's memory, which
// is no longer read by then.
struct ClusterTail {
  unsigned long long ck[kCCandCap];
  alignas(16) float p[kCCandCap + 8];
  int idx[kCCandCap];
  alignas(16) float prefix[kCCandCap + 4];
};

struct __align__(128) ClusterShared {
  union {
    unsigned short slice[kCSliceMax];  // this block's logits (bf16 bit patterns), row order
    ClusterTail tail;
  };
  float lut[kLutSize];               // bit pattern -> e, identical in every block of the cluster
  uint64_t exp_tab[kExpTableSize];
  unsigned long long mbar;           // completion barrier of the bulk copy
  // written by the peers through distributed shared memory
  float cmax[kCMaxCluster];          // block maxima
  double ctot[kCMaxCluster];         // block totals of the estimate
  // block-level reductions and scans
  float redf[kCWarps];
  double wtot[kCWarps];
  unsigned long long wx[kCWarps];
  int wev[kCWarps];
  int wklo[kCWarps];
  int ev_base;
  // leader only (rank 0); the peers write into the leader's copy
  int ev_total;
  int cand_count;
  int give_up;
  int ev_first[kCMaxCluster];
  int ev_count[kCMaxCluster];
  ChunkEvent events[kCEventCap];
  Entry cand[kCCandCap];
  // the leader's tail
  float sum;
  float coin;
  int sum_ok;
  int n_kept;
  int last;
  float cum;
  int first_above;
};
static_assert(sizeof(ClusterTail) <= kCSliceMax * sizeof(unsigned short), "the tail arrays must fit the slice");

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Bounded wait for the bulk copy (phase 0). Returns false if the copy has not landed after
// about a second; the row is then handed to the other kernel.
__device__ __forceinline__ bool wait_bulk_copy(unsigned long long* bar) {
  const uint32_t a = smem_addr(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(0u)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// e for one bf16 bit pattern: table where covered, direct evaluation otherwise.
__device__ __forceinline__ float cluster_term(const ClusterShared& sm, uint32_t h, float inv_t, float mx) {
  const uint32_t hb = h + kLutBias;
  if ((hb & 0x7000u) == 0x4000u) return sm.lut[(hb & 0x0FFFu) | ((hb >> 3) & 0x1000u)];
  return expf_ref(__fsub_rn(__fmul_rn(bits_f32(h << 16), inv_t), mx), sm.exp_tab);
}

// Terms of one chunk for the leader's walk: every lane of the walking warp fetches one term
// (from the leader's own slice, or from the row in global memory for the other slices) and
// the terms are handed out by shuffles. All lanes run the walk in lockstep.
struct LeaderTerms {
  const ClusterShared* sm;
  const unsigned short* row;
  int vocab;
  int slice_len;
  float inv_t;
  float mx;
  mutable float mine;
  __device__ __forceinline__ float operator()(int sl, int chunk, int j) const {
    if (j == 0) {
      const int lane = threadIdx.x & 31;
      const int local = chunk * kCTerms + lane;
      const int i = sl * slice_len + local;
      uint32_t h = 0xFF80u;  // -inf beyond the row
      if (sl == 0) {
        h = sm->slice[local];
      } else if (i < vocab) {
        h = __ldg(row + i);
      }
      mine = cluster_term(*sm, h, inv_t, mx);
    }
    return __shfl_sync(0xffffffffu, mine, j);
  }
};

__global__ void __launch_bounds__(kCThreads, 2) topp_cluster_kernel(
    const unsigned short* __restrict__ logits, int64_t rows, int vocab, int64_t row_stride,
    int slice_len, float inv_t, float topp, unsigned long long* __restrict__ rng_states,
    int64_t* __restrict__ out_ids, PeerOut peers, ExpTable table, int* __restrict__ retry_rows,
    int* __restrict__ retry_count, int* __restrict__ retry_count_next) {
  extern __shared__ __align__(128) unsigned char cluster_smem_raw[];
  ClusterShared& sm = *reinterpret_cast<ClusterShared*>(cluster_smem_raw);
  cg::cluster_group cluster = cg::this_cluster();
  const int csize = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t r = (int64_t)(blockIdx.x / csize);
  const unsigned short* row = logits + r * row_stride;
  ClusterShared* leader = cluster.map_shared_rank(&sm, 0);

  const int i0 = rank * slice_len;
  const int len = vocab - i0 < 0 ? 0 : (vocab - i0 < slice_len ? vocab - i0 : slice_len);
  const int n_chunks = (len + kCTerms - 1) / kCTerms;
  const int len16 = len & ~7;  // whole 16-byte units go by the bulk copy

  // ---- phase 0: the slice comes in; everything that does not need it meanwhile
  if (tid < kExpTableSize) sm.exp_tab[tid] = table.t[tid];
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(&sm.mbar)), "r"(1u));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (rank == 0) {
      sm.ev_total = 0;
      sm.cand_count = 0;
      sm.give_up = 0;
      // the counter the NEXT launch will use is cleared here (launches of a handle are ordered)
      if (blockIdx.x == 0) *retry_count_next = 0;
    }
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
  // the peers' shared memory must exist before anything is stored into it
  cluster.sync();
  bool copy_ok = true;
  if (len16 > 0) copy_ok = wait_bulk_copy(&sm.mbar);

  // ---- phase 1: this thread's chunk (four 128-bit reads, rotated per thread pair so that a
  // warp's reads fall into distinct banks) and the row maximum
  const bool active = tid < n_chunks;
  const int sw = (tid >> 1) & 3;
  uint4 raw[4];
  float gmax[4];  // maximum of each group of eight logits, for the candidate filter
  {
    const uint4* mine4 = reinterpret_cast<const uint4*>(sm.slice) + tid * 4;
    const __nv_bfloat162 ninf = neg_inf2(__nv_bfloat16());
    __nv_bfloat162 acc = ninf;
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
    if (tid < csize) {
      float b = sm.redf[0];
#pragma unroll
      for (int w = 1; w < kCWarps; ++w) b = fmaxf(b, sm.redf[w]);
      cluster.map_shared_rank(&sm, tid)->cmax[rank] = b;
    }
  }
  cluster.sync();
  float mx;
  {
    float b = sm.cmax[0];
    for (int c = 1; c < csize; ++c) b = fmaxf(b, sm.cmax[c]);
    mx = __fmul_rn(b, inv_t);  // x -> fl(x * inv_t) is monotone for inv_t > 0
  }

  // ---- phase 2: the table, built once per row by the whole cluster
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
  cluster.sync();

  // ---- phase 3: the 32 terms, their (inexact) sum, the candidates
  const float cutoff = __fdiv_rn(__fsub_rn(1.0f, topp), (float)(vocab - 1));
  const float e_floor = fmaxf(cutoff * 0.999999f, kGuessFloor);
  float e[kCTerms];
#pragma unroll
  for (int j = 0; j < kCTerms; ++j) e[j] = 0.0f;
  if (active) {
    const char* lut_bytes = reinterpret_cast<const char*>(sm.lut);
    uint32_t bad = 0u;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // both halves of the word at once (see RowMath::eval_raw)
        const uint32_t wb = w[j] + (kLutBias | (kLutBias << 16));
        bad |= wb ^ 0x40004000u;
        const uint32_t off0 = ((wb << 2) & 0x3FFCu) | ((wb >> 1) & 0x4000u);
        const uint32_t off1 = ((wb >> 14) & 0x3FFCu) | ((wb >> 17) & 0x4000u);
        e[q * 8 + 2 * j] = *reinterpret_cast<const float*>(lut_bytes + off0);
        e[q * 8 + 2 * j + 1] = *reinterpret_cast<const float*>(lut_bytes + off1);
      }
    }
    if ((bad & 0x70007000u) != 0u) {
      // rare: a zero, tiny, huge or non-finite logit (or padding) in this chunk
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          e[q * 8 + 2 * j] = cluster_term(sm, w[j] & 0xFFFFu, inv_t, mx);
          e[q * 8 + 2 * j + 1] = cluster_term(sm, w[j] >> 16, inv_t, mx);
        }
      }
    }
  }
  float est;
  {
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = (e[j] + e[j + 8]) + (e[j + 16] + e[j + 24]);
    est = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
  }
  {
    // Candidates: e >= e_floor. e is monotone in the logit, so a group of eight can only hold
    // one if its largest logit reaches a (generously low) bound; the exact test is on e.
    const float x_bound = (__logf(e_floor) + mx) / inv_t;
    const float x_low = x_bound - 0.03f * fabsf(x_bound) - 0.0625f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (gmax[q] >= x_low) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (e[q * 8 + j] >= e_floor) {
            const int slot = atomicAdd(&leader->cand_count, 1);
            if (slot < kCCandCap) {
              Entry en;
              en.key = f32_bits(e[q * 8 + j]);
              en.idx = i0 + tid * kCTerms + ((q ^ sw) << 3) + j;
              leader->cand[slot] = en;
            }
          }
        }
      }
    }
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
  double warp_pre = 0.0, block_tot = 0.0;
#pragma unroll
  for (int w = 0; w < kCWarps; ++w) {
    const double t = sm.wtot[w];
    if (w < warp) warp_pre += t;
    block_tot += t;
  }
  if (tid < csize) cluster.map_shared_rank(&sm, tid)->ctot[rank] = block_tot;
  cluster.sync();
  double row_pre = 0.0;
  for (int c = 0; c < rank; ++c) row_pre += sm.ctot[c];
  const float p_out = (float)(row_pre + warp_pre + (double)est_incl);
  const float p_in = (float)(row_pre + warp_pre + (double)(est_incl - est));

  // ---- phase 4: integer increments for the open binade(s); event records to the leader
  int klo = 1, khi = 1;
  SeqSummary slo, shi;
  seq_identity(&slo);
  seq_identity(&shi);
  unsigned flags = 0u;
  bool tie = false;
  if (active) {
    chunk_binades(p_in, p_out, binade_margin((long long)i0 + (long long)(tid + 1) * kCTerms), &klo, &khi);
    if (est == 0.0f) {
      flags = kEvLo | kEvHi | kEvZero;  // nothing but zeros: changes no sum
    } else {
      if (chunk_summarisable(klo, khi)) {
        bool half;
        const int inc = chunk_increment_fast(e, klo, &half);  // a sum of integers: any order
        slo.a0 = slo.a1 = inc;
        bool half_hi = false;
        if (khi != klo) {
          const int inc_hi = chunk_increment_fast(e, khi, &half_hi);
          shi.a0 = shi.a1 = inc_hi;
          flags = kEvLo | kEvHi;
        } else {
          flags = kEvLo;
        }
        if (half || half_hi) {
          // rare: an exact half-way term; the two-parity summary needs the terms in row order
          float ord[kCTerms];
#pragma unroll
          for (int j = 0; j < kCTerms; ++j) ord[(((j >> 3) ^ sw) << 3) | (j & 7)] = e[j];
          if (half) {
            slo = chunk_summary_exact(ord, klo);
            tie = tie || slo.a0 != slo.a1;
          }
          if (half_hi) {
            shi = chunk_summary_exact(ord, khi);
            tie = tie || shi.a0 != shi.a1;
          }
        }
      }
    }
  }
  const bool zero = (flags & kEvZero) != 0u;
  const bool wild = active && flags == 0u;
  const bool unsafe = active && !zero && (flags & kEvHi) != 0u;
  // a chunk whose binade differs from its predecessor's is an event; so is the first of a slice
  int prev_klo = __shfl_up_sync(0xffffffffu, klo, 1);
  if (lane == 31) sm.wklo[warp] = klo;
  __syncthreads();
  if (lane == 0) prev_klo = warp > 0 ? sm.wklo[warp - 1] : -1;
  const bool event = active && (tid == 0 || klo != prev_klo || wild || unsafe || tie);
  // exclusive scans over the block: increments of the ordinary chunks, and event slots
  const unsigned inc_mine = (active && !event) ? (unsigned)slo.a0 : 0u;  // < 2^24 for a valid run
  unsigned inc_incl = inc_mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned o = __shfl_up_sync(0xffffffffu, inc_incl, d);
    if (lane >= d) inc_incl += o;
  }
  const unsigned evb = __ballot_sync(0xffffffffu, event);
  if (lane == 31) {
    sm.wx[warp] = (unsigned long long)inc_incl;
    sm.wev[warp] = __popc(evb);
  }
  __syncthreads();
  unsigned long long x_pre = 0ull, x_tot = 0ull;
  int ev_pre = 0, ev_tot = 0;
#pragma unroll
  for (int w = 0; w < kCWarps; ++w) {
    const unsigned long long xv = sm.wx[w];
    const int c = sm.wev[w];
    if (w < warp) {
      x_pre += xv;
      ev_pre += c;
    }
    x_tot += xv;
    ev_tot += c;
  }
  if (tid == 0) {
    // one slot range per slice in the leader's list (plus the record that closes the slice)
    const int base = atomicAdd(&leader->ev_total, ev_tot + 1);
    const bool fits = base + ev_tot + 1 <= kCEventCap;
    leader->ev_first[rank] = fits ? base : 0;
    leader->ev_count[rank] = fits ? ev_tot + 1 : 0;
    if (!fits || !copy_ok) leader->give_up = 1;
    sm.ev_base = fits ? base : -1;
  }
  __syncthreads();
  const int ev_base = sm.ev_base;
  if (ev_base >= 0) {
    if (event) {
      ChunkEvent rec;
      rec.a0lo = slo.a0;
      rec.a1lo = slo.a1;
      rec.a0hi = shi.a0;
      rec.a1hi = shi.a1;
      rec.xbefore = x_pre + (unsigned long long)(inc_incl - inc_mine);
      rec.klo = (short)klo;
      rec.chunk = (short)tid;
      rec.flags = (unsigned short)flags;
      rec.pad = 0;
      leader->events[ev_base + ev_pre + __popc(evb & ((1u << lane) - 1u))] = rec;
    }
    if (tid == 0) {
      ChunkEvent rec;
      rec.a0lo = rec.a1lo = rec.a0hi = rec.a1hi = 0;
      rec.xbefore = x_tot;
      rec.klo = 0;
      rec.chunk = 0;
      rec.flags = (unsigned short)kEvTail;
      rec.pad = 0;
      leader->events[ev_base + ev_tot] = rec;
    }
  }
  cluster.sync();
  if (rank != 0) return;

  // ---- phase 5 (leader): the exact sequential sum, replayed by one warp
  if (warp == 0) {
    LeaderTerms terms;
    terms.sm = &sm;
    terms.row = row;
    terms.vocab = vocab;
    terms.slice_len = slice_len;
    terms.inv_t = inv_t;
    terms.mx = mx;
    terms.mine = 0.0f;
    float s = 0.0f;
    bool ok = sm.give_up == 0 && sm.cand_count <= kCCandCap;
    if (ok) ok = walk_events(sm.events, sm.ev_first, sm.ev_count, csize, kCEventCap, terms, &s);
    if (lane == 0) {
      sm.sum = s;
      sm.sum_ok = ok ? 1 : 0;
      sm.n_kept = 0;
      sm.first_above = 0x7fffffff;
      unsigned long long st = rng_states[r];
      sm.coin = next_coin(&st);  // the state is stored only when the row is decided
    }
  }
  __syncthreads();
  bool decided = sm.sum_ok != 0;
  const float sum = sm.sum;
  const float coin = sm.coin;

  // ---- phase 6 (leader): sample_topp (sampler.cpp:122-171) on the candidate list
  int token = 0;
  if (decided) {
    const int n_c = sm.cand_count;
    // crop (sampler.cpp:136-143) and sort key: probability descending, index ascending
    for (int i = tid; i < n_c; i += kCThreads) {
      const Entry en = sm.cand[i];
      const float p = __fdiv_rn(bits_f32(en.key), sum);
      if (p >= cutoff) {
        const int slot = atomicAdd(&sm.n_kept, 1);
        sm.tail.ck[slot] = ((unsigned long long)f32_bits(p) << 32) | (uint32_t)(0x7FFFFFFF - en.idx);
      }
    }
    __syncthreads();
    const int n_b = sm.n_kept;
    if (n_b > 0) {
      for (int i = tid; i < n_b; i += kCThreads) {
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
      for (int i0b = 0; i0b <= last; i0b += kCThreads) {
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
