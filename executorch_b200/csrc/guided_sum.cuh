// The exact sequential softmax denominator (sampler.cpp:199-203) of one 16-bit row by ONE
// thread block, without the block-wide rounds of seqsum_tile: the arithmetic of
// cluster_math.cuh (estimate-guided integer increments per chunk of 32 terms, a short replay
// over the few event chunks) applied inside sample_rows_kernel<..., kGuided = true>.
// Included by sampler_kernels.cu inside its unnamed namespace (uses its helpers).
//
// The row streams through shared memory twice, 16 384 logits (one chunk per thread) at a time,
// by bulk asynchronous copies (cp.async.bulk, completion on an mbarrier): the copy of the next
// tile is issued as soon as every thread holds the current one in registers.
//   sweep 1: approximate exponentials (ex2.approx) summed per chunk; a block scan per tile
//            gives every chunk an estimate of the running sum in front of and behind it, i.e.
//            the binade(s) the exact running sum can be in there;
//   sweep 2: the exact terms (table lookups), the candidates of top-p / top-k (appended to
//            list A in index order, as the rest of the kernel expects), the integer increments
//            for the open binade(s); event chunks leave a record (and, where they may have to
//            be added term by term, their terms) in shared memory;
//   replay:  one thread walks the event records (walk_events) and returns the exact sum.
// Returns false when the replay could not decide (a list overflowed, or an assumption about
// the estimate did not hold): the caller hands the row to the kernel without this pass.

#if defined(ETB200_PHASE_CLOCKS)
// Debug build only: clock64 stamps of block 0 / row 0, one per phase boundary.
__device__ long long g_phase_clock[16];
#define ETB_STAMP(k)                                                        \
  do {                                                                      \
    if (blockIdx.x == 0 && threadIdx.x == 0) g_phase_clock[k] = clock64();  \
  } while (0)
// time spent between the two macros, and event counts, accumulated into slot k
#define ETB_CLOCK_BEGIN() const long long etb_clock_t0 = clock64()
#define ETB_CLOCK_ADD(k)                                                                      \
  do {                                                                                        \
    if (blockIdx.x == 0 && threadIdx.x == 0) g_phase_clock[k] += clock64() - etb_clock_t0;   \
  } while (0)
// the GPU's global timer (nanoseconds), comparable between kernels and SMs
#define ETB_GSTAMP(k)                                                                   \
  do {                                                                                  \
    if (blockIdx.x == 0 && threadIdx.x == 0) {                                          \
      unsigned long long etb_gt;                                                        \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(etb_gt));                        \
      g_phase_clock[k] = (long long)etb_gt;                                             \
    }                                                                                   \
  } while (0)
#define ETB_COUNT(k)                                                \
  do {                                                              \
    if (blockIdx.x == 0 && threadIdx.x == 0) g_phase_clock[k] += 1; \
  } while (0)
#else
#define ETB_STAMP(k)
#define ETB_CLOCK_BEGIN()
#define ETB_CLOCK_ADD(k)
#define ETB_GSTAMP(k)
#define ETB_COUNT(k)
#endif

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute
// may start while its predecessor in the stream still runs. It must wait here before it touches
// anything the predecessor writes (the wait ends when the predecessor's grid has completed and
// its writes are visible; without the attribute it returns at once). The predecessor lets its
// dependents become resident early with grid_launch_dependents().
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Bounded wait for a bulk copy. Returns false if it has not landed after about a second.
__device__ __forceinline__ bool wait_bulk_copy(unsigned long long* bar, uint32_t parity) {
  const uint32_t a = smem_addr(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Tie-free increments of eight terms in one binade (see chunk_increment_fast).
__device__ __forceinline__ void inc8(const float (&e)[8], float inv_u, float (&acc)[2], float& md) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float t = __fmaf_rn(e[j], inv_u, 8388608.0f);
    const float q = __fsub_rn(t, 8388608.0f);
    const float d = __fmaf_rn(e[j], inv_u, -q);
    acc[j & 1] = __fadd_rn(acc[j & 1], q);
    md = fmaxf(md, fabsf(d));
  }
}

// The eight terms of one 128-bit group of 16-bit logits.
template <typename T, typename S>
__device__ __forceinline__ void terms8(const RowMath<T, S>& rm, const S& sm, const uint4& raw, float (&e)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  if constexpr (S::kHasLut) {
    const char* lut_bytes = reinterpret_cast<const char*>(sm.lut);
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
        e[2 * j] = rm.from_pattern(w[j] & 0xFFFFu, sm);
        e[2 * j + 1] = rm.from_pattern(w[j] >> 16, sm);
      }
    }
  } else {
    const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = rm.direct(to_f32(p[j]), sm);
  }
}

// fp32 value of a 16-bit logit pattern, for the approximate sweep.
template <typename T>
__device__ __forceinline__ float half_to_f32(uint32_t h) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return __uint_as_float(h << 16);
  } else {
    return __half2float(__ushort_as_half((unsigned short)h));
  }
}

template <typename T>
__device__ __forceinline__ unsigned short neg_inf_bits() {
  return std::is_same<T, __nv_bfloat16>::value ? (unsigned short)0xFF80u : (unsigned short)0xFC00u;
}

// The replay of walk_events() by one warp: the lanes take 32 consecutive event records at a
// time, a warp scan applies every record in front of the first one that needs more than an
// integer addition (a chunk that leaves the binade, one that has no summary for the current
// binade, one whose increment depends on parity), and that one is then handled by all lanes in
// step, exactly as walk_events() handles it. One slice (`n_ev` records, the last one kEvTail).
// Same result as walk_events(): the exact sum, or false.
__device__ bool walk_events_warp(const ChunkEvent* ev, int n_ev, const float (*pool)[kCTerms], int pool_cap,
                                 float* sum) {
  const int lane = threadIdx.x & 31;
  int k = 1, n = 0;   // the running sum as (binade, significand); warp-uniform
  int run_k = -1;     // binade of the ordinary chunks behind the last record that was applied
  unsigned long long x_prev = 0ull;
  int pos = 0;
  while (pos < n_ev) {
    const int i = pos + lane;
    const bool valid = i < n_ev;
    ChunkEvent r = ev[valid ? i : n_ev - 1];
    unsigned long long xb_prev = __shfl_up_sync(0xffffffffu, r.xbefore, 1);
    int klo_prev = __shfl_up_sync(0xffffffffu, (int)r.klo, 1);
    if (lane == 0) {
      xb_prev = x_prev;
      klo_prev = run_k;
    }
    const unsigned long long gap = r.xbefore - xb_prev;
    const bool tail = (r.flags & kEvTail) != 0u, zero = (r.flags & kEvZero) != 0u;
    int a0 = 0;
    bool have = false;
    if ((r.flags & kEvLo) && k == r.klo) {
      have = r.a0lo == r.a1lo;
      a0 = r.a0lo;
    } else if ((r.flags & kEvHi) && k == r.klo + 1) {
      have = r.a0hi == r.a1hi;
      a0 = r.a0hi;
    }
    // a record is simple when an integer addition applies it in the current binade
    const bool simple = valid && gap < (unsigned long long)kSeqLimit && (gap == 0ull || klo_prev == k) &&
                        (tail || zero || have);
    const unsigned inc = simple ? (unsigned)gap + ((tail || zero) ? 0u : (unsigned)a0) : 0u;  // < 2^26
    unsigned incl = inc;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    const bool stop = !simple || (unsigned)n + incl >= (unsigned)kSeqLimit;  // invalid lanes stop too
    const unsigned sb = __ballot_sync(0xffffffffu, stop);
    const int f = sb != 0u ? __ffs(sb) - 1 : 32;  // records in front of lane f are applied
    if (f > 0) {
      n += (int)__shfl_sync(0xffffffffu, incl, f - 1);
      x_prev = __shfl_sync(0xffffffffu, r.xbefore, f - 1);
      // the binade of the following run: that of the last record applied (a closing record has none)
      const int kl = __shfl_sync(0xffffffffu, (int)r.klo, f - 1);
      const unsigned fl = __shfl_sync(0xffffffffu, (unsigned)r.flags, f - 1);
      if ((fl & kEvTail) == 0u) run_k = kl;
      pos += f;
    }
    // the record at pos, if any, needs the long way; so do wild records right behind it
    while (pos < n_ev) {
      const ChunkEvent q = ev[pos];
      const unsigned long long g2 = q.xbefore - x_prev;
      if (g2 != 0ull) {
        if (run_k != k || g2 >= (unsigned long long)kSeqLimit) return false;
        n += (int)g2;
        if (n >= kSeqLimit) return false;
      }
      x_prev = q.xbefore;
      ++pos;
      if (q.flags & kEvTail) break;
      run_k = q.klo;
      if (q.flags & kEvZero) break;
      SeqSummary sm2;
      bool have2 = false;
      if ((q.flags & kEvLo) && k == q.klo) {
        sm2.a0 = q.a0lo;
        sm2.a1 = q.a1lo;
        have2 = true;
      } else if ((q.flags & kEvHi) && k == q.klo + 1) {
        sm2.a0 = q.a0hi;
        sm2.a1 = q.a1hi;
        have2 = true;
      }
      if (have2) {
        const int n2 = seq_apply(n, sm2);
        if (n2 < kSeqLimit) {
          n = n2;
          break;
        }
      }
      // the chunk leaves the binade (or has no summary for it): real float additions
      if (q.pool < 0 || q.pool >= pool_cap) return false;
      const float4* t4 = reinterpret_cast<const float4*>(pool[q.pool]);
      float s = seq_value(k, n);
#pragma unroll
      for (int j = 0; j < kCTerms / 4; ++j) {
        const float4 t = t4[j];
        s = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, t.x), t.y), t.z), t.w);
      }
      if (!(s < 3.0e38f)) return false;
      k = seq_kb(s);
      n = seq_n(s);
      // the start of a row is a run of such chunks: take the next one directly
      if (pos < n_ev && ev[pos].flags == 0u && ev[pos].xbefore == x_prev) continue;
      break;
    }
  }
  *sum = seq_value(k, n);
  return true;
}

template <typename T, typename S>
__device__ bool guided_sum_pass(S& sm, const RowMath<T, S>& rm, uint32_t& copy_parity, bool use_list,
                                float e_floor, Entry* listA, int* n_a_out, float* sum_out) {
  GuidedShared& g = sm.g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int vocab = rm.vocab;
  const int n_chunks = (vocab + kCTerms - 1) / kCTerms;
  const int n_tiles = (vocab + kGTile - 1) / kGTile;
  const unsigned short* row16 = reinterpret_cast<const unsigned short*>(rm.row);
  unsigned short* tile = reinterpret_cast<unsigned short*>(sm.u.stage);
  // the chunks' open binades: tiles 0..7 in g.kb, tiles 8..15 behind the tile buffer (the union
  // member is 40 KB, the tile 32 KB)
  unsigned short* kb_hi = tile + kGTile;
  static_assert(sizeof(sm.u.stage) >= (size_t)kGTile * 2 + (size_t)(kGMaxTiles - 8) * kThreads * 2,
                "the union buffer must hold a tile and the upper half of the binade table");
  const int sw = (tid >> 1) & 3;  // register group q holds the chunk's logits (q ^ sw) * 8 ...
  const float inv_t = rm.inv_t, mx = rm.mx;
  bool copies_ok = true;

  // Copy of tile r into the buffer: thread 0 issues the bulk copy of its whole 16-byte units;
  // all threads fill the ragged end and the padding of the last tile (-inf: e = 0). Called
  // right behind a barrier after which nobody reads the buffer's previous contents.
  auto start_tile = [&](int r) {
    const int left = vocab - r * kGTile;
    const int len = left < kGTile ? left : kGTile;
    const int len16 = len & ~7;
    if (tid == 0) {
      if (len16 > 0) {
        const uint32_t bytes = (uint32_t)len16 * 2u;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&g.mbar)),
                     "r"(bytes)
                     : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                smem_addr(tile)),
            "l"(row16 + (size_t)r * kGTile), "r"(bytes), "r"(smem_addr(&g.mbar))
            : "memory");
      } else {
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(&g.mbar)) : "memory");
      }
    }
    if (len < kGTile) {
      const int padded = ((len + kCTerms - 1) / kCTerms) * kCTerms;
      for (int i = len16 + tid; i < padded; i += kThreads) {
        tile[i] = i < len ? row16[(size_t)r * kGTile + i] : neg_inf_bits<T>();
      }
    }
  };
  // Waits for tile r and loads this thread's chunk of it (four 128-bit reads, rotated per
  // thread pair so that a warp's reads fall into distinct banks).
  auto take_tile = [&](int r, uint4 (&raw)[4], bool& active) {
#if defined(ETB200_PHASE_CLOCKS)
    const long long w0 = clock64();
#endif
    if (!wait_bulk_copy(&g.mbar, copy_parity)) copies_ok = false;
#if defined(ETB200_PHASE_CLOCKS)
    if (blockIdx.x == 0 && tid == 0) g_phase_clock[10] += clock64() - w0;
#endif
    copy_parity ^= 1u;
    if (vocab - r * kGTile < kGTile) __syncthreads();  // the ragged end was written by other threads
    active = r * kThreads + tid < n_chunks;
    const uint4* mine4 = reinterpret_cast<const uint4*>(tile) + tid * 4;
    const uint32_t ni = (uint32_t)neg_inf_bits<T>() * 0x10001u;
#pragma unroll
    for (int q = 0; q < 4; ++q) raw[q] = active ? mine4[q ^ sw] : make_uint4(ni, ni, ni, ni);
  };

  __syncthreads();  // the buffer (a union member) is free
  ETB_STAMP(2);
  start_tile(0);

  // ---- sweep 1: approximate sums, the binades each chunk can meet
  {
    const float c1 = inv_t * 1.4426950408889634f;
    const float c2 = -mx * 1.4426950408889634f;
    double base = 0.0;  // estimate of the sum in front of the tile (block-uniform)
    for (int r = 0; r < n_tiles; ++r) {
      uint4 raw[4];
      bool active;
      take_tile(r, raw, active);
      float est = 0.0f;
      if (active) {
        float a4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t w[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            a4[j] += ex2_approx(fmaf(half_to_f32<T>(w[j] & 0xFFFFu), c1, c2));
            a4[j] += ex2_approx(fmaf(half_to_f32<T>(w[j] >> 16), c1, c2));
          }
        }
        est = (a4[0] + a4[1]) + (a4[2] + a4[3]);
      }
      float incl = est;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const float o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      if (lane == 31) g.wtot[r & 1][warp] = (double)incl;
      __syncthreads();  // every thread holds its chunk of tile r; the warp totals are visible
      start_tile(r + 1 < n_tiles ? r + 1 : 0);  // behind the last tile: tile 0 again, for sweep 2
      double warp_pre = 0.0, tile_tot = 0.0;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const double t = g.wtot[r & 1][w];
        if (w < warp) warp_pre += t;
        tile_tot += t;
      }
      if (active) {
        const float p_out = (float)(base + warp_pre + (double)incl);
        const float p_in = (float)(base + warp_pre + (double)(incl - est));
        int klo, khi;
        chunk_binades(p_in, p_out, binade_margin((long long)(r * kThreads + tid + 1) * kCTerms), &klo, &khi);
        const int span = khi - klo < 3 ? khi - klo : 3;
        (r < 8 ? g.kb[r] : kb_hi + (r - 8) * kThreads)[tid] = (unsigned short)(klo | (span << 8));
      }
      base += tile_tot;
    }
  }

  ETB_STAMP(3);
  // ---- sweep 2: exact terms, candidates, integer increments, event records
  unsigned long long x_run = 0ull;  // increments of the ordinary chunks so far (block-uniform)
  int ev_n = 0, st_n = 0, n_a = 0;  // events, staged chunks, candidates so far (block-uniform)
  bool fits = true;
  // Candidates: e >= e_floor. e is monotone in the logit, so a group of eight can only hold one
  // if its largest logit reaches a (generously low) bound; the exact test is on e.
  const float x_bound = (__logf(e_floor) + mx) / inv_t;
  const float x_low = use_list ? x_bound - 0.03f * fabsf(x_bound) - 0.0625f : INFINITY;
  for (int r = 0; r < n_tiles; ++r) {
    uint4 raw[4];
    bool active;
    take_tile(r, raw, active);
    int klo = 1, khi = 1;
    if (active) {
      const unsigned kbv = (r < 8 ? g.kb[r] : kb_hi + (r - 8) * kThreads)[tid];
      klo = (int)(kbv & 0xFFu);
      khi = klo + (int)(kbv >> 8);
    }
    const bool can_sum = active && chunk_summarisable(klo, khi);
    const bool two = can_sum && khi != klo;
    // the second binade is summed by the whole warp whenever one of its chunks needs it
    const bool warp_two = __any_sync(0xffffffffu, two);
    int inc_lo = 0, inc_hi = 0;
    unsigned flags = 0u, cmask = 0u;
    if (active) {
      const float inv_lo = seq_inv_u(can_sum ? klo : 127), inv_hi = seq_inv_u(can_sum ? khi : 127);
      float acc_lo[2] = {0.0f, 0.0f}, acc_hi[2] = {0.0f, 0.0f};
      float md_lo = 0.0f, md_hi = 0.0f, top = -INFINITY;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float e[8];
        terms8(rm, sm, raw[q], e);
        using T2 = decltype(neg_inf2(T()));
        const T2* p = reinterpret_cast<const T2*>(&raw[q]);
        const T2 gm2 = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
        const float gm = fmaxf(to_f32(gm2.x), to_f32(gm2.y));
        top = fmaxf(top, gm);
        if (gm >= x_low) {
#pragma unroll
          for (int j = 0; j < 8; ++j) cmask |= (e[j] >= e_floor ? 1u : 0u) << (q * 8 + j);
        }
        inc8(e, inv_lo, acc_lo, md_lo);  // sums of integers: the order does not matter
        if (warp_two) inc8(e, inv_hi, acc_hi, md_hi);
      }
      // a chunk whose largest logit already gives e = 0 holds nothing but zeros
      if (__fsub_rn(__fmul_rn(top, inv_t), mx) < -0x1.9fe368p6f) {
        flags = kEvLo | kEvHi | kEvZero;
      } else {
        const float tlo = acc_lo[0] + acc_lo[1], thi = acc_hi[0] + acc_hi[1];
        inc_lo = (int)(tlo < 33554432.0f ? tlo : 33554432.0f);
        inc_hi = two ? (int)(thi < 33554432.0f ? thi : 33554432.0f) : 0;
        // a chunk with an exact half-way term is staged; its summary is formed after the sweep
        flags = chunk_flags(klo, khi, !(md_lo < 0.5f), two && !(md_hi < 0.5f));
      }
    }
    const bool staged = active && chunk_is_staged(flags);
    int prev_klo = __shfl_up_sync(0xffffffffu, klo, 1);
    if (lane == 31) g.wklo[r & 1][warp] = klo;
    __syncthreads();  // every thread holds its chunk of tile r; the warps' last binades are visible
    if (r + 1 < n_tiles) start_tile(r + 1);
    // a chunk whose binade differs from its predecessor's is an event; so is the row's first
    if (lane == 0) prev_klo = warp > 0 ? g.wklo[r & 1][warp - 1] : (r > 0 ? g.wklo[(r + 1) & 1][kWarps - 1] : -1);
    const bool event = active && (klo != prev_klo || staged);
    const unsigned inc_mine = (active && !event) ? (unsigned)inc_lo : 0u;  // < 2^24 for a valid run
    unsigned inc_incl = inc_mine;
    int cnd_incl = __popc(cmask);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned o = __shfl_up_sync(0xffffffffu, inc_incl, d);
      const int oc = __shfl_up_sync(0xffffffffu, cnd_incl, d);
      if (lane >= d) {
        inc_incl += o;
        cnd_incl += oc;
      }
    }
    const unsigned evb = __ballot_sync(0xffffffffu, event);
    const unsigned stb = __ballot_sync(0xffffffffu, staged);
    if (lane == 31) {
      g.wx[r & 1][warp] = (unsigned long long)inc_incl;
      g.wev[r & 1][warp] = __popc(evb);
      g.wst[r & 1][warp] = __popc(stb);
      g.wcand[r & 1][warp] = cnd_incl;
    }
    __syncthreads();
    unsigned long long x_pre = 0ull, x_tot = 0ull;
    int ev_pre = 0, ev_tot = 0, st_pre = 0, st_tot = 0, cn_pre = 0, cn_tot = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const unsigned long long xv = g.wx[r & 1][w];
      const int c = g.wev[r & 1][w], sc = g.wst[r & 1][w], cc = g.wcand[r & 1][w];
      if (w < warp) {
        x_pre += xv;
        ev_pre += c;
        st_pre += sc;
        cn_pre += cc;
      }
      x_tot += xv;
      ev_tot += c;
      st_tot += sc;
      cn_tot += cc;
    }
    if (ev_n + ev_tot + 1 > kGEventCap) fits = false;  // block-uniform
    if (fits && event) {
      int slot = -1;
      if (staged) {
        slot = st_n + st_pre + __popc(stb & ((1u << lane) - 1u));
        if (slot < kGPoolCap) {
          float4* dst = reinterpret_cast<float4*>(g.pool[slot]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float e[8];
            terms8(rm, sm, raw[q], e);
            dst[(q ^ sw) * 2] = make_float4(e[0], e[1], e[2], e[3]);
            dst[(q ^ sw) * 2 + 1] = make_float4(e[4], e[5], e[6], e[7]);
          }
        } else {
          slot = -1;  // no room: the replay gives up if it needs these terms
        }
      }
      ChunkEvent rec;
      rec.a0lo = rec.a1lo = inc_lo;
      rec.a0hi = rec.a1hi = inc_hi;
      rec.xbefore = x_run + x_pre + (unsigned long long)(inc_incl - inc_mine);
      rec.klo = (short)klo;
      rec.pool = (short)slot;
      rec.flags = (unsigned short)flags;
      rec.pad = 0;
      g.events[ev_n + ev_pre + __popc(evb & ((1u << lane) - 1u))] = rec;
    }
    if (cmask != 0u) {
      // candidates go to list A in index order: the chunks of a tile follow the threads, and
      // inside a chunk the register groups are visited in row order
      int off = n_a + cn_pre + cnd_incl - __popc(cmask);
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int q = b ^ sw;  // the register group that holds the chunk's logits b * 8 ...
        unsigned m = 0u;
#pragma unroll
        for (int qq = 0; qq < 4; ++qq) m = qq == q ? (cmask >> (qq * 8)) & 0xFFu : m;
        if (m != 0u) {
          uint4 rq = raw[0];
#pragma unroll
          for (int qq = 1; qq < 4; ++qq) rq = qq == q ? raw[qq] : rq;
          float e[8];
          terms8(rm, sm, rq, e);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (m & (1u << j)) {
              Entry en;
              en.key = f32_bits(e[j]);
              en.idx = (r * kThreads + tid) * kCTerms + b * 8 + j;
              listA[off++] = en;
            }
          }
        }
      }
    }
    x_run += x_tot;
    ev_n += ev_tot;
    st_n += st_tot;
    n_a += cn_tot;
  }
  if (tid == 0) {
    if (fits) {
      ChunkEvent rec;
      rec.a0lo = rec.a1lo = rec.a0hi = rec.a1hi = 0;
      rec.xbefore = x_run;
      rec.klo = 0;
      rec.pool = -1;
      rec.flags = (unsigned short)kEvTail;
      rec.pad = 0;
      g.events[ev_n] = rec;
    }
    g.ev_first[0] = 0;
    g.ev_count[0] = ev_n + 1;
  }
  __threadfence_block();
  __syncthreads();
  ETB_STAMP(4);
  // ---- pending two-parity summaries: one thread per event, side by side
  if (fits && tid < ev_n) {
    ChunkEvent* e = &g.events[tid];
    if ((e->flags & (kEvTieLo | kEvTieHi)) != 0u && e->pool >= 0) resolve_tie_event(e, g.pool[e->pool]);
  }
  __syncthreads();
  // ---- replay, by one warp
  if (warp == 0) {
    float s = 0.0f;
    bool ok = fits && copies_ok;
    if (ok) ok = walk_events_warp(g.events, ev_n + 1, g.pool, kGPoolCap, &s);
    if (lane == 0) {
      g.sum = s;
      g.ok = ok ? 1 : 0;
    }
  }
  __syncthreads();
  ETB_STAMP(5);
  *n_a_out = n_a;
  *sum_out = g.sum;
  return g.ok != 0;
}
