// Value-class tail of top-p sampling for 16-bit logits with a LONG nucleus (flat or very hot
// rows, where tens of thousands of tokens pass the cutoff crop of sampler.cpp:136-143).
//
// The probability of a token is a function of its logit's 16-bit pattern, and for a positive
// temperature it does not decrease with the logit. The reference's sorted candidate list
// (sampler.cpp:145, descending probability; equal probabilities by index) is therefore: value
// classes in descending key order, every class a run of `count` equal floats. Nothing is
// listed, compacted or sorted here:
//
//   1. count the row's patterns into a window of classes below the row maximum (shared-memory
//      histogram of kVcBins 32-bit counters; for a flat row, whose candidates span more classes,
//      2 * kVcBins 16-bit counters unless a class holds 65 536 or more logits; one read of the
//      row per window),
//   2. walk the classes, replaying `cumulative_prob += p` (sampler.cpp:151) over whole runs in
//      closed form (class_math.cuh) until the sum exceeds top-p; then again until it exceeds
//      r = coin * cumulative_prob (sampler.cpp:162-170). The result is a POSITION of the
//      sorted list and the probability found there,
//   3. classes whose float probabilities coincide form one group ordered by token index; one
//      more read of the row counts the tokens in front of the group and returns the member
//      of the wanted rank.
//
// Included by sampler_kernels.cu (inside its anonymous namespace), after RowMath.
#pragma once

template <typename T>
__device__ __forceinline__ float vc_logit_of_pattern(uint32_t pat) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return bits_f32(pat << 16);
  } else {
    return __half2float(__ushort_as_half((unsigned short)pat));
  }
}

// The window of class counts. The kernel variant with a table of exponentials lays it over the
// table and the union behind it (the tail evaluates its few classes directly; the next row
// rebuilds the table anyway); the other variant has a member for it.
template <typename S>
__device__ __forceinline__ unsigned* vc_hist(S& sm) {
  if constexpr (S::kHasLut) {
    static_assert(offsetof(S, u) == offsetof(S, lut) + sizeof(S::lut), "the union follows the table");
    static_assert(sizeof(S::lut) + sizeof(S::u) >= kVcBins * sizeof(unsigned), "window fits");
    return reinterpret_cast<unsigned*>(sm.lut);
  } else {
    return sm.u.vc.hist;
  }
}

// probability of the class with this key (rm.probs is off: rm yields e). Evaluated directly: the
// table's entries are these same values.
template <typename T, typename S>
__device__ __forceinline__ float vc_prob(const RowMath<T, S>& rm, const S& sm, uint32_t key, float sum) {
  const float e = rm.direct(vc_logit_of_pattern<T>(pattern_of_key16(key)), sm);
  return __fdiv_rn(e, sum);
}

// Eight consecutive patterns of the row starting at i0 (a multiple of 8), two per word.
// Positions beyond the row read as a NaN pattern, whose key lies above every real one.
template <typename T, typename S>
__device__ __forceinline__ void vc_load8(const RowMath<T, S>& rm, int i0, uint32_t (&w)[4]) {
  const unsigned short* row16 = reinterpret_cast<const unsigned short*>(rm.row);
  if (rm.vec_ok && i0 + 8 <= rm.vocab) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(row16 + i0));
    w[0] = raw.x;
    w[1] = raw.y;
    w[2] = raw.z;
    w[3] = raw.w;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = i0 + 2 * j < rm.vocab ? (uint32_t)row16[i0 + 2 * j] : 0x7FFFu;
      const uint32_t hi = i0 + 2 * j + 1 < rm.vocab ? (uint32_t)row16[i0 + 2 * j + 1] : 0x7FFFu;
      w[j] = lo | (hi << 16);
    }
  }
}

// Counts the row's patterns with keys in (win_hi - span, win_hi] into the window (vc_hist), slot
// win_hi - key: slot 0 is the window's largest value. With `pack16` the counters are 16 bits
// wide (two per word, span 2 * kVcBins): twice the classes per read of the row. A class of 65 536
// or more equal logits overflows such a counter; then the window's counters no longer add up to
// the number of logits counted, which is checked here, and the caller starts over with 32-bit
// counters. Returns false in that case (block-uniform).
template <typename T, typename S>
__device__ bool vc_histogram(S& sm, const RowMath<T, S>& rm, int win_hi, bool pack16) {
  const int tid = threadIdx.x;
  unsigned* hist = vc_hist(sm);
  __syncthreads();
  for (int i = tid; i < kVcBins / 4; i += kThreads) {
    reinterpret_cast<uint4*>(hist)[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  const uint32_t span = pack16 ? 2u * kVcBins : (uint32_t)kVcBins;
  const int nvec = (rm.vocab + 7) / 8;
  int added = 0;
  for (int q0 = tid; q0 < nvec; q0 += 4 * kThreads) {
    uint32_t w[4][4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int q = q0 + k * kThreads;
      if (q < nvec) {
        vc_load8(rm, q * 8, w[k]);
      } else {
        w[k][0] = w[k][1] = w[k][2] = w[k][3] = 0x7FFF7FFFu;
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t d0 = (uint32_t)win_hi - key_of_pattern16(w[k][j] & 0xFFFFu);
        const uint32_t d1 = (uint32_t)win_hi - key_of_pattern16(w[k][j] >> 16);
        if (pack16) {
          if (d0 < span) {
            atomicAdd(&hist[d0 >> 1], 1u << ((d0 & 1u) * 16u));
            ++added;
          }
          if (d1 < span) {
            atomicAdd(&hist[d1 >> 1], 1u << ((d1 & 1u) * 16u));
            ++added;
          }
        } else {
          if (d0 < span) atomicAdd(&hist[d0], 1u);
          if (d1 < span) atomicAdd(&hist[d1], 1u);
        }
      }
    }
  }
  __syncthreads();
  if (!pack16) return true;
  // every thread: the counters of its share of the window against what it added
  int diff = added;
  for (int i = tid; i < kVcBins / 4; i += kThreads) {
    const uint4 q = reinterpret_cast<const uint4*>(hist)[i];
    diff -= (int)((q.x & 0xFFFFu) + (q.x >> 16) + (q.y & 0xFFFFu) + (q.y >> 16) + (q.z & 0xFFFFu) + (q.z >> 16) +
                  (q.w & 0xFFFFu) + (q.w >> 16));
  }
  int total;
  block_excl_count(sm, diff, &total);
  return total == 0;
}

struct VcHit {
  bool overflow;  // a 16-bit class counter overflowed: nothing is decided, start over with 32-bit counters
  bool found;  // the running sum exceeded the threshold
  int pos;     // found: position (0-based) of the copy at which it did; else the number of candidates
  float p;     // found: the probability at that position
  float cum;   // the running sum there (found) or over all candidates
};

// One walk over the candidate classes, from the row maximum down, until the running float sum
// exceeds `thr` (strictly, as sampler.cpp:152 and :166 compare). The first walk of a row records
// the state at every window start; a later walk resumes from the last of those that is not
// beyond its threshold. Block-uniform result.
template <typename T, typename S>
__device__ VcHit vc_walk(S& sm, const RowMath<T, S>& rm, float sum, float cutoff, float thr, int key_max,
                         int key_min, bool first_walk, bool pack16) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  VcControl& vc = sm.vcc;
  const int span = pack16 ? 2 * kVcBins : kVcBins;  // classes per window
  int win_hi = key_max, kb = 1, n = 0, pos = 0;
  if (!first_walk) {
    const int nck = vc.n_ck;
    for (int i = 0; i < nck; ++i) {
      if (seq_value(vc.ck_kb[i], vc.ck_n[i]) <= thr) {
        win_hi = vc.ck_hi[i];
        kb = vc.ck_kb[i];
        n = vc.ck_n[i];
        pos = vc.ck_pos[i];
      }
    }
  }
  VcHit out;
  out.overflow = false;
  for (;;) {
    if (first_walk && tid == 0 && vc.n_ck < kVcCheckpoints) {
      const int i = vc.n_ck;
      vc.ck_hi[i] = win_hi;
      vc.ck_kb[i] = kb;
      vc.ck_n[i] = n;
      vc.ck_pos[i] = pos;
      vc.n_ck = i + 1;
    }
    if (pos >= rm.vocab) break;                                     // every token is consumed
    if (vc_prob(rm, sm, (uint32_t)win_hi, sum) < cutoff) break;     // nothing below is a candidate
    if (vc.loaded_hi != win_hi) {
      ETB_CLOCK_BEGIN();
      const bool counted = vc_histogram(sm, rm, win_hi, pack16);
      ETB_CLOCK_ADD(11);
      if (tid == 0) vc.loaded_hi = counted ? win_hi : -1;
      if (!counted) {
        out.overflow = true;
        out.found = false;
        out.pos = 0;
        out.p = 0.0f;
        out.cum = 0.0f;
        __syncthreads();
        return out;
      }
    }
    for (int t0 = 0; t0 < span; t0 += kVcTile) {
      const int b0 = t0 + tid * kVcPer;
      int c[kVcPer];
      if (pack16) {
        const uint2 cv = *reinterpret_cast<const uint2*>(reinterpret_cast<const unsigned short*>(vc_hist(sm)) + b0);
        c[0] = (int)(cv.x & 0xFFFFu);
        c[1] = (int)(cv.x >> 16);
        c[2] = (int)(cv.y & 0xFFFFu);
        c[3] = (int)(cv.y >> 16);
      } else {
        const uint4 cv = *reinterpret_cast<const uint4*>(&vc_hist(sm)[b0]);
        c[0] = (int)cv.x;
        c[1] = (int)cv.y;
        c[2] = (int)cv.z;
        c[3] = (int)cv.w;
      }
      float p[kVcPer];
      bool below = false;
      int low_key = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < kVcPer; ++j) {
        const int key = win_hi - (b0 + j);
        p[j] = 0.0f;
        if (key < key_min) c[j] = 0;
        if (c[j] > 0) {
          p[j] = vc_prob(rm, sm, (uint32_t)key, sum);
          if (p[j] < cutoff) {
            c[j] = 0;
            below = true;
          } else {
            low_key = key;
          }
        }
      }
      const int any = __syncthreads_or(c[0] | c[1] | c[2] | c[3]);
      if (below) vc.ended = 1;
      if (low_key != 0x7fffffff) atomicMin(&vc.last_key, (unsigned)low_key);
      while (any) {
        ETB_COUNT(12);
        // every thread: its classes' runs in the binade of the running sum
        SeqSummary s[kVcPer], mine;
        seq_identity(&mine);
        int cm = 0;
#pragma unroll
        for (int j = 0; j < kVcPer; ++j) {
          s[j] = rep_summary(p[j], c[j], kb);
          mine = seq_compose(mine, s[j]);
          cm += c[j];
        }
        SeqSummary inc = mine;
        int icnt = cm;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          SeqSummary o;
          o.a0 = __shfl_up_sync(0xffffffffu, inc.a0, d);
          o.a1 = __shfl_up_sync(0xffffffffu, inc.a1, d);
          const int oc = __shfl_up_sync(0xffffffffu, icnt, d);
          if (lane >= d) {
            inc = seq_compose(o, inc);
            icnt += oc;
          }
        }
        if (lane == 31) {
          vc.wsum[warp] = inc;
          vc.wcnt[warp] = icnt;
        }
        SeqSummary ex;  // the lanes in front of this one
        ex.a0 = __shfl_up_sync(0xffffffffu, inc.a0, 1);
        ex.a1 = __shfl_up_sync(0xffffffffu, inc.a1, 1);
        int ex_cnt = __shfl_up_sync(0xffffffffu, icnt, 1);
        if (lane == 0) {
          seq_identity(&ex);
          ex_cnt = 0;
        }
        __syncthreads();
        if (warp == 0) {
          // scan of the warps' totals: what lies in front of each warp, and the tile's total
          SeqSummary wi;
          seq_identity(&wi);
          int wic = 0;
          if (lane < kWarps) {
            wi = vc.wsum[lane];
            wic = vc.wcnt[lane];
          }
#pragma unroll
          for (int d = 1; d < kWarps; d <<= 1) {
            SeqSummary o;
            o.a0 = __shfl_up_sync(0xffffffffu, wi.a0, d);
            o.a1 = __shfl_up_sync(0xffffffffu, wi.a1, d);
            const int oc = __shfl_up_sync(0xffffffffu, wic, d);
            if (lane >= d) {
              wi = seq_compose(o, wi);
              wic += oc;
            }
          }
          SeqSummary we;
          we.a0 = __shfl_up_sync(0xffffffffu, wi.a0, 1);
          we.a1 = __shfl_up_sync(0xffffffffu, wi.a1, 1);
          int wec = __shfl_up_sync(0xffffffffu, wic, 1);
          if (lane == 0) {
            seq_identity(&we);
            wec = 0;
          }
          if (lane < kWarps) {
            vc.wpre[lane] = we;
            vc.wpre_cnt[lane] = wec;
          }
          if (lane == kWarps - 1) {
            vc.tot = wi;
            vc.tot_cnt = wic;
          }
        }
        __syncthreads();
        SeqSummary pre = vc.wpre[warp];
        int pre_cnt = vc.wpre_cnt[warp];
        const SeqSummary tot = vc.tot;
        const int tot_cnt = vc.tot_cnt;
        pre = seq_compose(pre, ex);
        pre_cnt += ex_cnt;
        int n_cur = seq_apply(n, pre);
        const int limit = thr_limit(thr, kb);
        int hit_j = -1, before = pre_cnt;
#pragma unroll
        for (int j = 0; j < kVcPer; ++j) {
          if (hit_j < 0 && c[j] > 0) {
            const int na = seq_apply(n_cur, s[j]);
            if (na >= limit) {
              hit_j = j;
            } else {
              n_cur = na;
              before += c[j];
            }
          }
        }
        if (hit_j >= 0) atomicMin(&vc.hit_tid, tid);
        __syncthreads();
        const int ht = vc.hit_tid;
        if (ht == 0x7fffffff) {
          n = seq_apply(n, tot);
          pos += tot_cnt;
          break;
        }
        if (tid == ht) {
          WalkState st;
          st.kb = kb;
          st.n = n_cur;
          bool found;
          float cum;
          float pj = p[0];
          int cj = c[0];
#pragma unroll
          for (int j = 1; j < kVcPer; ++j) {
            if (hit_j == j) {
              pj = p[j];
              cj = c[j];
            }
          }
          int copies = class_hit_step(&st, pj, cj, thr, &found, &cum);
          // a long run may carry the sum through further binades: stay with it instead of
          // paying a block round per binade
          while (!found && copies < cj) {
            const int rest = cj - copies;
            if (seq_apply(st.n, rep_summary(pj, rest, st.kb)) < thr_limit(thr, st.kb)) break;
            copies += class_hit_step(&st, pj, rest, thr, &found, &cum);
          }
          vc.found = found ? 1 : 0;
          vc.kb = st.kb;
          vc.n = st.n;
          vc.hit_b = b0 + hit_j;
          vc.hit_j = copies;
          vc.hit_pos = pos + before + copies - 1;
          vc.cum = cum;
          vc.p = pj;
        }
        __syncthreads();
        const bool found = vc.found != 0;
        const int hit_b = vc.hit_b, copies = vc.hit_j, hit_pos = vc.hit_pos;
        kb = vc.kb;
        n = vc.n;
        if (found) {
          out.found = true;
          out.pos = hit_pos;
          out.p = vc.p;
          out.cum = vc.cum;
          __syncthreads();
          if (tid == 0) vc.hit_tid = 0x7fffffff;
          return out;
        }
        pos = hit_pos + 1;
#pragma unroll
        for (int j = 0; j < kVcPer; ++j) {
          if (b0 + j < hit_b) c[j] = 0;
          if (b0 + j == hit_b) c[j] -= copies;
        }
        __syncthreads();  // everyone has read the record of this round
        if (tid == 0) vc.hit_tid = 0x7fffffff;
      }
      __syncthreads();
      if (vc.ended) goto done;
    }
    win_hi -= span;
    if (win_hi < key_min) break;
  }
done:
  out.found = false;
  out.pos = pos;
  out.cum = seq_value(kb, n);
  out.p = vc.last_key != 0xFFFFFFFFu ? vc_prob(rm, sm, vc.last_key, sum) : 0.0f;
  return out;
}

// The token at position `pos` of the sorted candidate list, where the probability is `pstar`.
// Classes with that same float probability form one group; inside it the list is ordered by
// token index (ties of the reference's comparator, pinned to index order). One read of the row
// counts the tokens in front of the group and the group's members per (tile, thread) in index
// order; the member of rank pos - (tokens in front) is then looked up in its thread's 32 logits.
// Returns -1 if the bookkeeping does not add up.
template <typename T, typename S>
__device__ int vc_select(S& sm, const RowMath<T, S>& rm, float sum, int key_max, int key_min, int pos,
                         float pstar) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  VcControl& vc = sm.vcc;
  __syncthreads();
  // the group's key range: probability does not decrease with the key
  if (tid == 0 || tid == 32) {
    int lo = key_min, hi = key_max;  // invariant: the answer lies in [lo, hi]
    if (tid == 0) {
      // largest key with p(key) <= pstar
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (vc_prob(rm, sm, (uint32_t)mid, sum) <= pstar) lo = mid; else hi = mid - 1;
      }
      vc.g_hi = lo;
    } else {
      // smallest key with p(key) >= pstar
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (vc_prob(rm, sm, (uint32_t)mid, sum) >= pstar) hi = mid; else lo = mid + 1;
      }
      vc.g_lo = lo;
    }
  }
  if (tid == 0) vc.token = -1;
  __syncthreads();
  const uint32_t g_lo = (uint32_t)vc.g_lo, g_hi = (uint32_t)vc.g_hi;
  const uint32_t span = g_hi - g_lo;                  // member:  key - g_lo <= span
  const uint32_t above_span = (uint32_t)key_max - g_hi;  // in front: 0 < key - g_hi <= above_span
  unsigned* cnts = vc_hist(sm);  // [tile][thread]; the class counts are not needed any more
  const int tiles = (rm.vocab + kVcSelTile - 1) / kVcSelTile;
  int above = 0;
  for (int t = 0; t < tiles; ++t) {
    const int i0 = t * kVcSelTile + tid * 32;
    int g = 0;
    uint32_t w[4][4];
#pragma unroll
    for (int k = 0; k < 4; ++k) vc_load8(rm, i0 + 8 * k, w[k]);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t k0 = key_of_pattern16(w[k][j] & 0xFFFFu), k1 = key_of_pattern16(w[k][j] >> 16);
        g += (k0 - g_lo <= span) + (k1 - g_lo <= span);
        above += (k0 - g_hi - 1u < above_span) + (k1 - g_hi - 1u < above_span);
      }
    }
    cnts[t * kThreads + tid] = (unsigned)g;
  }
  int n_above;
  block_excl_count(sm, above, &n_above);
  const int rank = pos - n_above;
  __syncthreads();
  for (int t = warp; t < tiles; t += kWarps) {
    unsigned sacc = 0;
#pragma unroll
    for (int k = 0; k < kThreads / 32; ++k) sacc += cnts[t * kThreads + lane + 32 * k];
    sacc = __reduce_add_sync(0xffffffffu, sacc);
    if (lane == 0) vc.tile_tot[t] = (int)sacc;
  }
  __syncthreads();
  int t_sel = -1, run = 0;
  if (rank >= 0) {
    for (int t = 0; t < tiles; ++t) {
      const int tt = vc.tile_tot[t];
      if (rank < run + tt) {
        t_sel = t;
        break;
      }
      run += tt;
    }
  }
  if (t_sel < 0) return -1;  // block-uniform
  const int g = (int)cnts[t_sel * kThreads + tid];
  int tot;
  const int pre = block_excl_count(sm, g, &tot);
  const int target = rank - run;
  if (pre <= target && target < pre + g) {
    int left = target - pre;  // members of this thread's run to skip
    const int i0 = t_sel * kVcSelTile + tid * 32;
    int token = -1;
    for (int k = 0; k < 4 && token < 0; ++k) {
      uint32_t w[4];
      vc_load8(rm, i0 + 8 * k, w);
      for (int j = 0; j < 8 && token < 0; ++j) {
        const uint32_t pat = (j & 1) ? (w[j >> 1] >> 16) : (w[j >> 1] & 0xFFFFu);
        if (key_of_pattern16(pat) - g_lo <= span) {
          if (left == 0) token = i0 + 8 * k + j;
          --left;
        }
      }
    }
    vc.token = token;
  }
  __syncthreads();
  return vc.token;
}

// The whole tail for one row: sample_topp (sampler.cpp:122-171) from the row's exact softmax sum.
// `raw_max` is the row's largest logit. Returns the token; -1 when the row has no candidate at all
// (undefined in the reference); -2 when the final lookup's counts do not add up.
template <typename T, typename S>
__device__ __forceinline__ int value_class_tail(S& sm, const RowMath<T, S>& rm, float sum, float cutoff, float topp, float coin,
                                float raw_max) {
  const int tid = threadIdx.x;
  VcControl& vc = sm.vcc;
  uint32_t max_pat;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    max_pat = f32_bits(raw_max) >> 16;
  } else {
    max_pat = (uint32_t)__half_as_ushort(__float2half_rn(raw_max));
  }
  const int key_max = (int)key_of_pattern16(max_pat);
  const int key_min = (int)key_of_pattern16(std::is_same<T, __nv_bfloat16>::value ? 0xFF80u : 0xFC00u);
  int pos = 0;
  float pstar = 0.0f;
  // A flat row (softmax sum of the order of the vocabulary size: most terms are close to the
  // largest) has candidates over more classes than one 32-bit window holds: 16-bit class counters
  // first for it (twice the classes per read of the row), and if one of them overflows (65 536 or
  // more equal logits) everything again with 32-bit counters. Other rows usually end inside the
  // first 32-bit window, where the packed form only costs (its check, and neighbouring classes
  // sharing a word).
  const bool flat = sum > 0.125f * (float)rm.vocab;
#pragma unroll 1
  for (int attempt = flat ? 0 : 1; attempt < 2; ++attempt) {
    const bool pack16 = attempt == 0;
    __syncthreads();
    if (tid == 0) {
      vc.hit_tid = 0x7fffffff;
      vc.ended = 0;
      vc.last_key = 0xFFFFFFFFu;
      vc.loaded_hi = -1;
      vc.n_ck = 0;
    }
    __syncthreads();
    ETB_STAMP(7);
    const VcHit first = vc_walk(sm, rm, sum, cutoff, topp, key_max, key_min, true, pack16);
    ETB_STAMP(8);
    if (first.overflow) continue;
    if (first.pos <= 0 && !first.found) return -1;  // no candidate at all
    // last_idx and the sum there (sampler.cpp:147-158); without a hit every candidate is kept
    pos = first.found ? first.pos : first.pos - 1;
    pstar = first.p;
    const float r = __fmul_rn(coin, first.cum);  // sampler.cpp:162
    if (r < first.cum) {
      // the first position whose running sum exceeds r lies at or before last_idx
      __syncthreads();
      if (tid == 0) vc.ended = 0;
      __syncthreads();
      const VcHit second = vc_walk(sm, rm, sum, cutoff, r, key_max, key_min, false, pack16);
      if (second.overflow) continue;
      if (second.found && second.pos <= pos) {
        pos = second.pos;
        pstar = second.p;
      }
    }
    break;
  }
  ETB_STAMP(9);
  const int token = vc_select(sm, rm, sum, key_max, key_min, pos, pstar);
  return token >= 0 ? token : -2;
}
