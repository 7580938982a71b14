// Low-latency round trip for small token counts: flags travel inside the data.
//
// Included by a2a.cu inside its unnamed namespace, after a2a_dedup.cuh.
//
// The regular one-launch round trip pays, for each of its two cross-rank
// hand-offs, a system-scope fence in the slowest CTA (its stores must be
// acknowledged), a grid-wide count, a second fence, the flag's flight and a poll:
// 10 to 20 us at eight ranks, whatever the payload.  With at most
// LL_MAX_TOKENS tokens per rank the payload is so small that it can carry its
// own arrival signal instead: every 8 bytes on the wire are 4 bytes of data and
// the 4-byte epoch of the call, written by one 8-byte-atomic store, and a reader
// polls the data itself until the epoch is there (the scheme NCCL calls LL).
// Twice the bytes, but no fence, no counter, no flag, no poller CTA, and no
// waiting between the CTAs of a rank:
//
//   dispatch  one row per (token, destination rank) as in a2a_dedup.cuh, written
//             in this format into the destination's landing area, with the
//             row's expert list and weights and the per-source row count in the
//             same format;
//   expert    polls the counts, then each (row, 256-vector block) unit polls its
//             vectors, computes sum_e w_e * round(scale(e) * x) and PUSHES the
//             partial row back into the source's landing area (the regular path
//             lets the source pull);
//   combine   polls the partial rows of its tokens and adds them in ascending
//             rank order.
//
// The reference has no counterpart (its smallest case costs six collectives and
// four host synchronisations, submission.py:59-163).  A slot is reused by the
// same writer only after the reader's answer to the previous call has come back,
// and epochs only grow, so a stale unit can never be mistaken for a fresh one.
constexpr int LL_MAX_TOKENS = 32;
constexpr int LL_BLOCK_VECS = A2A_THREADS;  // vectors of one expert-phase unit

// Landing areas of one rank inside the low-latency region: rows [world][ll_tmax][2 * row_bytes],
// partial rows (same shape), row metadata [world][ll_tmax][2k + 2] pairs, counts [2][world] lines.  A rank that
// sends a peer no row does not wait for that peer, so it can be one call ahead of it (never two: its next
// expert phase needs the peer's count): the count lines alternate with the epoch's parity.
struct LLLayout {
  size_t row2;      // bytes of a row in the wire format
  size_t back_off, meta_off, cnt_off;
};
__host__ __device__ inline LLLayout ll_layout(int world, int ll_tmax, int topk, int row_bytes) {
  LLLayout l;
  l.row2 = 2 * static_cast<size_t>(row_bytes);
  l.back_off = static_cast<size_t>(world) * ll_tmax * l.row2;
  l.meta_off = 2 * l.back_off;
  l.cnt_off = l.meta_off + static_cast<size_t>(world) * ll_tmax * (2 * topk + 2) * 8;
  return l;
}
__host__ __device__ inline size_t ll_region_bytes(int world, int ll_tmax, int topk, int row_bytes) {
  return ll_layout(world, ll_tmax, topk, row_bytes).cnt_off + 2 * static_cast<size_t>(world) * 128;
}

__device__ __forceinline__ uint8_t* ll_row(const A2aParams& p, const LLLayout& l, int on_rank, bool back, int src, int slot) {
  return reinterpret_cast<uint8_t*>(p.peer_base[on_rank]) + p.ll_off + (back ? l.back_off : 0) +
         (static_cast<size_t>(src) * p.ll_tmax + slot) * l.row2;
}
__device__ __forceinline__ uint2* ll_meta(const A2aParams& p, const LLLayout& l, int on_rank, int src, int slot) {
  return reinterpret_cast<uint2*>(p.peer_base[on_rank] + p.ll_off + l.meta_off) +
         (static_cast<size_t>(src) * p.ll_tmax + slot) * static_cast<size_t>(2 * p.k + 2);
}
__device__ __forceinline__ uint2* ll_cnt(const A2aParams& p, const LLLayout& l, int on_rank, int src) {
  return reinterpret_cast<uint2*>(p.peer_base[on_rank] + p.ll_off + l.cnt_off +
                                  (static_cast<size_t>(p.epoch & 1u) * p.world + src) * 128);
}

__device__ __forceinline__ void st_sys_v2(void* q, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(q), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_sys_v2(const void* q) {
  uint2 v;
  asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(q) : "memory");
  return v;
}
// One 16-byte data vector = two 16-byte wire units {d0, epoch, d1, epoch}; each 8-byte half is written atomically.
__device__ __forceinline__ void ll_store_vec(uint8_t* row, int v, const uint4& d, uint32_t f) {
  uint4* q = reinterpret_cast<uint4*>(row) + 2 * static_cast<size_t>(v);
  kb::st_sys_v4(q, make_uint4(d.x, f, d.y, f));
  kb::st_sys_v4(q + 1, make_uint4(d.z, f, d.w, f));
}
// Polls a wire vector until all four halves carry epoch `f`; false after limit_ns.
__device__ __forceinline__ bool ll_load_vec(const uint8_t* row, int v, uint32_t f, uint64_t limit_ns, uint4& d) {
  const uint4* q = reinterpret_cast<const uint4*>(row) + 2 * static_cast<size_t>(v);
  uint4 a = kb::ld_sys_v4(q), b = kb::ld_sys_v4(q + 1);
  if (!(a.y == f && a.w == f && b.y == f && b.w == f)) {
    const uint64_t t0 = kb::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
      a = kb::ld_sys_v4(q);
      b = kb::ld_sys_v4(q + 1);
      if (a.y == f && a.w == f && b.y == f && b.w == f) break;
      if ((++spins & 0x3fu) == 0 && kb::globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
  d = make_uint4(a.x, a.z, b.x, b.z);
  return true;
}
__device__ __forceinline__ bool ll_load_word(const uint2* q, uint32_t f, uint64_t limit_ns, uint32_t& value) {
  uint2 a = ld_sys_v2(q);
  if (a.y != f) {
    const uint64_t t0 = kb::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
      a = ld_sys_v2(q);
      if (a.y == f) break;
      if ((++spins & 0x3fu) == 0 && kb::globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
  value = a.x;
  return true;
}

template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_ll_kernel(const A2aParams p) {
  __shared__ int32_t s_pre[KB_MAX_WORLD], s_tot[KB_MAX_WORLD], s_n[KB_MAX_WORLD];
  __shared__ int32_t s_slot[LL_MAX_TOKENS * KB_MAX_WORLD];
  __shared__ uint32_t s_mask[LL_MAX_TOKENS];
  __shared__ uint32_t s_meta[2 * 64 + 2];
  const int tid = threadIdx.x;
  const int W = p.world;
  const uint32_t f = p.epoch;
  const LLLayout l = ll_layout(W, p.ll_tmax, p.k, p.row_bytes);
  const int mw = 2 * p.k + 2;
  stamp(p, ST_ENTRY);
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) {
    for (int i = 10; i < 16; ++i) p.trace[i] = i < 12 ? 0 : p.trace[ST_ENTRY];
  }
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  const int n_tok = t1 - t0;

  // ---- slots, as in dispatch_dedup_body ----
  if (tid < KB_MAX_WORLD) s_pre[tid] = s_tot[tid] = 0;
  __syncthreads();
  for (int t = tid; t < p.T; t += blockDim.x) {
    uint32_t m = rank_mask(p, t, blockIdx.x == 0);
    while (m) {
      const int r = __ffs(m) - 1;
      m &= m - 1;
      atomicAdd(&s_tot[r], 1);
      if (t < t0) atomicAdd(&s_pre[r], 1);
    }
  }
  for (int i = tid; i < n_tok; i += blockDim.x) s_mask[i] = rank_mask(p, t0 + i, false);
  __syncthreads();
  for (int q = tid; q < n_tok * W; q += blockDim.x) {
    const int i = q / W, r = q - i * W;
    int slot = -1;
    if ((s_mask[i] >> r) & 1u) {
      slot = s_pre[r];
      for (int i2 = 0; i2 < i; ++i2) slot += (s_mask[i2] >> r) & 1u;
      if (slot >= p.ll_tmax) {
        kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)((t0 + i) * p.k), p.epoch);
        slot = -1;
      }
    }
    s_slot[q] = slot;
  }
  __syncthreads();
  stamp(p, ST_SLOTS);

  // ---- dispatch: metadata, rows, counts, all carrying the epoch ----
  if (hs == 0) {
    for (int q = tid; q < n_tok * p.k; q += blockDim.x) {
      const int i = q / p.k, j = q - i * p.k;
      const int t = t0 + i;
      const int e = __ldg(p.idx + static_cast<size_t>(t) * p.k + j);
      if (e < 0 || e >= p.E) continue;
      const int r = e / p.El;
      const int slot = s_slot[i * W + r];
      if (slot < 0) continue;
      int pos = 0, cnt = 0;
      for (int j2 = 0; j2 < p.k; ++j2) {
        const int e2 = __ldg(p.idx + static_cast<size_t>(t) * p.k + j2);
        if (e2 >= 0 && e2 < p.E && e2 / p.El == r) {
          ++cnt;
          if (j2 < j) ++pos;
        }
      }
      uint2* m = ll_meta(p, l, r, p.rank, slot);
      st_sys_v2(m + 2 + pos, static_cast<uint32_t>(e - r * p.El), f);
      st_sys_v2(m + 2 + p.k + pos, __float_as_uint(__ldg(p.w + static_cast<size_t>(t) * p.k + j)), f);
      if (pos == 0) st_sys_v2(m, static_cast<uint32_t>(cnt), f);
    }
  }
  for (int i = 0; i < n_tok; ++i) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t0 + i) * p.row_bytes);
    for (int v = v0 + tid; v < v1; v += blockDim.x) {
      const uint4 d = kb::ld_nc_v4(src + v);
      for (int r = 0; r < W; ++r) {
        const int slot = s_slot[i * W + r];
        if (slot >= 0) ll_store_vec(ll_row(p, l, r, false, p.rank, slot), v, d, f);
      }
    }
  }
  if (blockIdx.x == 0 && tid < W) st_sys_v2(ll_cnt(p, l, tid, p.rank), static_cast<uint32_t>(s_tot[tid]), f);
  stamp(p, ST_PUSHED);
  stamp(p, ST_DISPATCH_FLAG);

  // ---- expert: (row, block of 256 vectors) units over all CTAs ----
  if (tid < W) {
    uint32_t n = 0;
    if (!ll_load_word(ll_cnt(p, l, p.rank, tid), f, p.limit_ns, n)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)tid, p.epoch);
      n = 0;
    }
    s_n[tid] = static_cast<int>(n > static_cast<uint32_t>(p.ll_tmax) ? p.ll_tmax : n);
  }
  __syncthreads();
  stamp(p, ST_EXPERT_GO);
  int rows_total = 0;
  for (int s = 0; s < W; ++s) rows_total += s_n[s];
  const int nblk = (p.vecs + LL_BLOCK_VECS - 1) / LL_BLOCK_VECS;
  for (int u = blockIdx.x; u < rows_total * nblk; u += gridDim.x) {
    int g = u / nblk;
    const int blk = u - g * nblk;
    int s = 0;
    while (g >= s_n[s]) {
      g -= s_n[s];
      ++s;
    }
    __syncthreads();  // the previous unit's readers of s_meta are done
    if (tid == 0) {
      uint32_t cnt = 0;
      if (!ll_load_word(ll_meta(p, l, p.rank, s, g), f, p.limit_ns, cnt)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)s, p.epoch);
        cnt = 0;
      }
      s_meta[0] = cnt > static_cast<uint32_t>(p.k) ? 0u : cnt;
    }
    __syncthreads();
    const int cnt = static_cast<int>(s_meta[0]);
    for (int q = tid; q < 2 * cnt; q += blockDim.x) {
      const int wi = q < cnt ? 2 + q : 2 + p.k + (q - cnt);
      uint32_t val = 0;
      if (!ll_load_word(ll_meta(p, l, p.rank, s, g) + wi, f, p.limit_ns, val)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)s, p.epoch);
      }
      s_meta[wi] = val;
    }
    __syncthreads();
    const int v = blk * LL_BLOCK_VECS + tid;
    if (v < p.vecs) {
      uint4 d;
      if (!ll_load_vec(ll_row(p, l, p.rank, false, s, g), v, f, p.limit_ns, d)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)s, p.epoch);
        d = make_uint4(0, 0, 0, 0);
      }
      float xin[Vec16<T>::N], acc[Vec16<T>::N];
      Vec16<T>::load(d, xin);
#pragma unroll
      for (int i = 0; i < Vec16<T>::N; ++i) acc[i] = 0.f;
      for (int j = 0; j < cnt; ++j) {
        const int le = static_cast<int>(s_meta[2 + j]);
        const float wj = __uint_as_float(s_meta[2 + p.k + j]);
        float scale = 1.0f;
        if (p.scale_mode == 1) scale = static_cast<float>(1 + p.rank);
        if (p.scale_mode == 2) scale = static_cast<float>(p.rank * p.El + le + 1) / static_cast<float>(p.E);
        float y[Vec16<T>::N];
#pragma unroll
        for (int i = 0; i < Vec16<T>::N; ++i) y[i] = xin[i] * scale;
        round_through<T>(y);
#pragma unroll
        for (int i = 0; i < Vec16<T>::N; ++i) acc[i] = fmaf(wj, y[i], acc[i]);
      }
      // the partial row goes straight back to the source's landing area
      ll_store_vec(ll_row(p, l, s, true, p.rank, g), v, Vec16<T>::store(acc), f);
    }
  }
  stamp(p, ST_EXPERT_ROWS);
  stamp(p, ST_EXPERT_FLAG);
  stamp(p, ST_COMBINE_GO);

  // ---- combine: this CTA's tokens and slice, partial rows in ascending rank order ----
  for (int i = 0; i < n_tok; ++i) {
    for (int v = v0 + tid; v < v1; v += blockDim.x) {
      float acc[Vec16<T>::N];
#pragma unroll
      for (int j = 0; j < Vec16<T>::N; ++j) acc[j] = 0.f;
      for (int r = 0; r < W; ++r) {
        const int slot = s_slot[i * W + r];
        if (slot < 0) continue;
        uint4 d;
        if (!ll_load_vec(ll_row(p, l, p.rank, true, r, slot), v, f, p.limit_ns, d)) {
          kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_COMB_FLAG, (uint32_t)r, p.epoch);
          continue;
        }
        float y[Vec16<T>::N];
        Vec16<T>::load(d, y);
#pragma unroll
        for (int j = 0; j < Vec16<T>::N; ++j) acc[j] += y[j];
      }
      reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t0 + i) * p.row_bytes)[v] = Vec16<T>::store(acc);
    }
  }
  stamp(p, ST_DONE);
}
