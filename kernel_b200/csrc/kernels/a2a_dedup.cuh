// The one-launch round trip with one row per (token, destination RANK).
//
// Included by a2a.cu inside its unnamed namespace, after the shared helpers.
//
// The split entry points (dispatch -> caller's expert kernel -> combine) place one
// row per (token, expert): an expert MLP wants its rows contiguous.  The task's
// round trip, whose expert is a scale, does not need that, and with top-8 routing
// over 8 ranks a token reaches 5.25 distinct ranks on average, with all experts
// on one rank exactly one.  Here a token row crosses the link once per
// destination rank, together with the list of its experts on that rank and
// their routing weights (2k + 2 words); the expert phase computes
//     partial = sum over those experts of  w_e * round(scale(e) * x)
// in fp32 (the rounding is the expert's output type) and writes ONE row; the
// combine pulls one row per (token, rank) and adds them in ascending rank order.
// NVLink bytes drop by a third at eight ranks (both directions), memory traffic
// by the top-k factor on one GPU.  The reference sends k copies of every token in
// each direction (reference.py:68-119, 177-234).
__device__ __forceinline__ int meta_words(const A2aParams& p) { return 2 * p.k + 2; }
// Metadata of unique row `slot` that `src` sent to `on_rank`: [count][unused][local expert ids x k][weights x k].
__device__ __forceinline__ uint32_t* meta_ptr(const A2aParams& p, int on_rank, int src, int slot) {
  return reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.meta_off) +
         (static_cast<size_t>(src) * p.tmax + slot) * static_cast<size_t>(meta_words(p));
}

// Bit r set: the token has at least one (valid) expert on rank r.  Eight routing
// entries are fetched before any is looked at.
__device__ __forceinline__ uint32_t rank_mask(const A2aParams& p, int t, bool report) {
  uint32_t mask = 0;
  const int32_t* row = p.idx + static_cast<size_t>(t) * p.k;
  for (int j0 = 0; j0 < p.k; j0 += 8) {
    int ev[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) ev[u] = (j0 + u < p.k) ? __ldg(row + j0 + u) : 0;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (j0 + u >= p.k) continue;
      const int e = ev[u];
      if (e < 0 || e >= p.E) {
        if (report) kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)(t * p.k + j0 + u), p.epoch);
        continue;
      }
      mask |= 1u << (e / p.El);
    }
  }
  return mask;
}

__device__ __forceinline__ void dispatch_dedup_body(const A2aParams& p, int32_t* sh, int nworkers) {
  int32_t* pre = sh;                          // [16] tokens before this CTA's that reach rank r
  int32_t* tot = sh + 16;                     // [16] tokens of this rank that reach rank r
  int32_t* slot_tab = sh + 32;                // [n_tok][world] unique-row slot of (token, rank), or -1
  int32_t* own_mask = slot_tab + DEDUP_MAX_SLOTS;  // [n_tok]
  uint8_t* rowbuf = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sh + table_ints(p.E)) + 127) & ~uintptr_t(127));
  uint64_t* rowbar = reinterpret_cast<uint64_t*>(rowbuf + 2 * ROWBUF_BYTES);
  const int tid = threadIdx.x;
  const int W = p.world;
  stamp(p, ST_ENTRY);
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  const int n_tok = t1 - t0;
  if (tid == 0) {
    kb::mbar_init(&rowbar[0], 1);
    kb::mbar_init(&rowbar[1], 1);
    kb::mbar_fence_init();
  }
  if (tid < 32) sh[tid] = 0;
  __syncthreads();
  // Every CTA walks the whole routing table once: how many earlier tokens reach
  // each rank decides the slots of its own tokens, no count exchange needed.
  // A thread counts in registers, a warp adds its threads' counts up, one lane
  // per warp touches the sixteen shared counters.
  {
    int cnt_tot[KB_MAX_WORLD], cnt_pre[KB_MAX_WORLD];
#pragma unroll
    for (int r = 0; r < KB_MAX_WORLD; ++r) cnt_tot[r] = cnt_pre[r] = 0;
    for (int t = tid; t < p.T; t += blockDim.x) {
      const uint32_t m = rank_mask(p, t, blockIdx.x == 0);
      const bool before = t < t0;
#pragma unroll
      for (int r = 0; r < KB_MAX_WORLD; ++r) {
        const int bit = static_cast<int>((m >> r) & 1u);
        cnt_tot[r] += bit;
        cnt_pre[r] += before ? bit : 0;
      }
    }
#pragma unroll
    for (int r = 0; r < KB_MAX_WORLD; ++r) {
      const int a = __reduce_add_sync(0xffffffffu, cnt_tot[r]);
      const int b = __reduce_add_sync(0xffffffffu, cnt_pre[r]);
      if ((tid & 31) == 0 && r < W) {
        if (a) atomicAdd(&tot[r], a);
        if (b) atomicAdd(&pre[r], b);
      }
    }
  }
  for (int i = tid; i < n_tok; i += blockDim.x) own_mask[i] = static_cast<int32_t>(rank_mask(p, t0 + i, false));
  __syncthreads();
  for (int q = tid; q < n_tok * W; q += blockDim.x) {
    const int i = q / W, r = q - i * W;
    int slot = -1;
    if ((static_cast<uint32_t>(own_mask[i]) >> r) & 1u) {
      slot = pre[r];
      for (int i2 = 0; i2 < i; ++i2) slot += (static_cast<uint32_t>(own_mask[i2]) >> r) & 1u;
      if (slot >= p.tmax) {
        kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)((t0 + i) * p.k), p.epoch);
        slot = -1;
      }
    }
    slot_tab[q] = slot;
    if (hs == 0) p.rank_slots[static_cast<size_t>(t0 + i) * W + r] = slot;
  }
  __syncthreads();
  stamp(p, ST_SLOTS);

  // Expert lists and weights of the unique rows (one CTA of each token group writes them).
  if (hs == 0) {
    for (int q = tid; q < n_tok * p.k; q += blockDim.x) {
      const int i = q / p.k, j = q - i * p.k;
      const int t = t0 + i;
      const int e = __ldg(p.idx + static_cast<size_t>(t) * p.k + j);
      if (e < 0 || e >= p.E) continue;
      const int r = e / p.El;
      const int slot = slot_tab[i * W + r];
      if (slot < 0) continue;
      int pos = 0, cnt = 0;
      for (int j2 = 0; j2 < p.k; ++j2) {
        const int e2 = __ldg(p.idx + static_cast<size_t>(t) * p.k + j2);
        if (e2 >= 0 && e2 < p.E && e2 / p.El == r) {
          ++cnt;
          if (j2 < j) ++pos;
        }
      }
      uint32_t* m = meta_ptr(p, r, p.rank, slot);
      kb::st_relaxed_sys_u32(m + 2 + pos, static_cast<uint32_t>(e - r * p.El));
      kb::st_relaxed_sys_u32(m + 2 + p.k + pos, __float_as_uint(__ldg(p.w + static_cast<size_t>(t) * p.k + j)));
      if (pos == 0) kb::st_relaxed_sys_u32(m, static_cast<uint32_t>(cnt));
    }
  }

  const int slice_bytes = (v1 - v0) * 16;
  if (slice_bytes >= p.bulk_min_bytes) {
    // Payload through the bulk-copy engine, driven by one thread (see dispatch_body).
    if (tid == 0) {
      const int pieces_per_row = (slice_bytes + ROWBUF_BYTES - 1) / ROWBUF_BYTES;
      const int n_pieces = n_tok * pieces_per_row;
      auto piece = [&](int n, int& i, int& off, int& bytes) {
        i = n / pieces_per_row;
        off = v0 * 16 + (n % pieces_per_row) * ROWBUF_BYTES;
        bytes = min(ROWBUF_BYTES, v0 * 16 + slice_bytes - off);
      };
      auto load = [&](int n) {
        int i, off, bytes;
        piece(n, i, off, bytes);
        kb::mbar_arrive_expect_tx(&rowbar[n & 1], static_cast<uint32_t>(bytes));
        kb::bulk_load(rowbuf + (n & 1) * ROWBUF_BYTES, p.x + static_cast<size_t>(t0 + i) * p.row_bytes + off, bytes, &rowbar[n & 1]);
      };
      if (n_pieces > 0) load(0);
      for (int n = 0; n < n_pieces; ++n) {
        if (n + 1 < n_pieces) {
          if (n >= 1) kb::bulk_wait_group_read<0>();
          load(n + 1);
        }
        if (!kb::mbar_wait_bounded(&rowbar[n & 1], (n >> 1) & 1u, p.limit_ns)) {
          kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_DISP_IDX, (uint32_t)n, p.epoch);
          break;
        }
        int i, off, bytes;
        piece(n, i, off, bytes);
        for (int r = 0; r < W; ++r) {
          const int slot = slot_tab[i * W + r];
          if (slot < 0) continue;
          kb::bulk_store(rows_ptr(p, r, p.recv_off, p.rank, slot) + off, rowbuf + (n & 1) * ROWBUF_BYTES, bytes);
        }
        kb::bulk_commit_group();
      }
      kb::bulk_wait_group<0>();
      kb::fence_proxy_async_global();
    }
  } else {
    for (int i = 0; i < n_tok; ++i) {
      const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t0 + i) * p.row_bytes);
      for (int vb = v0 + tid; vb < v1; vb += 4 * blockDim.x) {
        uint4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = vb + u * blockDim.x;
          if (v < v1) val[u] = kb::ld_nc_v4(src + v);
        }
        for (int r = 0; r < W; ++r) {
          const int slot = slot_tab[i * W + r];
          if (slot < 0) continue;
          uint4* d = reinterpret_cast<uint4*>(rows_ptr(p, r, p.recv_off, p.rank, slot));
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = vb + u * blockDim.x;
            if (v < v1) kb::st_sys_v4(d + v, val[u]);
          }
        }
      }
    }
  }
  stamp(p, ST_PUSHED);
  // How many unique rows every destination gets from this rank.
  if (blockIdx.x == 0 && tid < W) counts_ptr(p, tid, p.rank)[0] = tot[tid];
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  finish_phase(p, &sync[0], nworkers, 0);
  stamp(p, ST_DISPATCH_FLAG);
}

// Rounds a vector of fp32 values to the element type and back (the expert's output type).
template <typename T>
__device__ __forceinline__ void round_through(float* f) {
  const uint4 packed = Vec16<T>::store(f);
  Vec16<T>::load(packed, f);
}

// Expert phase over unique rows, in the batched rounds of expert_body.  The
// expert lists and weights of the two rows of a step (2k + 2 <= 130 words each)
// are staged in shared memory by the first threads of the CTA.
template <typename T>
__device__ __forceinline__ void expert_dedup_body(const A2aParams& p, int nworkers) {
  __shared__ uint32_t s_batch;
  __shared__ int32_t s_n[KB_MAX_WORLD], s_first[KB_MAX_WORLD];
  __shared__ uint32_t s_meta[2][2 * 64 + 2];
  const int tid = threadIdx.x;
  const uint32_t all = (1u << p.world) - 1u;
  const int mw = meta_words(p);
  uint32_t done = 0;
  uint64_t waited = 0;
  bool first_round = true;
  while (done != all) {
    if (tid == 0) {
      int s = p.rank;
      for (int si = 0; si < p.world; ++si) {
        s = (p.rank + si) % p.world;
        if (!((done >> s) & 1u)) break;
      }
      const uint64_t w0 = (p.trace != nullptr && blockIdx.x == 0) ? kb::globaltimer_ns() : 0;
      if (!wait_arrival<true>(p, 0, s)) kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)s, p.epoch);
      if (p.trace != nullptr && blockIdx.x == 0) waited += kb::globaltimer_ns() - w0;
      s_batch = 1u << s;
    }
    __syncthreads();
    if (tid < p.world && !((done >> tid) & 1u) && !((s_batch >> tid) & 1u)) {
      if (has_arrived<true>(p, 0, tid)) atomicOr(&s_batch, 1u << tid);
    }
    __syncthreads();
    const uint32_t batch = s_batch & ~done;
    if (first_round) stamp(p, ST_EXPERT_GO);
    first_round = false;
    if (tid < p.world) {
      int n = 0, first = 0;
      if ((batch >> tid) & 1u) {
        int rows = static_cast<int>(kb::ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts_ptr(p, p.rank, tid))));
        if (rows < 0) rows = 0;
        if (rows > p.tmax) rows = p.tmax;
        first = static_cast<int>((blockIdx.x + 37u * static_cast<unsigned>(tid)) % static_cast<unsigned>(nworkers));
        n = rows > first ? (rows - first + nworkers - 1) / nworkers : 0;
      }
      s_n[tid] = n;
      s_first[tid] = first;
    }
    __syncthreads();
    int n_tot = 0;
    for (int s = 0; s < p.world; ++s) n_tot += s_n[s];
    auto entry = [&](int j, int& src_rank, int& row) {
      int s = 0;
      while (j >= s_n[s]) {
        j -= s_n[s];
        ++s;
      }
      src_rank = s;
      row = s_first[s] + j * nworkers;
    };
    for (int j0 = 0; j0 < n_tot; j0 += 2) {
      bool have[2];
      const uint4* src[2];
      uint4* dst[2];
      const uint32_t* meta[2];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        have[b] = j0 + b < n_tot;
        int s = 0, row = 0;
        entry(have[b] ? j0 + b : j0, s, row);
        src[b] = reinterpret_cast<const uint4*>(rows_ptr(p, p.rank, p.recv_off, s, row));
        dst[b] = reinterpret_cast<uint4*>(rows_ptr(p, p.rank, p.y_off, s, row));
        meta[b] = meta_ptr(p, p.rank, s, row);
      }
      __syncthreads();  // the previous step's readers of s_meta are done
      for (int q = tid; q < 2 * mw; q += blockDim.x) {
        const int b = q / mw, wi = q - b * mw;
        s_meta[b][wi] = have[b] ? kb::ld_relaxed_sys_u32(meta[b] + wi) : 0u;
      }
      __syncthreads();
      int cnt[2];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        cnt[b] = static_cast<int>(s_meta[b][0]);
        if (cnt[b] < 0 || cnt[b] > p.k || !have[b]) cnt[b] = 0;
      }
      for (int vb = tid; vb < p.vecs; vb += 4 * blockDim.x) {
        uint4 in[2][4];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = vb + u * blockDim.x;
            if (have[b] && v < p.vecs) in[b][u] = kb::ld_sys_v4(src[b] + v);
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float acc[4][Vec16<T>::N];
          float xin[4][Vec16<T>::N];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            Vec16<T>::load(in[b][u], xin[u]);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) acc[u][i] = 0.f;
          }
          for (int j = 0; j < cnt[b]; ++j) {
            const int le = static_cast<int>(s_meta[b][2 + j]);
            const float wj = __uint_as_float(s_meta[b][2 + p.k + j]);
            float scale = 1.0f;
            if (p.scale_mode == 1) scale = static_cast<float>(1 + p.rank);
            if (p.scale_mode == 2) scale = static_cast<float>(p.rank * p.El + le + 1) / static_cast<float>(p.E);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float y[Vec16<T>::N];
#pragma unroll
              for (int i = 0; i < Vec16<T>::N; ++i) y[i] = xin[u][i] * scale;
              round_through<T>(y);
#pragma unroll
              for (int i = 0; i < Vec16<T>::N; ++i) acc[u][i] = fmaf(wj, y[i], acc[u][i]);
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = vb + u * blockDim.x;
            if (have[b] && v < p.vecs) dst[b][v] = Vec16<T>::store(acc[u]);
          }
        }
      }
    }
    done |= batch;
    __syncthreads();
  }
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[ST_WAITED_EXPERT] = waited;
  stamp(p, ST_EXPERT_ROWS);
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  finish_phase(p, &sync[1], nworkers, 1);
  stamp(p, ST_EXPERT_FLAG);
}

// Combine over unique rows: one partial row per (token, rank), pulled with peer
// loads (two vectors x up to eight ranks in flight per thread) and added in
// ascending rank order.  The slot table is the one the dispatch phase left in
// shared memory.
template <typename T>
__device__ __forceinline__ void combine_dedup_body(const A2aParams& p, const int32_t* slot_tab) {
  const int tid = threadIdx.x;
  const int W = p.world;
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  const uint64_t w0 = (p.trace != nullptr && blockIdx.x == 0 && tid == 0) ? kb::globaltimer_ns() : 0;
  if (tid < W) {
    if (!wait_arrival<true>(p, 1, tid)) kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_COMB_FLAG, (uint32_t)tid, p.epoch);
  }
  __syncthreads();
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[ST_WAITED_COMBINE] = kb::globaltimer_ns() - w0;
  stamp(p, ST_COMBINE_GO);
  for (int t = t0; t < t1; ++t) {
    const int32_t* ts = slot_tab + (t - t0) * W;
    for (int vb = v0 + tid; vb < v1; vb += 2 * blockDim.x) {
      float acc[2][Vec16<T>::N];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
#pragma unroll
        for (int i = 0; i < Vec16<T>::N; ++i) acc[b][i] = 0.f;
      }
      for (int r0 = 0; r0 < W; r0 += 8) {
        uint4 u[2][8];
        bool on[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int r = r0 + j;
          on[j] = r < W && ts[r] >= 0;
          u[0][j] = u[1][j] = make_uint4(0, 0, 0, 0);
          if (on[j]) {
            const uint4* row = reinterpret_cast<const uint4*>(rows_ptr(p, r, p.y_off, p.rank, ts[r]));
            u[0][j] = kb::ld_sys_v4(row + vb);
            if (vb + blockDim.x < v1) u[1][j] = kb::ld_sys_v4(row + vb + blockDim.x);
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if (!on[j]) continue;
            float f[Vec16<T>::N];
            Vec16<T>::load(u[b][j], f);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) acc[b][i] += f[i];
          }
        }
      }
      uint4* orow = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.row_bytes);
      orow[vb] = Vec16<T>::store(acc[0]);
      if (vb + blockDim.x < v1) orow[vb + blockDim.x] = Vec16<T>::store(acc[1]);
    }
  }
  stamp(p, ST_DONE);
}
