// MoE expert-parallel dispatch / combine over symmetric memory (sm_100a).
//
// Replaces the reference's six NCCL collectives, four host syncs, argsort and
// three local copies of the payload per direction (submission.py:37-189,
// reference.py:68-234) with three launches and no host involvement:
//
//   dispatch  every CTA histograms the routing table, derives for each
//             (token, k) copy its final row ("slot") in the owner rank's
//             receive region, and stores the token row there with 16-byte
//             peer stores.  Per-(source, expert) counts travel the same way.
//             The last CTA to finish publishes an epoch flag to every peer.
//   expert    (stand-in for the expert MLP) waits for all sources' flags and
//             writes y = scale(expert) * x into the pull region, then
//             publishes a second flag.
//   combine   because the sender chose the slots it already knows where each
//             copy lives: it pulls the k rows of a token with 16-byte peer
//             loads, accumulates w[t,k] * row in fp32 in fixed k order
//             (deterministic), and stores once.  No metadata crosses the wire.
//
// Layout of one rank's receive region: [world sources][capacity rows][H];
// a source's rows are grouped by local expert, in expert order.  Capacity is
// max_tokens * topk rows (a source can never send more to one rank).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdlib.h>

#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../include/kb200.h"

namespace {

constexpr int A2A_THREADS = 256;
constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_ENT_PER_CTA = 2048;
// Dispatch push through the bulk-copy engine: a slice of a token row is brought
// into one of two shared-memory buffers with one cp.async.bulk and sent to its k
// destinations with one cp.async.bulk each.
constexpr int ROWBUF_BYTES = 16384;
constexpr int BULK_MIN_BYTES = 1024;  // shorter slices go the load / store way
constexpr int DEDUP_MAX_SLOTS = 4096;  // one-launch round trip: (tokens of a CTA) x world entries of its slot table

// Words of the integer tables at the front of the dynamic shared memory of a
// kernel that runs a dispatch phase (the row buffers follow them).
__host__ __device__ inline int table_ints(int experts) {
  const int a = 3 * experts + 2 * MAX_ENT_PER_CTA;  // per-expert dispatch: tot, pre, off, entry experts, entry slots
  const int b = 32 + 2 * DEDUP_MAX_SLOTS;           // per-rank dispatch: pre[16], tot[16], slot table, rank masks
  return a > b ? a : b;
}
// Every (phase, source) flag sits on a 128-byte line of its own: a peer's flag
// store never queues behind polls of another source's flag.
constexpr int FLAG_STRIDE_WORDS = 32;
constexpr int GO_WORD_OFF = 32;   // sync region: words [0..3] block counters, [32..47] and [64..79] arrival words

enum Site : uint32_t { SITE_DISP_IDX = 11, SITE_EXP_FLAG = 12, SITE_COMB_FLAG = 13, SITE_COMB_SLOT = 14, SITE_POLLER = 15 };

struct A2aParams {
  int rank, world, E, El, k, H, T, cap;
  int row_bytes, vecs;  // bytes and 16-byte vectors per row
  int tok_groups, h_splits;
  const uint8_t* x;
  const int32_t* idx;
  const float* w;
  uint8_t* out;
  int32_t* slots;
  uint32_t epoch;
  char* peer_base[KB_MAX_WORLD];
  uint64_t recv_off, y_off, count_off, flag_off, sync_off;
  int scale_mode;
  uint32_t* status;
  uint64_t limit_ns;
  uint64_t* trace;
  int bulk_min_bytes;  // row slices at least this long are pushed by the bulk-copy engine; 0x7fffffff: never
  int tmax;            // max_tokens: capacity, in unique rows, of one source's share of a receive region
  uint64_t meta_off;   // one-launch round trip: [world][tmax][2k + 2] words, expert lists and weights of the unique rows
  int32_t* rank_slots; // one-launch round trip: local [T][world], slot of (token, rank) or -1
  uint64_t ll_off;     // low-latency round trip: landing areas in the wire format of a2a_ll.cuh; 0: none
  int ll_tmax;         // rows per source those areas hold
};

// Phase stamps (nanoseconds of the global timer) written by thread 0 of CTA 0.
// Words 10 and 11 hold the time that CTA spent inside the arrival waits of the
// expert pass and of the combine; words 12 to 15 are written by the CTA that
// finishes a phase last: when it arrived and when it had stored the flags, for
// the dispatch and for the expert phase.
enum Stamp { ST_ENTRY = 0, ST_SLOTS = 1, ST_PUSHED = 2, ST_DISPATCH_FLAG = 3, ST_EXPERT_GO = 4, ST_EXPERT_ROWS = 5,
             ST_EXPERT_FLAG = 6, ST_COMBINE_GO = 7, ST_DONE = 8, ST_WAITED_EXPERT = 10, ST_WAITED_COMBINE = 11 };
__device__ __forceinline__ void stamp(const A2aParams& p, int which) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.trace[which] = kb::globaltimer_ns();
}

__device__ __forceinline__ uint8_t* rows_ptr(const A2aParams& p, int on_rank, uint64_t region_off, int src, int slot) {
  return reinterpret_cast<uint8_t*>(p.peer_base[on_rank]) + region_off +
         (static_cast<size_t>(src) * p.cap + slot) * static_cast<size_t>(p.row_bytes);
}
__device__ __forceinline__ int32_t* counts_ptr(const A2aParams& p, int on_rank, int src) {
  return reinterpret_cast<int32_t*>(p.peer_base[on_rank] + p.count_off) + static_cast<size_t>(src) * p.El;
}
__device__ __forceinline__ uint32_t* flag_ptr(const A2aParams& p, int on_rank, int which, int src) {
  return reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off) +
         static_cast<size_t>(which * KB_MAX_WORLD + src) * FLAG_STRIDE_WORDS;
}
// Local arrival word of (phase, source), published by the poller CTA of a fused launch.
__device__ __forceinline__ uint32_t* go_ptr(const A2aParams& p, int which, int src) {
  return reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off) + GO_WORD_OFF * (1 + which) + src;
}
// With one rank nothing leaves this GPU and device scope is enough.
__device__ __forceinline__ void fence_for(const A2aParams& p) {
  if (p.world == 1) __threadfence();
  else kb::fence_sys();
}

// Counts this CTA as done with a phase (its writes ordered before the count) and,
// in the one CTA that arrives last, publishes this rank's flag of phase `which` on
// every rank.  One thread does the fence after the count and all the flag stores:
// fence + relaxed stores by the same thread is a release, and the critical path
// holds one system-scope fence here instead of one per posting thread.
__device__ __forceinline__ void finish_phase(const A2aParams& p, uint32_t* counter, uint32_t total, int which) {
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_for(p);
    const uint32_t old = atomicAdd(counter, 1u);
    if (old == total - 1u) {
      if (p.trace != nullptr) p.trace[12 + 2 * which] = kb::globaltimer_ns();  // the last CTA of the phase has arrived
      *counter = 0u;  // ready for the next launch
      fence_for(p);
      for (int dst = 0; dst < p.world; ++dst) {
        uint32_t* f = flag_ptr(p, dst, which, p.rank);
        if (p.world == 1) kb::st_release_gpu_u32(f, p.epoch);
        else kb::st_relaxed_sys_u32(f, p.epoch);
      }
      if (p.trace != nullptr) p.trace[13 + 2 * which] = kb::globaltimer_ns();  // its flags are on their way
    }
  }
  __syncthreads();
}

// Waits until source `src` has reached phase `which` of this epoch.  In a fused
// launch the data CTAs watch the local arrival word that the poller CTA
// publishes (one reader per CTA of a line nobody writes remotely); otherwise
// they watch the flag the peer writes.  One thread calls this.
template <bool kFused>
__device__ __forceinline__ bool wait_arrival(const A2aParams& p, int which, int src) {
  // The arrival words are written and read on this GPU only: device scope.  What
  // a peer wrote before its flag is ordered before the poller's system-scope
  // acquire, hence before the poller's release of the word, hence before this read.
  if (kFused) return kb::wait_flag_ge(go_ptr(p, which, src), p.epoch, 2 * p.limit_ns, 0, false);
  return kb::wait_flag_ge(flag_ptr(p, p.rank, which, src), p.epoch, p.limit_ns, 256, p.world > 1);
}

// The poller CTA of a fused launch: thread s watches the two flags source s
// sends and republishes each as a local arrival word.  It is the only reader of
// the lines the peers write.  After a time-out it reports and publishes anyway,
// so that the data CTAs do not each run into their own limit.
__device__ __forceinline__ void poller_body(const A2aParams& p) {
  const int s = threadIdx.x;
  if (s >= p.world) return;
  for (int which = 0; which < 2; ++which) {
    if (!kb::wait_flag_ge(flag_ptr(p, p.rank, which, s), p.epoch, p.limit_ns, 0, p.world > 1, true)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_POLLER, (uint32_t)(which * KB_MAX_WORLD + s), p.epoch);
    }
    kb::st_release_gpu_u32(go_ptr(p, which, s), p.epoch);
  }
}

// ------------------------------------------------------------------ dispatch ----
// Work unit u = (token group tg, hidden split hs); one unit per CTA.
__device__ __forceinline__ void unit_ranges(const A2aParams& p, int& t0, int& t1, int& v0, int& v1, int& hs) {
  const int tg = blockIdx.x / p.h_splits;
  hs = blockIdx.x - tg * p.h_splits;
  const int tok_per = (p.T + p.tok_groups - 1) / p.tok_groups;
  t0 = min(tg * tok_per, p.T);
  t1 = min(t0 + tok_per, p.T);
  const int v_per = (p.vecs + p.h_splits - 1) / p.h_splits;
  v0 = min(hs * v_per, p.vecs);
  v1 = min(v0 + v_per, p.vecs);
  if (blockIdx.x >= p.tok_groups * p.h_splits) {  // surplus CTAs
    t0 = t1 = p.T;
    v0 = v1 = 0;
  }
}

// off[e] = entries of the experts before e on e's owner rank: an exclusive block
// scan over all experts (four per thread), minus the scan value at the owner's
// first expert.  `tmp` holds E words.
__device__ __forceinline__ void expert_offsets(const int32_t* tot, int32_t* off, int32_t* tmp, int E, int El) {
  __shared__ int32_t s_warp[A2A_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int v[4];
  int sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = tid * 4 + j;
    v[j] = e < E ? tot[e] : 0;
    sum += v[j];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int run = incl - sum;
  for (int wv = 0; wv < warp; ++wv) run += s_warp[wv];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int e = tid * 4 + j;
    if (e < E) tmp[e] = run;
    run += v[j];
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) off[e] = tmp[e] - tmp[(e / El) * El];
}

__device__ __forceinline__ void dispatch_body(const A2aParams& p, int32_t* sh, int nworkers) {
  // behind the tables: two row buffers (128-byte aligned) and their two mbarriers
  uint8_t* rowbuf = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(sh + table_ints(p.E)) + 127) & ~uintptr_t(127));
  uint64_t* rowbar = reinterpret_cast<uint64_t*>(rowbuf + 2 * ROWBUF_BYTES);
  if (threadIdx.x == 0) {
    kb::mbar_init(&rowbar[0], 1);
    kb::mbar_init(&rowbar[1], 1);
    kb::mbar_fence_init();
  }
  int32_t* tot = sh;               // [E] entries per expert, whole rank
  int32_t* pre = tot + p.E;        // [E] entries per expert before this CTA's tokens
  int32_t* off = pre + p.E;        // [E] first slot of the expert inside its owner's region
  int32_t* ent_e = off + p.E;      // [MAX_ENT_PER_CTA] expert of each (token, k) entry of this CTA's tokens
  int32_t* ent_slot = ent_e + MAX_ENT_PER_CTA;  // [MAX_ENT_PER_CTA] its row in the owner's region, or -1

  const int tid = threadIdx.x;
  stamp(p, ST_ENTRY);
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  const int n_ent = (t1 - t0) * p.k;
  const int total_ent = p.T * p.k;

  for (int e = tid; e < p.E; e += blockDim.x) {
    tot[e] = 0;
    pre[e] = 0;
  }
  __syncthreads();
  // Sixteen entries per thread are fetched before any is counted: one memory
  // latency per sixteen entries instead of one per entry.
  for (int i0 = tid; i0 < total_ent; i0 += 16 * blockDim.x) {
    int ev[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int i = i0 + u * blockDim.x;
      ev[u] = i < total_ent ? __ldg(p.idx + i) : 0;
    }
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i >= total_ent) continue;
      const int e = ev[u];
      if (e < 0 || e >= p.E) {
        kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)i, p.epoch);
        continue;
      }
      atomicAdd(&tot[e], 1);
      if (i < t0 * p.k) atomicAdd(&pre[e], 1);
    }
  }
  __syncthreads();
  expert_offsets(tot, off, ent_slot, p.E, p.El);  // ent_slot is free until the ranking below
  for (int i = tid; i < n_ent; i += blockDim.x) ent_e[i] = p.idx[t0 * p.k + i];
  __syncthreads();
  // Rank of an entry among earlier entries of the same expert inside this
  // CTA's range; computed without atomics so that CTAs sharing a token range
  // (different hidden splits) agree on every slot.
  for (int i = tid; i < n_ent; i += blockDim.x) {
    const int e = ent_e[i];
    int slot = -1;
    if (e >= 0 && e < p.E) {
      int r = 0;
      for (int j = 0; j < i; ++j) r += (ent_e[j] == e) ? 1 : 0;
      slot = off[e] + pre[e] + r;
      if (slot >= p.cap) {
        kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)(t0 * p.k + i), p.epoch);
        slot = -1;
      }
    }
    ent_slot[i] = slot;
    if (hs == 0) p.slots[t0 * p.k + i] = slot;
  }
  __syncthreads();
  stamp(p, ST_SLOTS);

  const int slice_bytes = (v1 - v0) * 16;
  if (slice_bytes >= p.bulk_min_bytes) {
    // Payload through the bulk-copy engine, driven by one thread: piece n of the
    // CTA's rows (at most ROWBUF_BYTES of one token row) is loaded into buffer
    // n & 1 while the k stores of piece n - 1 are still leaving the other buffer.
    // The stores go to peer memory as large packets and cost the SM no issue
    // slots; their completion (wait_group 0) precedes this CTA's count below.
    if (tid == 0) {
      const int pieces_per_row = (slice_bytes + ROWBUF_BYTES - 1) / ROWBUF_BYTES;
      const int n_pieces = (t1 - t0) * pieces_per_row;
      auto piece = [&](int n, int& t, int& off, int& bytes) {
        t = t0 + n / pieces_per_row;
        off = v0 * 16 + (n % pieces_per_row) * ROWBUF_BYTES;
        bytes = min(ROWBUF_BYTES, v0 * 16 + slice_bytes - off);
      };
      auto load = [&](int n) {
        int t, off, bytes;
        piece(n, t, off, bytes);
        kb::mbar_arrive_expect_tx(&rowbar[n & 1], static_cast<uint32_t>(bytes));
        kb::bulk_load(rowbuf + (n & 1) * ROWBUF_BYTES, p.x + static_cast<size_t>(t) * p.row_bytes + off, bytes, &rowbar[n & 1]);
      };
      if (n_pieces > 0) load(0);
      for (int n = 0; n < n_pieces; ++n) {
        if (n + 1 < n_pieces) {
          if (n >= 1) kb::bulk_wait_group_read<0>();  // the stores of piece n - 1 have read the buffer piece n + 1 goes into
          load(n + 1);
        }
        if (!kb::mbar_wait_bounded(&rowbar[n & 1], (n >> 1) & 1u, p.limit_ns)) {
          kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_DISP_IDX, (uint32_t)n, p.epoch);
          break;
        }
        int t, off, bytes;
        piece(n, t, off, bytes);
        for (int kk = 0; kk < p.k; ++kk) {
          const int i = (t - t0) * p.k + kk;
          const int slot = ent_slot[i];
          if (slot < 0) continue;
          kb::bulk_store(rows_ptr(p, ent_e[i] / p.El, p.recv_off, p.rank, slot) + off, rowbuf + (n & 1) * ROWBUF_BYTES, bytes);
        }
        kb::bulk_commit_group();
      }
      kb::bulk_wait_group<0>();          // every store has been performed
      kb::fence_proxy_async_global();    // and is ordered before the ordinary accesses that follow (the count, the flag)
    }
  } else {
  // Payload: every 16-byte vector is read once and stored k times.  A thread
  // first issues all the loads of its (up to four) vectors of a row, so that the
  // load latency is paid once per row, not once per vector.
  for (int t = t0; t < t1; ++t) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.row_bytes);
    for (int vb = v0 + tid; vb < v1; vb += 4 * blockDim.x) {
      uint4 val[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = vb + u * blockDim.x;
        if (v < v1) val[u] = kb::ld_nc_v4(src + v);
      }
      for (int kk = 0; kk < p.k; ++kk) {
        const int i = (t - t0) * p.k + kk;
        const int slot = ent_slot[i];
        if (slot < 0) continue;
        const int dst = ent_e[i] / p.El;
        uint4* d = reinterpret_cast<uint4*>(rows_ptr(p, dst, p.recv_off, p.rank, slot));
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
  // Per-(source, expert) counts for every destination.
  if (blockIdx.x == 0) {
    for (int e = tid; e < p.E; e += blockDim.x) {
      counts_ptr(p, e / p.El, p.rank)[e % p.El] = tot[e];
    }
  }
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  finish_phase(p, &sync[0], nworkers, 0);
  stamp(p, ST_DISPATCH_FLAG);
}

__global__ void __launch_bounds__(A2A_THREADS) a2a_dispatch_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  dispatch_body(p, sh, gridDim.x);
}

// -------------------------------------------------------------- expert scale ----
template <typename T>
struct Vec16;
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const uint4& u, float* f) {
    float2 t;
    t = kb::unpack_bf16x2(u.x); f[0] = t.x; f[1] = t.y;
    t = kb::unpack_bf16x2(u.y); f[2] = t.x; f[3] = t.y;
    t = kb::unpack_bf16x2(u.z); f[4] = t.x; f[5] = t.y;
    t = kb::unpack_bf16x2(u.w); f[6] = t.x; f[7] = t.y;
  }
  __device__ static uint4 store(const float* f) {
    uint4 o;
    o.x = kb::pack_bf16x2(f[0], f[1]);
    o.y = kb::pack_bf16x2(f[2], f[3]);
    o.z = kb::pack_bf16x2(f[4], f[5]);
    o.w = kb::pack_bf16x2(f[6], f[7]);
    return o;
  }
};
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  __device__ static void load(const uint4& u, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ static uint4 store(const float* f) {
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return o;
  }
};
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x);
    f[1] = __uint_as_float(u.y);
    f[2] = __uint_as_float(u.z);
    f[3] = __uint_as_float(u.w);
  }
  __device__ static uint4 store(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

// Non-blocking form of wait_arrival: true if source `src` has reached phase `which`.
template <bool kFused>
__device__ __forceinline__ bool has_arrived(const A2aParams& p, int which, int src) {
  const bool sys = !kFused && p.world > 1;
  const uint32_t* word = kFused ? go_ptr(p, which, src) : flag_ptr(p, p.rank, which, src);
  const uint32_t v = sys ? kb::ld_relaxed_sys_u32(word) : kb::ld_relaxed_gpu_u32(word);
  if (static_cast<int32_t>(v - p.epoch) < 0) return false;
  if (sys) kb::fence_sys();
  else kb::fence_gpu();
  return true;
}

// The simulated expert, in rounds.  A round waits for the next missing source in
// ring order (starting with this rank, whose own rows are there first), takes
// along every other source whose dispatch flag has arrived meanwhile, and scales
// the rows of all of them in one batch: the counts of the batch's sources are
// scanned by different warps at the same time, and the CTA's rows of the whole
// batch form one list that is worked two rows per step (eight 16-byte loads per
// thread in flight).  When the ranks run aligned this is one round or two; when a
// source is late, everything that has arrived is done before the wait for it.
// Rows of a source are dealt round-robin to the data CTAs, starting at a CTA
// that depends on the source so that remainders spread out.
template <typename T, bool kFused>
__device__ __forceinline__ void expert_body(const A2aParams& p, int32_t* sh, int nworkers) {
  int32_t* incl = sh;  // [world][El] clamped inclusive prefix of each source's counts
  __shared__ uint32_t s_batch;
  __shared__ int32_t s_n[KB_MAX_WORLD], s_first[KB_MAX_WORLD];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const uint32_t all = p.world >= 32 ? 0xffffffffu : ((1u << p.world) - 1u);
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
      if (!wait_arrival<kFused>(p, 0, s)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)s, p.epoch);
      }
      if (p.trace != nullptr && blockIdx.x == 0) waited += kb::globaltimer_ns() - w0;
      s_batch = 1u << s;
    }
    __syncthreads();
    if (tid < p.world && !((done >> tid) & 1u) && !((s_batch >> tid) & 1u)) {
      if (has_arrived<kFused>(p, 0, tid)) atomicOr(&s_batch, 1u << tid);
    }
    __syncthreads();
    const uint32_t batch = s_batch & ~done;
    if (first_round) stamp(p, ST_EXPERT_GO);
    first_round = false;
    // Counts of the batch's sources -> clamped inclusive prefixes, one warp per source.
    for (int s = warp; s < p.world; s += A2A_THREADS / 32) {
      if (!((batch >> s) & 1u)) continue;
      const int32_t* counts = counts_ptr(p, p.rank, s);
      int carry = 0;
      for (int base = 0; base < p.El; base += 32) {
        const int le = base + lane;
        int v = 0;
        if (le < p.El) v = static_cast<int>(kb::ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + le)));
        if (v < 0) v = 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int n = __shfl_up_sync(0xffffffffu, v, o);
          if (lane >= o) v += n;
        }
        v += carry;
        if (v > p.cap) v = p.cap;
        if (le < p.El) incl[s * p.El + le] = v;
        carry = __shfl_sync(0xffffffffu, v, 31);
      }
    }
    __syncthreads();
    if (tid < p.world) {
      int n = 0, first = 0;
      if ((batch >> tid) & 1u) {
        const int rows = incl[tid * p.El + p.El - 1];
        first = static_cast<int>((blockIdx.x + 37u * static_cast<unsigned>(tid)) % static_cast<unsigned>(nworkers));
        n = rows > first ? (rows - first + nworkers - 1) / nworkers : 0;
      }
      s_n[tid] = n;
      s_first[tid] = first;
    }
    __syncthreads();
    int n_tot = 0;
    for (int s = 0; s < p.world; ++s) n_tot += s_n[s];
    // Entry j of this CTA's list -> (source, row): the sources' shares are laid end to end.
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
      float scale[2];
      const uint4* src[2];
      uint4* dst[2];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        have[b] = j0 + b < n_tot;
        int s = 0, row = 0;
        entry(have[b] ? j0 + b : j0, s, row);
        // first local expert whose inclusive prefix exceeds row
        const int32_t* in = incl + s * p.El;
        int lo = 0, hi = p.El - 1;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (in[mid] > row) hi = mid; else lo = mid + 1;
        }
        scale[b] = 1.0f;
        if (p.scale_mode == 1) scale[b] = static_cast<float>(1 + p.rank);
        if (p.scale_mode == 2) scale[b] = static_cast<float>(p.rank * p.El + lo + 1) / static_cast<float>(p.E);
        src[b] = reinterpret_cast<const uint4*>(rows_ptr(p, p.rank, p.recv_off, s, row));
        dst[b] = reinterpret_cast<uint4*>(rows_ptr(p, p.rank, p.y_off, s, row));
      }
      for (int vb = tid; vb < p.vecs; vb += 4 * blockDim.x) {
        uint4 in[2][4];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {  // all loads of this thread first: one latency per pair of rows
            const int v = vb + u * blockDim.x;
            if (have[b] && v < p.vecs) in[b][u] = kb::ld_sys_v4(src[b] + v);
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int v = vb + u * blockDim.x;
            if (have[b] && v < p.vecs) {
              float f[Vec16<T>::N];
              Vec16<T>::load(in[b][u], f);
#pragma unroll
              for (int i = 0; i < Vec16<T>::N; ++i) f[i] *= scale[b];
              dst[b][v] = Vec16<T>::store(f);
            }
          }
        }
      }
    }
    done |= batch;
    __syncthreads();  // s_batch, s_n and the prefixes are rewritten by the next round
  }
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[ST_WAITED_EXPERT] = waited;
  stamp(p, ST_EXPERT_ROWS);
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  finish_phase(p, &sync[1], nworkers, 1);
  stamp(p, ST_EXPERT_FLAG);
}

template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_expert_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  expert_body<T, false>(p, sh, gridDim.x);
}

// ------------------------------------------------------------------- combine ----
// `ent_e` / `ent_slot` hold expert and slot of the (token, k) entries of this
// CTA's tokens in shared memory: left there by the dispatch phase of a fused
// launch, or loaded by the prologue below when the combine runs as a launch of
// its own.  The k rows of a token are pulled with peer loads, two 16-byte
// vectors per thread and iteration (up to sixteen loads in flight), and
// accumulated in fp32 in fixed k order.
template <typename T, bool kFused>
__device__ __forceinline__ void combine_body(const A2aParams& p, int32_t* ent_e, int32_t* ent_slot) {
  const int tid = threadIdx.x;
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  if (!kFused) {
    const int n_ent = (t1 - t0) * p.k;
    for (int i = tid; i < n_ent; i += blockDim.x) {
      const int e = p.idx[t0 * p.k + i];
      const int slot = p.slots[t0 * p.k + i];
      const bool ok = e >= 0 && e < p.E && slot >= 0 && slot < p.cap;
      ent_e[i] = ok ? e : 0;
      ent_slot[i] = ok ? slot : -1;
    }
  }
  const uint64_t w0 = (p.trace != nullptr && blockIdx.x == 0 && tid == 0) ? kb::globaltimer_ns() : 0;
  if (tid < p.world) {
    if (!wait_arrival<kFused>(p, 1, tid)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_COMB_FLAG, (uint32_t)tid, p.epoch);
    }
  }
  __syncthreads();
  if (p.trace != nullptr && blockIdx.x == 0 && tid == 0) p.trace[ST_WAITED_COMBINE] = kb::globaltimer_ns() - w0;
  stamp(p, ST_COMBINE_GO);
  for (int t = t0; t < t1; ++t) {
    const int32_t* te = ent_e + (t - t0) * p.k;
    const int32_t* ts = ent_slot + (t - t0) * p.k;
    const float* tw = p.w + static_cast<size_t>(t) * p.k;
    for (int vb = v0 + tid; vb < v1; vb += 2 * blockDim.x) {
      float acc[2][Vec16<T>::N];
#pragma unroll
      for (int b = 0; b < 2; ++b) {
#pragma unroll
        for (int i = 0; i < Vec16<T>::N; ++i) acc[b][i] = 0.f;
      }
      for (int k0 = 0; k0 < p.k; k0 += 8) {
        uint4 u[2][8];
        float wk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int kk = k0 + j;
          wk[j] = 0.f;
          u[0][j] = u[1][j] = make_uint4(0, 0, 0, 0);
          if (kk < p.k && ts[kk] >= 0) {
            wk[j] = __ldg(tw + kk);
            const uint4* row = reinterpret_cast<const uint4*>(rows_ptr(p, te[kk] / p.El, p.y_off, p.rank, ts[kk]));
            u[0][j] = kb::ld_sys_v4(row + vb);
            if (vb + blockDim.x < v1) u[1][j] = kb::ld_sys_v4(row + vb + blockDim.x);
          }
        }
#pragma unroll
        for (int b = 0; b < 2; ++b) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float f[Vec16<T>::N];
            Vec16<T>::load(u[b][j], f);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) acc[b][i] = fmaf(wk[j], f[i], acc[b][i]);
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

template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_combine_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  combine_body<T, false>(p, sh, sh + MAX_ENT_PER_CTA);
}

#include "a2a_dedup.cuh"
#include "a2a_ll.cuh"

// All three phases in one cooperative launch (every CTA is resident, so CTAs may
// wait for one another).  The last CTA of the grid is the poller: it moves no
// rows, it is the only reader of the flag lines the peers write and republishes
// them locally.  The other CTAs are the data CTAs; their phases are separated
// only by the arrival words, this rank's own flags doubling as grid barrier.
// The phases are the per-rank ones of a2a_dedup.cuh: one row per (token, rank).
template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_fused_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  const int nworkers = static_cast<int>(gridDim.x) - 1;
  if (static_cast<int>(blockIdx.x) == nworkers) {
    poller_body(p);
    return;
  }
  dispatch_dedup_body(p, sh, nworkers);
  __syncthreads();
  expert_dedup_body<T>(p, nworkers);  // leaves the dynamic shared memory alone: the slot table stays intact
  __syncthreads();
  combine_dedup_body<T>(p, sh + 32);
}

// --------------------------------------------------------------- small utils ----
__global__ void wait_flags_kernel(const uint32_t* flags, int n, int stride_words, uint32_t want, uint64_t limit_ns,
                                  uint32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    if (!kb::wait_flag_ge(flags + static_cast<size_t>(i) * stride_words, want, limit_ns)) {
      kb::report_status(status, KB_DEV_TIMEOUT_FLAG, 21u, (uint32_t)i, want);
    }
  }
}

struct BarrierParams {
  char* peer_base[KB_MAX_WORLD];
};
__global__ void device_barrier_kernel(const BarrierParams bp, uint64_t pad_off, int rank, int world, uint32_t epoch,
                                      uint64_t limit_ns, uint32_t* status) {
  const int i = threadIdx.x;
  if (i < world) {
    kb::fence_sys();
    kb::st_release_sys_u32(reinterpret_cast<uint32_t*>(bp.peer_base[i] + pad_off) + rank, epoch);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(bp.peer_base[rank] + pad_off) + i;
    if (!kb::wait_flag_ge(mine, epoch, limit_ns)) {
      kb::report_status(status, KB_DEV_TIMEOUT_FLAG, 22u, (uint32_t)i, epoch);
    }
  }
}

// Tells every rank that this rank's expert outputs of `epoch` are in place
// (phase-1 flag), for callers that ran their own expert computation between
// kb_a2a_dispatch and kb_a2a_combine.
__global__ void post_ready_kernel(const A2aParams p) {
  const int i = threadIdx.x;
  if (i < p.world) {
    kb::fence_sys();
    kb::st_release_sys_u32(flag_ptr(p, i, 1, p.rank), p.epoch);
  }
}

// Dynamic shared memory of a kernel that runs the dispatch phase: the five tables,
// alignment slack, two row buffers, two mbarriers.
size_t dispatch_smem_bytes(int experts) {
  return static_cast<size_t>(table_ints(experts)) * sizeof(int32_t) + 128 + 2 * ROWBUF_BYTES + 16;
}

int fill_params(const KbA2aArgs* a, A2aParams* p, int sms) {
  if (a == nullptr) return KB_ERR_ARG;
  if (a->world < 1 || a->world > KB_MAX_WORLD || a->rank < 0 || a->rank >= a->world) {
    kb::set_error("a2a: bad rank/world %d/%d", a->rank, a->world);
    return KB_ERR_ARG;
  }
  if (a->num_experts <= 0 || a->num_experts > MAX_EXPERTS || a->num_experts % a->world != 0) {
    kb::set_error("a2a: num_experts=%d must be in (0,%d] and divisible by world=%d", a->num_experts, MAX_EXPERTS,
                  a->world);
    return KB_ERR_ARG;
  }
  if (a->num_tokens < 0 || a->num_tokens > a->max_tokens || a->topk <= 0 || a->topk > 64) {
    kb::set_error("a2a: num_tokens=%d (max %d), topk=%d out of range", a->num_tokens, a->max_tokens, a->topk);
    return KB_ERR_ARG;
  }
  const long long row_bytes = static_cast<long long>(a->hidden) * a->elem_bytes;
  if (a->hidden <= 0 || row_bytes % 16 != 0) {
    kb::set_error("a2a: hidden*elem_bytes=%lld must be a positive multiple of 16", row_bytes);
    return KB_ERR_ARG;
  }
  auto misaligned = [](const void* q, uintptr_t to) { return (reinterpret_cast<uintptr_t>(q) & (to - 1)) != 0; };
  if (misaligned(a->x, 16) || misaligned(a->out, 16) || misaligned(a->indices, 4) || misaligned(a->weights, 4) ||
      misaligned(a->slots, 4)) {
    kb::set_error("a2a: x and out must be 16-byte aligned, indices, weights and slots 4-byte aligned");
    return KB_ERR_ARG;
  }
  memset(p, 0, sizeof(*p));
  p->rank = a->rank;
  p->world = a->world;
  p->E = a->num_experts;
  p->El = a->num_experts / a->world;
  p->k = a->topk;
  p->H = a->hidden;
  p->T = a->num_tokens;
  p->cap = a->max_tokens * a->topk;
  p->row_bytes = static_cast<int>(row_bytes);
  p->vecs = static_cast<int>(row_bytes / 16);
  p->x = static_cast<const uint8_t*>(a->x);
  p->idx = a->indices;
  p->w = a->weights;
  p->out = static_cast<uint8_t*>(a->out);
  p->slots = a->slots;
  p->epoch = a->epoch;
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_base[r] == nullptr) {
      kb::set_error("a2a: peer_base[%d] is null", r);
      return KB_ERR_ARG;
    }
    p->peer_base[r] = static_cast<char*>(a->peer_base[r]);
  }
  p->recv_off = a->recv_off;
  p->y_off = a->y_off;
  p->count_off = a->count_off;
  p->flag_off = a->flag_off;
  p->sync_off = a->sync_off;
  p->scale_mode = a->scale_mode;
  p->status = a->status;
  p->limit_ns = a->wait_limit_ns ? a->wait_limit_ns : 2000000000ull;
  p->trace = a->trace;
  p->tmax = a->max_tokens;
  p->meta_off = a->meta_off;
  p->rank_slots = a->rank_slots;
  p->ll_off = a->ll_off;
  p->ll_tmax = a->ll_max_tokens;
  {
    static const int bulk_min = [] {
      const char* v = getenv("KB200_A2A_BULK");  // 0: ordinary loads and stores only
      return (v != nullptr && v[0] == '0') ? 0x7fffffff : BULK_MIN_BYTES;
    }();
    p->bulk_min_bytes = bulk_min;
  }
  // Work split: one unit per CTA, about two CTAs per SM (two slots stay free:
  // one for the poller CTA of the fused launch).  Units are token groups; with
  // few tokens every group is further split along the hidden dimension so that
  // more SMs take part.
  const int target = 2 * sms - 2 > 1 ? 2 * sms - 2 : 1;
  const int T = p->T > 0 ? p->T : 1;
  int tg = T < target ? T : target;
  // A CTA ranks the (tokens per group) * k entries of its group in a buffer of
  // MAX_ENT_PER_CTA words: the group count must keep ceil(T / tg) * k inside it.
  const int max_tok_per = MAX_ENT_PER_CTA / p->k;  // k <= 64, so at least 32
  const int min_tg = (T + max_tok_per - 1) / max_tok_per;
  if (tg < min_tg) tg = min_tg;
  int hs = target / tg;
  if (hs < 1) hs = 1;
  const int max_hs = (p->vecs + 31) / 32;  // at least a warp's worth of vectors per unit
  if (hs > max_hs) hs = max_hs;
  p->tok_groups = tg;
  p->h_splits = hs;
  return KB_OK;
}

// Function attributes and occupancy belong to a device's context, and a process may
// use several devices in its life (a pool worker that serves rank 3 in one case and
// rank 5 in the next): everything cached about a kernel is cached per device.
constexpr int MAX_DEVICES = 64;
int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return -1;
  return dev;
}

int device_sms(int* sms) {
  static int cached[64] = {0};
  int dev = 0;
  KB_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && cached[dev] > 0) {
    *sms = cached[dev];
    return KB_OK;
  }
  KB_CUDA_OK(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
  if (dev >= 0 && dev < 64) cached[dev] = *sms;
  return KB_OK;
}

}  // namespace

extern "C" uint64_t kb_a2a_flag_bytes(void) { return 2ull * KB_MAX_WORLD * FLAG_STRIDE_WORDS * 4; }
extern "C" uint64_t kb_a2a_sync_bytes(void) { return 512; }
extern "C" int kb_a2a_flag_stride_words(void) { return FLAG_STRIDE_WORDS; }

extern "C" uint64_t kb_a2a_meta_bytes(int world, int max_tokens, int topk) {
  const uint64_t b = (uint64_t)world * max_tokens * (2 * topk + 2) * 4;
  return (b + 255) / 256 * 256;
}

extern "C" int kb_a2a_ll_max_tokens(void) { return LL_MAX_TOKENS; }
extern "C" uint64_t kb_a2a_ll_bytes(int world, int max_tokens, int topk, int hidden, int elem_bytes) {
  if (max_tokens > LL_MAX_TOKENS) return 0;
  const uint64_t b = ll_region_bytes(world, max_tokens, topk, hidden * elem_bytes);
  return (b + 255) / 256 * 256;
}

extern "C" uint64_t kb_a2a_rows_bytes(int world, int max_tokens, int topk, int hidden, int elem_bytes) {
  const uint64_t b = (uint64_t)world * max_tokens * topk * hidden * elem_bytes;
  return (b + 255) / 256 * 256;
}

extern "C" int kb_a2a_dispatch(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  const size_t smem = dispatch_smem_bytes(p.E);
  static bool attr_set[MAX_DEVICES] = {};
  const int slot = current_device_slot();
  if (slot < 0 || !attr_set[slot]) {
    KB_CUDA_OK(cudaFuncSetAttribute(a2a_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dispatch_smem_bytes(MAX_EXPERTS)));
    if (slot >= 0) attr_set[slot] = true;
  }
  a2a_dispatch_kernel<<<p.tok_groups * p.h_splits, A2A_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

extern "C" int kb_a2a_post_ready(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  post_ready_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

extern "C" int kb_a2a_expert_scale(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  const size_t smem = p.E * sizeof(int32_t);
  const int grid = a->num_ctas > 0 ? a->num_ctas : 2 * sms;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case 0: a2a_expert_kernel<__nv_bfloat16><<<grid, A2A_THREADS, smem, st>>>(p); break;
    case 1: a2a_expert_kernel<__half><<<grid, A2A_THREADS, smem, st>>>(p); break;
    case 2: a2a_expert_kernel<float><<<grid, A2A_THREADS, smem, st>>>(p); break;
    default: kb::set_error("a2a: unknown dtype %d", a->dtype); return KB_ERR_ARG;
  }
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

extern "C" int kb_a2a_combine(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  const int want = p.tok_groups * p.h_splits;
  const size_t smem = 2 * MAX_ENT_PER_CTA * sizeof(int32_t);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case 0: a2a_combine_kernel<__nv_bfloat16><<<want, A2A_THREADS, smem, st>>>(p); break;
    case 1: a2a_combine_kernel<__half><<<want, A2A_THREADS, smem, st>>>(p); break;
    case 2: a2a_combine_kernel<float><<<want, A2A_THREADS, smem, st>>>(p); break;
    default: kb::set_error("a2a: unknown dtype %d", a->dtype); return KB_ERR_ARG;
  }
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

template <typename T>
static int launch_fused(const A2aParams& p, int sms, cudaStream_t st) {
  if (p.meta_off == 0 || p.rank_slots == nullptr) {
    kb::set_error("a2a fused: the workspace has no per-rank metadata region (meta_off, rank_slots)");
    return KB_ERR_UNSUPPORTED;
  }
  {
    const int tok_per = ((p.T > 0 ? p.T : 1) + p.tok_groups - 1) / p.tok_groups;
    if (tok_per * p.world > DEDUP_MAX_SLOTS) {
      kb::set_error("a2a fused: %d tokens per CTA x %d ranks exceed the slot table", tok_per, p.world);
      return KB_ERR_UNSUPPORTED;
    }
  }
  const size_t smem = dispatch_smem_bytes(p.E);  // the combine phase reuses the slot table at the front of it
  static bool attr_set[MAX_DEVICES] = {};
  const int slot = current_device_slot();
  if (slot < 0 || !attr_set[slot]) {
    KB_CUDA_OK(cudaFuncSetAttribute(a2a_fused_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dispatch_smem_bytes(MAX_EXPERTS)));
    if (slot >= 0) attr_set[slot] = true;
  }
  // The occupancy query costs microseconds of host time; its answer depends only
  // on the device, the kernel instance and the shared-memory size.
  static size_t cached_smem[MAX_DEVICES];
  static int cached_per_sm[MAX_DEVICES] = {};
  int per_sm = 0;
  if (slot >= 0 && cached_per_sm[slot] > 0 && cached_smem[slot] == smem) {
    per_sm = cached_per_sm[slot];
  } else {
    KB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a2a_fused_kernel<T>, A2A_THREADS, smem));
    if (slot >= 0) {
      cached_smem[slot] = smem;
      cached_per_sm[slot] = per_sm;
    }
  }
  const int units = p.tok_groups * p.h_splits + 1;  // data CTAs and the poller
  if (per_sm < 1 || units > per_sm * sms) {
    kb::set_error("a2a fused: %d CTAs cannot be co-resident (%d per SM)", units, per_sm);
    return KB_ERR_UNSUPPORTED;
  }
  A2aParams copy = p;
  void* args[] = {&copy};
  KB_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(a2a_fused_kernel<T>), dim3(units), dim3(A2A_THREADS),
                                         args, smem, st));
  return KB_OK;
}

// The low-latency kernel's CTAs poll data that other CTAs of peer ranks produce only after
// they themselves have been served by this rank: all of them must be resident.
template <typename T>
static int launch_ll(const A2aParams& p, int sms, cudaStream_t st) {
  static int cached_per_sm[MAX_DEVICES] = {};
  const int slot = current_device_slot();
  int per_sm = slot >= 0 ? cached_per_sm[slot] : 0;
  if (per_sm == 0) {
    KB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a2a_ll_kernel<T>, A2A_THREADS, 0));
    if (slot >= 0) cached_per_sm[slot] = per_sm;
  }
  const int units = p.tok_groups * p.h_splits;
  if (per_sm < 1 || units > per_sm * sms) {
    kb::set_error("a2a low-latency: %d CTAs cannot be co-resident (%d per SM)", units, per_sm);
    return KB_ERR_UNSUPPORTED;
  }
  A2aParams copy = p;
  void* args[] = {&copy};
  KB_CUDA_OK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(a2a_ll_kernel<T>), dim3(units), dim3(A2A_THREADS), args, 0, st));
  return KB_OK;
}

extern "C" int kb_a2a_round_trip(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The choice must be the same on every rank, so it depends on the context's capacity, not on this call's tokens.
  if (p.ll_off != 0 && p.ll_tmax >= p.tmax && p.tmax <= LL_MAX_TOKENS && p.T <= p.ll_tmax) {
    switch (a->dtype) {
      case 0: return launch_ll<__nv_bfloat16>(p, sms, st);
      case 1: return launch_ll<__half>(p, sms, st);
      case 2: return launch_ll<float>(p, sms, st);
    }
  }
  switch (a->dtype) {
    case 0: return launch_fused<__nv_bfloat16>(p, sms, st);
    case 1: return launch_fused<__half>(p, sms, st);
    case 2: return launch_fused<float>(p, sms, st);
  }
  kb::set_error("a2a: unknown dtype %d", a->dtype);
  return KB_ERR_ARG;
}

extern "C" int kb_wait_flags(const uint32_t* flags, int n, int stride_words, uint32_t want, uint64_t limit_ns,
                             uint32_t* status, void* stream) {
  if (n <= 0) return KB_OK;
  if (stride_words < 1) return KB_ERR_ARG;
  wait_flags_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(flags, n, stride_words, want, limit_ns,
                                                                                   status);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

extern "C" int kb_device_barrier(void* const* peer_bases, uint64_t pad_off, int rank, int world, uint32_t epoch,
                                 uint64_t limit_ns, uint32_t* status, void* stream) {
  if (world < 1 || world > KB_MAX_WORLD) return KB_ERR_ARG;
  BarrierParams bp;
  for (int i = 0; i < KB_MAX_WORLD; ++i) bp.peer_base[i] = i < world ? static_cast<char*>(peer_bases[i]) : nullptr;
  device_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(bp, pad_off, rank, world, epoch, limit_ns,
                                                                        status);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

// ------------------------------------------------- allocation-free entry point ----
// See a2a_static.h.  The workspace lives in a file-scope device array; host code
// must not pass the array's name to a kernel (on the host it is only a stand-in
// for the symbol), so its device address is looked up once per device.
#include <mutex>

#include "a2a_static.h"

static __device__ __align__(256) unsigned char g_a2a_static_scratch[KB_A2A_STATIC_BYTES];

namespace {
struct StaticSlot {
  unsigned char* base = nullptr;
  uint32_t epoch = 0;
};
StaticSlot g_static_slots[64];
std::mutex g_static_mu;  // guards g_static_slots (address look-up and epoch numbering)

// Layout inside the array (all offsets multiples of 256).
constexpr uint64_t ST_RECV_OFF = 0;
constexpr uint64_t ST_Y_OFF = KB_A2A_STATIC_ROW_BYTES;
constexpr uint64_t ST_SLOTS_OFF = 2ull * KB_A2A_STATIC_ROW_BYTES;
constexpr uint64_t ST_COUNT_OFF = ST_SLOTS_OFF + 4ull * KB_A2A_STATIC_MAX_ROWS;
constexpr uint64_t ST_FLAG_OFF = ST_COUNT_OFF + 4ull * KB_A2A_STATIC_MAX_EXPERTS;
constexpr uint64_t ST_SYNC_OFF = ST_FLAG_OFF + 2ull * KB_MAX_WORLD * FLAG_STRIDE_WORDS * 4;
constexpr uint64_t ST_STATUS_OFF = ST_SYNC_OFF + 512;
static_assert(ST_STATUS_OFF + 256 <= KB_A2A_STATIC_BYTES, "static workspace layout exceeds the array");

// Device index and workspace address of the current device (set-up on first use).
int static_slot(int* dev_out, unsigned char** base_out, bool next_epoch, uint32_t* epoch_out) {
  int dev = 0;
  KB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    kb::set_error("a2a static: device index %d out of range", dev);
    return KB_ERR_ARG;
  }
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticSlot& slot = g_static_slots[dev];
  if (slot.base == nullptr) {
    // Set-up, once per device, with that device current.
    unsigned char* ptr = nullptr;
    KB_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_a2a_static_scratch));
    slot.base = ptr;
  }
  if (next_epoch) ++slot.epoch;  // flags keep the previous call's epoch; epochs only grow
  if (epoch_out != nullptr) *epoch_out = slot.epoch;
  *dev_out = dev;
  *base_out = slot.base;
  return KB_OK;
}
}  // namespace

extern "C" int kb_a2a_round_trip_static(const void* x, const int32_t* indices, const float* weights, void* out,
                                        int num_tokens, int num_experts, int topk, int hidden, int dtype,
                                        int scale_mode, void* stream) {
  const int elem_bytes = (dtype == 2) ? 4 : 2;
  if (dtype < 0 || dtype > 2 || x == nullptr || indices == nullptr || weights == nullptr || out == nullptr) {
    kb::set_error("a2a static: null pointer or unknown dtype %d", dtype);
    return KB_ERR_ARG;
  }
  if (num_tokens < 0 || topk <= 0 || hidden <= 0 || num_experts <= 0) {
    kb::set_error("a2a static: sizes must be positive");
    return KB_ERR_ARG;
  }
  const unsigned long long rows = static_cast<unsigned long long>(num_tokens > 0 ? num_tokens : 1) * topk;
  const unsigned long long row_bytes = rows * hidden * elem_bytes;
  if (row_bytes > KB_A2A_STATIC_ROW_BYTES || rows > KB_A2A_STATIC_MAX_ROWS || num_experts > KB_A2A_STATIC_MAX_EXPERTS) {
    kb::set_error(
        "a2a static: request exceeds the built-in workspace (tokens*topk*hidden*elem = %llu > %u bytes, or rows %llu > %d, "
        "or experts %d > %d); use the regular entry points with an allocated workspace",
        row_bytes, KB_A2A_STATIC_ROW_BYTES, rows, KB_A2A_STATIC_MAX_ROWS, num_experts, KB_A2A_STATIC_MAX_EXPERTS);
    return KB_ERR_ARG;
  }
  int dev = 0;
  unsigned char* base = nullptr;
  uint32_t epoch = 0;
  int rc = static_slot(&dev, &base, true, &epoch);
  if (rc != KB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // The block counters must start at zero (a call that was cut short could have
  // left them elsewhere).  The status words are NOT cleared here: a failure stays
  // readable through kb_a2a_static_status until that call clears it.
  KB_CUDA_OK(cudaMemsetAsync(base + ST_SYNC_OFF, 0, 512, st));

  KbA2aArgs a;
  memset(&a, 0, sizeof(a));
  a.rank = 0;
  a.world = 1;
  a.num_experts = num_experts;
  a.topk = topk;
  a.hidden = hidden;
  a.max_tokens = num_tokens > 0 ? num_tokens : 1;
  a.num_tokens = num_tokens;
  a.elem_bytes = elem_bytes;
  a.dtype = dtype;
  a.x = x;
  a.indices = indices;
  a.weights = weights;
  a.out = out;
  a.slots = reinterpret_cast<int32_t*>(base + ST_SLOTS_OFF);
  a.epoch = epoch;
  a.peer_base[0] = base;
  a.recv_off = ST_RECV_OFF;
  a.y_off = ST_Y_OFF;
  a.count_off = ST_COUNT_OFF;
  a.flag_off = ST_FLAG_OFF;
  a.sync_off = ST_SYNC_OFF;
  a.scale_mode = scale_mode;
  a.status = reinterpret_cast<uint32_t*>(base + ST_STATUS_OFF);
  a.wait_limit_ns = 2000000000ull;
  rc = kb_a2a_dispatch(&a, st);
  if (rc != KB_OK) return rc;
  rc = kb_a2a_expert_scale(&a, st);
  if (rc != KB_OK) return rc;
  return kb_a2a_combine(&a, st);
}

extern "C" int kb_a2a_static_status(uint32_t* out8, int clear, void* stream) {
  if (out8 == nullptr) {
    kb::set_error("a2a static: status destination is null");
    return KB_ERR_ARG;
  }
  int dev = 0;
  unsigned char* base = nullptr;
  int rc = static_slot(&dev, &base, false, nullptr);
  if (rc != KB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  KB_CUDA_OK(cudaMemcpyAsync(out8, base + ST_STATUS_OFF, 8 * sizeof(uint32_t), cudaMemcpyDefault, st));
  if (clear) KB_CUDA_OK(cudaMemsetAsync(base + ST_STATUS_OFF, 0, 8 * sizeof(uint32_t), st));
  return KB_OK;
}
