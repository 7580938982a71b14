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

#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../include/kb200.h"

namespace {

constexpr int A2A_THREADS = 256;
constexpr int MAX_EXPERTS = 1024;
constexpr int MAX_ENT_PER_CTA = 2048;

enum Site : uint32_t { SITE_DISP_IDX = 11, SITE_EXP_FLAG = 12, SITE_COMB_FLAG = 13, SITE_COMB_SLOT = 14 };

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
};

// Phase stamps (nanoseconds of the global timer) written by thread 0 of CTA 0.
enum Stamp { ST_ENTRY = 0, ST_SLOTS = 1, ST_PUSHED = 2, ST_DISPATCH_FLAG = 3, ST_EXPERT_GO = 4, ST_COUNTS = 5, ST_EXPERT_ROWS = 6,
             ST_EXPERT_FLAG = 7, ST_COMBINE_GO = 8, ST_DONE = 9 };
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
  return reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off) + which * p.world + src;
}

// Last-block-done: returns true in exactly one CTA (the last to arrive) once
// the writes of all CTAs are ordered before it.
__device__ __forceinline__ bool last_block_done(uint32_t* counter, uint32_t total) {
  __shared__ uint32_t s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    kb::fence_sys();
    const uint32_t old = atomicAdd(counter, 1u);
    s_last = (old == total - 1u) ? 1u : 0u;
    if (s_last) {
      *counter = 0u;  // ready for the next launch
      kb::fence_sys();
    }
  }
  __syncthreads();
  return s_last != 0u;
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
  if (blockIdx.x >= p.tok_groups * p.h_splits) {  // surplus CTAs of a fused launch
    t0 = t1 = p.T;
    v0 = v1 = 0;
  }
}

__device__ __forceinline__ void dispatch_body(const A2aParams& p, int32_t* sh) {
  int32_t* tot = sh;               // [E] entries per expert, whole rank
  int32_t* pre = tot + p.E;        // [E] entries per expert before this CTA's tokens
  int32_t* off = pre + p.E;        // [E] first slot of the expert inside its owner's region
  int32_t* ent_e = off + p.E;      // [MAX_ENT_PER_CTA]
  int32_t* ent_slot = ent_e + MAX_ENT_PER_CTA;

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
  for (int i = tid; i < total_ent; i += blockDim.x) {
    const int e = p.idx[i];
    if (e < 0 || e >= p.E) {
      kb::report_status(p.status, KB_DEV_BAD_INDEX, SITE_DISP_IDX, (uint32_t)i, p.epoch);
      continue;
    }
    atomicAdd(&tot[e], 1);
    if (i < t0 * p.k) atomicAdd(&pre[e], 1);
  }
  __syncthreads();
  for (int e = tid; e < p.E; e += blockDim.x) {
    const int first = (e / p.El) * p.El;
    int acc = 0;
    for (int j = first; j < e; ++j) acc += tot[j];
    off[e] = acc;
  }
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
  stamp(p, ST_PUSHED);
  // Per-(source, expert) counts for every destination.
  if (blockIdx.x == 0) {
    for (int e = tid; e < p.E; e += blockDim.x) {
      counts_ptr(p, e / p.El, p.rank)[e % p.El] = tot[e];
    }
  }
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  if (last_block_done(&sync[0], gridDim.x)) {
    if (tid < p.world) kb::st_release_sys_u32(flag_ptr(p, tid, 0, p.rank), p.epoch);  // threads other than 0 need their own release
  }
  stamp(p, ST_DISPATCH_FLAG);
}

__global__ void __launch_bounds__(A2A_THREADS) a2a_dispatch_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  dispatch_body(p, sh);
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

template <typename T>
__device__ __forceinline__ void expert_body(const A2aParams& p, int32_t* sh) {
  int32_t* incl = sh;                        // [world][El] inclusive prefix of counts per source
  int32_t* src_end = incl + p.world * p.El;  // [world] inclusive prefix of per-source totals
  const int tid = threadIdx.x;

  if (tid < p.world) {
    if (!kb::wait_flag_ge(flag_ptr(p, p.rank, 0, tid), p.epoch, p.limit_ns)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)tid, p.epoch);
    }
  }
  __syncthreads();
  stamp(p, ST_EXPERT_GO);
  // All counts are fetched in parallel (one independent load per thread), then
  // scanned in shared memory.
  const int32_t* counts = counts_ptr(p, p.rank, 0);
  for (int i = tid; i < p.world * p.El; i += blockDim.x) {
    int v = static_cast<int>(kb::ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + i)));
    incl[i] = v < 0 ? 0 : v;
  }
  __syncthreads();
  if (tid < p.world) {
    int acc = 0;
    for (int le = 0; le < p.El; ++le) {
      acc += incl[tid * p.El + le];
      if (acc > p.cap) acc = p.cap;
      incl[tid * p.El + le] = acc;
    }
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int s = 0; s < p.world; ++s) {
      acc += incl[s * p.El + p.El - 1];
      src_end[s] = acc;
    }
  }
  __syncthreads();
  stamp(p, ST_COUNTS);
  const int total_rows = src_end[p.world - 1];
  for (int g = blockIdx.x; g < total_rows; g += gridDim.x) {
    int s = 0;
    while (src_end[s] <= g) ++s;
    const int row = g - (s ? src_end[s - 1] : 0);
    // first local expert whose inclusive prefix exceeds row
    int lo = 0, hi = p.El - 1;
    const int32_t* in = incl + s * p.El;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (in[mid] > row) hi = mid; else lo = mid + 1;
    }
    float scale = 1.0f;
    if (p.scale_mode == 1) scale = static_cast<float>(1 + p.rank);
    if (p.scale_mode == 2) scale = static_cast<float>(p.rank * p.El + lo + 1) / static_cast<float>(p.E);
    const uint4* src = reinterpret_cast<const uint4*>(rows_ptr(p, p.rank, p.recv_off, s, row));
    uint4* dst = reinterpret_cast<uint4*>(rows_ptr(p, p.rank, p.y_off, s, row));
    for (int vb = tid; vb < p.vecs; vb += 4 * blockDim.x) {
      uint4 in[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {  // all loads of this thread first: one latency per row
        const int v = vb + u * blockDim.x;
        if (v < p.vecs) in[u] = kb::ld_sys_v4(src + v);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = vb + u * blockDim.x;
        if (v < p.vecs) {
          float f[Vec16<T>::N];
          Vec16<T>::load(in[u], f);
#pragma unroll
          for (int i = 0; i < Vec16<T>::N; ++i) f[i] *= scale;
          dst[v] = Vec16<T>::store(f);
        }
      }
    }
  }
  stamp(p, ST_EXPERT_ROWS);
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  if (last_block_done(&sync[1], gridDim.x)) {
    if (tid < p.world) kb::st_release_sys_u32(flag_ptr(p, tid, 1, p.rank), p.epoch);
  }
  stamp(p, ST_EXPERT_FLAG);
}

template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_expert_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  expert_body<T>(p, sh);
}

// ------------------------------------------------------------------- combine ----
template <typename T>
__device__ __forceinline__ void combine_body(const A2aParams& p) {
  const int tid = threadIdx.x;
  if (tid < p.world) {
    if (!kb::wait_flag_ge(flag_ptr(p, p.rank, 1, tid), p.epoch, p.limit_ns)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_COMB_FLAG, (uint32_t)tid, p.epoch);
    }
  }
  __syncthreads();
  stamp(p, ST_COMBINE_GO);
  int t0, t1, v0, v1, hs;
  unit_ranges(p, t0, t1, v0, v1, hs);
  for (int t = t0; t < t1; ++t) {
    for (int v = v0 + tid; v < v1; v += blockDim.x) {
      float acc[Vec16<T>::N];
#pragma unroll
      for (int i = 0; i < Vec16<T>::N; ++i) acc[i] = 0.f;
      for (int k0 = 0; k0 < p.k; k0 += 8) {
        uint4 u[8];
        float wk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int kk = k0 + j;
          wk[j] = 0.f;
          u[j] = make_uint4(0, 0, 0, 0);
          if (kk < p.k) {
            const int e = p.idx[t * p.k + kk];
            const int slot = p.slots[t * p.k + kk];
            if (e >= 0 && e < p.E && slot >= 0 && slot < p.cap) {
              wk[j] = p.w[t * p.k + kk];
              u[j] = kb::ld_sys_v4(reinterpret_cast<const uint4*>(rows_ptr(p, e / p.El, p.y_off, p.rank, slot)) + v);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float f[Vec16<T>::N];
          Vec16<T>::load(u[j], f);
#pragma unroll
          for (int i = 0; i < Vec16<T>::N; ++i) acc[i] = fmaf(wk[j], f[i], acc[i]);
        }
      }
      reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.row_bytes)[v] = Vec16<T>::store(acc);
    }
  }
  stamp(p, ST_DONE);
}

template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_combine_kernel(const A2aParams p) {
  combine_body<T>(p);
}

// All three phases in one cooperative launch: the phases are separated only by
// the epoch flags (this rank's own flag doubles as the grid-wide barrier), so
// the two extra launches and their gaps disappear.  Needs every CTA resident,
// which the cooperative launch guarantees.
template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_fused_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  dispatch_body(p, sh);
  __syncthreads();
  expert_body<T>(p, sh);
  __syncthreads();
  combine_body<T>(p);
}

// --------------------------------------------------------------- small utils ----
__global__ void wait_flags_kernel(const uint32_t* flags, int n, uint32_t want, uint64_t limit_ns, uint32_t* status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    if (!kb::wait_flag_ge(flags + i, want, limit_ns)) {
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
  // Work split: one unit per CTA, about two CTAs per SM.  Units are token
  // groups; with few tokens every group is further split along the hidden
  // dimension so that more SMs take part.
  const int target = 2 * sms;
  const int T = p->T > 0 ? p->T : 1;
  int tg = T < target ? T : target;
  const int min_tg = (T * p->k + MAX_ENT_PER_CTA - 1) / MAX_ENT_PER_CTA;
  if (tg < min_tg) tg = min_tg;
  if (tg > T) {
    kb::set_error("a2a: topk=%d too large for the per-CTA ranking buffer", p->k);
    return KB_ERR_ARG;
  }
  int hs = target / tg;
  if (hs < 1) hs = 1;
  const int max_hs = (p->vecs + 31) / 32;  // at least a warp's worth of vectors per unit
  if (hs > max_hs) hs = max_hs;
  p->tok_groups = tg;
  p->h_splits = hs;
  return KB_OK;
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
  const size_t smem = (3 * p.E + 2 * MAX_ENT_PER_CTA) * sizeof(int32_t);
  a2a_dispatch_kernel<<<p.tok_groups * p.h_splits, A2A_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
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
  const size_t smem = (p.world * p.El + p.world) * sizeof(int32_t);
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case 0: a2a_combine_kernel<__nv_bfloat16><<<want, A2A_THREADS, 0, st>>>(p); break;
    case 1: a2a_combine_kernel<__half><<<want, A2A_THREADS, 0, st>>>(p); break;
    case 2: a2a_combine_kernel<float><<<want, A2A_THREADS, 0, st>>>(p); break;
    default: kb::set_error("a2a: unknown dtype %d", a->dtype); return KB_ERR_ARG;
  }
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

template <typename T>
static int launch_fused(const A2aParams& p, int sms, cudaStream_t st) {
  const size_t smem_d = (3 * p.E + 2 * MAX_ENT_PER_CTA) * sizeof(int32_t);
  const size_t smem_e = (p.world * p.El + p.world) * sizeof(int32_t);
  const size_t smem = smem_d > smem_e ? smem_d : smem_e;
  // The occupancy query costs microseconds of host time; its answer depends only
  // on the kernel instance and the shared-memory size.
  static size_t cached_smem = ~size_t(0);
  static int cached_per_sm = 0;
  int per_sm = cached_per_sm;
  if (cached_smem != smem) {
    KB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, a2a_fused_kernel<T>, A2A_THREADS, smem));
    cached_smem = smem;
    cached_per_sm = per_sm;
  }
  const int units = p.tok_groups * p.h_splits;
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

extern "C" int kb_a2a_round_trip(const KbA2aArgs* a, void* stream) {
  int sms = 0;
  int rc = device_sms(&sms);
  if (rc != KB_OK) return rc;
  A2aParams p;
  rc = fill_params(a, &p, sms);
  if (rc != KB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case 0: return launch_fused<__nv_bfloat16>(p, sms, st);
    case 1: return launch_fused<__half>(p, sms, st);
    case 2: return launch_fused<float>(p, sms, st);
  }
  kb::set_error("a2a: unknown dtype %d", a->dtype);
  return KB_ERR_ARG;
}

extern "C" int kb_wait_flags(const uint32_t* flags, int n, uint32_t want, uint64_t limit_ns, uint32_t* status,
                             void* stream) {
  if (n <= 0) return KB_OK;
  wait_flags_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(flags, n, want, limit_ns, status);
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
#include "a2a_static.h"

static __device__ __align__(256) unsigned char g_a2a_static_scratch[KB_A2A_STATIC_BYTES];

namespace {
struct StaticSlot {
  unsigned char* base = nullptr;
  uint32_t epoch = 0;
};
StaticSlot g_static_slots[64];
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
  KB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) {
    kb::set_error("a2a static: device index %d out of range", dev);
    return KB_ERR_ARG;
  }
  StaticSlot& slot = g_static_slots[dev];
  if (slot.base == nullptr) {
    // Set-up, once per device, with that device current.
    unsigned char* ptr = nullptr;
    KB_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_a2a_static_scratch));
    slot.base = ptr;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  // Layout inside the array (all offsets multiples of 256).
  const uint64_t recv_off = 0;
  const uint64_t y_off = KB_A2A_STATIC_ROW_BYTES;
  const uint64_t slots_off = 2ull * KB_A2A_STATIC_ROW_BYTES;
  const uint64_t count_off = slots_off + 4ull * KB_A2A_STATIC_MAX_ROWS;
  const uint64_t flag_off = count_off + 4ull * KB_A2A_STATIC_MAX_EXPERTS;
  const uint64_t sync_off = flag_off + 256;
  const uint64_t status_off = sync_off + 256;

  // The block counters must start at zero (a call that was cut short could have
  // left them elsewhere); the status words are cleared for this call.
  KB_CUDA_OK(cudaMemsetAsync(slot.base + sync_off, 0, 512, st));

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
  a.slots = reinterpret_cast<int32_t*>(slot.base + slots_off);
  a.epoch = ++slot.epoch;  // flags keep the previous call's epoch; epochs only grow
  a.peer_base[0] = slot.base;
  a.recv_off = recv_off;
  a.y_off = y_off;
  a.count_off = count_off;
  a.flag_off = flag_off;
  a.sync_off = sync_off;
  a.scale_mode = scale_mode;
  a.status = reinterpret_cast<uint32_t*>(slot.base + status_off);
  a.wait_limit_ns = 2000000000ull;
  int rc = kb_a2a_dispatch(&a, st);
  if (rc != KB_OK) return rc;
  rc = kb_a2a_expert_scale(&a, st);
  if (rc != KB_OK) return rc;
  return kb_a2a_combine(&a, st);
}
