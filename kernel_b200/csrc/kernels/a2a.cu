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
constexpr int MAX_ENT_PER_CTA = 512;

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
};

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
__global__ void __launch_bounds__(A2A_THREADS) a2a_dispatch_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  int32_t* tot = sh;               // [E] entries per expert, whole rank
  int32_t* pre = tot + p.E;        // [E] entries per expert before this CTA's tokens
  int32_t* off = pre + p.E;        // [E] first slot of the expert inside its owner's region
  int32_t* ent_e = off + p.E;      // [MAX_ENT_PER_CTA]
  int32_t* ent_slot = ent_e + MAX_ENT_PER_CTA;

  const int tid = threadIdx.x;
  const int tg = blockIdx.x, hs = blockIdx.y;
  const int tok_per = (p.T + p.tok_groups - 1) / p.tok_groups;
  const int t0 = min(tg * tok_per, p.T);
  const int t1 = min(t0 + tok_per, p.T);
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

  // Payload: one 16-byte vector per thread, read once, stored k times.
  const int v_per = (p.vecs + p.h_splits - 1) / p.h_splits;
  const int v0 = min(hs * v_per, p.vecs);
  const int v1 = min(v0 + v_per, p.vecs);
  for (int t = t0; t < t1; ++t) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.row_bytes);
    for (int v = v0 + tid; v < v1; v += blockDim.x) {
      const uint4 val = kb::ld_nc_v4(src + v);
      for (int kk = 0; kk < p.k; ++kk) {
        const int i = (t - t0) * p.k + kk;
        const int slot = ent_slot[i];
        if (slot < 0) continue;
        const int dst = ent_e[i] / p.El;
        uint4* d = reinterpret_cast<uint4*>(rows_ptr(p, dst, p.recv_off, p.rank, slot)) + v;
        kb::st_sys_v4(d, val);
      }
    }
  }
  // Per-(source, expert) counts for every destination.
  if (tg == 0 && hs == 0) {
    for (int e = tid; e < p.E; e += blockDim.x) {
      counts_ptr(p, e / p.El, p.rank)[e % p.El] = tot[e];
    }
  }
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  if (last_block_done(&sync[0], gridDim.x * gridDim.y)) {
    if (tid < p.world) kb::st_release_sys_u32(flag_ptr(p, tid, 0, p.rank), p.epoch);
  }
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
__global__ void __launch_bounds__(A2A_THREADS) a2a_expert_kernel(const A2aParams p) {
  extern __shared__ int32_t sh[];
  int32_t* incl = sh;                     // [world][El] inclusive prefix of counts per source
  int32_t* src_end = incl + p.world * p.El;  // [world] inclusive prefix of per-source totals
  const int tid = threadIdx.x;

  if (tid < p.world) {
    if (!kb::wait_flag_ge(flag_ptr(p, p.rank, 0, tid), p.epoch, p.limit_ns)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_EXP_FLAG, (uint32_t)tid, p.epoch);
    }
  }
  __syncthreads();
  for (int s = tid; s < p.world; s += blockDim.x) {
    const int32_t* c = counts_ptr(p, p.rank, s);
    int acc = 0;
    for (int le = 0; le < p.El; ++le) {
      int v = static_cast<int>(kb::ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(c + le)));
      if (v < 0) v = 0;
      acc += v;
      if (acc > p.cap) acc = p.cap;
      incl[s * p.El + le] = acc;
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
    for (int v = tid; v < p.vecs; v += blockDim.x) {
      float f[Vec16<T>::N];
      Vec16<T>::load(kb::ld_sys_v4(src + v), f);
#pragma unroll
      for (int i = 0; i < Vec16<T>::N; ++i) f[i] *= scale;
      dst[v] = Vec16<T>::store(f);
    }
  }
  uint32_t* sync = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.sync_off);
  if (last_block_done(&sync[1], gridDim.x)) {
    if (tid < p.world) kb::st_release_sys_u32(flag_ptr(p, tid, 1, p.rank), p.epoch);
  }
}

// ------------------------------------------------------------------- combine ----
template <typename T>
__global__ void __launch_bounds__(A2A_THREADS) a2a_combine_kernel(const A2aParams p) {
  const int tid = threadIdx.x;
  if (tid < p.world) {
    if (!kb::wait_flag_ge(flag_ptr(p, p.rank, 1, tid), p.epoch, p.limit_ns)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_COMB_FLAG, (uint32_t)tid, p.epoch);
    }
  }
  __syncthreads();
  const long long total = static_cast<long long>(p.T) * p.vecs;
  for (long long g = static_cast<long long>(blockIdx.x) * blockDim.x + tid; g < total;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(g / p.vecs);
    const int v = static_cast<int>(g - static_cast<long long>(t) * p.vecs);
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
  // Work split: enough CTAs to fill the machine about twice, token ranges
  // small enough for the in-CTA ranking, hidden split so that a thread owns
  // one vector of a row.
  const int target = 2 * sms;
  int hs = (p->vecs + A2A_THREADS - 1) / A2A_THREADS;
  if (hs < 1) hs = 1;
  int tg = (target + hs - 1) / hs;
  const int T = p->T > 0 ? p->T : 1;
  if (tg > T) tg = T;
  const int min_tg = (T * p->k + MAX_ENT_PER_CTA - 1) / MAX_ENT_PER_CTA;
  if (tg < min_tg) tg = min_tg;
  if (tg > T) {
    kb::set_error("a2a: topk=%d too large for the per-CTA ranking buffer", p->k);
    return KB_ERR_ARG;
  }
  // Few tokens: split rows finer so that more SMs take part.
  while (tg * hs < sms && hs * 2 * 32 <= p->vecs) hs *= 2;
  p->tok_groups = tg;
  p->h_splits = hs;
  return KB_OK;
}

int device_sms(int* sms) {
  int dev = 0;
  KB_CUDA_OK(cudaGetDevice(&dev));
  KB_CUDA_OK(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
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
  dim3 grid(p.tok_groups, p.h_splits);
  a2a_dispatch_kernel<<<grid, A2A_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(p);
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
  const long long total = static_cast<long long>(p.T) * p.vecs;
  long long want = (total + A2A_THREADS - 1) / A2A_THREADS;
  const long long cap = a->num_ctas > 0 ? a->num_ctas : 8LL * sms;
  if (want > cap) want = cap;
  if (want < 1) want = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (a->dtype) {
    case 0: a2a_combine_kernel<__nv_bfloat16><<<(int)want, A2A_THREADS, 0, st>>>(p); break;
    case 1: a2a_combine_kernel<__half><<<(int)want, A2A_THREADS, 0, st>>>(p); break;
    case 2: a2a_combine_kernel<float><<<(int)want, A2A_THREADS, 0, st>>>(p); break;
    default: kb::set_error("a2a: unknown dtype %d", a->dtype); return KB_ERR_ARG;
  }
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
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
