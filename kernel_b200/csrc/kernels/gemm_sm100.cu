// Persistent, warp-specialised bf16 GEMM for sm_100a with three epilogues:
//
//   PLAIN  out = A * B^T (+ bias)
//   RS     GEMM fused with reduce-scatter: every 128x256 tile is converted to
//          bf16 as it retires and its rows are stored straight into the row
//          owner's staging area over NVLink; the owner's own tiles run last
//          and their epilogue sums the peers' partials in fp32, adds the bias
//          and writes the output shard.  No collective library call, no
//          second kernel.
//   AG     all-gather fused with GEMM: extra "comm" warps of the same kernel
//          stream this rank's A rows into every peer's gather buffer while the
//          tensor cores already work on the rows that are present; the TMA
//          producer waits (bounded) on a per-row-block flag before it loads
//          rows that come from a peer.
//
// Mainloop: one TMA producer thread fills a 4-stage ring of 128x64 (A) and
// 256x64 (B) K-major tiles with 128-byte swizzle; one thread issues
// tcgen05.mma (M128 N256 K16) into one of two 256-column TMEM accumulators;
// four epilogue warps drain the other accumulator (tcgen05.ld -> bf16 ->
// swizzled smem -> 16-byte row-contiguous global accesses).
//
// The op replaces torch.matmul + bias add + reduce_scatter_tensor of the
// reference (gemm_rs/reference.py:49-60, gemm_rs/submission.py:23-28).
//
// TMA loads here are plain single-CTA loads from this GPU's own memory.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../include/kb200.h"

namespace {

using bf16 = __nv_bfloat16;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
// Single CTA: 128x256 tile, B stage = 256 rows, 4 stages of 48 KB.
// CTA pair (cta_group::2): 256x256 tile over two SMs, each CTA stages its 128
// rows of A and its 128 of the 256 B rows: 6 stages of 32 KB.
template <bool kPair>
struct Cfg {
  static constexpr int STAGES = kPair ? 6 : 4;
  static constexpr int B_ROWS = kPair ? 128 : 256;
  static constexpr int B_BYTES = B_ROWS * BK * 2;
};
constexpr int MAX_STAGES = 6;
constexpr int EPI_COLS = 128;                 // columns staged per epilogue pass
constexpr int EPI_ROW_BYTES = EPI_COLS * 2;   // 256
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int EPI_BYTES = 4 * EPI_WARP_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = 1024 + 4 * (A_BYTES + 32768) + EPI_BYTES + BAR_BYTES;  // same total for both configurations
constexpr int THREADS_BASE = 256;             // warps 0..3 control, 4..7 epilogue
constexpr int THREADS_AG = 384;               // + warps 8..11 comm

struct alignas(64) GemmParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmOwn;  // AG: this rank's own rows, read in place
  int mode, M, N, K;
  int MB, NB, KB;
  const bf16* bias;
  float bias_scale;
  bf16* out;
  int rank, world, rpo;
  uint32_t epoch;
  char* peer_base[KB_MAX_WORLD];
  uint64_t data_off, flag_off, counter_off;
  const bf16* a_local;
  uint32_t* status;
  uint64_t limit_ns;
  int own_lo_mb, own_hi_mb;
  int ag_parts;
  // Scheduling blocks: 128 rows (single CTA) or 256 rows (CTA pair).
  int MBQ, own_lo_q, own_hi_q;
  int group;  // scheduling blocks swept together (rasterisation)
  int ag_own_direct;  // AG: own row blocks are loaded straight from the input (no self copy)
  int ag_n_own;  // AG: scheduling blocks per source when they tile the rows evenly, else 0 (plain rotated order)
  int debug;  // experiments only (KB200_GEMM_DEBUG): 1 no global stores, 2 epilogue only releases TMEM, 4 every load reads tile (0,0), 8 timing words: status[5] max us waited on peers, [6] us until the pushes were out, [7] us until the last epilogue
};

enum Site : uint32_t {
  SITE_PROD_EMPTY = 1,
  SITE_MMA_FULL = 2,
  SITE_MMA_TEMPTY = 3,
  SITE_EPI_TFULL = 4,
  SITE_RS_FLAG = 5,
  SITE_AG_FLAG = 6,
};

struct Smem {
  uint8_t* a;
  uint8_t* b;
  uint8_t* epi;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* tfull;
  uint64_t* tempty;
  uint32_t* tmem_slot;
  volatile uint32_t* abort;
};

template <bool kPair>
__device__ __forceinline__ Smem carve(uint8_t* raw) {
  constexpr int STAGES = Cfg<kPair>::STAGES;
  Smem s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.a = base;
  s.b = base + STAGES * A_BYTES;
  s.epi = s.b + STAGES * Cfg<kPair>::B_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s.epi + EPI_BYTES);
  s.full = bars;
  s.empty = bars + MAX_STAGES;
  s.tfull = bars + 2 * MAX_STAGES;
  s.tempty = bars + 2 * MAX_STAGES + 2;
  s.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
  s.abort = s.tmem_slot + 1;
  return s;
}

// Position in the static schedule -> tile coordinates.
//
// Row blocks are visited in a rank-rotated sequence: RS starts just after the
// blocks this rank owns (so they come last and every owner is fed by a
// different peer at any time); AG starts with this rank's own rows (which need
// no transfer).  Inside the sequence, GROUP_M consecutive row blocks form a
// group that is swept column block by column block, so that the ~148 tiles in
// flight share few A and B panels (L2 reuse instead of HBM re-reads).  For RS
// the blocks this rank owns form a segment of their own at the very end: a CTA
// never has a push queued behind one of its own waits, which is what makes
// the cross-rank waits deadlock-free.
template <bool kPair>
__host__ __device__ __forceinline__ void tile_at(const GemmParams& p, int pos, int& mbq, int& nb) {
  const int GROUP_M = p.group;
  int start = 0;
  int first_len = p.MBQ;  // blocks in the first segment
  if (p.mode == KB_GEMM_RS) {
    start = p.own_hi_q + 1;
    first_len = p.MBQ - (p.own_hi_q - p.own_lo_q + 1);
  }
  if (p.mode == KB_GEMM_AG) start = p.own_lo_q;
  if (p.mode == KB_GEMM_AG && p.ag_n_own > 0) {
    // Own blocks first, then block c of every other source (nearest first) for
    // c = 0, 1, ...: the order in which the pushes arrive.  Groups of GROUP_M
    // consecutive sequence entries are swept column block by column block.
    const int per_group = GROUP_M * p.NB;
    const int g = pos / per_group;
    const int r = pos - g * per_group;
    int gs = p.MBQ - g * GROUP_M;
    if (gs > GROUP_M) gs = GROUP_M;
    nb = r / gs;
    const int j = g * GROUP_M + (r - nb * gs);
    if (j < p.ag_n_own) {
      mbq = p.own_lo_q + j;
    } else {
      const int jj = j - p.ag_n_own;
      const int c = jj / (p.world - 1);
      const int d = jj - c * (p.world - 1) + 1;
      mbq = ((p.rank + d) % p.world) * p.ag_n_own + c;
    }
    return;
  }
  int base = 0, blocks = first_len, q = pos;
  if (pos >= first_len * p.NB) {
    base = first_len;
    blocks = p.MBQ - first_len;
    q = pos - first_len * p.NB;
  }
  const int per_group = GROUP_M * p.NB;
  const int g = q / per_group;
  const int r = q - g * per_group;
  int gs = blocks - g * GROUP_M;
  if (gs > GROUP_M) gs = GROUP_M;
  nb = r / gs;
  const int j = base + g * GROUP_M + (r - nb * gs);
  mbq = (start + j) % p.MBQ;
}

__device__ __forceinline__ uint32_t* rs_flag(const GemmParams& p, int on_rank, int src, int tile) {
  const uint32_t parity = p.epoch & 1u;
  uint32_t* base = reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off);
  return base + (static_cast<size_t>(parity) * p.world + src) * (static_cast<size_t>(p.MB) * p.NB) + tile;
}
__device__ __forceinline__ bf16* rs_stage_row(const GemmParams& p, int on_rank, int src, int row_local) {
  const uint32_t parity = p.epoch & 1u;
  bf16* base = reinterpret_cast<bf16*>(p.peer_base[on_rank] + p.data_off);
  return base + ((static_cast<size_t>(parity) * p.world + src) * p.rpo + row_local) * static_cast<size_t>(p.N);
}
__device__ __forceinline__ uint32_t* ag_flag(const GemmParams& p, int on_rank, int src, int mb) {
  const uint32_t parity = p.epoch & 1u;
  uint32_t* base = reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off);
  return base + (static_cast<size_t>(parity) * p.world + src) * p.MB + mb;
}
__device__ __forceinline__ bf16* ag_gather_row(const GemmParams& p, int on_rank, int row) {
  const uint32_t parity = p.epoch & 1u;
  bf16* base = reinterpret_cast<bf16*>(p.peer_base[on_rank] + p.data_off);
  return base + (static_cast<size_t>(parity) * p.M + row) * static_cast<size_t>(p.K);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void comm_bar_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// TMEM -> bf16 -> this warp's 32 x 128 staging rows (16-byte chunks XOR-swizzled
// by row so both the row-per-thread writes and the row-contiguous reads are
// bank-conflict free).
__device__ __forceinline__ void stage_half(uint32_t taddr, uint8_t* warp_epi, int lane, const bf16* bias = nullptr,
                                           float bias_scale = 1.f, int col0 = 0, int n_cols = 0) {
#pragma unroll
  for (int c = 0; c < EPI_COLS / 32; ++c) {
    uint32_t r[32];
    kb::tmem_ld_32x32(taddr + c * 32, r);
    kb::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[8 * i + e]);
      if (bias != nullptr) {
        // Added in fp32 before the single rounding to bf16.  All lanes read
        // the same 16 bytes (they hold different rows of the same columns).
        const int col = col0 + c * 32 + i * 8;
        if (col < n_cols) {
          const uint4 bv = *reinterpret_cast<const uint4*>(bias + col);
          float2 t;
          t = kb::unpack_bf16x2(bv.x); f[0] += bias_scale * t.x; f[1] += bias_scale * t.y;
          t = kb::unpack_bf16x2(bv.y); f[2] += bias_scale * t.x; f[3] += bias_scale * t.y;
          t = kb::unpack_bf16x2(bv.z); f[4] += bias_scale * t.x; f[5] += bias_scale * t.y;
          t = kb::unpack_bf16x2(bv.w); f[6] += bias_scale * t.x; f[7] += bias_scale * t.y;
        }
      }
      uint4 v;
      v.x = kb::pack_bf16x2(f[0], f[1]);
      v.y = kb::pack_bf16x2(f[2], f[3]);
      v.z = kb::pack_bf16x2(f[4], f[5]);
      v.w = kb::pack_bf16x2(f[6], f[7]);
      const int j = c * 4 + i;
      const int phys = j ^ (lane & 15);
      *reinterpret_cast<uint4*>(warp_epi + lane * EPI_ROW_BYTES + phys * 16) = v;
    }
  }
}

// TMEM -> fp32 -> this warp's 32 x 64 staging rows (256 bytes per row, same XOR
// swizzle of the 16-byte chunks).
__device__ __forceinline__ void stage_quarter_f32(uint32_t taddr, uint8_t* warp_epi, int lane) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    kb::tmem_ld_32x32(taddr + c * 32, r);
    kb::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 v = make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
      const int j = c * 8 + i;
      *reinterpret_cast<uint4*>(warp_epi + lane * EPI_ROW_BYTES + ((j ^ (lane & 15)) * 16)) = v;
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  float2 t;
  t = kb::unpack_bf16x2(v.x); f[0] = t.x; f[1] = t.y;
  t = kb::unpack_bf16x2(v.y); f[2] = t.x; f[3] = t.y;
  t = kb::unpack_bf16x2(v.z); f[4] = t.x; f[5] = t.y;
  t = kb::unpack_bf16x2(v.w); f[6] = t.x; f[7] = t.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 o;
  o.x = kb::pack_bf16x2(f[0], f[1]);
  o.y = kb::pack_bf16x2(f[2], f[3]);
  o.z = kb::pack_bf16x2(f[4], f[5]);
  o.w = kb::pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ void load_bias8(const bf16* b, float scale, float* out) {
  const uint4 bv = *reinterpret_cast<const uint4*>(b);
  unpack8(bv, out);
#pragma unroll
  for (int e = 0; e < 8; ++e) out[e] *= scale;
}

template <int kMode, bool kPair>
__global__ void __launch_bounds__(kMode == KB_GEMM_AG ? THREADS_AG : THREADS_BASE, 1)
gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr bool kAG = (kMode == KB_GEMM_AG);
  constexpr bool kRS = (kMode == KB_GEMM_RS);
  constexpr int STAGES = Cfg<kPair>::STAGES;
  constexpr int B_BYTES = Cfg<kPair>::B_BYTES;
  // In a pair the even CTA leads: it issues the MMAs for both and owns the
  // barriers the MMA issuer waits on.
  const uint32_t cta_rank = kPair ? kb::cluster_ctarank() : 0u;
  const bool leader = (cta_rank == 0u);
  const int sched_id = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int sched_n = kPair ? (gridDim.x >> 1) : gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  Smem sm = carve<kPair>(smem_raw);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int total_tiles = p.MBQ * p.NB;
  const uint64_t t_start = kb::globaltimer_ns();  // for the optional timing words status[5..7]

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      kb::mbar_init(&sm.full[s], 1);
      kb::mbar_init(&sm.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      kb::mbar_init(&sm.tfull[a], 1);
      kb::mbar_init(&sm.tempty[a], kPair ? 8 : 4);  // epilogue warps of both CTAs release the leader's accumulator
    }
    *sm.abort = 0;
    kb::mbar_fence_init();
  }
  if (warp == 2) {
    if constexpr (kPair) {
      kb::tmem_alloc_pair(sm.tmem_slot, TMEM_COLS);
      kb::tmem_relinquish_pair();
    } else {
      kb::tmem_alloc(sm.tmem_slot, TMEM_COLS);
      kb::tmem_relinquish();
    }
  }
  if (warp == 0 && lane == 0) {
    kb::tma_prefetch_desc(&p.tmA);
    kb::tma_prefetch_desc(&p.tmB);
    if (kAG && p.ag_own_direct) kb::tma_prefetch_desc(&p.tmOwn);
  }
  kb::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) kb::cluster_sync_all();  // the partner's barriers exist before anything signals them
  kb::tc_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint64_t ready_mask[4] = {0ull, 0ull, 0ull, 0ull};  // row blocks already seen complete
      uint64_t waited_ns = 0;
      bool ok = true;
      for (int pos = sched_id; pos < total_tiles && ok; pos += sched_n) {
        int mbq, nb;
        tile_at<kPair>(p, pos, mbq, nb);
        const int mb = kPair ? 2 * mbq + static_cast<int>(cta_rank) : mbq;
        const bool own_direct = kAG && p.ag_own_direct && mb >= p.own_lo_mb && mb <= p.own_hi_mb;
        const CUtensorMap* map_a = own_direct ? &p.tmOwn : &p.tmA;
        const int a_row = own_direct ? mb * BM - p.rank * p.rpo : mb * BM;
        if (kAG && !own_direct && mb < p.MB && !(mb < 256 && ((ready_mask[mb >> 6] >> (mb & 63)) & 1ull))) {
          const int s_lo = (mb * BM) / p.rpo;
          int last_row = mb * BM + BM - 1;
          if (last_row > p.M - 1) last_row = p.M - 1;
          const int s_hi = last_row / p.rpo;
          const uint64_t w0 = kb::globaltimer_ns();
          for (int src = s_lo; src <= s_hi; ++src) {
            if (!kb::wait_flag_ge(ag_flag(p, p.rank, src, mb), p.epoch, p.limit_ns)) {
              kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_AG_FLAG, (uint32_t)src, p.epoch);
            }
          }
          waited_ns += kb::globaltimer_ns() - w0;
          kb::fence_proxy_async_global();
          if (mb < 256) ready_mask[mb >> 6] |= 1ull << (mb & 63);
        }
        for (int kb_i = 0; kb_i < p.KB; ++kb_i) {
          if (!kb::mbar_wait_bounded(&sm.empty[s], ph ^ 1u, p.limit_ns)) {
            kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_PROD_EMPTY, (uint32_t)pos, p.epoch);
            *sm.abort = 1;
            ok = false;
            break;
          }
          if constexpr (kPair) {
            // Both CTAs load their own boxes; all bytes are counted on the
            // leader's barrier, which expects the sum.
            const uint32_t bar = kb::map_to_cta(kb::smem_u32(&sm.full[s]), 0u);
            if (leader) kb::mbar_arrive_expect_tx(&sm.full[s], 2 * (A_BYTES + B_BYTES));
            kb::tma_load_2d_pair(sm.a + s * A_BYTES, map_a, bar, (p.debug & 4) ? 0 : kb_i * BK, (p.debug & 4) ? 0 : a_row);
            kb::tma_load_2d_pair(sm.b + s * B_BYTES, &p.tmB, bar, (p.debug & 4) ? 0 : kb_i * BK, (p.debug & 4) ? 0 : nb * BN + static_cast<int>(cta_rank) * 128);
          } else {
            kb::mbar_arrive_expect_tx(&sm.full[s], A_BYTES + B_BYTES);
            kb::tma_load_2d(sm.a + s * A_BYTES, map_a, &sm.full[s], (p.debug & 4) ? 0 : kb_i * BK, (p.debug & 4) ? 0 : a_row);
            kb::tma_load_2d(sm.b + s * B_BYTES, &p.tmB, &sm.full[s], (p.debug & 4) ? 0 : kb_i * BK, (p.debug & 4) ? 0 : nb * BN);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (kAG && p.status != nullptr && (p.debug & 8)) atomicMax(&p.status[5], static_cast<uint32_t>(waited_ns / 1000));
    }
    __syncwarp();
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer ----
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = kb::umma_idesc_bf16(kPair ? 2 * BM : BM, BN);
      int s = 0;
      uint32_t ph = 0;
      uint32_t it = 0;
      bool ok = true;
      for (int pos = sched_id; pos < total_tiles && ok; pos += sched_n, ++it) {
        const uint32_t acc = it & 1u;
        const uint32_t aph = (it >> 1) & 1u;
        if (!kb::mbar_wait_bounded(&sm.tempty[acc], aph ^ 1u, p.limit_ns)) {
          kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_MMA_TEMPTY, (uint32_t)pos, p.epoch);
          *sm.abort = 1;
          break;
        }
        kb::tc_fence_after_sync();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb_i = 0; kb_i < p.KB; ++kb_i) {
          if (!kb::mbar_wait_bounded(&sm.full[s], ph, p.limit_ns)) {
            kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_MMA_FULL, (uint32_t)pos, p.epoch);
            *sm.abort = 1;
            ok = false;
            break;
          }
          kb::tc_fence_after_sync();
          const uint32_t a_addr = kb::smem_u32(sm.a + s * A_BYTES);
          const uint32_t b_addr = kb::smem_u32(sm.b + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = kb::umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
            const uint64_t db = kb::umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
            if constexpr (kPair) {
              kb::umma_f16_pair(d, da, db, idesc, (kb_i | k) != 0 ? 1u : 0u);
            } else {
              kb::umma_f16(d, da, db, idesc, (kb_i | k) != 0 ? 1u : 0u);
            }
          }
          if constexpr (kPair) {
            // The stage is free in both CTAs once these MMAs have read it.
            const uint32_t e = kb::smem_u32(&sm.empty[s]);
            kb::umma_commit_pair(kb::map_to_cta(e, 0u));
            kb::umma_commit_pair(kb::map_to_cta(e, 1u));
          } else {
            kb::umma_commit(&sm.empty[s]);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) {
          if constexpr (kPair) {
            const uint32_t f = kb::smem_u32(&sm.tfull[acc]);
            kb::umma_commit_pair(kb::map_to_cta(f, 0u));
            kb::umma_commit_pair(kb::map_to_cta(f, 1u));
          } else {
            kb::umma_commit(&sm.tfull[acc]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ---------------------------------------------------------- epilogue ----
    const int q = warp - 4;
    const int et = tid - 128;
    uint8_t* warp_epi = sm.epi + q * EPI_WARP_BYTES;
    constexpr bool rs = kRS;  // the host maps single-rank calls to the plain kernel
    uint32_t it = 0;
    uint64_t rs_waited_ns = 0;
    // Releases this CTA's share of the accumulator: locally for the leader, on
    // the leader's barrier for its partner.
    auto release_acc = [&](uint32_t acc) {
      if constexpr (kPair) {
        if (leader) kb::mbar_arrive(&sm.tempty[acc]);
        else kb::mbar_arrive_cluster(kb::map_to_cta(kb::smem_u32(&sm.tempty[acc]), 0u));
      } else {
        kb::mbar_arrive(&sm.tempty[acc]);
      }
    };
    for (int pos = sched_id; pos < total_tiles; pos += sched_n, ++it) {
      int mbq, nb;
      tile_at<kPair>(p, pos, mbq, nb);
      const int mb = kPair ? 2 * mbq + static_cast<int>(cta_rank) : mbq;
      const uint32_t acc = it & 1u;
      const uint32_t aph = (it >> 1) & 1u;
      // After a failed wait the loop keeps its shape (the named barriers below
      // must be reached by all four warps) but stops waiting.
      if (*sm.abort == 0 && !kb::mbar_wait_bounded(&sm.tfull[acc], aph, p.limit_ns)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_EPI_TFULL, (uint32_t)pos, p.epoch);
        *sm.abort = 1;
      }
      kb::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int row0 = mb * BM;
      int last_row = row0 + BM - 1;
      if (last_row > p.M - 1) last_row = p.M - 1;
      int o_lo = 0, o_hi = 0;
      bool has_remote = false, has_own = true;
      if (rs && row0 < p.M) {
        o_lo = row0 / p.rpo;
        o_hi = last_row / p.rpo;
        has_own = (p.rank >= o_lo && p.rank <= o_hi);
        has_remote = !(o_lo == p.rank && o_hi == p.rank);
      }
      const int tile_id = mb * p.NB + nb;
      bool released = false;
      if (p.debug & 2) {
        kb::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
        continue;
      }

      if (kRS && has_remote) {
        // Phase A: rows that belong to other ranks go to their owners.
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          stage_half(taddr + h * EPI_COLS, warp_epi, lane);
          if (h == 1 && !has_own) {
            kb::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) release_acc(acc);
            released = true;
          }
          __syncwarp();
#pragma unroll 4
          for (int i = 0; i < 16; ++i) {
            const int row = i * 2 + (lane >> 4);
            const int j = lane & 15;
            const int gr = row0 + q * 32 + row;
            const int col = nb * BN + h * EPI_COLS + j * 8;
            if (gr < p.M && col < p.N) {
              const int owner = gr / p.rpo;
              if (owner != p.rank) {
                const uint4 v = *reinterpret_cast<const uint4*>(warp_epi + row * EPI_ROW_BYTES + ((j ^ (row & 15)) * 16));
                bf16* dst = rs_stage_row(p, owner, p.rank, gr - owner * p.rpo) + col;
                kb::st_sys_v4(dst, v);
              }
            }
          }
          __syncwarp();
        }
        epi_bar_sync();
        if (et == 0) {
          kb::fence_sys();
          for (int o = o_lo; o <= o_hi; ++o) {
            if (o != p.rank) kb::st_release_sys_u32(rs_flag(p, o, p.rank, tile_id), p.epoch);
          }
        }
      }

      if (has_own) {
        if (rs) {
          if (et < p.world && et != p.rank) {
            const uint64_t w0 = kb::globaltimer_ns();
            if (!kb::wait_flag_ge(rs_flag(p, p.rank, et, tile_id), p.epoch, p.limit_ns)) {
              kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_RS_FLAG, (uint32_t)et, p.epoch);
            }
            rs_waited_ns += kb::globaltimer_ns() - w0;
          }
          epi_bar_sync();
        }
        if constexpr (!kRS) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            stage_half(taddr + h * EPI_COLS, warp_epi, lane, p.bias, p.bias_scale, nb * BN + h * EPI_COLS, p.N);
            if (h == 1) {
              kb::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) release_acc(acc);
              released = true;
            }
            __syncwarp();
            const int j = lane & 15;
            const int col = nb * BN + h * EPI_COLS + j * 8;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
              const int row = i * 2 + (lane >> 4);
              const int gr = row0 + q * 32 + row;
              if (gr < p.M && col < p.N && !(p.debug & 1)) {
                const uint4 v = *reinterpret_cast<const uint4*>(warp_epi + row * EPI_ROW_BYTES + ((j ^ (row & 15)) * 16));
                *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(gr) * p.N + col) = v;
              }
            }
            __syncwarp();
          }
        } else {
          // Own rows of a reduce-scatter tile.  The local accumulator stays in
          // fp32 (staged 64 columns at a time); the peers' bf16 partials are
          // added in ascending source order, so the sum is bit-reproducible.
          // Loads are issued in batches of 8 rows x 4 sources per thread so
          // that enough of them are in flight to cover the memory latency.
#pragma unroll 1
          for (int qd = 0; qd < 4; ++qd) {
            stage_quarter_f32(taddr + qd * 64, warp_epi, lane);
            if (qd == 3) {
              kb::tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) release_acc(acc);
              released = true;
            }
            __syncwarp();
            const int c8 = lane & 7;
            const int col = nb * BN + qd * 64 + c8 * 8;
            float accv[8][8];
            int out_rows[8];
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int row = ii * 4 + (lane >> 3);
              const int gr = row0 + q * 32 + row;
              const bool mine = (gr < p.M) && (col < p.N) && (gr / p.rpo == p.rank);
              out_rows[ii] = mine ? gr - p.rank * p.rpo : -1;
              const uint8_t* rowp = warp_epi + row * EPI_ROW_BYTES;
              const float4 lo = *reinterpret_cast<const float4*>(rowp + (((2 * c8) ^ (row & 15)) * 16));
              const float4 hi = *reinterpret_cast<const float4*>(rowp + (((2 * c8 + 1) ^ (row & 15)) * 16));
              accv[ii][0] = lo.x; accv[ii][1] = lo.y; accv[ii][2] = lo.z; accv[ii][3] = lo.w;
              accv[ii][4] = hi.x; accv[ii][5] = hi.y; accv[ii][6] = hi.z; accv[ii][7] = hi.w;
            }
#pragma unroll 1
            for (int s0 = 0; s0 < p.world; s0 += 4) {
              uint4 u[8][4];
#pragma unroll
              for (int ii = 0; ii < 8; ++ii) {
#pragma unroll
                for (int sj = 0; sj < 4; ++sj) {
                  const int src = s0 + sj;
                  u[ii][sj] = make_uint4(0u, 0u, 0u, 0u);
                  if (out_rows[ii] >= 0 && src < p.world && src != p.rank) {
                    u[ii][sj] = kb::ld_sys_v4(rs_stage_row(p, p.rank, src, out_rows[ii]) + col);
                  }
                }
              }
#pragma unroll
              for (int ii = 0; ii < 8; ++ii) {
#pragma unroll
                for (int sj = 0; sj < 4; ++sj) {
                  float f[8];
                  unpack8(u[ii][sj], f);
#pragma unroll
                  for (int e = 0; e < 8; ++e) accv[ii][e] += f[e];
                }
              }
            }
            float bz[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (p.bias != nullptr && col < p.N) load_bias8(p.bias + col, p.bias_scale, bz);
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              if (out_rows[ii] >= 0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) accv[ii][e] += bz[e];
                *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(out_rows[ii]) * p.N + col) = pack8(accv[ii]);
              }
            }
            __syncwarp();
          }
        }
      }
      if (!released) {
        kb::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) release_acc(acc);
      }
    }
    if (p.status != nullptr && (p.debug & 8) && lane == 0) {
      if (kRS) atomicMax(&p.status[5], static_cast<uint32_t>(rs_waited_ns / 1000));
      atomicMax(&p.status[7], static_cast<uint32_t>((kb::globaltimer_ns() - t_start) / 1000));
    }
  } else if (kAG && warp >= 8) {
    // -------------------------------------------------- all-gather pusher ----
    const int ct = tid - 256;
    // Group of row blocks by group, all CTAs together.  A group is cut into
    // slices of 1024 vectors (16 KB); CTAs claim slices from a counter, so an SM
    // with a slower path to the links simply takes fewer of them and the group
    // completes at the aggregate rate instead of the slowest SM's.  A claimed
    // slice is read once (eight 16-byte loads per thread in flight) and stored
    // into the gather buffer of every other rank (and of this rank, unless the
    // GEMM reads its own rows in place).  Groups therefore arrive everywhere in
    // ascending order, which is the order in which the GEMMs consume them.  When
    // a CTA finds a group exhausted it fences and counts itself done; the last
    // one releases the group's flags on every rank and rewinds the claim counter.
    const int n_chunks = p.own_hi_mb - p.own_lo_mb + 1;
    const int own_row0 = p.rank * p.rpo;
    const int dd0 = p.ag_own_direct ? 1 : 0;
    uint32_t* counters = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.counter_off);  // [0..63] done, [64..127] claim
    const int group = (n_chunks + 7) / 8;  // at most eight groups per call
    const int n_groups = (n_chunks + group - 1) / group;
    constexpr size_t SLICE = 8 * 128;
    __shared__ uint32_t s_claim;
    for (int g = 0; g < n_groups; ++g) {
      const int c_lo = g * group;
      int c_hi = c_lo + group;
      if (c_hi > n_chunks) c_hi = n_chunks;
      int r_begin = (p.own_lo_mb + c_lo) * BM;
      if (r_begin < own_row0) r_begin = own_row0;
      int r_end = (p.own_lo_mb + c_hi) * BM;
      if (r_end > own_row0 + p.rpo) r_end = own_row0 + p.rpo;
      if (r_end > p.M) r_end = p.M;
      const size_t nvec = static_cast<size_t>(r_end - r_begin) * p.K / 8;
      const uint32_t n_slices = static_cast<uint32_t>((nvec + SLICE - 1) / SLICE);
      const uint4* src = reinterpret_cast<const uint4*>(p.a_local + static_cast<size_t>(r_begin - own_row0) * p.K);
      for (;;) {
        if (ct == 0) s_claim = atomicAdd(&counters[64 + g], 1u);
        comm_bar_sync();
        const uint32_t slice = s_claim;
        comm_bar_sync();  // everybody has read the claim before thread 0 overwrites it
        if (slice >= n_slices) break;
        const size_t base = static_cast<size_t>(slice) * SLICE;
        uint4 x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const size_t v = base + u * 128 + ct;
          if (v < nvec) x[u] = kb::ld_nc_v4(src + v);
        }
        for (int dd = dd0; dd < p.world; ++dd) {
          const int dst = (p.rank - dd + p.world) % p.world;
          uint4* dstp = reinterpret_cast<uint4*>(ag_gather_row(p, dst, r_begin));
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const size_t v = base + u * 128 + ct;
            if (v < nvec) kb::st_sys_v4(dstp + v, x[u]);
          }
        }
      }
      if (ct == 0) {
        kb::fence_sys();
        const uint32_t old = atomicAdd(&counters[g], 1u);
        if ((old + 1u) % gridDim.x == 0u) {
          counters[64 + g] = 0u;  // every CTA is past its last claim of this group
          kb::fence_sys();
          for (int cc = c_lo; cc < c_hi; ++cc) {
            for (int dd = dd0; dd < p.world; ++dd) {
              const int dst = (p.rank - dd + p.world) % p.world;
              kb::st_relaxed_sys_u32(ag_flag(p, dst, p.rank, p.own_lo_mb + cc), p.epoch);
            }
          }
        }
      }
    }
    if (ct == 0 && p.status != nullptr && (p.debug & 8)) {
      atomicMax(&p.status[6], static_cast<uint32_t>((kb::globaltimer_ns() - t_start) / 1000));
    }
  }

  kb::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) kb::cluster_sync_all();  // nobody leaves while the partner may still signal or read
  if (warp == 2) {
    kb::tc_fence_after_sync();
    if constexpr (kPair) kb::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else kb::tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host ----
int make_tmap(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  auto encode = KB_DRV(cuTensorMapEncodeTiled);
  if (encode == nullptr) return KB_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    kb::set_error("cuTensorMapEncodeTiled failed: CUresult %d (ptr %p rows %llu cols %llu)", (int)r, ptr,
                  (unsigned long long)rows, (unsigned long long)cols);
    return KB_ERR_CUDA;
  }
  return KB_OK;
}

inline uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

inline bool getenv_flag(const char* name) {
  const char* v = getenv(name);
  return v != nullptr && v[0] == '1';
}

}  // namespace

// Host replica of the device tile schedule, for tests of the index arithmetic:
// position -> (scheduling block, column block) for the given problem and rank.
// Returns the number of positions, or -1 for invalid arguments.
extern "C" int kb_gemm_schedule(int mode, int M, int N, int rank, int world, int pair, int pos, int* block, int* nb) {
  if (M <= 0 || N <= 0 || world < 1 || rank < 0 || rank >= world || (mode != KB_GEMM_PLAIN && M % world != 0)) return -1;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.mode = world > 1 ? mode : KB_GEMM_PLAIN;
  p.M = M;
  p.N = N;
  p.world = world;
  p.rank = rank;
  p.MB = (M + BM - 1) / BM;
  p.NB = (N + BN - 1) / BN;
  p.rpo = (p.mode == KB_GEMM_PLAIN) ? M : M / world;
  const int block_rows = pair ? 256 : 128;
  const bool dist_mode = p.mode != KB_GEMM_PLAIN;
  if (pair && dist_mode && (p.rpo % 256) != 0) return -1;
  p.MBQ = (M + block_rows - 1) / block_rows;
  p.own_lo_q = dist_mode ? (rank * p.rpo) / block_rows : 0;
  p.own_hi_q = dist_mode ? ((rank + 1) * p.rpo - 1) / block_rows : p.MBQ - 1;
  p.ag_n_own = (p.mode == KB_GEMM_AG && (p.rpo % block_rows) == 0) ? p.rpo / block_rows : 0;
  // 1024 rows are swept together (measured best among 512 to 4096 on 8192 x 8192 x 29568; for the all-gather
  // kernel it also makes the first group consist of this rank's own rows only at eight ranks).
  p.group = 1024 / block_rows;
  if (const char* g = getenv("KB200_GEMM_GROUP")) p.group = atoi(g) > 0 ? atoi(g) : p.group;
  const int total = p.MBQ * p.NB;
  if (pos >= 0 && pos < total && block != nullptr && nb != nullptr) {
    if (pair) tile_at<true>(p, pos, *block, *nb);
    else tile_at<false>(p, pos, *block, *nb);
  }
  return total;
}

extern "C" uint64_t kb_gemm_rs_data_bytes(int M, int N, int world) {
  return round_up(2ull * world * (uint64_t)(M / world) * N * 2, 256);
}
extern "C" uint64_t kb_gemm_rs_flag_bytes(int M, int N, int world) {
  const uint64_t tiles = (uint64_t)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return round_up(2ull * world * tiles * 4, 256);
}
extern "C" uint64_t kb_gemm_ag_data_bytes(int M, int K) { return round_up(2ull * (uint64_t)M * K * 2, 256); }
extern "C" uint64_t kb_gemm_ag_flag_bytes(int M, int world) {
  return round_up(2ull * world * ((M + BM - 1) / BM) * 4, 256);
}
extern "C" uint64_t kb_gemm_ag_counter_bytes(int M, int world) {
  (void)M;
  (void)world;
  return 1024;  // 64 completion counters and 64 claim counters (at most eight groups are used)
}

extern "C" int kb_gemm(const KbGemmArgs* a, void* stream_v) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (a == nullptr) return KB_ERR_ARG;
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || (a->K % 8) != 0 || (a->N % 8) != 0) {
    kb::set_error("kb_gemm: need M,N,K > 0 and N,K multiples of 8 (got %d %d %d)", a->M, a->N, a->K);
    return KB_ERR_ARG;
  }
  if (a->world < 1 || a->world > KB_MAX_WORLD || a->rank < 0 || a->rank >= a->world) {
    kb::set_error("kb_gemm: bad rank/world %d/%d", a->rank, a->world);
    return KB_ERR_ARG;
  }
  auto misaligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) != 0; };
  if (misaligned(a->A) || misaligned(a->B) || misaligned(a->out) || (a->bias && misaligned(a->bias))) {
    kb::set_error("kb_gemm: operand pointers must be 16-byte aligned");
    return KB_ERR_ARG;
  }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.mode = a->mode;
  p.M = a->M;
  p.N = a->N;
  p.K = a->K;
  p.MB = (a->M + BM - 1) / BM;
  p.NB = (a->N + BN - 1) / BN;
  p.KB = (a->K + BK - 1) / BK;
  p.bias = static_cast<const bf16*>(a->bias);
  p.bias_scale = a->bias_scale;
  p.out = static_cast<bf16*>(a->out);
  p.rank = a->rank;
  p.world = a->world;
  p.epoch = a->epoch;
  p.status = a->status;
  p.limit_ns = a->wait_limit_ns ? a->wait_limit_ns : 2000000000ull;
  p.data_off = a->data_off;
  p.flag_off = a->flag_off;
  p.counter_off = a->counter_off;
  p.ag_parts = 32;
  for (int r = 0; r < a->world; ++r) p.peer_base[r] = static_cast<char*>(a->peer_base[r]);

  const void* a_ptr = a->A;
  uint64_t a_rows = a->M;
  p.rpo = a->M;
  p.own_lo_mb = 0;
  p.own_hi_mb = p.MB - 1;
  const bool dist = a->mode != KB_GEMM_PLAIN && a->world > 1;
  if (a->mode == KB_GEMM_PLAIN || !dist) {
    if (a->mode == KB_GEMM_AG) {
      // Single rank: nothing to gather, read A in place.
      p.mode = KB_GEMM_PLAIN;
    }
    if (a->mode == KB_GEMM_RS) p.mode = KB_GEMM_PLAIN;
    p.world = 1;
    p.rank = 0;
  } else {
    if (a->M % a->world != 0) {
      kb::set_error("kb_gemm: M=%d must be divisible by world=%d", a->M, a->world);
      return KB_ERR_ARG;
    }
    p.rpo = a->M / a->world;
    if (!((p.rpo % BM) == 0 || (BM % p.rpo) == 0)) {
      kb::set_error("kb_gemm: rows per rank (%d) must divide or be a multiple of %d", p.rpo, BM);
      return KB_ERR_ARG;
    }
    for (int r = 0; r < a->world; ++r) {
      if (p.peer_base[r] == nullptr) {
        kb::set_error("kb_gemm: peer_base[%d] is null", r);
        return KB_ERR_ARG;
      }
    }
    p.own_lo_mb = (a->rank * p.rpo) / BM;
    p.own_hi_mb = ((a->rank + 1) * p.rpo - 1) / BM;
    if (a->mode == KB_GEMM_AG) {
      p.a_local = static_cast<const bf16*>(a->A);
      const uint32_t parity = a->epoch & 1u;
      a_ptr = p.peer_base[a->rank] + a->data_off + (uint64_t)parity * a->M * a->K * 2;
    }
  }

  // CTA pairs need 256-row scheduling blocks that do not straddle two ranks.
  // num_ctas bit 30 forces the single-CTA kernel (tests, comparisons).
  {
    const char* dbg = getenv("KB200_GEMM_DEBUG");
    p.debug = dbg ? atoi(dbg) : 0;

  }
  const bool forbid_pair = (a->num_ctas & (1 << 30)) != 0 || getenv_flag("KB200_GEMM_NO_PAIR");
  const int req_ctas = a->num_ctas & ~(1 << 30);
  const bool dist_mode = (p.mode != KB_GEMM_PLAIN);
  bool pair = !forbid_pair && a->M >= 256 && (!dist_mode || (p.rpo % 256) == 0);

  int dev = 0, sms = 0;
  KB_CUDA_OK(cudaGetDevice(&dev));
  KB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  int grid = req_ctas > 0 ? req_ctas : sms;
  if (grid > sms) grid = sms;
  if (pair) {
    grid &= ~1;
    if (grid < 2) pair = false;
  }
  const int block_rows = pair ? 256 : 128;
  p.MBQ = (a->M + block_rows - 1) / block_rows;
  p.own_lo_q = dist_mode ? (a->rank * p.rpo) / block_rows : 0;
  p.own_hi_q = dist_mode ? ((a->rank + 1) * p.rpo - 1) / block_rows : p.MBQ - 1;
  p.ag_n_own = (p.mode == KB_GEMM_AG && (p.rpo % block_rows) == 0) ? p.rpo / block_rows : 0;
  // 1024 rows are swept together (measured best among 512 to 4096 on 8192 x 8192 x 29568; for the all-gather
  // kernel it also makes the first group consist of this rank's own rows only at eight ranks).
  p.group = 1024 / block_rows;
  if (const char* g = getenv("KB200_GEMM_GROUP")) p.group = atoi(g) > 0 ? atoi(g) : p.group;

  int rc = make_tmap(&p.tmA, a_ptr, a_rows, a->K, BM);
  if (rc != KB_OK) return rc;
  rc = make_tmap(&p.tmB, a->B, a->N, a->K, pair ? 128 : BN);
  if (rc != KB_OK) return rc;
  p.ag_own_direct = 0;
  if (p.mode == KB_GEMM_AG && (p.rpo % BM) == 0) {
    rc = make_tmap(&p.tmOwn, a->A, p.rpo, a->K, BM);
    if (rc != KB_OK) return rc;
    p.ag_own_direct = 1;
  }

  const int total_units = p.MBQ * p.NB * (pair ? 2 : 1);
  const bool ag = (p.mode == KB_GEMM_AG);
  if (!ag && grid > total_units) grid = total_units;

  const int threads = ag ? THREADS_AG : THREADS_BASE;
  const void* fn = nullptr;
  if (pair) {
    fn = ag ? (const void*)gemm_kernel<KB_GEMM_AG, true>
            : (p.mode == KB_GEMM_RS ? (const void*)gemm_kernel<KB_GEMM_RS, true> : (const void*)gemm_kernel<KB_GEMM_PLAIN, true>);
  } else {
    fn = ag ? (const void*)gemm_kernel<KB_GEMM_AG, false>
            : (p.mode == KB_GEMM_RS ? (const void*)gemm_kernel<KB_GEMM_RS, false> : (const void*)gemm_kernel<KB_GEMM_PLAIN, false>);
  }
  KB_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (pair) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  void* args[] = {&p};
  KB_CUDA_OK(cudaLaunchKernelExC(&cfg, fn, args));
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}
