// Persistent, warp-specialised bf16 GEMM for sm_100a in three modes:
//
//   PLAIN  out = A * B^T (+ bias)
//   RS     GEMM fused with reduce-scatter.  Every rank computes its K-shard's
//          partial product tile by tile into its OWN half of a parity-buffered
//          [M, N] bf16 staging matrix in the symmetric heap and, per tile,
//          releases an epoch flag on the rank that owns the tile's rows.  Four
//          extra "reduce" warps per CTA walk the rows this rank owns in the order
//          in which the tiles complete everywhere, wait for the flags of all
//          ranks, pull the partials over NVLink (peer loads, or one
//          multimem.ld_reduce per 16 bytes that lets the switch add them), add the
//          bias and write the output shard.  The tensor-core pipeline never waits
//          for a peer, and the reduction of block c overlaps the GEMM of block c+1:
//          all ranks visit block c of every owner at about the same time.
//   AG     all-gather fused with GEMM: extra "comm" warps of the same kernel
//          stream this rank's A rows into every peer's gather buffer (peer stores,
//          or one multimem.st per 16 bytes that the switch replicates) while the
//          tensor cores already work on the rows that are present; the TMA
//          producer waits (bounded) on a per-row-block flag before it loads
//          rows that come from a peer.
//
// Mainloop: one TMA producer thread fills a ring of 128x64 (A) and 256x64 (B)
// K-major tiles with 128-byte swizzle; one thread issues tcgen05.mma into one of
// two 256-column TMEM accumulators; four epilogue warps drain the other
// accumulator.  Two epilogue variants: "tma" (PLAIN and AG only) goes tcgen05.ld ->
// bf16 -> 128-byte-swizzled shared memory -> cp.async.bulk.tensor store issued
// by one lane per warp, two staging boxes per warp; "direct" stores 16-byte
// vectors straight from the registers tcgen05.ld filled (a lane owns a row, so a
// warp's store touches 32 rows: more L2 transactions for the output, which is a
// few percent of the kernel's traffic) and needs no staging memory, which buys
// the CTA-pair configuration a seventh pipeline stage.  RS always stores
// directly: its stores must be ordered before a flag release as ordinary stores.
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
// rows of A and its 128 of the 256 B rows: 6 stages of 32 KB, 7 when the
// epilogue needs no staging memory.
template <bool kPair, bool kDirect>
struct Cfg {
  static constexpr int STAGES = kPair ? (kDirect ? 7 : 6) : 4;
  static constexpr int B_ROWS = kPair ? 128 : 256;
  static constexpr int B_BYTES = B_ROWS * BK * 2;
};
constexpr int MAX_STAGES = 7;
// Staging of the "tma" epilogue: per warp two boxes of 32 rows x 64 columns in
// the 128-byte-swizzle layout of the output tensor map.
constexpr int EPI_WARP_BYTES = 8192;
constexpr int EPI_BYTES = 4 * EPI_WARP_BYTES;
static_assert(6 * 32768 + EPI_BYTES <= 7 * 32768, "six pair stages plus the staging boxes fit where seven stages fit");
constexpr int OUT_BOX_COLS = 64;
constexpr int OUT_BOX_ROWS = 32;
constexpr int OUT_BOX_BYTES = OUT_BOX_ROWS * OUT_BOX_COLS * 2;  // 4 KB
constexpr int TMEM_COLS = 512;
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = 1024 + 7 * 32768 + BAR_BYTES;  // 6 pair stages + staging = 4 single stages + staging = 7 pair stages
constexpr int THREADS_BASE = 256;             // warps 0..3 control, 4..7 epilogue
constexpr int THREADS_COMM = 384;             // + warps 8..11: all-gather pushers or reduce-scatter reducers
constexpr int SCHED_RING = 4;                 // AG: claimed tile positions in flight between the claimer and the other roles
constexpr int AG_TILE_CLAIM = 128;            // AG: two words of the counter block (one per epoch parity) that hand out tile positions
constexpr int RS_ROW_GROUP = 64;              // rows of one reduction unit
constexpr int RS_UNIT_COLS = 128;             // columns of one reduction unit

struct alignas(64) GemmParams {
  CUtensorMap tmA;
  CUtensorMap tmB;
  CUtensorMap tmOwn;  // AG: this rank's own rows, read in place
  CUtensorMap tmOut;  // PLAIN/AG: the output, written with TMA stores
  int mode, M, N, K;
  int MB, NB, KB;
  const bf16* bias;
  float bias_scale;
  bf16* out;
  int rank, world, rpo;
  uint32_t epoch;
  char* peer_base[KB_MAX_WORLD];
  char* mc_base;  // multicast mapping of the heap, or null: peer loads / stores instead of multimem
  uint64_t data_off, flag_off, counter_off;
  const bf16* a_local;
  uint32_t* status;
  uint64_t limit_ns;
  int own_lo_mb, own_hi_mb;
  // Scheduling blocks: 128 rows (single CTA) or 256 rows (CTA pair).
  int MBQ, own_lo_q;
  int group;          // scheduling blocks swept together (rasterisation)
  int ag_own_direct;  // AG: own row blocks are loaded straight from the input (no self copy)
  int ag_n_own;       // AG: scheduling blocks per source when they tile the rows evenly, else 0 (plain rotated order)
  int rs_nq;          // RS: scheduling blocks per owner when they tile the rows evenly, else 0 (plain order)
  int timing;         // record timing words: status[5] max us waited on peers, [6] us until the pushes were out, [7] us until the last epilogue / reduction ended
};

enum Site : uint32_t {
  SITE_PROD_EMPTY = 1,
  SITE_MMA_FULL = 2,
  SITE_MMA_TEMPTY = 3,
  SITE_EPI_TFULL = 4,
  SITE_RS_FLAG = 5,
  SITE_AG_FLAG = 6,
  SITE_SCHED = 7,
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
  uint64_t* sfull;              // AG: a claimed position is in sched_pos[slot]
  uint64_t* sempty;             // AG: every role has read sched_pos[slot] (on the leader CTA)
  volatile int32_t* sched_pos;  // AG: ring of claimed schedule positions, -1 = no more tiles
};

template <bool kPair, bool kDirect>
__device__ __forceinline__ Smem carve(uint8_t* raw) {
  constexpr int STAGES = Cfg<kPair, kDirect>::STAGES;
  Smem s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.a = base;
  s.b = base + STAGES * A_BYTES;
  s.epi = s.b + STAGES * Cfg<kPair, kDirect>::B_BYTES;  // 1024-byte aligned: every stage is a multiple of 1024 bytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + 7 * 32768);  // behind the largest configuration
  s.full = bars;
  s.empty = bars + MAX_STAGES;
  s.tfull = bars + 2 * MAX_STAGES;
  s.tempty = bars + 2 * MAX_STAGES + 2;
  s.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
  s.abort = s.tmem_slot + 1;
  s.sfull = bars + 2 * MAX_STAGES + 5;
  s.sempty = s.sfull + SCHED_RING;
  s.sched_pos = reinterpret_cast<volatile int32_t*>(s.sempty + SCHED_RING);
  static_assert((2 * MAX_STAGES + 5 + 2 * SCHED_RING) * 8 + SCHED_RING * 4 <= BAR_BYTES, "barrier block too small");
  return s;
}

// Position in the static schedule -> tile coordinates.
//
// Scheduling blocks are visited in a sequence that depends on the mode; groups
// of GROUP_M consecutive sequence entries are swept column block by column
// block, so that the ~148 tiles in flight share few A and B panels (L2 reuse
// instead of HBM re-reads).
//   PLAIN  ascending.
//   RS     block c of every owner, then block c+1 of every owner, ... (owners in
//          ring order after this rank): all ranks finish block c of an owner at
//          about the same time, so its reduction overlaps the GEMM of block c+1.
//   AG     this rank's own blocks (no transfer needed), then block c of every
//          other source (nearest first) for c = 0, 1, ...: the order in which
//          the pushes arrive.
//
// PLAIN and RS walk the sequence statically (CTA or CTA pair i takes positions
// i, i + n, ...).  AG hands positions out from a counter: a CTA pair whose next
// tile waits for rows that have not arrived simply ends up with fewer tiles,
// instead of finishing late with its fixed share (with a static walk the pairs
// that start on remote rows lose the whole arrival time of the first blocks).
__host__ __device__ __forceinline__ void tile_at(const GemmParams& p, int pos, int& mbq, int& nb) {
  const int GROUP_M = p.group;
  const int per_group = GROUP_M * p.NB;
  const int g = pos / per_group;
  const int r = pos - g * per_group;
  int gs = p.MBQ - g * GROUP_M;
  if (gs > GROUP_M) gs = GROUP_M;
  nb = r / gs;
  const int j = g * GROUP_M + (r - nb * gs);  // index in the block sequence
  mbq = j;
  if (p.mode == KB_GEMM_RS && p.rs_nq > 0) {
    const int c = j / p.world;
    const int o = (p.rank + 1 + (j - c * p.world)) % p.world;
    mbq = o * p.rs_nq + c;
  } else if (p.mode == KB_GEMM_AG) {
    if (p.ag_n_own > 0) {
      if (j < p.ag_n_own) {
        mbq = p.own_lo_q + j;
      } else {
        const int jj = j - p.ag_n_own;
        const int c = jj / (p.world - 1);
        const int d = jj - c * (p.world - 1) + 1;
        mbq = ((p.rank + d) % p.world) * p.ag_n_own + c;
      }
    } else {
      mbq = (p.own_lo_q + j) % p.MBQ;
    }
  }
}

// RS: flag of (source rank, tile) on the rank that owns rows of the tile.
__device__ __forceinline__ uint32_t* rs_flag(const GemmParams& p, int on_rank, int src, int tile) {
  const uint32_t parity = p.epoch & 1u;
  uint32_t* base = reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off);
  return base + (static_cast<size_t>(parity) * p.world + src) * (static_cast<size_t>(p.MB) * p.NB) + tile;
}
// RS: element offset of row `row` of this epoch's [M, N] staging matrix inside a segment.
__device__ __forceinline__ size_t rs_stage_elem(const GemmParams& p, int row) {
  const uint32_t parity = p.epoch & 1u;
  return (static_cast<size_t>(parity) * p.M + row) * static_cast<size_t>(p.N);
}
__device__ __forceinline__ uint32_t* ag_flag(const GemmParams& p, int on_rank, int src, int mb) {
  const uint32_t parity = p.epoch & 1u;
  uint32_t* base = reinterpret_cast<uint32_t*>(p.peer_base[on_rank] + p.flag_off);
  return base + (static_cast<size_t>(parity) * p.world + src) * p.MB + mb;
}
__device__ __forceinline__ size_t ag_gather_elem(const GemmParams& p, int row) {
  const uint32_t parity = p.epoch & 1u;
  return (static_cast<size_t>(parity) * p.M + row) * static_cast<size_t>(p.K);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void comm_bar_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

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

// Eight fp32 accumulator values (+ bias, added in fp32 before the single rounding) -> eight bf16.
__device__ __forceinline__ uint4 cvt8(const uint32_t* r, const bf16* bias, float bias_scale, int col, int n_cols) {
  float f[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[e]);
  if (bias != nullptr && col < n_cols) {
    // All lanes read the same 16 bytes (they hold different rows of the same columns).
    float b[8];
    unpack8(*reinterpret_cast<const uint4*>(bias + col), b);
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] += bias_scale * b[e];
  }
  return pack8(f);
}

// TMEM -> bf16 (+ bias) -> global memory, 64 columns of this lane's row: eight
// 16-byte stores straight from the registers.
__device__ __forceinline__ void store_direct(uint32_t taddr, bf16* row_ptr, bool row_ok, const bf16* bias, float bias_scale,
                                             int col0, int n_cols) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    kb::tmem_ld_32x32(taddr + c * 32, r);
    kb::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int col = col0 + (c * 4 + i) * 8;
      const uint4 v = cvt8(r + 8 * i, bias, bias_scale, col, n_cols);
      if (row_ok && col < n_cols) *reinterpret_cast<uint4*>(row_ptr + col) = v;
    }
  }
}

// TMEM -> bf16 (+ bias) -> one 32 x 64 box in the 128-byte-swizzle layout of the
// output tensor map: row = lane, 16-byte chunk j of the row at position j ^ (row & 7).
__device__ __forceinline__ void stage_box(uint32_t taddr, uint8_t* box, int lane, const bf16* bias, float bias_scale,
                                          int col0, int n_cols) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    kb::tmem_ld_32x32(taddr + c * 32, r);
    kb::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int j = c * 4 + i;
      const uint4 v = cvt8(r + 8 * i, bias, bias_scale, col0 + j * 8, n_cols);
      *reinterpret_cast<uint4*>(box + lane * (OUT_BOX_COLS * 2) + ((j ^ (lane & 7)) * 16)) = v;
    }
  }
}

template <int kMode, bool kPair, bool kDirect>
__global__ void __launch_bounds__(kMode == KB_GEMM_PLAIN ? THREADS_BASE : THREADS_COMM, 1)
gemm_kernel(const __grid_constant__ GemmParams p) {
  constexpr bool kAG = (kMode == KB_GEMM_AG);
  constexpr bool kRS = (kMode == KB_GEMM_RS);
  static_assert(!kRS || kDirect, "the reduce-scatter epilogue stores directly");
  constexpr int STAGES = Cfg<kPair, kDirect>::STAGES;
  constexpr int B_BYTES = Cfg<kPair, kDirect>::B_BYTES;
  // In a pair the even CTA leads: it issues the MMAs for both and owns the
  // barriers the MMA issuer waits on.
  const uint32_t cta_rank = kPair ? kb::cluster_ctarank() : 0u;
  const bool leader = (cta_rank == 0u);
  const int sched_id = kPair ? (blockIdx.x >> 1) : blockIdx.x;
  const int sched_n = kPair ? (gridDim.x >> 1) : gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  Smem sm = carve<kPair, kDirect>(smem_raw);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int total_tiles = p.MBQ * p.NB;
  const uint64_t t_start = p.timing ? kb::globaltimer_ns() : 0;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      kb::mbar_init(&sm.full[s], 1);
      kb::mbar_init(&sm.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      kb::mbar_init(&sm.tfull[a], 1);
      kb::mbar_init(&sm.tempty[a], kPair ? 8 : 4);  // epilogue warps of both CTAs release the leader's accumulator
    }
    if (kAG) {
      for (int r = 0; r < SCHED_RING; ++r) {
        kb::mbar_init(&sm.sfull[r], 1);
        kb::mbar_init(&sm.sempty[r], kPair ? 10 : 5);  // MMA issuer, epilogue warps of both CTAs, the partner's producer
      }
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
  if (kAG && blockIdx.x == 0 && tid == 32) {
    reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.counter_off)[AG_TILE_CLAIM + ((p.epoch & 1u) ^ 1u)] = 0u;
  }
  if (warp == 0 && lane == 0) {
    kb::tma_prefetch_desc(&p.tmA);
    kb::tma_prefetch_desc(&p.tmB);
    if (kAG && p.ag_own_direct) kb::tma_prefetch_desc(&p.tmOwn);
    if (!kDirect) kb::tma_prefetch_desc(&p.tmOut);
  }
  kb::tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) kb::cluster_sync_all();  // the partner's barriers exist before anything signals them
  kb::tc_fence_after_sync();
  const uint32_t tmem_base = *sm.tmem_slot;

  // ---- AG: dynamic tile positions -------------------------------------------
  // The leader's producer thread claims the next position from a counter in this
  // rank's counter block and publishes it in a ring slot of both CTAs; every other
  // role reads it from its own CTA's slot and acknowledges on the leader's
  // barrier.  Calls alternate between two counters by epoch parity; a call zeroes
  // the counter of the other parity, which nobody uses while it runs, so the
  // counters are right whatever happened to the call before.
  auto claim_tile = [&](uint32_t iter) -> int {
    const int slot = static_cast<int>(iter % SCHED_RING);
    if (iter >= SCHED_RING && !kb::mbar_wait_bounded(&sm.sempty[slot], ((iter / SCHED_RING) - 1u) & 1u, p.limit_ns)) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_SCHED, iter, p.epoch);
      *sm.abort = 1;
      return -1;
    }
    uint32_t* counter = reinterpret_cast<uint32_t*>(p.peer_base[p.rank] + p.counter_off) + AG_TILE_CLAIM + (p.epoch & 1u);
    const uint32_t v = atomicAdd(counter, 1u);
    const int pos = v < static_cast<uint32_t>(total_tiles) ? static_cast<int>(v) : -1;
    sm.sched_pos[slot] = pos;
    if constexpr (kPair) {
      kb::st_shared_cluster_u32(kb::map_to_cta(kb::smem_u32(const_cast<int32_t*>(&sm.sched_pos[slot])), 1u), static_cast<uint32_t>(pos));
      kb::mbar_arrive_cluster(kb::map_to_cta(kb::smem_u32(&sm.sfull[slot]), 1u));
    }
    kb::mbar_arrive(&sm.sfull[slot]);
    return pos;
  };
  auto read_tile = [&](uint32_t iter) -> int {
    const int slot = static_cast<int>(iter % SCHED_RING);
    const uint32_t parity = (iter / SCHED_RING) & 1u;
    const bool ok = (kPair && !leader) ? kb::mbar_wait_bounded_cluster(&sm.sfull[slot], parity, p.limit_ns)
                                       : kb::mbar_wait_bounded(&sm.sfull[slot], parity, p.limit_ns);
    if (!ok) {
      kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_SCHED, iter, p.epoch);
      *sm.abort = 1;
      return -1;
    }
    const int pos = sm.sched_pos[slot];
    if (kPair && !leader) kb::mbar_arrive_cluster(kb::map_to_cta(kb::smem_u32(&sm.sempty[slot]), 0u));
    else kb::mbar_arrive(&sm.sempty[slot]);
    return pos;
  };

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint64_t ready_mask[4] = {0ull, 0ull, 0ull, 0ull};  // row blocks already seen complete
      uint64_t waited_ns = 0;
      bool ok = true;
      for (uint32_t iter = 0; ok; ++iter) {
        int pos;
        if constexpr (kAG) {
          pos = leader ? claim_tile(iter) : read_tile(iter);
          if (pos < 0) break;
        } else {
          pos = sched_id + static_cast<int>(iter) * sched_n;
          if (pos >= total_tiles) break;
        }
        int mbq, nb;
        tile_at(p, pos, mbq, nb);
        const int mb = kPair ? 2 * mbq + static_cast<int>(cta_rank) : mbq;
        const bool own_direct = kAG && p.ag_own_direct && mb >= p.own_lo_mb && mb <= p.own_hi_mb;
        const CUtensorMap* map_a = own_direct ? &p.tmOwn : &p.tmA;
        const int a_row = own_direct ? mb * BM - p.rank * p.rpo : mb * BM;
        if (kAG && !own_direct && mb < p.MB && !(mb < 256 && ((ready_mask[mb >> 6] >> (mb & 63)) & 1ull))) {
          const int s_lo = (mb * BM) / p.rpo;
          int last_row = mb * BM + BM - 1;
          if (last_row > p.M - 1) last_row = p.M - 1;
          const int s_hi = last_row / p.rpo;
          const uint64_t w0 = p.timing ? kb::globaltimer_ns() : 0;
          for (int src = s_lo; src <= s_hi; ++src) {
            // acquire loads, no system-scope fence: that fence would wait for the acknowledgements of
            // the pushes this GPU has in flight, microseconds per row block on the producer's path
            if (!kb::wait_flag_ge(ag_flag(p, p.rank, src, mb), p.epoch, p.limit_ns, 512, true, true)) {
              kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_AG_FLAG, (uint32_t)src, p.epoch);
            }
          }
          if (p.timing) waited_ns += kb::globaltimer_ns() - w0;
          kb::fence_proxy_async_global();
          if (mb < 256) ready_mask[mb >> 6] |= 1ull << (mb & 63);
        }
        for (int kb_i = 0; kb_i < p.KB; ++kb_i) {
          if (!kb::mbar_wait_bounded(&sm.empty[s], ph ^ 1u, p.limit_ns, 400)) {
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
            kb::tma_load_2d_pair(sm.a + s * A_BYTES, map_a, bar, kb_i * BK, a_row);
            kb::tma_load_2d_pair(sm.b + s * B_BYTES, &p.tmB, bar, kb_i * BK, nb * BN + static_cast<int>(cta_rank) * 128);
          } else {
            kb::mbar_arrive_expect_tx(&sm.full[s], A_BYTES + B_BYTES);
            kb::tma_load_2d(sm.a + s * A_BYTES, map_a, &sm.full[s], kb_i * BK, a_row);
            kb::tma_load_2d(sm.b + s * B_BYTES, &p.tmB, &sm.full[s], kb_i * BK, nb * BN);
          }
          if (++s == STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (kAG && p.status != nullptr && p.timing) atomicMax(&p.status[5], static_cast<uint32_t>(waited_ns / 1000));
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
      for (;; ++it) {
        int pos;
        if constexpr (kAG) {
          pos = read_tile(it);
        } else {
          pos = sched_id + static_cast<int>(it) * sched_n;
          if (pos >= total_tiles) pos = -1;
        }
        if (pos < 0 || !ok) break;
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
    uint32_t it = 0;
    // Releases this CTA's share of the accumulator: locally for the leader, on
    // the leader's barrier for its partner.
    auto release_acc = [&](uint32_t acc) {
      kb::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) {
          if (leader) kb::mbar_arrive(&sm.tempty[acc]);
          else kb::mbar_arrive_cluster(kb::map_to_cta(kb::smem_u32(&sm.tempty[acc]), 0u));
        } else {
          kb::mbar_arrive(&sm.tempty[acc]);
        }
      }
    };
    for (;; ++it) {
      int pos;
      if constexpr (kAG) {
        pos = 0;
        if (lane == 0) pos = read_tile(it);
        pos = __shfl_sync(0xffffffffu, pos, 0);
      } else {
        pos = sched_id + static_cast<int>(it) * sched_n;
        if (pos >= total_tiles) pos = -1;
      }
      if (pos < 0) break;
      int mbq, nb;
      tile_at(p, pos, mbq, nb);
      const int mb = kPair ? 2 * mbq + static_cast<int>(cta_rank) : mbq;
      const uint32_t acc = it & 1u;
      const uint32_t aph = (it >> 1) & 1u;
      // After a failed wait the loop keeps its shape (the named barriers below
      // must be reached by all four warps) but stops waiting.
      if (*sm.abort == 0 && !kb::mbar_wait_bounded(&sm.tfull[acc], aph, p.limit_ns, 2000)) {
        kb::report_status(p.status, KB_DEV_TIMEOUT_MBAR, SITE_EPI_TFULL, (uint32_t)pos, p.epoch);
        *sm.abort = 1;
      }
      kb::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      const int row0 = mb * BM;

      if constexpr (!kDirect) {
        // Four passes of 64 columns through two staging boxes; lane 0 owns the
        // bulk groups of this warp.  A box is rewritten only after the store that
        // last read it has finished reading (at most one younger group pending).
        const int gr0 = row0 + q * 32;
#pragma unroll 1
        for (int ps = 0; ps < BN / OUT_BOX_COLS; ++ps) {
          uint8_t* box = warp_epi + (ps & 1) * OUT_BOX_BYTES;
          if (lane == 0) kb::bulk_wait_group_read<1>();
          __syncwarp();
          const int col0 = nb * BN + ps * OUT_BOX_COLS;
          stage_box(taddr + ps * OUT_BOX_COLS, box, lane, p.bias, p.bias_scale, col0, p.N);
          if (ps == BN / OUT_BOX_COLS - 1) release_acc(acc);
          kb::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (gr0 < p.M && col0 < p.N) kb::tma_store_2d(&p.tmOut, box, col0, gr0);
            kb::bulk_commit_group();  // also when nothing was stored: one group per pass keeps the count simple
          }
        }
      } else {
        // A lane owns row (32 q + lane) of the tile and stores it 16 bytes at a
        // time.  RS: the row goes, without bias, into this rank's own staging
        // matrix (the partial product); then the owners of the tile's rows are told.
        const int gr = row0 + q * 32 + lane;
        bf16* row_ptr = kRS ? reinterpret_cast<bf16*>(p.peer_base[p.rank] + p.data_off) + rs_stage_elem(p, gr < p.M ? gr : 0)
                            : p.out + static_cast<size_t>(gr < p.M ? gr : 0) * p.N;
#pragma unroll 1
        for (int ps = 0; ps < BN / OUT_BOX_COLS; ++ps) {
          store_direct(taddr + ps * OUT_BOX_COLS, row_ptr, gr < p.M, kRS ? nullptr : p.bias, p.bias_scale,
                       nb * BN + ps * OUT_BOX_COLS, p.N);
        }
        release_acc(acc);
        if constexpr (kRS) {
          epi_bar_sync();
          if (et == 0 && row0 < p.M) {
            int last_row = row0 + BM - 1;
            if (last_row > p.M - 1) last_row = p.M - 1;
            const int tile_id = mb * p.NB + nb;
            kb::fence_sys();
            for (int o = row0 / p.rpo; o <= last_row / p.rpo; ++o) kb::st_relaxed_sys_u32(rs_flag(p, o, p.rank, tile_id), p.epoch);
          }
        }
      }
    }
    if constexpr (!kDirect) {
      if (lane == 0) kb::bulk_wait_group<0>();  // the staging boxes are read and the output is written before the CTA leaves
    }
    if (p.status != nullptr && p.timing && lane == 0 && !kRS) {
      atomicMax(&p.status[7], static_cast<uint32_t>((kb::globaltimer_ns() - t_start) / 1000));
    }
  } else if (kRS && warp >= 8) {
    // ------------------------------------------------ reduce-scatter reducer ----
    // Units of 64 rows x 128 columns of this rank's output shard, in ascending
    // row order (the order in which the tiles complete on all ranks), dealt
    // round-robin to the CTAs.  A unit waits for the tile's flag from every rank,
    // then sums the ranks' partials in ascending rank order in fp32, adds the
    // bias and writes the output.  Two 16-byte vectors per thread and up to
    // eight sources are in flight at a time.
    const int rt = tid - 256;
    const int row_begin = p.rank * p.rpo;
    const int row_end = row_begin + p.rpo;
    const int n_rg = (p.rpo + RS_ROW_GROUP - 1) / RS_ROW_GROUP;
    const int halves = BN / RS_UNIT_COLS;
    const int n_units = n_rg * p.NB * halves;
    uint64_t waited_ns = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x) {
      const int half = u % halves;
      const int t = u / halves;
      const int nb = t % p.NB;
      const int g = t / p.NB;
      const int r0 = row_begin + g * RS_ROW_GROUP;
      const int r1 = min(r0 + RS_ROW_GROUP, row_end);
      const int tile_id = (r0 / BM) * p.NB + nb;
      if (rt < p.world) {
        const uint64_t w0 = p.timing ? kb::globaltimer_ns() : 0;
        if (!kb::wait_flag_ge(rs_flag(p, p.rank, rt, tile_id), p.epoch, p.limit_ns, 256, true, true)) {
          kb::report_status(p.status, KB_DEV_TIMEOUT_FLAG, SITE_RS_FLAG, (uint32_t)rt, p.epoch);
        }
        if (p.timing) waited_ns += kb::globaltimer_ns() - w0;
      }
      comm_bar_sync();
      const int c0 = nb * BN + half * RS_UNIT_COLS;
      constexpr int VPR = RS_UNIT_COLS / 8;  // 16-byte vectors per unit row
      const int total = (r1 - r0) * VPR;
      auto finish = [&](float* accv, int row, int col) {
        if (p.bias != nullptr) {
          float bz[8];
          unpack8(*reinterpret_cast<const uint4*>(p.bias + col), bz);
#pragma unroll
          for (int e = 0; e < 8; ++e) accv[e] += p.bias_scale * bz[e];
        }
        *reinterpret_cast<uint4*>(p.out + static_cast<size_t>(row - row_begin) * p.N + col) = pack8(accv);
      };
      if (p.mc_base != nullptr) {
        // One multimem.ld_reduce per vector: the switch adds the ranks' values.
        // Eight vectors per thread in flight.
        const bf16* mc_stage = reinterpret_cast<const bf16*>(p.mc_base + p.data_off);
        for (int v0 = rt; v0 < total; v0 += 8 * 128) {
          uint4 x[8];
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const int v = v0 + b * 128;
            const int row = r0 + v / VPR, col = c0 + (v % VPR) * 8;
            x[b] = make_uint4(0u, 0u, 0u, 0u);
            if (v < total && col < p.N) x[b] = kb::multimem_ld_reduce_bf16x8(mc_stage + rs_stage_elem(p, row) + col);
          }
#pragma unroll
          for (int b = 0; b < 8; ++b) {
            const int v = v0 + b * 128;
            const int row = r0 + v / VPR, col = c0 + (v % VPR) * 8;
            if (v < total && col < p.N) {
              float accv[8];
              unpack8(x[b], accv);
              finish(accv, row, col);
            }
          }
        }
      } else {
        // Peer loads: two vectors per thread and up to eight sources in flight,
        // summed in ascending rank order.
        for (int v0 = rt; v0 < total; v0 += 2 * 128) {
          float accv[2][8];
          int rowv[2], colv[2];
          bool live[2];
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            const int v = v0 + b * 128;
            rowv[b] = r0 + v / VPR;
            colv[b] = c0 + (v % VPR) * 8;
            live[b] = v < total && colv[b] < p.N;
#pragma unroll
            for (int e = 0; e < 8; ++e) accv[b][e] = 0.f;
          }
#pragma unroll 1
          for (int s0 = 0; s0 < p.world; s0 += 8) {
            uint4 x[2][8];
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
              for (int sj = 0; sj < 8; ++sj) {
                x[b][sj] = make_uint4(0u, 0u, 0u, 0u);
                if (live[b] && s0 + sj < p.world) {
                  const bf16* src = reinterpret_cast<const bf16*>(p.peer_base[s0 + sj] + p.data_off) +
                                    rs_stage_elem(p, rowv[b]) + colv[b];
                  x[b][sj] = kb::ld_sys_v4(src);
                }
              }
            }
#pragma unroll
            for (int b = 0; b < 2; ++b) {
#pragma unroll
              for (int sj = 0; sj < 8; ++sj) {
                float f[8];
                unpack8(x[b][sj], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) accv[b][e] += f[e];
              }
            }
          }
#pragma unroll
          for (int b = 0; b < 2; ++b) {
            if (live[b]) finish(accv[b], rowv[b], colv[b]);
          }
        }
      }
    }
    if (p.status != nullptr && p.timing && rt < p.world) atomicMax(&p.status[5], static_cast<uint32_t>(waited_ns / 1000));
    if (p.status != nullptr && p.timing && rt == 0) {
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
    // GEMM reads its own rows in place): one peer store per rank, or a single
    // multimem store that the switch replicates.  Groups therefore arrive
    // everywhere in ascending order, which is the order in which the GEMMs
    // consume them.  When a CTA finds a group exhausted it fences and counts
    // itself done; the last one releases the group's flags on every rank and
    // rewinds both counters for the next call.
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
      const size_t dst_elem = ag_gather_elem(p, r_begin);
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
        if (p.mc_base != nullptr) {
          uint4* dstp = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.mc_base + p.data_off) + dst_elem);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const size_t v = base + u * 128 + ct;
            if (v < nvec) kb::multimem_st_v4(dstp + v, x[u]);
          }
        } else {
          for (int dd = dd0; dd < p.world; ++dd) {
            const int dst = (p.rank - dd + p.world) % p.world;
            uint4* dstp = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(p.peer_base[dst] + p.data_off) + dst_elem);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const size_t v = base + u * 128 + ct;
              if (v < nvec) kb::st_sys_v4(dstp + v, x[u]);
            }
          }
        }
      }
      if (ct == 0) {
        kb::fence_sys();
        const uint32_t old = atomicAdd(&counters[g], 1u);
        if (old == gridDim.x - 1u) {
          counters[g] = 0u;       // every CTA has counted itself: both counters start the next call at zero
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
    if (ct == 0 && p.status != nullptr && p.timing) {
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
int make_tmap(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_cols, uint32_t box_rows) {
  auto encode = KB_DRV(cuTensorMapEncodeTiled);
  if (encode == nullptr) return KB_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
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

// Environment switches, read once per process.
struct EnvConfig {
  bool no_pair;
  bool timing;
  bool tma_epilogue;
  int group_rows;
  EnvConfig() {
    const char* v = getenv("KB200_GEMM_NO_PAIR");
    no_pair = v != nullptr && v[0] == '1';
    v = getenv("KB200_GEMM_EPILOGUE");  // "tma" (default) or "direct"
    tma_epilogue = !(v != nullptr && v[0] == 'd');
    v = getenv("KB200_GEMM_TIMING");
    timing = v != nullptr && v[0] == '1';
    v = getenv("KB200_GEMM_GROUP_ROWS");
    group_rows = (v != nullptr && atoi(v) >= 256) ? atoi(v) : 1024;
  }
};
const EnvConfig& env_config() {
  static const EnvConfig cfg;
  return cfg;
}

// Fills the fields of the tile schedule.  Returns false when CTA pairs were
// asked for but the rows per rank are not a multiple of 256.
bool fill_schedule(GemmParams& p, int mode, int M, int N, int rank, int world, bool pair) {
  p.mode = world > 1 ? mode : KB_GEMM_PLAIN;
  p.M = M;
  p.N = N;
  p.world = world;
  p.rank = rank;
  p.MB = (M + BM - 1) / BM;
  p.NB = (N + BN - 1) / BN;
  const bool dist_mode = p.mode != KB_GEMM_PLAIN;
  p.rpo = dist_mode ? M / world : M;
  if (pair && dist_mode && (p.rpo % 256) != 0) return false;
  const int block_rows = pair ? 256 : 128;
  p.MBQ = (M + block_rows - 1) / block_rows;
  p.own_lo_q = dist_mode ? (rank * p.rpo) / block_rows : 0;
  p.ag_n_own = (p.mode == KB_GEMM_AG && (p.rpo % block_rows) == 0) ? p.rpo / block_rows : 0;
  p.rs_nq = (p.mode == KB_GEMM_RS && (p.rpo % block_rows) == 0) ? p.rpo / block_rows : 0;
  // 1024 rows are swept together (measured best among 512 to 4096 on 8192 x 8192 x 29568; for the all-gather
  // kernel it also makes the first group consist of this rank's own rows only at eight ranks).
  p.group = env_config().group_rows / block_rows;
  return true;
}

}  // namespace

// Host replica of the device tile schedule, for tests of the index arithmetic:
// position -> (scheduling block, column block) for the given problem and rank.
// Returns the number of positions, or -1 for invalid arguments.
extern "C" int kb_gemm_schedule(int mode, int M, int N, int rank, int world, int pair, int pos, int* block, int* nb) {
  if (M <= 0 || N <= 0 || world < 1 || rank < 0 || rank >= world || (mode != KB_GEMM_PLAIN && M % world != 0)) return -1;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  if (!fill_schedule(p, mode, M, N, rank, world, pair != 0)) return -1;
  const int total = p.MBQ * p.NB;
  if (pos >= 0 && pos < total && block != nullptr && nb != nullptr) tile_at(p, pos, *block, *nb);
  return total;
}

extern "C" uint64_t kb_gemm_rs_data_bytes(int M, int N, int world) {
  (void)world;
  return round_up(2ull * (uint64_t)M * N * 2, 256);  // two parities of this rank's [M, N] bf16 partial product
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
  return 1024;  // words 0..63 completion counters and 64..127 slice-claim counters of the pushes (at most eight groups are used), 128..129 tile-claim counters
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
  if (a->mode != KB_GEMM_PLAIN && a->mode != KB_GEMM_RS && a->mode != KB_GEMM_AG) {
    kb::set_error("kb_gemm: unknown mode %d", a->mode);
    return KB_ERR_ARG;
  }
  auto misaligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) != 0; };
  if (misaligned(a->A) || misaligned(a->B) || misaligned(a->out) || (a->bias && misaligned(a->bias))) {
    kb::set_error("kb_gemm: operand pointers must be 16-byte aligned");
    return KB_ERR_ARG;
  }
  const bool dist = a->mode != KB_GEMM_PLAIN && a->world > 1;
  int rpo = a->M;
  if (dist) {
    if (a->M % a->world != 0) {
      kb::set_error("kb_gemm: M=%d must be divisible by world=%d", a->M, a->world);
      return KB_ERR_ARG;
    }
    rpo = a->M / a->world;
    if (!((rpo % BM) == 0 || (BM % rpo) == 0)) {
      kb::set_error("kb_gemm: rows per rank (%d) must divide or be a multiple of %d", rpo, BM);
      return KB_ERR_ARG;
    }
    for (int r = 0; r < a->world; ++r) {
      if (a->peer_base[r] == nullptr) {
        kb::set_error("kb_gemm: peer_base[%d] is null", r);
        return KB_ERR_ARG;
      }
    }
  }

  // CTA pairs need 256-row scheduling blocks that do not straddle two ranks.
  // num_ctas bit 30 forces the single-CTA kernel (tests, comparisons).
  const EnvConfig& env = env_config();
  const bool forbid_pair = (a->num_ctas & (1 << 30)) != 0 || env.no_pair;
  const int req_ctas = a->num_ctas & ~(1 << 30);
  bool pair = !forbid_pair && a->M >= 256 && (!dist || (rpo % 256) == 0);
  int dev = 0, sms = 0;
  KB_CUDA_OK(cudaGetDevice(&dev));
  {
    static int cached_sms[64] = {0};
    if (dev >= 0 && dev < 64 && cached_sms[dev] > 0) {
      sms = cached_sms[dev];
    } else {
      KB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
      if (dev >= 0 && dev < 64) cached_sms[dev] = sms;
    }
  }
  int grid = req_ctas > 0 ? req_ctas : sms;
  if (grid > sms) grid = sms;
  if (pair) {
    grid &= ~1;
    if (grid < 2) pair = false;
  }

  GemmParams p;
  memset(&p, 0, sizeof(p));
  fill_schedule(p, a->mode, a->M, a->N, dist ? a->rank : 0, dist ? a->world : 1, pair);
  p.K = a->K;
  p.KB = (a->K + BK - 1) / BK;
  p.bias = static_cast<const bf16*>(a->bias);
  p.bias_scale = a->bias_scale;
  p.out = static_cast<bf16*>(a->out);
  p.epoch = a->epoch;
  p.status = a->status;
  p.limit_ns = a->wait_limit_ns ? a->wait_limit_ns : 2000000000ull;
  p.data_off = a->data_off;
  p.flag_off = a->flag_off;
  p.counter_off = a->counter_off;
  p.timing = env.timing ? 1 : 0;
  p.own_lo_mb = 0;
  p.own_hi_mb = p.MB - 1;
  const void* a_ptr = a->A;
  if (dist) {
    for (int r = 0; r < a->world; ++r) p.peer_base[r] = static_cast<char*>(a->peer_base[r]);
    p.mc_base = static_cast<char*>(a->mc_base);
    p.own_lo_mb = (a->rank * rpo) / BM;
    p.own_hi_mb = ((a->rank + 1) * rpo - 1) / BM;
    if (a->mode == KB_GEMM_AG) {
      p.a_local = static_cast<const bf16*>(a->A);
      const uint32_t parity = a->epoch & 1u;
      a_ptr = p.peer_base[a->rank] + a->data_off + (uint64_t)parity * a->M * a->K * 2;
    }
  }

  int rc = make_tmap(&p.tmA, a_ptr, a->M, a->K, BK, BM);
  if (rc != KB_OK) return rc;
  rc = make_tmap(&p.tmB, a->B, a->N, a->K, BK, pair ? 128 : BN);
  if (rc != KB_OK) return rc;
  if (p.mode == KB_GEMM_AG && (rpo % BM) == 0) {
    rc = make_tmap(&p.tmOwn, a->A, rpo, a->K, BK, BM);
    if (rc != KB_OK) return rc;
    p.ag_own_direct = 1;
  }
  const bool direct = p.mode == KB_GEMM_RS || !env.tma_epilogue;
  if (!direct) {
    rc = make_tmap(&p.tmOut, a->out, a->M, a->N, OUT_BOX_COLS, OUT_BOX_ROWS);
    if (rc != KB_OK) return rc;
  }

  const int total_units = p.MBQ * p.NB * (pair ? 2 : 1);
  if (p.mode == KB_GEMM_PLAIN && grid > total_units) grid = total_units;  // the fused modes keep every CTA: their extra warps share the transfers

  const int threads = p.mode == KB_GEMM_PLAIN ? THREADS_BASE : THREADS_COMM;
  const void* fns[2][2][3] = {
      {{(const void*)gemm_kernel<KB_GEMM_PLAIN, false, false>, nullptr, (const void*)gemm_kernel<KB_GEMM_AG, false, false>},
       {(const void*)gemm_kernel<KB_GEMM_PLAIN, false, true>, (const void*)gemm_kernel<KB_GEMM_RS, false, true>,
        (const void*)gemm_kernel<KB_GEMM_AG, false, true>}},
      {{(const void*)gemm_kernel<KB_GEMM_PLAIN, true, false>, nullptr, (const void*)gemm_kernel<KB_GEMM_AG, true, false>},
       {(const void*)gemm_kernel<KB_GEMM_PLAIN, true, true>, (const void*)gemm_kernel<KB_GEMM_RS, true, true>,
        (const void*)gemm_kernel<KB_GEMM_AG, true, true>}}};
  const void* fn = fns[pair ? 1 : 0][direct ? 1 : 0][p.mode];
  {
    static bool attr_set[64][2][2][3] = {};
    if (dev < 0 || dev >= 64 || !attr_set[dev][pair ? 1 : 0][direct ? 1 : 0][p.mode]) {
      KB_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
      if (dev >= 0 && dev < 64) attr_set[dev][pair ? 1 : 0][direct ? 1 : 0][p.mode] = true;
    }
  }
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
