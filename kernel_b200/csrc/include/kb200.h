// C ABI of libkb200: symmetric memory, the fused sm_100a kernels and their
// host launchers.  Everything is plain C so that Python can bind it with
// ctypes; no torch or pybind headers are involved.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KB_MAX_WORLD 16

// ---- error / status codes -------------------------------------------------
enum KbStatus {
  KB_OK = 0,
  KB_ERR_CUDA = 1,         // a CUDA runtime/driver call failed (see kb_last_error)
  KB_ERR_ARG = 2,          // invalid argument (shape, alignment, size limit)
  KB_ERR_TIMEOUT = 3,      // host-side rendezvous timed out
  KB_ERR_IO = 4,           // socket / fd error
  KB_ERR_UNSUPPORTED = 5,  // feature not available on this device/driver
};

// Device-side status word layout (uint32_t[8], zero = healthy).  A kernel that
// gives up on a wait records the first failure here and returns normally.
enum KbDevCode {
  KB_DEV_OK = 0,
  KB_DEV_TIMEOUT_MBAR = 1,    // intra-CTA pipeline barrier never completed
  KB_DEV_TIMEOUT_FLAG = 2,    // a peer's flag never reached the expected epoch
  KB_DEV_BAD_INDEX = 3,       // a bounds check rejected a computed slot/offset
};
// status[0]=code, [1]=site id, [2]=peer/tile waited on, [3]=epoch, [4]=blockIdx

const char* kb_last_error(void);

// ---- fd exchange (host only; testable without a GPU) -----------------------
// All ranks call with the same session/tag.  Rank r contributes `my_fd`
// (or -1 for "nothing"); on return out_fds[p] holds a duplicate of rank p's fd
// (or -1).  out_fds[rank] is a dup of my_fd.  Returns KbStatus.
int kb_fd_allgather(const char* session, const char* tag, int rank, int world, int my_fd, int* out_fds,
                    int timeout_ms);

// ---- symmetric heap ---------------------------------------------------------
enum KbBackend {
  KB_BACKEND_HOST = 0,  // memfd + mmap; CPU-only processes (tests, gloo ranks)
  KB_BACKEND_VMM = 1,   // cuMemCreate + POSIX fd export/import + cuMemMap
  KB_BACKEND_IPC = 2,   // cudaMalloc + cudaIpc handles (no multicast possible)
};

typedef struct KbSymmHeap KbSymmHeap;

// Phase 1: allocate the local segment and export it.  For KB_BACKEND_IPC the
// 64-byte handle is written to ipc_handle_out and exchanged by the caller.
int kb_symm_create(int backend, int rank, int world, uint64_t bytes, int device, KbSymmHeap** out);
uint64_t kb_symm_segment_bytes(const KbSymmHeap* h);
int kb_symm_local_fd(const KbSymmHeap* h);
int kb_symm_ipc_handle(const KbSymmHeap* h, void* out64);
// Phase 2: map every peer.  `fds` (VMM/HOST) or `ipc_handles` (IPC, world*64
// bytes) come from the exchange.  After this, kb_symm_peer_ptr works.
int kb_symm_map_peers(KbSymmHeap* h, const int* fds, const void* ipc_handles);
void* kb_symm_peer_ptr(const KbSymmHeap* h, int peer);
void* kb_symm_local_ptr(const KbSymmHeap* h);
// Optional NVLS multicast (VMM backend only).  Step A on rank 0 creates the
// object and returns its fd; step B on every rank imports (fd from rank 0),
// adds its device; step C (after a barrier across ranks) binds memory and maps.
int kb_symm_mc_supported(int device);
int kb_symm_mc_create(KbSymmHeap* h, int* fd_out);
int kb_symm_mc_join(KbSymmHeap* h, int fd_from_rank0);
int kb_symm_mc_bind(KbSymmHeap* h);
void* kb_symm_mc_ptr(const KbSymmHeap* h);
int kb_symm_destroy(KbSymmHeap* h);
// NVLS primitives over the multicast mapping (kernels/nvls_util.cu); bytes a multiple of 16.
// Store: every rank's segment receives `bytes` from local `src` at the offset `mc_dst` has in the mapping.
// Reduce: local `dst` receives the sum over all ranks of the bf16 values at `mc_src` (fp32 accumulation).
int kb_multimem_store(void* mc_dst, const void* src, uint64_t bytes, void* stream);
int kb_multimem_reduce_bf16(void* dst, const void* mc_src, uint64_t bytes, void* stream);

// Host-side epoch barrier over a KB_BACKEND_HOST heap (CPU atomics on the
// shared segment); `pad_off` is the byte offset of a world*4-byte flag pad.
int kb_symm_host_barrier(KbSymmHeap* h, uint64_t pad_off, uint32_t epoch, int timeout_ms);

// ---- device utilities -------------------------------------------------------
// Bounded wait kernel: waits until flag i >= want for i < n, or gives up
// after limit_ns and records KB_DEV_TIMEOUT_FLAG in status.
// Flag i is the word flags[i * stride_words].
int kb_wait_flags(const uint32_t* flags, int n, int stride_words, uint32_t want, uint64_t limit_ns, uint32_t* status,
                  void* stream);
// Cross-rank device barrier: post `epoch` into slot `rank` of every peer's pad,
// then wait for all `world` slots of the local pad.
int kb_device_barrier(void* const* peer_bases, uint64_t pad_off, int rank, int world, uint32_t epoch,
                      uint64_t limit_ns, uint32_t* status, void* stream);

// ---- GEMM family (tcgen05 / TMEM / TMA) ---------------------------------------
enum KbGemmMode {
  KB_GEMM_PLAIN = 0,  // out[M,N] = A[M,K] * B[N,K]^T (+ bias)
  KB_GEMM_RS = 1,     // K-sharded partials reduced into the row owner's shard
  KB_GEMM_AG = 2,     // A row-shards pushed to all peers while the GEMM runs
};

typedef struct KbGemmArgs {
  int mode;
  int M, N, K;             // GEMM extents seen by this rank (AG: M is the gathered M)
  const void* A;           // bf16 [M,K] (AG: local shard [M/world, K])
  const void* B;           // bf16 [N,K]
  const void* bias;        // bf16 [N] or NULL
  float bias_scale;        // multiplies bias (1, or world for per-rank-bias semantics)
  void* out;               // bf16; PLAIN/AG: [M,N]; RS: [M/world, N]
  int rank, world;
  uint32_t epoch;          // strictly increasing per call on a workspace
  void* peer_base[KB_MAX_WORLD];  // symmetric heap bases (RS/AG)
  uint64_t data_off;       // RS: this rank's partial product, bf16 [2][M][N], pulled by the row owners; AG: gather [2][M][K]
  uint64_t flag_off;       // RS: flags [2][world][tiles]; AG: flags [2][world][m_blocks]
  uint64_t counter_off;    // AG: local push counters [world][chunks] (uint32)
  uint32_t* status;        // device uint32[8]
  uint64_t wait_limit_ns;  // bound for every device-side wait
  int num_ctas;            // 0 = one per SM
  void* mc_base;           // multicast mapping of the heap (kb_symm_mc_ptr) or NULL: with it the RS reduction uses
                           // multimem.ld_reduce and the AG pushes multimem.st; without it peer loads and stores
} KbGemmArgs;

int kb_gemm(const KbGemmArgs* args, void* stream);
// The fused modes (RS, AG) run by a CPU rank over a KB_BACKEND_HOST heap: same
// schedule, staging layouts, flags and rounding points as the kernel (symm/gemm_host.cpp).
int kb_gemm_host(const KbGemmArgs* args, int timeout_ms);
// Host replica of the kernel's static tile schedule (tests of the index arithmetic).
int kb_gemm_schedule(int mode, int M, int N, int rank, int world, int pair, int pos, int* block, int* nb);
// Bytes each rank needs in the symmetric heap for the given problem.
uint64_t kb_gemm_rs_data_bytes(int M, int N, int world);
uint64_t kb_gemm_rs_flag_bytes(int M, int N, int world);
uint64_t kb_gemm_ag_data_bytes(int M, int K);
uint64_t kb_gemm_ag_flag_bytes(int M, int world);
uint64_t kb_gemm_ag_counter_bytes(int M, int world);

// ---- MoE dispatch / combine ----------------------------------------------------
typedef struct KbA2aArgs {
  int rank, world;
  int num_experts, topk, hidden, max_tokens;  // max_tokens: per-rank capacity
  int num_tokens;                             // tokens on this rank this call
  int elem_bytes;                             // 2 (bf16/fp16) or 4 (fp32)
  int dtype;                                  // 0 bf16, 1 fp16, 2 fp32
  const void* x;                              // [T, H]
  const int32_t* indices;                     // [T, k] global expert ids
  const float* weights;                       // [T, k]
  void* out;                                  // [T, H]
  int32_t* slots;                             // local scratch [max_tokens*topk]
  uint32_t epoch;
  void* peer_base[KB_MAX_WORLD];
  uint64_t recv_off;    // [world][max_tokens*topk][H] rows received from each source
  uint64_t y_off;       // same shape: expert outputs, pulled by the sources
  uint64_t count_off;   // int32 [world][experts_per_rank]
  uint64_t flag_off;    // kb_a2a_flag_bytes(): dispatch-done and y-ready epochs, flag (phase, source) at word
                        // (phase * KB_MAX_WORLD + source) * kb_a2a_flag_stride_words(), one 128-byte line each
  uint64_t sync_off;    // kb_a2a_sync_bytes(): local block counters and the arrival words of the fused launch
  int scale_mode;       // 0: y = x; 1: y = x*(1+rank); 2: y = x*(expert_id+1)/num_experts
  uint32_t* status;
  uint64_t wait_limit_ns;
  int num_ctas;
  uint64_t* trace;      // optional device uint64[16]: globaltimer stamps of CTA 0 at the phase boundaries
  uint64_t meta_off;    // kb_a2a_meta_bytes(): expert lists and weights of the one-launch round trip's unique rows
  int32_t* rank_slots;  // local scratch [max_tokens * world] of the one-launch round trip
  uint64_t ll_off;      // kb_a2a_ll_bytes(): landing areas of the low-latency round trip; 0 = not allocated
  int ll_max_tokens;    // rows per source those areas were sized for (the context's max_tokens)
} KbA2aArgs;

uint64_t kb_a2a_rows_bytes(int world, int max_tokens, int topk, int hidden, int elem_bytes);
uint64_t kb_a2a_meta_bytes(int world, int max_tokens, int topk);
// Low-latency round trip (contexts of at most kb_a2a_ll_max_tokens() tokens per rank): bytes of its landing
// areas, 0 when max_tokens is too large for it.
int kb_a2a_ll_max_tokens(void);
uint64_t kb_a2a_ll_bytes(int world, int max_tokens, int topk, int hidden, int elem_bytes);
uint64_t kb_a2a_flag_bytes(void);
uint64_t kb_a2a_sync_bytes(void);
int kb_a2a_flag_stride_words(void);
// Posts this rank's y-ready flag of args->epoch on every rank (after the caller's own expert computation).
int kb_a2a_post_ready(const KbA2aArgs* a, void* stream);
int kb_a2a_dispatch(const KbA2aArgs* a, void* stream);
int kb_a2a_expert_scale(const KbA2aArgs* a, void* stream);
int kb_a2a_combine(const KbA2aArgs* a, void* stream);
// The same round trip executed by a CPU rank over a KB_BACKEND_HOST heap (all
// pointers are host pointers; bf16, fp16 and fp32).  Returns KB_ERR_TIMEOUT naming
// the rank that never arrived.  The dispatch and combine phases are also callable
// on their own, around an expert computation of the caller.
int kb_a2a_round_trip_host(const KbA2aArgs* a, int timeout_ms);
// The low-latency protocol (flags inside the data, landing areas at a->ll_off) for CPU ranks.
int kb_a2a_round_trip_host_ll(const KbA2aArgs* a, int timeout_ms);
int kb_a2a_dispatch_host(const KbA2aArgs* a, int timeout_ms);
int kb_a2a_combine_host(const KbA2aArgs* a, int timeout_ms);
// dispatch + simulated expert + combine in ONE cooperative launch.
int kb_a2a_round_trip(const KbA2aArgs* a, void* stream);

#ifdef __cplusplus
}
#endif
