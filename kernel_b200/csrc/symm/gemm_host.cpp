// GEMM + reduce-scatter and all-gather + GEMM executed by CPU ranks over a
// host-backed symmetric heap (KB_BACKEND_HOST).  It is the protocol of
// kernels/gemm_sm100.cu with one worker per rank: the same 128 x 256 tiles
// visited in the order of the kernel's static schedule (kb_gemm_schedule), the
// same staging layouts (this rank's [parity][M][N] bf16 partial product for the
// reduce-scatter, which the row owners pull; [parity][row][K] gathered rows for
// the all-gather), the same per-(source, tile) and per-(source, row block) epoch
// flags with release/acquire ordering, fp32 accumulation, and the ranks' bf16
// partials added in fp32 in ascending rank order before the bias and the one
// rounding of the result.
// std::atomic stands in for system-scope PTX and memcpy for peer stores.
//
// Purpose: the index arithmetic, the epoch/parity protocol and the time-outs
// of the fused GEMMs can be exercised by processes without a GPU; a rank that
// never arrives makes the others return KB_ERR_TIMEOUT with its number, as the
// device waits report a status instead of hanging.
//
// Reference counterpart of the arithmetic: gemm_rs/submission.py:5-29 (matmul,
// bias, reduce_scatter_tensor); of the failure handling: eval.py:201,428.
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <vector>

#include "../common/host_util.h"
#include "../include/kb200.h"

namespace {

constexpr int BM = 128;
constexpr int BN = 256;

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {  // round to nearest even
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

struct Ctx {
  const KbGemmArgs* a;
  int MB, NB, rpo;
  uint32_t parity;
  int64_t deadline;
  char* base(int r) const { return static_cast<char*>(a->peer_base[r]); }
  // reduce-scatter
  std::atomic<uint32_t>* rs_flag(int on, int src, int tile) const {
    return reinterpret_cast<std::atomic<uint32_t>*>(base(on) + a->flag_off) +
           (static_cast<size_t>(parity) * a->world + src) * (static_cast<size_t>(MB) * NB) + tile;
  }
  // row `row` of rank `on`'s partial product of this epoch
  uint16_t* rs_row(int on, int row) const {
    return reinterpret_cast<uint16_t*>(base(on) + a->data_off) +
           (static_cast<size_t>(parity) * a->M + row) * static_cast<size_t>(a->N);
  }
  // all-gather
  std::atomic<uint32_t>* ag_flag(int on, int src, int mb) const {
    return reinterpret_cast<std::atomic<uint32_t>*>(base(on) + a->flag_off) +
           (static_cast<size_t>(parity) * a->world + src) * MB + mb;
  }
  uint16_t* ag_row(int on, int row) const {
    return reinterpret_cast<uint16_t*>(base(on) + a->data_off) +
           (static_cast<size_t>(parity) * a->M + row) * static_cast<size_t>(a->K);
  }
};

int wait_flag(const Ctx& c, std::atomic<uint32_t>* f, int src, const char* what) {
  while (static_cast<int32_t>(f->load(std::memory_order_acquire) - c.a->epoch) < 0) {
    if (now_ms() > c.deadline) {
      kb::set_error("gemm host: rank %d never delivered its %s of epoch %u (waited for by rank %d)", src, what, c.a->epoch,
                    c.a->rank);
      return KB_ERR_TIMEOUT;
    }
    usleep(20);
  }
  return KB_OK;
}

// acc[rows x cols] = A[rows x K] * B[cols x K]^T in fp32; `arow(i)` gives the bf16 row i of A.
template <typename RowFn>
void tile_matmul(RowFn arow, int rows, const uint16_t* B, int col0, int cols, int K, std::vector<float>& bt, float* acc) {
  // B tile transposed to [K][cols] fp32 once, then rank-1 updates along k (vectorisable inner loop)
  bt.resize(static_cast<size_t>(K) * cols);
  for (int j = 0; j < cols; ++j) {
    const uint16_t* b = B + static_cast<size_t>(col0 + j) * K;
    for (int k = 0; k < K; ++k) bt[static_cast<size_t>(k) * cols + j] = bf16_to_f32(b[k]);
  }
  for (int i = 0; i < rows; ++i) {
    float* out = acc + static_cast<size_t>(i) * cols;
    for (int j = 0; j < cols; ++j) out[j] = 0.f;
    const uint16_t* ar = arow(i);
    for (int k = 0; k < K; ++k) {
      const float av = bf16_to_f32(ar[k]);
      const float* brow = bt.data() + static_cast<size_t>(k) * cols;
      for (int j = 0; j < cols; ++j) out[j] += av * brow[j];
    }
  }
}

int run_rs(const Ctx& c) {
  const KbGemmArgs* a = c.a;
  const uint16_t* A = static_cast<const uint16_t*>(a->A);
  const uint16_t* B = static_cast<const uint16_t*>(a->B);
  const uint16_t* bias = static_cast<const uint16_t*>(a->bias);
  uint16_t* out = static_cast<uint16_t*>(a->out);
  const int total = kb_gemm_schedule(KB_GEMM_RS, a->M, a->N, a->rank, a->world, 0, -1, nullptr, nullptr);
  if (total < 0) {
    kb::set_error("gemm host: bad problem for the schedule");
    return KB_ERR_ARG;
  }
  // GEMM part: every tile of this rank's partial product goes, as bf16, into its
  // own staging matrix; the owners of the tile's rows are told.  Nothing here
  // waits for a peer.
  std::vector<float> acc(static_cast<size_t>(BM) * BN), bt;
  for (int pos = 0; pos < total; ++pos) {
    int mb = 0, nb = 0;
    kb_gemm_schedule(KB_GEMM_RS, a->M, a->N, a->rank, a->world, 0, pos, &mb, &nb);
    const int r0 = mb * BM, rows = (a->M - r0 < BM) ? a->M - r0 : BM;
    const int c0 = nb * BN, cols = (a->N - c0 < BN) ? a->N - c0 : BN;
    const int tile = mb * c.NB + nb;
    tile_matmul([&](int i) { return A + static_cast<size_t>(r0 + i) * a->K; }, rows, B, c0, cols, a->K, bt, acc.data());
    for (int i = 0; i < rows; ++i) {
      uint16_t* dst = c.rs_row(a->rank, r0 + i) + c0;
      const float* src = acc.data() + static_cast<size_t>(i) * cols;
      for (int j = 0; j < cols; ++j) dst[j] = f32_to_bf16(src[j]);
    }
    for (int o = r0 / c.rpo; o <= (r0 + rows - 1) / c.rpo; ++o) {
      c.rs_flag(o, a->rank, tile)->store(a->epoch, std::memory_order_release);
    }
  }
  // Reduction part: the rows this rank owns, in units of 64 rows x 128 columns in
  // ascending row order; a unit waits for its tile's flag from every rank and
  // pulls the partials.
  constexpr int RG = 64, UC = 128;
  const int row_begin = a->rank * c.rpo, row_end = row_begin + c.rpo;
  const int n_rg = (c.rpo + RG - 1) / RG;
  std::vector<float> sum(UC);
  for (int g = 0; g < n_rg; ++g) {
    const int r0 = row_begin + g * RG, r1 = (r0 + RG < row_end) ? r0 + RG : row_end;
    for (int nb = 0; nb < c.NB; ++nb) {
      const int tile = (r0 / BM) * c.NB + nb;
      for (int s = 0; s < a->world; ++s) {
        const int rc = wait_flag(c, c.rs_flag(a->rank, s, tile), s, "partial tile");
        if (rc != KB_OK) return rc;
      }
      for (int half = 0; half < BN / UC; ++half) {
        const int c0 = nb * BN + half * UC;
        const int cols = (a->N - c0 < UC) ? a->N - c0 : UC;
        if (cols <= 0) continue;
        for (int row = r0; row < r1; ++row) {
          for (int j = 0; j < cols; ++j) sum[j] = 0.f;
          for (int s = 0; s < a->world; ++s) {
            const uint16_t* st = c.rs_row(s, row) + c0;
            for (int j = 0; j < cols; ++j) sum[j] += bf16_to_f32(st[j]);
          }
          uint16_t* o = out + static_cast<size_t>(row - row_begin) * a->N + c0;
          for (int j = 0; j < cols; ++j) {
            const float b = bias != nullptr ? a->bias_scale * bf16_to_f32(bias[c0 + j]) : 0.f;
            o[j] = f32_to_bf16(sum[j] + b);
          }
        }
      }
    }
  }
  return KB_OK;
}

int run_ag(const Ctx& c) {
  const KbGemmArgs* a = c.a;
  const uint16_t* A = static_cast<const uint16_t*>(a->A);  // this rank's rows [rpo, K]
  const uint16_t* B = static_cast<const uint16_t*>(a->B);
  const uint16_t* bias = static_cast<const uint16_t*>(a->bias);
  uint16_t* out = static_cast<uint16_t*>(a->out);
  const int row_lo = a->rank * c.rpo;
  // push: this rank's rows into every peer's gathered buffer, then one flag per row block it has rows in
  for (int step = 1; step < a->world; ++step) {
    const int dst = (a->rank + step) % a->world;
    memcpy(c.ag_row(dst, row_lo), A, static_cast<size_t>(c.rpo) * a->K * 2);
    for (int mb = row_lo / BM; mb <= (row_lo + c.rpo - 1) / BM; ++mb) {
      c.ag_flag(dst, a->rank, mb)->store(a->epoch, std::memory_order_release);
    }
  }
  const int total = kb_gemm_schedule(KB_GEMM_AG, a->M, a->N, a->rank, a->world, 0, -1, nullptr, nullptr);
  if (total < 0) {
    kb::set_error("gemm host: bad problem for the schedule");
    return KB_ERR_ARG;
  }
  std::vector<float> acc(static_cast<size_t>(BM) * BN), bt;
  std::vector<char> ready(c.MB, 0);
  for (int pos = 0; pos < total; ++pos) {
    int mb = 0, nb = 0;
    kb_gemm_schedule(KB_GEMM_AG, a->M, a->N, a->rank, a->world, 0, pos, &mb, &nb);
    const int r0 = mb * BM, rows = (a->M - r0 < BM) ? a->M - r0 : BM;
    const int c0 = nb * BN, cols = (a->N - c0 < BN) ? a->N - c0 : BN;
    if (!ready[mb]) {
      for (int s = r0 / c.rpo; s <= (r0 + rows - 1) / c.rpo; ++s) {
        if (s == a->rank) continue;
        const int rc = wait_flag(c, c.ag_flag(a->rank, s, mb), s, "rows");
        if (rc != KB_OK) return rc;
      }
      ready[mb] = 1;
    }
    auto arow = [&](int i) -> const uint16_t* {
      const int gr = r0 + i;
      if (gr / c.rpo == a->rank) return A + static_cast<size_t>(gr - row_lo) * a->K;  // own rows in place
      return c.ag_row(a->rank, gr);
    };
    tile_matmul(arow, rows, B, c0, cols, a->K, bt, acc.data());
    for (int i = 0; i < rows; ++i) {
      const float* row = acc.data() + static_cast<size_t>(i) * cols;
      uint16_t* o = out + static_cast<size_t>(r0 + i) * a->N + c0;
      for (int j = 0; j < cols; ++j) {
        const float b = bias != nullptr ? a->bias_scale * bf16_to_f32(bias[c0 + j]) : 0.f;
        o[j] = f32_to_bf16(row[j] + b);
      }
    }
  }
  return KB_OK;
}

}  // namespace

// Same argument block as kb_gemm; `peer_base` are host pointers of a
// KB_BACKEND_HOST heap, A / B / bias / out host bf16 tensors.  Modes KB_GEMM_RS
// and KB_GEMM_AG with world >= 2 (a single rank has nothing to exchange).
extern "C" int kb_gemm_host(const KbGemmArgs* a, int timeout_ms) {
  if (a == nullptr || a->world < 2 || a->world > KB_MAX_WORLD || a->rank < 0 || a->rank >= a->world) {
    kb::set_error("gemm host: bad rank/world (needs world >= 2)");
    return KB_ERR_ARG;
  }
  if (a->mode != KB_GEMM_RS && a->mode != KB_GEMM_AG) {
    kb::set_error("gemm host: mode %d is not a fused mode", a->mode);
    return KB_ERR_ARG;
  }
  if (a->M <= 0 || a->N <= 0 || a->K <= 0 || a->M % a->world != 0) {
    kb::set_error("gemm host: need M, N, K > 0 and M divisible by the world size (got %d %d %d / %d)", a->M, a->N, a->K, a->world);
    return KB_ERR_ARG;
  }
  Ctx c;
  c.a = a;
  c.MB = (a->M + BM - 1) / BM;
  c.NB = (a->N + BN - 1) / BN;
  c.rpo = a->M / a->world;
  if (c.rpo % BM != 0 && BM % c.rpo != 0) {
    kb::set_error("gemm host: rows per rank (%d) must divide or be a multiple of %d", c.rpo, BM);
    return KB_ERR_ARG;
  }
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_base[r] == nullptr) {
      kb::set_error("gemm host: peer_base[%d] is null", r);
      return KB_ERR_ARG;
    }
  }
  if (a->A == nullptr || a->B == nullptr || a->out == nullptr) {
    kb::set_error("gemm host: null operand");
    return KB_ERR_ARG;
  }
  c.parity = a->epoch & 1u;
  c.deadline = now_ms() + (timeout_ms > 0 ? timeout_ms : 30000);
  return a->mode == KB_GEMM_RS ? run_rs(c) : run_ag(c);
}
