// MoE dispatch / expert / combine executed by CPU ranks over a host-backed
// symmetric heap (KB_BACKEND_HOST).  It is the protocol of kernels/a2a.cu --
// sender-computed slots, rows and per-(source, expert) counts stored straight
// into the owner's segment, epoch flags with release/acquire ordering, pull
// combine in fixed k order -- with std::atomic in place of system-scope PTX and
// memcpy in place of peer stores.  It lets the routing arithmetic, the epoch
// protocol and the time-outs be exercised by processes without a GPU: a rank
// that never shows up makes the others return KB_ERR_TIMEOUT with its number,
// exactly as the device waits report a status instead of hanging.
//
// Reference counterpart of the algorithm: PyTorchAllToAll.dispatch / combine
// (reference.py:68-234); of the failure handling: the pool time-outs of
// eval.py:201,428.
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <vector>

#include <cuda_fp16.h>  // host-callable fp16 <-> fp32 conversions

#include "../common/host_util.h"
#include "../include/kb200.h"

namespace {

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
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN stays NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

inline float f16_to_f32(uint16_t h) {
  __half_raw r;
  r.x = h;
  return __half2float(__half(r));
}
inline uint16_t f32_to_f16(float f) {  // round to nearest even
  return static_cast<__half_raw>(__float2half_rn(f)).x;
}

struct Layout {
  int rank, world, E, El, k, H, T, cap, eb, dtype;
  size_t row_bytes;
  char* base[KB_MAX_WORLD];
  uint64_t recv_off, y_off, count_off, flag_off;
  uint8_t* rows(int on, uint64_t region, int src, int slot) const {
    return reinterpret_cast<uint8_t*>(base[on]) + region + (static_cast<size_t>(src) * cap + slot) * row_bytes;
  }
  int32_t* counts(int on, int src) const {
    return reinterpret_cast<int32_t*>(base[on] + count_off) + static_cast<size_t>(src) * El;
  }
  std::atomic<uint32_t>* flag(int on, int which, int src) const {
    // same layout as the kernels: one 128-byte line per (phase, source)
    return reinterpret_cast<std::atomic<uint32_t>*>(base[on] + flag_off) + static_cast<size_t>(which * KB_MAX_WORLD + src) * 32;
  }
};

// Waits until flag `which` of every source has reached `epoch`; on expiry names
// the first source that is missing.
int wait_all(const Layout& L, int which, uint32_t epoch, int64_t deadline, const char* phase) {
  for (int s = 0; s < L.world; ++s) {
    while (static_cast<int32_t>(L.flag(L.rank, which, s)->load(std::memory_order_acquire) - epoch) < 0) {
      if (now_ms() > deadline) {
        kb::set_error("a2a host: rank %d never finished %s of epoch %u (waited for by rank %d)", s, phase, epoch, L.rank);
        return KB_ERR_TIMEOUT;
      }
      usleep(20);
    }
  }
  return KB_OK;
}

float expert_scale(const Layout& L, int mode, int owner_rank, int local_expert) {
  if (mode == 1) return static_cast<float>(1 + owner_rank);
  if (mode == 2) return static_cast<float>(owner_rank * L.El + local_expert + 1) / static_cast<float>(L.E);
  return 1.0f;
}

void scale_row(const Layout& L, const uint8_t* src, uint8_t* dst, float scale) {
  if (L.dtype == 2) {
    const float* s = reinterpret_cast<const float*>(src);
    float* d = reinterpret_cast<float*>(dst);
    for (int i = 0; i < L.H; ++i) d[i] = s[i] * scale;
  } else if (L.dtype == 1) {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
    for (int i = 0; i < L.H; ++i) d[i] = f32_to_f16(f16_to_f32(s[i]) * scale);
  } else {
    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
    for (int i = 0; i < L.H; ++i) d[i] = f32_to_bf16(bf16_to_f32(s[i]) * scale);
  }
}

int make_layout(const KbA2aArgs* a, Layout& L) {
  if (a == nullptr || a->world < 1 || a->world > KB_MAX_WORLD || a->rank < 0 || a->rank >= a->world) {
    kb::set_error("a2a host: bad rank/world");
    return KB_ERR_ARG;
  }
  if (a->dtype < 0 || a->dtype > 2) {
    kb::set_error("a2a host: dtype %d not supported on the host path (bf16, fp16 and fp32 are)", a->dtype);
    return KB_ERR_ARG;
  }
  if (a->num_experts <= 0 || a->num_experts % a->world != 0 || a->num_tokens < 0 || a->num_tokens > a->max_tokens) {
    kb::set_error("a2a host: bad expert or token count");
    return KB_ERR_ARG;
  }
  L.rank = a->rank;
  L.world = a->world;
  L.E = a->num_experts;
  L.El = a->num_experts / a->world;
  L.k = a->topk;
  L.H = a->hidden;
  L.T = a->num_tokens;
  L.cap = a->max_tokens * a->topk;
  L.eb = a->elem_bytes;
  L.dtype = a->dtype;
  L.row_bytes = static_cast<size_t>(a->hidden) * a->elem_bytes;
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_base[r] == nullptr) {
      kb::set_error("a2a host: peer_base[%d] is null", r);
      return KB_ERR_ARG;
    }
    L.base[r] = static_cast<char*>(a->peer_base[r]);
  }
  L.recv_off = a->recv_off;
  L.y_off = a->y_off;
  L.count_off = a->count_off;
  L.flag_off = a->flag_off;
  return KB_OK;
}

int64_t deadline_of(int timeout_ms) { return now_ms() + (timeout_ms > 0 ? timeout_ms : 30000); }

// Slot of entry i = first slot of its expert in the owner's region for this
// source + number of earlier entries with the same expert.  Rows and counts go
// straight into the owners' segments, then the dispatch flag; returns once every
// source's rows have arrived here.
int dispatch_phase(const KbA2aArgs* a, const Layout& L, int64_t deadline) {
  const uint8_t* x = static_cast<const uint8_t*>(a->x);
  std::vector<int> tot(L.E, 0), off(L.E, 0), seen(L.E, 0);
  const int n = L.T * L.k;
  for (int i = 0; i < n; ++i) {
    const int e = a->indices[i];
    if (e < 0 || e >= L.E) {
      kb::set_error("a2a host: expert id %d out of range at entry %d", e, i);
      return KB_ERR_ARG;
    }
    ++tot[e];
  }
  for (int e = 0; e < L.E; ++e) off[e] = (e % L.El == 0) ? 0 : off[e - 1] + tot[e - 1];
  for (int i = 0; i < n; ++i) {
    const int e = a->indices[i];
    const int slot = off[e] + seen[e]++;
    if (slot >= L.cap) {
      kb::set_error("a2a host: slot %d beyond capacity %d", slot, L.cap);
      return KB_ERR_ARG;
    }
    a->slots[i] = slot;
    memcpy(L.rows(e / L.El, L.recv_off, L.rank, slot), x + static_cast<size_t>(i / L.k) * L.row_bytes, L.row_bytes);
  }
  for (int e = 0; e < L.E; ++e) L.counts(e / L.El, L.rank)[e % L.El] = tot[e];
  for (int r = 0; r < L.world; ++r) L.flag(r, 0, L.rank)->store(a->epoch, std::memory_order_release);
  return wait_all(L, 0, a->epoch, deadline, "its dispatch");
}

// y = scale(expert) * x for every received row.
void expert_phase(const KbA2aArgs* a, const Layout& L) {
  for (int s = 0; s < L.world; ++s) {
    int row = 0;
    for (int le = 0; le < L.El; ++le) {
      int c = L.counts(L.rank, s)[le];
      if (c < 0) c = 0;
      const float scale = expert_scale(L, a->scale_mode, L.rank, le);
      for (int j = 0; j < c && row < L.cap; ++j, ++row) {
        scale_row(L, L.rows(L.rank, L.recv_off, s, row), L.rows(L.rank, L.y_off, s, row), scale);
      }
    }
  }
}

// Publishes this rank's expert outputs, waits for everybody's, then pulls the k
// rows of every token and sums them in fp32 in k order.
int combine_phase(const KbA2aArgs* a, const Layout& L, int64_t deadline) {
  uint8_t* out = static_cast<uint8_t*>(a->out);
  for (int r = 0; r < L.world; ++r) L.flag(r, 1, L.rank)->store(a->epoch, std::memory_order_release);
  const int rc = wait_all(L, 1, a->epoch, deadline, "its expert pass");
  if (rc != KB_OK) return rc;
  std::vector<float> acc(L.H);
  for (int t = 0; t < L.T; ++t) {
    for (int i = 0; i < L.H; ++i) acc[i] = 0.f;
    for (int kk = 0; kk < L.k; ++kk) {
      const int e = a->indices[t * L.k + kk];
      const uint8_t* row = L.rows(e / L.El, L.y_off, L.rank, a->slots[t * L.k + kk]);
      const float w = a->weights[t * L.k + kk];
      if (L.dtype == 2) {
        const float* r = reinterpret_cast<const float*>(row);
        for (int i = 0; i < L.H; ++i) acc[i] += w * r[i];
      } else if (L.dtype == 1) {
        const uint16_t* r = reinterpret_cast<const uint16_t*>(row);
        for (int i = 0; i < L.H; ++i) acc[i] += w * f16_to_f32(r[i]);
      } else {
        const uint16_t* r = reinterpret_cast<const uint16_t*>(row);
        for (int i = 0; i < L.H; ++i) acc[i] += w * bf16_to_f32(r[i]);
      }
    }
    if (L.dtype == 2) {
      memcpy(out + static_cast<size_t>(t) * L.row_bytes, acc.data(), L.row_bytes);
    } else if (L.dtype == 1) {
      uint16_t* o = reinterpret_cast<uint16_t*>(out + static_cast<size_t>(t) * L.row_bytes);
      for (int i = 0; i < L.H; ++i) o[i] = f32_to_f16(acc[i]);
    } else {
      uint16_t* o = reinterpret_cast<uint16_t*>(out + static_cast<size_t>(t) * L.row_bytes);
      for (int i = 0; i < L.H; ++i) o[i] = f32_to_bf16(acc[i]);
    }
  }
  return KB_OK;
}

}  // namespace

// Same arguments as the device entry points; `a->peer_base` are host pointers of
// a KB_BACKEND_HOST heap, `a->slots` host scratch, x / indices / weights / out
// host tensors.  dtype 0 (bf16), 1 (fp16) and 2 (fp32).
extern "C" int kb_a2a_round_trip_host(const KbA2aArgs* a, int timeout_ms) {
  Layout L;
  int rc = make_layout(a, L);
  if (rc != KB_OK) return rc;
  const int64_t deadline = deadline_of(timeout_ms);
  rc = dispatch_phase(a, L, deadline);
  if (rc != KB_OK) return rc;
  expert_phase(a, L);
  return combine_phase(a, L, deadline);
}

// The phases on their own, for callers that run their own expert computation
// between them: after kb_a2a_dispatch_host the receive region and the counts of
// this rank are complete; kb_a2a_combine_host expects the expert outputs in the
// y region, row for row, and uses the slots the dispatch of the same epoch left
// in `a->slots`.
extern "C" int kb_a2a_dispatch_host(const KbA2aArgs* a, int timeout_ms) {
  Layout L;
  const int rc = make_layout(a, L);
  if (rc != KB_OK) return rc;
  return dispatch_phase(a, L, deadline_of(timeout_ms));
}

extern "C" int kb_a2a_combine_host(const KbA2aArgs* a, int timeout_ms) {
  Layout L;
  const int rc = make_layout(a, L);
  if (rc != KB_OK) return rc;
  if (a->out == nullptr || a->weights == nullptr) {
    kb::set_error("a2a host: combine needs weights and an output");
    return KB_ERR_ARG;
  }
  return combine_phase(a, L, deadline_of(timeout_ms));
}
