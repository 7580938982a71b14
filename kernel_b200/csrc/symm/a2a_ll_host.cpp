// The low-latency MoE round trip (kernels/a2a_ll.cuh) executed by CPU ranks over
// a host-backed symmetric heap: the same wire format (every 8 bytes carry 4 bytes
// of payload and the call's epoch, written and read as one 8-byte atomic), the
// same landing areas, the same slot arithmetic, the same alternation of the count
// lines with the epoch's parity, and the same rounding points; no flag, counter or
// fence besides the data.  It lets processes without a GPU exercise what the
// protocol relies on: that a unit is rewritten only after its reader's answer to
// the previous call has come back, that a rank which sends a peer nothing can be
// one call ahead of it but never two, and that a missing rank ends the others'
// polls with KB_ERR_TIMEOUT naming it.
//
// The reference has no counterpart (six collectives and four host synchronisations
// per round trip, submission.py:59-163).
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
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
  __half_raw r;
  r.x = h;
  return __half2float(__half(r));
}
inline uint16_t f32_to_f16(float f) { return static_cast<__half_raw>(__float2half_rn(f)).x; }

using Unit = std::atomic<uint64_t>;  // {payload word, epoch}

// The landing areas of one rank, as a2a_ll.cuh lays them out.
struct LL {
  int rank, world, E, El, k, H, T, tmax, dtype;
  size_t row_bytes, words;  // payload bytes and 4-byte words per row
  uint32_t epoch;
  char* base[KB_MAX_WORLD];
  uint64_t off;
  size_t row2, back_off, meta_off, cnt_off;
  Unit* row(int on, bool back, int src, int slot) const {
    return reinterpret_cast<Unit*>(base[on] + off + (back ? back_off : 0) + (static_cast<size_t>(src) * tmax + slot) * row2);
  }
  Unit* meta(int on, int src, int slot) const {
    return reinterpret_cast<Unit*>(base[on] + off + meta_off) + (static_cast<size_t>(src) * tmax + slot) * static_cast<size_t>(2 * k + 2);
  }
  Unit* cnt(int on, int src) const {
    return reinterpret_cast<Unit*>(base[on] + off + cnt_off + (static_cast<size_t>(epoch & 1u) * world + src) * 128);
  }
};

inline void put(Unit* u, uint32_t payload, uint32_t epoch) {
  u->store(static_cast<uint64_t>(payload) | (static_cast<uint64_t>(epoch) << 32), std::memory_order_relaxed);
}
// Polls a unit until it carries `epoch`.
inline bool get(const Unit* u, uint32_t epoch, int64_t deadline, uint32_t* payload) {
  for (uint32_t spins = 0;; ++spins) {
    const uint64_t v = u->load(std::memory_order_relaxed);
    if (static_cast<uint32_t>(v >> 32) == epoch) {
      *payload = static_cast<uint32_t>(v);
      return true;
    }
    if ((spins & 0x3ffu) == 0x3ffu) {
      if (now_ms() > deadline) return false;
      usleep(20);
    }
  }
}

float to_f32(const LL& L, const uint32_t* words, int i) {
  if (L.dtype == 2) {
    float f;
    memcpy(&f, &words[i], 4);
    return f;
  }
  const uint16_t h = static_cast<uint16_t>(words[i / 2] >> (16 * (i & 1)));
  return L.dtype == 1 ? f16_to_f32(h) : bf16_to_f32(h);
}
// Rounds to the element type; returns the value back in fp32.
float round_to_type(const LL& L, float f) {
  if (L.dtype == 2) return f;
  return L.dtype == 1 ? f16_to_f32(f32_to_f16(f)) : bf16_to_f32(f32_to_bf16(f));
}
void pack(const LL& L, const std::vector<float>& v, std::vector<uint32_t>& words) {
  for (size_t w = 0; w < L.words; ++w) {
    if (L.dtype == 2) {
      memcpy(&words[w], &v[w], 4);
    } else {
      const uint16_t lo = L.dtype == 1 ? f32_to_f16(v[2 * w]) : f32_to_bf16(v[2 * w]);
      const uint16_t hi = L.dtype == 1 ? f32_to_f16(v[2 * w + 1]) : f32_to_bf16(v[2 * w + 1]);
      words[w] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
  }
}

}  // namespace

extern "C" uint64_t kb_a2a_ll_bytes(int world, int max_tokens, int topk, int hidden, int elem_bytes);

// Same arguments as kb_a2a_round_trip_host; `a->ll_off` / `a->ll_max_tokens` name the
// landing areas (kb_a2a_ll_bytes() bytes, zero-filled when the heap was made).
extern "C" int kb_a2a_round_trip_host_ll(const KbA2aArgs* a, int timeout_ms) {
  if (a == nullptr || a->world < 1 || a->world > KB_MAX_WORLD || a->rank < 0 || a->rank >= a->world || a->dtype < 0 ||
      a->dtype > 2 || a->num_experts <= 0 || a->num_experts % a->world != 0 || a->topk <= 0 || a->topk > 64) {
    kb::set_error("a2a host (low latency): bad rank, world, dtype, expert count or top-k");
    return KB_ERR_ARG;
  }
  if (a->ll_off == 0 || a->ll_max_tokens <= 0 || a->num_tokens < 0 || a->num_tokens > a->ll_max_tokens ||
      (static_cast<size_t>(a->hidden) * a->elem_bytes) % 16 != 0) {
    kb::set_error("a2a host (low latency): no landing areas, too many tokens (%d of %d) or a row that is not a multiple of 16 bytes",
                  a->num_tokens, a->ll_max_tokens);
    return KB_ERR_ARG;
  }
  LL L;
  L.rank = a->rank;
  L.world = a->world;
  L.E = a->num_experts;
  L.El = a->num_experts / a->world;
  L.k = a->topk;
  L.H = a->hidden;
  L.T = a->num_tokens;
  L.tmax = a->ll_max_tokens;
  L.dtype = a->dtype;
  L.row_bytes = static_cast<size_t>(a->hidden) * a->elem_bytes;
  L.words = L.row_bytes / 4;
  L.epoch = a->epoch;
  L.off = a->ll_off;
  L.row2 = 2 * L.row_bytes;
  L.back_off = static_cast<size_t>(L.world) * L.tmax * L.row2;
  L.meta_off = 2 * L.back_off;
  L.cnt_off = L.meta_off + static_cast<size_t>(L.world) * L.tmax * (2 * L.k + 2) * 8;
  {  // the kernel's own size function must agree with this layout
    const uint64_t mine = (L.cnt_off + 2 * static_cast<size_t>(L.world) * 128 + 255) / 256 * 256;
    const uint64_t theirs = kb_a2a_ll_bytes(L.world, L.tmax, L.k, L.H, a->elem_bytes);
    if (theirs != 0 && mine != theirs) {
      kb::set_error("a2a host (low latency): layout of %llu bytes, the kernels use %llu", (unsigned long long)mine,
                    (unsigned long long)theirs);
      return KB_ERR_ARG;
    }
  }
  for (int r = 0; r < L.world; ++r) {
    if (a->peer_base[r] == nullptr) {
      kb::set_error("a2a host (low latency): peer_base[%d] is null", r);
      return KB_ERR_ARG;
    }
    L.base[r] = static_cast<char*>(a->peer_base[r]);
  }
  const int64_t deadline = now_ms() + (timeout_ms > 0 ? timeout_ms : 30000);
  const int W = L.world, k = L.k;

  // ---- slots: a token's row on rank r lands behind the rows of the earlier tokens that reach r ----
  std::vector<int> slot(static_cast<size_t>(L.T) * W, -1), tot(W, 0);
  for (int t = 0; t < L.T; ++t) {
    uint32_t mask = 0;
    for (int j = 0; j < k; ++j) {
      const int e = a->indices[t * k + j];
      if (e < 0 || e >= L.E) {
        kb::set_error("a2a host (low latency): expert id %d out of range at entry %d", e, t * k + j);
        return KB_ERR_ARG;
      }
      mask |= 1u << (e / L.El);
    }
    for (int r = 0; r < W; ++r) {
      if ((mask >> r) & 1u) slot[static_cast<size_t>(t) * W + r] = tot[r]++;
    }
  }

  // ---- dispatch: metadata, rows and counts, every unit carrying the epoch ----
  const uint8_t* x = static_cast<const uint8_t*>(a->x);
  for (int t = 0; t < L.T; ++t) {
    const uint32_t* xw = reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(t) * L.row_bytes);
    for (int r = 0; r < W; ++r) {
      const int s = slot[static_cast<size_t>(t) * W + r];
      if (s < 0) continue;
      Unit* m = L.meta(r, L.rank, s);
      int cnt = 0;
      for (int j = 0; j < k; ++j) {
        const int e = a->indices[t * k + j];
        if (e / L.El != r) continue;
        uint32_t wbits;
        memcpy(&wbits, &a->weights[t * k + j], 4);
        put(m + 2 + cnt, static_cast<uint32_t>(e - r * L.El), L.epoch);
        put(m + 2 + k + cnt, wbits, L.epoch);
        ++cnt;
      }
      put(m, static_cast<uint32_t>(cnt), L.epoch);
      Unit* row = L.row(r, false, L.rank, s);
      for (size_t w = 0; w < L.words; ++w) put(row + w, xw[w], L.epoch);
    }
  }
  for (int r = 0; r < W; ++r) put(L.cnt(r, L.rank), static_cast<uint32_t>(tot[r]), L.epoch);

  // ---- expert: poll counts, metadata and rows; push one weighted partial row back per unique row ----
  std::vector<uint32_t> words(L.words), ids(k), wts(k);
  std::vector<float> acc(L.H);
  for (int si = 0; si < W; ++si) {
    const int s = (L.rank + si) % W;  // own rows first, as the kernels' rounds do
    uint32_t n = 0;
    if (!get(L.cnt(L.rank, s), L.epoch, deadline, &n)) {
      kb::set_error("a2a host (low latency): rank %d never sent its counts of epoch %u (waited for by rank %d)", s, L.epoch, L.rank);
      return KB_ERR_TIMEOUT;
    }
    if (n > static_cast<uint32_t>(L.tmax)) n = static_cast<uint32_t>(L.tmax);
    for (uint32_t g = 0; g < n; ++g) {
      const Unit* m = L.meta(L.rank, s, static_cast<int>(g));
      uint32_t cnt = 0;
      bool ok = get(m, L.epoch, deadline, &cnt);
      if (cnt > static_cast<uint32_t>(k)) cnt = 0;
      for (uint32_t j = 0; ok && j < cnt; ++j) ok = get(m + 2 + j, L.epoch, deadline, &ids[j]) && get(m + 2 + k + j, L.epoch, deadline, &wts[j]);
      const Unit* row = L.row(L.rank, false, s, static_cast<int>(g));
      for (size_t w = 0; ok && w < L.words; ++w) ok = get(row + w, L.epoch, deadline, &words[w]);
      if (!ok) {
        kb::set_error("a2a host (low latency): row %u of rank %d did not arrive in epoch %u (waited for by rank %d)", g, s, L.epoch, L.rank);
        return KB_ERR_TIMEOUT;
      }
      for (int i = 0; i < L.H; ++i) acc[i] = 0.f;
      for (uint32_t j = 0; j < cnt; ++j) {
        float scale = 1.0f;
        if (a->scale_mode == 1) scale = static_cast<float>(1 + L.rank);
        if (a->scale_mode == 2) scale = static_cast<float>(L.rank * L.El + static_cast<int>(ids[j]) + 1) / static_cast<float>(L.E);
        float wj;
        memcpy(&wj, &wts[j], 4);
        for (int i = 0; i < L.H; ++i) acc[i] += wj * round_to_type(L, to_f32(L, words.data(), i) * scale);
      }
      pack(L, acc, words);
      Unit* back = L.row(s, true, L.rank, static_cast<int>(g));
      for (size_t w = 0; w < L.words; ++w) put(back + w, words[w], L.epoch);
    }
  }

  // ---- combine: poll the partial rows of this rank's tokens, add them in ascending rank order ----
  uint8_t* out = static_cast<uint8_t*>(a->out);
  for (int t = 0; t < L.T; ++t) {
    for (int i = 0; i < L.H; ++i) acc[i] = 0.f;
    for (int r = 0; r < W; ++r) {
      const int s = slot[static_cast<size_t>(t) * W + r];
      if (s < 0) continue;
      const Unit* row = L.row(L.rank, true, r, s);
      for (size_t w = 0; w < L.words; ++w) {
        if (!get(row + w, L.epoch, deadline, &words[w])) {
          kb::set_error("a2a host (low latency): rank %d never returned row %d of epoch %u (waited for by rank %d)", r, s, L.epoch, L.rank);
          return KB_ERR_TIMEOUT;
        }
      }
      for (int i = 0; i < L.H; ++i) acc[i] += to_f32(L, words.data(), i);
    }
    pack(L, acc, words);
    memcpy(out + static_cast<size_t>(t) * L.row_bytes, words.data(), L.row_bytes);
  }
  return KB_OK;
}
