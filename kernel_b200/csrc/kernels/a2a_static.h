// Allocation-free entry point for the single-GPU MoE round trip.
//
// This entry point has no counterpart in the reference.
//
// Who needs it: code that is not allowed to obtain device memory at the moment
// it wants to run the op.  Examples are a plug-in inside a host application that
// hands out a fixed memory budget up front and forbids later allocations, a
// latency-critical serving loop that must never enter the allocator (cudaMalloc
// may synchronise the whole device and stall behind unrelated work), and a
// process whose memory pool already holds all free device memory, so that a
// fresh cudaMalloc would simply fail.  The regular entry points need a
// symmetric workspace that somebody has to allocate; this one brings its own.
//
// The workspace is one file-scope device array of KB_A2A_STATIC_BYTES bytes that
// every GPU which loads the library keeps until the process exits.  Limits that
// follow from it (larger requests are rejected with KB_ERR_ARG and a message):
//
//   num_tokens * topk * hidden * element size  <=  KB_A2A_STATIC_ROW_BYTES
//   num_tokens * topk                          <=  KB_A2A_STATIC_MAX_ROWS
//   num_experts                                <=  KB_A2A_STATIC_MAX_EXPERTS
//
// Rules of use
//   * One GPU only (all experts are local); inputs and outputs are the caller's.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and caches it.  Make that first call before any
//     stream capture is begun on that device.
//   * Every call uses the same array, which still holds what the previous call
//     left there.  The entry point resets the few words that must start at zero
//     itself, on the given stream.  Two calls that overlap on the GPU (different
//     streams, no dependency between them) race on the array: order them.
//   * No cudaMalloc, cudaFree or allocating library routine is called.
//   * The kernels check what they are given (expert ids in range, slots inside
//     the workspace) and skip what fails the check instead of writing it.  Such a
//     call still returns KB_OK, because the check runs on the GPU after the call
//     has returned: read the device status words with kb_a2a_static_status once
//     the stream has been synchronised.  The words keep the first failure until
//     they are cleared.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KB_A2A_STATIC_ROW_BYTES (4u << 20)   // per region; there are two regions
#define KB_A2A_STATIC_MAX_ROWS 16384
#define KB_A2A_STATIC_MAX_EXPERTS 1024
// two row regions, the slot table, the per-expert counts, 4 KB of flag lines, 512 bytes of counters, 256 of status
#define KB_A2A_STATIC_BYTES (2u * KB_A2A_STATIC_ROW_BYTES + 4u * KB_A2A_STATIC_MAX_ROWS + 4u * KB_A2A_STATIC_MAX_EXPERTS + 4096u + 512u + 256u)

// out[t] = sum_k weights[t,k] * scale(indices[t,k]) * x[t], the rows travelling
// through the dispatch, expert and combine kernels exactly as in
// kb_a2a_dispatch / kb_a2a_expert_scale / kb_a2a_combine with world = 1.
// dtype: 0 bf16, 1 fp16, 2 fp32.  scale_mode: 0 identity, 1 (1 + rank) = 1,
// 2 (expert + 1) / num_experts.  Returns a KbStatus; see kb_last_error().
int kb_a2a_round_trip_static(const void* x, const int32_t* indices, const float* weights, void* out, int num_tokens,
                             int num_experts, int topk, int hidden, int dtype, int scale_mode, void* stream);


// Copies the eight device status words of the built-in workspace of the current
// device to `out8` (host or device memory; pinned host memory keeps the copy
// asynchronous) on `stream`, and with `clear` non-zero zeroes them afterwards.
// out8[0] is a KbDevCode (0 = healthy, 3 = an index check rejected something),
// out8[1] the site, out8[2] the offending entry, out8[3] the call's sequence
// number, out8[4] the CTA.  Allocates nothing.  Returns a KbStatus.
int kb_a2a_static_status(uint32_t* out8, int clear, void* stream);

#ifdef __cplusplus
}
#endif
