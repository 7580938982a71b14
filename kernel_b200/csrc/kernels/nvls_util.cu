// Two small NVLS (NVSwitch multicast) primitives over the multicast mapping of a
// symmetric heap: a broadcast store and an all-rank reducing load.  They are the
// building blocks the fused GEMM kernels use (multimem.st for the all-gather
// pushes, multimem.ld_reduce for the reduce-scatter pull) as stand-alone
// launches, for bring-up tests and for callers that want the primitive itself.
//
// The reference reaches the same hardware only through NCCL
// (gemm_rs/reference.py:59 reduce_scatter_tensor).
#include <cuda_runtime.h>

#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../include/kb200.h"

namespace {

// dst (multicast address) <- src (local memory): every rank's segment receives the bytes.
__global__ void multimem_store_kernel(uint4* mc_dst, const uint4* src, size_t nvec) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    kb::multimem_st_v4(mc_dst + i, src[i]);
  }
}

// dst (local memory) <- sum over ranks of the bf16 values at mc_src (fp32 accumulation in the switch).
__global__ void multimem_reduce_kernel(uint4* dst, const uint4* mc_src, size_t nvec) {
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    dst[i] = kb::multimem_ld_reduce_bf16x8(mc_src + i);
  }
}

int check(const void* a, const void* b, uint64_t bytes) {
  if (a == nullptr || b == nullptr || bytes == 0 || (bytes % 16) != 0 || (reinterpret_cast<uintptr_t>(a) & 15u) != 0 ||
      (reinterpret_cast<uintptr_t>(b) & 15u) != 0) {
    kb::set_error("multimem: pointers must be non-null and 16-byte aligned, bytes a positive multiple of 16");
    return KB_ERR_ARG;
  }
  return KB_OK;
}

}  // namespace

extern "C" int kb_multimem_store(void* mc_dst, const void* src, uint64_t bytes, void* stream) {
  const int rc = check(mc_dst, src, bytes);
  if (rc != KB_OK) return rc;
  const size_t nvec = bytes / 16;
  const int grid = static_cast<int>(nvec / 256 + 1 < 592 ? nvec / 256 + 1 : 592);
  multimem_store_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(mc_dst),
                                                                             static_cast<const uint4*>(src), nvec);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}

extern "C" int kb_multimem_reduce_bf16(void* dst, const void* mc_src, uint64_t bytes, void* stream) {
  const int rc = check(dst, mc_src, bytes);
  if (rc != KB_OK) return rc;
  const size_t nvec = bytes / 16;
  const int grid = static_cast<int>(nvec / 256 + 1 < 592 ? nvec / 256 + 1 : 592);
  multimem_reduce_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint4*>(dst),
                                                                              static_cast<const uint4*>(mc_src), nvec);
  KB_CUDA_OK(cudaGetLastError());
  return KB_OK;
}
