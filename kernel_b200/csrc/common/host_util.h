// Host-side helpers shared by the launchers: error recording, lazy driver-API
// lookup (the library never links libcuda, so it also loads on machines with
// no driver), and device status reporting for kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../include/kb200.h"

namespace kb {

void set_error(const char* fmt, ...);

#define KB_CUDA_OK(expr)                                                                   \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      ::kb::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return KB_ERR_CUDA;                                                                  \
    }                                                                                      \
  } while (0)

// Looks a driver entry point up through the runtime.  Returns nullptr (and
// records an error) when the symbol or the driver is missing.
void* driver_fn(const char* name);

#define KB_DRV(name) reinterpret_cast<decltype(&name)>(::kb::driver_fn(#name))

#define KB_CU_OK(call_expr, what)                                                 \
  do {                                                                            \
    CUresult _r = (call_expr);                                                    \
    if (_r != CUDA_SUCCESS) {                                                     \
      ::kb::set_error("%s failed: CUresult %d (%s:%d)", what, (int)_r, __FILE__, __LINE__); \
      return KB_ERR_CUDA;                                                         \
    }                                                                             \
  } while (0)

#ifdef __CUDACC__
// First failure wins; later ones are dropped so the host sees the root cause.
__device__ __forceinline__ void report_status(uint32_t* status, uint32_t code, uint32_t site, uint32_t what,
                                              uint32_t epoch) {
  if (status == nullptr) return;
  if (atomicCAS(&status[0], 0u, code) == 0u) {
    status[1] = site;
    status[2] = what;
    status[3] = epoch;
    status[4] = blockIdx.x;
    __threadfence_system();
  }
}
#endif

}  // namespace kb
