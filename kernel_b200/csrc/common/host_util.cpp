#include "host_util.h"

#include <mutex>
#include <string>
#include <unordered_map>

namespace kb {

static thread_local char g_err[1024] = {0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

void* driver_fn(const char* name) {
  static std::mutex mu;
  static std::unordered_map<std::string, void*> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(name);
  if (it != cache.end()) return it->second;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
    set_error("driver entry point %s unavailable (%s)", name, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return nullptr;
  }
  cache.emplace(name, fn);
  return fn;
}

}  // namespace kb

extern "C" const char* kb_last_error(void) { return kb::g_err; }
