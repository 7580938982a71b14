// Symmetric heap: every rank allocates one segment of the same size and maps
// all peers' segments into its own address space, so a kernel can address
// "offset X on rank r" with plain loads and stores over NVLink.
//
// Backends
//   VMM   cuMemCreate (POSIX-fd shareable) -> fd exchange -> cuMemImport...
//         -> one reserved VA window of world * segment bytes, peer r mapped at
//         base + r * segment.  Optional NVLS multicast object bound to the
//         same physical memory and mapped at a second address.
//   IPC   cudaMalloc + cudaIpcGet/OpenMemHandle.  Fallback when fd passing or
//         cuMem export is refused.  No multicast.
//   HOST  memfd + mmap.  The same rendezvous and the same window layout for
//         CPU-only ranks; used by the host-side tests and by gloo runs.
//
// The reference has no such layer: its data plane is torch.distributed/NCCL
// (eval.py:176, reference.py:91-119, gemm_rs/reference.py:59).
#include <errno.h>
#include <string.h>
#include <sys/mman.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <vector>

#include "../common/host_util.h"
#include "../include/kb200.h"

struct KbSymmHeap {
  int backend = 0;
  int rank = 0;
  int world = 1;
  int device = 0;
  uint64_t seg_bytes = 0;
  int local_fd = -1;
  void* local_ptr = nullptr;                 // IPC: cudaMalloc pointer
  std::vector<void*> peer_ptr;
  // VMM
  CUmemGenericAllocationHandle local_handle = 0;
  std::vector<CUmemGenericAllocationHandle> peer_handles;
  CUdeviceptr window = 0;
  bool window_reserved = false;
  std::vector<char> mapped;
  // multicast
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_have = false, mc_bound = false, mc_mapped = false;
  CUdeviceptr mc_va = 0;
  uint64_t mc_bytes = 0;
  // HOST
  void* host_window = nullptr;
  // IPC
  cudaIpcMemHandle_t ipc_handle;
  std::vector<char> ipc_opened;
};

namespace {

uint64_t round_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

CUmemAllocationProp vmm_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

int vmm_create(KbSymmHeap* h, uint64_t bytes) {
  auto getGran = KB_DRV(cuMemGetAllocationGranularity);
  auto memCreate = KB_DRV(cuMemCreate);
  auto exportH = KB_DRV(cuMemExportToShareableHandle);
  if (!getGran || !memCreate || !exportH) return KB_ERR_UNSUPPORTED;
  KB_CUDA_OK(cudaSetDevice(h->device));
  KB_CUDA_OK(cudaFree(nullptr));  // make sure the primary context exists
  CUmemAllocationProp prop = vmm_prop(h->device);
  size_t gran = 0;
  KB_CU_OK(getGran(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  if (gran < (2u << 20)) gran = 2u << 20;
  h->seg_bytes = round_up(bytes, gran);
  KB_CU_OK(memCreate(&h->local_handle, h->seg_bytes, &prop, 0), "cuMemCreate");
  int fd = -1;
  KB_CU_OK(exportH(&fd, h->local_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
  h->local_fd = fd;
  return KB_OK;
}

int vmm_map(KbSymmHeap* h, const int* fds) {
  auto importH = KB_DRV(cuMemImportFromShareableHandle);
  auto reserve = KB_DRV(cuMemAddressReserve);
  auto memMap = KB_DRV(cuMemMap);
  auto setAccess = KB_DRV(cuMemSetAccess);
  if (!importH || !reserve || !memMap || !setAccess) return KB_ERR_UNSUPPORTED;
  KB_CUDA_OK(cudaSetDevice(h->device));
  KB_CU_OK(reserve(&h->window, h->seg_bytes * h->world, 0, 0, 0), "cuMemAddressReserve");
  h->window_reserved = true;
  h->peer_handles.assign(h->world, 0);
  h->mapped.assign(h->world, 0);
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  for (int r = 0; r < h->world; ++r) {
    CUmemGenericAllocationHandle hd = h->local_handle;
    if (r != h->rank) {
      if (fds == nullptr || fds[r] < 0) {
        kb::set_error("symm: no descriptor for peer %d", r);
        return KB_ERR_ARG;
      }
      KB_CU_OK(importH(&hd, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[r])),
                       CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
               "cuMemImportFromShareableHandle");
      h->peer_handles[r] = hd;
    }
    const CUdeviceptr va = h->window + static_cast<uint64_t>(r) * h->seg_bytes;
    KB_CU_OK(memMap(va, h->seg_bytes, 0, hd, 0), "cuMemMap");
    h->mapped[r] = 1;
    KB_CU_OK(setAccess(va, h->seg_bytes, &acc, 1), "cuMemSetAccess");
    h->peer_ptr[r] = reinterpret_cast<void*>(va);
  }
  KB_CUDA_OK(cudaMemset(h->peer_ptr[h->rank], 0, h->seg_bytes));
  KB_CUDA_OK(cudaDeviceSynchronize());
  return KB_OK;
}

int host_create(KbSymmHeap* h, uint64_t bytes) {
  h->seg_bytes = round_up(bytes, 1u << 16);
  const int fd = memfd_create("kb200-symm", MFD_CLOEXEC);
  if (fd < 0 || ftruncate(fd, static_cast<off_t>(h->seg_bytes)) != 0) {
    kb::set_error("memfd_create/ftruncate: %s", strerror(errno));
    if (fd >= 0) close(fd);
    return KB_ERR_IO;
  }
  h->local_fd = fd;
  return KB_OK;
}

int host_map(KbSymmHeap* h, const int* fds) {
  void* win = mmap(nullptr, h->seg_bytes * h->world, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (win == MAP_FAILED) {
    kb::set_error("mmap reserve: %s", strerror(errno));
    return KB_ERR_IO;
  }
  h->host_window = win;
  for (int r = 0; r < h->world; ++r) {
    const int fd = (r == h->rank) ? h->local_fd : (fds ? fds[r] : -1);
    if (fd < 0) {
      kb::set_error("symm: no descriptor for peer %d", r);
      return KB_ERR_ARG;
    }
    void* at = static_cast<char*>(win) + static_cast<uint64_t>(r) * h->seg_bytes;
    void* m = mmap(at, h->seg_bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
    if (m == MAP_FAILED) {
      kb::set_error("mmap peer %d: %s", r, strerror(errno));
      return KB_ERR_IO;
    }
    h->peer_ptr[r] = m;
  }
  return KB_OK;
}

int ipc_create(KbSymmHeap* h, uint64_t bytes) {
  KB_CUDA_OK(cudaSetDevice(h->device));
  h->seg_bytes = round_up(bytes, 2u << 20);
  KB_CUDA_OK(cudaMalloc(&h->local_ptr, h->seg_bytes));
  KB_CUDA_OK(cudaMemset(h->local_ptr, 0, h->seg_bytes));
  KB_CUDA_OK(cudaDeviceSynchronize());
  KB_CUDA_OK(cudaIpcGetMemHandle(&h->ipc_handle, h->local_ptr));
  return KB_OK;
}

int ipc_map(KbSymmHeap* h, const void* handles) {
  KB_CUDA_OK(cudaSetDevice(h->device));
  h->ipc_opened.assign(h->world, 0);
  for (int r = 0; r < h->world; ++r) {
    if (r == h->rank) {
      h->peer_ptr[r] = h->local_ptr;
      continue;
    }
    if (handles == nullptr) return KB_ERR_ARG;
    cudaIpcMemHandle_t hd;
    memcpy(&hd, static_cast<const char*>(handles) + static_cast<size_t>(r) * sizeof(hd), sizeof(hd));
    void* ptr = nullptr;
    KB_CUDA_OK(cudaIpcOpenMemHandle(&ptr, hd, cudaIpcMemLazyEnablePeerAccess));
    h->peer_ptr[r] = ptr;
    h->ipc_opened[r] = 1;
  }
  return KB_OK;
}

}  // namespace

extern "C" int kb_symm_create(int backend, int rank, int world, uint64_t bytes, int device, KbSymmHeap** out) {
  if (out == nullptr || world < 1 || world > KB_MAX_WORLD || rank < 0 || rank >= world || bytes == 0) {
    kb::set_error("kb_symm_create: bad arguments (rank %d world %d bytes %llu)", rank, world,
                  (unsigned long long)bytes);
    return KB_ERR_ARG;
  }
  KbSymmHeap* h = new KbSymmHeap();
  h->backend = backend;
  h->rank = rank;
  h->world = world;
  h->device = device;
  h->peer_ptr.assign(world, nullptr);
  int rc = KB_ERR_ARG;
  switch (backend) {
    case KB_BACKEND_HOST: rc = host_create(h, bytes); break;
    case KB_BACKEND_VMM: rc = vmm_create(h, bytes); break;
    case KB_BACKEND_IPC: rc = ipc_create(h, bytes); break;
    default: kb::set_error("kb_symm_create: unknown backend %d", backend);
  }
  if (rc != KB_OK) {
    kb_symm_destroy(h);
    return rc;
  }
  *out = h;
  return KB_OK;
}

extern "C" uint64_t kb_symm_segment_bytes(const KbSymmHeap* h) { return h ? h->seg_bytes : 0; }
extern "C" int kb_symm_local_fd(const KbSymmHeap* h) { return h ? h->local_fd : -1; }
extern "C" int kb_symm_ipc_handle(const KbSymmHeap* h, void* out64) {
  if (h == nullptr || out64 == nullptr || h->backend != KB_BACKEND_IPC) return KB_ERR_ARG;
  memcpy(out64, &h->ipc_handle, sizeof(h->ipc_handle));
  return KB_OK;
}

extern "C" int kb_symm_map_peers(KbSymmHeap* h, const int* fds, const void* ipc_handles) {
  if (h == nullptr) return KB_ERR_ARG;
  switch (h->backend) {
    case KB_BACKEND_HOST: return host_map(h, fds);
    case KB_BACKEND_VMM: return vmm_map(h, fds);
    case KB_BACKEND_IPC: return ipc_map(h, ipc_handles);
  }
  return KB_ERR_ARG;
}

extern "C" void* kb_symm_peer_ptr(const KbSymmHeap* h, int peer) {
  if (h == nullptr || peer < 0 || peer >= h->world) return nullptr;
  return h->peer_ptr[peer];
}
extern "C" void* kb_symm_local_ptr(const KbSymmHeap* h) { return h ? h->peer_ptr[h->rank] : nullptr; }

// ----------------------------------------------------------------- multicast ----
extern "C" int kb_symm_mc_supported(int device) {
  auto getAttr = KB_DRV(cuDeviceGetAttribute);
  if (!getAttr) return 0;
  int v = 0;
  if (getAttr(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v;
}

static CUmulticastObjectProp mc_prop(const KbSymmHeap* h, uint64_t bytes) {
  CUmulticastObjectProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.numDevices = static_cast<unsigned>(h->world);
  prop.size = bytes;
  prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

extern "C" int kb_symm_mc_create(KbSymmHeap* h, int* fd_out) {
  if (h == nullptr || fd_out == nullptr || h->backend != KB_BACKEND_VMM) return KB_ERR_ARG;
  auto getGran = KB_DRV(cuMulticastGetGranularity);
  auto create = KB_DRV(cuMulticastCreate);
  auto exportH = KB_DRV(cuMemExportToShareableHandle);
  if (!getGran || !create || !exportH) return KB_ERR_UNSUPPORTED;
  CUmulticastObjectProp prop = mc_prop(h, h->seg_bytes);
  size_t gran = 0;
  // The minimum granularity (the recommended one can be hundreds of megabytes); segments are whole
  // multiples of the 2 MB allocation granularity, which the minimum divides on NVSwitch systems.
  KB_CU_OK(getGran(&gran, &prop, CU_MULTICAST_GRANULARITY_MINIMUM), "cuMulticastGetGranularity");
  h->mc_bytes = round_up(h->seg_bytes, gran);
  if (h->mc_bytes != h->seg_bytes) {
    kb::set_error("multicast granularity %zu does not divide the segment size %llu", gran,
                  (unsigned long long)h->seg_bytes);
    return KB_ERR_UNSUPPORTED;
  }
  prop.size = h->mc_bytes;
  KB_CU_OK(create(&h->mc_handle, &prop), "cuMulticastCreate");
  h->mc_have = true;
  int fd = -1;
  KB_CU_OK(exportH(&fd, h->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "export multicast handle");
  *fd_out = fd;
  return KB_OK;
}

extern "C" int kb_symm_mc_join(KbSymmHeap* h, int fd_from_rank0) {
  if (h == nullptr || h->backend != KB_BACKEND_VMM) return KB_ERR_ARG;
  auto importH = KB_DRV(cuMemImportFromShareableHandle);
  auto addDev = KB_DRV(cuMulticastAddDevice);
  if (!importH || !addDev) return KB_ERR_UNSUPPORTED;
  if (!h->mc_have) {
    KB_CU_OK(importH(&h->mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd_from_rank0)),
                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
             "import multicast handle");
    h->mc_have = true;
    h->mc_bytes = h->seg_bytes;
  }
  KB_CU_OK(addDev(h->mc_handle, h->device), "cuMulticastAddDevice");
  return KB_OK;
}

extern "C" int kb_symm_mc_bind(KbSymmHeap* h) {
  if (h == nullptr || !h->mc_have) return KB_ERR_ARG;
  auto bindMem = KB_DRV(cuMulticastBindMem);
  auto reserve = KB_DRV(cuMemAddressReserve);
  auto memMap = KB_DRV(cuMemMap);
  auto setAccess = KB_DRV(cuMemSetAccess);
  if (!bindMem || !reserve || !memMap || !setAccess) return KB_ERR_UNSUPPORTED;
  KB_CU_OK(bindMem(h->mc_handle, 0, h->local_handle, 0, h->seg_bytes, 0), "cuMulticastBindMem");
  h->mc_bound = true;
  KB_CU_OK(reserve(&h->mc_va, h->mc_bytes, 0, 0, 0), "reserve multicast VA");
  KB_CU_OK(memMap(h->mc_va, h->mc_bytes, 0, h->mc_handle, 0), "map multicast handle");
  h->mc_mapped = true;
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = h->device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  KB_CU_OK(setAccess(h->mc_va, h->mc_bytes, &acc, 1), "set access on multicast VA");
  return KB_OK;
}

extern "C" void* kb_symm_mc_ptr(const KbSymmHeap* h) {
  return (h && h->mc_mapped) ? reinterpret_cast<void*>(h->mc_va) : nullptr;
}

extern "C" int kb_symm_destroy(KbSymmHeap* h) {
  if (h == nullptr) return KB_OK;
  if (h->backend == KB_BACKEND_VMM) {
    auto unmap = KB_DRV(cuMemUnmap);
    auto release = KB_DRV(cuMemRelease);
    auto addrFree = KB_DRV(cuMemAddressFree);
    auto unbind = KB_DRV(cuMulticastUnbind);
    if (unmap && release && addrFree) {
      cudaSetDevice(h->device);
      cudaDeviceSynchronize();
      if (h->mc_mapped) {
        unmap(h->mc_va, h->mc_bytes);
        addrFree(h->mc_va, h->mc_bytes);
      }
      if (h->mc_bound && unbind) unbind(h->mc_handle, h->device, 0, h->seg_bytes);
      if (h->mc_have) release(h->mc_handle);
      for (int r = 0; r < h->world && r < (int)h->mapped.size(); ++r) {
        if (h->mapped[r]) unmap(h->window + static_cast<uint64_t>(r) * h->seg_bytes, h->seg_bytes);
      }
      if (h->window_reserved) addrFree(h->window, h->seg_bytes * h->world);
      for (size_t r = 0; r < h->peer_handles.size(); ++r) {
        if (h->peer_handles[r]) release(h->peer_handles[r]);
      }
      if (h->local_handle) release(h->local_handle);
    }
  } else if (h->backend == KB_BACKEND_IPC) {
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    for (int r = 0; r < h->world && r < (int)h->ipc_opened.size(); ++r) {
      if (h->ipc_opened[r]) cudaIpcCloseMemHandle(h->peer_ptr[r]);
    }
    if (h->local_ptr) cudaFree(h->local_ptr);
  } else if (h->backend == KB_BACKEND_HOST) {
    if (h->host_window) munmap(h->host_window, h->seg_bytes * h->world);
  }
  if (h->local_fd >= 0) close(h->local_fd);
  delete h;
  return KB_OK;
}

extern "C" int kb_symm_host_barrier(KbSymmHeap* h, uint64_t pad_off, uint32_t epoch, int timeout_ms) {
  if (h == nullptr || h->backend != KB_BACKEND_HOST) return KB_ERR_ARG;
  if (pad_off + sizeof(uint32_t) * h->world > h->seg_bytes) return KB_ERR_ARG;
  for (int r = 0; r < h->world; ++r) {
    auto* slot = reinterpret_cast<std::atomic<uint32_t>*>(static_cast<char*>(h->peer_ptr[r]) + pad_off) + h->rank;
    slot->store(epoch, std::memory_order_release);
  }
  const int64_t deadline = now_ms() + (timeout_ms > 0 ? timeout_ms : 30000);
  auto* mine = reinterpret_cast<std::atomic<uint32_t>*>(static_cast<char*>(h->peer_ptr[h->rank]) + pad_off);
  for (int r = 0; r < h->world; ++r) {
    while (static_cast<int32_t>(mine[r].load(std::memory_order_acquire) - epoch) < 0) {
      if (now_ms() > deadline) {
        kb::set_error("host barrier: rank %d never reached epoch %u", r, epoch);
        return KB_ERR_TIMEOUT;
      }
      usleep(50);
    }
  }
  return KB_OK;
}
