// Symmetric heap: one allocation per rank of a group, mapped by every rank of the group into one contiguous
// address range (slot p of the range = rank p's memory), so that a kernel reaches a peer's copy of a buffer at
// `base + p * slot_bytes + offset` - plain arithmetic, no pointer table.
//
// Two backends share the bookkeeping and the exchange protocol:
//   * device memory through the CUDA virtual-memory-management driver API: cuMemCreate (a physical allocation
//     on this rank's GPU, exportable as a POSIX file descriptor), cuMemAddressReserve (the n-slot range),
//     cuMemImportFromShareableHandle + cuMemMap (the peers' allocations into their slots), cuMemSetAccess (read /
//     write for this rank's GPU).  The entry points are resolved at run time through the CUDA runtime, so the
//     library has no link-time dependency on the driver and loads on machines without one;
//   * host memory (memfd + mmap), with the same calls in the same order.  It is what the CPU tests run: ranks
//     are processes of one machine, "peer memory" is shared pages.  Nothing of the device backend is stubbed
//     for it - only the five memory calls differ.
//
// The file descriptors travel between processes in the Python layer (SCM_RIGHTS over abstract unix sockets whose
// names are agreed through the process group); this file never talks to another process.
//
// The reference project has no counterpart: its process groups (axonn/communication.py:124-236) move all data
// through NCCL.
#include <cerrno>
#include <cstdint>
#include <cstring>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <unistd.h>

#include "common.cuh"

namespace axb {

enum HeapBackend { HEAP_HOST = 0, HEAP_CUDA_VMM = 1 };

struct DriverApi {
  bool resolved = false, ok = false;
  CUresult (*memGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                         unsigned long long) = nullptr;
  CUresult (*memImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*memAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
};

static DriverApi g_drv;

template <typename F>
static bool resolve(const char* name, F* out) {
  void* f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess ||
      f == nullptr) {
    (void)cudaGetLastError();
    set_error("symmetric heap: the CUDA driver does not provide %s", name);
    return false;
  }
  *out = reinterpret_cast<F>(f);
  return true;
}

static bool driver_api() {
  if (g_drv.resolved) return g_drv.ok;
  g_drv.resolved = true;
  g_drv.ok = resolve("cuMemGetAllocationGranularity", &g_drv.memGetAllocationGranularity) &&
             resolve("cuMemCreate", &g_drv.memCreate) &&
             resolve("cuMemExportToShareableHandle", &g_drv.memExportToShareableHandle) &&
             resolve("cuMemImportFromShareableHandle", &g_drv.memImportFromShareableHandle) &&
             resolve("cuMemAddressReserve", &g_drv.memAddressReserve) &&
             resolve("cuMemAddressFree", &g_drv.memAddressFree) && resolve("cuMemMap", &g_drv.memMap) &&
             resolve("cuMemUnmap", &g_drv.memUnmap) && resolve("cuMemSetAccess", &g_drv.memSetAccess) &&
             resolve("cuMemRelease", &g_drv.memRelease);
  return g_drv.ok;
}

struct Heap {
  int backend = HEAP_HOST, device = 0, rank = 0, nranks = 1;
  size_t slot_bytes = 0;          // size of one rank's allocation, a multiple of the granularity
  uintptr_t base = 0;             // start of the n-slot address range
  int own_fd = -1;                // shareable handle of this rank's allocation
  std::vector<char> mapped;       // per slot: mapped into the range
  std::vector<CUmemGenericAllocationHandle> handles;   // device backend: per slot (0 = none)
};

static bool drv_ok(CUresult r, const char* what) {
  if (r == CUDA_SUCCESS) return true;
  set_error("symmetric heap: %s failed with driver error %d", what, static_cast<int>(r));
  return false;
}

static CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

static bool map_slot(Heap* h, int slot, int fd) {
  const uintptr_t at = h->base + static_cast<uintptr_t>(slot) * h->slot_bytes;
  if (h->backend == HEAP_HOST) {
    void* p = mmap(reinterpret_cast<void*>(at), h->slot_bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, fd, 0);
    if (p == MAP_FAILED) { set_error("symmetric heap: mmap of slot %d failed: %s", slot, strerror(errno)); return false; }
  } else {
    CUmemGenericAllocationHandle handle = h->handles[slot];
    if (handle == 0) {
      if (!drv_ok(g_drv.memImportFromShareableHandle(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                  "cuMemImportFromShareableHandle"))
        return false;
      h->handles[slot] = handle;
    }
    if (!drv_ok(g_drv.memMap(static_cast<CUdeviceptr>(at), h->slot_bytes, 0, handle, 0), "cuMemMap")) return false;
    CUmemAccessDesc access;
    memset(&access, 0, sizeof(access));
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = h->device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (!drv_ok(g_drv.memSetAccess(static_cast<CUdeviceptr>(at), h->slot_bytes, &access, 1), "cuMemSetAccess")) {
      g_drv.memUnmap(static_cast<CUdeviceptr>(at), h->slot_bytes);
      return false;
    }
  }
  h->mapped[slot] = 1;
  return true;
}

static void destroy(Heap* h) {
  if (h == nullptr) return;
  for (int s = 0; s < h->nranks; ++s) {
    const uintptr_t at = h->base + static_cast<uintptr_t>(s) * h->slot_bytes;
    if (h->backend == HEAP_CUDA_VMM) {
      if (h->mapped[s]) g_drv.memUnmap(static_cast<CUdeviceptr>(at), h->slot_bytes);
      if (h->handles[s] != 0) g_drv.memRelease(h->handles[s]);
    }
  }
  if (h->base != 0) {
    if (h->backend == HEAP_HOST) munmap(reinterpret_cast<void*>(h->base), h->slot_bytes * h->nranks);
    else g_drv.memAddressFree(static_cast<CUdeviceptr>(h->base), h->slot_bytes * h->nranks);
  }
  if (h->own_fd >= 0) close(h->own_fd);
  delete h;
}

}  // namespace axb

using namespace axb;

// Create this rank's allocation of at least `bytes` (rounded up to the allocation granularity, which every rank
// of one machine computes identically), reserve the n-slot range and map the allocation into slot `rank`.
// backend: 0 = host memory, 1 = device memory of GPU `device`.  Returns 0 and the heap in *out, or -1.
extern "C" int axb_heap_create(int backend, int device, int rank, int nranks, unsigned long long bytes, void** out) {
  if (out == nullptr || nranks < 1 || nranks > 64 || rank < 0 || rank >= nranks || bytes == 0 ||
      (backend != HEAP_HOST && backend != HEAP_CUDA_VMM)) {
    set_error("symmetric heap: bad arguments (backend %d, rank %d of %d, %llu bytes)", backend, rank, nranks, bytes);
    return -1;
  }
  Heap* h = new Heap;
  h->backend = backend; h->device = device; h->rank = rank; h->nranks = nranks;
  h->mapped.assign(nranks, 0);
  h->handles.assign(nranks, 0);
  size_t gran = 0;
  if (backend == HEAP_HOST) {
    gran = size_t(2) << 20;
    h->slot_bytes = (bytes + gran - 1) / gran * gran;
    h->own_fd = memfd_create("axonn_b200_symm_heap", MFD_CLOEXEC);
    if (h->own_fd < 0 || ftruncate(h->own_fd, static_cast<off_t>(h->slot_bytes)) != 0) {
      set_error("symmetric heap: memfd of %zu bytes: %s", h->slot_bytes, strerror(errno));
      destroy(h); return -1;
    }
    void* range = mmap(nullptr, h->slot_bytes * nranks, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (range == MAP_FAILED) {
      set_error("symmetric heap: reserving %zu bytes of address space: %s", h->slot_bytes * nranks, strerror(errno));
      destroy(h); return -1;
    }
    h->base = reinterpret_cast<uintptr_t>(range);
  } else {
    if (!driver_api()) { destroy(h); return -1; }
    if (check_cuda(cudaSetDevice(device), "cudaSetDevice") != 0 || check_cuda(cudaFree(nullptr), "context creation") != 0) {
      destroy(h); return -1;
    }
    const CUmemAllocationProp prop = device_prop(device);
    if (!drv_ok(g_drv.memGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                "cuMemGetAllocationGranularity") || gran == 0) {
      destroy(h); return -1;
    }
    h->slot_bytes = (bytes + gran - 1) / gran * gran;
    CUmemGenericAllocationHandle handle = 0;
    if (!drv_ok(g_drv.memCreate(&handle, h->slot_bytes, &prop, 0), "cuMemCreate")) { destroy(h); return -1; }
    h->handles[rank] = handle;
    int fd = -1;
    if (!drv_ok(g_drv.memExportToShareableHandle(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                "cuMemExportToShareableHandle")) {
      destroy(h); return -1;
    }
    h->own_fd = fd;
    CUdeviceptr range = 0;
    if (!drv_ok(g_drv.memAddressReserve(&range, h->slot_bytes * nranks, gran, 0, 0), "cuMemAddressReserve")) {
      destroy(h); return -1;
    }
    h->base = static_cast<uintptr_t>(range);
  }
  if (!map_slot(h, rank, h->own_fd)) { destroy(h); return -1; }
  *out = h;
  return 0;
}

// The shareable handle of this rank's allocation: a file descriptor that stays owned by the heap.
extern "C" int axb_heap_fd(void* heap) { return heap ? static_cast<Heap*>(heap)->own_fd : -1; }

// Map peer `peer`'s allocation, received as file descriptor `fd`, into its slot.  The descriptor stays the caller's
// to close (the mapping keeps the memory alive).
extern "C" int axb_heap_attach(void* heap, int peer, int fd) {
  Heap* h = static_cast<Heap*>(heap);
  if (h == nullptr || peer < 0 || peer >= h->nranks || peer == h->rank || fd < 0) {
    set_error("symmetric heap: cannot attach peer %d", peer);
    return -1;
  }
  if (h->mapped[peer]) { set_error("symmetric heap: peer %d is attached already", peer); return -1; }
  return map_slot(h, peer, fd) ? 0 : -1;
}

// what: 0 = base address of the range, 1 = bytes per slot, 2 = number of slots mapped so far, 3 = backend
extern "C" unsigned long long axb_heap_info(void* heap, int what) {
  const Heap* h = static_cast<const Heap*>(heap);
  if (h == nullptr) return 0;
  switch (what) {
    case 0: return h->base;
    case 1: return h->slot_bytes;
    case 2: { unsigned long long n = 0; for (char m : h->mapped) n += m; return n; }
    case 3: return static_cast<unsigned long long>(h->backend);
    default: return 0;
  }
}

// Unmap every slot, release the allocations and the address range.  The caller makes sure that no kernel of any
// rank still uses the memory (a barrier of the group after the last kernel has finished).
extern "C" int axb_heap_destroy(void* heap) {
  destroy(static_cast<Heap*>(heap));
  return 0;
}
