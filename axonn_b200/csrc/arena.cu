// Output arena: a host-side allocator over one peer-mapped ("symmetric") address range per device.
//
// The two-shot all-reduce epilogue of the fused GEMM stores finished values straight into C on every rank of
// the group, so C has to live in memory that the peers have mapped.  The range itself is a symmetric
// allocation made once by the Python layer (axonn_b200/parallel/symm.py) and registered here; this file only
// carves it up.  axb_arena_malloc / axb_arena_free have the signatures that torch's pluggable-allocator hook
// expects, so a torch.cuda.MemPool built on them lets PyTorch's caching allocator manage tensor lifetimes
// inside the range: outputs of the fused kernels are ordinary tensors whose storage happens to be peer-visible.
//
// Allocation is first-fit over a sorted free list with 2 MiB granularity (the caching allocator asks for whole
// segments and sub-allocates them itself).  No CUDA call is made here.  The reference project has no
// counterpart: all of its collectives go through NCCL's own staging buffers.
#include <cstdint>
#include <map>
#include <mutex>

#include "common.cuh"

namespace axb {

struct Arena {
  uintptr_t base = 0;
  size_t size = 0;
  std::map<uintptr_t, size_t> free_list;   // start -> length, coalesced
  std::map<uintptr_t, size_t> live;        // start -> length of blocks handed out
  size_t in_use = 0, high_water = 0;
  unsigned long long failed = 0;           // requests that did not fit
};

static std::mutex g_arena_mu;
static Arena g_arena[64];
constexpr size_t ARENA_ALIGN = size_t(2) << 20;

}  // namespace axb

using namespace axb;

// Register [base, base + nbytes) as device `device`'s arena (replaces an earlier registration; blocks that are
// still handed out from the earlier range are forgotten, which is only correct once they are all freed).
extern "C" int axb_arena_register(int device, void* base, unsigned long long nbytes) {
  if (device < 0 || device >= 64) { set_error("arena: bad device %d", device); return -1; }
  std::lock_guard<std::mutex> lock(g_arena_mu);
  Arena& a = g_arena[device];
  a.free_list.clear(); a.live.clear();
  a.in_use = a.high_water = 0; a.failed = 0;
  const uintptr_t lo = (reinterpret_cast<uintptr_t>(base) + ARENA_ALIGN - 1) / ARENA_ALIGN * ARENA_ALIGN;
  const uintptr_t hi = (reinterpret_cast<uintptr_t>(base) + nbytes) / ARENA_ALIGN * ARENA_ALIGN;
  a.base = reinterpret_cast<uintptr_t>(base);
  a.size = nbytes;
  if (base != nullptr && hi > lo) a.free_list[lo] = hi - lo;
  return 0;
}

// torch pluggable-allocator hook: returns a block of at least `size` bytes from the arena of `device`, or null
// when nothing fits (the caching allocator then reports out-of-memory for the pool).
extern "C" void* axb_arena_malloc(long long size, int device, void* /*stream*/) {
  if (device < 0 || device >= 64 || size <= 0) return nullptr;
  std::lock_guard<std::mutex> lock(g_arena_mu);
  Arena& a = g_arena[device];
  const size_t need = (static_cast<size_t>(size) + ARENA_ALIGN - 1) / ARENA_ALIGN * ARENA_ALIGN;
  for (auto it = a.free_list.begin(); it != a.free_list.end(); ++it) {
    if (it->second < need) continue;
    const uintptr_t start = it->first;
    const size_t len = it->second;
    a.free_list.erase(it);
    if (len > need) a.free_list[start + need] = len - need;
    a.live[start] = need;
    a.in_use += need;
    if (a.in_use > a.high_water) a.high_water = a.in_use;
    return reinterpret_cast<void*>(start);
  }
  ++a.failed;
  return nullptr;
}

extern "C" void axb_arena_free(void* ptr, long long /*size*/, int device, void* /*stream*/) {
  if (device < 0 || device >= 64 || ptr == nullptr) return;
  std::lock_guard<std::mutex> lock(g_arena_mu);
  Arena& a = g_arena[device];
  auto it = a.live.find(reinterpret_cast<uintptr_t>(ptr));
  if (it == a.live.end()) return;   // not ours (or from a replaced registration)
  uintptr_t start = it->first;
  size_t len = it->second;
  a.live.erase(it);
  a.in_use -= len;
  // coalesce with the neighbours
  auto next = a.free_list.lower_bound(start);
  if (next != a.free_list.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) { start = prev->first; len += prev->second; a.free_list.erase(prev); }
  }
  if (next != a.free_list.end() && start + len == next->first) { len += next->second; a.free_list.erase(next); }
  a.free_list[start] = len;
}

// what: 0 bytes handed out, 1 high-water mark, 2 registered size, 3 failed requests, 4 largest free block
extern "C" unsigned long long axb_arena_stat(int device, int what) {
  if (device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(g_arena_mu);
  const Arena& a = g_arena[device];
  switch (what) {
    case 0: return a.in_use;
    case 1: return a.high_water;
    case 2: return a.size;
    case 3: return a.failed;
    case 4: { size_t m = 0; for (auto& kv : a.free_list) if (kv.second > m) m = kv.second; return m; }
    default: return 0;
  }
}

// 1 when [ptr, ptr + nbytes) lies inside the registered range of `device`
extern "C" int axb_arena_contains(int device, const void* ptr, unsigned long long nbytes) {
  if (device < 0 || device >= 64) return 0;
  std::lock_guard<std::mutex> lock(g_arena_mu);
  const Arena& a = g_arena[device];
  const uintptr_t p = reinterpret_cast<uintptr_t>(ptr);
  return a.base != 0 && p >= a.base && p + nbytes <= a.base + a.size;
}
