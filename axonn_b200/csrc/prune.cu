// Gradient pruning: keep the k largest-magnitude entries of a tensor, zero the rest.
//
// The threshold (k-th largest |g|) comes from a radix select on the magnitude
// bits instead of a sort: one histogram pass over the top 15 magnitude bits
// (block-private shared-memory histograms, flushed with atomics), a one-block
// suffix scan that finds the bin holding the k-th element, for fp32 a second
// histogram over the next 16 bits restricted to that bin, then one masking
// pass.  bf16 tensors (15 magnitude bits in total) need exactly two passes
// over the data.  Ties at the threshold are all kept (|g| >= threshold), the
// same rule as thresholding with the k-th value of a sort.
//
// Scratch: 32768 + 65536 + 8 32-bit words, supplied by the caller.
#include <mutex>

#include "common.cuh"

namespace axb {

constexpr int PR_BINS1 = 32768;
constexpr int PR_BINS2 = 65536;
constexpr int PR_THREADS = 1024;
constexpr int PR_WORK_WORDS = PR_BINS1 + PR_BINS2 + 8;
// dtype codes are the library-wide ones of axonn_b200.h: 0 bf16, 1 fp16, 2 fp32
constexpr int PR_F32 = 2;

__device__ __forceinline__ uint32_t mag_bits(const void* g, long long i, int dtype) {
  if (dtype == PR_F32) return reinterpret_cast<const uint32_t*>(g)[i] & 0x7FFFFFFFu;
  return (static_cast<uint32_t>(reinterpret_cast<const uint16_t*>(g)[i]) & 0x7FFFu) << 16;
}

// level 1: histogram of the top 15 magnitude bits
__global__ void __launch_bounds__(PR_THREADS)
prune_hist1_kernel(const void* __restrict__ g, long long n, int dtype, unsigned int* __restrict__ hist) {
  extern __shared__ unsigned int sh[];
  for (int i = threadIdx.x; i < PR_BINS1; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  if (dtype != PR_F32 && (reinterpret_cast<uintptr_t>(g) & 15) == 0) {
    const long long nv = n / 8;
    const uint4* q = reinterpret_cast<const uint4*>(g);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
      const uint4 u = q[i];
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        atomicAdd(&sh[w[k] & 0x7FFFu], 1u);
        atomicAdd(&sh[(w[k] >> 16) & 0x7FFFu], 1u);
      }
    }
    for (long long i = nv * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
      atomicAdd(&sh[mag_bits(g, i, dtype) >> 16], 1u);
  } else {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
      atomicAdd(&sh[mag_bits(g, i, dtype) >> 16], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < PR_BINS1; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], sh[i]);
}

// One block: find the largest bin b with  count(bins > b) < k <= count(bins >= b).
// meta_out[0] = b, meta_out[1] = k - count(bins > b)  (rank of the target inside bin b)
template <int BINS>
__global__ void __launch_bounds__(PR_THREADS)
prune_select_kernel(const unsigned int* __restrict__ hist, const long long* __restrict__ k_in, long long k_const,
                    long long* __restrict__ meta_out) {
  __shared__ unsigned long long part[PR_THREADS];
  constexpr int PER = BINS / PR_THREADS;
  const long long k = k_in ? *k_in : k_const;
  // thread t owns bins [BINS - (t+1)*PER, BINS - t*PER): thread 0 holds the largest magnitudes
  const int hi = BINS - threadIdx.x * PER;
  unsigned long long mine = 0;
  for (int b = hi - PER; b < hi; ++b) mine += hist[b];
  part[threadIdx.x] = mine;
  __syncthreads();
  // inclusive prefix over threads (Hillis-Steele)
  for (int off = 1; off < PR_THREADS; off <<= 1) {
    unsigned long long v = threadIdx.x >= off ? part[threadIdx.x - off] : 0;
    __syncthreads();
    part[threadIdx.x] += v;
    __syncthreads();
  }
  const unsigned long long incl = part[threadIdx.x], excl = incl - mine;
  if (excl < (unsigned long long)k && (unsigned long long)k <= incl) {
    unsigned long long above = excl;
    for (int b = hi - 1; b >= hi - PER; --b) {
      const unsigned long long c = hist[b];
      if (above + c >= (unsigned long long)k) { meta_out[0] = b; meta_out[1] = k - (long long)above; return; }
      above += c;
    }
  }
  if (threadIdx.x == PR_THREADS - 1 && incl < (unsigned long long)k) { meta_out[0] = 0; meta_out[1] = 1; }  // k > n: keep all
}

// level 2 (fp32 only): histogram of the next 16 bits among elements whose top bits equal meta[0]
__global__ void prune_hist2_kernel(const void* __restrict__ g, long long n, const long long* __restrict__ meta,
                                   unsigned int* __restrict__ hist2) {
  const uint32_t top = (uint32_t)meta[0];
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const uint32_t m = reinterpret_cast<const uint32_t*>(g)[i] & 0x7FFFFFFFu;
    if ((m >> 16) == top) atomicAdd(&hist2[m & 0xFFFFu], 1u);
  }
}

// thr = 31-bit magnitude threshold: keep |g| bits >= thr
__global__ void prune_mask_kernel(void* __restrict__ g, long long n, int dtype, const long long* __restrict__ meta1,
                                  const long long* __restrict__ meta2) {
  const uint32_t thr = ((uint32_t)meta1[0] << 16) | (dtype == PR_F32 ? (uint32_t)meta2[0] : 0u);
  if (dtype != PR_F32 && (reinterpret_cast<uintptr_t>(g) & 15) == 0) {
    const long long nv = n / 8;
    uint4* q = reinterpret_cast<uint4*>(g);
    const uint32_t t16 = thr >> 16;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv; i += (long long)gridDim.x * blockDim.x) {
      uint4 u = q[i];
      uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if ((w[k] & 0x7FFFu) < t16) w[k] &= 0xFFFF0000u;
        if (((w[k] >> 16) & 0x7FFFu) < t16) w[k] &= 0x0000FFFFu;
      }
      q[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (long long i = nv * 8 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
      if (mag_bits(g, i, dtype) < thr) reinterpret_cast<uint16_t*>(g)[i] = 0;
  } else {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
      if (mag_bits(g, i, dtype) < thr) {
        if (dtype == PR_F32) reinterpret_cast<uint32_t*>(g)[i] = 0; else reinterpret_cast<uint16_t*>(g)[i] = 0;
      }
    }
  }
}

int sm_count(int device);

// Shared by the allocating and the static-scratch entry points.
int prune_topk_launch(void* g, long long n, int dtype, long long k, unsigned int* work, int device, cudaStream_t s) {
  if (n <= 0) return 0;
  if (k <= 0) { AXB_CUDA(cudaMemsetAsync(g, 0, (size_t)n * (dtype == PR_F32 ? 4 : 2), s)); return 0; }
  if (k >= n) return 0;
  unsigned int* hist1 = work;
  unsigned int* hist2 = work + PR_BINS1;
  long long* meta = reinterpret_cast<long long*>(work + PR_BINS1 + PR_BINS2);  // meta1 = meta[0..1], meta2 = meta[2..3]
  AXB_CUDA(cudaMemsetAsync(work, 0, sizeof(unsigned int) * PR_WORK_WORDS, s));
  static bool configured[64] = {false};
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(prune_hist1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PR_BINS1 * 4));
    configured[device & 63] = true;
  }
  const int sms = sm_count(device);
  prune_hist1_kernel<<<sms, PR_THREADS, PR_BINS1 * 4, s>>>(g, n, dtype, hist1);
  AXB_CUDA(cudaGetLastError());
  prune_select_kernel<PR_BINS1><<<1, PR_THREADS, 0, s>>>(hist1, nullptr, k, meta);
  AXB_CUDA(cudaGetLastError());
  if (dtype == PR_F32) {
    prune_hist2_kernel<<<sms * 4, 512, 0, s>>>(g, n, meta, hist2);
    AXB_CUDA(cudaGetLastError());
    prune_select_kernel<PR_BINS2><<<1, PR_THREADS, 0, s>>>(hist2, meta + 1, 0, meta + 2);
    AXB_CUDA(cudaGetLastError());
  }
  prune_mask_kernel<<<sms * 4, 512, 0, s>>>(g, n, dtype, meta, meta + 2);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace axb

extern "C" int axb_prune_workspace_words(void) { return axb::PR_WORK_WORDS; }

// g: gradient tensor (dtype 0 bf16, 1 fp16, 2 fp32: the library-wide codes), modified in place; keeps the k largest |g|.
// work: device scratch of axb_prune_workspace_words() 32-bit words (8-byte aligned).
extern "C" int axb_prune_topk(void* g, long long n, int dtype, long long k, void* work, int device, void* stream) {
  if (!work) { axb::set_error("prune: workspace is null"); return -1; }
  if (dtype < 0 || dtype > 2) { axb::set_error("prune: bad dtype %d (0 bf16, 1 fp16, 2 fp32)", dtype); return -1; }
  return axb::prune_topk_launch(g, n, dtype, k, static_cast<unsigned int*>(work), device, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Entry point for callers that must not allocate.
//
// Some programs that embed this library own every byte of device memory themselves (a serving
// process that hands the whole GPU to its own pool at start-up, or one that runs under a
// "nothing is allocated after initialisation" rule): asking the driver for a workspace in the
// middle of their step can fail or fragment their pool, so they cannot supply freshly allocated
// scratch and do not want this library to allocate it behind their back.  For them the
// radix-select scratch lives in the library image itself, in the array below.
//
// The array takes PR_WORK_WORDS * 4 bytes (32768 + 65536 + 8 words = 393,248 bytes) of every
// GPU that loads the library, from load until the process exits.
static __device__ __align__(256) unsigned int g_prune_static_scratch[axb::PR_WORK_WORDS];

namespace axb {
// Largest tensor the static entry point accepts: the histogram counters are 32-bit.
constexpr long long PR_STATIC_MAX_NUMEL = 2147483647LL;
// Device address of g_prune_static_scratch per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel can use, so the address is looked up once per
// device with cudaGetSymbolAddress while that device is current.
static unsigned int* g_prune_static_ptr[64] = {nullptr};
static std::mutex g_prune_static_mu;   // first-use lookup may race between host threads
}  // namespace axb

// Keep the k largest-magnitude entries of g (dtype 0 bf16, 1 fp16, 2 fp32), zero the rest, in place,
// like axb_prune_topk, but with no workspace argument and without allocating anything: no cudaMalloc,
// no cudaFree, no allocating library call.
//
// * `device` must be the calling thread's current device on every call (checked; the launches and the
//   clearing of the scratch go to the current device).  The first call on a device also looks up the
//   scratch array's device address: make that first call before starting any stream capture on the device.
// * n must not exceed 2,147,483,647 elements; larger tensors are rejected with an error.
// * All calls on a device share one scratch array.  It is cleared at the start of each call, so
//   nothing needs to be reset between calls, but two calls whose kernels may overlap on the GPU
//   (different streams without an ordering between them) race on it: serialise them.
extern "C" int axb_prune_topk_static(void* g, long long n, int dtype, long long k, int device, void* stream) {
  using namespace axb;
  if (n > PR_STATIC_MAX_NUMEL) {
    set_error("axb_prune_topk_static: %lld elements exceed the supported maximum of %lld", n, PR_STATIC_MAX_NUMEL);
    return -1;
  }
  if (device < 0 || device >= 64) { set_error("axb_prune_topk_static: bad device index %d", device); return -1; }
  if (dtype < 0 || dtype > 2) { set_error("axb_prune_topk_static: bad dtype %d", dtype); return -1; }
  int current = -1;
  AXB_CUDA(cudaGetDevice(&current));
  if (current != device) {
    set_error("axb_prune_topk_static: device %d must be the current device (current is %d)", device, current);
    return -1;
  }
  std::lock_guard<std::mutex> lock(g_prune_static_mu);
  if (g_prune_static_ptr[device] == nullptr) {
    unsigned int* p = nullptr;
    AXB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_prune_static_scratch));
    if (p == nullptr) { set_error("axb_prune_topk_static: scratch symbol has no device address"); return -1; }
    g_prune_static_ptr[device] = p;
  }
  return prune_topk_launch(g, n, dtype, k, g_prune_static_ptr[device], device, (cudaStream_t)stream);
}
