// Gradient all-reduce over NVLink peer memory with fused scale and dtype handling.
//
//   pack     a list of gradient tensors is copied into this rank's symmetric bucket (one launch over a
//            pointer table); the last CTA publishes READY = epoch to every peer;
//   reduce   two-shot in one kernel: rank k owns slice k of the bucket, loads that slice from every rank
//            (P2P loads, fp32 accumulation in rank order so that all ranks see identical bits), multiplies
//            by `scale` and stores the result into every rank's bucket (P2P stores).  Nobody else touches
//            slice k, so no further ordering is needed inside the kernel.  The last CTA publishes DONE;
//   unpack   waits for every peer's DONE (all slices of my bucket are final) and copies the bucket back
//            into the gradient tensors.
//
// Bytes on the wire per rank and direction: 2 (n-1)/n of the bucket, the two-shot optimum.  All waits
// are bounded and report through the device status word.
#include "common.cuh"

namespace axb {

struct CommCtx {
  int n, rank;
  unsigned int epoch;
  void* buf_peer[8];
  unsigned int* wait_local;      // [n] flags to wait on
  unsigned int* signal_peer[8];  // flag array on rank j (indexed by my rank) to publish completion
  unsigned int* counter;
  unsigned int* status;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ void c_st_release(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int c_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool comm_wait_all(const CommCtx& c, int* sh_ok) {
  if (threadIdx.x == 0) {
    int ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int j = 0; j < c.n && ok; ++j) {
      if (j == c.rank) continue;
      while (static_cast<int>(c_ld_acquire(c.wait_local + j) - c.epoch) < 0) {
        if (globaltimer_ns() - t0 > c.timeout_ns) {
          ok = 0;
          report_status(c.status, 0x301u);   // the first cause stays in the status word
          break;
        }
      }
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;
}
// Every CTA passes here exactly once per launch, also one whose wait ran out (`ok` false): the CTA counter
// returns to zero for the next call either way, and the completion flag is only published by a launch
// all of whose CTAs succeeded (peers of a failed launch run into their own deadline instead of reading
// an incomplete result).  c.counter + 1 collects the number of failed CTAs of the launch.
__device__ __forceinline__ void comm_signal_when_last(const CommCtx& c, bool ok = true) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicAdd(c.counter + 1, 1u);
    __threadfence_system();
    if (atomicAdd(c.counter, 1u) == gridDim.x - 1) {
      const unsigned int failed = atomicExch(c.counter + 1, 0u);
      *c.counter = 0;
      __threadfence_system();
      if (failed == 0)
        for (int j = 0; j < c.n; ++j)
          if (j != c.rank) c_st_release(c.signal_peer[j] + c.rank, c.epoch);
    }
  }
}

constexpr int PK_CHUNK = 1 << 15;

// table rows: {tensor ptr, numel, dtype (unused: all tensors share the bucket dtype), element offset in bucket,
//              chunk prefix}
__device__ __forceinline__ int pk_find(const long long* table, int n, long long chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (table[(size_t)mid * 5 + 4] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <typename T, bool TO_BUCKET>
__global__ void __launch_bounds__(256)
bucket_copy_kernel(const long long* __restrict__ table, int ntensors, long long total_chunks, T* bucket, CommCtx c,
                   int wait_first, int signal_last) {
  __shared__ int sh_ok;
  if (wait_first && c.n > 1 && !comm_wait_all(c, &sh_ok)) {
    if (signal_last) comm_signal_when_last(c, false);
    return;
  }
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int t = pk_find(table, ntensors, chunk);
    const long long* row = table + (size_t)t * 5;
    T* tensor = reinterpret_cast<T*>(row[0]);
    const long long numel = row[1];
    T* slot = bucket + row[3];
    const long long begin = (chunk - row[4]) * PK_CHUNK;
    const long long end = begin + PK_CHUNK < numel ? begin + PK_CHUNK : numel;
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
      if (TO_BUCKET) slot[i] = tensor[i]; else tensor[i] = slot[i];
    }
  }
  if (signal_last && c.n > 1) comm_signal_when_last(c);
}

template <typename T> struct V16;  // 16-byte vector of T <-> floats
template <> struct V16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};
template <> struct V16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return u;
  }
};

// nvec: number of 16-byte vectors in the bucket (padded so that nvec % n == 0)
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_twoshot_kernel(long long nvec, float scale, CommCtx c) {
  __shared__ int sh_ok;
  if (!comm_wait_all(c, &sh_ok)) { comm_signal_when_last(c, false); return; }
  const long long per = nvec / c.n;
  const long long lo = per * c.rank;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    float acc[V16<T>::N];
#pragma unroll
    for (int e = 0; e < V16<T>::N; ++e) acc[e] = 0.f;
    for (int j = 0; j < c.n; ++j) {
      const uint4 u = *(reinterpret_cast<const uint4*>(c.buf_peer[j]) + lo + i);
      float f[V16<T>::N];
      V16<T>::unpack(u, f);
#pragma unroll
      for (int e = 0; e < V16<T>::N; ++e) acc[e] += f[e];
    }
#pragma unroll
    for (int e = 0; e < V16<T>::N; ++e) acc[e] *= scale;
    const uint4 o = V16<T>::pack(acc);
    for (int j = 0; j < c.n; ++j) *(reinterpret_cast<uint4*>(c.buf_peer[j]) + lo + i) = o;
  }
  comm_signal_when_last(c);
}


// ----------------------------------------------------------------------------- in-switch (NVLS) all-reduce of the bucket
// Same contract as allreduce_twoshot_kernel, but the reduction happens inside the NVSwitch: rank k owns slice k of
// the bucket, loads the SUM of that slice over all ranks with one multimem.ld_reduce per 16 bytes (fp32 accumulation
// in the switch for bf16), scales it and broadcasts it to every rank's bucket with multimem.st.  `mc` is the
// multicast address of the bucket (the symmetric allocation is bound to an NVLink multicast object).  Per rank
// and direction only 1/n of the bucket crosses the link twice, independent of n.
template <typename T> struct MultiMem;
template <> struct MultiMem<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct MultiMem<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void* mc, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
                 ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

template <typename T>
__global__ void __launch_bounds__(512)
allreduce_nvls_kernel(long long nvec, float scale, uint8_t* mc, CommCtx c) {
  __shared__ int sh_ok;
  if (!comm_wait_all(c, &sh_ok)) { comm_signal_when_last(c, false); return; }
  const long long per = nvec / c.n;
  const long long lo = per * c.rank;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    uint8_t* addr = mc + (lo + i) * 16;
    uint4 u = MultiMem<T>::ld_reduce(addr);
    if (scale != 1.f) {
      float f[V16<T>::N];
      V16<T>::unpack(u, f);
#pragma unroll
      for (int e = 0; e < V16<T>::N; ++e) f[e] *= scale;
      u = V16<T>::pack(f);
    }
    MultiMem<T>::st(addr, u);
  }
  comm_signal_when_last(c);
}

// ----------------------------------------------------------------------------- one-kernel gradient all-reduce
// The whole data-parallel gradient all-reduce of a list of tensors in ONE launch, straight from and to the
// gradient tensors (no pack or unpack pass): the chunk list of the table is cut into n slices, rank k owns slice k.
//   phase 1  every rank reads its gradients of the slices it does not own and stores them into the owners'
//            receive slots (posted stores over NVLink);
//   phase 2  the owner adds its own gradients and the n-1 received partials in rank order (fp32 accumulation,
//            identical bits on every rank), multiplies by `scale`, writes the result back into its gradient
//            tensors and stores it into every peer's result area;
//   phase 3  every rank copies the slices it does not own from its result area into its gradient tensors.
// Phases are separated by epoch flags in peer memory (PUSHED, REDUCED); the last CTA of a phase publishes
// them.  All CTAs of the launch must be resident at once (grid <= 2 x #SMs at 512 threads); waits are bounded.
struct GradArCtx {
  int n, rank;
  unsigned int epoch;
  void* recv_peer[8];        // rank j's receive area: n slots (one per source rank) of slot_bytes
  void* result_peer[8];      // rank j's result area: one position per chunk of the table
  unsigned int* pushed_local;    // [n] epoch flags written by peers when their phase 1 is complete
  unsigned int* pushed_peer[8];
  unsigned int* reduced_local;   // [n] ... when their phase 2 is complete
  unsigned int* reduced_peer[8];
  unsigned int* counters;        // 3 words: CTA counters of phase 1 and 2, failed-CTA count (all zero between calls)
  unsigned long long slot_bytes;
  unsigned int* status;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ bool gar_wait_peers(const GradArCtx& c, const unsigned int* flags, int* sh_ok, unsigned int code) {
  if (threadIdx.x == 0) {
    int ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int j = 0; j < c.n && ok; ++j) {
      if (j == c.rank) continue;
      while (static_cast<int>(c_ld_acquire(flags + j) - c.epoch) < 0) {
        if (globaltimer_ns() - t0 > c.timeout_ns) { ok = 0; report_status(c.status, code); break; }
      }
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;
}
// The last CTA to pass publishes `epoch` into flag[rank] of every peer - unless a CTA of this launch passed with
// `ok` false (a wait of an earlier phase ran out; counters[2] counts those): the peers then run into their own
// deadline instead of consuming an incomplete result.  The counter is back at zero either way.
__device__ __forceinline__ void gar_phase_done(const GradArCtx& c, unsigned int* counter, unsigned int* const* flag_peer,
                                               bool ok = true) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicAdd(c.counters + 2, 1u);
    __threadfence_system();
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      const unsigned int failed = atomicExch(c.counters + 2, 0u);
      *counter = 0;
      __threadfence_system();
      if (failed == 0)
        for (int j = 0; j < c.n; ++j)
          if (j != c.rank) c_st_release(flag_peer[j] + c.rank, c.epoch);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(512)
grad_allreduce_kernel(const long long* __restrict__ table, int ntensors, long long total_chunks, long long chunks_per_slice,
                      float scale, GradArCtx c) {
  constexpr int VN = V16<T>::N;                 // elements per 16-byte vector
  __shared__ int sh_ok;
  const long long my_lo = chunks_per_slice * c.rank;
  const long long my_hi = my_lo + chunks_per_slice < total_chunks ? my_lo + chunks_per_slice : total_chunks;
  // ---- phase 1: my gradients of foreign slices -> the owners' receive slots
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    if (chunk >= my_lo && chunk < my_hi) continue;
    const int owner = static_cast<int>(chunk / chunks_per_slice);
    const int t = pk_find(table, ntensors, chunk);
    const long long* row = table + static_cast<size_t>(t) * 5;
    const T* tensor = reinterpret_cast<const T*>(row[0]);
    const long long numel = row[1];
    const long long begin = (chunk - row[4]) * PK_CHUNK;
    const long long end = begin + PK_CHUNK < numel ? begin + PK_CHUNK : numel;
    T* slot = reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(c.recv_peer[owner]) + c.rank * c.slot_bytes) +
              (chunk - owner * chunks_per_slice) * PK_CHUNK;
    if ((reinterpret_cast<uintptr_t>(tensor) & 15) == 0) {
      const long long nv = (end - begin) / VN;
      const uint4* sp = reinterpret_cast<const uint4*>(tensor + begin);
      uint4* dp = reinterpret_cast<uint4*>(slot);
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) dp[i] = sp[i];
      for (long long i = begin + nv * VN + threadIdx.x; i < end; i += blockDim.x) slot[i - begin] = tensor[i];
    } else {
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) slot[i - begin] = tensor[i];
    }
  }
  gar_phase_done(c, c.counters, c.pushed_peer);
  // ---- phase 2: reduce my slice, write it back and hand it to every peer
  bool ok = gar_wait_peers(c, c.pushed_local, &sh_ok, 0x302u);
  if (ok) {
    for (long long chunk = my_lo + blockIdx.x; chunk < my_hi; chunk += gridDim.x) {
      const int t = pk_find(table, ntensors, chunk);
      const long long* row = table + static_cast<size_t>(t) * 5;
      T* tensor = reinterpret_cast<T*>(row[0]);
      const long long numel = row[1];
      const long long begin = (chunk - row[4]) * PK_CHUNK;
      const long long end = begin + PK_CHUNK < numel ? begin + PK_CHUNK : numel;
      const long long in_slot = (chunk - my_lo) * PK_CHUNK;
      const bool vec = (reinterpret_cast<uintptr_t>(tensor) & 15) == 0;
      const long long nv = vec ? (end - begin) / VN : 0;
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
        float acc[VN];
#pragma unroll
        for (int e = 0; e < VN; ++e) acc[e] = 0.f;
        for (int j = 0; j < c.n; ++j) {       // rank order: identical bits on every rank
          uint4 u;
          if (j == c.rank) u = *(reinterpret_cast<const uint4*>(tensor + begin) + i);
          else u = *(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(c.recv_peer[c.rank]) +
                                                     j * c.slot_bytes) + in_slot) + i);
          float f[VN];
          V16<T>::unpack(u, f);
#pragma unroll
          for (int e = 0; e < VN; ++e) acc[e] += f[e];
        }
#pragma unroll
        for (int e = 0; e < VN; ++e) acc[e] *= scale;
        const uint4 o = V16<T>::pack(acc);
        *(reinterpret_cast<uint4*>(tensor + begin) + i) = o;
        for (int j = 0; j < c.n; ++j)
          if (j != c.rank) *(reinterpret_cast<uint4*>(reinterpret_cast<T*>(c.result_peer[j]) + chunk * PK_CHUNK) + i) = o;
      }
      for (long long i = begin + nv * VN + threadIdx.x; i < end; i += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < c.n; ++j) {
          const T v = (j == c.rank) ? tensor[i]
                                    : (reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(c.recv_peer[c.rank]) + j * c.slot_bytes) +
                                       in_slot)[i - begin];
          acc += static_cast<float>(v);
        }
        const T o = static_cast<T>(acc * scale);
        tensor[i] = o;
        for (int j = 0; j < c.n; ++j)
          if (j != c.rank) (reinterpret_cast<T*>(c.result_peer[j]) + chunk * PK_CHUNK)[i - begin] = o;
      }
    }
  }
  gar_phase_done(c, c.counters + 1, c.reduced_peer, ok);
  // ---- phase 3: the other slices come out of my result area
  ok = ok && gar_wait_peers(c, c.reduced_local, &sh_ok, 0x303u);
  if (!ok) return;
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    if (chunk >= my_lo && chunk < my_hi) continue;
    const int t = pk_find(table, ntensors, chunk);
    const long long* row = table + static_cast<size_t>(t) * 5;
    T* tensor = reinterpret_cast<T*>(row[0]);
    const long long numel = row[1];
    const long long begin = (chunk - row[4]) * PK_CHUNK;
    const long long end = begin + PK_CHUNK < numel ? begin + PK_CHUNK : numel;
    const T* res = reinterpret_cast<const T*>(c.result_peer[c.rank]) + chunk * PK_CHUNK;
    if ((reinterpret_cast<uintptr_t>(tensor) & 15) == 0) {
      const long long nv = (end - begin) / VN;
      const uint4* sp = reinterpret_cast<const uint4*>(res);
      uint4* dp = reinterpret_cast<uint4*>(tensor + begin);
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) dp[i] = sp[i];
      for (long long i = begin + nv * VN + threadIdx.x; i < end; i += blockDim.x) tensor[i] = res[i - begin];
    } else {
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) tensor[i] = res[i - begin];
    }
  }
}

}  // namespace axb

using namespace axb;

static int fill_comm(CommCtx& c, const AxbCommCtx* h, int device) {
  if (!h || h->n < 1 || h->n > 8) { set_error("allreduce: group size must be 1..8"); return -1; }
  c.n = h->n; c.rank = h->rank; c.epoch = h->epoch;
  for (int j = 0; j < 8; ++j) { c.buf_peer[j] = h->buf_peer[j]; c.signal_peer[j] = h->signal_peer[j]; }
  c.wait_local = h->wait_local; c.counter = h->counter;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("allreduce: no status word"); return -1; }
  c.status = st;
  c.timeout_ns = 2 * axb::wait_timeout_ns();
  return 0;
}

// direction 0: tensors -> bucket (then publish READY); direction 1: wait DONE, bucket -> tensors.
extern "C" int axb_bucket_copy(const long long* table, int ntensors, long long total_chunks, void* bucket, int dtype,
                               int direction, const AxbCommCtx* ctx, int device, void* stream) {
  CommCtx c;
  if (fill_comm(c, ctx, device)) return -1;
  const int cap = sm_count(device) * 8;
  const int grid = (int)(total_chunks < cap ? (total_chunks < 1 ? 1 : total_chunks) : cap);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) {
    if (direction == 0) bucket_copy_kernel<float, true><<<grid, 256, 0, s>>>(table, ntensors, total_chunks, (float*)bucket, c, 0, 1);
    else bucket_copy_kernel<float, false><<<grid, 256, 0, s>>>(table, ntensors, total_chunks, (float*)bucket, c, 1, 0);
  } else {
    if (direction == 0) bucket_copy_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(table, ntensors, total_chunks, (__nv_bfloat16*)bucket, c, 0, 1);
    else bucket_copy_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(table, ntensors, total_chunks, (__nv_bfloat16*)bucket, c, 1, 0);
  }
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// In-place two-shot all-reduce of every rank's bucket (nbytes, padded to a multiple of 16 * n), times `scale`.
extern "C" int axb_allreduce_twoshot(long long nbytes, int dtype, float scale, const AxbCommCtx* ctx, int device,
                                     void* stream) {
  CommCtx c;
  if (fill_comm(c, ctx, device)) return -1;
  if (nbytes % (16 * c.n)) { set_error("allreduce: bucket bytes must be a multiple of 16 * group size"); return -1; }
  const long long nvec = nbytes / 16;
  const long long per = nvec / c.n;
  long long blocks = (per + 511) / 512;
  const int cap = sm_count(device) * 4;
  const int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  if (dtype == 0) allreduce_twoshot_kernel<float><<<grid, 512, 0, (cudaStream_t)stream>>>(nvec, scale, c);
  else allreduce_twoshot_kernel<__nv_bfloat16><<<grid, 512, 0, (cudaStream_t)stream>>>(nvec, scale, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// Sum the tensors of `table` ({ptr, numel, -, -, chunk prefix} rows, chunks of 32768 elements) over the group,
// times `scale`, in place, in one kernel (see grad_allreduce_kernel).  `ctx` names the peer-mapped receive and
// result areas: recv holds n slots of chunks_per_slice * 32768 elements, result total_chunks * 32768 elements.
extern "C" int axb_grad_allreduce(const long long* table, int ntensors, long long total_chunks, long long chunks_per_slice,
                                  int dtype, float scale, const AxbGradArCtx* h, int device, void* stream) {
  if (!h || h->n < 2 || h->n > 8) { set_error("grad all-reduce: group size must be 2..8"); return -1; }
  if (chunks_per_slice * h->n < total_chunks) { set_error("grad all-reduce: slices do not cover the chunk list"); return -1; }
  GradArCtx c;
  c.n = h->n; c.rank = h->rank; c.epoch = h->epoch;
  for (int j = 0; j < 8; ++j) {
    c.recv_peer[j] = h->recv_peer[j]; c.result_peer[j] = h->result_peer[j];
    c.pushed_peer[j] = h->pushed_peer[j]; c.reduced_peer[j] = h->reduced_peer[j];
  }
  c.pushed_local = h->pushed_local; c.reduced_local = h->reduced_local; c.counters = h->counters;
  c.slot_bytes = h->slot_bytes;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("grad all-reduce: no status word"); return -1; }
  c.status = st;
  c.timeout_ns = 2 * axb::wait_timeout_ns();
  // all CTAs wait on each other's phases: keep the grid within what is resident at once
  const long long cap = static_cast<long long>(sm_count(device)) * 2;
  const int grid = static_cast<int>(total_chunks < cap ? (total_chunks < 1 ? 1 : total_chunks) : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) grad_allreduce_kernel<float><<<grid, 512, 0, s>>>(table, ntensors, total_chunks, chunks_per_slice, scale, c);
  else grad_allreduce_kernel<__nv_bfloat16><<<grid, 512, 0, s>>>(table, ntensors, total_chunks, chunks_per_slice, scale, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// In-place all-reduce of every rank's bucket through the NVSwitch (multimem); `mc_bucket` is the multicast
// address of the bucket.  Same flags as axb_allreduce_twoshot.
extern "C" int axb_allreduce_nvls(long long nbytes, int dtype, float scale, void* mc_bucket, const AxbCommCtx* ctx,
                                  int device, void* stream) {
  CommCtx c;
  if (fill_comm(c, ctx, device)) return -1;
  if (!mc_bucket) { set_error("allreduce (NVLS): no multicast address"); return -1; }
  if (nbytes % (16 * c.n)) { set_error("allreduce: bucket bytes must be a multiple of 16 * group size"); return -1; }
  const long long nvec = nbytes / 16;
  const long long per = nvec / c.n;
  long long blocks = (per + 511) / 512;
  const int cap = sm_count(device) * 2;
  const int grid = (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
  if (dtype == 0) allreduce_nvls_kernel<float><<<grid, 512, 0, (cudaStream_t)stream>>>(nvec, scale, (uint8_t*)mc_bucket, c);
  else allreduce_nvls_kernel<__nv_bfloat16><<<grid, 512, 0, (cudaStream_t)stream>>>(nvec, scale, (uint8_t*)mc_bucket, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
