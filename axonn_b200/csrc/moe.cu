// Expert-parallel token exchange over NVLink peer memory, fused with the
// permutation that routing implies.
//
//   scatter_rows  (dispatch; also the adjoint of gather_rows)
//       every routed (token, choice) copies its hidden row straight into the
//       buffer of the rank that owns the chosen expert, at the slot the router
//       assigned, with 16-byte peer stores; unused capacity slots are
//       zero-filled by the sender, so the owner's buffer is always fully defined.
//   gather_rows   (combine; also the adjoint of scatter_rows)
//       every routed (token, choice) pulls the row its expert produced from the
//       owner's buffer with 16-byte peer loads.
//
// Buffers are laid out [source rank][local expert][capacity][hidden] on the
// owner.  Cross-rank ordering uses monotonically increasing epoch flags in each
// rank's control block; every wait is bounded and reports through the device
// status word instead of hanging.
#include "common.cuh"

namespace axb {

struct MoeCtx {
  int n;                      // ranks in the expert-parallel group
  int rank;
  unsigned int epoch;
  int n_local;                // experts per rank
  void* buf_peer[8];          // exchange buffer of rank j
  unsigned int* wait_local;   // flags this kernel waits on before touching remote memory: [n]
  unsigned int wait_value;
  unsigned int* signal_peer[8];  // flag array (indexed by my rank) on rank j that this kernel sets when done
  unsigned int* counter;      // local CTA completion counter
  int* cnt_peer[8];           // dispatch: rank j's table [n_local][n] of the row counts per (expert, source)
  unsigned int* status;
  unsigned long long timeout_ns;
};

__device__ __forceinline__ void moe_st_release(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int moe_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads return true when every peer's flag has reached `value` (bounded).
__device__ __forceinline__ bool moe_wait_all(const MoeCtx& c, int* sh_ok) {
  if (threadIdx.x == 0) {
    int ok = 1;
    const uint64_t t0 = globaltimer_ns();
    for (int j = 0; j < c.n && ok; ++j) {
      if (j == c.rank) continue;
      while (static_cast<int>(moe_ld_acquire(c.wait_local + j) - c.wait_value) < 0) {
        if (globaltimer_ns() - t0 > c.timeout_ns) { ok = 0; report_status(c.status, 0x201u); break; }
      }
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;
}

// Every CTA passes here once per launch, also after a wait that ran out (`ok` false): the CTA counter is
// back at zero for the next call either way; the completion flag is published only when no CTA failed
// (c.counter + 1 counts the failed ones).
__device__ __forceinline__ void moe_signal_when_last(const MoeCtx& c, bool ok = true) {
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
          if (j != c.rank) moe_st_release(c.signal_peer[j] + c.rank, c.epoch);
    }
  }
}

// dest[a] = expert * C + slot for assignment a = token * k + choice; keep[a] != 0 when routed.
// counts[e] = number of kept assignments of expert e (<= C): slots >= counts[e] are zero-filled.
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ x, int x_by_token, const long long* __restrict__ dest,
                        const unsigned char* __restrict__ keep, const long long* __restrict__ counts, int T, int k,
                        int E, int C, int H, MoeCtx c) {
  __shared__ int sh_ok;
  if (!moe_wait_all(c, &sh_ok)) { moe_signal_when_last(c, false); return; }
  const int vec_per_row = H / 8;
  const long long n_assign = static_cast<long long>(T) * k;
  const long long n_slots = static_cast<long long>(E) * C;
  // work items: first the assignments, then the capacity slots (zero fill of the unused ones)
  for (long long item = blockIdx.x; item < n_assign + n_slots; item += gridDim.x) {
    uint4* dst;
    const uint4* src = nullptr;
    if (item < n_assign) {
      if (!keep[item]) continue;
      const long long d = dest[item];
      const int e = static_cast<int>(d / C), slot = static_cast<int>(d % C);
      const int owner = e / c.n_local, le = e % c.n_local;
      dst = reinterpret_cast<uint4*>(c.buf_peer[owner]) +
            ((static_cast<size_t>(le) * c.n + c.rank) * C + slot) * vec_per_row;
      const long long row = x_by_token ? item / k : item;
      src = reinterpret_cast<const uint4*>(x) + static_cast<size_t>(row) * vec_per_row;
    } else {
      const long long s = item - n_assign;
      const int e = static_cast<int>(s / C), slot = static_cast<int>(s % C);
      if (slot < counts[e]) continue;
      const int owner = e / c.n_local, le = e % c.n_local;
      dst = reinterpret_cast<uint4*>(c.buf_peer[owner]) +
            ((static_cast<size_t>(le) * c.n + c.rank) * C + slot) * vec_per_row;
    }
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x)
      dst[v] = src ? src[v] : make_uint4(0u, 0u, 0u, 0u);
  }
  // tell every owner how many of the capacity rows it received from this rank hold tokens (its expert GEMMs skip
  // the tiles without any)
  if (blockIdx.x == 0 && c.cnt_peer[0] != nullptr)
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      c.cnt_peer[e / c.n_local][(e % c.n_local) * c.n + c.rank] = static_cast<int>(counts[e]);
  moe_signal_when_last(c);
}

// out[a] = owner_buffer[dest[a]] for kept assignments, 0 otherwise.  out: [T*k, H].
__global__ void __launch_bounds__(256)
moe_gather_rows_kernel(__nv_bfloat16* __restrict__ out, const long long* __restrict__ dest,
                       const unsigned char* __restrict__ keep, int T, int k, int C, int H, MoeCtx c) {
  __shared__ int sh_ok;
  if (!moe_wait_all(c, &sh_ok)) { moe_signal_when_last(c, false); return; }
  const int vec_per_row = H / 8;
  const long long n_assign = static_cast<long long>(T) * k;
  for (long long item = blockIdx.x; item < n_assign; item += gridDim.x) {
    uint4* dst = reinterpret_cast<uint4*>(out) + static_cast<size_t>(item) * vec_per_row;
    if (!keep[item]) {
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const long long d = dest[item];
    const int e = static_cast<int>(d / C), slot = static_cast<int>(d % C);
    const int owner = e / c.n_local, le = e % c.n_local;
    const uint4* src = reinterpret_cast<const uint4*>(c.buf_peer[owner]) +
                       ((static_cast<size_t>(le) * c.n + c.rank) * C + slot) * vec_per_row;
    for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) dst[v] = src[v];
  }
  moe_signal_when_last(c);
}

// Copy `nvec` 16-byte words into a peer-readable buffer once every peer has released it (flags >= wait_value),
// then publish `epoch` to every peer: the publication step of the fused all-gather (a rank's weight shard goes
// into its outbox) as one launch instead of wait + copy + signal.
__global__ void __launch_bounds__(256)
copy_publish_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long nvec, MoeCtx c) {
  __shared__ int sh_ok;
  if (!moe_wait_all(c, &sh_ok)) { moe_signal_when_last(c, false); return; }
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
  moe_signal_when_last(c);
}

// One thread: publish `value` into flag[my rank] of every peer (after all prior work of the stream).
__global__ void moe_signal_kernel(MoeCtx c) {
  __threadfence_system();
  for (int j = 0; j < c.n; ++j)
    if (j != c.rank) moe_st_release(c.signal_peer[j] + c.rank, c.epoch);
}

// One block: bounded wait until every peer's flag reached wait_value.
__global__ void moe_wait_kernel(MoeCtx c) {
  __shared__ int sh_ok;
  moe_wait_all(c, &sh_ok);
}

int sm_count(int device);

}  // namespace axb

using namespace axb;

static int fill_ctx(MoeCtx& c, const AxbMoeCtx* h, int device) {
  if (!h || h->n < 1 || h->n > 8) { set_error("moe: group size must be 1..8"); return -1; }
  c.n = h->n; c.rank = h->rank; c.epoch = h->epoch; c.n_local = h->n_local;
  for (int j = 0; j < 8; ++j) { c.buf_peer[j] = h->buf_peer[j]; c.signal_peer[j] = h->signal_peer[j]; }
  c.wait_local = h->wait_local; c.wait_value = h->wait_value; c.counter = h->counter;
  for (int j = 0; j < 8; ++j) c.cnt_peer[j] = h->cnt_peer[j];
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("moe: no status word"); return -1; }
  c.status = st;
  c.timeout_ns = axb::wait_timeout_ns();
  return 0;
}

extern "C" int axb_moe_dispatch(const void* x, int x_by_token, const long long* dest, const unsigned char* keep,
                                const long long* counts, int T, int k, int E, int C, int H, const AxbMoeCtx* ctx,
                                int device, void* stream) {
  if (H % 8) { set_error("moe: hidden must be a multiple of 8"); return -1; }
  MoeCtx c;
  if (fill_ctx(c, ctx, device)) return -1;
  const long long items = static_cast<long long>(T) * k + static_cast<long long>(E) * C;
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  const int grid = static_cast<int>(items < cap ? (items < 1 ? 1 : items) : cap);
  moe_scatter_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, x_by_token, dest, keep,
                                                                 counts, T, k, E, C, H, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_moe_gather(void* out, const long long* dest, const unsigned char* keep, int T, int k, int C, int H,
                              const AxbMoeCtx* ctx, int device, void* stream) {
  if (H % 8) { set_error("moe: hidden must be a multiple of 8"); return -1; }
  MoeCtx c;
  if (fill_ctx(c, ctx, device)) return -1;
  const long long items = static_cast<long long>(T) * k;
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  const int grid = static_cast<int>(items < cap ? (items < 1 ? 1 : items) : cap);
  moe_gather_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)out, dest, keep, T, k, C, H, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// dst (this rank's peer-readable buffer) <- src, nbytes a multiple of 16, gated by the flags of `ctx` and followed
// by the publication of ctx->epoch to every peer.
extern "C" int axb_copy_publish(const void* src, void* dst, long long nbytes, const AxbMoeCtx* ctx, int device,
                                void* stream) {
  MoeCtx c;
  if (fill_ctx(c, ctx, device)) return -1;
  if (nbytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_error("axb_copy_publish: buffers must be 16-byte aligned and sized");
    return -1;
  }
  const long long nvec = nbytes / 16;
  const long long want = (nvec + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 2;
  const int grid = static_cast<int>(want < 1 ? 1 : (want > cap ? cap : want));
  copy_publish_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(dst), nvec, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_moe_signal(const AxbMoeCtx* ctx, int device, void* stream) {
  MoeCtx c;
  if (fill_ctx(c, ctx, device)) return -1;
  moe_signal_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_moe_wait(const AxbMoeCtx* ctx, int device, void* stream) {
  MoeCtx c;
  if (fill_ctx(c, ctx, device)) return -1;
  moe_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
