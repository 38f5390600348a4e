// Peer-memory data movement kernels that replace library collectives around the tensor-parallel layers:
//
//   a2a_rows        all-to-all-v of row blocks: every rank stores, for every destination, a 2-D block of its
//                   input (rows x row_bytes, arbitrary row pitch) straight into the destination's output tensor
//                   at a given offset and pitch, over NVLink.  One kernel covers the layout switches of the
//                   "easy" tensor-parallel mode - batch-gather/channel-scatter, channel-gather/batch-scatter
//                   and the all-gather-v of unequal row blocks (reference: the all_to_all calls of
//                   axonn/intra_layer/asym_communication.py:44,144,170) - without pack or unpack copies: the
//                   transposition is done by the addressing.
//   embedding rows  forward: every token fetches its row of the depth-sharded embedding table from the rank
//                   that owns it (reference: the whole table is all-gathered first,
//                   axonn/intra_layer/embedding.py:161-172); backward: token gradients are added into the
//                   owner's gradient shard with remote fp32 atomics.
//
// Outputs live in the peer-mapped output arena (see arena.cu); every rank announces the offset of its output
// through a mailbox in peer memory, so ranks need not allocate at equal offsets.  Every wait is bounded and
// reports through the device status word.
#include "common.cuh"

namespace axb {

struct P2pCtx {
  int n, rank;
  unsigned int epoch;
  void* arena_peer[8];
  unsigned int* mail_local;
  unsigned int* mail_peer[8];
  unsigned int* done_local;
  unsigned int* done_peer[8];
  unsigned int* counter;
  unsigned long long out_off;
  unsigned int* status;
  unsigned long long timeout_ns;
};

struct RowBlock {
  const uint8_t* src;            // first row of the block in my input
  long long src_pitch;           // bytes between rows of the input
  long long dst_off;             // byte offset of the block's first row inside the destination's output
  long long dst_pitch;           // bytes between rows of the destination's output
  long long rows;
  long long row_bytes;           // payload per row (multiple of 16)
};
struct RowBlocks { RowBlock b[8]; };

__device__ __forceinline__ void p2p_st_release(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int p2p_ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool p2p_wait_ge(const unsigned int* flag, unsigned int want, uint64_t timeout_ns) {
  const uint64_t t0 = globaltimer_ns();
  while (static_cast<int>(p2p_ld_acquire(flag) - want) < 0) {
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
  return true;
}

// Announce my output offset (block 0), then learn every peer's; leaves the peers' output base pointers in
// shared memory.  Returns false (all threads) when a peer never announced.
__device__ __forceinline__ bool p2p_exchange_offsets(const P2pCtx& c, unsigned long long* sh_out, int* sh_ok) {
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) {
      for (int j = 0; j < c.n; ++j) {
        if (j == c.rank) continue;
        unsigned int* rec = c.mail_peer[j] + c.rank * 8;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 0), "r"(static_cast<unsigned>(c.out_off)) : "memory");
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 1), "r"(static_cast<unsigned>(c.out_off >> 32)) : "memory");
        p2p_st_release(rec + 4, c.epoch);
      }
    }
    int ok = 1;
    for (int j = 0; j < c.n; ++j) {
      if (j == c.rank) { sh_out[j] = reinterpret_cast<unsigned long long>(c.arena_peer[j]) + c.out_off; continue; }
      const unsigned int* rec = c.mail_local + j * 8;
      if (!p2p_wait_ge(rec + 4, c.epoch, c.timeout_ns)) { ok = 0; report_status(c.status, 0x501u); break; }
      const unsigned long long off = (static_cast<unsigned long long>(__ldcv(rec + 1)) << 32) | __ldcv(rec + 0);
      sh_out[j] = reinterpret_cast<unsigned long long>(c.arena_peer[j]) + off;
    }
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok != 0;
}

// Every block passes here once: the last one publishes this rank's completion and waits (bounded) until every
// peer has finished storing into this rank's output.  `ok` false: a wait of this block ran out.
__device__ __forceinline__ void p2p_finish(const P2pCtx& c, bool ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!ok) atomicAdd(c.counter + 1, 1u);
    __threadfence_system();
    if (atomicAdd(c.counter, 1u) == gridDim.x - 1) {
      const unsigned int failed = atomicExch(c.counter + 1, 0u);
      *c.counter = 0;
      __threadfence_system();
      if (failed == 0) {
        for (int j = 0; j < c.n; ++j)
          if (j != c.rank) p2p_st_release(c.done_peer[j] + c.rank, c.epoch);
        for (int j = 0; j < c.n; ++j) {
          if (j == c.rank) continue;
          if (!p2p_wait_ge(c.done_local + j, c.epoch, c.timeout_ns)) { report_status(c.status, 0x502u); break; }
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256)
a2a_rows_kernel(RowBlocks blocks, P2pCtx c) {
  __shared__ unsigned long long sh_out[8];
  __shared__ int sh_ok;
  if (!p2p_exchange_offsets(c, sh_out, &sh_ok)) { p2p_finish(c, false); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long me = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  // destinations in ring order starting behind this rank, so that the ranks do not all store to the same peer
  for (int s = 1; s <= c.n; ++s) {
    const int j = (c.rank + s) % c.n;
    const RowBlock& b = blocks.b[j];
    uint8_t* dst = reinterpret_cast<uint8_t*>(sh_out[j]) + b.dst_off;
    // work unit = one 2 KB piece of one row (four 16-byte words per lane in flight), so that the parallelism
    // does not depend on the shape: a single row of 100 MB spreads over the whole grid like 100k short rows do
    const long long vecs = b.row_bytes >> 4;
    const long long pieces = (vecs + 127) >> 7;
    const long long units = b.rows * pieces;
    for (long long u = me; u < units; u += warps) {
      const long long row = u / pieces, v0 = (u - row * pieces) << 7;
      const uint4* sp = reinterpret_cast<const uint4*>(b.src + row * b.src_pitch) + v0;
      uint4* dp = reinterpret_cast<uint4*>(dst + row * b.dst_pitch) + v0;
      const long long left = vecs - v0;
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (lane + k * 32 < left) r[k] = sp[lane + k * 32];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (lane + k * 32 < left) dp[lane + k * 32] = r[k];
    }
  }
  p2p_finish(c, true);
}

// out[t, :] = table_shard(owner(ids[t]))[ids[t] % rows_per_shard, :]; rows of `row_bytes` (multiple of 16).
// shard_peer[j]: rank j's published shard.  One warp per token row, four 16-byte loads in flight per lane.
__global__ void __launch_bounds__(256)
embedding_fetch_kernel(const long long* __restrict__ ids, long long n_tokens, uint8_t* __restrict__ out,
                       long long row_bytes, long long rows_per_shard, P2pCtx c) {
  __shared__ int sh_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int j = 0; j < c.n && ok; ++j) {
      if (j == c.rank) continue;
      if (!p2p_wait_ge(c.mail_local + j * 8 + 4, c.epoch, c.timeout_ns)) { ok = 0; report_status(c.status, 0x503u); }
    }
    sh_ok = ok;
  }
  __syncthreads();
  if (!sh_ok) { p2p_finish(c, false); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  const long long vecs = row_bytes >> 4;
  for (long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp; t < n_tokens; t += warps) {
    const long long id = ids[t];
    const int owner = static_cast<int>(id / rows_per_shard);
    const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(c.arena_peer[owner]) +
                                                     (id - owner * rows_per_shard) * row_bytes);
    uint4* dp = reinterpret_cast<uint4*>(out + t * row_bytes);
    for (long long v0 = lane; v0 < vecs; v0 += 128) {
      uint4 r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (v0 + k * 32 < vecs) r[k] = __ldcg(sp + v0 + k * 32);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (v0 + k * 32 < vecs) dp[v0 + k * 32] = r[k];
    }
  }
  p2p_finish(c, true);
}

// grad_shard(owner(ids[t]))[ids[t] % rows_per_shard, :] += dy[t, :]  with fp32 atomics into the owner's
// (peer-mapped, fp32) gradient shard.  dy is bf16 [n_tokens, H].
__global__ void __launch_bounds__(256)
embedding_scatter_add_kernel(const long long* __restrict__ ids, long long n_tokens, const __nv_bfloat16* __restrict__ dy,
                             int H, long long rows_per_shard, P2pCtx c) {
  __shared__ int sh_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int j = 0; j < c.n && ok; ++j) {
      if (j == c.rank) continue;
      if (!p2p_wait_ge(c.mail_local + j * 8 + 4, c.epoch, c.timeout_ns)) { ok = 0; report_status(c.status, 0x504u); }
    }
    sh_ok = ok;
  }
  __syncthreads();
  if (!sh_ok) { p2p_finish(c, false); return; }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long warps = static_cast<long long>(gridDim.x) * (blockDim.x >> 5);
  for (long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp; t < n_tokens; t += warps) {
    const long long id = ids[t];
    const int owner = static_cast<int>(id / rows_per_shard);
    float* gp = reinterpret_cast<float*>(c.arena_peer[owner]) + (id - owner * rows_per_shard) * H;
    const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(dy + t * H);
    for (int h2 = lane; h2 < H / 2; h2 += 32) {
      const float2 v = __bfloat1622float2(sp[h2]);
      // two fp32 adds per 8 bytes; red (no return value) so that the remote atomics are posted
      asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(gp + 2 * h2), "f"(v.x) : "memory");
      asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(gp + 2 * h2 + 1), "f"(v.y) : "memory");
    }
  }
  p2p_finish(c, true);
}

// One thread: tell every peer that this rank's buffer (shard, or zeroed gradient shard) of call `epoch` is ready.
__global__ void p2p_publish_kernel(P2pCtx c) {
  __threadfence_system();
  for (int j = 0; j < c.n; ++j)
    if (j != c.rank) p2p_st_release(c.mail_peer[j] + c.rank * 8 + 4, c.epoch);
}

}  // namespace axb

using namespace axb;

static int fill_p2p(P2pCtx& c, const AxbP2pCtx* h, int device) {
  if (!h || h->n < 1 || h->n > 8) { set_error("p2p: group size must be 1..8"); return -1; }
  c.n = h->n; c.rank = h->rank; c.epoch = h->epoch;
  for (int j = 0; j < 8; ++j) { c.arena_peer[j] = h->base_peer[j]; c.mail_peer[j] = h->mail_peer[j]; c.done_peer[j] = h->done_peer[j]; }
  c.mail_local = h->mail_local; c.done_local = h->done_local; c.counter = h->counter; c.out_off = h->out_off;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("p2p: no status word"); return -1; }
  c.status = st;
  c.timeout_ns = wait_timeout_ns();
  return 0;
}

extern "C" int axb_a2a_rows(const AxbP2pCtx* ctx, const AxbRowBlock* blocks, int device, void* stream) {
  P2pCtx c;
  if (fill_p2p(c, ctx, device)) return -1;
  RowBlocks rb;
  long long rows_total = 0;
  for (int j = 0; j < 8; ++j) {
    RowBlock& b = rb.b[j];
    if (j < c.n) {
      b.src = static_cast<const uint8_t*>(blocks[j].src); b.src_pitch = blocks[j].src_pitch; b.dst_off = blocks[j].dst_off;
      b.dst_pitch = blocks[j].dst_pitch; b.rows = blocks[j].rows; b.row_bytes = blocks[j].row_bytes;
      if (b.rows > 0 && ((b.row_bytes | b.src_pitch | b.dst_pitch | b.dst_off) & 15 ||
                         (reinterpret_cast<uintptr_t>(b.src) & 15))) {
        set_error("axb_a2a_rows: rows, pitches and offsets must be multiples of 16 bytes");
        return -1;
      }
      rows_total += b.rows * ((b.row_bytes + 2047) / 2048);   // 2 KB work units
    } else {
      b = RowBlock{nullptr, 0, 0, 0, 0, 0};
    }
  }
  long long blocks_needed = (rows_total + 7) / 8;
  const long long cap = static_cast<long long>(sm_count(device)) * 4;
  const int grid = static_cast<int>(blocks_needed < 1 ? 1 : (blocks_needed > cap ? cap : blocks_needed));
  a2a_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(rb, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// Publish: after the stream's earlier work (the copy of my table shard into my peer-mapped buffer, or the
// zero fill of my gradient shard), raise epoch in every peer's mailbox.
extern "C" int axb_p2p_publish(const AxbP2pCtx* ctx, int device, void* stream) {
  P2pCtx c;
  if (fill_p2p(c, ctx, device)) return -1;
  p2p_publish_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_embedding_fetch(const long long* ids, long long n_tokens, void* out, long long row_bytes,
                                   long long rows_per_shard, const AxbP2pCtx* ctx, int device, void* stream) {
  P2pCtx c;
  if (fill_p2p(c, ctx, device)) return -1;
  if (row_bytes % 16 || rows_per_shard <= 0) { set_error("axb_embedding_fetch: rows must be multiples of 16 bytes"); return -1; }
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  const long long need = (n_tokens + 7) / 8;
  const int grid = static_cast<int>(need < 1 ? 1 : (need > cap ? cap : need));
  embedding_fetch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(ids, n_tokens, static_cast<uint8_t*>(out),
                                                                              row_bytes, rows_per_shard, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_embedding_scatter_add(const long long* ids, long long n_tokens, const void* dy, int H,
                                         long long rows_per_shard, const AxbP2pCtx* ctx, int device, void* stream) {
  P2pCtx c;
  if (fill_p2p(c, ctx, device)) return -1;
  if (H % 2 || rows_per_shard <= 0) { set_error("axb_embedding_scatter_add: hidden must be even"); return -1; }
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  const long long need = (n_tokens + 7) / 8;
  const int grid = static_cast<int>(need < 1 ? 1 : (need > cap ? cap : need));
  embedding_scatter_add_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, n_tokens, static_cast<const __nv_bfloat16*>(dy), H, rows_per_shard, c);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
