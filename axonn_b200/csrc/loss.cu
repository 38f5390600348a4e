// Softmax cross-entropy over (possibly vocabulary-sharded) logits.
//
// forward statistics, one block per row:  m = max_j z_j, s = sum_j exp(z_j - m),
// t = z_target when the target lies in this shard (else 0).  The caller turns
// (m, s, t) — all-reduced over the vocabulary shards when there are several —
// into lse = m + log s and loss = lse - t.
// backward, in place: z_j <- (exp(z_j - lse) - [j == target]) * scale.
#include "common.cuh"

namespace axb {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  v = l < nw ? red[l] : -INFINITY;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  v = l < nw ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void ld8bf(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}

// stats: [rows, 3] = (max, sumexp, target logit)
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
              float* __restrict__ stats, int rows, int V, int vocab_start) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* z = logits + (size_t)row * V;
    const int nchunk = V / 8;
    float m = -INFINITY;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
      float f[8]; ld8bf(z + c * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, f[i]);
    }
    m = block_max(m, red);
    float s = 0.f;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
      float f[8]; ld8bf(z + c * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) {
      const long long t = targets[row] - vocab_start;
      stats[3 * row] = m;
      stats[3 * row + 1] = s;
      stats[3 * row + 2] = (t >= 0 && t < V) ? __bfloat162float(z[t]) : 0.f;
    }
  }
}

// In place: logits <- dlogits.  scale_ptr: device scalar (upstream gradient x 1/num_tokens).
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
              const float* __restrict__ lse, const float* __restrict__ scale_ptr, int rows, int V, int vocab_start,
              long long ignore_index) {
  const float scale = *scale_ptr;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* z = logits + (size_t)row * V;
    const long long tgt = targets[row];
    const long long t = tgt - vocab_start;
    const float l = lse[row];
    const float rs = (tgt == ignore_index) ? 0.f : scale;
    const int nchunk = V / 8;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
      float f[8]; ld8bf(z + c * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float p = __expf(f[i] - l);
        if (c * 8 + i == t) p -= 1.f;
        f[i] = p * rs;
      }
      uint4 u;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
      for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      *reinterpret_cast<uint4*>(z + c * 8) = u;
    }
  }
}

}  // namespace axb

using namespace axb;

extern "C" int axb_ce_fwd(const void* logits, const long long* targets, float* stats, int rows, int V, int vocab_start,
                          void* stream) {
  if (V % 8) { set_error("cross entropy: vocab shard %d must be a multiple of 8", V); return -1; }
  const int cap = sm_count_current() * 8;
  const int grid = rows < cap ? rows : cap;
  ce_fwd_kernel<<<grid, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, targets, stats, rows, V,
                                                             vocab_start);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_ce_bwd(void* logits, const long long* targets, const float* lse, const float* scale, int rows, int V,
                          int vocab_start, long long ignore_index, void* stream) {
  if (V % 8) { set_error("cross entropy: vocab shard %d must be a multiple of 8", V); return -1; }
  const int cap = sm_count_current() * 8;
  const int grid = rows < cap ? rows : cap;
  ce_bwd_kernel<<<grid, CE_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, targets, lse, scale, rows, V,
                                                             vocab_start, ignore_index);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
