// LayerNorm / RMSNorm forward and backward for sm_100a.
//
// Rows are processed by persistent blocks (grid = a small multiple of the SM
// count); every thread owns fixed 8-element column chunks, so the backward
// kernel can accumulate its dgamma/dbeta partial sums in registers across all
// the rows the block visits and write one partial row per block; a second tiny
// kernel folds the partials.  All loads/stores are 16-byte vectors.
//
// Three modes serve tensor-parallel hidden dimensions (the row statistics are
// then sums over shards that the caller all-reduces between the two calls):
//   mode 0  statistics computed locally and applied in one kernel
//   mode 1  only emit per-row partial sums
//   mode 2  apply with externally supplied (already reduced) statistics
#include <cstdlib>

#include "common.cuh"

namespace axb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_CHUNKS = 8;  // hidden <= 256 * 8 * 8 = 16384

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<__half> {
  static __device__ __forceinline__ void load(const __half* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  }
  static __device__ __forceinline__ void store(__half* p, const float (&f)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

// f = T(f + d): the residual sum, rounded to the storage type exactly like a separate elementwise add would.
template <typename T> __device__ __forceinline__ float round_as(float v);
template <> __device__ __forceinline__ float round_as<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
template <> __device__ __forceinline__ float round_as<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_as<float>(float v) { return v; }
template <typename T>
__device__ __forceinline__ void add_rounded(float (&f)[8], const T* delta) {
  float d[8];
  Vec8<T>::load(delta, d);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = round_as<T>(f[i] + d[i]);
}

// Sum two values over the block; result broadcast to all threads.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red /* [2*32] */) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (l == 0) { red[w] = a; red[32 + w] = b; }
  __syncthreads();
  a = l < nw ? red[l] : 0.f; b = l < nw ? red[32 + l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
}

// stats layout: [rows, 2]: LayerNorm -> (sum x, sum x^2) in mode 1, (mean, rstd) otherwise;
// RMSNorm -> (unused, sum x^2) in mode 1, (0, rstd) otherwise.
template <typename T, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                T* __restrict__ y, float* __restrict__ stats, int rows, int H, int H_total, float eps, int mode,
                const T* __restrict__ delta, T* __restrict__ hout) {
  // delta != null (modes 0 and 1): the row that is normalised is h = x + delta, which is also written to hout
  // (the residual stream after the add); every thread re-reads only the chunks of hout that it wrote itself.
  __shared__ float red[64];
  const int nchunk = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * H;
    float mean = 0.f, rstd = 0.f;
    if (mode != 2 && mode != 3) {
      float s1 = 0.f, s2 = 0.f;
      for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
        float f[8]; Vec8<T>::load(xr + c * 8, f);
        if (delta) {
          add_rounded<T>(f, delta + static_cast<size_t>(row) * H + c * 8);
          Vec8<T>::store(hout + static_cast<size_t>(row) * H + c * 8, f);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { s1 += f[i]; s2 += f[i] * f[i]; }
      }
      block_sum2(s1, s2, red);
      if (mode == 1) {
        if (threadIdx.x == 0) { stats[2 * row] = s1; stats[2 * row + 1] = s2; }
        continue;
      }
      if (RMS) { mean = 0.f; rstd = rsqrtf(s2 / H_total + eps); }
      else { mean = s1 / H_total; rstd = rsqrtf(fmaxf(s2 / H_total - mean * mean, 0.f) + eps); }
      if (threadIdx.x == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
    } else if (mode == 3) {
      // stats hold (sum x, sum x^2) over the full hidden dimension (the partial sums of mode 1 after their
      // all-reduce): finish them here instead of in separate element-wise launches, keep (mean, rstd) for backward
      const float s1 = stats[2 * row], s2 = stats[2 * row + 1];
      if (RMS) { mean = 0.f; rstd = rsqrtf(s2 / H_total + eps); }
      else { mean = s1 / H_total; rstd = rsqrtf(fmaxf(s2 / H_total - mean * mean, 0.f) + eps); }
      __syncthreads();                               // every thread has read the sums
      if (threadIdx.x == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
    } else {
      mean = stats[2 * row]; rstd = stats[2 * row + 1];
    }
    if (delta && mode != 3) xr = hout + static_cast<size_t>(row) * H;
    T* yr = y + static_cast<size_t>(row) * H;
    for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
      float f[8], g[8], b[8];
      Vec8<T>::load(xr + c * 8, f);
      Vec8<T>::load(gamma + c * 8, g);
      if (!RMS && beta) Vec8<T>::load(beta + c * 8, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = (f[i] - mean) * rstd * g[i];
        if (!RMS && beta) v += b[i];
        f[i] = v;
      }
      Vec8<T>::store(yr + c * 8, f);
    }
  }
}

// Backward.  sums layout [rows, 2] = (sum g*dy, sum g*dy*xhat) over the full hidden dimension.
template <typename T, bool RMS, int CH>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                const float* __restrict__ stats, T* __restrict__ dx, float* __restrict__ sums,
                float* __restrict__ dgamma_part, float* __restrict__ dbeta_part, int rows, int H, int H_total,
                int mode, const T* __restrict__ dres) {
  // dres != null: gradient that reaches the normalised row through the residual path; it is added to dx
  __shared__ float red[64];
  const int nchunk = H / 8;
  float ag[CH][8], ab[CH][8];
#pragma unroll
  for (int k = 0; k < CH; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) { ag[k][i] = 0.f; ab[k][i] = 0.f; }

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* xr = x + static_cast<size_t>(row) * H;
    const T* dyr = dy + static_cast<size_t>(row) * H;
    const float mean = stats[2 * row], rstd = stats[2 * row + 1];
    float s1 = 0.f, s2 = 0.f;
    if (mode != 2) {
      for (int c = threadIdx.x; c < nchunk; c += blockDim.x) {
        float f[8], d[8], g[8];
        Vec8<T>::load(xr + c * 8, f); Vec8<T>::load(dyr + c * 8, d); Vec8<T>::load(gamma + c * 8, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float xh = (f[i] - mean) * rstd, gd = g[i] * d[i];
          s1 += gd; s2 += gd * xh;
        }
      }
      block_sum2(s1, s2, red);
      if (mode == 1) {
        if (threadIdx.x == 0) { sums[2 * row] = s1; sums[2 * row + 1] = s2; }
        continue;
      }
    } else {
      s1 = sums[2 * row]; s2 = sums[2 * row + 1];
    }
    const float m1 = RMS ? 0.f : s1 / H_total, m2 = s2 / H_total;
    T* dxr = dx + static_cast<size_t>(row) * H;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        float f[8], d[8], g[8], o[8];
        Vec8<T>::load(xr + c * 8, f); Vec8<T>::load(dyr + c * 8, d); Vec8<T>::load(gamma + c * 8, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float xh = (f[i] - mean) * rstd;
          o[i] = rstd * (g[i] * d[i] - m1 - xh * m2);
          ag[k][i] += d[i] * xh; ab[k][i] += d[i];
        }
        if (dres) {
          float r8[8];
          Vec8<T>::load(dres + static_cast<size_t>(row) * H + c * 8, r8);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r8[i];
        }
        Vec8<T>::store(dxr + c * 8, o);
      }
    }
  }
  if (mode != 1 && dgamma_part) {
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      if (c >= nchunk) continue;
      float* pg = dgamma_part + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) pg[i] = ag[k][i];
      if (!RMS && dbeta_part) {
        float* pb = dbeta_part + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) pb[i] = ab[k][i];
      }
    }
  }
}

// ---- mode-0 fast path (statistics local, hidden <= 256 * 8 * CH): a block handles R rows per iteration with one
// 8-element chunk per thread and CH, keeps the rows in registers between the statistics and the apply step
// (one global read per element) and needs a single block barrier per iteration: the loads of R rows are in
// flight together and the cross-warp sums of all R rows share the barrier.
template <int NV>
__device__ __forceinline__ void block_sum_n(float (&v)[NV], float* red /* [2][NV][8] */, int it) {
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[k] += __shfl_xor_sync(0xffffffffu, v[k], o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  float* buf = red + (it & 1) * NV * 8;     // double-buffered by iteration: one barrier per iteration
  if (l == 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) buf[k * 8 + w] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += buf[k * 8 + i];
    v[k] = t;
  }
}

template <typename T, bool RMS, int CH, int R>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_rows_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                     T* __restrict__ y, float* __restrict__ stats, int rows, int H, float eps,
                     const T* __restrict__ delta, T* __restrict__ hout) {
  __shared__ float red[2 * 2 * R * 8];
  const int nchunk = H / 8;
  float g[CH][8], b[CH][8];
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { g[k][i] = 0.f; b[k][i] = 0.f; }
    if (c < nchunk) {
      Vec8<T>::load(gamma + c * 8, g[k]);
      if (!RMS && beta) Vec8<T>::load(beta + c * 8, b[k]);
    }
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, ++it) {
    float f[R][CH][8];
    float sm[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      sm[2 * r] = 0.f; sm[2 * r + 1] = 0.f;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (row0 + r < rows && c < nchunk) {
          Vec8<T>::load(x + static_cast<size_t>(row0 + r) * H + c * 8, f[r][k]);
          if (delta) {
            add_rounded<T>(f[r][k], delta + static_cast<size_t>(row0 + r) * H + c * 8);
            Vec8<T>::store(hout + static_cast<size_t>(row0 + r) * H + c * 8, f[r][k]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) f[r][k][i] = 0.f;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int k = 0; k < CH; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) { sm[2 * r] += f[r][k][i]; sm[2 * r + 1] += f[r][k][i] * f[r][k][i]; }
    block_sum_n<2 * R>(sm, red, it);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) break;
      float mean, rstd;
      if (RMS) { mean = 0.f; rstd = rsqrtf(sm[2 * r + 1] / H + eps); }
      else { mean = sm[2 * r] / H; rstd = rsqrtf(fmaxf(sm[2 * r + 1] / H - mean * mean, 0.f) + eps); }
      if (threadIdx.x == 0) { stats[2 * (row0 + r)] = mean; stats[2 * (row0 + r) + 1] = rstd; }
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c >= nchunk) continue;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = (f[r][k][i] - mean) * rstd * g[k][i] + b[k][i];
        Vec8<T>::store(y + static_cast<size_t>(row0 + r) * H + c * 8, o);
      }
    }
  }
}

// Forward with one warp per row (hidden = 256 * VPL elements, the whole row in registers): the statistics need only
// warp shuffles, so there is no block barrier between the load and the store phase and the eight warps of a block
// run their rows independently - their loads stay in flight continuously.  gamma / beta are re-read per row (they
// stay in L1).
template <typename T, bool RMS, int VPL>
__global__ void __launch_bounds__(256)
norm_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                     T* __restrict__ y, float* __restrict__ stats, int rows, int H, float eps,
                     const T* __restrict__ delta, T* __restrict__ hout) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = static_cast<long long>(gridDim.x) * 8;
  for (long long row = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5); row < rows; row += nwarps) {
    const size_t base = static_cast<size_t>(row) * H;
    float f[VPL][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = (lane + 32 * k) * 8;
      Vec8<T>::load(x + base + c, f[k]);
      if (delta) {
        add_rounded<T>(f[k], delta + base + c);
        Vec8<T>::store(hout + base + c, f[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < VPL; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) { s1 += f[k][i]; s2 += f[k][i] * f[k][i]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    float mean, rstd;
    if (RMS) { mean = 0.f; rstd = rsqrtf(s2 / H + eps); }
    else { mean = s1 / H; rstd = rsqrtf(fmaxf(s2 / H - mean * mean, 0.f) + eps); }
    if (lane == 0) { stats[2 * row] = mean; stats[2 * row + 1] = rstd; }
#pragma unroll
    for (int k = 0; k < VPL; ++k) {
      const int c = (lane + 32 * k) * 8;
      float g[8], b[8], o[8];
      Vec8<T>::load(gamma + c, g);
      if (!RMS && beta) Vec8<T>::load(beta + c, b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = (f[k][i] - mean) * rstd * g[i];
        if (!RMS && beta) v += b[i];
        o[i] = v;
      }
      Vec8<T>::store(y + base + c, o);
    }
  }
}

template <typename T, bool RMS, int CH, int R>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_rows_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ gamma,
                     const float* __restrict__ stats, T* __restrict__ dx, float* __restrict__ dgamma_part,
                     float* __restrict__ dbeta_part, int rows, int H, const T* __restrict__ dres) {
  __shared__ float red[2 * 2 * R * 8];
  const int nchunk = H / 8;
  float g[CH][8], ag[CH][8], ab[CH][8];
#pragma unroll
  for (int k = 0; k < CH; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { g[k][i] = 0.f; ag[k][i] = 0.f; ab[k][i] = 0.f; }
    if (c < nchunk) Vec8<T>::load(gamma + c * 8, g[k]);
  }
  int it = 0;
  for (int row0 = blockIdx.x * R; row0 < rows; row0 += gridDim.x * R, ++it) {
    float xh[R][CH][8], d[R][CH][8];
    float rstd[R];
    float sm[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const bool live = row0 + r < rows;
      const float mean = live ? stats[2 * (row0 + r)] : 0.f;
      rstd[r] = live ? stats[2 * (row0 + r) + 1] : 0.f;
      sm[2 * r] = 0.f; sm[2 * r + 1] = 0.f;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (live && c < nchunk) {
          Vec8<T>::load(x + static_cast<size_t>(row0 + r) * H + c * 8, xh[r][k]);
          Vec8<T>::load(dy + static_cast<size_t>(row0 + r) * H + c * 8, d[r][k]);
#pragma unroll
          for (int i = 0; i < 8; ++i) xh[r][k][i] = (xh[r][k][i] - mean) * rstd[r];
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) { xh[r][k][i] = 0.f; d[r][k][i] = 0.f; }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int k = 0; k < CH; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float gd = g[k][i] * d[r][k][i];
          sm[2 * r] += gd; sm[2 * r + 1] += gd * xh[r][k][i];
          ag[k][i] += d[r][k][i] * xh[r][k][i]; ab[k][i] += d[r][k][i];
        }
    block_sum_n<2 * R>(sm, red, it);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (row0 + r >= rows) break;
      const float m1 = RMS ? 0.f : sm[2 * r] / H, m2 = sm[2 * r + 1] / H;
#pragma unroll
      for (int k = 0; k < CH; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c >= nchunk) continue;
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd[r] * (g[k][i] * d[r][k][i] - m1 - xh[r][k][i] * m2);
        if (dres) {
          float r8[8];
          Vec8<T>::load(dres + static_cast<size_t>(row0 + r) * H + c * 8, r8);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r8[i];
        }
        Vec8<T>::store(dx + static_cast<size_t>(row0 + r) * H + c * 8, o);
      }
    }
  }
  if (dgamma_part) {
#pragma unroll
    for (int k = 0; k < CH; ++k) {
      const int c = threadIdx.x + k * blockDim.x;
      if (c >= nchunk) continue;
      float4* pg = reinterpret_cast<float4*>(dgamma_part + static_cast<size_t>(blockIdx.x) * H + c * 8);
      pg[0] = make_float4(ag[k][0], ag[k][1], ag[k][2], ag[k][3]);
      pg[1] = make_float4(ag[k][4], ag[k][5], ag[k][6], ag[k][7]);
      if (!RMS && dbeta_part) {
        float4* pb = reinterpret_cast<float4*>(dbeta_part + static_cast<size_t>(blockIdx.x) * H + c * 8);
        pb[0] = make_float4(ab[k][0], ab[k][1], ab[k][2], ab[k][3]);
        pb[1] = make_float4(ab[k][4], ab[k][5], ab[k][6], ab[k][7]);
      }
    }
  }
}

// out[c] = sum_b part[b, c]   (optionally two tables at once).  Block = 32 columns x 32 row-groups; every
// thread keeps four independent loads in flight.
// Results are written in `out_dtype` (0 bf16, 1 fp16, 2 fp32) - the dtype of the parameter whose gradient this is -
// so that no separate cast kernel follows.
__device__ __forceinline__ void fold_store(void* o, int out_dtype, int c, float v) {
  if (out_dtype == 2) reinterpret_cast<float*>(o)[c] = v;
  else if (out_dtype == 0) reinterpret_cast<__nv_bfloat16*>(o)[c] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(o)[c] = __float2half_rn(v);
}
__global__ void fold_partials_kernel(const float* __restrict__ pa, const float* __restrict__ pb, void* __restrict__ oa,
                                     void* __restrict__ ob, int nblocks, int H, int out_dtype) {
  __shared__ float sa[32][33], sb[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float a[4] = {0.f, 0.f, 0.f, 0.f}, b[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < H) {
    for (int r = threadIdx.y; r < nblocks; r += 128) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + 32 * u;
        if (rr < nblocks) {
          a[u] += pa[static_cast<size_t>(rr) * H + c];
          if (pb) b[u] += pb[static_cast<size_t>(rr) * H + c];
        }
      }
    }
  }
  sa[threadIdx.y][threadIdx.x] = (a[0] + a[1]) + (a[2] + a[3]);
  sb[threadIdx.y][threadIdx.x] = (b[0] + b[1]) + (b[2] + b[3]);
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float ta = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) { ta += sa[k][threadIdx.x]; tb += sb[k][threadIdx.x]; }
    fold_store(oa, out_dtype, c, ta);
    if (pb) fold_store(ob, out_dtype, c, tb);
  }
}

// Column sums of a row-major [rows, N] matrix (bias gradients): block = 32 column vectors (8 columns each)
// x 8 row groups, grid = (column blocks, row splits); every thread keeps four 16-byte loads in flight and one
// partial row per row split is written for fold_partials_kernel.
template <typename T>
__global__ void __launch_bounds__(256)
colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ part, int rows, int N) {
  __shared__ float red[8][32][9];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < N) {
    const int stride = gridDim.y * 8;
    for (int r = blockIdx.y * 8 + w; r < rows; r += 4 * stride) {
      float f[4][8];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int rr = r + u * stride;
        if (rr < rows) Vec8<T>::load(x + static_cast<size_t>(rr) * N + c, f[u]);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) f[u][i] = 0.f;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[u][i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[w][lane][i] = acc[i];
  __syncthreads();
  // thread (w, lane) folds column i = w of lane's vector over the 8 row groups
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane][w];
    part[static_cast<size_t>(blockIdx.y) * N + c + w] = t;
  }
}

// dx = dy * gelu'(x) together with the column sums of dx (the bias gradient of the layer that produced x):
// same thread layout as colsum_partial_kernel, one extra load and one store per element.
template <typename T>
__global__ void __launch_bounds__(256, 6)
gelu_bwd_colsum_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                       float* __restrict__ part, int rows, int N) {
  __shared__ float red[8][32][9];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + lane) * 8;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < N) {
    // one row per iteration and few registers: the arithmetic of one warp hides behind the loads of the many
    // other resident warps (48 per SM) instead of behind a deep per-thread batch
    const int stride = gridDim.y * 8;
    for (int r = blockIdx.y * 8 + w; r < rows; r += stride) {
      float fx[8], fd[8], o[8];
      Vec8<T>::load(x + static_cast<size_t>(r) * N + c, fx);
      Vec8<T>::load(dy + static_cast<size_t>(r) * N + c, fd);
#pragma unroll
      for (int i = 0; i < 8; ++i) { o[i] = fd[i] * gelu_tanh_grad(fx[i]); acc[i] += o[i]; }
      Vec8<T>::store(dx + static_cast<size_t>(r) * N + c, o);
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[w][lane][i] = acc[i];
  __syncthreads();
  if (c < N) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += red[k][lane][w];
    part[static_cast<size_t>(blockIdx.y) * N + c + w] = t;
  }
}

int sm_count(int device);

// The warp-per-row forward serves hidden sizes 1024 / 2048 / 4096; AXONN_NORM_WARP=0 keeps the block-per-rows kernel
// for them too (read once).
static bool norm_warp_rows_enabled() {
  static const bool on = [] {
    const char* e = getenv("AXONN_NORM_WARP");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename T>
static int norm_fwd_t(const void* x, const void* gamma, const void* beta, void* y, float* stats, int rows, int H,
                      int H_total, float eps, int rms, int mode, int grid, cudaStream_t s, const void* delta, void* hout) {
  const int threads = (H / 8 <= 128) ? 128 : NORM_THREADS;  // no idle threads for narrow (sharded) rows
  if (mode == 0 && H == H_total && norm_warp_rows_enabled() && (H == 1024 || H == 2048 || H == 4096)) {
    const int wgrid = min((rows + 7) / 8, grid * 2);
#define AXB_NORM_FWD_WARP(RMS_, VPL_)                                                                           \
  norm_fwd_warp_kernel<T, RMS_, VPL_><<<wgrid, 256, 0, s>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y, \
                                                           stats, rows, H, eps, (const T*)delta, (T*)hout)
    if (rms) { if (H == 1024) AXB_NORM_FWD_WARP(true, 4); else if (H == 2048) AXB_NORM_FWD_WARP(true, 8); else AXB_NORM_FWD_WARP(true, 16); }
    else { if (H == 1024) AXB_NORM_FWD_WARP(false, 4); else if (H == 2048) AXB_NORM_FWD_WARP(false, 8); else AXB_NORM_FWD_WARP(false, 16); }
#undef AXB_NORM_FWD_WARP
    AXB_CUDA(cudaGetLastError());
    return 0;
  }
  if (mode == 0 && H == H_total && H / 8 <= 2 * NORM_THREADS && H / 8 > 128) {
    const int ch = (H / 8 + NORM_THREADS - 1) / NORM_THREADS;
#define AXB_NORM_FWD_ROWS(RMS_, CH_, R_)                                                                         \
  norm_fwd_rows_kernel<T, RMS_, CH_, R_><<<min(grid, (rows + R_ - 1) / R_), NORM_THREADS, 0, s>>>(              \
      (const T*)x, (const T*)gamma, (const T*)beta, (T*)y, stats, rows, H, eps, (const T*)delta, (T*)hout)
    if (rms) { if (ch == 1) AXB_NORM_FWD_ROWS(true, 1, 4); else AXB_NORM_FWD_ROWS(true, 2, 2); }
    else { if (ch == 1) AXB_NORM_FWD_ROWS(false, 1, 4); else AXB_NORM_FWD_ROWS(false, 2, 2); }
#undef AXB_NORM_FWD_ROWS
    AXB_CUDA(cudaGetLastError());
    return 0;
  }
  if (rms)
    norm_fwd_kernel<T, true><<<grid, threads, 0, s>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y,
                                                     stats, rows, H, H_total, eps, mode, (const T*)delta, (T*)hout);
  else
    norm_fwd_kernel<T, false><<<grid, threads, 0, s>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)y,
                                                      stats, rows, H, H_total, eps, mode, (const T*)delta, (T*)hout);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

template <typename T>
static int norm_bwd_t(const void* dy, const void* x, const void* gamma, const float* stats, void* dx, float* sums,
                      float* dgp, float* dbp, int rows, int H, int H_total, int rms, int mode, int grid,
                      cudaStream_t s, int* blocks_launched, const void* dres) {
  *blocks_launched = grid;
  const int nchunk = H / 8;
  const int threads = (nchunk <= 128) ? 128 : NORM_THREADS;
  const int ch = (nchunk + threads - 1) / threads;
  if (mode == 0 && H == H_total && nchunk <= 2 * NORM_THREADS && nchunk > 128) {
#define AXB_NORM_BWD_ROWS(RMS_, CH_, R_)                                                                       \
  *blocks_launched = min(grid, (rows + R_ - 1) / R_);                                                          \
  norm_bwd_rows_kernel<T, RMS_, CH_, R_><<<*blocks_launched, NORM_THREADS, 0, s>>>(                            \
      (const T*)dy, (const T*)x, (const T*)gamma, stats, (T*)dx, dgp, dbp, rows, H, (const T*)dres)
    if (rms) { if (ch == 1) { AXB_NORM_BWD_ROWS(true, 1, 2); } else { AXB_NORM_BWD_ROWS(true, 2, 1); } }
    else { if (ch == 1) { AXB_NORM_BWD_ROWS(false, 1, 2); } else { AXB_NORM_BWD_ROWS(false, 2, 1); } }
#undef AXB_NORM_BWD_ROWS
    AXB_CUDA(cudaGetLastError());
    return 0;
  }
#define AXB_NORM_BWD(RMS_, CH_)                                                                              \
  norm_bwd_kernel<T, RMS_, CH_><<<grid, threads, 0, s>>>((const T*)dy, (const T*)x, (const T*)gamma, stats, \
                                                              (T*)dx, sums, dgp, dbp, rows, H, H_total, mode, (const T*)dres)
  if (rms) {
    if (ch <= 1) AXB_NORM_BWD(true, 1); else if (ch <= 2) AXB_NORM_BWD(true, 2);
    else if (ch <= 4) AXB_NORM_BWD(true, 4); else AXB_NORM_BWD(true, 8);
  } else {
    if (ch <= 1) AXB_NORM_BWD(false, 1); else if (ch <= 2) AXB_NORM_BWD(false, 2);
    else if (ch <= 4) AXB_NORM_BWD(false, 4); else AXB_NORM_BWD(false, 8);
  }
#undef AXB_NORM_BWD
  AXB_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace axb

extern "C" int axb_norm_grid(int device, int rows) {
  int g = 8 * axb::sm_count(device);
  return rows < g ? rows : g;
}

// y = norm(x + delta) and hout = x + delta when delta is non-null (the residual add fused into the norm; not in
// mode 2, which applies given statistics to a row that has already been summed); y = norm(x) otherwise.
extern "C" int axb_add_norm_fwd(const void* x, const void* delta, void* hout, const void* gamma, const void* beta,
                                void* y, float* stats, int rows, int H, int H_total, float eps, int rms, int mode,
                                int dtype, int device, void* stream) {
  using namespace axb;
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAX_CHUNKS) { set_error("norm: hidden %d unsupported", H); return -1; }
  if (delta && (mode == 2 || !hout)) { set_error("norm: the fused residual add needs an output for x + delta and mode 0 or 1"); return -1; }
  if (rows <= 0) return 0;
  const int grid = axb_norm_grid(device, rows);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) return norm_fwd_t<__nv_bfloat16>(x, gamma, beta, y, stats, rows, H, H_total, eps, rms, mode, grid, s, delta, hout);
  if (dtype == 1) return norm_fwd_t<__half>(x, gamma, beta, y, stats, rows, H, H_total, eps, rms, mode, grid, s, delta, hout);
  return norm_fwd_t<float>(x, gamma, beta, y, stats, rows, H, H_total, eps, rms, mode, grid, s, delta, hout);
}

extern "C" int axb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* stats, int rows, int H,
                            int H_total, float eps, int rms, int mode, int dtype, int device, void* stream) {
  return axb_add_norm_fwd(x, nullptr, nullptr, gamma, beta, y, stats, rows, H, H_total, eps, rms, mode, dtype, device, stream);
}

// dgamma_part / dbeta_part: [grid, H] fp32 scratch (grid from axb_norm_grid); dgamma/dbeta: [H] fp32 outputs.
extern "C" int axb_add_norm_bwd(const void* dy, const void* dres, const void* x, const void* gamma, const float* stats,
                                void* dx, float* sums, float* dgamma_part, float* dbeta_part, void* dgamma, void* dbeta,
                                int rows, int H, int H_total, int rms, int mode, int dtype, int param_dtype, int device,
                                void* stream);
extern "C" int axb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* stats, void* dx,
                            float* sums, float* dgamma_part, float* dbeta_part, void* dgamma, void* dbeta, int rows,
                            int H, int H_total, int rms, int mode, int dtype, int param_dtype, int device, void* stream) {
  return axb_add_norm_bwd(dy, nullptr, x, gamma, stats, dx, sums, dgamma_part, dbeta_part, dgamma, dbeta, rows, H, H_total,
                          rms, mode, dtype, param_dtype, device, stream);
}

// dx = norm_backward(dy) + dres (dres, optional: the gradient arriving through the residual path of a fused add + norm)
extern "C" int axb_add_norm_bwd(const void* dy, const void* dres, const void* x, const void* gamma, const float* stats,
                                void* dx, float* sums, float* dgamma_part, float* dbeta_part, void* dgamma, void* dbeta,
                                int rows, int H, int H_total, int rms, int mode, int dtype, int param_dtype, int device,
                                void* stream) {
  using namespace axb;
  if (H % 8 || H > NORM_THREADS * 8 * NORM_MAX_CHUNKS) { set_error("norm: hidden %d unsupported", H); return -1; }
  if (rows <= 0) return 0;
  const int grid = axb_norm_grid(device, rows);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc, nblocks = grid;
  if (dtype == 0) rc = norm_bwd_t<__nv_bfloat16>(dy, x, gamma, stats, dx, sums, dgamma_part, dbeta_part, rows, H, H_total, rms, mode, grid, s, &nblocks, dres);
  else if (dtype == 1) rc = norm_bwd_t<__half>(dy, x, gamma, stats, dx, sums, dgamma_part, dbeta_part, rows, H, H_total, rms, mode, grid, s, &nblocks, dres);
  else rc = norm_bwd_t<float>(dy, x, gamma, stats, dx, sums, dgamma_part, dbeta_part, rows, H, H_total, rms, mode, grid, s, &nblocks, dres);
  if (rc) return rc;
  if (mode != 1 && dgamma_part && dgamma) {
    fold_partials_kernel<<<(H + 31) / 32, dim3(32, 32), 0, s>>>(dgamma_part, rms ? nullptr : dbeta_part, dgamma,
                                                              rms ? nullptr : dbeta, nblocks, H, param_dtype);
    AXB_CUDA(cudaGetLastError());
  }
  return 0;
}

extern "C" int axb_colsum_splits(int device, int rows, int N) {
  const int col_blocks = (N / 8 + 31) / 32;
  int splits = (8 * axb::sm_count(device) + col_blocks - 1) / col_blocks;
  const int max_splits = (rows + 31) / 32;       // at least four rows per thread
  if (splits > max_splits) splits = max_splits;
  return splits < 1 ? 1 : splits;
}

// out[c] = sum_r x[r, c]; part: [axb_colsum_splits, N] fp32 scratch, out: [N] fp32.  N must be a multiple of 8.
extern "C" int axb_colsum(const void* x, float* part, void* out, int rows, int N, int dtype, int out_dtype, int device,
                          void* stream) {
  using namespace axb;
  if (N % 8 || rows <= 0) { set_error("colsum: N must be a multiple of 8 and rows positive"); return -1; }
  const int splits = axb_colsum_splits(device, rows, N);
  dim3 grid((N / 8 + 31) / 32, splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) colsum_partial_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, part, rows, N);
  else if (dtype == 1) colsum_partial_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, part, rows, N);
  else colsum_partial_kernel<float><<<grid, 256, 0, s>>>((const float*)x, part, rows, N);
  AXB_CUDA(cudaGetLastError());
  fold_partials_kernel<<<(N + 31) / 32, dim3(32, 32), 0, s>>>(part, nullptr, out, nullptr, splits, N, out_dtype);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// dx = dy * gelu'(x) (tanh form) and colsum[c] = sum_r dx[r, c] in one pass.  part: [axb_colsum_splits, N] fp32.
extern "C" int axb_gelu_bwd_colsum(const void* dy, const void* x, void* dx, float* part, void* colsum, int rows,
                                   int N, int dtype, int out_dtype, int device, void* stream) {
  using namespace axb;
  if (N % 8 || rows <= 0) { set_error("gelu_bwd_colsum: N must be a multiple of 8 and rows positive"); return -1; }
  if (dtype != 0 && dtype != 1) { set_error("gelu_bwd_colsum: bf16 or fp16 only"); return -1; }
  const int splits = axb_colsum_splits(device, rows, N);
  dim3 grid((N / 8 + 31) / 32, splits);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    gelu_bwd_colsum_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                              (__nv_bfloat16*)dx, part, rows, N);
  else
    gelu_bwd_colsum_kernel<__half><<<grid, 256, 0, s>>>((const __half*)dy, (const __half*)x, (__half*)dx, part, rows, N);
  AXB_CUDA(cudaGetLastError());
  fold_partials_kernel<<<(N + 31) / 32, dim3(32, 32), 0, s>>>(part, nullptr, colsum, nullptr, splits, N, out_dtype);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
