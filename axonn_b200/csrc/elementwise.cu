// Activation and rotary-embedding kernels (memory-bound, 16-byte vectors).
//   gelu (tanh form) forward / backward
//   swiglu: out = silu(gate) * up, forward / backward; gate and up are interleaved in
//           blocks of 8 columns of one [T, 2F] tensor: cols [16i, 16i+8) = gate, [16i+8, 16i+16) = up
//   rope: rotate (i, i + D/2) pairs of each head in place, forward or inverse
#include "common.cuh"

namespace axb {

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8]; ld8(x + i * 8, f);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = gelu_tanh(f[k]);
    st8(y + i * 8, f);
  }
}
// dx = dy * gelu'(x)
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                __nv_bfloat16* __restrict__ dx, size_t n8) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8], d[8]; ld8(x + i * 8, f); ld8(dy + i * 8, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) d[k] *= gelu_tanh_grad(f[k]);
    st8(dx + i * 8, d);
  }
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

// gu: [T, 2F] interleaved-8; out: [T, F]
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int T, int F) {
  const size_t per_row = F / 8, total = (size_t)T * per_row;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per_row, c = (i % per_row) * 8;
    float g[8], u[8];
    ld8(gu + r * 2 * F + 2 * c, g); ld8(gu + r * 2 * F + 2 * c + 8, u);
#pragma unroll
    for (int k = 0; k < 8; ++k) g[k] = g[k] * sigmoidf_(g[k]) * u[k];
    st8(out + r * F + c, g);
  }
}
// dgu: [T, 2F]
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ dgu, int T, int F) {
  const size_t per_row = F / 8, total = (size_t)T * per_row;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / per_row, c = (i % per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    ld8(gu + r * 2 * F + 2 * c, g); ld8(gu + r * 2 * F + 2 * c + 8, u); ld8(dout + r * F + c, d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = sigmoidf_(g[k]);
      const float silu = g[k] * s;
      du[k] = d[k] * silu;
      dg[k] = d[k] * u[k] * (s + silu * (1.f - s));
    }
    st8(dgu + r * 2 * F + 2 * c, dg); st8(dgu + r * 2 * F + 2 * c + 8, du);
  }
}

// x: [rows, nh, D] with rows = B * S * pos_div; position of a row = (row / pos_div) % S.
// cs: [S, D/2, 2] fp32 (cos, sin); sign = +1 forward, -1 inverse (backward).
// row_stride = elements between consecutive rows (allows q/k heads packed inside a wider qkv tensor).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, size_t rows, int S, int nh,
                            int D, int pos_div, size_t row_stride, float sign) {
  const int half = D / 2, per_head = half / 8;
  const size_t total = rows * nh * per_head;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_head) * 8;
    const size_t t = i / per_head;
    const int h = (int)(t % nh);
    const size_t bs = t / nh;
    const int s = (int)((bs / pos_div) % S);
    __nv_bfloat16* p = x + bs * row_stride + (size_t)h * D + c;
    float a[8], b[8];
    ld8(p, a); ld8(p + half, b);
    const float* t0 = cs + ((size_t)s * half + c) * 2;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float co = t0[2 * k], si = sign * t0[2 * k + 1];
      const float x0 = a[k], x1 = b[k];
      a[k] = x0 * co - x1 * si;
      b[k] = x1 * co + x0 * si;
    }
    st8(p, a); st8(p + half, b);
  }
}

static inline int ew_grid(size_t work, int threads) {
  size_t g = (work + threads - 1) / threads;
  const size_t cap = static_cast<size_t>(sm_count_current()) * 16;
  return (int)(g > cap ? cap : (g == 0 ? 1 : g));
}

}  // namespace axb

using namespace axb;

extern "C" int axb_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n % 8) { set_error("gelu: numel must be a multiple of 8"); return -1; }
  gelu_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n / 8);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream) {
  if (n % 8) { set_error("gelu: numel must be a multiple of 8"); return -1; }
  gelu_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                                      (__nv_bfloat16*)dx, n / 8);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_swiglu_fwd(const void* gu, void* out, int T, int F, void* stream) {
  if (F % 8) { set_error("swiglu: F must be a multiple of 8"); return -1; }
  swiglu_fwd_kernel<<<ew_grid((size_t)T * F / 8, 256), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu,
                                                                                    (__nv_bfloat16*)out, T, F);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_swiglu_bwd(const void* dout, const void* gu, void* dgu, int T, int F, void* stream) {
  if (F % 8) { set_error("swiglu: F must be a multiple of 8"); return -1; }
  swiglu_bwd_kernel<<<ew_grid((size_t)T * F / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, T, F);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_rope(void* x, const float* cs, long long rows, int S, int nh, int D, int pos_div,
                        long long row_stride, int inverse, void* stream) {
  if (D % 16) { set_error("rope: head_dim must be a multiple of 16"); return -1; }
  if (row_stride % 8) { set_error("rope: row stride must be a multiple of 8 elements"); return -1; }
  const size_t work = (size_t)rows * nh * (D / 16);
  rope_kernel<<<ew_grid(work, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, cs, (size_t)rows, S, nh, D, pos_div,
                                                                   (size_t)row_stride, inverse ? -1.f : 1.f);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
