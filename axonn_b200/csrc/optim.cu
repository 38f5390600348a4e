// Multi-tensor kernels: fused AdamW step, squared L2 norm, in-place scale.
//
// A launch covers a whole list of tensors through a device table; work is cut
// into fixed-size chunks and a grid-stride loop maps chunk -> (tensor, offset)
// by binary search in the table's chunk prefix sums, so one launch replaces
// hundreds of per-parameter launches.
#include <mutex>

#include "common.cuh"

namespace axb {

constexpr int MT_CHUNK = 1 << 16;
constexpr int MT_THREADS = 512;
constexpr int ADAM_UNROLL = 4;

// table row for norm/scale: {ptr, numel, dtype (0 fp32, 1 bf16, 2 fp16), chunk_prefix}
// table row for adamw:      {master fp32, model bf16 or 0, grad, exp_avg, exp_avg_sq, numel, grad dtype, chunk_prefix}
__device__ __forceinline__ int find_tensor(const long long* table, int width, int prefix_col, int n, long long chunk) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (table[(size_t)mid * width + prefix_col] <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float load_as_f32(const void* p, long long i, int dtype) {
  if (dtype == 0) return reinterpret_cast<const float*>(p)[i];
  if (dtype == 1) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, long long i, int dtype, float v) {
  if (dtype == 0) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == 1) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

__global__ void __launch_bounds__(MT_THREADS)
multi_l2norm_sq_kernel(const long long* __restrict__ table, int n, long long total_chunks, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int t = find_tensor(table, 4, 3, n, chunk);
    const long long* row = table + (size_t)t * 4;
    const void* p = reinterpret_cast<const void*>(row[0]);
    const long long numel = row[1];
    const int dtype = (int)row[2];
    const long long begin = (chunk - row[3]) * MT_CHUNK;
    const long long end = begin + MT_CHUNK < numel ? begin + MT_CHUNK : numel;
    const bool vec = (reinterpret_cast<uintptr_t>(p) & 15) == 0;
    if (vec && dtype == 1) {
      const long long nv = (end - begin) / 8;
      const uint4* q = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + begin);
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
        uint4 u = q[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int k = 0; k < 4; ++k) { float2 f = __bfloat1622float2(h[k]); acc += f.x * f.x + f.y * f.y; }
      }
      for (long long i = begin + nv * 8 + threadIdx.x; i < end; i += blockDim.x) {
        float v = load_as_f32(p, i, dtype); acc += v * v;
      }
    } else if (vec && dtype == 0) {
      const long long nv = (end - begin) / 4;
      const float4* q = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + begin);
      for (long long i = threadIdx.x; i < nv; i += blockDim.x) {
        float4 f = q[i]; acc += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
      }
      for (long long i = begin + nv * 4 + threadIdx.x; i < end; i += blockDim.x) {
        float v = load_as_f32(p, i, dtype); acc += v * v;
      }
    } else {
      for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float v = load_as_f32(p, i, dtype); acc += v * v;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(out, acc);
  }
}

__global__ void __launch_bounds__(MT_THREADS)
multi_scale_kernel(const long long* __restrict__ table, int n, long long total_chunks, const float* __restrict__ scale_ptr) {
  const float s = *scale_ptr;
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int t = find_tensor(table, 4, 3, n, chunk);
    const long long* row = table + (size_t)t * 4;
    void* p = reinterpret_cast<void*>(row[0]);
    const long long numel = row[1];
    const int dtype = (int)row[2];
    const long long begin = (chunk - row[3]) * MT_CHUNK;
    const long long end = begin + MT_CHUNK < numel ? begin + MT_CHUNK : numel;
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x)
      store_from_f32(p, i, dtype, load_as_f32(p, i, dtype) * s);
  }
}

// SGD with momentum (torch.optim.SGD semantics without dampening / Nesterov): g' = g * grad_scale + wd * p,
// buf = mu * buf + g', p -= lr * buf.  Table rows: {param, grad, momentum buffer (fp32), numel, param dtype,
// grad dtype, chunk prefix, -}.
__global__ void __launch_bounds__(MT_THREADS)
multi_sgd_kernel(const long long* __restrict__ table, int n, long long total_chunks, float lr, float momentum,
                 float weight_decay, const float* __restrict__ grad_scale, const unsigned int* __restrict__ status) {
  if (status && *reinterpret_cast<const volatile unsigned int*>(status) != 0u) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int t = find_tensor(table, 8, 6, n, chunk);
    const long long* row = table + (size_t)t * 8;
    void* p = reinterpret_cast<void*>(row[0]);
    const void* g = reinterpret_cast<const void*>(row[1]);
    float* buf = reinterpret_cast<float*>(row[2]);
    const long long numel = row[3];
    const int pdtype = (int)row[4], gdtype = (int)row[5];
    const long long begin = (chunk - row[6]) * MT_CHUNK;
    const long long end = begin + MT_CHUNK < numel ? begin + MT_CHUNK : numel;
    for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
      const float w = load_as_f32(p, i, pdtype);
      const float gi = load_as_f32(g, i, gdtype) * gs + weight_decay * w;
      const float b = momentum * buf[i] + gi;
      buf[i] = b;
      store_from_f32(p, i, pdtype, w - lr * b);
    }
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2;
  const float* grad_scale;       // device scalar multiplied into every gradient (may be null)
  const float* found_inf;        // device scalar; non-zero => skip the whole step (may be null)
  const unsigned int* status;    // copy, in device memory, of the device status word taken just before this launch;
                                 // non-zero (a bounded wait of an earlier kernel expired: gradients may be
                                 // incomplete) => skip the whole step (may be null)
};

__global__ void __launch_bounds__(MT_THREADS)
multi_adamw_kernel(const long long* __restrict__ table, int n, long long total_chunks, AdamArgs a) {
  if (a.found_inf && *a.found_inf != 0.f) return;
  if (a.status && *reinterpret_cast<const volatile unsigned int*>(a.status) != 0u) return;
  const float gs = a.grad_scale ? *a.grad_scale : 1.f;
  const float decay = 1.f - a.lr * a.weight_decay;
  const float step = a.lr / a.bias_c1;
  const float inv_sqrt_c2 = rsqrtf(a.bias_c2);
  for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
    const int t = find_tensor(table, 8, 7, n, chunk);
    const long long* row = table + (size_t)t * 8;
    float* master = reinterpret_cast<float*>(row[0]);
    __nv_bfloat16* model = reinterpret_cast<__nv_bfloat16*>(row[1]);
    const void* grad = reinterpret_cast<const void*>(row[2]);
    float* m = reinterpret_cast<float*>(row[3]);
    float* v = reinterpret_cast<float*>(row[4]);
    const long long numel = row[5];
    const int gdtype = (int)row[6];
    const long long begin = (chunk - row[7]) * MT_CHUNK;
    const long long end = begin + MT_CHUNK < numel ? begin + MT_CHUNK : numel;
    const bool aligned = ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
                           reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad) |
                           reinterpret_cast<uintptr_t>(model)) & 15) == 0;
    long long scalar_from = begin;
    if (aligned && gdtype != 2) {
      // 4 elements per vector: 16-byte accesses to the fp32 state, 8-byte to bf16 tensors.  Every thread
      // loads ADAM_UNROLL vectors of all four streams before it computes, so that enough bytes are in
      // flight per SM to cover the DRAM latency; the state is touched once per step, hence streaming hints.
      const long long nv = (end - begin) / 4;
      for (long long q0 = threadIdx.x; q0 < nv; q0 += (long long)blockDim.x * ADAM_UNROLL) {
        float4 p4[ADAM_UNROLL], m4[ADAM_UNROLL], v4[ADAM_UNROLL];
        float g4[ADAM_UNROLL][4];
#pragma unroll
        for (int u = 0; u < ADAM_UNROLL; ++u) {
          const long long q = q0 + (long long)u * blockDim.x;
          if (q < nv) {
            const long long i = begin + q * 4;
            p4[u] = __ldcs(reinterpret_cast<const float4*>(master + i));
            m4[u] = __ldcs(reinterpret_cast<const float4*>(m + i));
            v4[u] = __ldcs(reinterpret_cast<const float4*>(v + i));
            if (gdtype == 0) {
              const float4 t = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grad) + i));
              g4[u][0] = t.x; g4[u][1] = t.y; g4[u][2] = t.z; g4[u][3] = t.w;
            } else {
              const uint2 t = __ldcs(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(grad) + i));
              const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
              const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
              g4[u][0] = __bfloat162float(lo.x); g4[u][1] = __bfloat162float(lo.y);
              g4[u][2] = __bfloat162float(hi.x); g4[u][3] = __bfloat162float(hi.y);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < ADAM_UNROLL; ++u) {
          const long long q = q0 + (long long)u * blockDim.x;
          if (q >= nv) continue;
          const long long i = begin + q * 4;
          float pp[4] = {p4[u].x, p4[u].y, p4[u].z, p4[u].w}, mm[4] = {m4[u].x, m4[u].y, m4[u].z, m4[u].w},
                vv[4] = {v4[u].x, v4[u].y, v4[u].z, v4[u].w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float g = g4[u][k] * gs;
            mm[k] = a.beta1 * mm[k] + (1.f - a.beta1) * g;
            vv[k] = a.beta2 * vv[k] + (1.f - a.beta2) * g * g;
            const float denom = sqrtf(vv[k]) * inv_sqrt_c2 + a.eps;
            pp[k] = pp[k] * decay - step * mm[k] / denom;
          }
          __stcs(reinterpret_cast<float4*>(master + i), make_float4(pp[0], pp[1], pp[2], pp[3]));
          __stcs(reinterpret_cast<float4*>(m + i), make_float4(mm[0], mm[1], mm[2], mm[3]));
          __stcs(reinterpret_cast<float4*>(v + i), make_float4(vv[0], vv[1], vv[2], vv[3]));
          if (model) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
            uint2 o;
            o.x = *reinterpret_cast<const uint32_t*>(&lo); o.y = *reinterpret_cast<const uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(model + i) = o;
          }
        }
      }
      scalar_from = begin + nv * 4;
    }
    for (long long i = scalar_from + threadIdx.x; i < end; i += blockDim.x) {
      const float g = load_as_f32(grad, i, gdtype) * gs;
      const float mi = a.beta1 * m[i] + (1.f - a.beta1) * g;
      const float vi = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
      m[i] = mi; v[i] = vi;
      const float denom = sqrtf(vi) * inv_sqrt_c2 + a.eps;
      const float p = master[i] * decay - step * mi / denom;
      master[i] = p;
      if (model) model[i] = __float2bfloat16_rn(p);
    }
  }
}

// The status word itself lives in mapped host memory (the host polls it without synchronising); a read of it
// costs a PCIe round trip per warp, which serialises to milliseconds when every warp of a large grid does it.
// One thread copies it into device memory first and the optimizer's blocks read that copy.
__global__ void status_gate_kernel(const unsigned int* __restrict__ status, unsigned int* __restrict__ gate) {
  *gate = *reinterpret_cast<const volatile unsigned int*>(status);
}

int sm_count(int device);
static inline int mt_grid(long long chunks) {
  const long long cap = static_cast<long long>(sm_count_current()) * 8;
  return (int)(chunks < cap ? (chunks < 1 ? 1 : chunks) : cap);
}

}  // namespace axb

using namespace axb;

extern "C" int axb_multi_l2norm_sq(const long long* table, int n, long long total_chunks, float* out, void* stream) {
  multi_l2norm_sq_kernel<<<mt_grid(total_chunks), MT_THREADS, 0, (cudaStream_t)stream>>>(table, n, total_chunks, out);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
extern "C" int axb_multi_scale(const long long* table, int n, long long total_chunks, const float* scale, void* stream) {
  multi_scale_kernel<<<mt_grid(total_chunks), MT_THREADS, 0, (cudaStream_t)stream>>>(table, n, total_chunks, scale);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
// Device-memory copy of the status word of the current device, refreshed on `stream` (see status_gate_kernel);
// null when the device has no status word.
static unsigned int* refreshed_status_gate(cudaStream_t stream) {
  int dev = 0;
  unsigned int* status = nullptr;
  unsigned int* gate = nullptr;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    device_status_word(dev, &status);
    static unsigned int* gates[64] = {nullptr};
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (status && !gates[dev]) {
      if (cudaMalloc(&gates[dev], sizeof(unsigned int)) != cudaSuccess) { gates[dev] = nullptr; cudaGetLastError(); }
    }
    gate = status ? gates[dev] : nullptr;
  }
  if (gate) status_gate_kernel<<<1, 1, 0, stream>>>(status, gate);
  return gate;
}

extern "C" int axb_multi_sgd(const long long* table, int n, long long total_chunks, float lr, float momentum,
                             float weight_decay, const float* grad_scale, void* stream) {
  unsigned int* gate = refreshed_status_gate((cudaStream_t)stream);
  AXB_CUDA(cudaGetLastError());
  multi_sgd_kernel<<<mt_grid(total_chunks), MT_THREADS, 0, (cudaStream_t)stream>>>(table, n, total_chunks, lr, momentum,
                                                                                weight_decay, grad_scale, gate);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int axb_multi_adamw(const long long* table, int n, long long total_chunks, float lr, float beta1, float beta2,
                               float eps, float weight_decay, float bias_c1, float bias_c2, const float* grad_scale,
                               const float* found_inf, void* stream) {
  // The step is also skipped when a kernel that ran before it on this device reported an expired wait:
  // its output (activations or gradients) is incomplete, and the host learns of it at its next check_status.
  unsigned int* gate = refreshed_status_gate((cudaStream_t)stream);
  AXB_CUDA(cudaGetLastError());
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale, found_inf, gate};
  multi_adamw_kernel<<<mt_grid(total_chunks), MT_THREADS, 0, (cudaStream_t)stream>>>(table, n, total_chunks, a);
  AXB_CUDA(cudaGetLastError());
  return 0;
}
