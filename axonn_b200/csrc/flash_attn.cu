// Causal flash attention forward on tcgen05 tensor cores (sm_100a), grouped-query aware.
//
// Input is the fused projection output, packed [B, S, G, q_per_kv + 2, D]: for every KV group its query
// heads, then its key head, then its value head.  One CTA handles one (batch, query head, 128-row query
// tile) and walks the KV tiles up to the diagonal:
//
//   warp 0   TMA: Q once, then K_j / V_j into a 2-stage shared-memory ring (128-byte swizzle)
//   warp 1   MMA: S_j = Q K_j^T into one of two TMEM score buffers (issued one tile ahead), then
//            PV_j = P_j V_j into one of two TMEM output buffers; P_j is read from shared memory
//            (K-major), V_j is consumed in place as an MN-major operand - no transposes
//   warps 2-5 softmax: one thread per query row; tcgen05.ld the scores, online max / exp2 / row sum,
//            write P_j (bf16) into shared memory in the tensor core's canonical swizzled layout,
//            and fold the previous tile's PV product into the register-resident output row
//            (o = o * alpha + PV), so score MMAs, exponentials and PV MMAs of neighbouring tiles
//            overlap.
//
// Outputs: O [B, S, heads, D] bf16 and the per-row log-sum-exp (natural log, of the scaled scores)
// [B, heads, S] fp32 for the backward pass.  All waits are bounded.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace axb {

int make_tmap_2d_16bit(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, int dtype);
int make_tmap_2d_f32(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows);

struct FaParams {
  __nv_bfloat16* out;
  float* lse;
  int B, S, G, qpk;
  float scale_log2;
  unsigned int* status;
  unsigned long long timeout_ns;
  int debug;   // ablation builds only (-DAXB_ABLATION, read once from AXB_FA_DEBUG; otherwise 0 and compiled out): 4 phase timers of the two-tile forward
};

constexpr int FA_BQ = 128, FA_BKV = 128, FA_THREADS = 320;   // TMA warp, MMA warp, 8 softmax warps

template <int HD>
struct FaSmem {
  static constexpr int TILE = 128 * HD * 2;       // Q, K or V tile bytes
  static constexpr int P_BYTES = 128 * 128 * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = TILE;               // 2 stages
  static constexpr int V_OFF = 3 * TILE;           // 2 stages
  static constexpr int P_OFF = 5 * TILE;
  static constexpr int BAR_OFF = P_OFF + P_BYTES;
  static constexpr int NBARS = 1 + 2 + 2 + 2 + 2 + 2 + 1 + 1 + 2 + 2;
  // exchange between the two threads of a query row: maxima [2][2][128], row sums [2][128], sequence tags [2][128]
  static constexpr int XCH_OFF = BAR_OFF + NBARS * 8 + 16;
  static constexpr int TOTAL = XCH_OFF + 8 * 128 * 4 + 1024;
};

// Bounded wait until the other thread of a query row has published sequence number `want`.
__device__ __forceinline__ bool wait_partner(volatile int* flag, int want, volatile int* abort_flag, uint64_t timeout_ns) {
  uint64_t start = 0;
  for (uint32_t it = 0; *flag < want; ++it) {
    if ((it & 0xff) == 0xff) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (start == 0) start = now;
      else if (now - start > timeout_ns) { *abort_flag = 1; return false; }
    }
  }
  __threadfence_block();
  return true;
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const FaParams p) {
  using S_ = FaSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = bars + 3;
  uint64_t* kv_empty = bars + 5;
  uint64_t* s_full = bars + 7;
  uint64_t* s_empty = bars + 9;
  uint64_t* p_full = bars + 11;
  uint64_t* p_empty = bars + 12;
  uint64_t* o_full = bars + 13;
  uint64_t* o_empty = bars + 15;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + S_::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.S / FA_BQ;
  const int qt = nq - 1 - static_cast<int>(blockIdx.z);  // heaviest tiles first, over the whole grid
  const int head = blockIdx.x;
  const int b = blockIdx.y;
  const int g = head / p.qpk, jq = head % p.qpk;
  const int n_kv = qt + 1;                               // causal: tiles 0..qt
  const int row0 = b * p.S + qt * FA_BQ;                 // row in the [B*S, G*(qpk+2)*HD] view
  const int col_q = (g * (p.qpk + 2) + jq) * HD;
  const int col_k = (g * (p.qpk + 2) + p.qpk) * HD;
  const int col_v = col_k + HD;
  const uint64_t timeout = p.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 8);
      mbar_init(&o_full[i], 1); mbar_init(&o_empty[i], 8);
    }
    mbar_init(p_full, 8); mbar_init(p_empty, 1);
    for (int i = 0; i < 256; ++i) reinterpret_cast<volatile int*>(smem + S_::XCH_OFF + 6 * 128 * 4)[i] = 0;
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) tma_prefetch_desc(&tmQKV);
  if (warp == 1) { tmem_alloc(tmem_ptr_smem, 512); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tmem_s = tmem_base;          // 2 x 128 columns
  const uint32_t tmem_o = tmem_base + 256;    // 2 x HD columns

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_expect_tx(q_full, S_::TILE);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) tma_load_2d(smem + S_::Q_OFF + c * 16384, &tmQKV, q_full, col_q + 64 * c, row0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&kv_empty[st], ph ^ 1, abort_flag, timeout)) { ok = false; break; }
        const int krow = b * p.S + j * FA_BKV;
        mbar_expect_tx(&k_full[st], S_::TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + S_::K_OFF + st * S_::TILE + c * 16384, &tmQKV, &k_full[st], col_k + 64 * c, krow);
        mbar_expect_tx(&v_full[st], S_::TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_2d(smem + S_::V_OFF + st * S_::TILE + c * 16384, &tmQKV, &v_full[st], col_v + 64 * c, krow);
      }
      if (!ok) {
        // drain: give in-flight copies time to land before the CTA exits
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
        report_status(p.status, 0x401u);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = true;
      const uint32_t idesc_s = umma_idesc(1, 0, 0, 128, 128);
      const uint32_t idesc_o = umma_idesc(1, 0, 1, 128, HD);
      const uint32_t q_addr = smem_u32(smem + S_::Q_OFF);
      const uint32_t p_addr = smem_u32(smem + S_::P_OFF);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(smem + S_::K_OFF + (j & 1) * S_::TILE);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_f16(tmem_s + (j & 1) * 128, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024),
                   idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      ok = mbar_wait(q_full, 0, abort_flag, timeout) && mbar_wait(&k_full[0], 0, abort_flag, timeout);
      if (ok) { tcgen05_fence_after(); issue_s(0); }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int u = j + 1;
          if (!mbar_wait(&k_full[u & 1], (u >> 1) & 1, abort_flag, timeout) ||
              !mbar_wait(&s_empty[u & 1], ((u >> 1) & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
          tcgen05_fence_after();
          issue_s(u);
        }
        if (!mbar_wait(p_full, j & 1, abort_flag, timeout) || !mbar_wait(&v_full[j & 1], (j >> 1) & 1, abort_flag, timeout) ||
            !mbar_wait(&o_empty[j & 1], ((j >> 1) & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t v_addr = smem_u32(smem + S_::V_OFF + (j & 1) * S_::TILE);
#pragma unroll
        for (int kk = 0; kk < FA_BKV / 16; ++kk) {
          const uint64_t adesc = umma_smem_desc(p_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
          // V: MN-major, 64-wide column chunks 16 KB apart (leading), 8-row groups 1 KB apart (stride)
          const uint64_t bdesc = umma_smem_desc(v_addr + kk * 2048, 16384, 1024);
          umma_f16(tmem_o + (j & 1) * HD, adesc, bdesc, idesc_o, kk != 0 ? 1u : 0u);
        }
        umma_commit(&o_full[j & 1]);
        umma_commit(p_empty);
        umma_commit(&kv_empty[j & 1]);
      }
      if (!ok) report_status(p.status, 0x402u);
    }
  } else {
    // ------------------------------------------------------------------ softmax + output accumulation
    // Eight warps: two share each TMEM lane quarter; thread = (query row r, column half).  A thread owns 64 of
    // the 128 score columns of its row and HD/2 of the output columns, so that a KV tile costs it one TMEM
    // read of the scores (kept in registers between the max and the exponentials) and one of the PV product.
    // The two threads of a row exchange their partial row maxima through shared memory (one 64-thread named
    // barrier per tile); the partial row sums are only combined at the end.
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;                 // query row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    constexpr int OC = HD / 2;                    // output columns per thread
    float o[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    bool ok = true;
    uint8_t* p_row = smem + S_::P_OFF + (r >> 3) * 1024 + (r & 7) * 128 + half * 16384;
    volatile float* xch = reinterpret_cast<volatile float*>(smem + S_::XCH_OFF);   // [2 tile parities][2 halves][128 rows]
    volatile int* xflag = reinterpret_cast<volatile int*>(smem + S_::XCH_OFF + 6 * 128 * 4);   // [2 halves][128 rows]
    for (int j = 0; j < n_kv; ++j) {
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t s_addr = tmem_s + lane_base + (j & 1) * 128 + half * 64;
      const bool diag = (j == qt);
      uint32_t sv[64];
      tmem_ld_32x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
      tmem_ld_32x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
      tmem_ld_wait();
      // the score buffer can be reused by the MMA warp as soon as both halves hold it in registers
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[j & 1]);
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (!diag || (half * 64 + i) <= r) mx = fmaxf(mx, __uint_as_float(sv[i]));
      mx *= p.scale_log2;                       // the scale is positive: scale the maximum once
      xch[((j & 1) * 2 + half) * 128 + r] = mx;
      __threadfence_block();
      xflag[half * 128 + r] = j + 1;
      if (!wait_partner(xflag + (half ^ 1) * 128 + r, j + 1, abort_flag, timeout)) { ok = false; break; }
      mx = fmaxf(mx, xch[((j & 1) * 2 + (half ^ 1)) * 128 + r]);
      const float m_new = fmaxf(m, mx);
      const float alpha = exp2f(m - m_new);
      if (!mbar_wait(p_empty, (j & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
      // exponentials, partial row sum, this thread's half of the P row (bf16, swizzled K-major layout)
      float rowsum = 0.f;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float e0 = exp2f(__uint_as_float(sv[c * 32 + 2 * i]) * p.scale_log2 - m_new);
          float e1 = exp2f(__uint_as_float(sv[c * 32 + 2 * i + 1]) * p.scale_log2 - m_new);
          if (diag) {
            if (half * 64 + c * 32 + 2 * i > r) e0 = 0.f;
            if (half * 64 + c * 32 + 2 * i + 1 > r) e1 = 0.f;
          }
          const __nv_bfloat162 h = __floats2bfloat162_rn(e0, e1);
          rowsum += e0 + e1;
          packed[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        // columns half*64 + [c*32, c*32+32): 16-byte chunks (c * 4 + t), t = 0..3, of the 64-column block
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int chunk = (c * 4 + t) ^ (r & 7);
          *reinterpret_cast<uint4*>(p_row + chunk * 16) =
              make_uint4(packed[4 * t], packed[4 * t + 1], packed[4 * t + 2], packed[4 * t + 3]);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      l = l * alpha + rowsum;
      m = m_new;
      // fold the previous tile's PV product into the output row
      if (j > 0) {
        const int u = j - 1;
        if (!mbar_wait(&o_full[u & 1], (u >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t o_addr = tmem_o + lane_base + (u & 1) * HD + half * OC;
        uint32_t v[OC];
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) tmem_ld_32x32(o_addr + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&o_empty[u & 1]);
#pragma unroll
        for (int i = 0; i < OC; ++i) o[i] = o[i] * alpha_prev + __uint_as_float(v[i]);
      }
      alpha_prev = alpha;
    }
    if (ok) {
      const int u = n_kv - 1;
      if (mbar_wait(&o_full[u & 1], (u >> 1) & 1, abort_flag, timeout)) {
        tcgen05_fence_after();
        // total row sum = sum of the two halves' partial sums
        volatile float* lx = xch + 4 * 128;        // [2 halves][128 rows], used once
        lx[half * 128 + r] = l;
        __threadfence_block();
        xflag[half * 128 + r] = n_kv + 1;
        if (!wait_partner(xflag + (half ^ 1) * 128 + r, n_kv + 1, abort_flag, timeout)) ok = false;
        l += lx[(half ^ 1) * 128 + r];
        const uint32_t o_addr = tmem_o + lane_base + (u & 1) * HD + half * OC;
        const float inv_l = 1.f / l;
        const size_t heads = static_cast<size_t>(p.G) * p.qpk;
        __nv_bfloat16* dst = p.out + ((static_cast<size_t>(b) * p.S + qt * FA_BQ + r) * heads + head) * HD + half * OC;
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(o_addr + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = t * 8 + i * 2;
              const float a0 = (o[c * 32 + e] * alpha_prev + __uint_as_float(v[e])) * inv_l;
              const float a1 = (o[c * 32 + e + 1] * alpha_prev + __uint_as_float(v[e + 1])) * inv_l;
              const __nv_bfloat162 h = __floats2bfloat162_rn(a0, a1);
              w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + c * 32 + t * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        if (half == 0)
          p.lse[(static_cast<size_t>(b) * heads + head) * p.S + qt * FA_BQ + r] = (m + log2f(l)) * 0.6931471805599453f;
      } else {
        ok = false;
      }
    }
    if (!ok && lane == 0) report_status(p.status, 0x404u);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int HD>
static int fa_launch(const CUtensorMap& tm, const FaParams& p, int device, cudaStream_t s) {
  using S_ = FaSmem<HD>;
  static bool configured[64] = {false};
  auto kern = fa_fwd_kernel<HD>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S_::TOTAL));
    configured[device & 63] = true;
  }
  dim3 grid(p.G * p.qpk, p.B, p.S / FA_BQ);   // z (slowest) = query tile, heaviest tiles first
  kern<<<grid, FA_THREADS, S_::TOTAL, s>>>(tm, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}


// -----------------------------------------------------------------------------------------------------
// Forward, two query tiles at a time ("ping-pong"), persistent CTAs.  A work item is the pair of adjacent
// 128-row query tiles A = 2u and B = 2u + 1 of one (batch, head); they share every K_j / V_j tile that the TMA
// warp loads.  One CTA per SM walks its share of the items (longest first): the loads and the first score MMAs
// of the next item overlap the previous item's last softmax steps and its output stores.
//
//   warp 0      TMA: Q_A, Q_B once; K_j and V_j into separate 2-stage rings
//   warps 1, 2  MMA of tile A and of tile B: S_X = Q_X K^T for 64 keys into one of the two score buffers of tile X, then O_X += P_X V
//               with the A operand P_X read from tensor memory (bf16, in the first 32 columns of the score
//               buffer, written there by the softmax threads) and O_X accumulating in tensor memory
//   warp 3      idle: it completes the first warpgroup, which hands most of its registers to the others
//   warps 4-7   softmax of tile A, one thread per query row (TMEM lane): one read of the step's 64 scores, row
//   warps 8-11  maximum, exponentials, row sum, P back into tensor memory.  (8-11: the same for tile B.)
//
// The work of a query tile proceeds in steps of 64 key columns, and the 128 score columns of the tile are two
// 64-column buffers used alternately: while the softmax threads work on step s, the scores of step s + 1 are
// already complete in the other buffer (S(s + 2) is issued right after the PV MMA of step s, which is the last
// reader of that buffer), so the threads go from one step to the next without waiting for the tensor core, and
// the tensor core always has the other tile's and the next step's MMAs queued.  The running maximum of a row is
// only raised when a step's maximum exceeds it by more than 2^8 (the probabilities then stay below 256, exact
// in the final normalisation because the row sum uses the same reference); only then the row's O accumulator
// is rescaled in tensor memory, by the softmax thread itself, after waiting for the previous step's PV MMA.
template <int HD>
struct Fa2Smem {
  static constexpr int TILE = 128 * HD * 2;
  static constexpr int Q_OFF = 0;                  // Q_A, Q_B
  static constexpr int K_OFF = 2 * TILE;           // 2 stages
  static constexpr int V_OFF = 4 * TILE;           // 2 stages
  static constexpr int BAR_OFF = 6 * TILE;
  static constexpr int NBARS = 2 + 8 + 4 + 4 + 2;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16 + 1024;
};

constexpr int FA2_THREADS = 384;
#ifndef FA2_POLY_OF_8
#define FA2_POLY_OF_8 3     // pairs of every 8 whose exponential runs on the FMA pipes instead of the ex2 unit
#endif
#ifndef FA2_PACKED
#define FA2_PACKED 1        // packed fp32x2 arithmetic for the scale-and-subtract and the row sum
#endif

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Work item `idx` of the persistent grid: pairs of query tiles sorted by decreasing length (pair u has 4u + 3 tile
// steps), dealt to the CTAs in a snake (0..G-1, G-1..0, ...) so that every CTA gets nearly the same total.
struct Fa2Item { int u, head, b; };
__device__ __forceinline__ bool fa2_item(const FaParams& p, int k, Fa2Item& w) {
  const int G = gridDim.x, c = blockIdx.x;
  const int heads = p.G * p.qpk, bh = p.B * heads, npairs = p.S / (2 * FA_BQ);
  const int idx = k * G + ((k & 1) ? G - 1 - c : c);
  if (idx >= bh * npairs) return false;
  w.u = npairs - 1 - idx / bh;
  const int rem = idx % bh;
  w.head = rem % heads;
  w.b = rem / heads;
  return true;
}

template <int HD>
__global__ void __launch_bounds__(FA2_THREADS, 1)
fa_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tmQKV, const FaParams p) {
  using S_ = Fa2Smem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_::BAR_OFF);
  uint64_t* q_full = bars;         // one arrival per work item
  uint64_t* q_empty = bars + 1;    // both Q tiles may be overwritten (the item's last score MMAs are done)
  uint64_t* k_full = bars + 2;
  uint64_t* k_empty = bars + 4;
  uint64_t* v_full = bars + 6;
  uint64_t* v_empty = bars + 8;
  uint64_t* s_full = bars + 10;    // [query tile][score buffer]
  uint64_t* p_full = bars + 14;    // [query tile][score buffer]
  uint64_t* pv_done = bars + 18;   // per query tile: one phase per step, completed by that step's PV MMA
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + S_::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t timeout = p.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 2);           // "empty": one release per MMA warp
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 2); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 2);
      mbar_init(&pv_done[i], 1);
    }
    for (int i = 0; i < 4; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) tma_prefetch_desc(&tmQKV);
  if (warp == 1) { tmem_alloc(tmem_ptr_smem, 512); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // columns: score buffers of A [0,64) [64,128), of B [128,192) [192,256) (P = the first 32 columns of a
  // buffer), O_A [256,256+HD), O_B [384,384+HD)
  // the register budget of a role must be set inside its branch: after a join the compiler assumes the smaller one
  if (warp < 4) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
   if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      uint32_t kvc = 0;                                     // KV tiles loaded so far: ring stage and phase
      Fa2Item w;
      for (int it = 0; ok && fa2_item(p, it, w); ++it) {
        const int g = w.head / p.qpk, jq = w.head % p.qpk;
        const int col_q = (g * (p.qpk + 2) + jq) * HD;
        const int col_k = (g * (p.qpk + 2) + p.qpk) * HD;
        const int col_v = col_k + HD;
        const int row0 = w.b * p.S + 2 * w.u * FA_BQ;
        const int n_b = 2 * w.u + 2;                         // KV tiles of 128 keys
        if (!mbar_wait(q_empty, (it & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
        mbar_expect_tx(q_full, 2 * S_::TILE);
#pragma unroll
        for (int x = 0; x < 2; ++x)
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + S_::Q_OFF + x * S_::TILE + c * 16384, &tmQKV, q_full, col_q + 64 * c, row0 + x * FA_BQ);
        for (int j = 0; j < n_b && ok; ++j, ++kvc) {
          const int st = kvc & 1;
          const uint32_t ph = (kvc >> 1) & 1;
          const int krow = w.b * p.S + j * FA_BKV;
          if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, timeout)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], S_::TILE);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + S_::K_OFF + st * S_::TILE + c * 16384, &tmQKV, &k_full[st], col_k + 64 * c, krow);
          if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, timeout)) { ok = false; break; }
          mbar_expect_tx(&v_full[st], S_::TILE);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + S_::V_OFF + st * S_::TILE + c * 16384, &tmQKV, &v_full[st], col_v + 64 * c, krow);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();     // give in-flight copies time to land before the CTA exits
        while (globaltimer_ns() - t0 < 200000ull) {}
        report_status(p.status, 0x405u);
      }
    }
   } else if (warp <= 2) {
    // ------------------------------------------------------------------ MMA issue: warp 1 for tile A, warp 2 for B
    // (one thread cannot issue both tiles' 24 instructions per step as fast as the tensor core retires them)
    if (elect_one()) {
      bool ok = true;
      const int x = warp - 1;
      const uint32_t idesc_s = umma_idesc(1, 0, 0, 128, 64);
      const uint32_t idesc_o = umma_idesc(1, 0, 1, 128, HD);
      const uint32_t s_tmem = tmem_base + x * 128, o_tmem = tmem_base + 256 + x * 128;
      const uint64_t qd = umma_smem_desc(smem_u32(smem + S_::Q_OFF + x * S_::TILE), 16, 1024);
      // descriptors of a k-step = the tile's descriptor + a constant in the (16-byte unit) address field
      // scores of step s (keys [64 s, 64 s + 64)): rows (s & 1) * 64 .. of K tile kv, into score buffer s & 1
      auto issue_s = [&](uint32_t kv, int sb) {
        const uint64_t kd = umma_smem_desc(smem_u32(smem + S_::K_OFF + (kv & 1) * S_::TILE) + sb * 8192, 16, 1024);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_f16(s_tmem + sb * 64, qd + off, kd + off, idesc_s, kk != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](uint32_t kv, int sb, bool first) {
        // V: MN-major, 64-wide column chunks 16 KB apart (leading), 8-row groups 1 KB apart (stride)
        const uint64_t vd = umma_smem_desc(smem_u32(smem + S_::V_OFF + (kv & 1) * S_::TILE) + sb * 8192, 16384, 1024);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_f16_ts(o_tmem, s_tmem + sb * 64 + kk * 8, vd + ((kk * 2048) >> 4), idesc_o, (first && kk == 0) ? 0u : 1u);
      };
      uint32_t kvc = 0;            // KV tiles of earlier items
      uint32_t tc = 0;             // steps of earlier items and of this one so far (barrier phases)
      const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0 && x == 0;
      long long pw_p = 0, pw_kv = 0, p_mark = 0, p_t0 = probe ? clock64() : 0;
      Fa2Item w;
      for (int it = 0; ok && fa2_item(p, it, w); ++it) {
        const int n_b = 4 * w.u + 4, n_x = n_b - 2 + 2 * x;     // steps of 64 keys: causal, tiles 2u and 2u + 1
        if (!mbar_wait(q_full, it & 1, abort_flag, timeout) ||
            !mbar_wait(&k_full[kvc & 1], (kvc >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        // both score buffers are free: the previous item's PV MMAs, which read P from them, were issued earlier
#pragma unroll
        for (int sb = 0; sb < 2; ++sb) { issue_s(kvc, sb); umma_commit(&s_full[x * 2 + sb]); }
        umma_commit(&k_empty[kvc & 1]);
        if (n_x == 2) umma_commit(q_empty);                    // a two-step tile has no further score MMAs
        for (int st = 0; st < n_x && ok; ++st) {
          const uint32_t kv = kvc + (st >> 1);
          const int sb = st & 1;
          if (probe) p_mark = clock64();
          if (!mbar_wait(&p_full[x * 2 + sb], (tc >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          if (probe) { const long long now = clock64(); pw_p += now - p_mark; p_mark = now; }
          if (!mbar_wait(&v_full[kv & 1], (kv >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          if (probe) pw_kv += clock64() - p_mark;
          ++tc;
          tcgen05_fence_after();
          issue_pv(kv, sb, st == 0);
          umma_commit(&pv_done[x]);
          if (sb == 1) umma_commit(&v_empty[kv & 1]);
          if (st + 2 < n_x) {
            const uint32_t kn = kv + 1;                        // step st + 2 reads the next K tile
            if (probe) p_mark = clock64();
            if (!mbar_wait(&k_full[kn & 1], (kn >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
            if (probe) pw_kv += clock64() - p_mark;
            tcgen05_fence_after();
            issue_s(kn, sb);
            umma_commit(&s_full[x * 2 + sb]);
            if (sb == 1) {
              umma_commit(&k_empty[kn & 1]);                   // this tile's last read of that K tile
              if (st + 3 == n_x) umma_commit(q_empty);         // ... and of Q: the item's last score MMAs
            }
          }
        }
        if (x == 0 && ok) {
          // Tile A does not read the item's last KV tile, but the ring counts two releases per tile.  The release
          // may only be given once that tile has been loaded: before that, the stage still belongs to the tile
          // two steps earlier, and an early arrival would complete that tile's "empty" phase while tile B's warp
          // is still reading it.
          const uint32_t last = kvc + (n_b >> 1) - 1;
          if (!mbar_wait(&k_full[last & 1], (last >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          umma_commit(&k_empty[last & 1]);
          if (!mbar_wait(&v_full[last & 1], (last >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          umma_commit(&v_empty[last & 1]);
        }
        kvc += n_b >> 1;
      }
      if (probe) {
        volatile unsigned int* wd = reinterpret_cast<volatile unsigned int*>(p.status);
        wd[13] = static_cast<unsigned>(pw_p); wd[14] = static_cast<unsigned>(pw_kv);
        wd[15] = static_cast<unsigned>(clock64() - p_t0);
      }
      if (!ok) report_status(p.status, 0x406u);
    }
   }
  } else {
    // ------------------------------------------------------------------ softmax of query tile x
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int x = (warp - 4) >> 2;
    const int q4 = warp & 3;                         // the TMEM lane quarter this warp may access
    const int r = q4 * 32 + lane;                    // query row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    const uint32_t s_addr = tmem_base + lane_base + x * 128;
    const uint32_t o_addr = tmem_base + lane_base + 256 + x * 128;
    bool ok = true;
    uint32_t tc = 0;                                 // steps so far (all items): barrier phases
    const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0 && warp == 4 && lane == 0;
    long long pw_s = 0, pt_ld = 0, pt_max = 0, pt_exp = 0, pt_epi = 0, p_mark = 0;
    Fa2Item w;
    for (int it = 0; ok && fa2_item(p, it, w); ++it) {
      const int n_x = 4 * w.u + 2 + 2 * x;           // steps of 64 keys; the item's step counts are even, so the
      float m = -INFINITY, l = 0.f;                  // score buffer of a step is also (tc & 1)
      for (int st = 0; st < n_x; ++st, ++tc) {
        const int sb = st & 1;
        if (probe) p_mark = clock64();
        if (!mbar_wait(&s_full[x * 2 + sb], (tc >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const long long now = clock64(); pw_s += now - p_mark; p_mark = now; }
        tcgen05_fence_after();
        uint32_t sv[64];
        tmem_ld_32x32(s_addr + sb * 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32(s_addr + sb * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_wait();
        if (probe) { const long long now = clock64(); pt_ld += now - p_mark; p_mark = now; }
        // key column 64 st + i is visible to query row 256 u + 128 x + r when it is not to the right of it
        const int d = 64 * st - 128 * x - 256 * w.u;
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        if (d + 63 > 0) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (d + i > r) sv[i] = 0xff800000u;         // -inf: exp2 gives exactly 0
        }
#pragma unroll
        for (int i = 0; i < 64; i += 8) {              // three-input maxima, four independent chains
          mx0 = fmax3(mx0, __uint_as_float(sv[i]), __uint_as_float(sv[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(sv[i + 2]), __uint_as_float(sv[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(sv[i + 4]), __uint_as_float(sv[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(sv[i + 6]), __uint_as_float(sv[i + 7]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;   // the scale is positive
        const float m_new = (mx - m > 8.f) ? mx : m;   // first step: m = -inf, always raised (key 0 is visible)
        float alpha = 1.f;                             // stays 1 when no row of the warp raises its reference
        if (__any_sync(0xffffffffu, m_new != m)) {
          alpha = exp2f(m - m_new);
          if (st > 0) {
            // rescale O in place once the previous step's PV MMA has completed (phase tc - 1 of pv_done)
            if (!mbar_wait(&pv_done[x], (tc - 1) & 1, abort_flag, timeout)) { ok = false; break; }
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < HD / 32; ++c) {
              uint32_t v[32];
              tmem_ld_32x32(o_addr + c * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tmem_st_32x32(o_addr + c * 32, v);
            }
          }
          l *= alpha;
          m = m_new;
        }
        if (probe) { const long long now = clock64(); pt_max += now - p_mark; p_mark = now; }
        // Exponentials of the step's 64 scores, two at a time with packed fp32 arithmetic.  The special-function
        // unit (ex2) is the scarcest resource of this kernel, so FA2_POLY_OF_8 of every 8 pairs are computed on
        // the FMA pipes instead: 2^x = 2^n * 2^f with n = round(x) (taken from the mantissa of x + 1.5 * 2^23)
        // and a cubic for 2^f on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding of P; the row sum
        // uses the same values, so the normalisation stays consistent).
        const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m, -m);
        float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
#if FA2_PACKED
          float2 xx = __ffma2_rn(make_float2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), sc2, nm2);
#else
          float2 xx = make_float2(fmaf(__uint_as_float(sv[2 * i]), sc2.x, nm2.x), fmaf(__uint_as_float(sv[2 * i + 1]), sc2.x, nm2.x));
#endif
          float2 e;
          if ((i & 7) < FA2_POLY_OF_8) {
            xx.x = fmaxf(xx.x, -125.f); xx.y = fmaxf(xx.y, -125.f);     // masked scores (-inf) become 2^-125
            const float2 t = __fadd2_rn(xx, make_float2(12582912.f, 12582912.f));
            const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
            const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), xx);
            float2 q = __ffma2_rn(make_float2(0.05517147481441498f, 0.05517147481441498f), f,
                                  make_float2(0.242610901594162f, 0.242610901594162f));
            q = __ffma2_rn(q, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
            q = __ffma2_rn(q, f, make_float2(0.9999281167984009f, 0.9999281167984009f));
            e.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
            e.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
          } else {
            e.x = exp2f(xx.x); e.y = exp2f(xx.y);
          }
#if FA2_PACKED
          if (i & 1) acc1 = __fadd2_rn(acc1, e); else acc0 = __fadd2_rn(acc0, e);
#else
          if (i & 1) { acc1.x += e.x; acc1.y += e.y; } else { acc0.x += e.x; acc0.y += e.y; }
#endif
          const __nv_bfloat162 h = __floats2bfloat162_rn(e.x, e.y);
          packed[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        tmem_st_32x32(s_addr + sb * 64, packed);
        l += (acc0.x + acc0.y) + (acc1.x + acc1.y);
        // A parity wait is only meaningful while the barrier is at most one phase ahead of the waiter, so every
        // phase of pv_done is observed, in order: the previous step's PV MMA here - it has had this whole step to
        // complete, and this step's cannot be issued before the arrival below.
        if (st >= 1 && !mbar_wait(&pv_done[x], (tc - 1) & 1, abort_flag, timeout)) { ok = false; break; }
        tmem_st_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[x * 2 + sb]);
        if (probe) { const long long now = clock64(); pt_exp += now - p_mark; p_mark = now; }
      }
      if (probe) p_mark = clock64();
      // the item's last PV MMA: phase tc - 1 of pv_done (tc - 2 was observed in the last step)
      if (!ok || !mbar_wait(&pv_done[x], (tc - 1) & 1, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      const float inv_l = 1.f / l;
      const size_t heads = static_cast<size_t>(p.G) * p.qpk;
      const size_t qrow = static_cast<size_t>(w.b) * p.S + (2 * w.u + x) * FA_BQ + r;
      __nv_bfloat16* dst = p.out + (qrow * heads + w.head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(o_addr + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t wv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = t * 8 + i * 2;
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[e]) * inv_l, __uint_as_float(v[e + 1]) * inv_l);
            wv[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + c * 32 + t * 8) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
      p.lse[(static_cast<size_t>(w.b) * heads + w.head) * p.S + (2 * w.u + x) * FA_BQ + r] = (m + log2f(l)) * 0.6931471805599453f;
      // the next item's first PV MMA overwrites O: it waits for this thread's next arrival on p_full, which follows
      // these reads in program order
      tcgen05_fence_before();
      if (probe) pt_epi += clock64() - p_mark;
    }
    if (probe) {
      volatile unsigned int* wd = reinterpret_cast<volatile unsigned int*>(p.status);
      wd[8] = static_cast<unsigned>(pw_s); wd[9] = static_cast<unsigned>(pt_ld); wd[10] = static_cast<unsigned>(pt_max);
      wd[11] = static_cast<unsigned>(pt_exp); wd[12] = static_cast<unsigned>(pt_epi); wd[7] = tc;
    }
    if (!ok && lane == 0) report_status(p.status, 0x407u);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int HD>
static int fa_launch_pingpong(const CUtensorMap& tm, const FaParams& p, int device, cudaStream_t s) {
  using S_ = Fa2Smem<HD>;
  static bool configured[64] = {false};
  auto kern = fa_fwd_pingpong_kernel<HD>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S_::TOTAL));
    configured[device & 63] = true;
  }
  const long long items = static_cast<long long>(p.B) * p.G * p.qpk * (p.S / (2 * FA_BQ));
  const int sms = sm_count(device);
  kern<<<static_cast<int>(items < sms ? items : sms), FA2_THREADS, S_::TOTAL, s>>>(tm, p);   // persistent CTAs
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// AXONN_FA_FWD=single keeps the one-tile-per-CTA forward for every shape (A/B runs); read once.
static bool fa_pingpong_enabled() {
  static const bool on = [] {
    const char* e = getenv("AXONN_FA_FWD");
    return !(e && e[0] == 's');
  }();
  return on;
}

}  // namespace axb

// qkv: [B, S, G, qpk + 2, D] bf16 contiguous; out: [B, S, G*qpk, D] bf16; lse: [B, G*qpk, S] fp32.
extern "C" int axb_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int G, int qpk, int D,
                                  float scale, int device, void* stream) {
  using namespace axb;
  if (D != 64 && D != 128) { set_error("flash attention: head_dim must be 64 or 128"); return -1; }
  if (S % 128) { set_error("flash attention: sequence length must be a multiple of 128"); return -1; }
  CUtensorMap tm;
  if (make_tmap_2d_16bit(&tm, qkv, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(G) * (qpk + 2) * D, 128, 0))
    return -1;
  FaParams p;
  p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.B = B; p.S = S; p.G = G; p.qpk = qpk;
  p.scale_log2 = scale * 1.4426950408889634f;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("flash attention: no status word"); return -1; }
  p.status = st; p.timeout_ns = wait_timeout_ns();
  p.debug = 0;
#ifdef AXB_ABLATION
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("AXB_FA_DEBUG"); dbg = e ? atoi(e) : 0; } p.debug = dbg; }
#endif
  if (S % 256 == 0 && fa_pingpong_enabled()) {
    if (D == 128) return fa_launch_pingpong<128>(tm, p, device, static_cast<cudaStream_t>(stream));
    return fa_launch_pingpong<64>(tm, p, device, static_cast<cudaStream_t>(stream));
  }
  if (D == 128) return fa_launch<128>(tm, p, device, static_cast<cudaStream_t>(stream));
  return fa_launch<64>(tm, p, device, static_cast<cudaStream_t>(stream));
}

// =====================================================================================================
// Backward.  One CTA owns one (batch, KV group, 128-row KV tile): K and V stay in shared memory, dK and dV
// accumulate in TMEM, and the CTA walks every (query tile on or below the diagonal, query head of the
// group).  Per step:
//   MMA      S = Q K^T and dP = dO V^T into TMEM
//   softmax  P = exp2(S * scale_log2 - lse * log2e), dS = P * (dP - delta) * scale, both written as bf16
//            tiles in the canonical swizzled layout (one thread per query row)
//   MMA      dV += P^T dO, dK += dS^T Q (A operands read MN-major: the same bytes, transposed by the
//            descriptor), dQ_partial = dS K into the TMEM columns S occupied
//   softmax  dQ_partial -> fp32 global accumulator with vector reductions (red.global.add.v4.f32)
// delta = rowsum(dO * O) comes from a small pre-kernel.  dK/dV are written straight into the packed
// gradient tensor; dQ is converted from the fp32 accumulator by the caller.
namespace axb {

struct FaBwdParams {
  const float* lse;     // [B, heads, S]
  const float* delta;   // [B, heads, S]
  float* dq_acc;        // [B, S, heads, D] fp32, zero-initialised
  __nv_bfloat16* dqkv;  // [B, S, G, qpk + 2, D]
  int B, S, G, qpk;
  float scale, scale_log2;
  unsigned int* status;
  unsigned long long timeout_ns;
  int debug;   // ablation builds only (-DAXB_ABLATION, then read once from AXB_FA_DEBUG; otherwise 0 and every branch on it is compiled out): 1 no dQ reductions, 2 no exponentials, 4 phase timers, 8 release Q/dO after the dQ MMAs
};

template <int HD>
struct FaBwdSmem {
  static constexpr int TILE = 128 * HD * 2;
  static constexpr int K_OFF = 0, V_OFF = TILE, Q_OFF = 2 * TILE, DO_OFF = 3 * TILE;
  static constexpr int P_OFF = 4 * TILE, DS_OFF = P_OFF + 32768;
  // After the MMAs of an iteration the P / dS tiles are dead until the next iteration writes them; the dQ
  // partial (fp32) is staged there as 32-row x 32-column boxes (4 KB, 128-byte swizzle), HD / 64 per warp,
  // for the bulk tensor reductions into global memory.
  static constexpr int DQ_BOX_BYTES = 32 * 32 * 4;
  static constexpr int BAR_OFF = P_OFF + 65536;
  static constexpr int NBARS = 7;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16 + 1024;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// thread r holds KV row r of the dK (which = 0) or dV (which = 1) accumulator: TMEM -> packed gradient tensor
template <int HD>
__device__ __forceinline__ void fa_store_kv_grad(const FaBwdParams& p, uint32_t src, int b, int jt, int g, int r, int which) {
  const size_t kvpos = static_cast<size_t>(b) * p.S + jt * 128 + r;
  __nv_bfloat16* dst = p.dqkv + (kvpos * p.G + g) * (p.qpk + 2) * HD + static_cast<size_t>(p.qpk + which) * HD;
#pragma unroll 1
  for (int c = 0; c < HD / 32; ++c) {
    uint32_t v[32];
    tmem_ld_32x32(src + c * 32, v);
    tmem_ld_wait();
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[t * 8 + 2 * k]), __uint_as_float(v[t * 8 + 2 * k + 1]));
        w[k] = *reinterpret_cast<const uint32_t*>(&h);
      }
      *reinterpret_cast<uint4*>(dst + c * 32 + t * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

constexpr int FA_BWD_THREADS = 320;   // TMA warp, MMA warp, 8 softmax / reduction warps

template <int HD>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO,
              const __grid_constant__ CUtensorMap tmDQ, const FaBwdParams p) {
  using S_ = FaBwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* pds_full = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* s_free = bars + 6;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + S_::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile int* reads_done = reinterpret_cast<volatile int*>(tmem_ptr_smem + 2);   // dQ staging boxes read back, per warp and iteration

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.S / 128;
  const int jt = blockIdx.z;            // KV tile; tile 0 has the most work and its CTAs are scheduled first
  const int g = blockIdx.x, b = blockIdx.y;
  const int heads = p.G * p.qpk;
  const int n_iter = (nq - jt) * p.qpk;  // (query tile, query head) pairs
  const int col_k = (g * (p.qpk + 2) + p.qpk) * HD, col_v = col_k + HD;
  const int kvrow = b * p.S + jt * 128;
  const uint64_t timeout = p.timeout_ns;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8); mbar_init(dq_full, 1); mbar_init(s_free, 8);
    *abort_flag = 0;
    *reads_done = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO); tma_prefetch_desc(&tmDQ); }
  if (warp == 1) { tmem_alloc(tmem_ptr_smem, 512); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dk = tmem_base + 256, tm_dv = tmem_base + 384;

  if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      mbar_expect_tx(kv_full, 2 * S_::TILE);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_2d(smem + S_::K_OFF + c * 16384, &tmQKV, kv_full, col_k + 64 * c, kvrow);
        tma_load_2d(smem + S_::V_OFF + c * 16384, &tmQKV, kv_full, col_v + 64 * c, kvrow);
      }
      for (int it = 0; it < n_iter && ok; ++it) {
        const int i = jt + it / p.qpk, jq = it % p.qpk;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
        const int qrow = b * p.S + i * 128;
        const int col_q = (g * (p.qpk + 2) + jq) * HD;
        const int col_do = (g * p.qpk + jq) * HD;
        mbar_expect_tx(qdo_full, 2 * S_::TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(smem + S_::Q_OFF + c * 16384, &tmQKV, qdo_full, col_q + 64 * c, qrow);
          tma_load_2d(smem + S_::DO_OFF + c * 16384, &tmDO, qdo_full, col_do + 64 * c, qrow);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) {}
        report_status(p.status, 0x411u);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = mbar_wait(kv_full, 0, abort_flag, timeout);
      const uint32_t idesc_s = umma_idesc(1, 0, 0, 128, 128);      // S, dP: K-major x K-major
      const uint32_t idesc_t = umma_idesc(1, 1, 1, 128, HD);       // dV, dK: A^T (MN-major) x MN-major
      const uint32_t idesc_q = umma_idesc(1, 0, 1, 128, HD);       // dQ: K-major x MN-major
      const uint32_t k_addr = smem_u32(smem + S_::K_OFF), v_addr = smem_u32(smem + S_::V_OFF);
      const uint32_t q_addr = smem_u32(smem + S_::Q_OFF), do_addr = smem_u32(smem + S_::DO_OFF);
      const uint32_t p_addr = smem_u32(smem + S_::P_OFF), ds_addr = smem_u32(smem + S_::DS_OFF);
      const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
      uint64_t w_qdo = 0, w_sfree = 0, w_pds = 0, t_mark = probe ? globaltimer_ns() : 0;
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (probe) t_mark = globaltimer_ns();
        if (!mbar_wait(qdo_full, ph, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const uint64_t now = globaltimer_ns(); w_qdo += now - t_mark; t_mark = now; }
        tcgen05_fence_after();
        // dP first: its TMEM columns are free already, while the S columns still hold the previous
        // iteration's dQ until the reduction warps have drained it
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_f16(tm_dp, umma_smem_desc(do_addr + off, 16, 1024), umma_smem_desc(v_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        if (probe) t_mark = globaltimer_ns();
        if (!mbar_wait(s_free, ph ^ 1, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const uint64_t now = globaltimer_ns(); w_sfree += now - t_mark; t_mark = now; }
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_f16(tm_s, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(sdp_full);
        if (probe) t_mark = globaltimer_ns();
        if (!mbar_wait(pds_full, ph, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const uint64_t now = globaltimer_ns(); w_pds += now - t_mark; t_mark = now; }
        tcgen05_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // reduction over the 128 query rows, 16 per step
          umma_f16(tm_dv, umma_smem_desc(p_addr + kk * 2048, 16384, 1024), umma_smem_desc(do_addr + kk * 2048, 16384, 1024),
                   idesc_t, (it | kk) != 0);
          umma_f16(tm_dk, umma_smem_desc(ds_addr + kk * 2048, 16384, 1024), umma_smem_desc(q_addr + kk * 2048, 16384, 1024),
                   idesc_t, (it | kk) != 0);
        }
        if (!AXB_DBG(p, 8)) umma_commit(qdo_empty);   // Q and dO are free once dV / dK are done: the next loads overlap dQ
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // reduction over the 128 KV rows
          umma_f16(tm_s, umma_smem_desc(ds_addr + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                   umma_smem_desc(k_addr + kk * 2048, 16384, 1024), idesc_q, kk != 0);
        }
        umma_commit(dq_full);
        if AXB_DBG(p, 8) umma_commit(qdo_empty);
      }
      if (probe) {
        volatile unsigned int* w = reinterpret_cast<volatile unsigned int*>(p.status);
        w[2] = static_cast<unsigned>(w_qdo); w[3] = static_cast<unsigned>(w_sfree); w[4] = static_cast<unsigned>(w_pds);
        w[7] = static_cast<unsigned>(n_iter);
      }
      if (!ok) report_status(p.status, 0x412u);
    }
  } else {
    // ---- 8 softmax / reduction warps: thread = (query row r, column half): two warps share each TMEM lane
    // quarter and split the 128 score columns (and the HD columns of dQ) between them
    const int q4 = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    uint8_t* p_row = smem + S_::P_OFF + (r >> 3) * 1024 + (r & 7) * 128;
    uint8_t* ds_row = smem + S_::DS_OFF + (r >> 3) * 1024 + (r & 7) * 128;
    bool ok = true;
    const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && warp == 2 && lane == 0;
    uint64_t w_sdp = 0, t_a = 0, w_dq = 0, t_b = 0, t_b1 = 0, t_b2 = 0, t_mark = 0;
    for (int it = 0; it < n_iter; ++it) {
      const uint32_t ph = it & 1;
      const int i = jt + it / p.qpk, jq = it % p.qpk;
      const int head = g * p.qpk + jq;
      const size_t srow = static_cast<size_t>(i) * 128 + r;   // query position of this thread's row
      if (probe) t_mark = globaltimer_ns();
      const float lse2 = p.lse[(static_cast<size_t>(b) * heads + head) * p.S + srow] * 1.4426950408889634f;
      const float dl = p.delta[(static_cast<size_t>(b) * heads + head) * p.S + srow];
      if (!mbar_wait(sdp_full, ph, abort_flag, timeout)) { ok = false; break; }
      if (probe) { const uint64_t now = globaltimer_ns(); w_sdp += now - t_mark; t_mark = now; }
      tcgen05_fence_after();
      const bool diag = (i == jt);
#pragma unroll 1
      for (int c = 2 * half; c < 2 * half + 2; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tm_s + lane_base + c * 32, sv);
        tmem_ld_32x32(tm_dp + lane_base + c * 32, dv);
        tmem_ld_wait();
        uint32_t pp[16], dd[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float p0 = AXB_DBG(p, 2) ? __uint_as_float(sv[2 * k]) : exp2f(__uint_as_float(sv[2 * k]) * p.scale_log2 - lse2);
          float p1 = AXB_DBG(p, 2) ? __uint_as_float(sv[2 * k + 1]) : exp2f(__uint_as_float(sv[2 * k + 1]) * p.scale_log2 - lse2);
          if (diag) {   // key position (column) beyond the query position (row) is masked
            if (c * 32 + 2 * k > r) p0 = 0.f;
            if (c * 32 + 2 * k + 1 > r) p1 = 0.f;
          }
          const float d0 = p0 * (__uint_as_float(dv[2 * k]) - dl) * p.scale;
          const float d1 = p1 * (__uint_as_float(dv[2 * k + 1]) - dl) * p.scale;
          const __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
          pp[k] = *reinterpret_cast<const uint32_t*>(&hp);
          dd[k] = *reinterpret_cast<const uint32_t*>(&hd);
        }
        if (it > 0 && c == 2 * half) {
          // the P / dS tiles still hold the previous iteration's dQ staging boxes until the copy engine has read
          // them: every warp waits for its own reductions' reads and counts itself, all wait for the eight
          // counts - here, after the first chunk's arithmetic, so that the wait is usually over already
          if (lane == 0) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __threadfence_block();
            atomicAdd(const_cast<int*>(reads_done), 1);
          }
          if (!wait_partner(reads_done, 8 * it, abort_flag, timeout)) ok = false;
        }
        const int blk = (c >> 1) * 16384;
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const int chunk = ((c & 1) * 4 + t) ^ (r & 7);
          *reinterpret_cast<uint4*>(p_row + blk + chunk * 16) = make_uint4(pp[4 * t], pp[4 * t + 1], pp[4 * t + 2], pp[4 * t + 3]);
          *reinterpret_cast<uint4*>(ds_row + blk + chunk * 16) = make_uint4(dd[4 * t], dd[4 * t + 1], dd[4 * t + 2], dd[4 * t + 3]);
        }
      }
      if (!ok) break;
      tcgen05_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      if (probe) { const uint64_t now = globaltimer_ns(); t_a += now - t_mark; t_mark = now; }
      // dQ partial of this (query tile, head): TMEM -> fp32 accumulator in global memory
      if (!mbar_wait(dq_full, ph, abort_flag, timeout)) { ok = false; break; }
      if (probe) { const uint64_t now = globaltimer_ns(); w_dq += now - t_mark; t_mark = now; }
      tcgen05_fence_after();
      // this warp's 32 rows x HD/2 columns: TMEM -> swizzled 32x32 fp32 boxes in shared memory -> one bulk
      // tensor reduce-add per box into the fp32 accumulator (16 copy-engine operations per tile in all)
      constexpr int NBOX = HD / 64;                 // boxes per warp
      uint8_t* wstage = smem + S_::P_OFF + (warp - 2) * (NBOX * S_::DQ_BOX_BYTES);
#pragma unroll 1
      for (int cc = 0; cc < NBOX; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32(tm_s + lane_base + (half * NBOX + cc) * 32, v);
        tmem_ld_wait();
        uint8_t* row = wstage + cc * S_::DQ_BOX_BYTES + lane * 128;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          *reinterpret_cast<uint4*>(row + ((k ^ (lane & 7)) * 16)) = make_uint4(v[4 * k], v[4 * k + 1], v[4 * k + 2], v[4 * k + 3]);
      }
      tcgen05_fence_before();
      if (probe) { const uint64_t now = globaltimer_ns(); t_b1 += now - t_mark; }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && !AXB_DBG(p, 1)) {
        const int y = b * p.S + i * 128 + q4 * 32;
#pragma unroll
        for (int cc = 0; cc < NBOX; ++cc) {
          const int x = head * HD + (half * NBOX + cc) * 32;
          asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                       ::"l"(reinterpret_cast<uint64_t>(&tmDQ)), "r"(x), "r"(y), "r"(smem_u32(wstage + cc * S_::DQ_BOX_BYTES))
                       : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        if (probe) { const uint64_t now = globaltimer_ns(); t_b2 += now - t_mark; }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      if (probe) { const uint64_t now = globaltimer_ns(); t_b += now - t_mark; t_mark = now; }
    }
    if (probe) {
      volatile unsigned int* w = reinterpret_cast<volatile unsigned int*>(p.status);
      w[8] = static_cast<unsigned>(w_sdp); w[9] = static_cast<unsigned>(t_a); w[10] = static_cast<unsigned>(w_dq);
      w[11] = static_cast<unsigned>(t_b); w[12] = static_cast<unsigned>(t_b1); w[13] = static_cast<unsigned>(t_b2);
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    // dK (column half 0) and dV (half 1) of this KV tile: every MMA has completed (last dq_full seen)
    if (ok) {
      fa_store_kv_grad<HD>(p, (half == 0 ? tm_dk : tm_dv) + lane_base, b, jt, g, r, half);
    } else if (lane == 0) {
      report_status(p.status, 0x414u);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row
__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                float* __restrict__ delta, int B, int S, int H, int D) {
  const long long rows = static_cast<long long>(B) * S * H;
  const int lane = threadIdx.x & 31;
  for (long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; row < rows;
       row += ((long long)gridDim.x * blockDim.x) >> 5) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(o + row * D);
    const __nv_bfloat162* c = reinterpret_cast<const __nv_bfloat162*>(d_o + row * D);
    float acc = 0.f;
    for (int i = lane; i < D / 2; i += 32) {
      const float2 x = __bfloat1622float2(a[i]), y = __bfloat1622float2(c[i]);
      acc += x.x * y.x + x.y * y.y;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
      const long long h = row % H, bs = row / H, s = bs % S, bb = bs / S;
      delta[(bb * H + h) * S + s] = acc;
    }
  }
}

template <int HD>
static int fa_bwd_launch(const CUtensorMap& tq, const CUtensorMap& td, const CUtensorMap& tdq, const FaBwdParams& p,
                         int device, cudaStream_t s) {
  using S_ = FaBwdSmem<HD>;
  static bool configured[64] = {false};
  auto kern = fa_bwd_kernel<HD>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S_::TOTAL));
    configured[device & 63] = true;
  }
  dim3 grid(p.G, p.B, p.S / 128);   // z (slowest) = KV tile: all CTAs with the most iterations are scheduled first
  kern<<<grid, FA_BWD_THREADS, S_::TOTAL, s>>>(tq, td, tdq, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace axb

// Backward of axb_flash_attn_fwd.  qkv [B,S,G,qpk+2,D], out / d_out [B,S,G*qpk,D] bf16, lse [B,G*qpk,S];
// delta [B,G*qpk,S] fp32 scratch; dq_acc [B,S,G*qpk,D] fp32, zero on entry, holds dQ on return;
// dqkv [B,S,G,qpk+2,D]: its K and V slots receive dK and dV (the Q slots are left to the caller).
extern "C" int axb_flash_attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
                                  float* dq_acc, void* dqkv, int B, int S, int G, int qpk, int D, float scale,
                                  int device, void* stream) {
  using namespace axb;
  if (D != 64 && D != 128) { set_error("flash attention: head_dim must be 64 or 128"); return -1; }
  if (S % 128) { set_error("flash attention: sequence length must be a multiple of 128"); return -1; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int H = G * qpk;
  const long long rows = static_cast<long long>(B) * S * H;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  const int blocks = static_cast<int>(rows / 8 < cap ? (rows / 8 < 1 ? 1 : rows / 8) : cap);
  fa_delta_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(d_out),
                                         delta, B, S, H, D);
  AXB_CUDA(cudaGetLastError());
  CUtensorMap tq, td, tdq;
  if (make_tmap_2d_16bit(&tq, qkv, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(G) * (qpk + 2) * D, 128, 0)) return -1;
  if (make_tmap_2d_16bit(&td, d_out, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(H) * D, 128, 0)) return -1;
  if (make_tmap_2d_f32(&tdq, dq_acc, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(H) * D, 32)) return -1;
  FaBwdParams p;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc; p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.B = B; p.S = S; p.G = G; p.qpk = qpk; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("flash attention: no status word"); return -1; }
  p.status = st; p.timeout_ns = wait_timeout_ns();
  p.debug = 0;
#ifdef AXB_ABLATION
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("AXB_FA_DEBUG"); dbg = e ? atoi(e) : 0; } p.debug = dbg; }
#endif
  if (D == 128) return fa_bwd_launch<128>(tq, td, tdq, p, device, s);
  return fa_bwd_launch<64>(tq, td, tdq, p, device, s);
}
