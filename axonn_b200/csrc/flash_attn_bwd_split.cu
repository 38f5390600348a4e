// Causal flash attention backward as two tcgen05 kernels without atomics (sm_100a), grouped-query aware.
//
// The one-kernel backward (flash_attn.cu) keeps dK and dV in tensor memory and has to push dQ partials through
// the score columns and a global fp32 accumulator, which serialises every step.  Here the work is split the way
// the forward kernel is organised - persistent CTAs, every probability / score-gradient tile goes from the
// softmax threads back into tensor memory as the A operand of the next MMA, nothing is staged in shared memory:
//
//   fa_bwd_dq_kernel   one 128-row query tile per work item, walks the key tiles up to the diagonal:
//                      S = Q K^T and dP = dO V^T (128 x 128 each) into tensor memory, the softmax threads read
//                      them into registers (the MMA warp then already issues the next tile's S and dP),
//                      dS = P (dP - delta) scale goes back as bf16 and dQ += dS K accumulates in tensor memory.
//                      dQ is written once, as bf16, into the packed gradient tensor.
//   fa_bwd_dkv_kernel  one 128-row key tile per work item, walks the query tiles from the diagonal down (and the
//                      query heads of the group) in steps of 64 queries: S^T = K Q^T and dP^T = V dO^T into
//                      double-buffered 64-column score buffers (a thread owns a key row), P^T and dS^T go back as
//                      bf16, dV += P^T dO and dK += dS^T Q accumulate in tensor memory; one MMA warp per
//                      accumulator.
//
// Both recompute S, so the pair does 7 MMA units per tile against 5 of the one-kernel form, but neither has a
// serial chain through shared memory, global reductions or the fp32 accumulator (no zero fill, no conversion).
// delta = rowsum(dO * O) comes from a small pre-kernel.  All waits are bounded.
#include <cstdlib>

#include "common.cuh"

namespace axb {

int make_tmap_2d_16bit(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, int dtype);
int sm_count(int device);

struct FaSplitParams {
  const float* lse;      // [B, heads, S], natural log
  const float* delta;    // [B, heads, S]
  __nv_bfloat16* dqkv;   // [B, S, G, qpk + 2, D]
  int B, S, G, qpk;
  float scale, scale_log2;
  unsigned int* status;
  unsigned long long timeout_ns;
  int debug;   // ablation builds only (-DAXB_ABLATION, read once from AXB_FA_DEBUG; otherwise 0 and compiled out): 4 phase timers
};

constexpr int FS_THREADS = 384;   // TMA warp, MMA warp(s), idle warps of the first warpgroup, 8 softmax warps

// delta[b, h, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (b, s, h) row
__global__ void fa_split_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
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

// ------------------------------------------------------------------------------------------------ dQ
template <int HD>
struct DqSmem {
  static constexpr int TILE = 128 * HD * 2;
  static constexpr int Q_OFF = 0, DO_OFF = TILE;
  // K is held from the step's S MMA until its dQ MMA, a whole step later, so it gets three stages; V is released
  // as soon as dP has completed and gets two (7 tiles = 224 KB at head_dim 128).
  static constexpr int K_OFF = 2 * TILE;           // 3 stages
  static constexpr int V_OFF = 5 * TILE;           // 2 stages
  static constexpr int BAR_OFF = 7 * TILE;
  static constexpr int NBARS = 2 + 6 + 4 + 4;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16 + 1024;
};

// Work item k of this CTA: query tiles sorted by decreasing length (tile i walks i + 1 key tiles), dealt to the
// persistent CTAs in a snake.
struct DqItem { int i, head, b; };
__device__ __forceinline__ bool dq_item(const FaSplitParams& p, int k, DqItem& w) {
  const int G = gridDim.x, c = blockIdx.x;
  const int heads = p.G * p.qpk, bh = p.B * heads, nq = p.S / 128;
  const int idx = k * G + ((k & 1) ? G - 1 - c : c);
  if (idx >= bh * nq) return false;
  w.i = nq - 1 - idx / bh;
  const int rem = idx % bh;
  w.head = rem % heads;
  w.b = rem / heads;
  return true;
}

template <int HD>
__global__ void __launch_bounds__(FS_THREADS, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const FaSplitParams p) {
  using S_ = DqSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_::BAR_OFF);
  uint64_t* q_full = bars;          // Q and dO of the item
  uint64_t* q_empty = bars + 1;
  uint64_t* k_full = bars + 2;      // [3]
  uint64_t* k_empty = bars + 5;     // [3]
  uint64_t* v_full = bars + 8;      // [2]
  uint64_t* v_empty = bars + 10;    // [2]
  uint64_t* sdp_full = bars + 12;   // S and dP of a step are complete
  uint64_t* sdp_free = bars + 13;   // ... and held in registers: their columns may be overwritten
  uint64_t* ds_full = bars + 14;    // dS of a step is in tensor memory
  uint64_t* dq_done = bars + 15;    // the step's dQ MMA has completed (dS may be overwritten; at the end: dQ final)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + S_::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t timeout = p.timeout_ns;
  const int heads = p.G * p.qpk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 2); }   // released by both MMA warps
    for (int i = 0; i < 2; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(sdp_full, 1); mbar_init(sdp_free, 8); mbar_init(ds_full, 8); mbar_init(dq_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO); }
  if (warp == 1) { tmem_alloc(tmem_ptr_smem, 512); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // columns: S [0,128), dP [128,256), dS (bf16, 128 keys) [256,320), dQ [384,384+HD)
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_ds = tmem_base + 256, tm_dq = tmem_base + 384;

  if (warp < 4) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
   if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      uint32_t kvc = 0;
      DqItem w;
      for (int it = 0; ok && dq_item(p, it, w); ++it) {
        const int g = w.head / p.qpk, jq = w.head % p.qpk;
        const int col_q = (g * (p.qpk + 2) + jq) * HD;
        const int col_k = (g * (p.qpk + 2) + p.qpk) * HD;
        const int col_v = col_k + HD;
        const int row0 = w.b * p.S + w.i * 128;
        if (!mbar_wait(q_empty, (it & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
        mbar_expect_tx(q_full, 2 * S_::TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(smem + S_::Q_OFF + c * 16384, &tmQKV, q_full, col_q + 64 * c, row0);
          tma_load_2d(smem + S_::DO_OFF + c * 16384, &tmDO, q_full, w.head * HD + 64 * c, row0);
        }
        for (int j = 0; j <= w.i && ok; ++j, ++kvc) {
          const int st = kvc % 3;
          const uint32_t ph = (kvc / 3) & 1;
          const int krow = w.b * p.S + j * 128;
          if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, timeout)) { ok = false; break; }
          mbar_expect_tx(&k_full[st], S_::TILE);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + S_::K_OFF + st * S_::TILE + c * 16384, &tmQKV, &k_full[st], col_k + 64 * c, krow);
          if (!mbar_wait(&v_empty[kvc & 1], ((kvc >> 1) & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
          mbar_expect_tx(&v_full[kvc & 1], S_::TILE);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c)
            tma_load_2d(smem + S_::V_OFF + (kvc & 1) * S_::TILE + c * 16384, &tmQKV, &v_full[kvc & 1], col_v + 64 * c, krow);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();     // give in-flight copies time to land before the CTA exits
        while (globaltimer_ns() - t0 < 200000ull) {}
        report_status(p.status, 0x421u);
      }
    }
   } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA warp 1: S = Q K^T and dP = dO V^T
    if (elect_one()) {
      bool ok = true;
      const uint32_t idesc_s = umma_idesc(1, 0, 0, 128, 128);
      const uint64_t qd = umma_smem_desc(smem_u32(smem + S_::Q_OFF), 16, 1024);
      const uint64_t dod = umma_smem_desc(smem_u32(smem + S_::DO_OFF), 16, 1024);
      auto issue_sdp = [&](uint32_t kv) {
        const uint64_t kd = umma_smem_desc(smem_u32(smem + S_::K_OFF + (kv % 3) * S_::TILE), 16, 1024);
        const uint64_t vd = umma_smem_desc(smem_u32(smem + S_::V_OFF + (kv & 1) * S_::TILE), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_f16(tm_s, qd + off, kd + off, idesc_s, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_f16(tm_dp, dod + off, vd + off, idesc_s, kk != 0 ? 1u : 0u);
        }
      };
      uint32_t kvc = 0, c = 0;     // key tiles and steps of earlier items (ring stages, barrier phases)
      const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0;
      long long pw_free = 0, pw_kv = 0, p_mark = 0, p_t0 = probe ? clock64() : 0;
      DqItem w;
      for (int it = 0; ok && dq_item(p, it, w); ++it) {
        const int n = w.i + 1;
        if (!mbar_wait(q_full, it & 1, abort_flag, timeout)) { ok = false; break; }
        for (int j = 0; j < n && ok; ++j, ++c) {
          const uint32_t kv = kvc + j;
          // S and dP columns are free once the softmax threads hold the previous step's tile in registers
          if (probe) p_mark = clock64();
          if (c >= 1 && !mbar_wait(sdp_free, (c - 1) & 1, abort_flag, timeout)) { ok = false; break; }
          if (probe) { const long long now = clock64(); pw_free += now - p_mark; p_mark = now; }
          if (!mbar_wait(&k_full[kv % 3], (kv / 3) & 1, abort_flag, timeout) ||
              !mbar_wait(&v_full[kv & 1], (kv >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          if (probe) pw_kv += clock64() - p_mark;
          tcgen05_fence_after();
          issue_sdp(kv);
          umma_commit(sdp_full);
          umma_commit(&v_empty[kv & 1]);
          umma_commit(&k_empty[kv % 3]);              // first of the two releases of this K tile
          if (j + 1 == n) umma_commit(q_empty);       // the item's last reads of Q and dO
        }
        kvc += n;
      }
      if (probe) {
        volatile unsigned int* wd = reinterpret_cast<volatile unsigned int*>(p.status);
        wd[12] = static_cast<unsigned>(pw_free); wd[13] = static_cast<unsigned>(pw_kv);
        wd[15] = static_cast<unsigned>(clock64() - p_t0);
      }
      if (!ok) report_status(p.status, 0x422u);
    }
   } else if (warp == 2) {
    // ------------------------------------------------------------------ MMA warp 2: dQ += dS K
    if (elect_one()) {
      bool ok = true;
      const uint32_t idesc_dq = umma_idesc(1, 0, 1, 128, HD);
      uint32_t kvc = 0, c = 0;
      const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0;
      long long pw_ds = 0, p_mark = 0;
      DqItem w;
      for (int it = 0; ok && dq_item(p, it, w); ++it) {
        const int n = w.i + 1;
        for (int j = 0; j < n && ok; ++j, ++c) {
          const uint32_t kv = kvc + j;
          if (probe) p_mark = clock64();
          // dS of the step is in tensor memory (the softmax threads saw S of this K tile, so the tile is loaded)
          if (!mbar_wait(ds_full, c & 1, abort_flag, timeout)) { ok = false; break; }
          if (probe) pw_ds += clock64() - p_mark;
          tcgen05_fence_after();
          // K as the B operand of dQ = dS K: keys are the reduction dimension, head_dim is contiguous (MN-major):
          // 64-wide column chunks 16 KB apart (leading), 8-row groups 1 KB apart (stride)
          const uint64_t kmn = umma_smem_desc(smem_u32(smem + S_::K_OFF + (kv % 3) * S_::TILE), 16384, 1024);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_f16_ts(tm_dq, tm_ds + kk * 8, kmn + ((kk * 2048) >> 4), idesc_dq, (j == 0 && kk == 0) ? 0u : 1u);
          umma_commit(dq_done);
          umma_commit(&k_empty[kv % 3]);              // second release of this K tile
        }
        kvc += n;
      }
      if (probe) reinterpret_cast<volatile unsigned int*>(p.status)[14] = static_cast<unsigned>(pw_ds);
      if (!ok) report_status(p.status, 0x424u);
    }
   }
  } else {
    // ------------------------------------------------------------------ P, dS: thread = (query row, key half)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int q4 = warp & 3;
    const int half = (warp - 4) >> 2;
    const int r = q4 * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    uint32_t c = 0;
    const bool probe = AXB_DBG(p, 4) && blockIdx.x == 0 && warp == 4 && lane == 0;
    long long pw_s = 0, pt_ld = 0, pt_cmp = 0, pw_dq = 0, pt_st = 0, p_mark = 0;
    DqItem w;
    for (int it = 0; ok && dq_item(p, it, w); ++it) {
      const int n = w.i + 1;
      const size_t srow = static_cast<size_t>(w.i) * 128 + r;
      const float lse2 = p.lse[(static_cast<size_t>(w.b) * heads + w.head) * p.S + srow] * 1.4426950408889634f;
      const float dl = p.delta[(static_cast<size_t>(w.b) * heads + w.head) * p.S + srow];
      for (int j = 0; j < n; ++j, ++c) {
        if (probe) p_mark = clock64();
        if (!mbar_wait(sdp_full, c & 1, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const long long now = clock64(); pw_s += now - p_mark; p_mark = now; }
        tcgen05_fence_after();
        uint32_t sv[64], dv[64];
        tmem_ld_32x32(tm_s + lane_base + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32(tm_s + lane_base + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_32x32(tm_dp + lane_base + half * 64, *reinterpret_cast<uint32_t(*)[32]>(&dv[0]));
        tmem_ld_32x32(tm_dp + lane_base + half * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&dv[32]));
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_free);          // the MMA warp may issue the next tile's S and dP
        if (probe) { const long long now = clock64(); pt_ld += now - p_mark; p_mark = now; }
        const bool diag = (j == w.i);
        uint32_t packed[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float p0 = exp2f(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -lse2));
          float p1 = exp2f(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -lse2));
          if (diag) {
            if (half * 64 + 2 * i > r) p0 = 0.f;
            if (half * 64 + 2 * i + 1 > r) p1 = 0.f;
          }
          const float d0 = p0 * (__uint_as_float(dv[2 * i]) - dl) * p.scale;
          const float d1 = p1 * (__uint_as_float(dv[2 * i + 1]) - dl) * p.scale;
          const __nv_bfloat162 h = __floats2bfloat162_rn(d0, d1);
          packed[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        // the previous step's dQ MMA (of this or of the previous item) has read its dS: every phase is observed
        if (probe) { const long long now = clock64(); pt_cmp += now - p_mark; p_mark = now; }
        if (c >= 1 && !mbar_wait(dq_done, (c - 1) & 1, abort_flag, timeout)) { ok = false; break; }
        if (probe) { const long long now = clock64(); pw_dq += now - p_mark; p_mark = now; }
        tmem_st_32x32(tm_ds + lane_base + half * 32, packed);
        tmem_st_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
        if (probe) { const long long now = clock64(); pt_st += now - p_mark; p_mark = now; }
      }
      if (!ok || !mbar_wait(dq_done, (c - 1) & 1, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      // dQ row r, columns [half * HD/2, +HD/2) -> packed gradient tensor, query slot of this head
      const int g = w.head / p.qpk, jq = w.head % p.qpk;
      const size_t pos = static_cast<size_t>(w.b) * p.S + srow;
      __nv_bfloat16* dst = p.dqkv + ((pos * p.G + g) * (p.qpk + 2) + jq) * HD + half * (HD / 2);
#pragma unroll
      for (int cc = 0; cc < HD / 64; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32(tm_dq + lane_base + half * (HD / 2) + cc * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t wv[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[t * 8 + 2 * i]), __uint_as_float(v[t * 8 + 2 * i + 1]));
            wv[i] = *reinterpret_cast<const uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + cc * 32 + t * 8) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
      // the next item's first dQ MMA overwrites these columns; it waits for ds_full, which this thread arrives on
      // after these reads
      tcgen05_fence_before();
    }
    if (probe) {
      volatile unsigned int* wd = reinterpret_cast<volatile unsigned int*>(p.status);
      wd[6] = c; wd[7] = static_cast<unsigned>(pw_s); wd[8] = static_cast<unsigned>(pt_ld); wd[9] = static_cast<unsigned>(pt_cmp);
      wd[10] = static_cast<unsigned>(pw_dq); wd[11] = static_cast<unsigned>(pt_st);
    }
    if (!ok && lane == 0) report_status(p.status, 0x423u);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int HD>
static int dq_launch(const CUtensorMap& tq, const CUtensorMap& td, const FaSplitParams& p, int device, cudaStream_t s) {
  using S_ = DqSmem<HD>;
  static bool configured[64] = {false};
  auto kern = fa_bwd_dq_kernel<HD>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S_::TOTAL));
    configured[device & 63] = true;
  }
  const long long items = static_cast<long long>(p.B) * p.G * p.qpk * (p.S / 128);
  const int sms = sm_count(device);
  kern<<<static_cast<int>(items < sms ? items : sms), FS_THREADS, S_::TOTAL, s>>>(tq, td, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------ dK, dV
template <int HD>
struct DkvSmem {
  static constexpr int TILE = 128 * HD * 2;
  static constexpr int K_OFF = 0, V_OFF = TILE;
  static constexpr int Q_OFF = 2 * TILE;           // 2 stages
  static constexpr int DO_OFF = 4 * TILE;          // 2 stages
  static constexpr int LSE_OFF = 6 * TILE;         // [2 stages][lse, delta][128] fp32
  static constexpr int BAR_OFF = LSE_OFF + 2048;
  static constexpr int NBARS = 2 + 4 + 2 + 2 + 1;
  static constexpr int TOTAL = BAR_OFF + NBARS * 8 + 16 + 1024;
};

// Work item k of this CTA: key tiles sorted by decreasing length (tile jt is visited by (nq - jt) * qpk query
// tiles), dealt to the persistent CTAs in a snake.
struct DkvItem { int jt, g, b; };
__device__ __forceinline__ bool dkv_item(const FaSplitParams& p, int k, DkvItem& w) {
  const int G = gridDim.x, c = blockIdx.x;
  const int bg = p.B * p.G, nq = p.S / 128;
  const int idx = k * G + ((k & 1) ? G - 1 - c : c);
  if (idx >= bg * nq) return false;
  w.jt = idx / bg;
  const int rem = idx % bg;
  w.g = rem % p.G;
  w.b = rem / p.G;
  return true;
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      : : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// global -> shared bulk copy (16-byte aligned, size a multiple of 16) that completes on an mbarrier
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int HD>
__global__ void __launch_bounds__(FS_THREADS, 1)
fa_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQKV, const __grid_constant__ CUtensorMap tmDO, const FaSplitParams p) {
  using S_ = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_::BAR_OFF);
  uint64_t* kv_full = bars;          // K and V of the item
  uint64_t* kv_empty = bars + 1;     // both MMA warps are done with them
  uint64_t* qdo_full = bars + 2;     // [stage]: Q, dO, lse, delta of a query tile
  uint64_t* qdo_empty = bars + 4;    // [stage]: 2 MMA warps + 8 softmax warps
  uint64_t* sdp_full = bars + 6;     // [score buffer]: S^T and dP^T of a step (one arrival per MMA warp)
  uint64_t* pds_full = bars + 8;     // [score buffer]: P^T and dS^T of a step are in tensor memory
  uint64_t* acc_done = bars + 10;    // dK and dV of the item are final (one arrival per MMA warp)
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(bars + S_::NBARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  float* lse_s = reinterpret_cast<float*>(smem + S_::LSE_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint64_t timeout = p.timeout_ns;
  const int heads = p.G * p.qpk, nq = p.S / 128;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(kv_empty, 2); mbar_init(acc_done, 2);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 10);
      mbar_init(&sdp_full[i], 2); mbar_init(&pds_full[i], 8);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmQKV); tma_prefetch_desc(&tmDO); }
  if (warp == 1) { tmem_alloc(tmem_ptr_smem, 512); tmem_relinquish(); }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  // columns: S^T buffers [0,64) [64,128), dP^T buffers [128,192) [192,256) (P^T / dS^T of a buffer's queries
  // [0,32) in its columns [0,16), of queries [32,64) in [32,48)), dK [256,256+HD), dV [384,384+HD)

  if (warp < 4) {
   asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
   if (warp == 0) {
    if (elect_one()) {
      bool ok = true;
      uint32_t tq = 0;                 // query tiles loaded so far: ring stage and phase
      DkvItem w;
      for (int it = 0; ok && dkv_item(p, it, w); ++it) {
        const int col_k = (w.g * (p.qpk + 2) + p.qpk) * HD;
        const int krow = w.b * p.S + w.jt * 128;
        if (!mbar_wait(kv_empty, (it & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
        mbar_expect_tx(kv_full, 2 * S_::TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_2d(smem + S_::K_OFF + c * 16384, &tmQKV, kv_full, col_k + 64 * c, krow);
          tma_load_2d(smem + S_::V_OFF + c * 16384, &tmQKV, kv_full, col_k + HD + 64 * c, krow);
        }
        const int per_head = nq - w.jt;
        for (int t = 0; t < per_head * p.qpk && ok; ++t, ++tq) {
          const int jq = t / per_head, i = w.jt + t % per_head;
          const int head = w.g * p.qpk + jq;
          const int st = tq & 1;
          const int row0 = w.b * p.S + i * 128;
          if (!mbar_wait(&qdo_empty[st], ((tq >> 1) & 1) ^ 1, abort_flag, timeout)) { ok = false; break; }
          mbar_expect_tx(&qdo_full[st], 2 * S_::TILE + 1024);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c) {
            tma_load_2d(smem + S_::Q_OFF + st * S_::TILE + c * 16384, &tmQKV, &qdo_full[st],
                        (w.g * (p.qpk + 2) + jq) * HD + 64 * c, row0);
            tma_load_2d(smem + S_::DO_OFF + st * S_::TILE + c * 16384, &tmDO, &qdo_full[st], head * HD + 64 * c, row0);
          }
          const size_t vec = (static_cast<size_t>(w.b) * heads + head) * p.S + static_cast<size_t>(i) * 128;
          bulk_load_1d(lse_s + st * 256, p.lse + vec, 512, &qdo_full[st]);
          bulk_load_1d(lse_s + st * 256 + 128, p.delta + vec, 512, &qdo_full[st]);
        }
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();     // give in-flight copies time to land before the CTA exits
        while (globaltimer_ns() - t0 < 200000ull) {}
        report_status(p.status, 0x431u);
      }
    }
   } else if (warp <= 2) {
    // ------------------------------------------------------------------ MMA: warp 1 = S^T and dV, warp 2 = dP^T and dK
    if (elect_one()) {
      bool ok = true;
      const int which = warp - 1;                              // 0: scores / dV (operands K, Q | P^T, dO); 1: dP^T / dK (V, dO | dS^T, Q)
      const uint32_t idesc_t = umma_idesc(1, 0, 0, 128, 64);
      const uint32_t idesc_acc = umma_idesc(1, 0, 1, 128, HD);
      const uint32_t t_buf = tmem_base + which * 128;          // this warp's two 64-column buffers
      const uint32_t t_acc = tmem_base + (which ? 256 : 384);  // dK | dV
      const uint64_t ad = umma_smem_desc(smem_u32(smem + (which ? S_::V_OFF : S_::K_OFF)), 16, 1024);
      const int b_off = which ? S_::DO_OFF : S_::Q_OFF;        // B operand of the transposed score MMA
      const int m_off = which ? S_::Q_OFF : S_::DO_OFF;        // B operand (MN-major) of the accumulator MMA
      // scores of step s = (query tile, half hq): 64 query rows of the tile in ring stage st, into buffer hq
      auto issue_t = [&](int st, int hq) {
        const uint64_t bd = umma_smem_desc(smem_u32(smem + b_off + st * S_::TILE) + hq * 8192, 16, 1024);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t off = ((kk >> 2) * 16384 + (kk & 3) * 32) >> 4;
          umma_f16(t_buf + hq * 64, ad + off, bd + off, idesc_t, kk != 0 ? 1u : 0u);
        }
      };
      auto issue_acc = [&](int st, int hq, bool first) {
        // dO (or Q) as an MN-major B operand: the 64 queries of the half step are the reduction dimension
        const uint64_t md = umma_smem_desc(smem_u32(smem + m_off + st * S_::TILE) + hq * 8192, 16384, 1024);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          // P^T / dS^T of queries [32 h, 32 h + 32) sit in the first 16 of the 32 columns that thread half h read
          umma_f16_ts(t_acc, t_buf + hq * 64 + (kk >> 1) * 32 + (kk & 1) * 8, md + ((kk * 2048) >> 4), idesc_acc,
                      (first && kk == 0) ? 0u : 1u);
      };
      uint32_t tq = 0, c = 0;          // query tiles and steps of earlier items
      DkvItem w;
      for (int it = 0; ok && dkv_item(p, it, w); ++it) {
        const int ns = 2 * (nq - w.jt) * p.qpk;
        if (!mbar_wait(kv_full, it & 1, abort_flag, timeout) ||
            !mbar_wait(&qdo_full[tq & 1], (tq >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        // both buffers are free: the previous item's accumulator MMAs, which read them, were issued earlier
        issue_t(tq & 1, 0); umma_commit(&sdp_full[0]);
        issue_t(tq & 1, 1); umma_commit(&sdp_full[1]);
        for (int s = 0; s < ns && ok; ++s, ++c) {
          const uint32_t tile = tq + (s >> 1);
          const int hq = s & 1;
          if (!mbar_wait(&pds_full[hq], (c >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
          tcgen05_fence_after();
          issue_acc(tile & 1, hq, s == 0);
          if (hq == 1) umma_commit(&qdo_empty[tile & 1]);        // this warp's last read of the tile
          if (s + 2 < ns) {
            const uint32_t tn = tile + 1;
            if (!mbar_wait(&qdo_full[tn & 1], (tn >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
            tcgen05_fence_after();
            issue_t(tn & 1, hq);
            umma_commit(&sdp_full[hq]);
          }
        }
        umma_commit(acc_done);
        umma_commit(kv_empty);
        tq += ns >> 1;
      }
      if (!ok) report_status(p.status, 0x432u);
    }
   }
  } else {
    // ------------------------------------------------------------------ P^T, dS^T: thread = (key row, 32 of the step's 64 queries)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
    const int q4 = warp & 3;
    const int half = (warp - 4) >> 2;
    const int r = q4 * 32 + lane;                     // key row inside the tile
    const uint32_t lane_base = static_cast<uint32_t>(q4 * 32) << 16;
    bool ok = true;
    uint32_t tq = 0, c = 0;
    DkvItem w;
    for (int it = 0; ok && dkv_item(p, it, w); ++it) {
      const int per_head = nq - w.jt;
      const int ns = 2 * per_head * p.qpk;
      for (int s = 0; s < ns; ++s, ++c) {
        const uint32_t tile = tq + (s >> 1);
        const int hq = s & 1, st = tile & 1;
        const int i = w.jt + (s >> 1) % per_head;
        // lse / delta of the tile arrive with its Q and dO
        if (hq == 0 && !mbar_wait(&qdo_full[st], (tile >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        if (!mbar_wait(&sdp_full[hq], (c >> 1) & 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        uint32_t sv[32], dv[32];
        tmem_ld_32x32(tmem_base + lane_base + hq * 64 + half * 32, sv);
        tmem_ld_32x32(tmem_base + lane_base + 128 + hq * 64 + half * 32, dv);
        tmem_ld_wait();
        const int qc0 = hq * 64 + half * 32;           // first query column of this thread inside the tile
        const float4* lv = reinterpret_cast<const float4*>(lse_s + st * 256 + qc0);
        const float4* dvv = reinterpret_cast<const float4*>(lse_s + st * 256 + 128 + qc0);
        const bool diag = (i == w.jt);
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int v4 = 0; v4 < 8; ++v4) {
          const float4 l4 = lv[v4], d4 = dvv[v4];
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
          float pr[4], dsr[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = v4 * 4 + e;
            float pv = exp2f(fmaf(__uint_as_float(sv[col]), p.scale_log2, -ls[e] * 1.4426950408889634f));
            if (diag && r > qc0 + col) pv = 0.f;        // the key lies after the query
            pr[e] = pv;
            dsr[e] = pv * (__uint_as_float(dv[col]) - ds[e]) * p.scale;
          }
          const __nv_bfloat162 a0 = __floats2bfloat162_rn(pr[0], pr[1]), a1 = __floats2bfloat162_rn(pr[2], pr[3]);
          const __nv_bfloat162 b0 = __floats2bfloat162_rn(dsr[0], dsr[1]), b1 = __floats2bfloat162_rn(dsr[2], dsr[3]);
          pp[v4 * 2] = *reinterpret_cast<const uint32_t*>(&a0); pp[v4 * 2 + 1] = *reinterpret_cast<const uint32_t*>(&a1);
          pd[v4 * 2] = *reinterpret_cast<const uint32_t*>(&b0); pd[v4 * 2 + 1] = *reinterpret_cast<const uint32_t*>(&b1);
        }
        // into this thread's own score columns: the other half's thread of the row may not have read its scores yet
        tmem_st_32x16(tmem_base + lane_base + hq * 64 + half * 32, pp);
        tmem_st_32x16(tmem_base + lane_base + 128 + hq * 64 + half * 32, pd);
        tmem_st_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&pds_full[hq]);
          if (hq == 1) mbar_arrive(&qdo_empty[st]);      // lse / delta of the tile have been read
        }
      }
      if (!ok || !mbar_wait(acc_done, it & 1, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      // half 0 stores dK row r, half 1 stores dV row r into the key / value slots of the packed gradient tensor
      const size_t kvpos = static_cast<size_t>(w.b) * p.S + w.jt * 128 + r;
      __nv_bfloat16* dst = p.dqkv + ((kvpos * p.G + w.g) * (p.qpk + 2) + p.qpk + half) * HD;
      const uint32_t src = tmem_base + lane_base + (half ? 384 : 256);
#pragma unroll
      for (int cc = 0; cc < HD / 32; ++cc) {
        uint32_t v[32];
        tmem_ld_32x32(src + cc * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint32_t wv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[t * 8 + 2 * e]), __uint_as_float(v[t * 8 + 2 * e + 1]));
            wv[e] = *reinterpret_cast<const uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(dst + cc * 32 + t * 8) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        }
      }
      // the next item's first accumulator MMAs overwrite dK / dV; they wait for pds_full, on which this thread
      // arrives after these reads
      tcgen05_fence_before();
      tq += ns >> 1;
    }
    if (!ok && lane == 0) report_status(p.status, 0x433u);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int HD>
static int dkv_launch(const CUtensorMap& tq, const CUtensorMap& td, const FaSplitParams& p, int device, cudaStream_t s) {
  using S_ = DkvSmem<HD>;
  static bool configured[64] = {false};
  auto kern = fa_bwd_dkv_kernel<HD>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S_::TOTAL));
    configured[device & 63] = true;
  }
  const long long items = static_cast<long long>(p.B) * p.G * (p.S / 128);
  const int sms = sm_count(device);
  kern<<<static_cast<int>(items < sms ? items : sms), FS_THREADS, S_::TOTAL, s>>>(tq, td, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace axb

// which: bit 0 = dQ kernel (writes the query slots of dqkv), bit 1 = dK / dV kernel (writes the key and value slots).
// qkv [B,S,G,qpk+2,D], out / d_out [B,S,G*qpk,D] bf16; lse [B,G*qpk,S]; delta [B,G*qpk,S] fp32 scratch.
extern "C" int axb_flash_attn_bwd_split(const void* qkv, const void* out, const void* d_out, const float* lse,
                                        float* delta, void* dqkv, int B, int S, int G, int qpk, int D, float scale,
                                        int which, int device, void* stream) {
  using namespace axb;
  if (D != 64 && D != 128) { set_error("flash attention: head_dim must be 64 or 128"); return -1; }
  if (S % 128) { set_error("flash attention: sequence length must be a multiple of 128"); return -1; }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int H = G * qpk;
  const long long rows = static_cast<long long>(B) * S * H;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  const int blocks = static_cast<int>(rows / 8 < cap ? (rows / 8 < 1 ? 1 : rows / 8) : cap);
  fa_split_delta_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(out),
                                               static_cast<const __nv_bfloat16*>(d_out), delta, B, S, H, D);
  AXB_CUDA(cudaGetLastError());
  CUtensorMap tq, td;
  if (make_tmap_2d_16bit(&tq, qkv, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(G) * (qpk + 2) * D, 128, 0)) return -1;
  if (make_tmap_2d_16bit(&td, d_out, static_cast<uint64_t>(B) * S, static_cast<uint64_t>(H) * D, 128, 0)) return -1;
  FaSplitParams p;
  p.lse = lse; p.delta = delta; p.dqkv = static_cast<__nv_bfloat16*>(dqkv);
  p.B = B; p.S = S; p.G = G; p.qpk = qpk; p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  unsigned int* st = nullptr;
  if (!device_status_word(device, &st)) { set_error("flash attention: no status word"); return -1; }
  p.status = st; p.timeout_ns = wait_timeout_ns();
  p.debug = 0;
#ifdef AXB_ABLATION
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("AXB_FA_DEBUG"); dbg = e ? atoi(e) : 0; } p.debug = dbg; }
#endif
  if (which & 2) {
    if (D == 128) { if (dkv_launch<128>(tq, td, p, device, s)) return -1; }
    else          { if (dkv_launch<64>(tq, td, p, device, s)) return -1; }
  }
  if (which & 1) {
    if (D == 128) { if (dq_launch<128>(tq, td, p, device, s)) return -1; }
    else          { if (dq_launch<64>(tq, td, p, device, s)) return -1; }
  }
  return 0;
}
