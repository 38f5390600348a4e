// bf16/fp16 GEMM on 5th-generation tensor cores (tcgen05) for sm_100a.
//
// Two kernels share the pipeline below.
//
// gemm_tcgen05_kernel: one persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: streams 128xBK (A) and BNxBK (B) tiles into a
//               multi-stage shared-memory ring (128-byte swizzle, mbarrier
//               transaction counts);
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma (M=128, N=BN,
//               K=16) from shared-memory descriptors into one of two TMEM
//               accumulators (2 x BN fp32 columns), and commits to mbarriers
//               to recycle smem stages and to publish finished accumulators;
//   warps 2-5   epilogue: tcgen05.ld the accumulator (each warp its 32 TMEM
//               lanes), apply bias / GELU / accumulate, convert and store; runs
//               concurrently with the next tile's main loop thanks to the
//               double-buffered accumulator;
//   warps 6-15  only active when the GEMM carries an all-reduce / reduce-scatter
//               over peer memory: eight reducer warps, a flagger and a watcher
//               (described at reducer_warps / watcher_thread below).
//
// gemm_pair_kernel: clusters of two CTAs (tcgen05.mma.cta_group::2) compute
// 256x256 tiles for plain GEMMs; warps 0-5 as above in each CTA, MMAs issued
// by the even CTA for both.
//
// Operand layouts: each of A and B is either K-major (row = M/N index, K
// contiguous) or MN-major (row = K index, M/N contiguous); both are expressed
// to the tensor core through the majorness bits of the instruction descriptor
// and the matching canonical shared-memory layout, so forward (A Bt), input
// gradient (A B) and weight gradient (At B) need no transposed copies.
//
// Every wait is bounded; on expiry the CTA raises an abort flag, records the
// reason in the device status word, drains its TMA copies, frees TMEM and
// returns.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace axb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int REDUCER_THREADS = 256;
constexpr int GEMM_THREADS = 192 + REDUCER_THREADS + 64;   // TMA warp, MMA warp, 4 epilogue warps, 8 reducer warps, flagger warp, watcher warp
constexpr int FLAGGER_WARP = (192 + REDUCER_THREADS) / 32;
constexpr int WATCHER_WARP = FLAGGER_WARP + 1;

struct GemmParams {
  void* C;
  const void* bias;
  void* aux;
  int M, N, K;
  int tiles_m, tiles_n;
  int out_dtype;  // 0 bf16, 1 fp16, 2 fp32
  int in_dtype;   // 0 bf16, 1 fp16
  int epilogue;
  int accumulate;
  unsigned int* status;
  unsigned long long timeout_ns;
  AxbArCtx ar;  // ar.n <= 1: plain GEMM; otherwise the epilogue all-reduces C over ar.n ranks
  AxbAgCtx ag;  // ag.n <= 1: B is complete; otherwise B's row blocks are gathered from the peers in-kernel
  int tn_offset;  // rotation of the N-tile order (all-gather mode: tiles of the local shard first)
  int kb_offset;  // rotation of the K-block order (all-gather mode, B rows = K: local shard first)
  int gemm_ctas;  // number of CTAs in the grid (every CTA computes tiles and, in the fused modes, reduces them)
  int pair;       // 1: CTA pairs (clusters of two) compute 256 x BN tiles, each CTA owning 128 rows of them
  int flag_batch; // tiles whose partial-arrival flags share one system-scope fence (fused all-reduce / reduce-scatter)
  // Batched mode of the plain CTA-pair kernel: nb independent M x N x K problems of one shape in one launch.
  // Problem e reads and writes its operands e * {a,b,c}_batch_rows rows further down the (stacked) 2-D arrays.
  int nb, a_batch_rows, b_batch_rows, c_batch_rows;
  // Row mask of the batched mode (capacity buffers of a mixture-of-experts layer): the masked dimension of
  // problem e (mask_mode 1: the M rows; 2: the K rows of layout 2) consists of nseg segments of seg_rows rows of
  // which only the first seg_counts[e * nseg + s] hold data, the rest being zero.  Tiles (mode 1) or K blocks
  // (mode 2) without a data row are not computed; a skipped tile is stored as zeros.
  const int* seg_counts;
  int seg_rows, nseg, mask_mode;
  int debug;      // ablation builds only (-DAXB_ABLATION, then read once from AXB_AR_DEBUG; otherwise 0 and every branch on it is compiled out): 1 no flagger fence, 2 no peer stores, 4 no reducer fence, 8 no reduction, 16 no partial stores, 128 register-path reducer instead of the shared-memory ring
};

// Time that the fused kernels spent stalled on peers since the last reset, in units of ns / 1024: every CTA of a
// communicating launch adds (its wait for weight shards + the tail after its last tile's epilogue, in which only
// the reduction of peer data and the end-of-call handshake remain) * 1024 / number of CTAs, i.e. each launch
// contributes the mean over its CTAs.  Read by axb_comm_stall_ms.
static __device__ unsigned long long g_comm_stall;

template <int BN, bool PAIR = false>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BK * 2;   // a CTA of a pair stages its half of the B tile
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256 && !PAIR) ? 4 : 6;
  // Two-rank all-reduce with 128x256 tiles: the operand ring runs with RING_STAGES stages and the space
  // behind them stages the inbox slots that the reducer warps sum (2 groups x 2 ranks x 16 KB, bulk copies).
  static constexpr int RING_STAGES = PAIR ? 4 : 3;
  static constexpr int RING_SLOT_BYTES = 32 * BN * 2;          // one (tile, warp) slot of one rank
  static constexpr int RING_OFFSET = RING_STAGES * STAGE_BYTES;
  static constexpr int RING_BYTES = (BN == 256) ? 4 * RING_SLOT_BYTES : 0;
  // All-gather mode: two 8 KB bounce buffers through which one thread per CTA moves its slice of the peers'
  // weight shards (bulk copy peer memory -> shared memory -> local staging).
  static constexpr int PULL_BUF_BYTES = 8192;
  static constexpr int PULL_OFFSET = (STAGES * STAGE_BYTES > RING_OFFSET + RING_BYTES) ? STAGES * STAGE_BYTES
                                                                                       : RING_OFFSET + RING_BYTES;
  static constexpr int BAR_OFFSET = PULL_OFFSET + 2 * PULL_BUF_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], ring_full[2], ring_empty[2], pull[2], tmem ptr,
  // flags, peer output pointers (two-shot all-reduce: C and aux of every rank, 16 x 8 bytes)
  // + two 8-byte words of stall accounting
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 10) * 8 + 16 + 128 + 16 + 1024 /* alignment slack */;
};

// Does any of the rows [r0, r0 + len) of problem e hold data (see GemmParams::seg_counts)?
__device__ __forceinline__ bool rows_hold_data(const int* __restrict__ seg_counts, int seg_rows, int nseg, int e, int r0,
                                               int len) {
  const int* cnt = seg_counts + e * nseg;
  const int r1 = min(r0 + len, nseg * seg_rows);
  for (int s = r0 / seg_rows; s < nseg && s * seg_rows < r1; ++s)
    if (max(r0, s * seg_rows) < s * seg_rows + __ldg(cnt + s)) return true;
  return false;
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int group, int& tm, int& tn) {
  const int per_group = group * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group;
  const int gsize = min(group, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsize;
  tn = r / gsize;
}

// Tile schedule of a CTA.  Single CTAs walk the tile list with stride = grid size; CTA pairs walk the list of
// 256-row tile pairs with stride = number of pairs and each CTA of a pair takes the 128 rows of its cluster rank.
// `tile` is the index under which a 128 x BN tile is known to the communication buffers (inbox slots, flags):
// the same on every rank for the same rows and columns of C.
struct Sched { int first, total, stride, crank; };
template <bool PAIR>
__device__ __forceinline__ Sched make_sched(const GemmParams& p) {
  Sched s;
  if (PAIR) {
    s.crank = static_cast<int>(cluster_cta_rank());
    s.first = blockIdx.x >> 1; s.stride = gridDim.x >> 1; s.total = ((p.tiles_m + 1) >> 1) * p.tiles_n;
  } else {
    s.crank = 0; s.first = blockIdx.x; s.stride = p.gemm_ctas; s.total = p.tiles_m * p.tiles_n;
  }
  return s;
}
template <bool PAIR>
__device__ __forceinline__ void sched_tile(const GemmParams& p, const Sched& s, int it, int group, int& tile, int& tm, int& tn) {
  if (PAIR) {
    int tm2; tile_coords(it, (p.tiles_m + 1) >> 1, p.tiles_n, 8, tm2, tn);
    tm = 2 * tm2 + s.crank; tile = it * 2 + s.crank;
  } else {
    tile_coords(it, p.tiles_m, p.tiles_n, group, tm, tn); tile = it;
  }
}

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ uint32_t pack2(float a, float b, int dtype) {
  if (dtype == 0) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack2(uint32_t u, int dtype, float& a, float& b) {
  if (dtype == 0) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    a = __bfloat162float(v.x); b = __bfloat162float(v.y);
  } else {
    __half2 v = *reinterpret_cast<__half2*>(&u);
    a = __half2float(v.x); b = __half2float(v.y);
  }
}

// Store 8 consecutive elements starting at element offset `off` (16-byte aligned for 16-bit outputs).
__device__ __forceinline__ void store_vec8(void* base, int out_dtype, size_t off, const float* v, bool accumulate) {
  if (out_dtype == 2) {
    float* p = reinterpret_cast<float*>(base) + off;
    float4 a = make_float4(v[0], v[1], v[2], v[3]), b = make_float4(v[4], v[5], v[6], v[7]);
    if (accumulate) {
      const float4 oa = *reinterpret_cast<float4*>(p), ob = *reinterpret_cast<float4*>(p + 4);
      a.x += oa.x; a.y += oa.y; a.z += oa.z; a.w += oa.w; b.x += ob.x; b.y += ob.y; b.z += ob.z; b.w += ob.w;
    }
    *reinterpret_cast<float4*>(p) = a; *reinterpret_cast<float4*>(p + 4) = b;
  } else {
    uint16_t* p = reinterpret_cast<uint16_t*>(base) + off;
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = v[i];
    if (accumulate) {
      const uint4 old = *reinterpret_cast<uint4*>(p);
      float a, b;
      unpack2(old.x, out_dtype, a, b); f[0] += a; f[1] += b;
      unpack2(old.y, out_dtype, a, b); f[2] += a; f[3] += b;
      unpack2(old.z, out_dtype, a, b); f[4] += a; f[5] += b;
      unpack2(old.w, out_dtype, a, b); f[6] += a; f[7] += b;
    }
    uint4 o;
    o.x = pack2(f[0], f[1], out_dtype); o.y = pack2(f[2], f[3], out_dtype);
    o.z = pack2(f[4], f[5], out_dtype); o.w = pack2(f[6], f[7], out_dtype);
    *reinterpret_cast<uint4*>(p) = o;
  }
}

// Store 32 consecutive columns of one output row (fp32 values in v).
__device__ __forceinline__ void store_row32(void* base, int out_dtype, size_t row, int ld, int col, int N,
                                            const float (&v)[32], bool accumulate) {
  if (out_dtype == 2) {
    float* p = reinterpret_cast<float*>(base) + row * ld + col;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      if (col + g * 4 + 4 <= N) {
        float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        if (accumulate) {
          float4 old = *reinterpret_cast<float4*>(p + g * 4);
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        *reinterpret_cast<float4*>(p + g * 4) = o;
      }
    }
  } else {
    uint16_t* p = reinterpret_cast<uint16_t*>(base) + row * ld + col;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      if (col + g * 8 + 8 <= N) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = v[g * 8 + i];
        if (accumulate) {
          uint4 old = *reinterpret_cast<uint4*>(p + g * 8);
          float a, b;
          unpack2(old.x, out_dtype, a, b); f[0] += a; f[1] += b;
          unpack2(old.y, out_dtype, a, b); f[2] += a; f[3] += b;
          unpack2(old.z, out_dtype, a, b); f[4] += a; f[5] += b;
          unpack2(old.w, out_dtype, a, b); f[6] += a; f[7] += b;
        }
        uint4 o;
        o.x = pack2(f[0], f[1], out_dtype); o.y = pack2(f[2], f[3], out_dtype);
        o.z = pack2(f[4], f[5], out_dtype); o.w = pack2(f[6], f[7], out_dtype);
        *reinterpret_cast<uint4*>(p + g * 8) = o;
      }
    }
  }
}

// Named-barrier OR-reduction over the 128 epilogue threads (barrier 1): returns true if all passed true.
__device__ __forceinline__ bool __syncthreads_or_named(bool ok) {
  __shared__ int sh_fail;
  if ((threadIdx.x - 64) == 0) sh_fail = 0;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  if (!ok) sh_fail = 1;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  return sh_fail == 0;
}

// ---- peer-memory helpers of the fused all-reduce epilogue
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded spin until *flag >= want (flags are monotonically increasing epochs).
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* flag, unsigned int want, volatile int* abort_flag,
                                             uint64_t timeout_ns) {
  uint64_t start = 0;
  for (uint32_t it = 0;; ++it) {
    if (static_cast<int>(ld_acquire_sys(flag) - want) >= 0) return true;
    if ((it & 0x3f) == 0x3f) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (start == 0) start = now;
      else if (now - start > timeout_ns) { *abort_flag = 1; return false; }
    }
  }
}

// Rank that reduces the 32-row unit (tile, warp-row q): -1 = every rank (one-shot all-reduce), the owner of
// the rows (reduce-scatter), or round-robin over the units (two-shot all-reduce).
__device__ __forceinline__ int unit_owner(const GemmParams& p, int tile, int tm, int q) {
  if (p.ar.mode == 1) return (tm * BM + q * 32) / p.ar.rows_per_shard;
  if (p.ar.mode == 2) return (tile * 4 + q) % p.ar.n;
  return -1;
}
__device__ __forceinline__ unsigned unit_mask(const GemmParams& p, int tile, int tm) {
  unsigned mine = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int o = unit_owner(p, tile, tm, q);
    if (o < 0 || o == p.ar.rank) mine |= 1u << q;
  }
  return mine;
}

__device__ __forceinline__ uint4 pack8(const float* v, int dtype) {
  uint4 o;
  o.x = pack2(v[0], v[1], dtype); o.y = pack2(v[2], v[3], dtype);
  o.z = pack2(v[4], v[5], dtype); o.w = pack2(v[6], v[7], dtype);
  return o;
}

// Finish 8 consecutive reduced values of one output row: bias / GELU / store.  Two-shot all-reduce
// (`peer_out` non-null: C pointers of all ranks at [0..8), aux pointers at [8..16), null for this rank): the
// finished values also go to the same position of C (and aux) on every peer with 16-byte stores over NVLink.
__device__ __forceinline__ void comm_finish8(const GemmParams& p, float* v, size_t row, int col,
                                             const unsigned long long* peer_out = nullptr) {
  if (p.epilogue == 1 || p.epilogue == 2) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      v[e] += (p.in_dtype == 0) ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + e])
                                : __half2float(reinterpret_cast<const __half*>(p.bias)[col + e]);
  }
  const size_t out_row = (p.ar.mode == 1) ? row - static_cast<size_t>(p.ar.rank) * p.ar.rows_per_shard : row;
  const size_t off = out_row * p.N + col;
  // debug builds: the 8 values must lie inside C (and, on the peers, inside the tensor they announced)
  if (!AXB_IN_RANGE(p.status, off * 2ull, 16ull,
                    static_cast<unsigned long long>(p.ar.mode == 1 ? p.ar.rows_per_shard : p.M) * p.N * 2ull, 0x702u)) return;
  if (p.epilogue >= 2) {
    if (p.aux != nullptr) {
      store_vec8(p.aux, p.out_dtype, off, v, false);
      if (peer_out != nullptr) {   // 16-bit outputs only (checked by the launcher)
        const uint4 o = pack8(v, p.out_dtype);
        for (int j = 0; j < p.ar.n; ++j)
          if (peer_out[8 + j]) *(reinterpret_cast<uint4*>(peer_out[8 + j]) + (off >> 3)) = o;
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = gelu_tanh(v[e]);
  }
  store_vec8(p.C, p.out_dtype, off, v, p.accumulate != 0);
  if (peer_out != nullptr) {
    const uint4 o = pack8(v, p.out_dtype);
    for (int j = 0; j < p.ar.n; ++j)
      if (peer_out[j]) *(reinterpret_cast<uint4*>(peer_out[j]) + (off >> 3)) = o;
  }
}

__device__ __forceinline__ void acc_vec8(float* acc, const uint4& u, int dtype) {
  float a, b;
  unpack2(u.x, dtype, a, b); acc[0] += a; acc[1] += b;
  unpack2(u.y, dtype, a, b); acc[2] += a; acc[3] += b;
  unpack2(u.z, dtype, a, b); acc[4] += a; acc[5] += b;
  unpack2(u.w, dtype, a, b); acc[6] += a; acc[7] += b;
}

// ---- reducer warps (warps 6-9 of every CTA): second half of the fused all-reduce / reduce-scatter.
// They follow the CTA's own tile sequence: for each tile they wait (bounded) until the (tile, warp) flags of
// all ranks are up - the peers' partials were pushed into this rank's inbox over NVLink by their epilogues,
// this CTA's epilogue stored its own -, then sum the inbox slots of all ranks in rank order (identical bits
// on every rank; loads of all ranks are issued before any is used), apply bias / GELU and write C.  They
// only wait on memory, so they run beside the MMA and epilogue warps of the same SM: the reduction of every
// tile is spread over all SMs without taking any away from the GEMM.  In reduce-scatter mode only the
// 32-row groups owned by this rank exist in the inbox and are reduced.
// ---- watcher (one thread per CTA): runs ahead of the reducer warps over the CTA's tile sequence, waits
// (bounded) until the (tile, warp) flags of all ranks are up, performs the acquire fence once per tile and
// publishes the count of ready tiles in shared memory, so that polling global memory and the system-scope
// fence overlap the reduction of the previous tile instead of preceding each one.
template <int BN, bool PAIR>
__device__ __forceinline__ void watcher_thread(const GemmParams& p, const Sched& sc, int group, volatile int* abort_flag,
                                               volatile unsigned int* ready_tiles, unsigned long long* peer_out,
                                               uint8_t* ring = nullptr, uint64_t* ring_full = nullptr,
                                               uint64_t* ring_empty = nullptr) {
  constexpr int WVEC = (BN / 32) * 4 * 32;    // 16-byte words per (tile, warp) slot
  constexpr int SLOT = WVEC * 16;
  int issued = 0;                             // ring mode: units handed to the reducer warps so far
  int t = 0;
  if (p.ar.mode == 2) {
    // Two-shot all-reduce: learn where every peer keeps its C (and aux) inside its arena.  Each rank wrote the
    // offsets of this call into its peers' mailboxes when its kernel started; the pointers are left in shared
    // memory for the reducer warps, which see them through the ready signal of the first tile.
    for (int j = 0; j < p.ar.n; ++j) {
      peer_out[j] = 0ull; peer_out[8 + j] = 0ull;
      if (j == p.ar.rank) continue;
      const unsigned int* rec = p.ar.mail_local + j * 8;
      if (!wait_flag_ge(rec + 4, p.ar.epoch, abort_flag, p.timeout_ns)) { report_status(p.status, 0x124u); return; }
      const unsigned long long c_off = (static_cast<unsigned long long>(__ldcv(rec + 1)) << 32) | __ldcv(rec + 0);
      const unsigned long long a_off = (static_cast<unsigned long long>(__ldcv(rec + 3)) << 32) | __ldcv(rec + 2);
      peer_out[j] = reinterpret_cast<unsigned long long>(p.ar.arena_peer[j]) + c_off;
      if (p.aux != nullptr) peer_out[8 + j] = reinterpret_cast<unsigned long long>(p.ar.arena_peer[j]) + a_off;
    }
    __threadfence_block();
  }
  for (int it_ = sc.first; it_ < sc.total; it_ += sc.stride, ++t) {
    int tile, tm, tn; sched_tile<PAIR>(p, sc, it_, group, tile, tm, tn);
    const unsigned mine = unit_mask(p, tile, tm);
    if (mine != 0) {
      // the four (tile, warp) flags of a rank are one aligned 16-byte word
      uint64_t t0 = 0;
      bool good = true;
      for (uint32_t it = 0;; ++it) {
        bool all = true;
        for (int j = 0; j < p.ar.n; ++j) {
          const uint4 f = __ldcv(reinterpret_cast<const uint4*>(p.ar.flags_local + static_cast<size_t>(j) * p.ar.flags_per_src + tile * 4));
          const unsigned int fv[4] = {f.x, f.y, f.z, f.w};
          for (int q = 0; q < 4; ++q)
            if ((mine & (1u << q)) && static_cast<int>(fv[q] - p.ar.epoch) < 0) all = false;
        }
        if (all) break;
        if ((it & 0x3f) == 0x3f) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (*abort_flag || now - t0 > p.timeout_ns) { *abort_flag = 1; good = false; break; }
        }
      }
      if (!good) {
        report_status(p.status, 0x121u);
        return;
      }
      if (!AXB_DBG(p, 4)) __threadfence_system();   // acquire side of the flags, once per tile
      if (ring != nullptr) {
        // two-rank ring mode: bring the tile's inbox slots (own partial and the peer's, 16 KB each per warp-row)
        // into shared memory with bulk copies, one ring group per warp-row, as soon as the group is free
        asm volatile("fence.proxy.async;" ::: "memory");   // the slots were written with ordinary stores
        for (int q = 0; q < 4; ++q) {
          if (!(mine & (1u << q))) continue;
          const int g = issued & 1;
          if (!mbar_wait(&ring_empty[g], ((issued >> 1) & 1) ^ 1, abort_flag, p.timeout_ns)) {
            report_status(p.status, 0x123u);
            return;
          }
          mbar_expect_tx(&ring_full[g], 2 * SLOT);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ar.inbox_local) +
                                 (static_cast<size_t>(j) * p.ar.inbox_vecs_per_src + (static_cast<size_t>(tile) * 4 + q) * WVEC) * 16;
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(ring + (g * 2 + j) * SLOT)), "l"(src), "r"(SLOT), "r"(smem_u32(&ring_full[g]))
                         : "memory");
          }
          ++issued;
        }
      }
    }
    __threadfence_block();
    *ready_tiles = static_cast<unsigned>(t + 1);
  }
}

// 16-byte L2 load whose position among the other loads and the pins below is fixed for the compiler
__device__ __forceinline__ uint4 ld_cg_ordered(const uint4* ptr) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
// keeps a loaded word from being consumed before every load that precedes this statement was issued
__device__ __forceinline__ void pin(uint4& v) { asm volatile("" : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)); }

template <int BN, int NR, bool PAIR>
__device__ __forceinline__ void reducer_warps(const GemmParams& p, const Sched& sc, int group, volatile int* abort_flag,
                                              volatile unsigned int* ready_tiles, const unsigned long long* peer_out) {
  constexpr int CH = BN / 32;                 // 32-column chunks per tile row
  constexpr int WVEC = CH * 4 * 32;           // 16-byte words per (tile, warp) slot
  constexpr int TVEC = 4 * WVEC;
  constexpr int RG = NR < 4 ? NR : 4;         // ranks whose words are in flight together
  constexpr int UB = 4 / RG;                  // units per thread and batch: RG * UB * 4 = 16 loads in flight
  constexpr int UNITS = TVEC / 4;
  const int tid = threadIdx.x - 192;          // 0 .. REDUCER_THREADS-1
  bool ok = true;
  int t = -1;
  const bool probe = AXB_DBG(p, 64) && blockIdx.x == 0 && tid == 0;
  uint64_t ns_wait = 0, ns_work = 0, ns_mark = probe ? globaltimer_ns() : 0;
  for (int it_ = sc.first; it_ < sc.total && ok; it_ += sc.stride) {
    ++t;
    int tile, tm, tn; sched_tile<PAIR>(p, sc, it_, group, tile, tm, tn);
    const unsigned mine = unit_mask(p, tile, tm);
    if (mine == 0) continue;
    if (tid == 0) {
      // the watcher warp has seen (and acquired) the flags of all ranks for tiles [0, *ready_tiles)
      uint64_t t0 = 0;
      for (uint32_t it = 0; static_cast<int>(*ready_tiles - static_cast<unsigned>(t + 1)) < 0; ++it) {
        if (*abort_flag) break;
        if ((it & 0xfff) == 0xfff) {
          const uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > p.timeout_ns) { *abort_flag = 1; break; }
        }
      }
      __threadfence_block();
    }
    asm volatile("bar.sync 3, %0;" ::"n"(REDUCER_THREADS) : "memory");
    if (*abort_flag) { ok = false; break; }
    if (probe) { const uint64_t now = globaltimer_ns(); ns_wait += now - ns_mark; ns_mark = now; }
    if AXB_DBG(p, 8) continue;
    const uint4* inbox = reinterpret_cast<const uint4*>(p.ar.inbox_local) + static_cast<size_t>(tile) * TVEC;
    // A unit is one output row segment of 32 columns (4 vectors of one lane of one chunk): the thread that
    // reduces it writes 64 contiguous bytes of C, so every 32-byte sector of C is written in one piece.
    for (int base = tid; base < UNITS; base += REDUCER_THREADS * UB) {
      float acc[UB][4][8];
#pragma unroll
      for (int k = 0; k < UB; ++k)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[k][i][e] = 0.f;
#pragma unroll
      for (int j0 = 0; j0 < NR; j0 += RG) {
        if (j0 >= p.ar.n) break;
        uint4 in[RG][UB][4];
#pragma unroll
        for (int jj = 0; jj < RG; ++jj) {
          const int j = j0 + jj;
          const uint4* src = inbox + static_cast<size_t>(j < p.ar.n ? j : 0) * p.ar.inbox_vecs_per_src;
#pragma unroll
          for (int k = 0; k < UB; ++k) {
            const int u = base + k * REDUCER_THREADS;
            const int q = u / (CH * 32), c = (u >> 5) % CH, ln = u & 31;
            const bool live = j < p.ar.n && u < UNITS && (mine & (1u << q));
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // words of a slot are stored lane-permuted (see the epilogue): word w of row ln sits at w*32 + (ln ^ w)
              if (live) in[jj][k][i] = ld_cg_ordered(src + q * WVEC + (c * 4 + i) * 32 + (ln ^ ((c * 4 + i) & 31)));
              else in[jj][k][i] = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
#pragma unroll
        for (int jj = 0; jj < RG; ++jj)
#pragma unroll
          for (int k = 0; k < UB; ++k)
#pragma unroll
            for (int i = 0; i < 4; ++i) pin(in[jj][k][i]);
#pragma unroll
        for (int jj = 0; jj < RG; ++jj)   // rank order: identical bits on every rank
#pragma unroll
          for (int k = 0; k < UB; ++k)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc_vec8(acc[k][i], in[jj][k][i], p.in_dtype);
      }
#pragma unroll
      for (int k = 0; k < UB; ++k) {
        const int u = base + k * REDUCER_THREADS;
        if (u >= UNITS) continue;
        const int q = u / (CH * 32), c = (u >> 5) % CH, ln = u & 31;
        if (!(mine & (1u << q))) continue;
        const size_t row = static_cast<size_t>(tm) * BM + q * 32 + ln;
        if (row >= static_cast<size_t>(p.M)) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = tn * BN + c * 32 + i * 8;
          if (col >= p.N) continue;
          comm_finish8(p, acc[k][i], row, col, p.ar.mode == 2 ? peer_out : nullptr);
        }
      }
    }
    if (probe) { const uint64_t now = globaltimer_ns(); ns_work += now - ns_mark; ns_mark = now; }
  }
  if (probe) {
    volatile unsigned int* w = reinterpret_cast<volatile unsigned int*>(p.status);
    w[2] = static_cast<unsigned>(ns_wait); w[3] = static_cast<unsigned>(ns_work); w[7] = static_cast<unsigned>(t + 1);
  }
  if (!ok && tid == 0) report_status(p.status, 0x120u);
}

// ---- reducer warps, two ranks, 128x256 tiles: the inbox slots go through shared memory.
// One (tile, warp-row q) unit = two 16 KB slots (own partial and the peer's), each contiguous in the inbox.  The
// watcher thread copies them into a two-group ring behind the operand stages with bulk copies as soon as the
// tile's flags are up (32 - 64 KB in flight per SM without holding registers); the eight reducer warps wait for
// a group and read it row-wise: each of the eight warps takes four of the unit's 32 rows, a lane the 16-byte
// word `lane` of the row (the slot's words are stored lane-permuted, word w of row r at w*32 + (r ^ w), so these
// reads hit distinct banks), sums the two ranks in rank order, applies bias / GELU and stores 16 bytes: one warp
// instruction writes 512 contiguous bytes of a row of C - locally and, in the two-shot all-reduce, over NVLink
// into the peer's C as well - then the group is handed back.
template <int BN, bool PAIR>
__device__ __forceinline__ void reducer_ring(const GemmParams& p, const Sched& sc, int group, volatile int* abort_flag,
                                             uint8_t* ring, uint64_t* ring_full, uint64_t* ring_empty,
                                             const unsigned long long* peer_out) {
  constexpr int CH = BN / 32;
  constexpr int WVEC = CH * 4 * 32;           // 16-byte words per slot
  constexpr int SLOT = WVEC * 16;
  static_assert(CH * 4 == 32, "row-wise ring reducer: one 16-byte word of a row per lane");
  const int tid = threadIdx.x - 192;
  const int wr = tid >> 5, ln = tid & 31;     // wr: rows 4*wr .. 4*wr+3 of the unit, ln: 16-byte word of the row
  const unsigned long long* peers = p.ar.mode == 2 ? peer_out : nullptr;
  bool ok = true;
  int consumed = 0;                           // ring group = consumed & 1, phase = (consumed >> 1) & 1
  for (int it_ = sc.first; it_ < sc.total && ok; it_ += sc.stride) {
    int tile, tm, tn; sched_tile<PAIR>(p, sc, it_, group, tile, tm, tn);
    const unsigned mine = unit_mask(p, tile, tm);
    for (int q = 0; q < 4; ++q) {
      if (!(mine & (1u << q))) continue;
      const int g = consumed & 1;
      if (!mbar_wait(&ring_full[g], (consumed >> 1) & 1, abort_flag, p.timeout_ns)) { ok = false; break; }
      ++consumed;
      if (!AXB_DBG(p, 8)) {
        const uint4* s0 = reinterpret_cast<const uint4*>(ring + (g * 2) * SLOT);
        const uint4* s1 = reinterpret_cast<const uint4*>(ring + (g * 2 + 1) * SLOT);
        const int col = tn * BN + ln * 8;
        uint4 a[4], b[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int r = wr * 4 + k;
          a[k] = s0[ln * 32 + (r ^ ln)]; b[k] = s1[ln * 32 + (r ^ ln)];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const size_t row = static_cast<size_t>(tm) * BM + q * 32 + wr * 4 + k;
          if (row >= static_cast<size_t>(p.M) || col >= p.N) continue;
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
          acc_vec8(acc, a[k], p.in_dtype);     // rank order: identical bits on both ranks
          acc_vec8(acc, b[k], p.in_dtype);
          comm_finish8(p, acc, row, col, peers);
        }
      }
      __syncwarp();
      if (ln == 0) mbar_arrive(&ring_empty[g]);
    }
  }
  if (!ok && tid == 0) report_status(p.status, 0x122u);
}

// ---- all-gather puller (one thread per CTA): brings this CTA's slice of every shard of B - own shard first,
// then the peers' in ring order - from the owners' outboxes into the local staging copy of B.  The bytes never
// pass through registers: a bulk copy lands 8 KB of the (peer-mapped) outbox in shared memory, a second bulk copy
// writes them to staging, two buffers alternate so that two remote reads are in flight per SM all the time
// (148 SMs x 16 KB per NVLink round trip).  When the CTA's slice of a shard is complete it adds one to the
// shard's arrival counter; the TMA producers of all CTAs wait for the counter to reach the number of CTAs
// before they read tiles of that shard.
template <int BN>
__device__ __forceinline__ void ag_puller(const GemmParams& p, uint8_t* buf, uint64_t* pull_bar,
                                          volatile int* abort_flag) {
  constexpr uint32_t CHB = GemmSmem<BN, false>::PULL_BUF_BYTES;
  const unsigned long long total = p.ag.shard_bytes;
  unsigned long long per = (total + gridDim.x - 1) / gridDim.x;
  per = (per + 15ull) & ~15ull;                              // bulk copies move multiples of 16 bytes
  const unsigned long long lo = per * blockIdx.x < total ? per * blockIdx.x : total;
  const unsigned long long hi = lo + per < total ? lo + per : total;
  const uint32_t nch = static_cast<uint32_t>((hi - lo + CHB - 1) / CHB);
  uint32_t loads = 0, waited = 0;   // bulk loads issued / awaited so far: buffer = index & 1, phase = (index >> 1) & 1
  bool ok = true;
  for (int s = 0; s < p.ag.n && ok; ++s) {
    const int z = (p.ag.rank + s) % p.ag.n;
    if (z != p.ag.rank && !wait_flag_ge(p.ag.wait_local + z, p.ag.epoch, abort_flag, p.timeout_ns)) { ok = false; break; }
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag.outbox_peer[z]);
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.ag.staging) + static_cast<unsigned long long>(z) * total;
    auto chunk_bytes = [&](uint32_t k) {
      const unsigned long long off = lo + static_cast<unsigned long long>(k) * CHB;
      return static_cast<uint32_t>(hi - off < CHB ? hi - off : CHB);
    };
    auto issue_load = [&](uint32_t k) {
      const uint32_t b = loads & 1u, bytes = chunk_bytes(k);
      mbar_expect_tx(&pull_bar[b], bytes);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(smem_u32(buf + b * CHB)), "l"(src + lo + static_cast<unsigned long long>(k) * CHB), "r"(bytes),
                     "r"(smem_u32(&pull_bar[b])) : "memory");
      ++loads;
    };
    if (nch > 0) issue_load(0);
    for (uint32_t k = 0; k < nch; ++k) {
      if (k + 1 < nch) {
        // the other buffer was last read by the store of chunk k-1: that read must be over before it is refilled
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        issue_load(k + 1);
      }
      const uint32_t b = waited & 1u;
      if (!mbar_wait(&pull_bar[b], (waited >> 1) & 1u, abort_flag, p.timeout_ns)) { ok = false; break; }
      ++waited;
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                   ::"l"(dst + lo + static_cast<unsigned long long>(k) * CHB), "r"(smem_u32(buf + b * CHB)), "r"(chunk_bytes(k))
                   : "memory");
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store of this slice has been written
    if (!ok) break;
    asm volatile("fence.proxy.async;" ::: "memory");            // bulk-copy writes -> visible to the TMA reads of all CTAs
    __threadfence();
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.ag.shard_ready + z) : "memory");
  }
  if (!ok) {
    // loads still in flight must land before the CTA's shared memory goes away (bounded)
    for (; waited < loads; ++waited) {
      const uint64_t t0 = globaltimer_ns();
      while (!mbar_try_wait(&pull_bar[waited & 1u], (waited >> 1) & 1u) && globaltimer_ns() - t0 < 2000000ull) {}
    }
    report_status(p.status, 0x110u);
  }
}

template <int BN, int A_MN, int B_MN, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const GemmParams p) {
  // PAIR: launched as clusters of two CTAs (tcgen05.mma.cta_group::2): the pair computes a 256 x BN tile, each
  // CTA stages its own 128 rows of A and its half of the B tile (no multicast loads), the even CTA issues the
  // MMAs for both, and each CTA's epilogue, flagger, watcher and reducer warps handle the 128 rows held in its
  // own TMEM exactly like a single CTA handles a 128 x BN tile.
  using S = GemmSmem<BN, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + S::STAGES;
  uint64_t* tmem_full = empty_bar + S::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint64_t* ring_full = tmem_empty + 2;
  uint64_t* ring_empty = ring_full + 2;
  uint64_t* pull_bar = ring_empty + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(pull_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);
  volatile unsigned int* parts_done = reinterpret_cast<volatile unsigned int*>(tmem_ptr_smem + 2);
  volatile unsigned int* ready_tiles = reinterpret_cast<volatile unsigned int*>(tmem_ptr_smem + 3);
  unsigned long long* peer_out = reinterpret_cast<unsigned long long*>(tmem_ptr_smem + 4);   // [16], 8-byte aligned
  unsigned long long* stall_words = peer_out + 16;   // [0] time the last epilogue warp finished, [1] ns the producer waited for shards

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + BK - 1) / BK;
  const int group = (BN == 256) ? 16 : 8;
  const uint64_t timeout = p.timeout_ns;
  const Sched sc = make_sched<PAIR>(p);
  const int crank = sc.crank;           // rank inside the CTA pair (0 without pairs)
  // two ranks, 128x256 tiles: the reducer stages inbox slots in shared memory behind a shortened operand ring
  const bool ring_mode = BN == 256 && p.ar.n == 2 && !AXB_DBG(p, 128);
  const int nstages = ring_mode ? S::RING_STAGES : S::STAGES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], PAIR ? 8 : 4); }
    for (int b = 0; b < 2; ++b) { mbar_init(&ring_full[b], 1); mbar_init(&ring_empty[b], REDUCER_THREADS / 32); }
    for (int b = 0; b < 2; ++b) mbar_init(&pull_bar[b], 1);
    *abort_flag = 0;
    *parts_done = 0;
    *ready_tiles = 0;
    stall_words[0] = 0ull; stall_words[1] = 0ull;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(tmem_ptr_smem, 2 * BN); tmem_relinquish_pair(); }
    else { tmem_alloc(tmem_ptr_smem, 2 * BN); tmem_relinquish(); }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) { __syncwarp(); cluster_sync_all(); }   // both CTAs' barriers exist before any remote arrival or TMA signal
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (p.ar.n > 1 && threadIdx.x == 64) {
    // The inbox (double-buffered by call parity) was last read by the peers in call epoch-2:
    // do not overwrite it before they are done with that call.
    for (int j = 0; j < p.ar.n; ++j) {
      if (j == p.ar.rank) continue;
      if (!wait_flag_ge(p.ar.done_local + j, p.ar.epoch - 2u, abort_flag, timeout)) {
        report_status(p.status, 0x108u);
        break;
      }
    }
    if (p.ar.mode == 2 && blockIdx.x == 0) {
      // two-shot all-reduce: tell every peer where this rank's C and aux of this call lie inside its arena
      for (int j = 0; j < p.ar.n; ++j) {
        if (j == p.ar.rank) continue;
        unsigned int* rec = p.ar.mail_peer[j] + p.ar.rank * 8;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 0), "r"(static_cast<unsigned>(p.ar.c_off)) : "memory");
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 1), "r"(static_cast<unsigned>(p.ar.c_off >> 32)) : "memory");
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 2), "r"(static_cast<unsigned>(p.ar.aux_off)) : "memory");
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(rec + 3), "r"(static_cast<unsigned>(p.ar.aux_off >> 32)) : "memory");
        st_release_sys(rec + 4, p.ar.epoch);
      }
    }
  }
  if (p.ar.n > 1) __syncthreads();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      uint32_t armed_mask = 0, armed_parity = 0;
      uint32_t ag_ready_mask = 0;
      bool ok = true;
      for (int it_ = sc.first; it_ < sc.total && ok; it_ += sc.stride) {
        int tile, tm, tn; sched_tile<PAIR>(p, sc, it_, group, tile, tm, tn);
        tn += p.tn_offset; if (tn >= p.tiles_n) tn -= p.tiles_n;
        const int m0 = tm * BM, n0 = tn * BN + (PAIR ? crank * (BN / 2) : 0);   // a pair's CTA loads its half of the B tile
        for (int kbi = 0; kbi < num_kb; ++kbi) {
          int kb = kbi + p.kb_offset; if (kb >= num_kb) kb -= num_kb;
          if (p.ag.n > 1) {
            // B row block needed by this load: rows n0.. (B is [N,K]) or rows k0.. (B is [K,N])
            const int brow = (B_MN == 0) ? n0 : kb * BK;
            const int shard = brow / p.ag.rows_per_shard;
            if (!(ag_ready_mask & (1u << shard))) {
              uint64_t t0 = 0;
              const uint64_t t_wait = globaltimer_ns();
              for (uint32_t it = 0;; ++it) {
                unsigned int v;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.ag.shard_ready + shard) : "memory");
                if (static_cast<int>(v - p.ag.ready_target) >= 0) break;
                if ((it & 0x3f) == 0x3f) {
                  const uint64_t now = globaltimer_ns();
                  if (t0 == 0) t0 = now;
                  else if (*abort_flag || now - t0 > timeout) { *abort_flag = 1; ok = false; break; }
                }
              }
              if (!ok) break;
              asm volatile("fence.proxy.async;" ::: "memory");
              ag_ready_mask |= 1u << shard;
              stall_words[1] += globaltimer_ns() - t_wait;
            }
          }
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, timeout)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          const int k0 = kb * BK;
          if (PAIR) {
            // the leader's barrier counts the bytes of both CTAs' loads of this stage
            if (crank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
            if (A_MN == 0) {
              tma_load_2d_pair(sA, &tmA, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sA + j * (BK * 128), &tmA, &full_bar[stage], m0 + 64 * j, k0);
            }
            if (B_MN == 0) {
              tma_load_2d_pair(sB, &tmB, &full_bar[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sB + j * (BK * 128), &tmB, &full_bar[stage], n0 + 64 * j, k0);
            }
          } else {
            mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
            armed_mask |= 1u << stage;
            armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
            if (A_MN == 0) {
              tma_load_2d(sA, &tmA, &full_bar[stage], k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) tma_load_2d(sA + j * (BK * 128), &tmA, &full_bar[stage], m0 + 64 * j, k0);
            }
            if (B_MN == 0) {
              tma_load_2d(sB, &tmB, &full_bar[stage], k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j) tma_load_2d(sB + j * (BK * 128), &tmB, &full_bar[stage], n0 + 64 * j, k0);
            }
          }
          if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        // drain: wait (bounded) until every copy this thread started has landed
        for (int s = 0; s < S::STAGES; ++s) {
          if (armed_mask & (1u << s)) {
            uint32_t par = (armed_parity >> s) & 1u;
            uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(&full_bar[s], par) && globaltimer_ns() - t0 < 2000000ull) {}
          }
        }
        report_status(p.status, 0x101u);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if ((!PAIR || crank == 0) && elect_one()) {   // in a pair the even CTA issues for both
      const uint32_t idesc = umma_idesc(p.in_dtype == 0 ? 1 : 0, A_MN, B_MN, PAIR ? 2 * BM : BM, BN);
      // K-major: 8-row groups 1024 B apart, K step = 32 B inside the swizzle row.
      // MN-major: 64-wide MN chunks BK*128 B apart (leading), 8-K-row groups
      // 1024 B apart (stride), K step = 16 rows * 128 B.
      const uint32_t a_lbo = A_MN ? BK * 128 : 16, a_sbo = 1024, a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_lbo = B_MN ? BK * 128 : 16, b_sbo = 1024, b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int it_ = sc.first; it_ < sc.total && ok; it_ += sc.stride, ++t) {
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, timeout)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * a_kstep, a_lbo, a_sbo);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * b_kstep, b_lbo, b_sbo);
            if (PAIR) umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
            else umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(&empty_bar[stage]);   // frees the stage in both CTAs
          else umma_commit(&empty_bar[stage]);
          if (++stage == nstages) { stage = 0; phase ^= 1; }
        }
        if (ok) { if (PAIR) umma_commit_pair(&tmem_full[buf]); else umma_commit(&tmem_full[buf]); }
      }
      if (!ok) {
        // MMAs issued before the abort may still be running: give them time before TMEM is released
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000ull) {}
        report_status(p.status, 0x102u);
      }
    }
  } else if (warp == FLAGGER_WARP) {
    // ------------------------------------------------------------------ flagger: publishes finished partials
    // One thread waits until the four epilogue warps have stored a tile's partial (shared counter), runs
    // the single system-scope fence the tile needs and raises its flags on the reducing ranks, so that the
    // fence latency is off the epilogue's path.
    // (lane 16 of the same warp is the all-gather puller; the two run as independent threads)
    if (p.ag.n > 1 && lane == 16) {
      ag_puller<BN>(p, smem + S::PULL_OFFSET, pull_bar, abort_flag);
    } else if (p.ar.n > 1 && lane == 0) {
      // The system-scope fence is the expensive part (it waits for every store the SM has in flight over
      // NVLink), so the flags of `flag_batch` consecutive tiles share one fence; the last tiles of the CTA
      // are published one by one so that the peers' reducers do not wait at the end of the kernel.
      const int my_tiles = sc.first < sc.total ? (sc.total - sc.first + sc.stride - 1) / sc.stride : 0;
      int batch = p.flag_batch < 1 ? 1 : p.flag_batch;
      int t = 0, published = 0;
      bool good = true;
      while (published < my_tiles && good) {
        const int upto = (my_tiles - published <= batch) ? published + 1 : published + batch;   // tiles [published, upto)
        uint64_t t0 = 0;
        for (uint32_t it = 0; static_cast<int>(*parts_done - 4u * upto) < 0; ++it) {
          if ((it & 0xff) == 0xff) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (*abort_flag || now - t0 > timeout) { good = false; break; }
          }
        }
        if (!good) break;
        if (!AXB_DBG(p, 1)) __threadfence_system();
        for (t = published; t < upto; ++t) {
          int tile, tm, tn; sched_tile<PAIR>(p, sc, sc.first + t * sc.stride, group, tile, tm, tn);
          for (int qq = 0; qq < 4; ++qq) {
            const int own = unit_owner(p, tile, tm, qq);
            for (int j = 0; j < p.ar.n; ++j) {
              if (own >= 0 && j != own && !(p.ar.loopback && own == p.ar.rank)) continue;
              if (!AXB_IN_RANGE(p.status, static_cast<unsigned long long>(tile) * 4 + qq, 1ull, p.ar.flags_per_src, 0x703u)) continue;
              unsigned int* f = (j == p.ar.rank ? p.ar.flags_local : p.ar.flags_peer[j]) +
                                static_cast<size_t>(p.ar.rank) * p.ar.flags_per_src + tile * 4 + qq;
              asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f), "r"(p.ar.epoch) : "memory");
            }
          }
        }
        published = upto;
      }
    }
  } else if (warp == WATCHER_WARP) {
    if (p.ar.n > 1 && lane == 0) {
      if (ring_mode) watcher_thread<BN, PAIR>(p, sc, group, abort_flag, ready_tiles, peer_out, smem + S::RING_OFFSET, ring_full, ring_empty);
      else watcher_thread<BN, PAIR>(p, sc, group, abort_flag, ready_tiles, peer_out);
    }
  } else if (warp >= 6) {
    bool done = false;
    if constexpr (BN == 256) {
      if (ring_mode) {
        reducer_ring<BN, PAIR>(p, sc, group, abort_flag, smem + S::RING_OFFSET, ring_full, ring_empty, peer_out);
        done = true;
      }
    }
    if (done) {
    } else if (p.ar.n == 2) reducer_warps<BN, 2, PAIR>(p, sc, group, abort_flag, ready_tiles, peer_out);
    else if (p.ar.n > 2 && p.ar.n <= 4) reducer_warps<BN, 4, PAIR>(p, sc, group, abort_flag, ready_tiles, peer_out);
    else if (p.ar.n > 4) reducer_warps<BN, 8, PAIR>(p, sc, group, abort_flag, ready_tiles, peer_out);
  } else {
    // ------------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    bool ok = true;
    int t = 0;
    // Finish one tile: values v (one row, 32 columns) -> bias / GELU -> C.
    auto finish_chunk = [&](float (&v)[32], size_t out_row, int col, bool store_ok) {
      if (p.epilogue == 1 || p.epilogue == 2) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (col + i < p.N) {
            float b = (p.in_dtype == 0)
                          ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + i])
                          : __half2float(reinterpret_cast<const __half*>(p.bias)[col + i]);
            v[i] += b;
          }
        }
      }
      if (p.epilogue >= 2) {
        if (p.aux != nullptr && store_ok) store_row32(p.aux, p.out_dtype, out_row, p.N, col, p.N, v, false);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
      }
      if (store_ok) store_row32(p.C, p.out_dtype, out_row, p.N, col, p.N, v, p.accumulate != 0);
    };

    for (int it_ = sc.first; it_ < sc.total && ok; it_ += sc.stride, ++t) {
      int tile, tm, tn; sched_tile<PAIR>(p, sc, it_, group, tile, tm, tn);
      tn += p.tn_offset; if (tn >= p.tiles_n) tn -= p.tiles_n;
      const int buf = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      if (!mbar_wait(&tmem_full[buf], acc_phase, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      const size_t row = static_cast<size_t>(tm) * BM + q * 32 + lane;
      const bool row_ok = row < static_cast<size_t>(p.M);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      if (p.ar.n <= 1) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          const int col = tn * BN + c * 32;
          if (col >= p.N) break;  // uniform across the warp
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          finish_chunk(v, row, col, row_ok);
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) { if (PAIR) mbar_arrive_leader(&tmem_empty[buf]); else mbar_arrive(&tmem_empty[buf]); }
        continue;
      }
      // ---- communication mode: the epilogue moves this warp's bf16 partial (32 rows x BN columns) out of
      // TMEM into the inbox of every rank that reduces these rows - with posted 16-byte stores over NVLink
      // for the peers, plain stores for this rank - then the flagger raises the (tile, warp) flags; the reducer warps of the
      // reducing ranks sum the inbox slots locally.  Slot layout of a (tile, warp): [chunk][vec 0..3][lane]
      // 16-byte words, so every store instruction of a warp covers 512 contiguous bytes.
      // Words are lane-permuted inside their 512 bytes (word w of row `lane` at w*32 + (lane ^ w)): a store
      // instruction still covers the same 512 contiguous bytes, and the reducer warps can read a slot row by
      // row from shared memory without bank conflicts.
      const int owner = unit_owner(p, tile, tm, q);
      const bool own_unit = owner < 0 || owner == p.ar.rank;
      const size_t slot_vec = static_cast<size_t>(p.ar.rank) * p.ar.inbox_vecs_per_src +
                              (static_cast<size_t>(tile) * 4 + q) * (BN / 32) * 4 * 32;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        if (tn * BN + c * 32 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        uint4 w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i].x = pack2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]), p.in_dtype);
          w[i].y = pack2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]), p.in_dtype);
          w[i].z = pack2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]), p.in_dtype);
          w[i].w = pack2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]), p.in_dtype);
        }
        for (int j = 0; j < p.ar.n; ++j) {
          // one-shot: every rank gets the partial; otherwise only the unit's owner (in the one-GPU emulation
          // an owned unit is also stored for the other source slot, which stands in for the peer's partial)
          if (owner >= 0 && j != owner && !(p.ar.loopback && own_unit)) continue;
          if (AXB_DBG(p, 2) && j != p.ar.rank) continue;
          if AXB_DBG(p, 16) continue;
          uint4* dst = reinterpret_cast<uint4*>(j == p.ar.rank ? p.ar.inbox_local : p.ar.inbox_peer[j]) + slot_vec;
          // debug builds: the slot must lie inside rank j's inbox (n sources x inbox_vecs_per_src 16-byte words)
          if (!AXB_IN_RANGE(p.status, (slot_vec + (c * 4 + 3) * 32 + 31) * 16ull, 16ull,
                            p.ar.inbox_vecs_per_src * 16ull * p.ar.n, 0x701u)) continue;
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[(c * 4 + i) * 32 + (lane ^ ((c * 4 + i) & 31))] = w[i];
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) { if (PAIR) mbar_arrive_leader(&tmem_empty[buf]); else mbar_arrive(&tmem_empty[buf]); }   // accumulator is free: the MMA warp runs ahead
      // hand the stored partial to the flagger warp (release at CTA scope on a monotonic counter)
      if (lane == 0) {
        __threadfence_block();
        atomicAdd(const_cast<unsigned int*>(parts_done), 1u);
      }
    }
    if (!ok && lane == 0) report_status(p.status, 0x104u);
    if (lane == 0 && (p.ar.n > 1 || p.ag.n > 1)) atomicMax(stall_words, static_cast<unsigned long long>(globaltimer_ns()));
  }

  tcgen05_fence_before();
  __syncthreads();
  if (PAIR) {
    // the peer CTA's shared memory and TMEM stay valid until every MMA and remote arrival of the pair is done
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) { tcgen05_fence_after(); tmem_dealloc_pair(tmem_base, 2 * BN); }
  } else if (warp == 1) { __syncwarp(); tcgen05_fence_after(); tmem_dealloc(tmem_base, 2 * BN); }
  if (p.ag.n > 1 && threadIdx.x == 32) {
    __threadfence();
    if (atomicAdd(p.ag.counter, 1u) == gridDim.x - 1) {
      *p.ag.counter = 0;
      __threadfence_system();
      for (int j = 0; j < p.ag.n; ++j)
        if (j != p.ag.rank) st_release_sys(p.ag.done_peer[j] + p.ag.rank, p.ag.epoch);
    }
  }
  if (p.ar.n > 1 && threadIdx.x == 0) {
    // the CTA's stores into the peers' inboxes (and, in the two-shot all-reduce, into their C) are ordered
    // before the CTA counter at system scope; the last CTA then tells the peers that this rank is done
    if (p.ar.mode == 2) __threadfence_system(); else __threadfence();
    if (atomicAdd(p.ar.counter, 1u) == gridDim.x - 1) {
      *p.ar.counter = 0;
      __threadfence_system();
      for (int j = 0; j < p.ar.n; ++j)
        if (j != p.ar.rank) st_release_sys(p.ar.done_peer[j] + p.ar.rank, p.ar.epoch);
      if (p.ar.mode == 2) {
        // two-shot all-reduce: the rows of C that the peers own are written by their reducer warps; C is
        // complete on this rank once every peer has reported the end of its call (bounded wait)
        for (int j = 0; j < p.ar.n; ++j) {
          if (j == p.ar.rank) continue;
          if (!wait_flag_ge(p.ar.done_local + j, p.ar.epoch, abort_flag, timeout)) { report_status(p.status, 0x109u); break; }
        }
      }
    }
  }
  if ((p.ar.n > 1 || p.ag.n > 1) && threadIdx.x == 0) {
    unsigned long long stall = stall_words[1];
    if (p.ar.n > 1 && stall_words[0] != 0ull) stall += globaltimer_ns() - stall_words[0];
    atomicAdd(&g_comm_stall, stall * 1024ull / gridDim.x);
  }
}

// ----------------------------------------------------------------------------- CTA-pair GEMM (cta_group::2)
// Plain GEMM (no in-kernel communication) on pairs of CTAs: a cluster of two CTAs computes one 256x256 output
// tile with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its own 128 of the 256
// rows/columns of B per K block (32 KB per stage instead of 48 KB, six stages), the leader CTA issues the
// MMAs for both, and each CTA's epilogue drains the 128 accumulator rows held in its own TMEM.  Shared-memory
// traffic per SM and flop drops by a third against the single-CTA 128x256 tile, which is what bounds that
// kernel's tensor-pipe utilisation.  TMA loads carry no multicast; the only cluster-wide signals are the
// tcgen05.commit arrivals and plain remote mbarrier arrivals.
constexpr int PAIR_THREADS = 192;   // TMA warp, MMA warp, 4 epilogue warps
constexpr int PAIR_BN = 256;
struct PairSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (PAIR_BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 6;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024 /* alignment slack */;
};

// Masked batched mode: is the 256-row tile pair tm2 of problem e computed at all?  (mode 1: one of its rows holds
// data; mode 2: one of the problem's K blocks does.)  All three roles of the kernel ask the same question.
__device__ __forceinline__ bool pair_tile_computed(const GemmParams& p, int e, int tm2, int num_kb) {
  if (p.mask_mode == 1) return rows_hold_data(p.seg_counts, p.seg_rows, p.nseg, e, tm2 * 2 * BM, 2 * BM);
  if (p.mask_mode == 2) return rows_hold_data(p.seg_counts, p.seg_rows, p.nseg, e, 0, num_kb * BK);
  return true;
}

template <int A_MN, int B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PAIR_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  using S = PairSmem;
  constexpr int BN = PAIR_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + S::STAGES;
  uint64_t* tmem_full = empty_bar + S::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_ptr_smem = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_ptr_smem + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();         // 0: leader (issues the MMAs), 1: peer
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_kb = (p.K + BK - 1) / BK;
  const int tiles_m2 = (p.tiles_m + 1) >> 1;         // 256-row tile rows
  const int per_batch = tiles_m2 * p.tiles_n;
  const int total = per_batch * p.nb;
  const uint64_t timeout = p.timeout_ns;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 8); }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); }
  if (warp == 1) { tmem_alloc_pair(tmem_ptr_smem, 2 * BN); tmem_relinquish_pair(); }
  tcgen05_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();     // both CTAs' barriers are initialised before any remote arrival or TMA signal
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int it = pair_id; it < total && ok; it += num_pairs) {
        const int e = it / per_batch;
        int tm2, tn; tile_coords(it - e * per_batch, tiles_m2, p.tiles_n, 8, tm2, tn);
        const int m0 = (2 * tm2 + static_cast<int>(rank)) * BM;
        const int n0 = tn * BN + static_cast<int>(rank) * (BN / 2);   // this CTA's half of the B tile
        // row coordinate of problem e in the stacked operands (rows = M or N for a K-major operand, K otherwise)
        const int a_r = e * p.a_batch_rows, b_r = e * p.b_batch_rows;
        if (p.mask_mode == 1 && !rows_hold_data(p.seg_counts, p.seg_rows, p.nseg, e, tm2 * 2 * BM, 2 * BM)) continue;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (p.mask_mode == 2 && !rows_hold_data(p.seg_counts, p.seg_rows, p.nseg, e, kb * BK, BK)) continue;
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, timeout)) { ok = false; break; }
          uint8_t* sA = smem + stage * S::STAGE_BYTES;
          uint8_t* sB = sA + S::A_BYTES;
          // the leader's barrier counts the bytes of both CTAs' loads of this stage
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
          const int k0 = kb * BK;
          if (A_MN == 0) {
            tma_load_2d_pair(sA, &tmA, &full_bar[stage], k0, m0 + a_r);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d_pair(sA + j * (BK * 128), &tmA, &full_bar[stage], m0 + 64 * j, k0 + a_r);
          }
          if (B_MN == 0) {
            tma_load_2d_pair(sB, &tmB, &full_bar[stage], k0, n0 + b_r);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j) tma_load_2d_pair(sB + j * (BK * 128), &tmB, &full_bar[stage], n0 + 64 * j, k0 + b_r);
          }
          if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) report_status(p.status, 0x141u);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = umma_idesc(p.in_dtype == 0 ? 1 : 0, A_MN, B_MN, 2 * BM, BN);
      const uint32_t a_lbo = A_MN ? BK * 128 : 16, a_sbo = 1024, a_kstep = A_MN ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_lbo = B_MN ? BK * 128 : 16, b_sbo = 1024, b_kstep = B_MN ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      int t = 0;
      for (int it = pair_id; it < total && ok; it += num_pairs) {
        const int e = it / per_batch;
        if (p.mask_mode != 0) {
          int tm2, tn; tile_coords(it - e * per_batch, tiles_m2, p.tiles_n, 8, tm2, tn);
          if (!pair_tile_computed(p, e, tm2, num_kb)) continue;      // no accumulator buffer is used for it
        }
        const int buf = t & 1;
        const uint32_t acc_phase = (t >> 1) & 1;
        ++t;
        if (!mbar_wait(&tmem_empty[buf], acc_phase ^ 1, abort_flag, timeout)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool first = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (p.mask_mode == 2 && !rows_hold_data(p.seg_counts, p.seg_rows, p.nseg, e, kb * BK, BK)) continue;
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, timeout)) { ok = false; break; }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = umma_smem_desc(a_addr + k * a_kstep, a_lbo, a_sbo);
            const uint64_t bdesc = umma_smem_desc(b_addr + k * b_kstep, b_lbo, b_sbo);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (first && k == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit_pair(&empty_bar[stage]);      // frees this stage in both CTAs
          if (++stage == S::STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(&tmem_full[buf]);   // accumulator complete: both epilogues may read
      }
      if (!ok) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 50000ull) {}   // let MMAs in flight finish before TMEM is released
        report_status(p.status, 0x142u);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    bool ok = true;
    int t = 0;
    for (int it = pair_id; it < total && ok; it += num_pairs) {
      const int e = it / per_batch;
      int tm2, tn; tile_coords(it - e * per_batch, tiles_m2, p.tiles_n, 8, tm2, tn);
      const int tm = 2 * tm2 + static_cast<int>(rank);
      const size_t local_row = static_cast<size_t>(tm) * BM + q * 32 + lane;
      const bool row_ok = local_row < static_cast<size_t>(p.M);     // rows past M belong to the next problem
      const size_t row = local_row + static_cast<size_t>(e) * p.c_batch_rows;
      if (p.mask_mode != 0 && !pair_tile_computed(p, e, tm2, num_kb)) {
        // a tile without data: zeros (nothing to add when accumulating), no accumulator buffer involved
        if (row_ok && !p.accumulate) {
          float z[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) z[i] = 0.f;
          for (int c = 0; c < BN / 32 && tn * BN + c * 32 < p.N; ++c)
            store_row32(p.C, p.out_dtype, row, p.N, tn * BN + c * 32, p.N, z, false);
        }
        continue;
      }
      const int buf = t & 1;
      const uint32_t acc_phase = (t >> 1) & 1;
      ++t;
      if (!mbar_wait(&tmem_full[buf], acc_phase, abort_flag, timeout)) { ok = false; break; }
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col = tn * BN + c * 32;
        if (col >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (p.epilogue == 1 || p.epilogue == 2) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col + i < p.N) {
              v[i] += (p.in_dtype == 0) ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col + i])
                                        : __half2float(reinterpret_cast<const __half*>(p.bias)[col + i]);
            }
          }
        }
        if (p.epilogue >= 2) {
          if (p.aux != nullptr && row_ok) store_row32(p.aux, p.out_dtype, row, p.N, col, p.N, v, false);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = gelu_tanh(v[i]);
        }
        if (row_ok) store_row32(p.C, p.out_dtype, row, p.N, col, p.N, v, p.accumulate != 0);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);   // 8 arrivals (4 warps x 2 CTAs) free the buffer
    }
    if (!ok && lane == 0) report_status(p.status, 0x144u);
  }

  tcgen05_fence_before();
  __syncthreads();
  __syncwarp();
  cluster_sync_all();     // the peer's shared memory and TMEM stay valid until every MMA and arrival is done
  if (warp == 1) { tcgen05_fence_after(); tmem_dealloc_pair(tmem_base, 2 * BN); }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] of 16-bit elements; box = box_rows x 64 columns (128 B), 128 B swizzle.
int make_tmap_2d_16bit(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       int dtype) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { set_error("cuTensorMapEncodeTiled entry point not available"); return -1; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) { set_error("TMA base address must be 16-byte aligned"); return -1; }
  if ((cols * 2) % 16 != 0) { set_error("TMA row pitch must be a multiple of 16 bytes (cols=%llu)", (unsigned long long)cols); return -1; }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                   const_cast<void*>(ptr), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r); return -1; }
  return 0;
}

// Row-major fp32 [rows, cols] with 32 x `box_rows` boxes (128-byte rows, 128-byte swizzle): destination of
// bulk tensor reductions.
int make_tmap_2d_f32(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { set_error("cuTensorMapEncodeTiled entry point not available"); return -1; }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (cols * 4) % 16 != 0) {
    set_error("TMA tensor must be 16-byte aligned with a row pitch that is a multiple of 16 bytes");
    return -1;
  }
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * 4};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (fp32) failed with CUresult %d", (int)r); return -1; }
  return 0;
}

int sm_count(int device) {
  static int cached[64] = {0};
  if (device < 0 || device >= 64) return 148;
  if (!cached[device]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
    cached[device] = n;
  }
  return cached[device];
}

int sm_count_current() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  return sm_count(dev);
}

// Communicating GEMM on CTA pairs: the kernel above with PAIR = true, launched as clusters of two.
// Upper bound on the CTAs of the next GEMM launches (0 = all SMs): lets two GEMMs that are launched on different
// streams - a communication-bound fused kernel and a compute-bound one - share the GPU instead of queueing behind
// each other (a persistent grid of one CTA per SM leaves no room for a second kernel).
static int g_max_ctas = 0;
static inline int usable_sms(int device) {
  const int sms = sm_count(device);
  return (g_max_ctas >= 2 && g_max_ctas < sms) ? g_max_ctas : sms;
}

template <int A_MN, int B_MN>
static int launch_comm_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int device, cudaStream_t stream) {
  using S = GemmSmem<256, true>;
  static bool configured[64] = {false};
  auto kern = gemm_tcgen05_kernel<256, A_MN, B_MN, true>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + 255) / 256;
  p.pair = 1;
  const int total = ((p.tiles_m + 1) / 2) * p.tiles_n;
  const int pairs = usable_sms(device) / 2;
  const int grid = 2 * (total < pairs ? total : pairs);
  p.gemm_ctas = grid;
  if (p.ag.n > 1) { p.ag.n_copy = grid; p.ag.ready_target = static_cast<unsigned int>(grid); }   // every CTA pulls a slice
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(GEMM_THREADS); cfg.dynamicSmemBytes = S::TOTAL; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  AXB_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, p));
  return 0;
}

template <int BN, int A_MN, int B_MN>
static int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int device, cudaStream_t stream) {
  using S = GemmSmem<BN>;
  static bool configured[64] = {false};
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, false>;
  p.pair = 0;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int sms = usable_sms(device);
  // every CTA must be resident at once (reducer warps wait for partials of the same launch): grid <= #SMs
  p.gemm_ctas = tiles < sms ? tiles : sms;
  if (p.ag.n > 1) { p.ag.n_copy = p.gemm_ctas; p.ag.ready_target = static_cast<unsigned int>(p.gemm_ctas); }   // every CTA pulls a slice
  const int grid = p.gemm_ctas;
  kern<<<grid, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

template <int A_MN, int B_MN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, int device, cudaStream_t stream) {
  using S = PairSmem;
  static bool configured[64] = {false};
  auto kern = gemm_pair_kernel<A_MN, B_MN>;
  if (!configured[device & 63]) {
    AXB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
    configured[device & 63] = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + PAIR_BN - 1) / PAIR_BN;
  const int total = ((p.tiles_m + 1) / 2) * p.tiles_n * p.nb;
  const int pairs = usable_sms(device) / 2;
  const int grid = 2 * (total < pairs ? total : pairs);
  p.gemm_ctas = grid;
  kern<<<grid, PAIR_THREADS, S::TOTAL, stream>>>(tmA, tmB, p);
  AXB_CUDA(cudaGetLastError());
  return 0;
}

// Tiles per system-scope fence in the fused reductions (AXONN_FLAG_BATCH, default 4, 1..16).
static int flag_batch_setting() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("AXONN_FLAG_BATCH");
    int b = e ? atoi(e) : 4;
    v = b < 1 ? 1 : (b > 16 ? 16 : b);
  }
  return v;
}

// CTA pairs are used for plain GEMMs wide enough to fill the GPU with 256x256 tiles (AXONN_GEMM_2CTA=0 disables).
static bool pair_mode_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("AXONN_GEMM_2CTA"); v = (e && e[0] == '0') ? 0 : 1; }
  return v == 1;
}

}  // namespace axb

static int gemm_common(int layout, const void* A, const void* B, void* C, const void* bias, void* aux, int M, int N,
                       int K, int in_dtype, int out_dtype, int epilogue, int accumulate, int device, void* stream,
                       const AxbArCtx* ar, const AxbAgCtx* ag = nullptr) {
  using namespace axb;
  if (M <= 0 || N <= 0 || K <= 0) { set_error("axb_gemm: empty problem"); return -1; }
  if (layout < 0 || layout > 2) { set_error("axb_gemm: bad layout %d", layout); return -1; }
  if (in_dtype != 0 && in_dtype != 1) { set_error("axb_gemm: operands must be bf16 or fp16"); return -1; }
  if ((N % 8) || (K % 8) || (layout == 2 && (M % 8))) { set_error("axb_gemm: dims must be multiples of 8"); return -1; }
  if ((epilogue == 1 || epilogue == 2) && !bias) { set_error("axb_gemm: epilogue needs bias"); return -1; }
  unsigned int* status_dev = nullptr;
  if (!device_status_word(device, &status_dev)) { set_error("axb_gemm: no status word"); return -1; }

  const int tiles_m = (M + BM - 1) / BM;
  const bool wide = static_cast<long long>(tiles_m) * ((N + 255) / 256) >= sm_count(device);
  int BN = (ar && ar->n > 1) ? ar->bn : (wide ? 256 : 128);
  const bool comm = (ar && ar->n > 1) || (ag && ag->n > 1);
  const bool enough_pairs = static_cast<long long>((tiles_m + 1) / 2) * ((N + 255) / 256) >= sm_count(device) / 2;
  // Communicating GEMMs run on CTA pairs too (same main loop as the plain pair kernel) when the problem fills
  // the GPU with 256-wide tiles; a gathered B (layout 0) then needs shards that are multiples of the 128 rows
  // one CTA of a pair loads.
  const bool comm_pair = comm && BN == 256 && enough_pairs && pair_mode_enabled() &&
                         !(ag && ag->n > 1 && layout == 0 && ag->rows_per_shard % 128 != 0);
  if (!comm_pair && ag && ag->n > 1 && layout == 0 && ag->rows_per_shard % BN != 0) BN = 128;
  const int a_mn = (layout == 2) ? 1 : 0;
  const int b_mn = (layout == 0) ? 0 : 1;

  CUtensorMap tmA, tmB;
  // K-major operand [R, K]: box 64(K) x tile rows.  MN-major operand [K, R]: box 64(R) x 64(K).
  if (a_mn == 0) { if (make_tmap_2d_16bit(&tmA, A, M, K, BM, in_dtype)) return -1; }
  else           { if (make_tmap_2d_16bit(&tmA, A, K, M, BK, in_dtype)) return -1; }
  const bool pair = !comm && BN == 256 && pair_mode_enabled() && enough_pairs;
  if (b_mn == 0) { if (make_tmap_2d_16bit(&tmB, B, N, K, (pair || comm_pair) ? BN / 2 : BN, in_dtype)) return -1; }
  else           { if (make_tmap_2d_16bit(&tmB, B, K, N, BK, in_dtype)) return -1; }

  GemmParams p;
  p.C = C; p.bias = bias; p.aux = aux; p.M = M; p.N = N; p.K = K;
  p.out_dtype = out_dtype; p.in_dtype = in_dtype; p.epilogue = epilogue; p.accumulate = accumulate;
  p.status = status_dev; p.timeout_ns = wait_timeout_ns();
  if (ar && ar->n > 1) {
    p.ar = *ar;
    // CTA pairs index tiles by (pair, CTA of the pair): an odd number of tile rows leaves one unused index per column
    const long long tiles = static_cast<long long>(comm_pair ? (tiles_m + 1) / 2 * 2 : tiles_m) * ((N + BN - 1) / BN);
    if (tiles * 4 > ar->flags_per_src || tiles * 4 * (BN / 32) * 128 > ar->inbox_vecs_per_src) {
      set_error("axb_gemm_ar: communication buffers too small for %lld tiles", tiles);
      return -1;
    }
  } else {
    p.ar.n = 1;
  }
  p.tn_offset = 0; p.kb_offset = 0;
  p.nb = 1; p.a_batch_rows = p.b_batch_rows = p.c_batch_rows = 0;
  p.seg_counts = nullptr; p.seg_rows = 0; p.nseg = 0; p.mask_mode = 0;
  p.flag_batch = flag_batch_setting();
  p.debug = 0;
#ifdef AXB_ABLATION
  { static int dbg = -1; if (dbg < 0) { const char* e = getenv("AXB_AR_DEBUG"); dbg = e ? atoi(e) : 0; } p.debug = dbg; }
#endif
  if (ag && ag->n > 1) {
    p.ag = *ag;
    AXB_CUDA(cudaMemsetAsync(p.ag.shard_ready, 0, 8 * sizeof(unsigned int), static_cast<cudaStream_t>(stream)));
    if (layout == 0) {
      if (ag->rows_per_shard % (comm_pair ? 128 : BN) != 0 || static_cast<long long>(ag->rows_per_shard) * ag->n != N) {
        set_error("axb_ag_gemm: shard rows (%d) must be a multiple of %d and n*rows == N", ag->rows_per_shard, comm_pair ? 128 : BN);
        return -1;
      }
      // With the all-reduce epilogue every rank must walk the tiles in the same order (partials are matched
      // by tile index and a rank waits for its peers' partial of the tile it finished one step earlier).
      p.tn_offset = (ar && ar->n > 1) ? 0 : ag->rank * (ag->rows_per_shard / BN);
    } else if (layout == 1) {
      if (ag->rows_per_shard % BK != 0 || static_cast<long long>(ag->rows_per_shard) * ag->n != K) {
        set_error("axb_ag_gemm: shard rows (%d) must be a multiple of %d and n*rows == K", ag->rows_per_shard, BK);
        return -1;
      }
      p.kb_offset = ag->rank * (ag->rows_per_shard / BK);
    } else {
      set_error("axb_ag_gemm: layout must be 0 or 1");
      return -1;
    }
  } else {
    p.ag.n = 1;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (comm_pair) {
    if (layout == 0) return launch_comm_pair<0, 0>(tmA, tmB, p, device, s);
    if (layout == 1) return launch_comm_pair<0, 1>(tmA, tmB, p, device, s);
    return launch_comm_pair<1, 1>(tmA, tmB, p, device, s);
  }
  if (pair) {
    if (layout == 0) return launch_pair<0, 0>(tmA, tmB, p, device, s);
    if (layout == 1) return launch_pair<0, 1>(tmA, tmB, p, device, s);
    return launch_pair<1, 1>(tmA, tmB, p, device, s);
  }
#define AXB_DISPATCH(BN_, A_, B_) return launch<BN_, A_, B_>(tmA, tmB, p, device, s)
  if (BN == 256) {
    if (layout == 0) AXB_DISPATCH(256, 0, 0);
    if (layout == 1) AXB_DISPATCH(256, 0, 1);
    AXB_DISPATCH(256, 1, 1);
  } else {
    if (layout == 0) AXB_DISPATCH(128, 0, 0);
    if (layout == 1) AXB_DISPATCH(128, 0, 1);
    AXB_DISPATCH(128, 1, 1);
  }
#undef AXB_DISPATCH
}

// Milliseconds the fused GEMM kernels spent stalled on peers since the last reset (sum over launches of the mean
// over each launch's CTAs).  Synchronises the device; `device` must be current.  A diagnostic for reporting exposed
// communication, not for use inside a timed region.
extern "C" void axb_gemm_set_max_ctas(int n) { axb::g_max_ctas = n; }

extern "C" double axb_comm_stall_ms(int device, int reset) {
  (void)device;
  unsigned long long v = 0;
  if (cudaMemcpyFromSymbol(&v, axb::g_comm_stall, sizeof(v)) != cudaSuccess) return -1.0;
  if (reset) {
    const unsigned long long z = 0;
    cudaMemcpyToSymbol(axb::g_comm_stall, &z, sizeof(z));
  }
  return static_cast<double>(v) / 1024.0 / 1e6;
}

// nb problems of one shape in one launch of the CTA-pair kernel (the expert GEMMs of a mixture-of-experts layer):
// A, B and C are 2-D arrays in which problem e starts e * {a,b,c}_batch_rows rows below problem 0.  Layouts as in
// axb_gemm.  Tiles may run past a problem's M and N (those rows and columns are not stored), but an operand whose
// rows are the reduction dimension (B in layout 1, A and B in layout 2) needs K to be a multiple of 64 so that no
// K block reads the next problem's rows.
//
// seg_counts (device, int32 [nb, nseg]; nullptr = no mask): the M rows (layouts 0 and 1) or the K rows (layout 2)
// of every problem are nseg segments of seg_rows rows, of which only the first seg_counts[e][s] hold data and the
// others are zero.  Tiles (K blocks in layout 2) without a data row are skipped; a skipped tile is stored as zeros.
extern "C" int axb_gemm_batched(int layout, const void* A, const void* B, void* C, int nb, int M, int N, int K,
                                int a_batch_rows, int b_batch_rows, int c_batch_rows, int in_dtype, int out_dtype,
                                int accumulate, const int* seg_counts, int seg_rows, int nseg, int device,
                                void* stream) {
  using namespace axb;
  if (nb <= 0 || M <= 0 || N <= 0 || K <= 0) { set_error("axb_gemm_batched: empty problem"); return -1; }
  if (layout < 0 || layout > 2) { set_error("axb_gemm_batched: bad layout %d", layout); return -1; }
  if (in_dtype != 0 && in_dtype != 1) { set_error("axb_gemm_batched: operands must be bf16 or fp16"); return -1; }
  if ((N % 8) || (K % 8) || (layout == 2 && (M % 8))) { set_error("axb_gemm_batched: dims must be multiples of 8"); return -1; }
  if (layout != 0 && K % BK) { set_error("axb_gemm_batched: K must be a multiple of %d in layouts 1 and 2", BK); return -1; }
  const int a_mn = (layout == 2) ? 1 : 0, b_mn = (layout == 0) ? 0 : 1;
  const int a_rows = a_mn ? K : M, b_rows = b_mn ? K : N;
  if (a_batch_rows < a_rows || b_batch_rows < b_rows || c_batch_rows < M) {
    set_error("axb_gemm_batched: problems overlap (batch strides %d %d %d)", a_batch_rows, b_batch_rows, c_batch_rows);
    return -1;
  }
  unsigned int* status_dev = nullptr;
  if (!device_status_word(device, &status_dev)) { set_error("axb_gemm_batched: no status word"); return -1; }
  CUtensorMap tmA, tmB;
  const uint64_t a_total = static_cast<uint64_t>(a_batch_rows) * (nb - 1) + a_rows;
  const uint64_t b_total = static_cast<uint64_t>(b_batch_rows) * (nb - 1) + b_rows;
  if (a_total > 0x7fffffffull || b_total > 0x7fffffffull) { set_error("axb_gemm_batched: stacked operands too tall"); return -1; }
  if (a_mn == 0) { if (make_tmap_2d_16bit(&tmA, A, a_total, K, BM, in_dtype)) return -1; }
  else           { if (make_tmap_2d_16bit(&tmA, A, a_total, M, BK, in_dtype)) return -1; }
  if (b_mn == 0) { if (make_tmap_2d_16bit(&tmB, B, b_total, K, PAIR_BN / 2, in_dtype)) return -1; }
  else           { if (make_tmap_2d_16bit(&tmB, B, b_total, N, BK, in_dtype)) return -1; }
  GemmParams p;
  p.C = C; p.bias = nullptr; p.aux = nullptr; p.M = M; p.N = N; p.K = K;
  p.out_dtype = out_dtype; p.in_dtype = in_dtype; p.epilogue = 0; p.accumulate = accumulate;
  p.status = status_dev; p.timeout_ns = wait_timeout_ns();
  p.ar.n = 1; p.ag.n = 1; p.tn_offset = 0; p.kb_offset = 0; p.flag_batch = 1; p.debug = 0; p.pair = 1;
  p.nb = nb; p.a_batch_rows = a_batch_rows; p.b_batch_rows = b_batch_rows; p.c_batch_rows = c_batch_rows;
  p.seg_counts = nullptr; p.seg_rows = 0; p.nseg = 0; p.mask_mode = 0;
  if (seg_counts) {
    const long long masked = (layout == 2) ? K : M;
    if (seg_rows <= 0 || nseg <= 0 || static_cast<long long>(seg_rows) * nseg != masked) {
      set_error("axb_gemm_batched: %d segments of %d rows do not cover the masked dimension (%lld)", nseg, seg_rows, masked);
      return -1;
    }
    p.seg_counts = seg_counts; p.seg_rows = seg_rows; p.nseg = nseg; p.mask_mode = (layout == 2) ? 2 : 1;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (layout == 0) return launch_pair<0, 0>(tmA, tmB, p, device, s);
  if (layout == 1) return launch_pair<0, 1>(tmA, tmB, p, device, s);
  return launch_pair<1, 1>(tmA, tmB, p, device, s);
}

extern "C" int axb_gemm(int layout, const void* A, const void* B, void* C, const void* bias, void* aux, int M, int N,
                        int K, int in_dtype, int out_dtype, int epilogue, int accumulate, int device, void* stream) {
  return gemm_common(layout, A, B, C, bias, aux, M, N, K, in_dtype, out_dtype, epilogue, accumulate, device, stream,
                     nullptr);
}

// C = allreduce_over_ranks(op(A) op(B)) (+bias, GELU): every rank of the group calls this with its partial
// operands; the epilogue exchanges bf16 partial tiles through peer-mapped inboxes (see AxbArCtx).
// C = op(A) op(B) where B ([N,K] for layout 0, [K,N] for layout 1) is the concatenation along its rows of one
// shard per rank: the kernel pulls the shards from the ranks' outboxes into `ag->staging` (which holds the
// complete B afterwards) while the tiles that only need already-present shards are being computed.  The B
// argument of the GEMM is `ag->staging`.  May be combined with the all-reduce epilogue (`ar`, optional).
extern "C" int axb_ag_gemm(int layout, const void* A, void* C, const void* bias, void* aux, int M, int N, int K,
                           int in_dtype, int out_dtype, int epilogue, int device, void* stream, const AxbAgCtx* ag,
                           const AxbArCtx* ar) {
  if (!ag || ag->n < 2 || ag->n > 8) { axb::set_error("axb_ag_gemm: group size must be 2..8"); return -1; }
  if (ag->shard_bytes % 16) { axb::set_error("axb_ag_gemm: shard size must be a multiple of 16 bytes"); return -1; }
  return gemm_common(layout, A, ag->staging, C, bias, aux, M, N, K, in_dtype, out_dtype, epilogue, 0, device, stream,
                     (ar && ar->n > 1) ? ar : nullptr, ag);
}

// C_shard[rows_per_shard, N] (+)= reduce_scatter_over_ranks(op(A) op(B)) along the rows of the product:
// rank o receives rows [o * rows_per_shard, (o + 1) * rows_per_shard).  M must equal n * rows_per_shard.
extern "C" int axb_gemm_rs(int layout, const void* A, const void* B, void* C_shard, int M, int N, int K, int in_dtype,
                           int out_dtype, int accumulate, int device, void* stream, const AxbArCtx* ar) {
  if (!ar || ar->n < 2 || ar->n > 8) { axb::set_error("axb_gemm_rs: group size must be 2..8"); return -1; }
  if (ar->mode != 1 || ar->rows_per_shard <= 0 || ar->rows_per_shard % 32 != 0 ||
      static_cast<long long>(ar->rows_per_shard) * ar->n != M) {
    axb::set_error("axb_gemm_rs: rows_per_shard must be a multiple of 32 with n * rows_per_shard == M");
    return -1;
  }
  if (ar->bn != 128 && ar->bn != 256) { axb::set_error("axb_gemm_rs: bn must be 128 or 256"); return -1; }
  return gemm_common(layout, A, B, C_shard, nullptr, nullptr, M, N, K, in_dtype, out_dtype, 0, accumulate, device,
                     stream, ar);
}

extern "C" int axb_gemm_ar(int layout, const void* A, const void* B, void* C, const void* bias, void* aux, int M,
                           int N, int K, int in_dtype, int out_dtype, int epilogue, int device, void* stream,
                           const AxbArCtx* ar) {
  if (!ar || ar->n < 2 || ar->n > 8) { axb::set_error("axb_gemm_ar: group size must be 2..8"); return -1; }
  if (ar->bn != 128 && ar->bn != 256) { axb::set_error("axb_gemm_ar: bn must be 128 or 256"); return -1; }
  if (ar->mode != 0 && ar->mode != 2) { axb::set_error("axb_gemm_ar: context is not in all-reduce mode"); return -1; }
  if (ar->mode == 2 && out_dtype == 2) { axb::set_error("axb_gemm_ar: the two-shot all-reduce stores 16-bit outputs only"); return -1; }
  return gemm_common(layout, A, B, C, bias, aux, M, N, K, in_dtype, out_dtype, epilogue, 0, device, stream, ar);
}
