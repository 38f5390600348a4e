/* C interface of libaxonn_b200.so: launchers for the sm_100a kernels.
 *
 * Every function returns 0 on success and non-zero on failure, in which case
 * axb_last_error() describes the problem.  Pointers are device pointers unless
 * said otherwise; `stream` is a cudaStream_t.  Launchers never synchronise.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* axb_last_error(void);
/* Status word set by kernels whose bounded waits expired (0 = clean); reading
 * clears it when `clear` is non-zero.  Host-mapped: no device sync needed. */
unsigned int axb_device_status(int device, int clear);

/* dtype codes: 0 = bf16, 1 = fp16, 2 = fp32 */

/* C[M,N] = op(A) * op(B) on tcgen05 tensor cores (fp32 accumulate in TMEM).
 *   layout 0: A[M,K] row-major, B[N,K] row-major   (C = A  B^T)
 *   layout 1: A[M,K] row-major, B[K,N] row-major   (C = A  B)
 *   layout 2: A[K,M] row-major, B[K,N] row-major   (C = A^T B)
 * epilogue: 0 none, 1 +bias[N], 2 +bias then GELU(tanh), 3 GELU; with GELU the
 * pre-activation is also written to `aux` when it is non-null.
 * accumulate != 0: C += result.  Dimensions must be multiples of 8. */
/* nb problems of one shape in one launch: problem e starts e * {a,b,c}_batch_rows rows below problem 0 in the
   stacked 2-D operands; layouts 1 and 2 need K % 64 == 0.  With seg_counts the masked dimension (M; K in layout 2)
   is nseg segments of seg_rows rows whose first seg_counts[e][s] rows hold data (the rest are zero): tiles or K
   blocks without data are skipped, skipped tiles are stored as zeros */
int axb_gemm_batched(int layout, const void* A, const void* B, void* C, int nb, int M, int N, int K,
                     int a_batch_rows, int b_batch_rows, int c_batch_rows, int in_dtype, int out_dtype,
                     int accumulate, const int* seg_counts /* device int32 [nb, nseg] or NULL */, int seg_rows,
                     int nseg, int device, void* stream);
/* cap on the CTAs of the following GEMM launches (0: one per SM), for GEMMs that share the GPU from two streams */
void axb_gemm_set_max_ctas(int n);
int axb_gemm(int layout, const void* A, const void* B, void* C, const void* bias, void* aux,
             int M, int N, int K, int in_dtype, int out_dtype, int epilogue, int accumulate,
             int device, void* stream);

/* Peer-memory context of the fused GEMM + all-reduce / reduce-scatter.  All pointers are device addresses:
 * the *_local ones in this rank's symmetric buffer, the *_peer[j] ones the same regions of rank j mapped
 * into this process.  `inbox_*` holds bf16 partial tiles indexed [source rank][tile][warp]: every rank's
 * GEMM epilogue pushes its partial into the inbox of the ranks that reduce those rows (posted stores over
 * NVLink for peers), whose reducer warps sum the slots locally.  Flag
 * arrays are indexed [source rank][tile * 4 + warp]; `epoch` increases by one per call on the group and
 * selects (by parity, done by the caller) which of two outbox/flag sets is used. */
typedef struct AxbArCtx {
  int n;                      /* ranks in the group (2..8) */
  int rank;                   /* this rank's index in the group */
  unsigned int epoch;         /* call sequence number (>= 2) */
  int bn;                     /* tile width all ranks agreed on: 128 or 256 */
  void* inbox_local;          /* my inbox: partial tiles written by peers */
  void* inbox_peer[8];        /* peer j's inbox */
  unsigned int* flags_local;  /* per (source, tile, warp) arrival flags written by peers */
  unsigned int* flags_peer[8];
  unsigned int* done_local;   /* [source] last call the peer has completed */
  unsigned int* done_peer[8];
  unsigned int* counter;      /* local CTA completion counter (zero between calls) */
  unsigned long long inbox_vecs_per_src; /* 16-byte words per source in an inbox */
  unsigned long long flags_per_src;      /* flags per source */
  int mode;                   /* 0: one-shot all-reduce of C (every rank receives and sums every partial);
                                 1: reduce-scatter of C by row blocks;
                                 2: two-shot all-reduce: every 32-row unit (tile, warp) has one owner rank,
                                    (tile * 4 + warp) % n, which receives the partials, sums them and stores the
                                    finished values into C on every rank.  C (and aux) must then lie in a range
                                    that all ranks of the group have mapped ("arena"); each rank announces the
                                    offsets of its C and aux in that range through the mailbox, and the kernel
                                    returns only after every peer has finished writing into this rank's C. */
  int rows_per_shard;         /* mode 1: rows of C owned by each rank (multiple of 32) */
  int comm_ctas;              /* reserved, must be 0 */
  int loopback;               /* mode 2 on one GPU with aliased peer pointers (tests, profiling): owned units are
                                 stored for both source slots, so that the kernel only waits on its own flags */
  unsigned long long c_off;   /* mode 2: byte offset of C inside this rank's arena */
  unsigned long long aux_off; /* mode 2: byte offset of aux inside this rank's arena (unused when aux is null) */
  void* arena_peer[8];        /* mode 2: base of rank j's arena as mapped in this process */
  unsigned int* mail_local;   /* mode 2: [source] records of 8 words {c_off lo, hi, aux_off lo, hi, epoch, -, -, -} */
  unsigned int* mail_peer[8];
} AxbArCtx;

/* Peer-memory context of the fused all-gather -> GEMM: B's row blocks ("shards", one per rank) are pulled
 * from the owners' outboxes into a local staging copy of B while the tiles that need only shards already
 * present are computed.  Every CTA of the GEMM brings in its slice of every shard: one thread per CTA runs
 * bulk copies peer outbox -> shared memory -> staging, two 8 KB buffers in flight.  `wait_local[j]` reaches
 * `epoch` when rank j has published its shard; `shard_ready[z]` is a local counter that reaches the number
 * of CTAs when shard z is complete (`n_copy` and `ready_target` are set by the launcher). */
typedef struct AxbAgCtx {
  int n, rank;
  unsigned int epoch;
  int n_copy;
  const void* outbox_peer[8];
  void* staging;
  unsigned long long shard_bytes;
  unsigned int* shard_ready;
  unsigned int ready_target;
  int rows_per_shard;
  unsigned int* wait_local;
  unsigned int* done_peer[8];
  unsigned int* counter;
} AxbAgCtx;

int axb_ag_gemm(int layout, const void* A, void* C, const void* bias, void* aux, int M, int N, int K, int in_dtype,
                int out_dtype, int epilogue, int device, void* stream, const AxbAgCtx* ag, const AxbArCtx* ar);

int axb_gemm_rs(int layout, const void* A, const void* B, void* C_shard, int M, int N, int K, int in_dtype,
                int out_dtype, int accumulate, int device, void* stream, const AxbArCtx* ar);

int axb_gemm_ar(int layout, const void* A, const void* B, void* C, const void* bias, void* aux, int M, int N, int K,
                int in_dtype, int out_dtype, int epilogue, int device, void* stream, const AxbArCtx* ar);

/* Peer-memory context of the MoE token exchange kernels.  `wait_local[j]` must reach `wait_value` before the
 * kernel touches remote memory; when the kernel has finished it writes `epoch` to `signal_peer[j][rank]`. */
typedef struct AxbMoeCtx {
  int n, rank;
  unsigned int epoch;
  int n_local;
  void* buf_peer[8];
  unsigned int* wait_local;
  unsigned int wait_value;
  unsigned int* signal_peer[8];
  unsigned int* counter;
  int* cnt_peer[8];   /* dispatch only, may be NULL: rank j's table [n_local][n] of rows that every source sent per expert */
} AxbMoeCtx;

int axb_moe_dispatch(const void* x, int x_by_token, const long long* dest, const unsigned char* keep,
                     const long long* counts, int T, int k, int E, int C, int H, const AxbMoeCtx* ctx, int device,
                     void* stream);
int axb_moe_gather(void* out, const long long* dest, const unsigned char* keep, int T, int k, int C, int H,
                   const AxbMoeCtx* ctx, int device, void* stream);
int axb_moe_signal(const AxbMoeCtx* ctx, int device, void* stream);
/* wait for the flags of ctx, copy src into this rank's peer-readable dst, publish ctx->epoch: one launch */
int axb_copy_publish(const void* src, void* dst, long long nbytes, const AxbMoeCtx* ctx, int device, void* stream);
int axb_moe_wait(const AxbMoeCtx* ctx, int device, void* stream);

/* Peer-memory context of the gradient all-reduce kernels (see AxbMoeCtx for the flag conventions). */
typedef struct AxbCommCtx {
  int n, rank;
  unsigned int epoch;
  int pad;
  void* buf_peer[8];
  unsigned int* wait_local;
  unsigned int* signal_peer[8];
  unsigned int* counter;
} AxbCommCtx;

/* Peer-memory context of the row all-to-all and embedding kernels (p2p.cu).  `base_peer[j]`: for the row
 * all-to-all the base of rank j's output arena (the destination tensor of rank j lies at the offset rank j
 * announces through the mailbox); for the embedding kernels rank j's published table shard / gradient shard.
 * Mailbox records are 8 words per source rank: {offset lo, offset hi, -, -, epoch, -, -, -}. */
typedef struct AxbP2pCtx {
  int n, rank;
  unsigned int epoch;
  int pad;
  void* base_peer[8];
  unsigned int* mail_local;
  unsigned int* mail_peer[8];
  unsigned int* done_local;
  unsigned int* done_peer[8];
  unsigned int* counter;       /* two words: CTA counter, failed-CTA counter (zero between calls) */
  unsigned long long out_off;  /* row all-to-all: byte offset of my output tensor inside my arena */
} AxbP2pCtx;

/* One row block per destination rank: `rows` rows of `row_bytes` bytes, read from `src` with pitch `src_pitch`
 * and stored into the destination's output at byte offset `dst_off` with pitch `dst_pitch` (all multiples of 16). */
typedef struct AxbRowBlock {
  const void* src;
  long long src_pitch, dst_off, dst_pitch, rows, row_bytes;
} AxbRowBlock;

int axb_a2a_rows(const AxbP2pCtx* ctx, const AxbRowBlock* blocks /* [n] */, int device, void* stream);
int axb_p2p_publish(const AxbP2pCtx* ctx, int device, void* stream);
int axb_embedding_fetch(const long long* ids, long long n_tokens, void* out, long long row_bytes,
                        long long rows_per_shard, const AxbP2pCtx* ctx, int device, void* stream);
int axb_embedding_scatter_add(const long long* ids, long long n_tokens, const void* dy_bf16, int H,
                              long long rows_per_shard, const AxbP2pCtx* ctx, int device, void* stream);

int axb_bucket_copy(const long long* table, int ntensors, long long total_chunks, void* bucket, int dtype, int direction,
                    const AxbCommCtx* ctx, int device, void* stream);
int axb_allreduce_twoshot(long long nbytes, int dtype, float scale, const AxbCommCtx* ctx, int device, void* stream);
/* the same reduction inside the NVSwitch (multimem.ld_reduce / multimem.st on the bucket's multicast address) */
int axb_allreduce_nvls(long long nbytes, int dtype, float scale, void* mc_bucket, const AxbCommCtx* ctx, int device,
                       void* stream);

/* Peer-memory context of the one-kernel gradient all-reduce (allreduce.cu::grad_allreduce_kernel). */
typedef struct AxbGradArCtx {
  int n, rank;
  unsigned int epoch;
  int pad;
  void* recv_peer[8];            /* rank j's receive area: n slots (one per source rank) of slot_bytes */
  void* result_peer[8];          /* rank j's result area */
  unsigned int* pushed_local;    /* [n] epoch flags */
  unsigned int* pushed_peer[8];
  unsigned int* reduced_local;
  unsigned int* reduced_peer[8];
  unsigned int* counters;        /* 3 words, zero between calls */
  unsigned long long slot_bytes;
} AxbGradArCtx;
/* dtype here: 0 fp32, 1 bf16 (the bucket kernels' own codes) */
int axb_grad_allreduce(const long long* table, int ntensors, long long total_chunks, long long chunks_per_slice,
                       int dtype, float scale, const AxbGradArCtx* ctx, int device, void* stream);

/* ---- runtime helpers (common.cu) */
void axb_set_wait_timeout_ms(unsigned int ms);   /* deadline of every device-side wait; default 120000 */
unsigned int axb_debug_word(int device, int index, int clear);   /* diagnostic words 1..15 next to the status word */
double axb_comm_stall_ms(int device, int reset); /* time the fused GEMM kernels spent stalled on peers; synchronises */

/* ---- elementwise kernels (elementwise.cu); bf16 tensors, n / F multiples of 8 */
int axb_gelu_fwd(const void* x, void* y, long long n, void* stream);
int axb_gelu_bwd(const void* dy, const void* x, void* dx, long long n, void* stream);
int axb_swiglu_fwd(const void* gate_up, void* out, int T, int F, void* stream);   /* gate|up interleaved in blocks of 8 */
int axb_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, int T, int F, void* stream);
/* rotary embedding in place on rows of nh heads of D elements; cs: [positions, D/2, 2] cos/sin table */
int axb_rope(void* x, const float* cs, long long rows, int S, int nh, int D, int pos_div, long long row_stride,
             int inverse, void* stream);

/* ---- flash attention on the packed projection output [B, S, G, qpk + 2, D] (flash_attn.cu); D 64 or 128, S % 128 == 0 */
int axb_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int G, int qpk, int D, float scale,
                       int device, void* stream);
int axb_flash_attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta, float* dq_acc,
                       void* dqkv, int B, int S, int G, int qpk, int D, float scale, int device, void* stream);
/* two-kernel backward without atomics; which: bit 0 = dQ kernel (query slots of dqkv), bit 1 = dK / dV kernel */
int axb_flash_attn_bwd_split(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
                             void* dqkv, int B, int S, int G, int qpk, int D, float scale, int which, int device,
                             void* stream);

/* ---- cross entropy on a vocabulary shard of bf16 logits (loss.cu); backward overwrites the logits with their gradient */
int axb_ce_fwd(const void* logits, const long long* targets, float* stats, int rows, int V, int vocab_start, void* stream);
int axb_ce_bwd(void* logits, const long long* targets, const float* lse, const float* scale, int rows, int V,
               int vocab_start, long long ignore_index, void* stream);

/* ---- LayerNorm / RMSNorm and column sums (norm.cu) */
int axb_norm_grid(int device, int rows);
int axb_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* stats, int rows, int H, int H_total,
                 float eps, int rms, int mode, int dtype, int device, void* stream);
/* dgamma / dbeta are written in `param_dtype`, column sums in `out_dtype` (the dtype codes above) */
int axb_norm_bwd(const void* dy, const void* x, const void* gamma, const float* stats, void* dx, float* sums,
                 float* dgamma_part, float* dbeta_part, void* dgamma, void* dbeta, int rows, int H, int H_total, int rms,
                 int mode, int dtype, int param_dtype, int device, void* stream);
/* the residual add fused into the norm: y = norm(x + delta), hout = x + delta; dx = norm_backward(dy) + dres */
int axb_add_norm_fwd(const void* x, const void* delta, void* hout, const void* gamma, const void* beta, void* y,
                     float* stats, int rows, int H, int H_total, float eps, int rms, int mode, int dtype, int device,
                     void* stream);
int axb_add_norm_bwd(const void* dy, const void* dres, const void* x, const void* gamma, const float* stats, void* dx,
                     float* sums, float* dgamma_part, float* dbeta_part, void* dgamma, void* dbeta, int rows, int H,
                     int H_total, int rms, int mode, int dtype, int param_dtype, int device, void* stream);
int axb_colsum_splits(int device, int rows, int N);
int axb_colsum(const void* x, float* part, void* out, int rows, int N, int dtype, int out_dtype, int device, void* stream);
int axb_gelu_bwd_colsum(const void* dy, const void* x, void* dx, float* part, void* colsum, int rows, int N, int dtype,
                        int out_dtype, int device, void* stream);

/* ---- multi-tensor kernels over a device table of tensor pointers (optim.cu) */
int axb_multi_l2norm_sq(const long long* table, int n, long long total_chunks, float* out, void* stream);
int axb_multi_scale(const long long* table, int n, long long total_chunks, const float* scale, void* stream);
/* SGD with momentum over a pointer table (rows {param, grad, fp32 momentum buffer, numel, param dtype, grad dtype,
   chunk prefix, 0}; dtype codes 0 fp32, 1 bf16, 2 fp16) */
int axb_multi_sgd(const long long* table, int n, long long total_chunks, float lr, float momentum, float weight_decay,
                  const float* grad_scale, void* stream);
int axb_multi_adamw(const long long* table, int n, long long total_chunks, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bias_c1, float bias_c2, const float* grad_scale, const float* found_inf,
                    void* stream);

/* ---- output arena (arena.cu): host-side allocator over a registered peer-mapped range; the malloc / free pair
 * has the signature of torch's pluggable-allocator hook */
int axb_arena_register(int device, void* base, unsigned long long nbytes);
void* axb_arena_malloc(long long size, int device, void* stream);
void axb_arena_free(void* ptr, long long size, int device, void* stream);
unsigned long long axb_arena_stat(int device, int what);
int axb_arena_contains(int device, const void* ptr, unsigned long long nbytes);

/* ---- symmetric heap (symm_heap.cu): one allocation per rank (backend 0: host memory, 1: device memory through the
 * CUDA virtual-memory-management API), all ranks' allocations mapped into one range, slot p = rank p.  The file
 * descriptors returned by axb_heap_fd travel between the processes in the Python layer.  axb_heap_info: 0 = base
 * address, 1 = bytes per slot, 2 = slots mapped, 3 = backend. */
int axb_heap_create(int backend, int device, int rank, int nranks, unsigned long long bytes, void** out_heap);
int axb_heap_fd(void* heap);
int axb_heap_attach(void* heap, int peer, int fd);
unsigned long long axb_heap_info(void* heap, int what);
int axb_heap_destroy(void* heap);

/* ---- top-k gradient pruning (prune.cu): keep the k largest |g|, zero the rest, in place.
 * dtype: the codes above (0 bf16, 1 fp16, 2 fp32).  `work`: device scratch of axb_prune_workspace_words() 32-bit words. */
int axb_prune_workspace_words(void);
int axb_prune_topk(void* g, long long n, int dtype, long long k, void* work, int device, void* stream);

/* Top-k gradient pruning for callers that cannot allocate device memory (programs that own the whole GPU
 * through their own pool, or that forbid allocation after start-up).  This entry point has no counterpart
 * in the reference project.  Same result and same dtype codes (0 bf16, 1 fp16, 2 fp32) as axb_prune_topk,
 * but the radix-select scratch is a 393,248-byte array inside the library image, held on every GPU that
 * loads the library until the process exits.  `device` must be the calling thread's current device on
 * every call (checked).  The first call on a device also resolves the array's address: make it before any
 * stream capture.  n is limited to 2,147,483,647 elements.  Calls share the scratch: they must not overlap
 * on the GPU. */
int axb_prune_topk_static(void* g, long long n, int dtype, long long k, int device, void* stream);

#ifdef __cplusplus
}
#endif
