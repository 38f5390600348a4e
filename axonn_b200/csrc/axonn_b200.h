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
int axb_gemm(int layout, const void* A, const void* B, void* C, const void* bias, void* aux,
             int M, int N, int K, int in_dtype, int out_dtype, int epilogue, int accumulate,
             int device, void* stream);

#ifdef __cplusplus
}
#endif
