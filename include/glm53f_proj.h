/* The projections either side of the KDA core, for B200 (sm_100a): a bf16 GEMM on the tcgen05 tensor cores.
 *
 * What this replaces.  A KDA layer of the reference projects its normed input with Gemm::bf16
 * (crates/glm53f-forward/src/gemm.rs:212-235) at crates/glm53f-forward/src/forward.rs:3494-3542 (the fused
 * [q|k|v|b] weight 4096 -> 24,640; the low-rank gate pair 4096 -> 256 and, in two groups, 128 -> 8192) and
 * forward.rs:3772-3790 (o_proj 8192 -> 4096).  Gemm::bf16 sends 1..8 rows to the crate's CUDA-core GEMV
 *
 *     glm53f_fwd_gemv_bf16   crates/glm53f-forward/kernels/glm53f_forward.h:19-40, bound by src/ffi.rs
 *
 * and more rows to cuBLAS (gemm.rs:296-324).  The call below takes the GEMV's arguments (minus its split-K scratch)
 * with the same meaning and serves every row count, so the forward would call it in place of both.
 */
#ifndef GLM53F_PROJ_H
#define GLM53F_PROJ_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GLM53F_STREAM_T_DEFINED
#define GLM53F_STREAM_T_DEFINED
typedef struct CUstream_st* glm53f_stream_t; /* cudaStream_t; NULL = the legacy default stream */
#endif

/* out[g][m][o] = sum_k x[g][m][k] * w[g][o][k] for groups g < groups, rows m < rows, outputs o < n:
 * x at x + g * x_gstride + m * ldx, w row o at w + g * w_gstride + o * ldw, out at out + g * o_gstride + m * ldo
 * (strides in elements; x and w bf16; out bf16, or f32 when out_f32 != 0).  Products are exact, sums accumulate in
 * f32 in k order; in launches of up to 512 rows a row's result depends on that row and on (groups, n, k) only, never on
 * `rows` (bit for bit: the tile shape's accumulation and the K split are chosen from (groups, n, k)); larger launches
 * use wider tiles without a K split and agree with them to the order of the f32 sums.
 *
 * n % 8 == 0; k % 64 == 0; ldx, ldw, x_gstride, w_gstride % 8 == 0; ldx, ldw >= k; ldo >= n; x and w 16-byte
 * aligned.  The group strides are read only when groups > 1.  rows == 0 launches nothing.  Returns 0, 1
 * (cudaErrorInvalidValue) for a rejected argument, or another cudaError_t value.  Asynchronous on `stream`;
 * allocates nothing. */
int32_t glm53f_kda_proj_bf16(const uint16_t* x, int64_t ldx, int64_t x_gstride, const uint16_t* w, int64_t ldw,
                             int64_t w_gstride, int32_t groups, int32_t rows, int32_t n, int32_t k, void* out,
                             int32_t out_f32, int64_t ldo, int64_t o_gstride, glm53f_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GLM53F_PROJ_H */
