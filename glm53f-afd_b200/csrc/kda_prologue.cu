// The layer prologue of the chunked forms: projection rows to the core's inputs.
//
// The layer entry points take the engine's rows (q | k | v projections, beta logits, the forget-gate row); the chunked
// tensor-core kernels take what the recurrence is defined on: q and k after the short convolution, SiLU and the L2
// norms, v after the convolution and SiLU, the per-channel decay and beta.  This kernel computes those with the
// chain's own arithmetic (reference kernels/kda.cu:129-165 = kernels/kda_prefill.cu:121-208; this file is compiled
// without multiply-add contraction like the chain): four taps summed in order, one bf16 rounding after the SiLU, decay
// exp(lower * sigmoid(exp(A_log) (a + dt_bias))), beta = bf16(sigmoid(b)), each L2 norm as a lane's four consecutive
// channels summed in order, then the xor butterfly.  (Bit for bit in the verify sink; the prefill sink uses the
// hardware's approximate division, exponential and reciprocal root, see sigmoid_ below.)
//
// One warp per (request, head, row); a lane owns four consecutive channels, so the norms need no shared memory.  The
// work is bound by instruction issue (about 850 instructions per row and lane, most of them IEEE divisions and
// exponentials), so a warp takes ONE row and reads its three predecessors again (the four warps of a block take four
// consecutive rows; the predecessors come from L1/L2): every load of a warp is in flight at once and 79 registers
// allow 24 resident warps per SM.  (A warp that walks 16 rows with the three earlier rows sliding in registers needs
// 143 registers and was half as fast.)
//
// Two sinks:
//  * a prefill pass: dense core inputs for one pass of rows in the caller's workspace.  q and k are rounded to fp16
//    (they lie in [-1, 1]; eleven mantissa bits), the one place where the chunked prefill departs from the chain's
//    FP32 q and k before the tensor-core products: with bf16's eight bits the rounding of k alone, which reaches the
//    state through K^T D, would take the state's whole error budget when few rows dominate it.  The decay is kept as
//    its logarithm.
//  * a verify call (VERIFY): the call's own buffers take the results, so nothing is allocated -- k (f32), v, the decay
//    multiplier exp(log decay) and beta go to the replay saves, which a verify call must write anyway and which hold
//    exactly these values (the bits the exact form saves), and q goes, as fp16, to the 256 bytes of `out` that the
//    same (row, head) output will overwrite.  Windows of up to 16 rows.

#include <cuda_fp16.h>

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"

namespace kda {
namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr int kVerifyWindow = 16;

struct ProParams {
    int H, batch, pass_rows, row_shift;  // rows row_shift .. row_shift + pass_rows - 1 of every request
    const int32_t* cu;
    const uint16_t* P;
    long long p_stride, b_off;
    const uint16_t* A;
    long long a_stride;
    const uint16_t* conv;
    const long long* conv_off;
    const uint16_t* cw;
    const float* a_log;
    const float* dt_bias;
    float lower;
    // prefill pass: [batch * pass_rows][H][128] (beta [batch * pass_rows][H])
    uint16_t *q, *k, *v;
    float *g, *beta;
    // verify: q as fp16 into the output rows (through `q`), the rest into the replay saves
    long long out_stride;
    float *k_save, *g_save, *b_save;
    uint16_t* v_save;
};

// The verify sink keeps the chain's IEEE arithmetic (its results are the replay saves, bit for bit); the prefill sink
// feeds tensor-core products that round every operand to bf16 anyway, so there the divisions, exponentials and
// reciprocal roots are the hardware approximations (a few ulp of FP32): a third of the instructions.
template <bool FAST>
__device__ __forceinline__ float sigmoid_(float x) {
    if constexpr (FAST) return __fdividef(1.0f, 1.0f + __expf(-x));
    else return 1.0f / (1.0f + expf(-x));
}
template <bool FAST>
__device__ __forceinline__ float silu_(float x) {
    if constexpr (FAST) return __fdividef(x, 1.0f + __expf(-x));
    else return x / (1.0f + expf(-x));
}
template <bool FAST>
__device__ __forceinline__ float inv_norm_(float ss) {
    if constexpr (FAST) return rsqrtf(ss + 1e-6f);
    else return 1.0f / sqrtf(ss + 1e-6f);
}
__device__ __forceinline__ float butterfly(float x) {
#pragma unroll
    for (int o = 16; o; o >>= 1) x = x + __shfl_xor_sync(FULL, x, o);
    return x;
}
__device__ __forceinline__ void unpack4(uint2 w, float (&x)[4]) {
    x[0] = __uint_as_float(w.x << 16);
    x[1] = __uint_as_float(w.x & 0xffff0000u);
    x[2] = __uint_as_float(w.y << 16);
    x[3] = __uint_as_float(w.y & 0xffff0000u);
}
__device__ __forceinline__ uint2 pack4_fp16(const float (&x)[4]) {
    const __half2 lo = __floats2half2_rn(x[0], x[1]), hi = __floats2half2_rn(x[2], x[3]);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}
__device__ __forceinline__ uint2 pack4(const float (&x)[4]) {
    return make_uint2((uint32_t)f32_to_bf16_bits(x[0]) | ((uint32_t)f32_to_bf16_bits(x[1]) << 16),
                      (uint32_t)f32_to_bf16_bits(x[2]) | ((uint32_t)f32_to_bf16_bits(x[3]) << 16));
}

template <bool VERIFY>
__global__ void __launch_bounds__(128, 6) layer_prologue_kernel(const ProParams p) {
    const int lane = threadIdx.x & 31, H = p.H;
    // a block = four consecutive rows of one (request, head): neighbours share their predecessors in L1
    const int quads = p.pass_rows / 4;
    const long long unit = blockIdx.x / quads;
    const int j_first = (int)(blockIdx.x % quads) * 4 + (threadIdx.x >> 5);  // row of the pass
    const int h = (int)(unit % H), b = (int)(unit / H);
    // A prefill pass covers pass_rows rows of every request.  A verify window is meant to have at most 16 rows; should one be
    // longer (the chunk kernel then reports status 122 and leaves the rows past 16 without outputs), its replay saves are
    // still written for EVERY row, so that a commit of any prefix replays real values: the warp goes on in steps of 16.
    const int r0 = p.cu[b], n_all = max(p.cu[b + 1] - r0 - p.row_shift, 0), n = VERIFY ? n_all : min(n_all, p.pass_rows);
    for (int j = j_first; j < n; j += p.pass_rows) {
    const int c0 = lane * 4, jj = p.row_shift + j;  // row of the request
    const long long C = 3LL * H * DK, gr = (long long)r0 + jj;
    const uint16_t* window = p.conv + p.conv_off[b];
    uint2 x[TAPS][3];  // [tap: rows jj-3 .. jj][part]; rows before the request's first come from the conv window
#pragma unroll
    for (int d = 0; d < TAPS; ++d) {
        const int rr = jj - 3 + d;
        const uint16_t* row = rr < 0 ? window + (long long)(WINDOW + rr) * C : p.P + ((long long)r0 + rr) * p.p_stride;
#pragma unroll
        for (int part = 0; part < 3; ++part) x[d][part] = *reinterpret_cast<const uint2*>(row + ((long long)part * H + h) * DK + c0);
    }
    uint4 wq[3][2];
#pragma unroll
    for (int part = 0; part < 3; ++part) {
        const uint4* src = reinterpret_cast<const uint4*>(p.cw + (((long long)part * H + h) * DK + c0) * TAPS);
        wq[part][0] = src[0];
        wq[part][1] = src[1];
    }
    const uint2 a_bits = *reinterpret_cast<const uint2*>(p.A + gr * p.a_stride + (long long)h * DK + c0);
    const float4 dtb4 = *reinterpret_cast<const float4*>(p.dt_bias + (long long)h * DK + c0);
    const float blogit = bf16_bits_to_f32(p.P[gr * p.p_stride + p.b_off + h]);
    const float decay_rate = expf(p.a_log[h]);

    float act[3][4];
#pragma unroll
    for (int part = 0; part < 3; ++part) {
        float xv[TAPS][4];
#pragma unroll
        for (int d = 0; d < TAPS; ++d) unpack4(x[d][part], xv[d]);
        const uint32_t ww[8] = {wq[part][0].x, wq[part][0].y, wq[part][0].z, wq[part][0].w, wq[part][1].x, wq[part][1].y, wq[part][1].z, wq[part][1].w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float acc = 0.0f;
            acc = acc + __uint_as_float(ww[2 * c] << 16) * xv[0][c];
            acc = acc + __uint_as_float(ww[2 * c] & 0xffff0000u) * xv[1][c];
            acc = acc + __uint_as_float(ww[2 * c + 1] << 16) * xv[2][c];
            acc = acc + __uint_as_float(ww[2 * c + 1] & 0xffff0000u) * xv[3][c];
            // q reaches only the outputs, which carry bf16-operand rounding in both chunked forms: always the fast form
            act[part][c] = bf16_round(part == 0 ? silu_<true>(acc) : silu_<!VERIFY>(acc));
        }
    }
    // L2 norms of q and k (eps 1e-6 inside the root), q also times 128^-0.5.
    float qn[4], kn[4];
    {
        float sq = 0.0f, sk = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            sq = sq + act[0][c] * act[0][c];
            sk = sk + act[1][c] * act[1][c];
        }
        sq = butterfly(sq);
        sk = butterfly(sk);
        const float iq = inv_norm_<true>(sq), ik = inv_norm_<!VERIFY>(sk);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            qn[c] = (act[0][c] * iq) * (1.0f / sqrtf((float)DK));
            kn[c] = act[1][c] * ik;
        }
    }
    float a4[4], lg[4];
    unpack4(a_bits, a4);
    const float dtb[4] = {dtb4.x, dtb4.y, dtb4.z, dtb4.w};
#pragma unroll
    for (int c = 0; c < 4; ++c) lg[c] = p.lower * sigmoid_<!VERIFY>(decay_rate * (a4[c] + dtb[c]));
    const float bt = bf16_round(sigmoid_<!VERIFY>(blogit));
    if constexpr (VERIFY) {
        const long long sv = (gr * H + h) * DK + c0;
        if (j < p.pass_rows) *reinterpret_cast<uint2*>(p.q + gr * p.out_stride + (long long)h * DK + c0) = pack4_fp16(qn);  // rows past 16 get no output: leave theirs alone
        *reinterpret_cast<float4*>(p.k_save + sv) = make_float4(kn[0], kn[1], kn[2], kn[3]);
        *reinterpret_cast<uint2*>(p.v_save + sv) = pack4(act[2]);
        *reinterpret_cast<float4*>(p.g_save + sv) = make_float4(expf(lg[0]), expf(lg[1]), expf(lg[2]), expf(lg[3]));
        if (lane == 0) p.b_save[gr * H + h] = bt;
    } else {
        const long long orow = (long long)b * p.pass_rows + j, at = (orow * H + h) * DK + c0;
        *reinterpret_cast<uint2*>(p.q + at) = pack4_fp16(qn);
        *reinterpret_cast<uint2*>(p.k + at) = pack4_fp16(kn);
        *reinterpret_cast<uint2*>(p.v + at) = pack4(act[2]);
        *reinterpret_cast<float4*>(p.g + at) = make_float4(lg[0], lg[1], lg[2], lg[3]);
        if (lane == 0) p.beta[orow * H + h] = bt;
    }
    }
}

template <bool VERIFY>
int launch(const ProParams& pp, cudaStream_t stream) {
    const long long blocks = (long long)pp.batch * pp.H * (pp.pass_rows / 4);
    if (blocks > 0x7fffffffLL) return kInvalid;
    layer_prologue_kernel<VERIFY><<<(unsigned)blocks, 128, 0, stream>>>(pp);
    return (int)cudaGetLastError();
}

}  // namespace

int layer_prologue_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t pass_rows, int32_t row_shift,
                          const glm53f_bf16* p, int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride,
                          const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w, const float* a_log,
                          const float* dt_bias, float lower, glm53f_bf16* q, glm53f_bf16* k, glm53f_bf16* v, float* g, float* beta,
                          cudaStream_t stream) {
    if (pass_rows < 16 || pass_rows % 16 != 0) return kInvalid;
    ProParams pp{};
    pp.H = heads; pp.batch = batch; pp.pass_rows = pass_rows; pp.row_shift = row_shift;
    pp.cu = cu_rows;
    pp.P = p; pp.p_stride = p_stride; pp.b_off = b_off;
    pp.A = a; pp.a_stride = a_stride;
    pp.conv = conv; pp.conv_off = reinterpret_cast<const long long*>(conv_off); pp.cw = conv_w;
    pp.a_log = a_log; pp.dt_bias = dt_bias; pp.lower = lower;
    pp.q = q; pp.k = k; pp.v = v; pp.g = g; pp.beta = beta;
    return launch<false>(pp, stream);
}

// The prologue of the chunked verify: windows of up to 16 rows per request; see the head of the file for where the
// results go.  The caller checks the alignment of every row.
int verify_prologue_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                           const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* conv, const int64_t* conv_off,
                           const glm53f_bf16* conv_w, const float* a_log, const float* dt_bias, float lower, glm53f_bf16* out,
                           int64_t out_stride, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream) {
    ProParams pp{};
    pp.H = heads; pp.batch = batch; pp.pass_rows = kVerifyWindow; pp.row_shift = 0;
    pp.cu = cu_rows;
    pp.P = p; pp.p_stride = p_stride; pp.b_off = b_off;
    pp.A = a; pp.a_stride = a_stride;
    pp.conv = conv; pp.conv_off = reinterpret_cast<const long long*>(conv_off); pp.cw = conv_w;
    pp.a_log = a_log; pp.dt_bias = dt_bias; pp.lower = lower;
    pp.q = out; pp.out_stride = out_stride;
    pp.k_save = k_save; pp.v_save = v_save; pp.g_save = g_save; pp.b_save = b_save;
    return launch<true>(pp, stream);
}

}  // namespace kda
