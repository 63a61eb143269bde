// Draft verification on the tensor cores: a verify window of up to 16 rows is one 16-row chunk.
//
// The exact verify (kda_chain.cu) walks a window's rows one after the other through the delta rule, each row a full
// pass over the 128 x 128 state in registers: 16 serial passes, bound by instruction issue.  The chunked form reads the
// state once and does the state-sized work as two small tensor-core products.  For the rows i = 0..15 of a window,
// with G the cumulative log decay, Gm = G_8 (the middle row: every decay factor formed below stays within e^+-47 for
// the model's gate bound of -5.8 per row) and S the window's incoming state [v][k]:
//
//   L = beta_i (k_i a_i).(k_j / a_j) for j < i,  M = (q_i a_i).(k_j / a_j) for j <= i,   a = exp(G - Gm)
//                         as L^T, M^T = Kc x Kgb^T, Kc x Qgb^T (tcgen05, M = 128 of which 16 rows are real, N = 16)
//   W = (I + L)^-1 diag(beta) Kg,  U = (I + L)^-1 diag(beta) V   forward substitution down the 16 rows, FP32 on the CUDA
//                         cores (thread = channel: 136 multiply-adds each; no explicit inverse), Kg = k exp(G)
//   (W S)^T, (Qg S)^T     = S x W^T, S x Qg^T: tcgen05, M = 128 value channels, N = 16 rows, K = 128 key channels; the
//                         bf16 state tile is the A operand exactly as it lies in HBM (rows of 128 key channels)
//   D = U - W S,  O = Qg S + M D   FP32, thread = value channel (its tensor-memory lane)
//
// The state is not written (a verify leaves it to the commit) and the replay saves are the exact path's, bit for bit
// (k widened, v copied, exp(g) by the same expf, beta copied), so verify + commit still leaves the states of serial
// decode steps; only the window's OUTPUTS differ from the serial steps', by the rounding of bf16 operands (within the
// task's tolerance: max-abs 2e-2, rel-L2 5e-3).  Selected by GLM53F_KDA_CORE_TENSOR on glm53f_kda_core_verify_batch.
//
// The layer form (LAYER = true; the chunked form of glm53f_kda_chain_batch_bf16state, glm53f_kda_verify_mode) runs after
// the verify prologue (kda_prologue.cu) and takes a unit's rows from where that kernel left them: k, v, the decay
// multiplier and beta from the replay saves, q as fp16 from the output rows; it writes no saves and fuses the gated
// RMSNorm into its outputs.
//
// One block of 128 threads per (request, head) unit, three blocks per SM, blocks walk the units persistently.  A unit's
// rows and state arrive by asynchronous 16-byte copies issued one unit ahead (the state straight into the 128-byte
// swizzle the tensor core reads), so one unit's arithmetic covers the next one's loads.  All waits are bounded.

#include <cuda_fp16.h>

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"
#include "tc.cuh"

namespace kda {
namespace {

constexpr int WIN = 16, kVThreads = 128;
// Shared memory map (bytes).  Tiles are boxes of R rows x 128 bytes in the 128-byte swizzle (16-byte piece p of row r at
// piece p ^ (r & 7)), two boxes per tile (channels 0-63, 64-127).  The column-side tile Kc comes first: as the M = 128
// operand of L^T and M^T its descriptor walks 128 rows although 16 are real, and what follows it is the state tile.
// Once those two products are done Kc is dead, and L and M (FP32, 2.1 KB) take its place until the unit ends.
constexpr int vKc = 0, vS = 4096, vKgb = vS + 32768, vQgb = vKgb + 4096, vQg = vQgb + 4096, vRaw = vQg + 4096;
constexpr int vW = vKgb;                                                 // W replaces Kgb once L^T is done
constexpr int vStage = vKgb;                                             // layer form: FP32 outputs [16][128] over W and Qgb
constexpr int vL = vKc, vM = vL + WIN * 17 * 4;
static_assert(vM + WIN * WIN * 4 <= vS, "L and M fit the dead column-side tile");
// Raw rows of a unit.  Core form: q, k, v bf16 (256 bytes a row), log decay f32 (512), beta.  Layer form: q fp16, v bf16,
// k f32, the decay multiplier f32, beta.
template <bool LAYER>
struct Raw {
    static constexpr int Q = 0, V = 4096, K = 8192, G = LAYER ? 16384 : 12288, B = G + 8192, kBytes = B + 128;
};
template <bool LAYER>
struct Map {
    static constexpr int vBeta = vRaw + Raw<LAYER>::kBytes, vBar = vBeta + 64, vCtl = vBar + 16, kSmem = vCtl + 16;
    static_assert(vBar % 8 == 0 && kSmem <= 75 * 1024, "three blocks per SM");
};
constexpr uint32_t kVCols = 32;  // tensor memory: [0, 16) L^T then (W S)^T, [16, 32) M^T then (Qg S)^T

struct VParams {
    int H;
    long long units;
    const int32_t* cu;
    const uint16_t *q, *k, *v;  // core form: bf16 rows
    const float* g;
    const float* beta;
    const uint16_t* state;
    const long long* state_off;
    uint16_t* out;              // layer form: holds q as fp16 on entry
    long long out_stride;
    float* k_save;              // layer form: the sources of k, v, decay and beta
    uint16_t* v_save;
    float* g_save;
    float* b_save;
    const uint16_t* gate;       // layer form: the output gate rows, the norm weight, eps
    long long gate_stride;
    const uint16_t* norm_w;
    float eps;
    int* status;
};

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Byte offset in a tile with R rows per box of the bf16 element (row r, channel c).
__device__ __forceinline__ int sw_elem(int R, int r, int c) {
    return (c >> 6) * R * 128 + r * 128 + (((((c & 63) >> 3) ^ (r & 7))) << 4) + (c & 7) * 2;
}
// The output gate: these outputs carry the rounding of bf16 operands already, so the hardware's approximate exponential
// and division do (the file's other divisions and exponentials keep IEEE arithmetic for the replay saves).
__device__ __forceinline__ float sigmoid_(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

struct Unit {
    int b, h, n;
    long long row0, s_elem;
};
__device__ __forceinline__ Unit unit_of(const VParams& p, long long u) {
    Unit x;
    x.b = (int)(u / p.H);
    x.h = (int)(u % p.H);
    const int r0 = p.cu[x.b];
    x.row0 = r0;
    x.n = p.cu[x.b + 1] - r0;
    x.s_elem = p.state_off[x.b] + (long long)x.h * DV * DK;
    return x;
}

// The unit's raw rows; rows past the window's end become zero.
template <bool LAYER>
__device__ __forceinline__ void fetch_rows(const VParams& p, unsigned char* smem, const Unit& un, int t) {
    using R = Raw<LAYER>;
    const int n = min(max(un.n, 0), WIN);
    unsigned char* raw = smem + vRaw;
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int e = t; e < WIN * 16; e += kVThreads) {  // 16-byte pieces of the 256-byte rows
        const int r = e >> 4, pc = e & 15;
        const long long at = ((un.row0 + r) * p.H + un.h) * DK + pc * 8;
        if (r < n) {
            if constexpr (LAYER) {
                cp_async16(raw + R::Q + e * 16, p.out + (un.row0 + r) * p.out_stride + (long long)un.h * DK + pc * 8);
                cp_async16(raw + R::V + e * 16, p.v_save + at);
            } else {
                cp_async16(raw + R::Q + e * 16, p.q + at);
                cp_async16(raw + R::K + e * 16, p.k + at);
                cp_async16(raw + R::V + e * 16, p.v + at);
            }
        } else {
            *reinterpret_cast<uint4*>(raw + R::Q + e * 16) = z;
            if constexpr (!LAYER) *reinterpret_cast<uint4*>(raw + R::K + e * 16) = z;
            *reinterpret_cast<uint4*>(raw + R::V + e * 16) = z;
        }
    }
    for (int e = t; e < WIN * 32; e += kVThreads) {  // and of the 512-byte rows
        const int r = e >> 5, pc = e & 31;
        const long long at = ((un.row0 + r) * p.H + un.h) * DK + pc * 4;
        if (r < n) {
            if constexpr (LAYER) {
                cp_async16(raw + R::K + e * 16, p.k_save + at);
                cp_async16(raw + R::G + e * 16, p.g_save + at);
            } else {
                cp_async16(raw + R::G + e * 16, p.g + at);
            }
        } else {
            if constexpr (LAYER) *reinterpret_cast<uint4*>(raw + R::K + e * 16) = z;
            *reinterpret_cast<uint4*>(raw + R::G + e * 16) = z;
        }
    }
    if (t < WIN) {
        const float* src = LAYER ? p.b_save : p.beta;
        reinterpret_cast<float*>(raw + R::B)[t] = t < n ? src[(un.row0 + t) * p.H + un.h] : 0.0f;
    }
    cp_async_commit();
}
// The unit's state, 2,048 pieces of 16 bytes, into the swizzled tile.
__device__ __forceinline__ void fetch_state(const VParams& p, unsigned char* smem, const Unit& un, int t) {
    const uint16_t* src = p.state + un.s_elem;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int e = t + i * kVThreads, v = e >> 4, pk = e & 15;
            cp_async16(smem + vS + (pk >> 3) * 16384 + v * 128 + (((pk & 7) ^ (v & 7)) << 4), src + (long long)e * 8);
        }
    } else {  // a state that is not 16-byte aligned: element by element
        for (int e = t; e < DV * DK; e += kVThreads) *reinterpret_cast<uint16_t*>(smem + vS + sw_elem(DV, e >> 7, e & 127)) = src[e];
    }
    cp_async_commit();
}

template <bool LAYER>
__global__ void __launch_bounds__(kVThreads, 3) verify_tc_kernel(const __grid_constant__ VParams p) {
    using R = Raw<LAYER>;
    using MP = Map<LAYER>;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + MP::vBar);
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + MP::vCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    if (t == 0) {
        mbar_init(bar, 1);
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, kVCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const WaitCtx ctx{ctl, ctl + 1, p.status};
    uint32_t phase = 0;
    float* Lf = reinterpret_cast<float*>(smem + vL);
    float* Mf = reinterpret_cast<float*>(smem + vM);
    float* betas = reinterpret_cast<float*>(smem + MP::vBeta);
    float nw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if constexpr (LAYER) {
#pragma unroll
        for (int i = 0; i < 4; ++i) nw[i] = bf16_bits_to_f32(p.norm_w[lane * 4 + i]);
    }

    long long u = blockIdx.x;
    if (u < p.units) {
        const Unit first = unit_of(p, u);
        fetch_rows<LAYER>(p, smem, first, t);
        fetch_state(p, smem, first, t);
    }
    for (; u < p.units; u += gridDim.x) {
        const Unit un = unit_of(p, u);
        const long long u_next = u + gridDim.x;
        const bool more = u_next < p.units;
        Unit nxt = un;
        if (more) nxt = unit_of(p, u_next);
        if (un.n > WIN && t == 0) atomicCAS(p.status, 0, kStatusVerifyWindow);
        const int n = min(max(un.n, 0), WIN);

        cp_async_wait<1>();  // this unit's rows have landed (its state may still be on the way)
        __syncthreads();     // and every thread is done with the previous unit's L, M and staged outputs

        // ---- A. thread = channel c: the decay scan, the operand tiles, the replay saves ----------------------------------
        float kg[WIN], vv[WIN], qe[WIN];
        {
            const int c = t;
            const unsigned char* raw = smem + vRaw;
            float G[WIN], acc = 0.0f;
#pragma unroll
            for (int r = 0; r < WIN; ++r) {
                const float x = reinterpret_cast<const float*>(raw + R::G)[r * DK + c];
                // layer form: the saved multiplier exp(log decay) in (0, 1]; the rows past the window decay by nothing
                acc += LAYER ? (r < n ? __logf(x) : 0.0f) : x;
                G[r] = acc;
            }
            const float gm = G[WIN / 2];
            float amax = 0.0f;
#pragma unroll
            for (int r = 0; r < WIN; ++r) {
                float kf, qf;
                if constexpr (LAYER) {
                    kf = reinterpret_cast<const float*>(raw + R::K)[r * DK + c];
                    qf = __half2float(reinterpret_cast<const __half*>(raw + R::Q)[r * DK + c]);
                } else {
                    kf = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(raw + R::K)[r * DK + c]);
                    qf = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(raw + R::Q)[r * DK + c]);
                }
                const uint16_t vb = reinterpret_cast<const uint16_t*>(raw + R::V)[r * DK + c];
                const float a = __expf(G[r] - gm), e = __expf(G[r]);
                amax = fmaxf(amax, a);
                kg[r] = kf * e;
                vv[r] = bf16_bits_to_f32(vb);
                *reinterpret_cast<uint16_t*>(smem + vKgb + sw_elem(WIN, r, c)) = f32_to_bf16_bits(kf * a);
                *reinterpret_cast<uint16_t*>(smem + vQgb + sw_elem(WIN, r, c)) = f32_to_bf16_bits(qf * a);
                *reinterpret_cast<uint16_t*>(smem + vKc + sw_elem(WIN, r, c)) = f32_to_bf16_bits(kf * __fdividef(1.0f, a));
                qe[r] = qf * e;  // the Qg tile is written while the first products run
                if constexpr (!LAYER) {
                    if (r < n && p.k_save != nullptr) {
                        const long long at = ((un.row0 + r) * p.H + un.h) * DK + c;
                        p.k_save[at] = kf;
                        p.v_save[at] = vb;
                        p.g_save[at] = expf(reinterpret_cast<const float*>(raw + R::G)[r * DK + c]);
                    }
                }
            }
            if (!(amax < 1e37f)) atomicCAS(p.status, 0, kStatusPrefillRange);
            if (t < WIN) {
                const float bt = reinterpret_cast<const float*>(raw + R::B)[t];
                betas[t] = bt;
                if constexpr (!LAYER) {
                    if (t < n && p.b_save != nullptr) p.b_save[(un.row0 + t) * p.H + un.h] = bt;
                }
            }
        }
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();
        // The raw rows are consumed: the next unit's may come in.
        if (more) fetch_rows<LAYER>(p, smem, nxt, t);
        else cp_async_commit();

        // ---- B. L^T and M^T -------------------------------------------------------------------------------------------------
        if (t == 0) {
            constexpr uint32_t id = tc::idesc_bf16(128, WIN, 0, 0, 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm, tc::desc_sw128_kmajor(smem + vKc, WIN, k0), tc::desc_sw128_kmajor(smem + vKgb, WIN, k0), id, k0 > 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + 16, tc::desc_sw128_kmajor(smem + vKc, WIN, k0), tc::desc_sw128_kmajor(smem + vQgb, WIN, k0), id, k0 > 0);
            tc::mma_commit(bar);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
#pragma unroll
        for (int r = 0; r < WIN; ++r) *reinterpret_cast<uint16_t*>(smem + vQg + sw_elem(WIN, r, t)) = f32_to_bf16_bits(qe[r]);
        bool ok = mbar_wait(bar, phase, ctx, kStatusWaitPrefill);
        phase ^= 1u;
        if (!__syncthreads_and(ok)) break;
        tc::fence_after_sync();
        if (warp == 0) {  // lanes 0..15 hold column j of L and of M; tensor-memory column = row i.  Kc is dead: L, M go over it.
            uint32_t l16[16], m16[16];
            tc::tmem_ld16(tc::tmem_addr(tm, 0, 0), l16);
            tc::tmem_ld16(tc::tmem_addr(tm, 0, 16), m16);
            tc::tmem_ld_wait();
            if (lane < WIN) {
                const int j = lane;
#pragma unroll
                for (int i = 0; i < WIN; ++i) {
                    Lf[i * 17 + j] = i > j ? betas[i] * __uint_as_float(l16[i]) : 0.0f;
                    Mf[i * WIN + j] = i >= j ? __uint_as_float(m16[i]) : 0.0f;
                }
            }
        }
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- C. W = (I + L)^-1 diag(beta) Kg into its tile (thread = channel), U = (I + L)^-1 diag(beta) V in registers
        //         (thread = value channel), both by forward substitution down the 16 rows: the same multiply-adds as a product
        //         with an explicit inverse, without the inverse
        float U[WIN];
        {
            float W[WIN];
#pragma unroll
            for (int i = 0; i < WIN; ++i) {
                const float bi = betas[i];
                float w0 = bi * kg[i], w1 = 0.0f, u0 = bi * vv[i], u1 = 0.0f;
#pragma unroll
                for (int j = 0; j < i; ++j) {
                    const float l = Lf[i * 17 + j];
                    if (j & 1) {
                        w1 = fmaf(-l, W[j], w1);
                        u1 = fmaf(-l, U[j], u1);
                    } else {
                        w0 = fmaf(-l, W[j], w0);
                        u0 = fmaf(-l, U[j], u0);
                    }
                }
                W[i] = w0 + w1;
                U[i] = u0 + u1;
                *reinterpret_cast<uint16_t*>(smem + vW + sw_elem(WIN, i, t)) = f32_to_bf16_bits(W[i]);
            }
        }
        cp_async_wait<1>();  // this unit's state has landed (the next unit's rows may still be on the way)
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- D. (W S)^T and (Qg S)^T: the state tile as it lies in memory is the M operand ---------------------------------------
        if (t == 0) {
            constexpr uint32_t id = tc::idesc_bf16(128, WIN, 0, 0, 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm, tc::desc_sw128_kmajor(smem + vS, DV, k0), tc::desc_sw128_kmajor(smem + vW, WIN, k0), id, k0 > 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + 16, tc::desc_sw128_kmajor(smem + vS, DV, k0), tc::desc_sw128_kmajor(smem + vQg, WIN, k0), id, k0 > 0);
            tc::mma_commit(bar);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        ok = mbar_wait(bar, phase, ctx, kStatusWaitPrefill);
        phase ^= 1u;
        if (!__syncthreads_and(ok)) break;
        tc::fence_after_sync();
        // The state tile is consumed: the next unit's may come in.
        if (more) fetch_state(p, smem, nxt, t);
        else cp_async_commit();

        // ---- E. D = U - W S,  O = Qg S + M D; thread = value channel = its tensor-memory lane -----------------------------------------
        {
            uint32_t ws[16], qs[16];
            tc::tmem_ld16(tc::tmem_addr(tm, warp, 0), ws);
            tc::tmem_ld16(tc::tmem_addr(tm, warp, 16), qs);
            tc::tmem_ld_wait();
            float D[WIN];
#pragma unroll
            for (int j = 0; j < WIN; ++j) D[j] = U[j] - __uint_as_float(ws[j]);
#pragma unroll
            for (int i = 0; i < WIN; ++i) {
                float o = __uint_as_float(qs[i]);
#pragma unroll
                for (int j = 0; j <= i; ++j) o = fmaf(Mf[i * WIN + j], D[j], o);
                if constexpr (LAYER) reinterpret_cast<float*>(smem + vStage)[i * DV + t] = o;  // W and Qgb are dead
                else if (i < n) p.out[(un.row0 + i) * p.out_stride + (long long)un.h * DV + t] = f32_to_bf16_bits(o);
            }
        }
        tc::fence_before_sync();  // the next unit's products overwrite these tensor-memory columns
        if constexpr (LAYER) {
            // The gated RMSNorm (reference kda.cu:188-201): a warp takes four rows, a lane four value channels.
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = warp * 4 + k;
                if (i >= n) break;
                const float4 y4 = *reinterpret_cast<const float4*>(smem + vStage + (i * DV + lane * 4) * 4);
                const float y[4] = {y4.x, y4.y, y4.z, y4.w};
                float ss = 0.0f;
#pragma unroll
                for (int x = 0; x < 4; ++x) ss = ss + y[x] * y[x];
#pragma unroll
                for (int o = 16; o; o >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, o);
                const float rinv = rsqrtf(ss * (1.0f / (float)DV) + p.eps);
                const long long gr = un.row0 + i;
                const uint2 gw = *reinterpret_cast<const uint2*>(p.gate + gr * p.gate_stride + (long long)un.h * DV + lane * 4);
                const float gt[4] = {__uint_as_float(gw.x << 16), __uint_as_float(gw.x & 0xffff0000u), __uint_as_float(gw.y << 16),
                                     __uint_as_float(gw.y & 0xffff0000u)};
                uint32_t o2[2];
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const float lo = (nw[2 * x] * (y[2 * x] * rinv)) * sigmoid_(gt[2 * x]);
                    const float hi = (nw[2 * x + 1] * (y[2 * x + 1] * rinv)) * sigmoid_(gt[2 * x + 1]);
                    o2[x] = (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
                }
                *reinterpret_cast<uint2*>(p.out + gr * p.out_stride + (long long)un.h * DV + lane * 4) = make_uint2(o2[0], o2[1]);
            }
        }
    }
    cp_async_wait<0>();
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tm, kVCols);
}

// ---- the commit as chunks of 16 rows ---------------------------------------------------------------------------------
// The state after the first keep[b] saved rows, for every (request, layer, head): S <- E S + Kdec^T D per chunk of up to
// 16 rows, with D = U - W S as above, E = exp(G_last) and Kdec_i = k_i exp(G_last - G_i).  The inputs are the replay
// saves (k and the decay multiplier f32, v bf16, beta).  The bf16 state tile is the A operand of S W^T where it lies;
// the update D^T x Kdec (M = 128 value rows, N = 128 key channels, K = 16 rows) runs as three products of bf16 hi/lo
// halves (the path into the state keeps 16 bits of operand mantissa, as in the prefill), its FP32 accumulator is read
// back lane = value row, E S is added in FP32 and the rounded row goes back into the tile, which is then the next
// chunk's state or is copied out.  Unlike the exact replay this rounds the state to bf16 once per chunk instead of
// after every row, and its sums run in another order: the committed state agrees with serial decode steps to the last
// bits of bf16, not bit for bit (glm53f_kda_commit_mode).
// Four blocks per SM (128 registers a thread, all 512 columns of tensor memory, 52.6 KB of shared memory each): the stages
// of a unit are serial, so what overlaps one unit's waits is the other resident blocks' work.  To fit, the hi half of D^T
// shares its 4 KB with Kc and L: Kc is read by the L^T product only, L by the forward substitution only, and D^T is written
// after the (W S)^T product, which comes after both.
constexpr int cS = 0, cDT = 32768, cKc = cDT, cKgb = cDT + 8192, cKdT = cKgb + 4096, cE = cKdT + 8192, cBeta = cE + 512;
constexpr int cBar = cBeta + 64, cCtl = cBar + 16, kCSmem = cCtl + 16;
constexpr int cW = cKgb, cL = cKc;                    // W replaces Kgb, L replaces Kc once L^T is done
constexpr uint32_t kCCols = 128;                      // tensor memory: L^T, then (W S)^T, then the 128 x 128 update
constexpr int kCBlocks = 4;
static_assert(kCBlocks * (kCSmem + 1024) <= 228 * 1024 && kCBlocks * kCCols <= 512, "four blocks per SM");

struct CParams {
    int H, layers, rows1;
    long long units;
    const int32_t* cu;
    const int32_t* keep;
    const uint16_t* state_in;
    uint16_t* state_out;
    long long state_stride;
    const long long* state_off;
    const float* k_save;
    const uint16_t* v_save;
    const float* g_save;
    const float* b_save;
    long long kv_stride, b_stride;
    int* status;
};

__device__ __forceinline__ int state_piece(int v, int pk) { return cS + (pk >> 3) * 16384 + v * 128 + (((pk & 7) ^ (v & 7)) << 4); }

__global__ void __launch_bounds__(kVThreads, kCBlocks) commit_tc_kernel(const __grid_constant__ CParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + cBar);
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + cCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    if (t == 0) {
        mbar_init(bar, 1);
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, kCCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const WaitCtx ctx{ctl, ctl + 1, p.status};
    uint32_t phase = 0;
    float* Lf = reinterpret_cast<float*>(smem + cL);
    float* En = reinterpret_cast<float*>(smem + cE);
    float* betas = reinterpret_cast<float*>(smem + cBeta);
    bool ok = true;

    for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
        const int h = (int)(u % p.H), layer = (int)((u / p.H) % p.layers), b = (int)(u / ((long long)p.H * p.layers));
        const long long row0 = p.cu ? p.cu[b] : 0;
        int n = p.keep ? p.keep[b] : p.rows1;
        if (n < 0) n = 0;
        const long long s_elem = (long long)layer * p.state_stride + (p.state_off ? p.state_off[b] : 0) + (long long)h * DV * DK;
        const uint16_t* src = p.state_in + s_elem;
        uint16_t* dst = p.state_out + s_elem;
        if (n == 0 && dst == src) continue;
        const long long kv_base = (long long)layer * p.kv_stride, b_base = (long long)layer * p.b_stride;
        __syncthreads();  // the previous unit's tile has been copied out
        // The unit's state into the swizzled tile.
        const bool vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0;
        if (vec) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int e = t + i * kVThreads;
                cp_async16(smem + state_piece(e >> 4, e & 15), src + (long long)e * 8);
            }
        } else {
            for (int e = t; e < DV * DK; e += kVThreads) *reinterpret_cast<uint16_t*>(smem + cS + sw_elem(DV, e >> 7, e & 127)) = src[e];
        }
        cp_async_commit();

        for (int c0 = 0; c0 < n && ok; c0 += WIN) {
            const int nr = min(WIN, n - c0);
            // ---- A. thread = channel: the decay scan and the operand tiles; thread = value channel: v ----------------------
            float kg[WIN], vv[WIN];
            {
                float kf[WIN], G[WIN], acc = 0.0f;
#pragma unroll
                for (int r = 0; r < WIN; ++r) {
                    const long long at = kv_base + ((row0 + c0 + r) * p.H + h) * DK + t;
                    const bool live = r < nr;
                    kf[r] = live ? p.k_save[at] : 0.0f;
                    vv[r] = live ? bf16_bits_to_f32(p.v_save[at]) : 0.0f;
                    acc += live ? __logf(p.g_save[at]) : 0.0f;
                    G[r] = acc;
                }
                const float gm = G[WIN / 2], gl = G[WIN - 1];
                float amax = 0.0f;
                uint32_t dh[WIN / 2], dl[WIN / 2];
#pragma unroll
                for (int r = 0; r < WIN; r += 2) {
                    float hi[2], lo[2];
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const float a = __expf(G[r + x] - gm);
                        amax = fmaxf(amax, a);
                        kg[r + x] = kf[r + x] * __expf(G[r + x]);
                        *reinterpret_cast<uint16_t*>(smem + cKgb + sw_elem(WIN, r + x, t)) = f32_to_bf16_bits(kf[r + x] * a);
                        *reinterpret_cast<uint16_t*>(smem + cKc + sw_elem(WIN, r + x, t)) = f32_to_bf16_bits(kf[r + x] * __fdividef(1.0f, a));
                        tc::split_bf16(kf[r + x] * __expf(gl - G[r + x]), hi[x], lo[x]);
                    }
                    dh[r / 2] = tc::bf16x2(hi[0], hi[1]);
                    dl[r / 2] = tc::bf16x2(lo[0], lo[1]);
                }
                // Kdec^T: row = key channel t, 16 row indices along K = two 16-byte cells
                *reinterpret_cast<uint4*>(smem + cKdT + (0 * DK + t) * 16) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(smem + cKdT + (1 * DK + t) * 16) = make_uint4(dh[4], dh[5], dh[6], dh[7]);
                *reinterpret_cast<uint4*>(smem + cKdT + 4096 + (0 * DK + t) * 16) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4*>(smem + cKdT + 4096 + (1 * DK + t) * 16) = make_uint4(dl[4], dl[5], dl[6], dl[7]);
                En[t] = __expf(gl);
                if (!(amax < 1e37f)) atomicCAS(p.status, 0, kStatusPrefillRange);
                if (t < WIN) betas[t] = t < nr ? p.b_save[b_base + (row0 + c0 + t) * p.H + h] : 0.0f;
            }
            fence_proxy_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            tc::fence_after_sync();

            // ---- B. L^T ---------------------------------------------------------------------------------------------------
            if (t == 0) {
                constexpr uint32_t id = tc::idesc_bf16(128, WIN, 0, 0, 0);
                for (int k0 = 0; k0 < DK; k0 += 16)
                    tc::mma_bf16(tm, tc::desc_sw128_kmajor(smem + cKc, WIN, k0), tc::desc_sw128_kmajor(smem + cKgb, WIN, k0), id, k0 > 0);
                tc::mma_commit(bar);
                atomicAdd(const_cast<uint32_t*>(ctl), 1u);
            }
            ok = mbar_wait(bar, phase, ctx, kStatusWaitPrefill);
            phase ^= 1u;
            ok = __syncthreads_and(ok);
            if (!ok) break;
            tc::fence_after_sync();
            if (warp == 0) {
                uint32_t l16[16];
                tc::tmem_ld16(tc::tmem_addr(tm, 0, 0), l16);
                tc::tmem_ld_wait();
                if (lane < WIN) {
#pragma unroll
                    for (int i = 0; i < WIN; ++i) Lf[i * 17 + lane] = i > lane ? betas[i] * __uint_as_float(l16[i]) : 0.0f;
                }
            }
            tc::fence_before_sync();
            __syncthreads();
            tc::fence_after_sync();

            // ---- C. W and U by forward substitution ---------------------------------------------------------------------------
            float U[WIN];
            {
                float W[WIN];
#pragma unroll
                for (int i = 0; i < WIN; ++i) {
                    const float bi = betas[i];
                    float w0 = bi * kg[i], w1 = 0.0f, u0 = bi * vv[i], u1 = 0.0f;
#pragma unroll
                    for (int j = 0; j < i; ++j) {
                        const float l = Lf[i * 17 + j];
                        if (j & 1) {
                            w1 = fmaf(-l, W[j], w1);
                            u1 = fmaf(-l, U[j], u1);
                        } else {
                            w0 = fmaf(-l, W[j], w0);
                            u0 = fmaf(-l, U[j], u0);
                        }
                    }
                    W[i] = w0 + w1;
                    U[i] = u0 + u1;
                    *reinterpret_cast<uint16_t*>(smem + cW + sw_elem(WIN, i, t)) = f32_to_bf16_bits(W[i]);  // over Kgb, which is consumed
                }
            }
            cp_async_wait<0>();  // the state has landed (first chunk)
            fence_proxy_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            tc::fence_after_sync();

            // ---- D. (W S)^T = S W^T --------------------------------------------------------------------------------------------
            if (t == 0) {
                constexpr uint32_t id = tc::idesc_bf16(128, WIN, 0, 0, 0);
                for (int k0 = 0; k0 < DK; k0 += 16)
                    tc::mma_bf16(tm, tc::desc_sw128_kmajor(smem + cS, DV, k0), tc::desc_sw128_kmajor(smem + cW, WIN, k0), id, k0 > 0);
                tc::mma_commit(bar);
                atomicAdd(const_cast<uint32_t*>(ctl), 1u);
            }
            ok = mbar_wait(bar, phase, ctx, kStatusWaitPrefill);
            phase ^= 1u;
            ok = __syncthreads_and(ok);
            if (!ok) break;
            tc::fence_after_sync();

            // ---- E. D = U - W S as the A operand D^T (row = value channel t, hi and lo halves) ------------------------------
            {
                uint32_t ws[16];
                tc::tmem_ld16(tc::tmem_addr(tm, warp, 0), ws);
                tc::tmem_ld_wait();
                uint32_t dh[WIN / 2], dl[WIN / 2];
#pragma unroll
                for (int i = 0; i < WIN; i += 2) {
                    float hi[2], lo[2];
                    tc::split_bf16(U[i] - __uint_as_float(ws[i]), hi[0], lo[0]);
                    tc::split_bf16(U[i + 1] - __uint_as_float(ws[i + 1]), hi[1], lo[1]);
                    dh[i / 2] = tc::bf16x2(hi[0], hi[1]);
                    dl[i / 2] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(smem + cDT + (0 * DV + t) * 16) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(smem + cDT + (1 * DV + t) * 16) = make_uint4(dh[4], dh[5], dh[6], dh[7]);
                *reinterpret_cast<uint4*>(smem + cDT + 4096 + (0 * DV + t) * 16) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4*>(smem + cDT + 4096 + (1 * DV + t) * 16) = make_uint4(dl[4], dl[5], dl[6], dl[7]);
            }
            fence_proxy_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            tc::fence_after_sync();

            // ---- F. the update D^T x Kdec: [value row][key channel], three products of halves ------------------------------------
            if (t == 0) {
                constexpr uint32_t id = tc::idesc_bf16(128, 128, 0, 0, 0);
                tc::mma_bf16(tm, tc::desc_kmajor_bf16(smem + cDT, DV, 0, 0), tc::desc_kmajor_bf16(smem + cKdT, DK, 0, 0), id, false);
                tc::mma_bf16(tm, tc::desc_kmajor_bf16(smem + cDT, DV, 0, 0), tc::desc_kmajor_bf16(smem + cKdT + 4096, DK, 0, 0), id, true);
                tc::mma_bf16(tm, tc::desc_kmajor_bf16(smem + cDT + 4096, DV, 0, 0), tc::desc_kmajor_bf16(smem + cKdT, DK, 0, 0), id, true);
                tc::mma_commit(bar);
                atomicAdd(const_cast<uint32_t*>(ctl), 1u);
            }
            ok = mbar_wait(bar, phase, ctx, kStatusWaitPrefill);
            phase ^= 1u;
            ok = __syncthreads_and(ok);
            if (!ok) break;
            tc::fence_after_sync();

            // ---- G. S <- E S + update, rounded to bf16, back into the tile (thread = value row) ------------------------------
#pragma unroll 1
            for (int cg = 0; cg < DK / 32; ++cg) {
                uint32_t a16[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cg * 32), a16);
                tc::tmem_ld_wait();
#pragma unroll
                for (int half = 0; half < 4; ++half) {
                    unsigned char* at = smem + state_piece(t, cg * 4 + half);
                    const uint4 sv = *reinterpret_cast<const uint4*>(at);
                    const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
                    uint32_t out[4];
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const int k = cg * 32 + half * 8 + 2 * x;
                        const float2 e2 = *reinterpret_cast<const float2*>(&En[k]);
                        const float lo = fmaf(e2.x, __uint_as_float(sw[x] << 16), __uint_as_float(a16[half * 8 + 2 * x]));
                        const float hi = fmaf(e2.y, __uint_as_float(sw[x] & 0xffff0000u), __uint_as_float(a16[half * 8 + 2 * x + 1]));
                        out[x] = tc::bf16x2(lo, hi);
                    }
                    *reinterpret_cast<uint4*>(at) = make_uint4(out[0], out[1], out[2], out[3]);
                }
            }
            fence_proxy_async_smem();  // the next chunk's S W^T reads the tile through the async proxy
            tc::fence_before_sync();
            __syncthreads();
            tc::fence_after_sync();
        }
        if (!ok) break;
        cp_async_wait<0>();  // a unit without rows: its state is only copied
        __syncthreads();
        // ---- the tile back to global memory, coalesced ------------------------------------------------------------------------
        if (vec) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int e = t + i * kVThreads;
                *reinterpret_cast<uint4*>(dst + (long long)e * 8) = *reinterpret_cast<const uint4*>(smem + state_piece(e >> 4, e & 15));
            }
        } else {
            for (int e = t; e < DV * DK; e += kVThreads) dst[e] = *reinterpret_cast<const uint16_t*>(smem + cS + sw_elem(DV, e >> 7, e & 127));
        }
    }
    cp_async_wait<0>();
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tm, kCCols);
}

template <bool LAYER>
int launch_verify(const VParams& p, cudaStream_t stream) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(verify_tc_kernel<LAYER>, cudaFuncAttributeMaxDynamicSharedMemorySize, Map<LAYER>::kSmem);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    const long long cap = 3LL * sm_count();
    verify_tc_kernel<LAYER><<<(unsigned)(p.units < cap ? p.units : cap), kVThreads, Map<LAYER>::kSmem, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace

// The chunked verify of the core entry point: bf16 states, no state written, no fused norm, 16-byte aligned rows (the
// caller checks).
int core_verify_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q, const glm53f_bf16* k,
                          const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, const int64_t* state_off,
                          glm53f_bf16* out, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream) {
    VParams p{};
    p.H = heads;
    p.units = (long long)heads * batch;
    p.cu = cu_rows;
    p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta;
    p.state = reinterpret_cast<const uint16_t*>(state_in);
    p.state_off = reinterpret_cast<const long long*>(state_off);
    p.out = out;
    p.out_stride = (long long)heads * DV;
    p.k_save = k_save; p.v_save = v_save; p.g_save = g_save; p.b_save = b_save;
    p.status = status_word();
    return launch_verify<false>(p, stream);
}

// The chunked verify of the layer entry point, after verify_prologue_launch on the same stream: the saves hold k, v, the
// decay multiplier and beta of every window row, `out` holds q as fp16 and receives the gated, normalised outputs.
int layer_verify_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const void* state_in, const int64_t* state_off,
                           const glm53f_bf16* gate, int64_t gate_stride, const glm53f_bf16* norm_w, float eps, glm53f_bf16* out,
                           int64_t out_stride, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream) {
    VParams p{};
    p.H = heads;
    p.units = (long long)heads * batch;
    p.cu = cu_rows;
    p.state = reinterpret_cast<const uint16_t*>(state_in);
    p.state_off = reinterpret_cast<const long long*>(state_off);
    p.out = out;
    p.out_stride = out_stride;
    p.k_save = k_save; p.v_save = v_save; p.g_save = g_save; p.b_save = b_save;
    p.gate = gate; p.gate_stride = gate_stride; p.norm_w = norm_w; p.eps = eps;
    p.status = status_word();
    return launch_verify<true>(p, stream);
}

// The chunked commit (bf16 states; the caller checks that the saves are 4-byte aligned, which every float array is).
int commit_tc_launch(int32_t heads, int32_t layers, int32_t batch, const int32_t* cu_rows, const int32_t* keep, int32_t rows1, const void* state_in,
                     void* state_out, int64_t state_stride, const int64_t* state_off, const float* k_save, const glm53f_bf16* v_save,
                     const float* g_save, const float* b_save, int64_t kv_stride, int64_t b_stride, cudaStream_t stream) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(commit_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCSmem);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    CParams p{};
    p.H = heads; p.layers = layers; p.rows1 = rows1;
    p.units = (long long)heads * layers * batch;
    p.cu = cu_rows; p.keep = keep;
    p.state_in = reinterpret_cast<const uint16_t*>(state_in);
    p.state_out = reinterpret_cast<uint16_t*>(state_out);
    p.state_stride = state_stride;
    p.state_off = reinterpret_cast<const long long*>(state_off);
    p.k_save = k_save; p.v_save = v_save; p.g_save = g_save; p.b_save = b_save;
    p.kv_stride = kv_stride; p.b_stride = b_stride;
    p.status = status_word();
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    const long long cap = (long long)kCBlocks * sm_count();
    commit_tc_kernel<<<(unsigned)(p.units < cap ? p.units : cap), kVThreads, kCSmem, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace kda
