// Chunked KDA prefill on the 5th-generation tensor cores (tcgen05 + TMEM), chunk = 64 rows.
//
// One block of 128 threads per (sequence, head) walks the sequence's chunks in order; the head's 128x128 state
// stays in tensor memory (FP32 accumulator, 128 lanes = key channel, 128 columns = value channel) from the first
// chunk to the last and touches HBM twice: once in, once out.  Per chunk (the algebra of the reference's CPU
// definition crates/glm53f-kda/src/chunked.rs:67-198, which itself restates chunk_kimi_delta_attention):
//
//   G_i   = g_0 + ... + g_i per key channel (FP32 scan, thread = channel), E = exp(G), E_last = exp(G_63)
//   Kg = k*E, Qg = q*E, Kinv = k/E, Kdec = k * E_last/E                       (operand tiles, written by hand)
//   [L; M] = [Kg; Qg] Kinv^T          one 128x64x128 MMA; L strictly lower * beta_i, M lower incl. diagonal
//   T  = (I + L)^-1                   FP32 on the CUDA cores: 16x16 diagonal blocks by substitution, the
//                                     off-diagonal blocks by block back-substitution;  T' = T diag(beta)
//   W  = T' Kg,  U = T' V             64x128x64 MMAs; T' as bf16 hi + lo for U
//   D  = U - W S,  QS = Qg S          64x128x128 MMAs on a bf16 copy of S; D accumulates in place (negated A)
//   O  = QS + M D                     64x128x64 MMA
//   S <- E_last * S + Kdec^T D        128x128x64 MMAs, Kdec and D as bf16 hi + lo (three products)
//
// Operand precision follows a CPU study of this exact scheme on the benchmark's input distribution: bf16
// operands are enough for every product that only reaches the output (M, QS, M D) and for L, W and W S, but not
// for U and Kdec^T D, which carry the state: those use two-term bf16 splits (16 mantissa bits).  With that mix
// the final state is within 5e-4 rel-L2 of the FP32 recurrence (limit 1e-3) and the bf16 outputs within 4e-3
// (limit 5e-3).
//
// Every exponent the scheme evaluates stays representable only while a chunk's cumulative log decay stays above
// about -80 per channel (1/E is formed explicitly).  The benchmark's gates (log sigmoid(N(3,1)), about -4.5 per
// chunk) are far inside that range; the model's gate bound of -5 per row is not, so the layer entry points
// (glm53f_kda_prefill*) keep the exact row-by-row path, and this kernel records kStatusPrefillRange when a chunk
// leaves the range.
//
// Raw inputs arrive by bulk asynchronous copies (one per row and tensor) into padded row-major staging buffers;
// operands are written in the un-swizzled "cell" layout of tc.cuh.  All waits are bounded.

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"
#include "tc.cuh"

namespace kda {
namespace {

constexpr int CH = 64;            // rows per chunk
constexpr int kThreadsTc = 128;   // thread t <-> TMEM lane t
constexpr int RS16 = 272;         // staging row stride, bf16 tensors (256 + 16: rows 4 banks apart)
constexpr int RS32 = 528;         // staging row stride, f32 tensor
// Shared memory map (bytes).
constexpr int oRawQ = 0, oRawK = oRawQ + CH * RS16, oRawV = oRawK + CH * RS16, oRawG = oRawV + CH * RS16;
constexpr int kRegionA = oRawG + CH * RS32;            // 86,016
// Region A is reused once the operands are built: L, T, P (FP32) during the inversion, then S16 / D_hi / D_lo.
constexpr int LS = 65;                                  // FP32 row stride of L and T
constexpr int oL = 0, oT = oL + CH * LS * 4, oP = oT + CH * LS * 4;  // P: [16][49]
constexpr int oS16 = 0, oDhi = oS16 + 128 * 16 * 16, oDlo = oDhi + CH * 16 * 16;
static_assert(oP + 16 * 49 * 4 <= kRegionA && oDlo + CH * 16 * 16 <= kRegionA, "region A overflow");
constexpr int XR = 192;                                 // X rows: Kg 0..63, Qg 64..127, W 128..191
constexpr int oX = kRegionA, oKinv = oX + XR * 16 * 16, oKdHi = oKinv + CH * 16 * 16, oKdLo = oKdHi + CH * 16 * 16;
constexpr int oTpHi = oKdLo + CH * 16 * 16, oTpLo = oTpHi + CH * 8 * 16, oMm = oTpLo + CH * 8 * 16, oV = oMm + CH * 8 * 16;
constexpr int oBeta = oV + CH * 16 * 16, oEGL = oBeta + CH * 4, oBars = oEGL + 128 * 4, oCtl = oBars + 16;
constexpr int kSmemTc = oCtl + 32;
static_assert(kSmemTc <= 232448, "shared memory budget");
// Tensor memory columns.
constexpr uint32_t cS = 0, cLM = 128, cW = 192, cQS = 192, cU = 320, kTmemCols = 512;

struct TcParams {
    int H;
    const int32_t* cu;
    const uint16_t *q, *k, *v;
    const float* g;
    const float* beta;
    const void* state_in;
    void* state_out;
    const long long* state_off;
    int state_bf16;
    const uint16_t* gate;
    const uint16_t* norm_w;
    float eps;
    uint16_t* out;
    int* status;
};

__device__ __forceinline__ unsigned char* cell(unsigned char* tile, int R, int c, int r) { return tile + ((size_t)c * R + r) * 16; }

__global__ void __launch_bounds__(kThreadsTc, 1) prefill_tc_kernel(const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bar_raw = reinterpret_cast<uint64_t*>(smem + oBars);
    uint64_t* bar_mma = bar_raw + 1;
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    float* betas = reinterpret_cast<float*>(smem + oBeta);
    float* egl = reinterpret_cast<float*>(smem + oEGL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x, b = blockIdx.y, H = p.H;
    const long long row0 = p.cu[b];
    const int T = p.cu[b + 1] - p.cu[b];
    const long long s_elem = p.state_off[b] + (long long)h * DV * DK;

    if (tid == 0) {
        mbar_init(bar_raw, 1);
        mbar_init(bar_mma, 1);
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const WaitCtx ctx{ctl, ctl + 1, p.status};
    uint32_t raw_phase = 0, mma_phase = 0;
    bool alive = true;

    // ---- the incoming state into tensor memory: thread = key channel, columns = value channel ----------------------
    for (int c0 = 0; c0 < 4; ++c0) {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const long long at = s_elem + (long long)(c0 * 32 + j) * DK + tid;
            const float x = p.state_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.state_in)[at])
                                         : reinterpret_cast<const float*>(p.state_in)[at];
            r[j] = __float_as_uint(x);
        }
        tc::tmem_st32(tc::tmem_addr(tm, warp, cS + c0 * 32), r);
    }
    tc::tmem_st_wait();

    for (int s = 0; s < T && alive; s += CH) {
        const int n = min(CH, T - s);
        const long long gr0 = row0 + s;
        // ---- 0. raw rows: bulk copies, one per row and tensor; rows past the end are zero ------------------------
        if (tid == 0) mbar_arrive_expect_tx(bar_raw, (uint32_t)n * (3 * 256 + 512));
        if (tid < n) {
            const long long at = ((gr0 + tid) * H + h) * DK;
            bulk_load(smem + oRawQ + tid * RS16, p.q + at, 256, bar_raw);
            bulk_load(smem + oRawK + tid * RS16, p.k + at, 256, bar_raw);
            bulk_load(smem + oRawV + tid * RS16, p.v + at, 256, bar_raw);
            bulk_load(smem + oRawG + tid * RS32, p.g + at, 512, bar_raw);
        } else if (tid < CH) {
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int e = 0; e < 16; ++e) {
                *reinterpret_cast<uint4*>(smem + oRawQ + tid * RS16 + e * 16) = z;
                *reinterpret_cast<uint4*>(smem + oRawK + tid * RS16 + e * 16) = z;
                *reinterpret_cast<uint4*>(smem + oRawV + tid * RS16 + e * 16) = z;
            }
            for (int e = 0; e < 32; ++e) *reinterpret_cast<uint4*>(smem + oRawG + tid * RS32 + e * 16) = z;
        }
        if (tid < CH) betas[tid] = tid < n ? p.beta[(gr0 + tid) * H + h] : 0.0f;
        if (!mbar_wait(bar_raw, raw_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        raw_phase ^= 1u;
        __syncthreads();

        // ---- 1. cumulative log decay per key channel; the staging buffer keeps E = exp(G) ---------------------------
        {
            float G = 0.0f, e = 1.0f;
            for (int r = 0; r < CH; ++r) {
                float* at = reinterpret_cast<float*>(smem + oRawG + r * RS32) + tid;
                G += *at;
                e = expf(G);
                *at = e;
            }
            egl[tid] = e;
            if (!(e > 1e-34f)) atomicCAS(p.status, 0, kStatusPrefillRange);
        }
        __syncthreads();

        // ---- 2. operand tiles: lane <-> row, 8 channels (one 16-byte cell) at a time -------------------------------
        {
            const int r = tid & 63, half = tid >> 6;
            for (int cc = 0; cc < 8; ++cc) {
                const int c = half * 8 + cc;
                const uint4 k8 = *reinterpret_cast<const uint4*>(smem + oRawK + r * RS16 + c * 16);
                const uint4 q8 = *reinterpret_cast<const uint4*>(smem + oRawQ + r * RS16 + c * 16);
                const uint4 v8 = *reinterpret_cast<const uint4*>(smem + oRawV + r * RS16 + c * 16);
                const float4 e0 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32);
                const float4 e1 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32 + 16);
                const float4 l0 = *reinterpret_cast<const float4*>(egl + c * 8);
                const float4 l1 = *reinterpret_cast<const float4*>(egl + c * 8 + 4);
                const float E[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
                const float EL[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
                const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w}, qw[4] = {q8.x, q8.y, q8.z, q8.w};
                uint32_t kg[4], qg[4], ki[4], dh[4], dl[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float kf[2] = {__uint_as_float(kw[j] << 16), __uint_as_float(kw[j] & 0xffff0000u)};
                    float qf[2] = {__uint_as_float(qw[j] << 16), __uint_as_float(qw[j] & 0xffff0000u)};
                    float a[2], bq[2], ci[2], hi[2], lo[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float e = E[2 * j + u], einv = __frcp_rn(e);
                        a[u] = kf[u] * e;
                        bq[u] = qf[u] * e;
                        ci[u] = kf[u] * einv;
                        tc::split_bf16(kf[u] * (EL[2 * j + u] * einv), hi[u], lo[u]);
                    }
                    kg[j] = tc::bf16x2(a[0], a[1]);
                    qg[j] = tc::bf16x2(bq[0], bq[1]);
                    ki[j] = tc::bf16x2(ci[0], ci[1]);
                    dh[j] = tc::bf16x2(hi[0], hi[1]);
                    dl[j] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(cell(smem + oX, XR, c, r)) = make_uint4(kg[0], kg[1], kg[2], kg[3]);
                *reinterpret_cast<uint4*>(cell(smem + oX, XR, c, 64 + r)) = make_uint4(qg[0], qg[1], qg[2], qg[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKinv, CH, c, r)) = make_uint4(ki[0], ki[1], ki[2], ki[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdHi, CH, c, r)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdLo, CH, c, r)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4*>(cell(smem + oV, CH, c, r)) = v8;
            }
        }
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- 3. [L; M] = [Kg; Qg] Kinv^T ---------------------------------------------------------------------------
        if (tid == 0) {
            constexpr uint32_t id = tc::idesc_bf16(128, 64, 0, 0, 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + cLM, tc::desc_kmajor_bf16(smem + oX, XR, 0, k0), tc::desc_kmajor_bf16(smem + oKinv, CH, 0, k0), id, k0 > 0);
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        mma_phase ^= 1u;
        tc::fence_after_sync();

        // ---- 4. L (FP32, strictly lower, times beta_i) and M (bf16 cells, lower with the diagonal) ------------------
        {
            const int i = tid & 63;
            float* Lr = reinterpret_cast<float*>(smem + oL) + i * LS;
            float* Tr = reinterpret_cast<float*>(smem + oT) + i * LS;
            const float bi = betas[i];
            for (int c0 = 0; c0 < 2; ++c0) {
                uint32_t r[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cLM + c0 * 32), r);
                tc::tmem_ld_wait();
                if (tid < 64) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = c0 * 32 + j;
                        Lr[col] = col < i ? bi * __uint_as_float(r[j]) : 0.0f;
                        Tr[col] = 0.0f;
                    }
                } else {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t w[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int col = c0 * 32 + cc * 8 + 2 * j;
                            const float x0 = col <= i ? __uint_as_float(r[cc * 8 + 2 * j]) : 0.0f;
                            const float x1 = col + 1 <= i ? __uint_as_float(r[cc * 8 + 2 * j + 1]) : 0.0f;
                            w[j] = tc::bf16x2(x0, x1);
                        }
                        *reinterpret_cast<uint4*>(cell(smem + oMm, CH, c0 * 4 + cc, i)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
        __syncthreads();

        // ---- 5. T = (I + L)^-1 in FP32 ------------------------------------------------------------------------------
        {
            const float* Lm = reinterpret_cast<const float*>(smem + oL);
            float* Tm = reinterpret_cast<float*>(smem + oT);
            float* Pm = reinterpret_cast<float*>(smem + oP);
            // 5a. the four 16x16 diagonal blocks by forward substitution: thread j keeps column j of its block.
            if (tid < 64) {
                const int blk = tid >> 4, jj = tid & 15, base = blk * 16;
                float tcol[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) tcol[m] = m == jj ? 1.0f : 0.0f;
#pragma unroll
                for (int ii = 1; ii < 16; ++ii) {
                    float acc = Lm[(base + ii) * LS + base + jj];
#pragma unroll
                    for (int m = 1; m < 15; ++m)
                        if (m > jj && m < ii) acc = fmaf(Lm[(base + ii) * LS + base + m], tcol[m], acc);
                    if (jj < ii) tcol[ii] = -acc;
                }
#pragma unroll
                for (int m = 0; m < 16; ++m) Tm[(base + m) * LS + base + jj] = tcol[m];
            }
            __syncthreads();
            // 5b. block rows 1..3: P = L[I, 0..I) T[0..I, 0..I), then T[I, 0..I) = -T[I,I] P.
            for (int I = 1; I < 4; ++I) {
                const int cols = 16 * I;
                for (int e = tid; e < 16 * cols; e += kThreadsTc) {
                    const int i = e / cols, j = e % cols;
                    const float* Lrow = Lm + (16 * I + i) * LS;
                    float a0 = 0.0f, a1 = 0.0f;
                    for (int m = j & ~15; m < cols; m += 2) {  // T[m][j] is zero above its block's diagonal
                        a0 = fmaf(Lrow[m], Tm[m * LS + j], a0);
                        a1 = fmaf(Lrow[m + 1], Tm[(m + 1) * LS + j], a1);
                    }
                    Pm[i * 49 + j] = a0 + a1;
                }
                __syncthreads();
                for (int e = tid; e < 16 * cols; e += kThreadsTc) {
                    const int i = e / cols, j = e % cols;
                    const float* Trow = Tm + (16 * I + i) * LS + 16 * I;
                    float acc = 0.0f;
                    for (int m = 0; m <= i; ++m) acc = fmaf(Trow[m], Pm[m * 49 + j], acc);
                    Tm[(16 * I + i) * LS + j] = -acc;
                }
                __syncthreads();
            }
            // 5c. T' = T diag(beta) as bf16 hi + lo cells.
            const int i = tid & 63, half = tid >> 6;
            for (int cc = 0; cc < 4; ++cc) {
                const int c = half * 4 + cc;
                uint32_t wh[4], wl[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float hi[2], lo[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int col = c * 8 + 2 * j + u;
                        const float t = col <= i ? Tm[i * LS + col] * betas[col] : 0.0f;
                        tc::split_bf16(t, hi[u], lo[u]);
                    }
                    wh[j] = tc::bf16x2(hi[0], hi[1]);
                    wl[j] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(cell(smem + oTpHi, CH, c, i)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                *reinterpret_cast<uint4*>(cell(smem + oTpLo, CH, c, i)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            }
        }
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- 6. W = T' Kg (bf16 T'), U = T' V (T' hi + lo) -----------------------------------------------------------
        if (tid == 0) {
            constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cW, tc::desc_kmajor_bf16(smem + oTpHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oX, XR, 0, k0), id, k0 > 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oTpHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oV, CH, 0, k0), id, k0 > 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oTpLo, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oV, CH, 0, k0), id, true);
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        mma_phase ^= 1u;
        tc::fence_after_sync();

        // ---- 7. W to bf16 cells (rows 128.. of X); 8. S to bf16 cells, and the decayed S back to tensor memory -------
        {
            const int i = warp * 16 + lane;  // valid for lane < 16: row of an M = 64 accumulator
            for (int c0 = 0; c0 < 4; ++c0) {
                uint32_t r[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cW + c0 * 32), r);
                tc::tmem_ld_wait();
                if (lane < 16) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        *reinterpret_cast<uint4*>(cell(smem + oX, XR, c0 * 4 + cc, 128 + i)) =
                            make_uint4(tc::bf16x2(__uint_as_float(r[cc * 8 + 0]), __uint_as_float(r[cc * 8 + 1])),
                                       tc::bf16x2(__uint_as_float(r[cc * 8 + 2]), __uint_as_float(r[cc * 8 + 3])),
                                       tc::bf16x2(__uint_as_float(r[cc * 8 + 4]), __uint_as_float(r[cc * 8 + 5])),
                                       tc::bf16x2(__uint_as_float(r[cc * 8 + 6]), __uint_as_float(r[cc * 8 + 7])));
                }
            }
            const float el = egl[tid];
            for (int c0 = 0; c0 < 4; ++c0) {
                uint32_t r[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cS + c0 * 32), r);
                tc::tmem_ld_wait();
                if (p.state_bf16) {  // a bf16 state is rounded once per chunk
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(bf16_round(__uint_as_float(r[j])));
                }
#pragma unroll
                for (int cc = 0; cc < 4; ++cc)
                    *reinterpret_cast<uint4*>(cell(smem + oS16, 128, c0 * 4 + cc, tid)) =
                        make_uint4(tc::bf16x2(__uint_as_float(r[cc * 8 + 0]), __uint_as_float(r[cc * 8 + 1])),
                                   tc::bf16x2(__uint_as_float(r[cc * 8 + 2]), __uint_as_float(r[cc * 8 + 3])),
                                   tc::bf16x2(__uint_as_float(r[cc * 8 + 4]), __uint_as_float(r[cc * 8 + 5])),
                                   tc::bf16x2(__uint_as_float(r[cc * 8 + 6]), __uint_as_float(r[cc * 8 + 7])));
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * el);
                tc::tmem_st32(tc::tmem_addr(tm, warp, cS + c0 * 32), r);
            }
            tc::tmem_st_wait();
        }
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- 9. QS = Qg S;  D = U - W S (negated A, accumulated onto U) -------------------------------------------------
        if (tid == 0) {
            constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0), idn = tc::idesc_bf16(64, 128, 0, 1, 1);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + cQS, tc::desc_kmajor_bf16(smem + oX, XR, 64, k0), tc::desc_mnmajor_bf16(smem + oS16, 128, 0, k0), id, k0 > 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oX, XR, 128, k0), tc::desc_mnmajor_bf16(smem + oS16, 128, 0, k0), idn, true);
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        mma_phase ^= 1u;
        tc::fence_after_sync();

        // ---- 10. D as bf16 hi + lo cells --------------------------------------------------------------------------------
        {
            const int i = warp * 16 + lane;
            for (int c0 = 0; c0 < 4; ++c0) {
                uint32_t r[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cU + c0 * 32), r);
                tc::tmem_ld_wait();
                if (lane < 16) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t wh[4], wl[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float h0, l0, h1, l1;
                            tc::split_bf16(__uint_as_float(r[cc * 8 + 2 * j]), h0, l0);
                            tc::split_bf16(__uint_as_float(r[cc * 8 + 2 * j + 1]), h1, l1);
                            wh[j] = tc::bf16x2(h0, h1);
                            wl[j] = tc::bf16x2(l0, l1);
                        }
                        *reinterpret_cast<uint4*>(cell(smem + oDhi, CH, c0 * 4 + cc, i)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                        *reinterpret_cast<uint4*>(cell(smem + oDlo, CH, c0 * 4 + cc, i)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                    }
                }
            }
        }
        fence_proxy_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();

        // ---- 11. O = QS + M D;  S += Kdec^T D (hi hi + hi lo + lo hi) --------------------------------------------------
        if (tid == 0) {
            constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0), ids = tc::idesc_bf16(128, 128, 1, 1, 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cQS, tc::desc_kmajor_bf16(smem + oMm, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), id, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), ids, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDlo, CH, 0, k0), ids, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdLo, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), ids, true);
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        mma_phase ^= 1u;
        tc::fence_after_sync();

        // ---- 12. outputs: bf16(y), or the gated RMSNorm of bf16(y) --------------------------------------------------------
        {
            const int i = warp * 16 + lane;
            const bool live = lane < 16 && i < n;
            const long long at = ((gr0 + i) * H + h) * DV;
            float y[128];
            for (int c0 = 0; c0 < 4; ++c0) {
                uint32_t r[32];
                tc::tmem_ld32(tc::tmem_addr(tm, warp, cQS + c0 * 32), r);
                tc::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) y[c0 * 32 + j] = bf16_round(__uint_as_float(r[j]));
            }
            if (live) {
                float rinv = 1.0f;
                if (p.gate != nullptr) {
                    float ss = 0.0f;
#pragma unroll
                    for (int j = 0; j < 128; ++j) ss = fmaf(y[j], y[j], ss);
                    rinv = 1.0f / sqrtf(ss / (float)DV + p.eps);
                }
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    float o[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = y[c * 8 + j];
                    if (p.gate != nullptr) {
                        const uint4 g8 = *reinterpret_cast<const uint4*>(p.gate + at + c * 8);
                        const uint4 w8 = *reinterpret_cast<const uint4*>(p.norm_w + c * 8);
                        const uint32_t gw[4] = {g8.x, g8.y, g8.z, g8.w}, ww[4] = {w8.x, w8.y, w8.z, w8.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
                            const float w0 = __uint_as_float(ww[j] << 16), w1 = __uint_as_float(ww[j] & 0xffff0000u);
                            o[2 * j] = w0 * (o[2 * j] * rinv) * (1.0f / (1.0f + expf(-g0)));
                            o[2 * j + 1] = w1 * (o[2 * j + 1] * rinv) * (1.0f / (1.0f + expf(-g1)));
                        }
                    }
                    *reinterpret_cast<uint4*>(p.out + at + c * 8) =
                        make_uint4(tc::bf16x2(o[0], o[1]), tc::bf16x2(o[2], o[3]), tc::bf16x2(o[4], o[5]), tc::bf16x2(o[6], o[7]));
                }
            }
        }
        tc::fence_before_sync();
        __syncthreads();
        tc::fence_after_sync();
    }

    // ---- the outgoing state -------------------------------------------------------------------------------------------
    if (alive) {
        for (int c0 = 0; c0 < 4; ++c0) {
            uint32_t r[32];
            tc::tmem_ld32(tc::tmem_addr(tm, warp, cS + c0 * 32), r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const long long at = s_elem + (long long)(c0 * 32 + j) * DK + tid;
                if (p.state_bf16) reinterpret_cast<uint16_t*>(p.state_out)[at] = f32_to_bf16_bits(__uint_as_float(r[j]));
                else reinterpret_cast<float*>(p.state_out)[at] = __uint_as_float(r[j]);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tm, kTmemCols);
}

}  // namespace

int core_prefill_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, const glm53f_bf16* q, const glm53f_bf16* k,
                           const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, void* state_out,
                           const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate, const glm53f_bf16* norm_w,
                           float eps, glm53f_bf16* out, cudaStream_t stream) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    TcParams p{};
    p.H = heads;
    p.cu = cu_seqlens;
    p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta;
    p.state_in = state_in; p.state_out = state_out;
    p.state_off = reinterpret_cast<const long long*>(state_off);
    p.state_bf16 = bf16_state ? 1 : 0;
    p.gate = gate; p.norm_w = norm_w; p.eps = eps;
    p.out = out;
    p.status = status_word();
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    prefill_tc_kernel<<<dim3(heads, batch), kThreadsTc, kSmemTc, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace kda
