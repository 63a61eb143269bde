// Chunked KDA prefill on the 5th-generation tensor cores (tcgen05 + TMEM), chunk = 64 rows.
//
// One block (16 compute warps + 1 loader warp) per (sequence, head) walks the sequence's chunks in order; the head's 128x128 state
// stays in tensor memory (FP32 accumulator, 128 lanes = key channel, 128 columns = value channel) from the first
// chunk to the last and touches HBM twice: once in, once out.  Per chunk (the algebra of the reference's CPU
// definition crates/glm53f-kda/src/chunked.rs:67-198, which itself restates chunk_kimi_delta_attention):
//
//   G_i   = g_0 + ... + g_i per key channel (FP32 scan, thread = channel), E = exp(G), E_last = exp(G_63)
//   Kg = k*E, Qg = q*E, Kinv = k/E, Kdec = k * E_last/E                       (operand tiles, written by hand)
//   L = Kg Kinv^T, M = Qg Kinv^T      64x64x128 MMAs; L strictly lower * beta_i, M lower incl. diagonal
//   T  = (I + L)^-1                   FP32 on the CUDA cores by recursive doubling: the lower-left block of every
//                                     2sz x 2sz diagonal block is -T22 (L21 T11), sz = 1 .. 32;  T' = T diag(beta)
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

#include <cuda_fp16.h>

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"
#include "prefill_common.cuh"
#include "tc.cuh"

namespace kda {
namespace {

using namespace pf;

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
    // A pass of a layer prefill (pass_rows > 0): sequence b's inputs are rows b * pass_rows .. of q, k, v, g, beta (its
    // rows row_shift .. row_shift + pass_rows - 1, as many as it has), its outputs and gate rows are rows
    // cu[b] + row_shift .. of `out` and `gate`.  Otherwise inputs and outputs are both rows cu[b] .. cu[b + 1] - 1.
    int pass_rows, row_shift;
    long long gate_stride;  // elements between consecutive gate rows
};

// Two 16-bit values of a q or k row to FP32: bf16 (the core entry points' inputs), or fp16 when the layer prologue
// produced them (normalised q and k lie in [-1, 1]; eleven mantissa bits instead of eight keep the rounding of k, which
// goes into the state through Kdec, below the state's error budget).
template <bool QK16>
__device__ __forceinline__ void widen2(uint32_t w, float& lo, float& hi) {
    if constexpr (QK16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        lo = f.x;
        hi = f.y;
    } else {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xffff0000u);
    }
}

template <bool QK16>
__global__ void __launch_bounds__(kThreadsTc, 1) prefill_tc_kernel(const __grid_constant__ TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bar_raw = reinterpret_cast<uint64_t*>(smem + oBars);
    uint64_t* bar_mma = bar_raw + 1;
    uint64_t* bar_free = bar_raw + 2;  // the staging area may be overwritten
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    float* betas2 = reinterpret_cast<float*>(smem + oBeta);  // [2][64]: the loader fills the next chunk's
    float* egl = reinterpret_cast<float*>(smem + oEGL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, cg = warp >> 2;   // TMEM lane quadrant, column group
    const int lane_row128 = quad * 32 + lane;     // row of an M = 128 accumulator this thread reaches
    const int lane_row64 = quad * 16 + lane;      // row of an M = 64 accumulator (lanes 0..15 only)
    const int h = blockIdx.x, b = blockIdx.y, H = p.H;
    long long in0, out0;
    int T;
    {
        const int r0 = p.cu[b], len = p.cu[b + 1] - r0;
        if (p.pass_rows > 0) {
            T = min(max(len - p.row_shift, 0), p.pass_rows);
            in0 = (long long)b * p.pass_rows;
            out0 = (long long)r0 + p.row_shift;
        } else {
            T = len;
            in0 = out0 = r0;
        }
    }
    const long long s_elem = p.state_off[b] + (long long)h * DV * DK;

    if (tid == 0) {
        mbar_init(bar_raw, 1);
        mbar_init(bar_mma, 1);
        mbar_init(bar_free, 1);
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

    // ---- the loader warp: for every chunk, once the staging area is free, one bulk copy per row and tensor ----------
    if (warp == kCompute / 32) {
        uint32_t free_phase = 0;
        for (int s = 0, it = 0; s < T; s += CH, ++it) {
            if (it > 0) {
                if (!mbar_wait(bar_free, free_phase, ctx, kStatusWaitPrefill)) break;
                free_phase ^= 1u;
            }
            const int n = min(CH, T - s);
            const long long gr0 = in0 + s;
            float* bt = betas2 + (it & 1) * CH;
            for (int r = lane; r < CH; r += 32) {
                bt[r] = r < n ? p.beta[(gr0 + r) * H + h] : 0.0f;
                if (r >= n) {  // rows past the end of the sequence are zero
                    const uint4 z = make_uint4(0, 0, 0, 0);
                    for (int e = 0; e < 16; ++e) {
                        *reinterpret_cast<uint4*>(smem + oRawQ + r * RS16 + e * 16) = z;
                        *reinterpret_cast<uint4*>(smem + oRawK + r * RS16 + e * 16) = z;
                        *reinterpret_cast<uint4*>(smem + oRawV + r * RS16 + e * 16) = z;
                    }
                    for (int e = 0; e < 32; ++e) *reinterpret_cast<uint4*>(smem + oRawG + r * RS32 + e * 16) = z;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_expect_tx(bar_raw, (uint32_t)n * (3 * 256 + 512));  // releases beta and the zero rows
            for (int r = lane; r < n; r += 32) {
                const long long at = ((gr0 + r) * H + h) * DK;
                bulk_load(smem + oRawQ + r * RS16, p.q + at, 256, bar_raw);
                bulk_load(smem + oRawK + r * RS16, p.k + at, 256, bar_raw);
                bulk_load(smem + oRawV + r * RS16, p.v + at, 256, bar_raw);
                bulk_load(smem + oRawG + r * RS32, p.g + at, 512, bar_raw);
            }
        }
        tc::fence_before_sync();
        __syncthreads();  // the block's final barrier
        return;
    }

    // One round of MMAs: thread 0 issues and commits, everybody waits for the tensor core.
    auto mma_round = [&](auto&& issue) -> bool {
        if (tid == 0) {
            issue();
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) return false;
        mma_phase ^= 1u;
        tc::fence_after_sync();
        return true;
    };
    auto publish_operands = [&]() {  // generic-proxy writes -> tensor core, and TMEM accesses ordered across the block
        fence_proxy_async_smem();
        tc::fence_before_sync();
        compute_sync();
        tc::fence_after_sync();
    };

    // ---- the incoming state into tensor memory: lane = key channel, columns = value channel -----------------------
    {
        uint32_t r[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const long long at = s_elem + (long long)(cg * 32 + j) * DK + lane_row128;
            const float x = p.state_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(p.state_in)[at])
                                         : reinterpret_cast<const float*>(p.state_in)[at];
            r[j] = __float_as_uint(x);
        }
        tc::tmem_st32(tc::tmem_addr(tm, quad, cS + cg * 32), r);
        tc::tmem_st_wait();
    }

    for (int s = 0; s < T; s += CH) {
        const int n = min(CH, T - s);
        const long long gr0 = out0 + s;
        const float* betas = betas2 + ((s / CH) & 1) * CH;
        if (!mbar_wait(bar_raw, raw_phase, ctx, kStatusWaitPrefill)) { alive = false; break; }
        raw_phase ^= 1u;

        bool mild;
        // ---- 1. per key channel: the cumulative log decay G, a = exp(G - Gm) of every row relative to the middle row of
        // its block of 16 (left in the staging buffer in place of g), and the per-block factor tables.
        // Thread (part, d): rows 16*part .. 16*part+15 of channel d, which is exactly row block J = part.
        {
            const int part = tid >> 7, d = tid & 127;
            float* col = reinterpret_cast<float*>(smem + oRawG + (part * 16) * RS32) + d;
            float* totals = reinterpret_cast<float*>(smem + oScan);
            float* tab = reinterpret_cast<float*>(smem + oTab) + d;
            float loc[16], G = 0.0f;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                G += *reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(col) + r * RS32);
                loc[r] = G;
            }
            totals[part * 128 + d] = G;
            tab[part * 128] = loc[8];  // the block's middle row, relative to the block's start, until the tables are written
            float amax = 0.0f;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const float av = __expf(loc[r] - loc[8]);
                amax = fmaxf(amax, av);
                *reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(col) + r * RS32) = av;
            }
            // Eight rows of decay must stay below e^85: per-row log decays below about -10.6 (or positive ones) do not.
            if (!(amax < 1e37f)) atomicCAS(p.status, 0, kStatusPrefillRange);
            compute_sync();
            float start[5];  // G before each block's first row, and after the last row
            start[0] = 0.0f;
#pragma unroll
            for (int q2 = 0; q2 < 4; ++q2) start[q2 + 1] = start[q2] + totals[q2 * 128 + d];
            float gm[4];
#pragma unroll
            for (int q2 = 0; q2 < 4; ++q2) gm[q2] = start[q2] + tab[q2 * 128];
            compute_sync();  // the relative middles have been read: the tables may be written over them
            tab[(tE0 + part) * 128] = __expf(gm[part]);
            tab[(tEL + part) * 128] = __expf(start[4] - gm[part]);
#pragma unroll
            for (int I = 1; I < 4; ++I)
                if (I > part) tab[(tF + I * (I - 1) / 2 + part) * 128] = __expf(gm[I] - gm[part]);
            if (part == 3) egl[d] = __expf(start[4]);
            mild = start[4] > -60.0f;
        }
        // A chunk whose whole decay stays above e^-60 in every channel takes one reference row (the chunk's start): one
        // column-side tile, one product each for L^T and M^T, no second operand pass.  The block decides together (the
        // barrier carries the vote) from the chunk's own gates.
        const bool narrow = named_bar_all(1, kCompute, mild);

        if (narrow) {
            const int r = tid & 63, cgrp = tid >> 6, J = r >> 4;
            const float* tabs = reinterpret_cast<const float*>(smem + oTab);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = cgrp * 2 + cc;
                const uint4 k8 = *reinterpret_cast<const uint4*>(smem + oRawK + r * RS16 + c * 16);
                const uint4 q8 = *reinterpret_cast<const uint4*>(smem + oRawQ + r * RS16 + c * 16);
                const uint4 v8 = *reinterpret_cast<const uint4*>(smem + oRawV + r * RS16 + c * 16);
                const float4 a0 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32);
                const float4 a1 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32 + 16);
                const float4 e0 = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8);
                const float4 e1 = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8 + 4);
                const float4 l0 = *reinterpret_cast<const float4*>(egl + c * 8);
                const float4 l1 = *reinterpret_cast<const float4*>(egl + c * 8 + 4);
                const float E[8] = {a0.x * e0.x, a0.y * e0.y, a0.z * e0.z, a0.w * e0.w, a1.x * e1.x, a1.y * e1.y, a1.z * e1.z, a1.w * e1.w};
                const float EL[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
                const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w}, qw[4] = {q8.x, q8.y, q8.z, q8.w};
                uint32_t kg[4], qg[4], ki[4], dh[4], dl[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float kf[2], qf[2], vi[2], hi[2], lo[2];
                    widen2<QK16>(kw[j], kf[0], kf[1]);
                    widen2<QK16>(qw[j], qf[0], qf[1]);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float einv = __fdividef(1.0f, E[2 * j + u]);
                        vi[u] = kf[u] * einv;
                        tc::split_bf16(kf[u] * (EL[2 * j + u] * einv), hi[u], lo[u]);
                    }
                    kg[j] = tc::bf16x2(kf[0] * E[2 * j], kf[1] * E[2 * j + 1]);
                    qg[j] = tc::bf16x2(qf[0] * E[2 * j], qf[1] * E[2 * j + 1]);
                    ki[j] = tc::bf16x2(vi[0], vi[1]);
                    dh[j] = tc::bf16x2(hi[0], hi[1]);
                    dl[j] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(cell(smem + oKg, CH, c, r)) = make_uint4(kg[0], kg[1], kg[2], kg[3]);
                *reinterpret_cast<uint4*>(cell(smem + oQg, CH, c, r)) = make_uint4(qg[0], qg[1], qg[2], qg[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKc + kc_tile(3), CH, c, r)) = make_uint4(ki[0], ki[1], ki[2], ki[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdHi, CH, c, r)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdLo, CH, c, r)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4*>(cell(smem + oV, CH, c, r)) = v8;
            }
            publish_operands();
            if (tid == 0 && s + CH < T) mbar_arrive(bar_free);  // the staging area is free for the next chunk's rows
            if (!mma_round([&] {
                    constexpr uint32_t id = tc::idesc_bf16(64, 64, 0, 0, 0);
                    const unsigned char* kit = smem + oKc + kc_tile(3);
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + cL, tc::desc_kmajor_bf16(kit, CH, 0, k0), tc::desc_kmajor_bf16(smem + oKg, CH, 0, k0), id, k0 > 0);
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + cMm, tc::desc_kmajor_bf16(kit, CH, 0, k0), tc::desc_kmajor_bf16(smem + oQg, CH, 0, k0), id, k0 > 0);
                })) { alive = false; break; }
        } else {
        // ---- 2. operand tiles: lane <-> row, one 16-byte cell (8 channels) at a time.  Row sides Kgb = K a -> oKg, Qgb = Q a ->
        // oQg; the column sides K exp(Gm_I - G) into the four tiles I >= J; Kdec = K exp(G_last - G) as bf16 hi + lo; V as it is.
        {
            const int r = tid & 63, cgrp = tid >> 6, J = r >> 4;
            const float* tabs = reinterpret_cast<const float*>(smem + oTab);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = cgrp * 2 + cc;
                const uint4 k8 = *reinterpret_cast<const uint4*>(smem + oRawK + r * RS16 + c * 16);
                const uint4 q8 = *reinterpret_cast<const uint4*>(smem + oRawQ + r * RS16 + c * 16);
                const uint4 v8 = *reinterpret_cast<const uint4*>(smem + oRawV + r * RS16 + c * 16);
                const float4 a0 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32);
                const float4 a1 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32 + 16);
                const float4 l0 = *reinterpret_cast<const float4*>(tabs + (tEL + J) * 128 + c * 8);
                const float4 l1 = *reinterpret_cast<const float4*>(tabs + (tEL + J) * 128 + c * 8 + 4);
                const float A[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const float EL[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
                const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w}, qw[4] = {q8.x, q8.y, q8.z, q8.w};
                uint32_t kgb[4], qgb[4], kcd[4], dh[4], dl[4];
                float kc[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float kf[2], qf[2];
                    widen2<QK16>(kw[j], kf[0], kf[1]);
                    widen2<QK16>(qw[j], qf[0], qf[1]);
                    float hi[2], lo[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        kc[2 * j + u] = kf[u] * __fdividef(1.0f, A[2 * j + u]);
                        tc::split_bf16(kc[2 * j + u] * EL[2 * j + u], hi[u], lo[u]);
                    }
                    kgb[j] = tc::bf16x2(kf[0] * A[2 * j], kf[1] * A[2 * j + 1]);
                    qgb[j] = tc::bf16x2(qf[0] * A[2 * j], qf[1] * A[2 * j + 1]);
                    kcd[j] = tc::bf16x2(kc[2 * j], kc[2 * j + 1]);
                    dh[j] = tc::bf16x2(hi[0], hi[1]);
                    dl[j] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(cell(smem + oKg, CH, c, r)) = make_uint4(kgb[0], kgb[1], kgb[2], kgb[3]);
                *reinterpret_cast<uint4*>(cell(smem + oQg, CH, c, r)) = make_uint4(qgb[0], qgb[1], qgb[2], qgb[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdHi, CH, c, r)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(cell(smem + oKdLo, CH, c, r)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
                *reinterpret_cast<uint4*>(cell(smem + oV, CH, c, r)) = v8;
                *reinterpret_cast<uint4*>(cell(smem + oKc + kc_tile(J), 16 * (J + 1), c, r)) = make_uint4(kcd[0], kcd[1], kcd[2], kcd[3]);
                for (int I = J + 1; I < 4; ++I) {  // the later row blocks see this row through exp(Gm_I - Gm_J) <= 1
                    const float* f = tabs + (tF + I * (I - 1) / 2 + J) * 128 + c * 8;
                    const float4 fa = *reinterpret_cast<const float4*>(f), fb = *reinterpret_cast<const float4*>(f + 4);
                    *reinterpret_cast<uint4*>(cell(smem + oKc + kc_tile(I), 16 * (I + 1), c, r)) =
                        make_uint4(tc::bf16x2(kc[0] * fa.x, kc[1] * fa.y), tc::bf16x2(kc[2] * fa.z, kc[3] * fa.w),
                                   tc::bf16x2(kc[4] * fb.x, kc[5] * fb.y), tc::bf16x2(kc[6] * fb.z, kc[7] * fb.w));
                }
            }
        }
        publish_operands();

        // ---- 3. L^T and M^T, one block column of 16 rows i at a time: [64 j x 16 i] = column side (tile I) x row side (block I)^T
        if (!mma_round([&] {
                constexpr uint32_t id = tc::idesc_bf16(64, 16, 0, 0, 0);
                for (int I = 0; I < 4; ++I) {
                    const unsigned char* kct = smem + oKc + kc_tile(I);
                    const int R = 16 * (I + 1);
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + cL + 16 * I, tc::desc_kmajor_bf16(kct, R, 0, k0), tc::desc_kmajor_bf16(smem + oKg, CH, 16 * I, k0), id, k0 > 0);
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + cMm + 16 * I, tc::desc_kmajor_bf16(kct, R, 0, k0), tc::desc_kmajor_bf16(smem + oQg, CH, 16 * I, k0), id, k0 > 0);
                }
            })) { alive = false; break; }

        // ---- 3b. the tiles that take the decay from the chunk's start, over the row sides (the tensor core is done with
        // them): Kg = K exp(G) for W, Qg = Q exp(G) for Q S.  Then the staging area is free.
        {
            const int r = tid & 63, cgrp = tid >> 6, J = r >> 4;
            const float* tabs = reinterpret_cast<const float*>(smem + oTab);
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = cgrp * 2 + cc;
                const uint4 k8 = *reinterpret_cast<const uint4*>(smem + oRawK + r * RS16 + c * 16);
                const uint4 q8 = *reinterpret_cast<const uint4*>(smem + oRawQ + r * RS16 + c * 16);
                const float4 a0 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32);
                const float4 a1 = *reinterpret_cast<const float4*>(smem + oRawG + r * RS32 + c * 32 + 16);
                const float4 e0 = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8);
                const float4 e1 = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8 + 4);
                const float E[8] = {a0.x * e0.x, a0.y * e0.y, a0.z * e0.z, a0.w * e0.w, a1.x * e1.x, a1.y * e1.y, a1.z * e1.z, a1.w * e1.w};
                const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w}, qw[4] = {q8.x, q8.y, q8.z, q8.w};
                uint32_t kg[4], qg[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float kf[2], qf[2];
                    widen2<QK16>(kw[j], kf[0], kf[1]);
                    widen2<QK16>(qw[j], qf[0], qf[1]);
                    kg[j] = tc::bf16x2(kf[0] * E[2 * j], kf[1] * E[2 * j + 1]);
                    qg[j] = tc::bf16x2(qf[0] * E[2 * j], qf[1] * E[2 * j + 1]);
                }
                *reinterpret_cast<uint4*>(cell(smem + oKg, CH, c, r)) = make_uint4(kg[0], kg[1], kg[2], kg[3]);
                *reinterpret_cast<uint4*>(cell(smem + oQg, CH, c, r)) = make_uint4(qg[0], qg[1], qg[2], qg[3]);
            }
        }
        compute_sync();  // every thread is done with the staging area and the tables (M goes over them next)
        // The staging area is free: the loader streams the next chunk's rows in behind this chunk's arithmetic.
        if (tid == 0 && s + CH < T) mbar_arrive(bar_free);
        }

        // ---- 4. from L^T and M^T (lane = column j, tensor-memory column = row i): L (FP32, strictly lower, times beta_i); M
        // (lower with the diagonal) as bf16 cells of eight consecutive rows i, [8 cells][64 columns j].  Column groups 0, 1
        // take the two halves (of i) of L, groups 2, 3 those of M; lanes 0..15 hold the columns.
        {
            uint32_t r[32];
            const int half = cg & 1, j = lane_row64;
            tc::tmem_ld32(tc::tmem_addr(tm, quad, (cg < 2 ? cL : cMm) + half * 32), r);
            tc::tmem_ld_wait();
            if (lane < 16) {
                if (cg < 2) {  // L stays transposed: this thread's column j, 32 consecutive rows i
                    float* Lt = reinterpret_cast<float*>(smem + oL) + j * LS + half * 32;
#pragma unroll
                    for (int i4 = 0; i4 < 8; ++i4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(betas + half * 32 + i4 * 4);
                        const int i = half * 32 + i4 * 4;
                        *reinterpret_cast<float4*>(Lt + i4 * 4) = make_float4(i > j ? b4.x * __uint_as_float(r[i4 * 4]) : 0.0f, i + 1 > j ? b4.y * __uint_as_float(r[i4 * 4 + 1]) : 0.0f,
                                                                              i + 2 > j ? b4.z * __uint_as_float(r[i4 * 4 + 2]) : 0.0f, i + 3 > j ? b4.w * __uint_as_float(r[i4 * 4 + 3]) : 0.0f);
                    }
                } else {
#pragma unroll
                    for (int i2 = 0; i2 < 32; ++i2)
                        if (half * 32 + i2 < j) r[i2] = 0u;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(cell(smem + oMm, CH, half * 4 + cc, j)) = pack8(r + cc * 8);
                }
            }
        }
        compute_sync();

        // ---- 5. T = (I + L)^-1 in FP32 ------------------------------------------------------------------------------------------
        {
            const float* Lm = reinterpret_cast<const float*>(smem + oL);
            float* Tm = reinterpret_cast<float*>(smem + oT);
            float* Pm = reinterpret_cast<float*>(smem + oP);
            // Recursive doubling.  T starts as the identity; at block size sz the lower-left sz x sz block of every
            // 2sz x 2sz diagonal block is -T22 (L21 T11), all blocks and elements in parallel.
            invert_diag16(Lm, Tm, tid);
            invert_level<4>(Lm, Tm, Pm, tid);
            invert_level<5>(Lm, Tm, Pm, tid);
            // 5c. T' = T diag(beta) as bf16 hi + lo cells.  T' lands on the scratch itself, so every thread first reads
            // its eight values of T, then the block synchronises, then the cells are written.
            {
                const int i = tid & 63, c = tid >> 6;
                float t8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) t8[j] = Tm[i * LS + c * 8 + j] * betas[c * 8 + j];
                compute_sync();
                uint32_t wh[4], wl[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float h0, l0, h1, l1;
                    tc::split_bf16(t8[2 * j], h0, l0);
                    tc::split_bf16(t8[2 * j + 1], h1, l1);
                    wh[j] = tc::bf16x2(h0, h1);
                    wl[j] = tc::bf16x2(l0, l1);
                }
                *reinterpret_cast<uint4*>(cell(smem + oTpHi, CH, c, i)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                *reinterpret_cast<uint4*>(cell(smem + oTpLo, CH, c, i)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            }
        }
        publish_operands();

        // ---- 6. W = T' Kg (bf16 T'), U = T' V (T' hi + lo) -------------------------------------------------------------------
        if (!mma_round([&] {
                constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cW, tc::desc_kmajor_bf16(smem + oTpHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oKg, CH, 0, k0), id, k0 > 0);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oTpHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oV, CH, 0, k0), id, k0 > 0);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oTpLo, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oV, CH, 0, k0), id, true);
            })) { alive = false; break; }

        // ---- 7. W to bf16 cells; 8. S to bf16 cells (over Kg | Kinv, both dead), the decayed S back to tensor memory ------------
        {
            uint32_t r[32];
            tc::tmem_ld32(tc::tmem_addr(tm, quad, cW + cg * 32), r);
            tc::tmem_ld_wait();
            if (lane < 16) {
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(cell(smem + oW, CH, cg * 4 + cc, lane_row64)) = pack8(r + cc * 8);
            }
            tc::tmem_ld32(tc::tmem_addr(tm, quad, cS + cg * 32), r);
            tc::tmem_ld_wait();
            if (p.state_bf16) {  // a bf16 state is rounded once per chunk
#pragma unroll
                for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(bf16_round(__uint_as_float(r[j])));
            }
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(cell(smem + oS16, 128, cg * 4 + cc, lane_row128)) = pack8(r + cc * 8);
            const float el = egl[lane_row128];
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * el);
            tc::tmem_st32(tc::tmem_addr(tm, quad, cS + cg * 32), r);
            tc::tmem_st_wait();
        }
        publish_operands();

        // ---- 9. QS = Qg S;  D = U - W S (negated A, accumulated onto U) ----------------------------------------------------------
        if (!mma_round([&] {
                constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0), idn = tc::idesc_bf16(64, 128, 0, 1, 1);
                for (int k0 = 0; k0 < DK; k0 += 16)
                    tc::mma_bf16(tm + cQS, tc::desc_kmajor_bf16(smem + oQg, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oS16, 128, 0, k0), id, k0 > 0);
                for (int k0 = 0; k0 < DK; k0 += 16)
                    tc::mma_bf16(tm + cU, tc::desc_kmajor_bf16(smem + oW, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oS16, 128, 0, k0), idn, true);
            })) { alive = false; break; }

        // ---- 10. D as bf16 hi + lo cells (over T' | V, both dead) -------------------------------------------------------------------
        {
            uint32_t r[32];
            tc::tmem_ld32(tc::tmem_addr(tm, quad, cU + cg * 32), r);
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
                    *reinterpret_cast<uint4*>(cell(smem + oDhi, CH, cg * 4 + cc, lane_row64)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *reinterpret_cast<uint4*>(cell(smem + oDlo, CH, cg * 4 + cc, lane_row64)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
            }
        }
        publish_operands();

        // ---- 11. O = QS + M D;  S += Kdec^T D (hi hi + hi lo + lo hi) ------------------------------------------------------------------
        if (!mma_round([&] {
                constexpr uint32_t idm = tc::idesc_bf16(64, 128, 1, 1, 0), ids = tc::idesc_bf16(128, 128, 1, 1, 0);  // M has its rows contiguous
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cQS, tc::desc_mnmajor_bf16(smem + oMm, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), idm, true);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), ids, true);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdHi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDlo, CH, 0, k0), ids, true);
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + cS, tc::desc_mnmajor_bf16(smem + oKdLo, CH, 0, k0), tc::desc_mnmajor_bf16(smem + oDhi, CH, 0, k0), ids, true);
            })) { alive = false; break; }

        // ---- 12. outputs: bf16(y), or the gated RMSNorm of bf16(y); a thread holds 32 columns of its row -------------------------------
        {
            uint32_t r[32];
            tc::tmem_ld32(tc::tmem_addr(tm, quad, cQS + cg * 32), r);
            tc::tmem_ld_wait();
            const int i = lane_row64;
            const bool live = lane < 16 && i < n;
            const long long at = ((gr0 + i) * H + h) * DV + cg * 32;
            float y[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) y[j] = bf16_round(__uint_as_float(r[j]));
            if (p.gate != nullptr) {
                float* red = reinterpret_cast<float*>(smem + oRed);
                float ss = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) ss = fmaf(y[j], y[j], ss);
                if (lane < 16) red[cg * CH + i] = ss;
                compute_sync();
                if (live) {
                    const float tot = (red[i] + red[CH + i]) + (red[2 * CH + i] + red[3 * CH + i]);
                    const float rinv = 1.0f / sqrtf(tot / (float)DV + p.eps);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float gt = bf16_bits_to_f32(p.gate[(gr0 + i) * p.gate_stride + h * DV + cg * 32 + j]), w = bf16_bits_to_f32(p.norm_w[cg * 32 + j]);
                        y[j] = w * (y[j] * rinv) * (1.0f / (1.0f + __expf(-gt)));
                    }
                }
            }
            if (live) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(p.out + at + c * 8) = make_uint4(tc::bf16x2(y[c * 8], y[c * 8 + 1]), tc::bf16x2(y[c * 8 + 2], y[c * 8 + 3]),
                                                                            tc::bf16x2(y[c * 8 + 4], y[c * 8 + 5]), tc::bf16x2(y[c * 8 + 6], y[c * 8 + 7]));
            }
        }
        tc::fence_before_sync();
        compute_sync();
        tc::fence_after_sync();
    }

    // ---- the outgoing state -------------------------------------------------------------------------------------------------------
    if (alive) {
        uint32_t r[32];
        tc::tmem_ld32(tc::tmem_addr(tm, quad, cS + cg * 32), r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const long long at = s_elem + (long long)(cg * 32 + j) * DK + lane_row128;
            if (p.state_bf16) reinterpret_cast<uint16_t*>(p.state_out)[at] = f32_to_bf16_bits(__uint_as_float(r[j]));
            else reinterpret_cast<float*>(p.state_out)[at] = __uint_as_float(r[j]);
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
                           float eps, glm53f_bf16* out, cudaStream_t stream, const PrefillWindow* win) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTc);
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
    p.gate_stride = (long long)heads * DV;
    if (win != nullptr) {
        p.pass_rows = win->pass_rows;
        p.row_shift = win->row_shift;
        p.gate_stride = win->gate_stride;
    }
    p.status = status_word();
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    if (win != nullptr && win->qk_fp16) prefill_tc_kernel<true><<<dim3(heads, batch), kThreadsTc, kSmemTc, stream>>>(p);
    else prefill_tc_kernel<false><<<dim3(heads, batch), kThreadsTc, kSmemTc, stream>>>(p);
    return (int)cudaGetLastError();
}

}  // namespace kda
