// Pieces shared by the chunk-64 tensor-core prefill kernels: the chunk geometry, the shared-memory map of the
// state-independent ("intra") phase, the cell helpers and the FP32 triangular inverse.
#pragma once

#include "common.cuh"
#include "tc.cuh"

namespace kda {
namespace pf {

constexpr int CH = 64;            // rows per chunk
constexpr int kCompute = 512;     // 16 compute warps: warp w reaches TMEM lanes 32*(w%4).., and takes columns 32*(w/4)..
constexpr int kThreadsTc = kCompute + 32;  // + one loader warp that streams the next chunk's rows in
constexpr int RS16 = 272;         // staging row stride, bf16 tensors (256 + 16: rows 4 banks apart)
constexpr int RS32 = 528;         // staging row stride, f32 tensor
// Shared memory map (bytes).  Tiles are 64-row (R = 64) cell arrays unless noted; buffers whose lifetimes do not
// overlap inside a chunk share space, so that the staging area is free again as soon as the operands are built and
// the next chunk's rows can stream in behind the current chunk's arithmetic.
constexpr int kTile = CH * 16 * 16;  // 16 KiB: 64 rows x 128 bf16
constexpr int oRawQ = 0, oRawK = oRawQ + CH * RS16, oRawV = oRawK + CH * RS16, oRawG = oRawV + CH * RS16;
constexpr int oKg = oRawG + CH * RS32;   // Kg                       (steps 2-6)   } later S16 [128 rows] (steps 8-9)
constexpr int oKinv = oKg + kTile;        // Kinv (2-3)                             }
constexpr int oTp = oKinv + kTile;        // T' hi | T' lo (5c-6), later D hi (steps 10-11)
constexpr int oW = oTp + kTile;           // W                        (steps 7-9)
constexpr int oV = oW + kTile;            // V                        (steps 2-6), later D lo
constexpr int oQg = oV + kTile;           // Qg                       (steps 2-9)
constexpr int oKdHi = oQg + kTile, oKdLo = oKdHi + kTile;  // Kdec hi, lo (steps 2-11)
constexpr int oMm = oKdLo + kTile;        // M, 64 x 64 bf16          (steps 4-11)
constexpr int oS16 = oKg, oDhi = oTp, oDlo = oV, oTpHi = oTp, oTpLo = oTp + kTile / 2;
// The column sides of L and M, one tile per row block I (rows 0 .. 16 I + 15, 256 bytes a row), over Kinv | T' | W
// (steps 2-3); the per-block decay factor tables (14 x 128 floats: E0[4], EL[4], F[6]) over M (steps 1-3).
constexpr int oKc = oKinv, oTab = oMm, kTabs = 14, tE0 = 0, tEL = 4, tF = 8;
__device__ __forceinline__ int kc_tile(int I) { return 2048 * I * (I + 1); }
static_assert(2 * 128 * (16 + 32 + 48 + 64) <= 3 * kTile && kTabs * 512 <= kTile / 2, "column-side tiles and tables");
// FP32 scratch of the inversion (steps 4-5) over Kinv | T' | W, all dead then: T, P, L.  Rows are padded to 68
// floats so that one lane per row spreads over the banks while float4 loads stay aligned.
constexpr int LS = 68;
constexpr int oT = oKinv, oP = oT + CH * LS * 4, oL = oKinv + 24576;
static_assert(oP + 32 * 32 * 4 <= oL && oL + CH * LS * 4 <= oKinv + 3 * kTile, "inversion scratch");
constexpr int oBeta = oMm + kTile / 2, oEGL = oBeta + 2 * CH * 4, oScan = oEGL + 128 * 4, oRed = oScan + 4 * 128 * 4;
constexpr int oBars = oRed + 4 * CH * 4, oCtl = oBars + 32;
constexpr int kSmemTc = oCtl + 32;
static_assert(kSmemTc <= 232448, "shared memory budget");
// Tensor memory columns.
constexpr uint32_t cS = 0, cL = 128, cMm = 192, cW = 256, cQS = 256, cU = 384, kTmemCols = 512;


__device__ __forceinline__ void compute_sync() { named_bar_sync(1, kCompute); }

__device__ __forceinline__ unsigned char* cell(unsigned char* tile, int R, int c, int r) { return tile + ((size_t)c * R + r) * 16; }

// Eight FP32 values (TMEM words) to one 16-byte cell of bf16.
__device__ __forceinline__ uint4 pack8(const uint32_t* r) {
    return make_uint4(tc::bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])), tc::bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                      tc::bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])), tc::bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
}

// One level of the recursive-doubling inverse of I + L (L strictly lower, 64 x 64).  L is held TRANSPOSED, as the
// tensor core delivers it (Lm[j * LS + i] = L[i][j]); T is held row by row (row stride LS).  Given T correct on
// every sz x sz diagonal block, fills the lower-left sz x sz block of every 2sz x 2sz diagonal block with
// -T22 (L21 T11).  A thread computes VJ consecutive columns of one row; the loops run over the full block (the
// triangular halves that are zero cost a few multiply-adds and keep the trip counts fixed and unrolled).
// NT threads (numbered tid = 0..NT-1) take part and meet at named barrier `bar`.
template <int LG, int NT = kCompute>
__device__ __forceinline__ void invert_level(const float* Lm, float* Tm, float* Pm, int tid, int bar = 1) {
    constexpr int sz = 1 << LG, nblk = 32 >> LG, VJ = sz >= 4 ? 4 : sz, cols = sz / VJ, per = sz * cols, total = nblk * per;
    for (int e = tid; e < total; e += NT) {
        const int blk = e / per, rem = e % per, i = rem / cols, j0 = (rem % cols) * VJ;
        const int c0 = blk * 2 * sz, r0 = c0 + sz;
        const float* Lrow = Lm + c0 * LS + r0 + i;  // L is held transposed: L[r0 + i][c0 + m] at (c0 + m) * LS + r0 + i
        const float* Tc = Tm + c0 * LS + c0 + j0;
        float acc[VJ];
#pragma unroll
        for (int v = 0; v < VJ; ++v) acc[v] = 0.0f;
#pragma unroll
        for (int m = 0; m < sz; ++m) {
            const float l = Lrow[m * LS];
            if constexpr (VJ == 4) {
                const float4 t = *reinterpret_cast<const float4*>(Tc + m * LS);
                acc[0] = fmaf(l, t.x, acc[0]); acc[1] = fmaf(l, t.y, acc[1]); acc[2] = fmaf(l, t.z, acc[2]); acc[3] = fmaf(l, t.w, acc[3]);
            } else {
#pragma unroll
                for (int v = 0; v < VJ; ++v) acc[v] = fmaf(l, Tc[m * LS + v], acc[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < VJ; ++v) Pm[blk * sz * sz + i * sz + j0 + v] = acc[v];
    }
    named_bar_sync(bar, NT);
    for (int e = tid; e < total; e += NT) {
        const int blk = e / per, rem = e % per, i = rem / cols, j0 = (rem % cols) * VJ;
        const int c0 = blk * 2 * sz, r0 = c0 + sz;
        const float* Trow = Tm + (r0 + i) * LS + r0;
        const float* Pc = Pm + blk * sz * sz + j0;
        float acc[VJ];
#pragma unroll
        for (int v = 0; v < VJ; ++v) acc[v] = 0.0f;
#pragma unroll
        for (int m = 0; m < sz; ++m) {
            const float t = Trow[m];
            if constexpr (VJ == 4) {
                const float4 pv = *reinterpret_cast<const float4*>(Pc + m * sz);
                acc[0] = fmaf(t, pv.x, acc[0]); acc[1] = fmaf(t, pv.y, acc[1]); acc[2] = fmaf(t, pv.z, acc[2]); acc[3] = fmaf(t, pv.w, acc[3]);
            } else {
#pragma unroll
                for (int v = 0; v < VJ; ++v) acc[v] = fmaf(t, Pc[m * sz + v], acc[v]);
            }
        }
#pragma unroll
        for (int v = 0; v < VJ; ++v) Tm[(r0 + i) * LS + c0 + j0 + v] = -acc[v];
    }
    named_bar_sync(bar, NT);
}

// The start of the inverse: the four 16 x 16 diagonal blocks of (I + L)^-1 by forward substitution, one thread per
// column (a column needs only its own earlier rows, so the 64 threads never talk to each other), while the other
// threads clear every entry outside those blocks.  Ends with a barrier; levels 4 and 5 of invert_level follow.
template <int NT = kCompute>
__device__ __forceinline__ void invert_diag16(const float* Lm, float* Tm, int tid, int bar = 1) {
    if (tid < 64) {
        const int o = (tid >> 4) * 16, j = tid & 15;
        float t[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const float* Lr = Lm + o * LS + o + i;  // L[o + i][o + m] at (o + m) * LS + o + i
            float a0 = i == j ? 1.0f : 0.0f, a1 = 0.0f;
#pragma unroll
            for (int m = 0; m < i; ++m) {
                if (m & 1) a1 = fmaf(-Lr[m * LS], t[m], a1);
                else a0 = fmaf(-Lr[m * LS], t[m], a0);
            }
            t[i] = a0 + a1;
            Tm[(o + i) * LS + o + j] = t[i];
        }
    } else {
        for (int e = tid - 64; e < CH * CH; e += NT - 64) {
            const int i = e >> 6, j = e & 63;
            if ((i >> 4) != (j >> 4)) Tm[i * LS + j] = 0.0f;
        }
    }
    named_bar_sync(bar, NT);
}

}  // namespace pf
}  // namespace kda
