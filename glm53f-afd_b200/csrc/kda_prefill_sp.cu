// Chunk-64 tensor-core prefill in two passes over a caller-provided workspace, for launches with few (sequence,
// head) chains: a single long sequence, or a GPU's shard of heads.
//
// The arithmetic is that of kda_prefill_tc.cu (same operand tiles, same products, same precision mix).  What
// changes is where it runs.  Everything of a chunk that does not need the recurrent state -- the decay scan, the
// operand tiles, L, M, the triangular inverse, W = T'Kg and U = T'V, about two thirds of a chunk's time -- is
// independent from chunk to chunk, so the *intra role* spreads those (chain, chunk) items over every SM and leaves
// per item, in the workspace, exactly what the state recurrence consumes: Qg, W, M, Kdec hi/lo (bf16 cell tiles),
// U (FP32) and exp(G_last).  The *state role*, one block per chain, walks the chunks in order with the state in
// tensor memory and only the short dependent part per chunk: S as bf16 operand, QS = Qg S and -W S, D = U - W S,
// O = QS + M D, S <- E_last S + Kdec^T D.
//
// The sequence is cut into segments sized by the workspace.  One kernel launch runs the state role for segment s-1
// (blocks 0..chains-1) and the intra role for segment s (every block, the chain blocks after their state work; items
// are handed out through a counter in the workspace), on two halves of the workspace that swap from launch to
// launch.  Stream order between launches is the only synchronisation: no block ever waits on another block.
//
// Workspace slot of one (chain, chunk) item, bytes: Qg 0 | W 16,384 | M 32,768 | Kdec hi 40,960 | Kdec lo 57,344 |
// U 73,728 (FP32, 32 cells of four value channels x 64 rows) | E_last 106,496 (128 floats); 107,008 per slot = 1,672 per row and head, inside
// the 2,176 the reference's prefill workspace formula provides (kernels/kda_prefill.cu:40-43, 695-698).  The last
// 256 bytes of the workspace hold the two item counters.

#include <cstdlib>

#include <cuda.h>

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"
#include "prefill_common.cuh"
#include "tc.cuh"

namespace kda {
namespace {

using namespace pf;

// U is kept in FP32 as 16-byte cells of four value channels, [32 cells][64 rows], so that both its writer (a thread
// holds a row's channels) and its reader store and load consecutive cells.
constexpr int wQg = 0, wW = kTile, wMm = 2 * kTile, wKdHi = wMm + kTile / 2, wKdLo = wKdHi + kTile, wU = wKdLo + kTile;
constexpr int kUBytes = CH * DV * 4, wEgl = wU + kUBytes, kSlotBytes = wEgl + 512;
static_assert(kSlotBytes == 107008 && wU == 73728, "workspace slot layout");

// Staging of a chunk's raw rows in the intra kernel: dense boxes of 64 rows x 128 bytes written by tiled tensor copies
// with the 128-byte swizzle (16-byte piece p of row r sits at piece p ^ (r & 7)), so that threads walking down the
// rows of one column spread over all banks.  q, k, v: two boxes each (channels 0-63, 64-127); the log decays: four.
constexpr int kBox = CH * 128;  // 8 KiB
// Byte offset inside a tensor's staging of the 16-byte piece `piece` (0..15 for bf16 rows, 0..31 for f32 rows) of row r.
__device__ __forceinline__ int box_piece(int r, int piece) { return (piece >> 3) * kBox + r * 128 + (((piece & 7) ^ (r & 7)) << 4); }

struct SpParams {
    alignas(64) CUtensorMap tm_q, tm_k, tm_v, tm_g;  // [rows][H][128] as (128, H, rows); boxes of 64 rows x 128 bytes, 128-byte swizzle
    alignas(64) CUtensorMap tm_out;                  // the shard-local output, the same way
    alignas(64) CUtensorMap tm_full[8];              // every rank's full output buffer: (128, heads_total, rows)
    int H, batch;
    const int32_t* cu;
    const uint16_t *q, *k, *v;
    const float* g;
    const float* beta;
    const void* state_in;   // segment 0 reads the caller's state, later segments the state written so far
    void* state_out;
    const long long* state_off;
    int state_bf16;
    const uint16_t* gate;
    const uint16_t* norm_w;
    float eps;
    uint16_t* out;
    int seg_chunks;          // chunks of every sequence per segment = slots per chain in a workspace half
    unsigned char* ws_intra; // intra role: chunks [intra_chunk0, intra_chunk0 + seg_chunks) of every sequence, or none
    int intra_chunk0, has_intra;
    unsigned char* ws_state; // state role: chunks [state_chunk0, state_chunk0 + seg_chunks) of every sequence, or none
    int state_chunk0, has_state;
    uint16_t* full[8];       // head-sharded launches: every rank's full [rows][heads_total][128] output buffer, or none
    int ranks, heads_total, head0;
    int parts;               // state-role blocks per chain: 1, or 2 (each owns half of the value channels)
    unsigned int* counters;  // [2] item counters: this launch hands items out of counters[ctr], and zeroes the other
    int ctr;
    int* status;
    // The scan over segments of the sequence (scan_pass != 0; FP32 states; the workspace holds every chunk).  Segment s of
    // a chain covers chunks [s * scan_chunks, (s + 1) * scan_chunks).
    //   pass 1  blocks (chain, s < K - 1, kind): the walk of segment s without outputs, from the zero state (kind 0: its
    //           end state is the segment's offset B_s) and from the identity with U = 0 (kind 1: its end state is the
    //           segment's transition A_s), written to scan_ab
    //   pass 2  blocks (chain, s): the walk of segment s with outputs from its true incoming state scan_start (composed
    //           from the A_s, B_s between the two passes); the last segment writes the final state
    int scan_pass, scan_k, scan_chunks;
    int scan_open;      // the last segment runs to the sequence's end (the call's last super-block), else to the end of
                        // this launch's chunk range [state_chunk0, state_chunk0 + seg_chunks)
    int scan_p1;        // segments pass 1 walks: K - 1, or K when the state after the range is wanted before pass 2 runs
    const float* scan_carry_in;  // super-blocks: the FP32 state before this launch's range, [chain][128 x 128] (NULL: state_in)
    float* scan_carry_out;       // super-blocks: the FP32 state after this launch's range (scan_p1 == K)
    float* scan_ab;     // [chain][K - 1][2][128 x 128]: B_s, A_s in the state's layout
    float* scan_start;  // [chain][K][128 x 128]: the state before each segment (segment 0: unused, the caller's state)
};

__device__ __forceinline__ unsigned char* slot_of(unsigned char* ws, int seg_chunks, int chain, int jj) {
    return ws + ((size_t)chain * seg_chunks + jj) * kSlotBytes;
}

// The state role's barriers sit behind every tile (set up once at kernel entry, never repurposed).  The intra role's
// live inside its two groups' areas, which the state role -- it runs first in a block -- uses as tile space, so they are
// set up when the intra role starts.
constexpr int oBarsState = kSmemTc, kSmemSp = kSmemTc + 128;
// 16 compute warps, the loader warp, and (state role only) a warp that moves finished output rows to global memory.
constexpr int kThreadsSp = kCompute + 64, kLoaderWarp = kCompute / 32, kOutWarp = kCompute / 32 + 1;
static_assert(kSmemSp <= 232448, "shared memory budget");

// =====================================================================================================================
// Pass 1: the state-independent part of every (chain, chunk) item of the segment, items handed out by a counter.
//
// A block runs two items at a time: two groups of eight warps, each with its own staging, tensor-memory columns,
// barriers and loader warp, so that one group's waits (tensor-core rounds, tensor-memory reads, its own barriers) are
// filled by the other group's arithmetic.  To fit two items, a group keeps 96 KiB: q, k, v and the log decays arrive
// by tiled tensor copies in the 128-byte swizzle, which is an operand layout of the tensor core (K-major for the
// products over key channels, MN-major for the products over rows), so k and q are turned into Kg and Qg in place and
// v is used as it lands; the log decays become E in place; the inverse's FP32 scratch goes over E and Kinv once they
// are dead; and everything the state role needs leaves for the workspace straight from registers (Qg, Kdec hi/lo,
// E_last, M, W, U), in the un-swizzled cell layout the state role reads, so no result tile lives in shared memory.
// =====================================================================================================================
constexpr int kGroupThreads = 256, kGroups = 2;
// Decay range.  L and M hold exp(G_i - G_j) for every pair of rows j <= i of a chunk, and a tensor-core product can
// only form it as (row factor) x (column factor).  With the model's gate bound (log decay down to -5.8 per row, -371
// per chunk) neither exp(G) nor exp(-G) is representable, so the pair is split at a reference row r between j and i:
// exp(G_i - G_r) exp(G_r - G_j).  Rows are grouped in blocks of 16 and the reference of row block I is its middle row
// (16 I + 8).  The row side k_i exp(G_i - Gm_I) then stays within e^+-47; the column side for row block I is
// k_j exp(Gm_I - G_j) for every j below the end of block I: at most e^47 inside the block and at most 1 (vanishing
// harmlessly where the true product vanishes) in earlier blocks.  It depends on I, so there are four column-side
// tiles of 16, 32, 48 and 64 rows, and L^T, M^T are formed block column by block column (N = 16) with the column side
// as the M operand: rows past a tile's end produce entries above the diagonal, which are discarded.
constexpr int kKcBytes = 2 * 128 * (16 + 32 + 48 + 64);  // the four column-side tiles, boxes of R x 128 bytes
// Tile I starts at pf::kc_tile(I).  Byte offset inside tile I (R = 16 (I + 1) rows per box) of the 16-byte piece `piece` (0..15) of row r.
__device__ __forceinline__ int kc_piece(int I, int r, int piece) {
    return kc_tile(I) + (piece >> 3) * (I + 1) * 2048 + r * 128 + (((piece & 7) ^ (r & 7)) << 4);
}
constexpr int gQ = 0, gK = kTile, gV = 2 * kTile, gKb = 3 * kTile, gG = 4 * kTile, gKc = gG;  // Q/Qgb | K/Kg | V | Kgb | g/G, then the column-side tiles
constexpr int gT = gKc, gL = gT + CH * LS * 4, gP = gL + CH * LS * 4, gTp = gL;              // inverse scratch over the column-side tiles; T' (hi | lo box) over L
static_assert(gTp % 1024 == 0 && gKc % 1024 == 0, "swizzled tiles are 1024-byte aligned");
// Per-block decay factors, 128 channels each: E0[J] = exp(Gm_J), EL[J] = exp(G_last - Gm_J), F[I(I-1)/2 + J] =
// exp(Gm_I - Gm_J) for I > J.  The scan's totals use the first two rows before the tables are written.
constexpr int gTab = gKc + kKcBytes, gBeta = gTab + kTabs * 512, gBars = gBeta + CH * 4, gItem = gBars + 32, gGl = gItem + 16;  // gGl: exp(G_last) [128]
constexpr int kGroupBytes = 114688;
static_assert(4 * kBox <= kKcBytes && gP + 32 * 32 * 4 <= gKc + kKcBytes && gTp + kTile <= gP && gGl + 512 <= kGroupBytes && kGroupBytes % 1024 == 0, "group map");
static_assert(kGroups * kGroupBytes <= oCtl, "two groups must fit below the block's control words");
constexpr uint32_t gcL = 0, gcM = 64, gcW = 0, gcU = 128, kGroupCols = 256;

// G = 0 or 1, a runtime value: both groups run the same instructions (one copy of this code in the instruction cache).
__device__ __forceinline__ void intra_group(const SpParams& p, unsigned char* smem, const uint32_t tm_block, const WaitCtx& ctx, const int G) {
    const int BAR = 2 + G;
    unsigned char* gs = smem + G * kGroupBytes;
    const uint32_t tm = tm_block + G * kGroupCols;
    uint64_t* bar_raw = reinterpret_cast<uint64_t*>(gs + gBars);
    uint64_t* bar_mma = bar_raw + 1;
    uint64_t* bar_lm = bar_raw + 2;  // the eight products of L^T and M^T: eight issuing threads arrive
    uint64_t* bar_free = bar_raw + 3;
    volatile int* item_slot = reinterpret_cast<volatile int*>(gs + gItem);
    float* betas = reinterpret_cast<float*>(gs + gBeta);
    const int gt = threadIdx.x - G * kGroupThreads, gw = gt >> 5, lane = gt & 31;
    const int quad = gw & 3, cg = gw >> 2;  // a warp reaches tensor-memory lanes 32 * (warp % 4)..; cg picks a half of the columns
    const int lane_row64 = quad * 16 + lane;
    const int H = p.H, chains = p.batch * H;
    auto group_sync = [&]() { named_bar_sync(BAR, kGroupThreads); };
    auto publish = [&]() {
        fence_proxy_async_smem();
        tc::fence_before_sync();
        group_sync();
        tc::fence_after_sync();
    };
    auto mma_issue = [&](uint64_t* bar, auto&& issue) {
        if (gt == 0) {
            issue();
            tc::mma_commit(bar);
            atomicAdd(const_cast<uint32_t*>(ctx.progress), 1u);
        }
    };
    uint32_t raw_phase = 0, mma_phase = 0, lm_phase = 0;
    auto mma_wait = [&](uint64_t* bar, uint32_t& phase) -> bool {
        if (!mbar_wait(bar, phase, ctx, kStatusWaitPrefill)) return false;
        phase ^= 1u;
        tc::fence_after_sync();
        return true;
    };

    for (;;) {
        if (!mbar_wait(bar_raw, raw_phase, ctx, kStatusWaitPrefill)) break;
        raw_phase ^= 1u;
        const int item = *item_slot;
        if (item < 0) break;
        const int chain = item % chains, jj = item / chains;
        unsigned char* slot = slot_of(p.ws_intra, p.seg_chunks, chain, jj);

        bool mild;
        // ---- 1. per key channel: the cumulative log decay; a = exp(G - Gm), every row relative to the middle row of its block of
        // 16, left in the staging boxes in place of g; then the per-block factor tables.  Thread (part, d): rows 32 part ..
        // 32 part + 31 of channel d, i.e. row blocks 2 part and 2 part + 1 (a needs nothing from the other half).
        {
            const int part = gt >> 7, d = gt & 127;
            // Row r of this thread's channel: box d / 32, piece (d % 32) / 4 swizzled by r & 7, float d % 4.
            unsigned char* col = gs + gG + (d >> 5) * kBox + part * 32 * 128 + (d & 3) * 4;
            const int pc = (d >> 2) & 7;
            float* tmp = reinterpret_cast<float*>(gs + gKb);  // totals [2][128], middles [4][128]: the Kgb tile is not in use yet
            float run[32], acc = 0.0f;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                acc += *reinterpret_cast<const float*>(col + r * 128 + ((pc ^ (r & 7)) << 4));
                run[r] = acc;
            }
            tmp[part * 128 + d] = acc;
            tmp[(2 + 2 * part) * 128 + d] = run[8];
            tmp[(3 + 2 * part) * 128 + d] = run[24];
            float amax = 0.0f;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const float av = __expf(run[r] - run[(r & 16) | 8]);
                amax = fmaxf(amax, av);
                *reinterpret_cast<float*>(col + r * 128 + ((pc ^ (r & 7)) << 4)) = av;
            }
            // Eight rows of decay must stay below e^85: per-row log decays below about -10.6 (or positive ones) do not.
            if (!(amax < 1e37f)) atomicCAS(p.status, 0, kStatusPrefillRange);
            group_sync();
            const float base1 = tmp[d];
            const float gm0 = tmp[2 * 128 + d], gm1 = tmp[3 * 128 + d], gm2 = base1 + tmp[4 * 128 + d], gm3 = base1 + tmp[5 * 128 + d];
            const float gl = base1 + tmp[128 + d];
            float* tab = reinterpret_cast<float*>(gs + gTab) + d;
            if (part == 0) {
                tab[(tE0 + 0) * 128] = __expf(gm0); tab[(tE0 + 1) * 128] = __expf(gm1); tab[(tE0 + 2) * 128] = __expf(gm2); tab[(tE0 + 3) * 128] = __expf(gm3);
                tab[(tEL + 0) * 128] = __expf(gl - gm0); tab[(tEL + 1) * 128] = __expf(gl - gm1);
                tab[(tEL + 2) * 128] = __expf(gl - gm2); tab[(tEL + 3) * 128] = __expf(gl - gm3);
            } else {
                tab[(tF + 0) * 128] = __expf(gm1 - gm0);
                tab[(tF + 1) * 128] = __expf(gm2 - gm0); tab[(tF + 2) * 128] = __expf(gm2 - gm1);
                tab[(tF + 3) * 128] = __expf(gm3 - gm0); tab[(tF + 4) * 128] = __expf(gm3 - gm1); tab[(tF + 5) * 128] = __expf(gm3 - gm2);
                const float egl = __expf(gl);
                reinterpret_cast<float*>(slot + wEgl)[d] = egl;
                reinterpret_cast<float*>(gs + gGl)[d] = egl;
            }
            mild = gl > -60.0f;
        }
        // A chunk whose whole decay stays above e^-60 in every channel needs no block-wise references: exp(G) and exp(-G) from
        // the chunk's start are both representable with room for small q and k, one column-side tile serves every row, and L^T,
        // M^T are one product each.  The group decides together (the barrier carries the vote); the choice depends on the chunk's
        // own gates only, so it is the same however the call is batched or cut into passes.
        const bool narrow = named_bar_all(BAR, kGroupThreads, mild);

        // ---- 2. a of this thread's row and 32 channels into registers -----------------------------------------------------------
        const int r = gt & 63, cq = gt >> 6, J = r >> 4;
        float a[32];
#pragma unroll
        for (int pp = 0; pp < 8; ++pp) {
            const float4 x = *reinterpret_cast<const float4*>(gs + gG + box_piece(r, cq * 8 + pp));
            a[pp * 4 + 0] = x.x; a[pp * 4 + 1] = x.y; a[pp * 4 + 2] = x.z; a[pp * 4 + 3] = x.w;
        }
        group_sync();  // nobody reads the staged a (or the scan's scratch) any more: the tiles may go over them

        // ---- 3. operand tiles, first those made from k.  Row side Kgb = K a; Kg = K exp(G) (over K) for W; Kdec =
        // K exp(G_last - G) as bf16 hi + lo out to the workspace; column sides K exp(Gm_I - G) into the tiles I >= J.
        const float* tabs = reinterpret_cast<const float*>(gs + gTab);
        if (narrow) {
            // One reference (the chunk's start): Kg = K exp(G) (over K) is the row side of L and the operand of W, Kinv = K exp(-G)
            // the one column-side tile (the 64-row tile), Kdec = Kinv exp(G_last).
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int c = cq * 4 + cc;
                const uint4 k8 = *reinterpret_cast<const uint4*>(gs + gK + box_piece(r, c));
                const float4 e0a = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8), e0b = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8 + 4);
                const float4 gla = *reinterpret_cast<const float4*>(gs + gGl + c * 32), glb = *reinterpret_cast<const float4*>(gs + gGl + c * 32 + 16);
                const float E0[8] = {e0a.x, e0a.y, e0a.z, e0a.w, e0b.x, e0b.y, e0b.z, e0b.w};
                const float GL[8] = {gla.x, gla.y, gla.z, gla.w, glb.x, glb.y, glb.z, glb.w};
                const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w};
                uint32_t kg[4], ki[4], dh[4], dl[4];
#pragma unroll
                for (int u2 = 0; u2 < 4; ++u2) {
                    const float kf[2] = {__uint_as_float(kw[u2] << 16), __uint_as_float(kw[u2] & 0xffff0000u)};
                    float v_kg[2], v_ki[2], hi[2], lo[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const float e = a[cc * 8 + 2 * u2 + u] * E0[2 * u2 + u], einv = __fdividef(1.0f, e);
                        v_kg[u] = kf[u] * e;
                        v_ki[u] = kf[u] * einv;
                        tc::split_bf16(kf[u] * (GL[2 * u2 + u] * einv), hi[u], lo[u]);
                    }
                    kg[u2] = tc::bf16x2(v_kg[0], v_kg[1]);
                    ki[u2] = tc::bf16x2(v_ki[0], v_ki[1]);
                    dh[u2] = tc::bf16x2(hi[0], hi[1]);
                    dl[u2] = tc::bf16x2(lo[0], lo[1]);
                }
                *reinterpret_cast<uint4*>(gs + gK + box_piece(r, c)) = make_uint4(kg[0], kg[1], kg[2], kg[3]);
                *reinterpret_cast<uint4*>(gs + gKc + kc_piece(3, r, c)) = make_uint4(ki[0], ki[1], ki[2], ki[3]);
                *reinterpret_cast<uint4*>(cell(slot + wKdHi, CH, c, r)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
                *reinterpret_cast<uint4*>(cell(slot + wKdLo, CH, c, r)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
            }
        } else {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const int c = cq * 4 + cc;
            const uint4 k8 = *reinterpret_cast<const uint4*>(gs + gK + box_piece(r, c));
            const float4 e0a = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8), e0b = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8 + 4);
            const float4 ela = *reinterpret_cast<const float4*>(tabs + (tEL + J) * 128 + c * 8), elb = *reinterpret_cast<const float4*>(tabs + (tEL + J) * 128 + c * 8 + 4);
            const float E0[8] = {e0a.x, e0a.y, e0a.z, e0a.w, e0b.x, e0b.y, e0b.z, e0b.w};
            const float EL[8] = {ela.x, ela.y, ela.z, ela.w, elb.x, elb.y, elb.z, elb.w};
            const uint32_t kw[4] = {k8.x, k8.y, k8.z, k8.w};
            uint32_t kg[4], kgb[4], kcd[4], dh[4], dl[4];
            float kc[8];  // K exp(Gm_J - G): the column side inside the row's own block
#pragma unroll
            for (int u2 = 0; u2 < 4; ++u2) {
                const float kf[2] = {__uint_as_float(kw[u2] << 16), __uint_as_float(kw[u2] & 0xffff0000u)};
                float v_kg[2], v_kgb[2], hi[2], lo[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float av = a[cc * 8 + 2 * u2 + u], inva = __fdividef(1.0f, av);
                    v_kgb[u] = kf[u] * av;
                    v_kg[u] = kf[u] * (av * E0[2 * u2 + u]);
                    kc[2 * u2 + u] = kf[u] * inva;
                    tc::split_bf16(kc[2 * u2 + u] * EL[2 * u2 + u], hi[u], lo[u]);
                }
                kg[u2] = tc::bf16x2(v_kg[0], v_kg[1]);
                kgb[u2] = tc::bf16x2(v_kgb[0], v_kgb[1]);
                kcd[u2] = tc::bf16x2(kc[2 * u2], kc[2 * u2 + 1]);
                dh[u2] = tc::bf16x2(hi[0], hi[1]);
                dl[u2] = tc::bf16x2(lo[0], lo[1]);
            }
            *reinterpret_cast<uint4*>(gs + gK + box_piece(r, c)) = make_uint4(kg[0], kg[1], kg[2], kg[3]);
            *reinterpret_cast<uint4*>(gs + gKb + box_piece(r, c)) = make_uint4(kgb[0], kgb[1], kgb[2], kgb[3]);
            *reinterpret_cast<uint4*>(cell(slot + wKdHi, CH, c, r)) = make_uint4(dh[0], dh[1], dh[2], dh[3]);
            *reinterpret_cast<uint4*>(cell(slot + wKdLo, CH, c, r)) = make_uint4(dl[0], dl[1], dl[2], dl[3]);
            *reinterpret_cast<uint4*>(gs + gKc + kc_piece(J, r, c)) = make_uint4(kcd[0], kcd[1], kcd[2], kcd[3]);
            for (int I = J + 1; I < 4; ++I) {  // the later row blocks see this row through exp(Gm_I - Gm_J) <= 1
                const float* f = tabs + (tF + I * (I - 1) / 2 + J) * 128 + c * 8;
                const float4 fa = *reinterpret_cast<const float4*>(f), fb = *reinterpret_cast<const float4*>(f + 4);
                *reinterpret_cast<uint4*>(gs + gKc + kc_piece(I, r, c)) =
                    make_uint4(tc::bf16x2(kc[0] * fa.x, kc[1] * fa.y), tc::bf16x2(kc[2] * fa.z, kc[3] * fa.w),
                               tc::bf16x2(kc[4] * fb.x, kc[5] * fb.y), tc::bf16x2(kc[6] * fb.z, kc[7] * fb.w));
            }
        }
        }
        publish();
        // ---- 3a. L^T, one block column of 16 rows i a warp: [64 j x 16 i] = column side (tile I) x row side (block I)^T.  Eight
        // threads (lane 0 of every warp) issue the eight small products of L^T and M^T, so none of them issues for long; each
        // commits to the same barrier, which completes when all eight have.
        if (lane == 0 && gw < 4) {
            if (narrow) {  // one product, all 64 rows i at once, row side Kg (a commit with nothing pending arrives at once)
                constexpr uint32_t id64 = tc::idesc_bf16(64, 64, 0, 0, 0);
                if (gw == 0)
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + gcL, tc::desc_sw128_kmajor(gs + gKc + kc_tile(3), CH, k0), tc::desc_sw128_kmajor(gs + gK, CH, k0), id64, k0 > 0);
            } else {
            constexpr uint32_t id = tc::idesc_bf16(64, 16, 0, 0, 0);
            const int I = gw;
            const unsigned char* kct = gs + gKc + kc_tile(I);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + gcL + 16 * I, tc::desc_sw128_kmajor(kct, 16 * (I + 1), k0), tc::desc_sw128_kmajor(gs + gKb + I * 2048, CH, k0), id, k0 > 0);
            }
            tc::mma_commit(bar_lm);
            atomicAdd(const_cast<uint32_t*>(ctx.progress), 1u);
        }
        // ---- 3b. the tiles made from q, while L^T runs: row side Qgb = Q a (over Q); Qg = Q exp(G) out to the workspace -------
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const int c = cq * 4 + cc;
            const uint4 q8 = *reinterpret_cast<const uint4*>(gs + gQ + box_piece(r, c));
            const float4 e0a = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8), e0b = *reinterpret_cast<const float4*>(tabs + (tE0 + J) * 128 + c * 8 + 4);
            const float E0[8] = {e0a.x, e0a.y, e0a.z, e0a.w, e0b.x, e0b.y, e0b.z, e0b.w};
            const uint32_t qw[4] = {q8.x, q8.y, q8.z, q8.w};
            uint32_t qg[4], qgb[4];
#pragma unroll
            for (int u2 = 0; u2 < 4; ++u2) {
                const float q0 = __uint_as_float(qw[u2] << 16), q1 = __uint_as_float(qw[u2] & 0xffff0000u);
                const float a0 = a[cc * 8 + 2 * u2], a1 = a[cc * 8 + 2 * u2 + 1];
                qgb[u2] = tc::bf16x2(q0 * a0, q1 * a1);
                qg[u2] = tc::bf16x2(q0 * (a0 * E0[2 * u2]), q1 * (a1 * E0[2 * u2 + 1]));
            }
            // narrow: Qg itself is M's row side
            *reinterpret_cast<uint4*>(gs + gQ + box_piece(r, c)) = narrow ? make_uint4(qg[0], qg[1], qg[2], qg[3]) : make_uint4(qgb[0], qgb[1], qgb[2], qgb[3]);
            *reinterpret_cast<uint4*>(cell(slot + wQg, CH, c, r)) = make_uint4(qg[0], qg[1], qg[2], qg[3]);
        }
        publish();
        // ---- 3c. M^T the same way, by the other four warps ------------------------------------------------------------------------
        if (lane == 0 && gw >= 4) {
            if (narrow) {
                constexpr uint32_t id64 = tc::idesc_bf16(64, 64, 0, 0, 0);
                if (gw == 4)
                    for (int k0 = 0; k0 < DK; k0 += 16)
                        tc::mma_bf16(tm + gcM, tc::desc_sw128_kmajor(gs + gKc + kc_tile(3), CH, k0), tc::desc_sw128_kmajor(gs + gQ, CH, k0), id64, k0 > 0);
            } else {
            constexpr uint32_t id = tc::idesc_bf16(64, 16, 0, 0, 0);
            const int I = gw - 4;
            const unsigned char* kct = gs + gKc + kc_tile(I);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + gcM + 16 * I, tc::desc_sw128_kmajor(kct, 16 * (I + 1), k0), tc::desc_sw128_kmajor(gs + gQ + I * 2048, CH, k0), id, k0 > 0);
            }
            tc::mma_commit(bar_lm);
            atomicAdd(const_cast<uint32_t*>(ctx.progress), 1u);
        }
        if (!mma_wait(bar_lm, lm_phase)) break;

        // ---- 4. from L^T and M^T (lane = column j, tensor-memory column = row i): L (FP32, strictly lower, times beta_i) into
        // the scratch; M (lower with the diagonal) out as bf16 cells of eight consecutive rows i, [8 cells][64 columns j] ----------
        {
            const int j = lane_row64;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t rr[32];
                tc::tmem_ld32(tc::tmem_addr(tm, quad, (cg == 0 ? gcL : gcM) + half * 32), rr);
                tc::tmem_ld_wait();
                if (lane < 16) {
                    if (cg == 0) {  // L stays transposed: this thread's column j, 32 consecutive rows i
                        float* Lt = reinterpret_cast<float*>(gs + gL) + j * LS + half * 32;
#pragma unroll
                        for (int i4 = 0; i4 < 8; ++i4) {
                            const float4 b4 = *reinterpret_cast<const float4*>(betas + half * 32 + i4 * 4);
                            const int i = half * 32 + i4 * 4;
                            *reinterpret_cast<float4*>(Lt + i4 * 4) = make_float4(i > j ? b4.x * __uint_as_float(rr[i4 * 4]) : 0.0f, i + 1 > j ? b4.y * __uint_as_float(rr[i4 * 4 + 1]) : 0.0f,
                                                                                  i + 2 > j ? b4.z * __uint_as_float(rr[i4 * 4 + 2]) : 0.0f, i + 3 > j ? b4.w * __uint_as_float(rr[i4 * 4 + 3]) : 0.0f);
                        }
                    } else {
#pragma unroll
                        for (int i2 = 0; i2 < 32; ++i2)
                            if (half * 32 + i2 < j) rr[i2] = 0u;
#pragma unroll
                        for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(cell(slot + wMm, CH, half * 4 + cc, j)) = pack8(rr + cc * 8);
                    }
                }
            }
        }
        tc::fence_before_sync();
        group_sync();

        // ---- 5. T = (I + L)^-1 in FP32, T' = T diag(beta) as bf16 hi + lo cells (over L, dead by then) -----------------------
        {
            const float* Lm = reinterpret_cast<const float*>(gs + gL);
            float* Tm = reinterpret_cast<float*>(gs + gT);
            float* Pm = reinterpret_cast<float*>(gs + gP);
            invert_diag16<kGroupThreads>(Lm, Tm, gt, BAR);
            invert_level<4, kGroupThreads>(Lm, Tm, Pm, gt, BAR);
            invert_level<5, kGroupThreads>(Lm, Tm, Pm, gt, BAR);
            const int i = gt & 63, cq = gt >> 6;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                const int c = cq + cc * 4;
                uint32_t wh[4], wl[4];
#pragma unroll
                for (int j2 = 0; j2 < 4; ++j2) {
                    float h0, l0, h1, l1;
                    tc::split_bf16(Tm[i * LS + c * 8 + 2 * j2] * betas[c * 8 + 2 * j2], h0, l0);
                    tc::split_bf16(Tm[i * LS + c * 8 + 2 * j2 + 1] * betas[c * 8 + 2 * j2 + 1], h1, l1);
                    wh[j2] = tc::bf16x2(h0, h1);
                    wl[j2] = tc::bf16x2(l0, l1);
                }
                *reinterpret_cast<uint4*>(gs + gTp + box_piece(i, c)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                *reinterpret_cast<uint4*>(gs + gTp + kBox + box_piece(i, c)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
            }
        }
        publish();

        // ---- 6. W = T' Kg (bf16 T'), U = T' V (T' hi + lo) -------------------------------------------------------------------
        mma_issue(bar_mma, [&] {
            constexpr uint32_t id = tc::idesc_bf16(64, 128, 0, 1, 0);
            const unsigned char* tph = gs + gTp;
            const unsigned char* tpl = gs + gTp + kBox;
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + gcW, tc::desc_sw128_kmajor(tph, CH, k0), tc::desc_sw128_mnmajor(gs + gK, CH, k0), id, k0 > 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + gcU, tc::desc_sw128_kmajor(tph, CH, k0), tc::desc_sw128_mnmajor(gs + gV, CH, k0), id, k0 > 0);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + gcU, tc::desc_sw128_kmajor(tpl, CH, k0), tc::desc_sw128_mnmajor(gs + gV, CH, k0), id, true);
        });
        if (!mma_wait(bar_mma, mma_phase)) break;
        // Nothing of this item is left in the group's shared memory: the loader may bring the next item in.
        if (gt == 0) mbar_arrive(bar_free);

        // ---- 7. W as bf16 cells and U as FP32 rows, from tensor memory to the workspace ---------------------------------------
        {
            const int i = lane_row64;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                uint32_t r[32];
                const int col = cg * 64 + half * 32;
                tc::tmem_ld32(tc::tmem_addr(tm, quad, gcW + col), r);
                tc::tmem_ld_wait();
                if (lane < 16) {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) *reinterpret_cast<uint4*>(cell(slot + wW, CH, col / 8 + cc, i)) = pack8(r + cc * 8);
                }
                tc::tmem_ld32(tc::tmem_addr(tm, quad, gcU + col), r);
                tc::tmem_ld_wait();
                if (lane < 16) {
#pragma unroll
                    for (int j2 = 0; j2 < 8; ++j2)
                        *reinterpret_cast<uint4*>(cell(slot + wU, CH, col / 4 + j2, i)) = make_uint4(r[j2 * 4], r[j2 * 4 + 1], r[j2 * 4 + 2], r[j2 * 4 + 3]);
                }
            }
        }
        tc::fence_before_sync();
        group_sync();
        tc::fence_after_sync();
    }
}

// The loader warp of group G: takes items off the counter and brings each one's rows into the group's staging.  A full
// chunk arrives by ten tiled tensor copies issued by one lane; a sequence's last, partial chunk is copied by the
// warp's own loads and stores (rows past the sequence's end are not read, they become zero), so no copy ever reaches
// past the rows the caller's metadata names.
__device__ __forceinline__ void intra_loader(const SpParams& p, unsigned char* smem, const WaitCtx& ctx, const int G) {
    unsigned char* gs = smem + G * kGroupBytes;
    uint64_t* bar_raw = reinterpret_cast<uint64_t*>(gs + gBars);
    uint64_t* bar_free = bar_raw + 3;
    volatile int* item_slot = reinterpret_cast<volatile int*>(gs + gItem);
    float* betas = reinterpret_cast<float*>(gs + gBeta);
    const int lane = threadIdx.x & 31;
    const int H = p.H, chains = p.batch * H;
    const long long items = (long long)chains * p.seg_chunks;  // item = jj * chains + chain: chunk-major
    uint32_t free_phase = 0;
    for (int it = 0;;) {
        long long item = 0;
        if (lane == 0) item = atomicAdd(&p.counters[p.ctr], 1u);
        item = __shfl_sync(0xffffffffu, item, 0);
        const bool last = item >= items;
        int h = 0, n = 0;
        long long gr0 = 0;
        if (!last) {
            const int chain = (int)(item % chains), j = p.intra_chunk0 + (int)(item / chains);
            const int b = chain / H;
            h = chain % H;
            const int r0 = p.cu[b], T = p.cu[b + 1] - r0;
            if ((long long)j * CH >= T) continue;  // the sequence has no such chunk
            gr0 = (long long)r0 + (long long)j * CH;
            n = min(CH, T - j * CH);
        }
        float b0 = 0.0f, b1 = 0.0f;
        if (lane < n) b0 = p.beta[(gr0 + lane) * H + h];
        if (lane + 32 < n) b1 = p.beta[(gr0 + lane + 32) * H + h];
        if (it > 0) {
            if (!mbar_wait(bar_free, free_phase, ctx, kStatusWaitPrefill)) break;
            free_phase ^= 1u;
        }
        ++it;
        if (last) {  // tell the compute warps that there is nothing more
            if (lane == 0) {
                *item_slot = -1;
                mbar_arrive(bar_raw);
            }
            break;
        }
        betas[lane] = b0;
        betas[lane + 32] = b1;
        if (lane == 0) *item_slot = (int)item;
        if (n == CH) {
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_expect_tx(bar_raw, 3u * kTile + 4u * kBox);
                const int row = (int)gr0;
                for (int x = 0; x < 4; ++x) tensor_load_3d(gs + gG + x * kBox, &p.tm_g, x * 32, h, row, bar_raw);
                for (int x = 0; x < 2; ++x) tensor_load_3d(gs + gK + x * kBox, &p.tm_k, x * 64, h, row, bar_raw);
                for (int x = 0; x < 2; ++x) tensor_load_3d(gs + gQ + x * kBox, &p.tm_q, x * 64, h, row, bar_raw);
                for (int x = 0; x < 2; ++x) tensor_load_3d(gs + gV + x * kBox, &p.tm_v, x * 64, h, row, bar_raw);
            }
        } else {
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int e = lane; e < CH * 16; e += 32) {
                const int r = e >> 4, c = e & 15;
                const long long at = ((gr0 + r) * H + h) * DK + c * 8;
                const bool in = r < n;
                *reinterpret_cast<uint4*>(gs + gQ + box_piece(r, c)) = in ? *reinterpret_cast<const uint4*>(p.q + at) : z;
                *reinterpret_cast<uint4*>(gs + gK + box_piece(r, c)) = in ? *reinterpret_cast<const uint4*>(p.k + at) : z;
                *reinterpret_cast<uint4*>(gs + gV + box_piece(r, c)) = in ? *reinterpret_cast<const uint4*>(p.v + at) : z;
            }
            for (int e = lane; e < CH * 32; e += 32) {
                const int r = e >> 5, piece = e & 31;
                const long long at = ((gr0 + r) * H + h) * DK + piece * 4;
                *reinterpret_cast<uint4*>(gs + gG + box_piece(r, piece)) = r < n ? *reinterpret_cast<const uint4*>(p.g + at) : z;
            }
            fence_proxy_async_smem();  // V is read by the tensor core as it stands
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_raw);
        }
    }
}

__device__ void intra_role(const SpParams& p, unsigned char* smem, const uint32_t tm) {
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oCtl);
    const WaitCtx ctx{ctl, ctl + 1, p.status};
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        for (int g = 0; g < kGroups; ++g) {
            uint64_t* b = reinterpret_cast<uint64_t*>(smem + g * kGroupBytes + gBars);
            for (int i = 0; i < 4; ++i) mbar_init(b + i, i == 2 ? 8 : 1);  // raw, mma, L^T/M^T (eight issuers), free
        }
        mbar_init_fence();
    }
    __syncthreads();
    if (warp == kLoaderWarp || warp == kOutWarp) intra_loader(p, smem, ctx, warp == kLoaderWarp ? 0 : 1);
    else intra_group(p, smem, tm, ctx, warp < kGroupThreads / 32 ? 0 : 1);
    tc::fence_before_sync();
    __syncthreads();
}

// =====================================================================================================================
// Pass 2: the state recurrence of one chain over the segment's chunks, from the workspace.
// =====================================================================================================================
// Shared memory mirrors a workspace slot (three groups, each with its own full/empty barrier pair, refilled by the
// loader warp as soon as the tensor core has consumed them), then S as bf16 cells and D hi/lo.
constexpr int sSlot = 0, sS16 = (kSlotBytes + 1023) / 1024 * 1024, sDhi = sS16 + 2 * kTile, sDlo = sDhi + kTile, sRed = sDlo + kTile;
// Finished output rows (bf16) wait in one of two tiles for the output warp: two boxes of 64 rows x 128 bytes each (value
// channels 0-63, 64-127) in the 128-byte swizzle of box_piece(), which is what the tiled tensor stores read.
constexpr int sOut = sRed + 4 * CH * 4, kOutTile = 2 * kBox;
static_assert(sOut % 1024 == 0 && sOut + 2 * kOutTile <= oBars, "state role shared memory");
constexpr uint32_t tS = 0, tQS = 128, tD = 256, tQS1 = 384;  // QS/O accumulators alternate between chunks

// NV = the value channels this block owns (all 128, or 64: a chain's value columns never interact, so two blocks can
// share a chain when chains are few and the serial walk over the chunks is what takes the time); value channels
// [vpart * NV, vpart * NV + NV).  A warp then covers C = NV / 4 accumulator columns.
// What one walk of the state role covers: chunks [ja, jb) of its chain, where the state comes from and goes to, whether
// U takes part (not in the walk that yields a segment's transition) and whether outputs are produced.
struct Walk {
    int ja, jb;
    int init;          // 0: the state buffer (state_in for the first chunk of a sequence, else state_out); 1: zero; 2: identity; 3: FP32 `from`
    const float* from;
    int fin;           // where the end state goes: 0 state_out, 1 the FP32 buffer `to`, 2 nowhere
    float* to;
    bool use_u, emit;
};

template <int NV>
__device__ void state_role(const SpParams& p, unsigned char* smem, const uint32_t tm, const int chain, const int vpart, const Walk wk) {
    constexpr int C = NV / 4, CELLS = C / 8;
    const int v0 = vpart * NV;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + oBarsState);  // [3]
    uint64_t* empty = full + 3;                                       // [3]
    uint64_t* bar_mma = full + 6;
    uint64_t* out_full = full + 7;   // [2]
    uint64_t* out_empty = full + 9;  // [2]
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oCtl);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, cg = warp >> 2;
    const int lane_row128 = quad * 32 + lane, lane_row64 = quad * 16 + lane;
    const int H = p.H, b = chain / H, h = chain % H;
    const long long row0 = p.cu[b];
    const int T = p.cu[b + 1] - p.cu[b];
    const int nch = (T + CH - 1) / CH;
    const int j0 = min(wk.ja, nch), j1 = min(nch, wk.jb);
    const long long s_elem = p.state_off[b] + (long long)h * DV * DK;
    // A chain with no chunk in this range: only the first segment has anything to do (an empty sequence copies its state);
    // a scan walk always delivers its end state.
    if (p.scan_pass == 0 && j0 >= j1 && !(j0 == 0 && p.state_out != p.state_in)) return;
    const WaitCtx ctx{ctl, ctl + 1, p.status};

    if (warp == kOutWarp && !wk.emit) {
        tc::fence_before_sync();
        __syncthreads();
        return;
    }
    if (warp == kOutWarp) {
        // The output warp: each finished tile of rows goes to the shard-local `out` and, for a head-sharded launch, into
        // every rank's full buffer -- the all-gather, done here: a peer's buffer is reached over NVLink.  A full chunk
        // leaves by tiled tensor stores (two per destination), off the compute warps' path; a sequence's last, partial
        // chunk by the warp's own stores, so that no row beyond the sequence is touched.
        for (int j = j0; j < j1; ++j) {
            const int c = j - j0, n = min(CH, T - j * CH);
            const long long gr0 = row0 + (long long)j * CH;
            if (!mbar_wait(&out_full[c & 1], (uint32_t)((c >> 1) & 1), ctx, kStatusWaitPrefill)) break;
            const unsigned char* tile = smem + sOut + (c & 1) * kOutTile;
            if (n == CH) {
                if (lane == 0) {
                    for (int x = 0; x < NV / 64; ++x) {
                        if (p.out != nullptr) tensor_store_3d(&p.tm_out, v0 + x * 64, h, (int)gr0, tile + x * kBox);
                        for (int pe = 0; pe < p.ranks; ++pe) tensor_store_3d(&p.tm_full[pe], v0 + x * 64, p.head0 + h, (int)gr0, tile + x * kBox);
                    }
                    bulk_commit();
                    bulk_wait_read<0>();  // the tile has been read: the compute warps may refill it
                }
            } else {
                for (int e = lane; e < n * (NV / 8); e += 32) {
                    const int r = e / (NV / 8), piece = e % (NV / 8);
                    const uint4 v4 = *reinterpret_cast<const uint4*>(tile + box_piece(r, piece));
                    if (p.out != nullptr) *reinterpret_cast<uint4*>(p.out + ((gr0 + r) * H + h) * DV + v0 + piece * 8) = v4;
                    const long long at_full = ((gr0 + r) * p.heads_total + p.head0 + h) * DV + v0 + piece * 8;
                    for (int pe = 0; pe < p.ranks; ++pe) *reinterpret_cast<uint4*>(p.full[pe] + at_full) = v4;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&out_empty[c & 1]);
        }
        if (lane == 0) bulk_wait_all<0>();
        tc::fence_before_sync();
        __syncthreads();
        return;
    }
    if (warp == kLoaderWarp) {
        if (lane == 0) {
            uint32_t ph = 1;  // the empty barriers start released
            for (int j = j0; j < j1; ++j) {
                const unsigned char* slot = slot_of(p.ws_state, p.seg_chunks, chain, j - p.state_chunk0);
                if (!mbar_wait(&empty[0], ph, ctx, kStatusWaitPrefill)) break;
                mbar_arrive_expect_tx(&full[0], 2 * kTile + 512);
                bulk_load(smem + sSlot + wQg, slot + wQg, 2 * kTile, &full[0]);
                bulk_load(smem + sSlot + wEgl, slot + wEgl, 512, &full[0]);
                if (!mbar_wait(&empty[1], ph, ctx, kStatusWaitPrefill)) break;
                mbar_arrive_expect_tx(&full[1], NV * CH * 4);
                bulk_load(smem + sSlot + wU, slot + wU + (size_t)(v0 / 4) * CH * 16, NV * CH * 4, &full[1]);
                if (!mbar_wait(&empty[2], ph, ctx, kStatusWaitPrefill)) break;
                mbar_arrive_expect_tx(&full[2], kTile / 2 + 2 * kTile);
                bulk_load(smem + sSlot + wMm, slot + wMm, kTile / 2 + 2 * kTile, &full[2]);
                ph ^= 1u;
            }
        }
        tc::fence_before_sync();
        __syncthreads();
        return;
    }

    uint32_t mma_phase = 0;
    bool alive = true;
    auto mma_issue = [&](auto&& issue) {
        if (tid == 0) {
            issue();
            tc::mma_commit(bar_mma);
            atomicAdd(const_cast<uint32_t*>(ctl), 1u);
        }
    };
    auto mma_wait = [&]() -> bool {
        if (!mbar_wait(bar_mma, mma_phase, ctx, kStatusWaitPrefill)) return false;
        mma_phase ^= 1u;
        tc::fence_after_sync();
        return true;
    };
    auto publish_operands = [&]() {
        fence_proxy_async_smem();
        tc::fence_before_sync();
        compute_sync();
        tc::fence_after_sync();
    };
    // S as bf16 cells for chunk c's products, the decayed S back to tensor memory, then QS = Qg S and -W S are started
    // (not waited for) into the chunk's accumulators.
    auto begin_chunk = [&](int c) -> bool {
        if (!mbar_wait(&full[0], (uint32_t)(c & 1), ctx, kStatusWaitPrefill)) return false;
        const float* egl = reinterpret_cast<const float*>(smem + sSlot + wEgl);
        {
            uint32_t r[C];
            tc::tmem_ld<C>(tc::tmem_addr(tm, quad, tS + cg * C), r);
            tc::tmem_ld_wait();
            if (p.state_bf16) {
#pragma unroll
                for (int jj = 0; jj < C; ++jj) r[jj] = __float_as_uint(bf16_round(__uint_as_float(r[jj])));
            }
#pragma unroll
            for (int cc = 0; cc < CELLS; ++cc) *reinterpret_cast<uint4*>(cell(smem + sS16, 128, cg * CELLS + cc, lane_row128)) = pack8(r + cc * 8);
            const float el = egl[lane_row128];
#pragma unroll
            for (int jj = 0; jj < C; ++jj) r[jj] = __float_as_uint(__uint_as_float(r[jj]) * el);
            tc::tmem_st<C>(tc::tmem_addr(tm, quad, tS + cg * C), r);
            tc::tmem_st_wait();
        }
        publish_operands();
        const uint32_t tO = (c & 1) ? tQS1 : tQS;
        mma_issue([&] {
            constexpr uint32_t id = tc::idesc_bf16(64, NV, 0, 1, 0), idn = tc::idesc_bf16(64, NV, 0, 1, 1);
            if (wk.emit)
                for (int k0 = 0; k0 < DK; k0 += 16)
                    tc::mma_bf16(tm + tO, tc::desc_kmajor_bf16(smem + sSlot + wQg, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sS16, 128, 0, k0), id, k0 > 0);
            for (int k0 = 0; k0 < DK; k0 += 16)
                tc::mma_bf16(tm + tD, tc::desc_kmajor_bf16(smem + sSlot + wW, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sS16, 128, 0, k0), idn, k0 > 0);
        });
        return true;
    };

    // ---- the incoming state into tensor memory: lane = key channel, columns = value channel -----------------------
    {
        const void* src = j0 == 0 ? p.state_in : p.state_out;
        uint32_t r[C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int vch = v0 + cg * C + j;
            const long long at = s_elem + (long long)vch * DK + lane_row128;
            float x;
            if (wk.init == 1) x = 0.0f;
            else if (wk.init == 2) x = vch == lane_row128 ? 1.0f : 0.0f;
            else if (wk.init == 3) x = wk.from[vch * DK + lane_row128];
            else x = p.state_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(src)[at]) : reinterpret_cast<const float*>(src)[at];
            r[j] = __float_as_uint(x);
        }
        tc::tmem_st<C>(tc::tmem_addr(tm, quad, tS + cg * C), r);
        tc::tmem_st_wait();
    }
    tc::fence_before_sync();
    compute_sync();
    tc::fence_after_sync();
    if (j0 < j1 && !begin_chunk(0)) alive = false;

    for (int j = j0; alive && j < j1; ++j) {
        const int c = j - j0, n = min(CH, T - j * CH);
        const uint32_t par = (uint32_t)(c & 1), tO = (c & 1) ? tQS1 : tQS;
        const long long gr0 = row0 + (long long)j * CH;
        if (!mma_wait()) { alive = false; break; }
        if (tid == 0) mbar_arrive(&empty[0]);  // Qg, W and exp(G_last) are consumed (begin_chunk read E_last before the products)

        // ---- D = U - W S as bf16 hi + lo cells ---------------------------------------------------------------------------
        if (!mbar_wait(&full[1], par, ctx, kStatusWaitPrefill)) { alive = false; break; }
        {
            uint32_t r[C];
            tc::tmem_ld<C>(tc::tmem_addr(tm, quad, tD + cg * C), r);
            tc::tmem_ld_wait();
            if (lane < 16) {
                unsigned char* Ut = smem + sSlot + wU;  // this block's slice of U: NV / 4 cells of four value channels
#pragma unroll
                for (int cc = 0; cc < CELLS; ++cc) {
                    const float4 u0 = *reinterpret_cast<const float4*>(cell(Ut, CH, cg * (C / 4) + cc * 2, lane_row64));
                    const float4 u1 = *reinterpret_cast<const float4*>(cell(Ut, CH, cg * (C / 4) + cc * 2 + 1, lane_row64));
                    const float uu[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
                    uint32_t wh[4], wl[4];
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        float h0, l0, h1, l1;
                        tc::split_bf16((wk.use_u ? uu[2 * jj] : 0.0f) + __uint_as_float(r[cc * 8 + 2 * jj]), h0, l0);
                        tc::split_bf16((wk.use_u ? uu[2 * jj + 1] : 0.0f) + __uint_as_float(r[cc * 8 + 2 * jj + 1]), h1, l1);
                        wh[jj] = tc::bf16x2(h0, h1);
                        wl[jj] = tc::bf16x2(l0, l1);
                    }
                    *reinterpret_cast<uint4*>(cell(smem + sDhi, CH, cg * CELLS + cc, lane_row64)) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
                    *reinterpret_cast<uint4*>(cell(smem + sDlo, CH, cg * CELLS + cc, lane_row64)) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
                }
            }
        }
        publish_operands();
        if (tid == 0) mbar_arrive(&empty[1]);

        // ---- O = QS + M D;  S += Kdec^T D (hi hi + hi lo + lo hi) ------------------------------------------------------------
        if (!mbar_wait(&full[2], par, ctx, kStatusWaitPrefill)) { alive = false; break; }
        mma_issue([&] {
            constexpr uint32_t idm = tc::idesc_bf16(64, NV, 1, 1, 0), ids = tc::idesc_bf16(128, NV, 1, 1, 0);  // M arrives with its rows contiguous
            const unsigned char* kdhi = smem + sSlot + wKdHi;
            const unsigned char* kdlo = smem + sSlot + wKdLo;
            if (wk.emit)
                for (int k0 = 0; k0 < CH; k0 += 16)
                    tc::mma_bf16(tm + tO, tc::desc_mnmajor_bf16(smem + sSlot + wMm, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sDhi, CH, 0, k0), idm, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + tS, tc::desc_mnmajor_bf16(kdhi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sDhi, CH, 0, k0), ids, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + tS, tc::desc_mnmajor_bf16(kdhi, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sDlo, CH, 0, k0), ids, true);
            for (int k0 = 0; k0 < CH; k0 += 16)
                tc::mma_bf16(tm + tS, tc::desc_mnmajor_bf16(kdlo, CH, 0, k0), tc::desc_mnmajor_bf16(smem + sDhi, CH, 0, k0), ids, true);
        });
        if (!mma_wait()) { alive = false; break; }
        if (tid == 0) mbar_arrive(&empty[2]);

        // The next chunk's first products run on the tensor core while this chunk's outputs leave.
        if (j + 1 < j1 && !begin_chunk(c + 1)) { alive = false; break; }

        // ---- outputs: bf16(y), or the gated RMSNorm of bf16(y) ------------------------------------------------------------------
        if (wk.emit) {
            uint32_t r[C];
            tc::tmem_ld<C>(tc::tmem_addr(tm, quad, tO + cg * C), r);
            tc::tmem_ld_wait();
            const int i = lane_row64;
            const bool live = lane < 16 && i < n;
            const long long at = ((gr0 + i) * H + h) * DV + v0 + cg * C;
            float y[C];
#pragma unroll
            for (int jj = 0; jj < C; ++jj) y[jj] = bf16_round(__uint_as_float(r[jj]));
            if (NV == DV && p.gate != nullptr) {  // the norm needs a row's every value channel: whole-head blocks only
                float* red = reinterpret_cast<float*>(smem + sRed);
                float ss = 0.0f;
#pragma unroll
                for (int jj = 0; jj < C; ++jj) ss = fmaf(y[jj], y[jj], ss);
                if (lane < 16) red[cg * CH + i] = ss;
                compute_sync();
                if (live) {
                    const float tot = (red[i] + red[CH + i]) + (red[2 * CH + i] + red[3 * CH + i]);
                    const float rinv = 1.0f / sqrtf(tot / (float)DV + p.eps);
#pragma unroll
                    for (int jj = 0; jj < C; ++jj) {
                        const float gt = bf16_bits_to_f32(p.gate[at + jj]), w = bf16_bits_to_f32(p.norm_w[cg * C + jj]);
                        y[jj] = w * (y[jj] * rinv) * (1.0f / (1.0f + __expf(-gt)));
                    }
                }
                compute_sync();  // the partial sums are read before the next chunk's are written
            }
            // Into the output tile (the output warp takes it from there).
            if (!mbar_wait(&out_empty[c & 1], (uint32_t)(((c >> 1) & 1) ^ 1), ctx, kStatusWaitPrefill)) { alive = false; break; }
            if (lane < 16) {
                unsigned char* dst = smem + sOut + (c & 1) * kOutTile;
#pragma unroll
                for (int c4 = 0; c4 < CELLS; ++c4)
                    *reinterpret_cast<uint4*>(dst + box_piece(i, cg * CELLS + c4)) = make_uint4(tc::bf16x2(y[c4 * 8], y[c4 * 8 + 1]), tc::bf16x2(y[c4 * 8 + 2], y[c4 * 8 + 3]),
                                                                          tc::bf16x2(y[c4 * 8 + 4], y[c4 * 8 + 5]), tc::bf16x2(y[c4 * 8 + 6], y[c4 * 8 + 7]));
            }
            fence_proxy_async_smem();  // the tensor stores read the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&out_full[c & 1]);
        }
    }

    // ---- the outgoing state ---------------------------------------------------------------------------------------------
    if (alive) {
        uint32_t r[C];
        tc::tmem_ld<C>(tc::tmem_addr(tm, quad, tS + cg * C), r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const long long at = s_elem + (long long)(v0 + cg * C + j) * DK + lane_row128;
            if (wk.fin == 2) continue;
            if (wk.fin == 1) wk.to[(v0 + cg * C + j) * DK + lane_row128] = __uint_as_float(r[j]);
            else if (p.state_bf16) reinterpret_cast<uint16_t*>(p.state_out)[at] = f32_to_bf16_bits(__uint_as_float(r[j]));
            else reinterpret_cast<float*>(p.state_out)[at] = __uint_as_float(r[j]);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
}

// One launch: the state role of one segment on the chain blocks, then the intra role of the next segment on all blocks.
__global__ void __launch_bounds__(kThreadsSp, 1) prefill_sp_kernel(const __grid_constant__ SpParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        uint64_t* bs = reinterpret_cast<uint64_t*>(smem + oBarsState);
        for (int i = 0; i < 7; ++i) mbar_init(bs + i, 1);  // state role: full[3], empty[3], mma
        for (int i = 0; i < 2; ++i) mbar_init(bs + 7 + i, kCompute / 32);  // output tile full: one arrival per compute warp
        for (int i = 0; i < 2; ++i) mbar_init(bs + 9 + i, 1);               // output tile empty
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
        // the next launch's counter; nobody reads it during this launch.  (A scan pass leaves the counters alone: it may run
        // beside the next super-block's intra launch on another stream.)
        if (blockIdx.x == 0 && p.scan_pass == 0) p.counters[p.ctr ^ 1] = 0u;
    }
    if (warp == 0) tc::tmem_alloc(tmem_slot, kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const int chains = p.batch * p.H;
    if (p.scan_pass == 1) {  // (chain, segment s < scan_p1, kind): the segment's offset and transition
        const int kind = blockIdx.x & 1, sg = (blockIdx.x >> 1) % p.scan_p1, chain = (blockIdx.x >> 1) / p.scan_p1;
        if (chain < chains) {
            const int hi = p.state_chunk0 + p.seg_chunks;  // the launch's chunk range ends here
            const bool last = sg == p.scan_k - 1;
            const int end = last ? (p.scan_open ? 0x7fffffff : hi) : min(p.state_chunk0 + (sg + 1) * p.scan_chunks, hi);
            const Walk wk{min(p.state_chunk0 + sg * p.scan_chunks, hi), end, kind ? 2 : 1, nullptr, 1,
                          p.scan_ab + (((size_t)chain * p.scan_p1 + sg) * 2 + kind) * DV * DK, kind == 0, false};
            state_role<DV>(p, smem, tm, chain, 0, wk);
        }
    } else if (p.scan_pass == 2) {  // (chain, segment): the walk with outputs from the segment's true incoming state
        const int sg = blockIdx.x % p.scan_k, chain = blockIdx.x / p.scan_k;
        if (chain < chains) {
            // Only the last segment delivers the sequence's final state; the others end where the next one starts.
            const bool last = sg == p.scan_k - 1;
            const int hi = p.state_chunk0 + p.seg_chunks;
            const int end = last ? (p.scan_open ? 0x7fffffff : hi) : min(p.state_chunk0 + (sg + 1) * p.scan_chunks, hi);
            const bool carried = sg == 0 && p.scan_carry_in != nullptr;  // a later super-block: its incoming state is a composed one
            const Walk wk{min(p.state_chunk0 + sg * p.scan_chunks, hi), end, sg == 0 && !carried ? 0 : 3,
                          carried ? p.scan_carry_in + (size_t)chain * DV * DK : p.scan_start + ((size_t)chain * p.scan_k + sg) * DV * DK,
                          last ? 0 : 2, nullptr, true, true};
            state_role<DV>(p, smem, tm, chain, 0, wk);
        }
    } else if (p.has_state && blockIdx.x < (unsigned)(chains * p.parts)) {
        const Walk wk{p.state_chunk0, p.state_chunk0 + p.seg_chunks, 0, nullptr, 0, nullptr, true, true};
        if (p.parts == 2) state_role<64>(p, smem, tm, (int)(blockIdx.x >> 1), (int)(blockIdx.x & 1), wk);
        else state_role<DV>(p, smem, tm, (int)blockIdx.x, 0, wk);
        tc::fence_after_sync();
    }
    if (p.has_intra && ctl[1] == 0u) intra_role(p, smem, tm);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tm, kTmemCols);
}

// Between the two scan passes: the state before every segment, S_start[s + 1] = A_s S_start[s] + B_s in FP32, from the
// caller's state.  A state's value columns never mix, so a block owns two of them (held in shared memory across the
// segments) and a thread one key channel: acc[v] += A_s[k][k'] S[k'][v] with A_s read along k (coalesced; A_s lies in
// the state's layout, entry [k'][k]).
constexpr int kComposeCols = 2;  // value columns per block: 64 blocks a chain (with eight columns, 16 blocks, a launch took 0.3 ms)
__global__ void __launch_bounds__(128) scan_compose_kernel(const __grid_constant__ SpParams p) {
    constexpr int kCols = kComposeCols;
    __shared__ float S[kCols][DK];
    const int chain = blockIdx.x / (DV / kCols), v0 = (blockIdx.x % (DV / kCols)) * kCols, k = threadIdx.x;
    const int b = chain / p.H, h = chain % p.H;
    const float* s0 = p.scan_carry_in != nullptr ? p.scan_carry_in + (size_t)chain * DV * DK
                                                 : reinterpret_cast<const float*>(p.state_in) + p.state_off[b] + (long long)h * DV * DK;
#pragma unroll
    for (int vi = 0; vi < kCols; ++vi) S[vi][k] = s0[(v0 + vi) * DK + k];
    __syncthreads();
    for (int sg = 0; sg < p.scan_p1; ++sg) {
        const float* B = p.scan_ab + ((size_t)chain * p.scan_p1 + sg) * 2 * DV * DK;
        const float* A = B + DV * DK;
        float acc[kCols];
#pragma unroll
        for (int vi = 0; vi < kCols; ++vi) acc[vi] = B[(v0 + vi) * DK + k];
#pragma unroll 8
        for (int kp = 0; kp < DK; ++kp) {
            const float a = A[kp * DK + k];
#pragma unroll
            for (int vi = 0; vi < kCols; ++vi) acc[vi] = fmaf(a, S[vi][kp], acc[vi]);
        }
        __syncthreads();
        // the state before segment sg + 1, or, after the last segment (scan_p1 == K), the state after the launch's range
        float* out = sg + 1 < p.scan_k ? p.scan_start + ((size_t)chain * p.scan_k + sg + 1) * DV * DK : p.scan_carry_out + (size_t)chain * DV * DK;
#pragma unroll
        for (int vi = 0; vi < kCols; ++vi) {
            S[vi][k] = acc[vi];
            out[(v0 + vi) * DK + k] = acc[vi];
        }
        __syncthreads();
    }
}

}  // namespace

// The driver's tensor-map encoder, looked up once through the runtime (the library does not link libcuda).
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiled>(f);
    }();
    return fn;
}

// A [rows][H][128] tensor of `elem`-byte elements as (128, H, rows) with boxes of 64 rows of one head, 128 bytes wide.
static bool row_tensor_map(CUtensorMap* tm, const void* base, int elem, int H, long long rows) {
    EncodeTiled enc = encode_tiled();
    if (enc == nullptr) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)DK, (cuuint64_t)H, (cuuint64_t)rows};
    const cuuint64_t strides[2] = {(cuuint64_t)DK * elem, (cuuint64_t)H * DK * elem};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / elem), 1u, (cuuint32_t)CH};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(tm, elem == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr long long kCounterBytes = 256;  // tail of the workspace: the two item counters

int64_t core_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t chunks_per_pass) {
    if (heads < 1 || batch < 1 || chunks_per_pass < 1) return 0;
    return (int64_t)heads * batch * chunks_per_pass * kSlotBytes + kCounterBytes;
}

// The launches over every segment of the longest sequence, in stream order.  A workspace of two or more chunks per
// chain is split into halves so that the state role of one segment runs beside the intra role of the next; a
// workspace of one chunk per chain alternates intra-only and state-only launches.
// Two side streams and their events per device, made on the first head-sharded scan (host objects only; no device memory).
constexpr int kMaxSuperBlocks = 16;
struct SideStreams {
    cudaStream_t a = nullptr, b = nullptr;
    cudaEvent_t fork = nullptr, join_a = nullptr, join_b = nullptr, ready[kMaxSuperBlocks] = {};
};
static SideStreams* side_streams() {
    constexpr int kMaxDevices = 64;
    static SideStreams table[kMaxDevices];
    static bool made[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    SideStreams& t = table[dev];
    if (!made[dev]) {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);  // hi is the numerically lowest = the most urgent
        bool ok = cudaStreamCreateWithPriority(&t.a, cudaStreamNonBlocking, lo) == cudaSuccess &&
                  cudaStreamCreateWithPriority(&t.b, cudaStreamNonBlocking, hi) == cudaSuccess;  // the stores go first
        ok = ok && cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&t.join_a, cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&t.join_b, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; ok && i < kMaxSuperBlocks; ++i) ok = cudaEventCreateWithFlags(&t.ready[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            return nullptr;
        }
        made[dev] = true;
    }
    return &t;
}

int core_prefill_sp_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len, const glm53f_bf16* q,
                           const glm53f_bf16* k, const glm53f_bf16* v, const float* g, const float* beta, const void* state_in,
                           void* state_out, const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate,
                           const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                           cudaStream_t stream, const PrefillScatter* scatter) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_sp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemSp);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    const long long chains = (long long)heads * batch;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15) != 0 || workspace_bytes < kCounterBytes) return kInvalid;
    const long long usable = (workspace_bytes - kCounterBytes) & ~15ll;
    const long long whole = usable / (chains * kSlotBytes);
    if (whole < 1) return kInvalid;
    const bool overlap = whole >= 2;
    long long seg = overlap ? whole / 2 : whole;
    const long long need = ((long long)max_len + CH - 1) / CH;
    if (seg > need) seg = need > 0 ? need : 1;
    SpParams p{};
    p.H = heads; p.batch = batch; p.cu = cu_seqlens;
    p.q = q; p.k = k; p.v = v; p.g = g; p.beta = beta;
    p.state_in = state_in; p.state_out = state_out;
    p.state_off = reinterpret_cast<const long long*>(state_off);
    p.state_bf16 = bf16_state ? 1 : 0;
    p.gate = gate; p.norm_w = norm_w; p.eps = eps; p.out = out;
    if (scatter != nullptr) {
        if (scatter->ranks < 1 || scatter->ranks > 8 || scatter->head0 < 0 || scatter->head0 + heads > scatter->heads_total) return kInvalid;
        for (int r = 0; r < scatter->ranks; ++r) {
            if (scatter->full[r] == nullptr || (reinterpret_cast<uintptr_t>(scatter->full[r]) & 15) != 0) return kInvalid;
            p.full[r] = scatter->full[r];
        }
        p.ranks = scatter->ranks; p.heads_total = scatter->heads_total; p.head0 = scatter->head0;
    } else if (out == nullptr) {
        return kInvalid;
    }
    // Few chains: the serial walk over a chain's chunks is the critical path, so two blocks share each chain.  (Not with
    // the fused output norm, which needs a row's every value channel in one block.)
    p.parts = (gate == nullptr && chains * 2 <= 64) ? 2 : 1;
    p.seg_chunks = (int)seg;
    unsigned char* base = reinterpret_cast<unsigned char*>(workspace);
    unsigned char* half[2] = {base, overlap ? base + chains * seg * kSlotBytes : base};
    p.counters = reinterpret_cast<unsigned int*>(base + usable);
    p.status = status_word();
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    // Tensor copies fetch full chunks only, whose rows the caller's metadata vouches for; the extent written into the
    // maps is the most rows the batch can hold.
    long long rows_cap = (long long)batch * max_len;
    rows_cap = rows_cap < CH ? CH : (rows_cap > 0x7fffffffll ? 0x7fffffffll : rows_cap);
    if (!row_tensor_map(&p.tm_q, q, 2, heads, rows_cap) || !row_tensor_map(&p.tm_k, k, 2, heads, rows_cap) ||
        !row_tensor_map(&p.tm_v, v, 2, heads, rows_cap) || !row_tensor_map(&p.tm_g, g, 4, heads, rows_cap))
        return (int)cudaErrorNotSupported;
    if (out != nullptr && !row_tensor_map(&p.tm_out, out, 2, heads, rows_cap)) return (int)cudaErrorNotSupported;
    for (int r = 0; r < p.ranks; ++r)
        if (!row_tensor_map(&p.tm_full[r], p.full[r], 2, p.heads_total, rows_cap)) return (int)cudaErrorNotSupported;
    cudaError_t e = cudaMemsetAsync(p.counters, 0, 2 * sizeof(unsigned int), stream);
    if (e != cudaSuccess) return (int)e;
    const long long sms = sm_count();
    // Few chains and a long sequence: the serial walk over a chain's chunks is the critical path whatever the number of
    // idle SMs.  The recurrence is affine in the state (S_end = A S_start + B over any run of chunks), so the sequence is
    // cut into K segments that are walked at the same time: once from the zero state and once from the identity without
    // U (their end states are B and A), then, after the K - 1 compositions, once more from the true incoming states with
    // the outputs.  Needs FP32 states (a bf16 state is rounded every chunk, which is not affine) and a workspace that
    // holds every chunk of the call plus (3K - 2) states per chain.  K follows from the number of chains, the SM count and
    // the length (or GLM53F_KDA_PREFILL_SEGMENTS); the results depend on K, not otherwise on the workspace size.
    {
        long long K = 1;
        if (const char* env = getenv("GLM53F_KDA_PREFILL_SEGMENTS")) K = atoll(env);
        else if (chains <= 16) {  // measured, 2^20 tokens: 8 chains 41.0 -> 17.0 ms, 16 chains 42.1 -> 33.8 ms, 32 chains 55.3 -> 61.9 ms
            const long long ka = sms / (2 * chains) + 1, kc = sms / chains;
            K = ka < kc ? ka : kc;
            if (K > 16) K = 16;
            if (K > need / 32) K = need / 32;  // a segment of fewer than 32 chunks is not worth three walks
        }
        if (K > need) K = need;
        // A head-sharded launch sends every output row to every rank, and the scan emits all outputs in its last pass: the
        // NVLink time (15 GB per GPU at 8 ranks) would follow the compute instead of running beside it.  So there the
        // sequence is cut into super-blocks, each scanned on its own: the intra role and pass 1 of super-block b + 1 run on
        // one side stream while the composition and pass 2 of super-block b -- the stores -- run on another.  Pass 2 then
        // holds SMs while it waits for the links, so it gets fewer, longer segments (K <= 48 / chains).
        // GLM53F_KDA_PREFILL_SUPERBLOCKS overrides the count (1 = off).
        long long SB = (scatter != nullptr && scatter->ranks > 1) ? 8 : 1;
        long long min_seg = 32;  // a segment of fewer than 32 chunks is not worth three walks (an override may ask for any)
        if (const char* env = getenv("GLM53F_KDA_PREFILL_SUPERBLOCKS")) {
            SB = atoll(env);
            min_seg = 1;
        }
        if (SB > kMaxSuperBlocks) SB = kMaxSuperBlocks;
        if (SB > 1 && K >= 2 && !bf16_state) {
            long long Ks = K;
            if (getenv("GLM53F_KDA_PREFILL_SEGMENTS") == nullptr && Ks > 48 / chains) Ks = 48 / chains > 2 ? 48 / chains : 2;
            while (SB > 1 && need / (SB * Ks) < min_seg) --SB;
            const long long sb = (need + SB - 1) / SB;
            // per super-block: K transitions and offsets, K incoming states, and the state after the super-block
            const long long scratch_sb = chains * (3 * Ks + 1) * (long long)(DV * DK * sizeof(float));
            SideStreams* side = SB > 1 && chains * SB * sb * kSlotBytes + SB * scratch_sb <= usable ? side_streams() : nullptr;
            if (side != nullptr) {
                if ((e = cudaEventRecord(side->fork, stream)) != cudaSuccess) return (int)e;
                cudaStreamWaitEvent(side->a, side->fork, 0);
                cudaStreamWaitEvent(side->b, side->fork, 0);
                unsigned char* scratch0 = base + chains * SB * sb * kSlotBytes;
                const float* carry = nullptr;
                for (long long b = 0; b < SB; ++b) {
                    const long long c0 = b * sb, cnt = (need - c0) < sb ? (need - c0) : sb;
                    if (cnt <= 0) break;
                    const long long Kb = cnt >= min_seg * Ks ? Ks : (cnt / min_seg > 1 ? cnt / min_seg : 1);
                    p.parts = 1;
                    p.seg_chunks = (int)cnt;
                    p.intra_chunk0 = p.state_chunk0 = (int)c0;
                    p.ws_intra = p.ws_state = base + b * chains * sb * kSlotBytes;
                    p.ctr = (int)(b & 1);
                    p.scan_k = (int)Kb;
                    p.scan_p1 = (int)Kb;  // every segment: the state after the super-block is composed, not walked for
                    p.scan_chunks = (int)((cnt + Kb - 1) / Kb);
                    p.scan_open = (c0 + cnt >= need) ? 1 : 0;
                    p.scan_ab = reinterpret_cast<float*>(scratch0 + b * scratch_sb);
                    p.scan_start = p.scan_ab + chains * Kb * 2 * DV * DK;
                    p.scan_carry_in = carry;
                    p.scan_carry_out = p.scan_start + chains * Kb * DV * DK;
                    // one stream: everything up to the states before this super-block's segments and after it -- the intra
                    // role, both walks of every segment, the composition (which needs the previous super-block's, not its
                    // pass 2)
                    p.has_intra = 1; p.has_state = 0; p.scan_pass = 0;
                    // The intra blocks are persistent: on every SM they would keep the previous super-block's output pass,
                    // which is ready about now, off the machine until they are done, and the links idle.  From the second
                    // super-block on they leave that pass its SMs (measured on 8 GPUs, 2^20 tokens: 28.6 -> 26.1 ms).
                    const long long items = chains * cnt, room = b == 0 ? sms : (sms - Kb * chains > sms / 2 ? sms - Kb * chains : sms / 2);
                    prefill_sp_kernel<<<(unsigned)(items < room ? items : room), kThreadsSp, kSmemSp, side->a>>>(p);
                    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
                    p.has_intra = 0; p.has_state = 1; p.scan_pass = 1;
                    prefill_sp_kernel<<<(unsigned)(2 * Kb * chains), kThreadsSp, kSmemSp, side->a>>>(p);
                    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
                    scan_compose_kernel<<<(unsigned)(chains * (DV / kComposeCols)), 128, 0, side->a>>>(p);
                    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
                    cudaEventRecord(side->ready[b], side->a);
                    // the other: the walks with the outputs (and the stores to the peers), super-block after super-block
                    cudaStreamWaitEvent(side->b, side->ready[b], 0);
                    p.scan_pass = 2;
                    prefill_sp_kernel<<<(unsigned)(Kb * chains), kThreadsSp, kSmemSp, side->b>>>(p);
                    if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
                    carry = p.scan_carry_out;
                }
                cudaEventRecord(side->join_a, side->a);
                cudaEventRecord(side->join_b, side->b);
                cudaStreamWaitEvent(stream, side->join_a, 0);
                if ((e = cudaStreamWaitEvent(stream, side->join_b, 0)) != cudaSuccess) return (int)e;
                return 0;
            }
        }
        const long long scratch = chains * (3 * K - 2) * (long long)(DV * DK * sizeof(float));
        if (K >= 2 && !bf16_state && chains * need * kSlotBytes + scratch <= usable) {
            p.seg_chunks = (int)need;
            p.parts = 1;
            p.ws_intra = p.ws_state = base;
            p.intra_chunk0 = p.state_chunk0 = 0;
            p.ctr = 0;
            p.scan_k = (int)K;
            p.scan_chunks = (int)((need + K - 1) / K);
            p.scan_ab = reinterpret_cast<float*>(base + chains * need * kSlotBytes);
            p.scan_start = p.scan_ab + chains * (K - 1) * 2 * DV * DK;
            p.scan_open = 1;
            p.scan_p1 = (int)K - 1;
            p.scan_carry_in = nullptr; p.scan_carry_out = nullptr;
            p.has_intra = 1; p.has_state = 0; p.scan_pass = 0;
            const long long items = chains * need;
            prefill_sp_kernel<<<(unsigned)(items < sms ? items : sms), kThreadsSp, kSmemSp, stream>>>(p);
            if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
            p.has_intra = 0; p.has_state = 1; p.scan_pass = 1;
            prefill_sp_kernel<<<(unsigned)(2 * (K - 1) * chains), kThreadsSp, kSmemSp, stream>>>(p);
            if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
            scan_compose_kernel<<<(unsigned)(chains * (DV / kComposeCols)), 128, 0, stream>>>(p);
            if ((e = cudaGetLastError()) != cudaSuccess) return (int)e;
            p.scan_pass = 2;
            prefill_sp_kernel<<<(unsigned)(K * chains), kThreadsSp, kSmemSp, stream>>>(p);
            return (int)cudaGetLastError();
        }
    }
    const long long segs = need > 0 ? (need + seg - 1) / seg : 0;
    int launch_no = 0;
    auto launch = [&](long long intra_seg, long long state_seg) -> int {
        p.has_intra = intra_seg >= 0 ? 1 : 0;
        p.has_state = state_seg >= 0 ? 1 : 0;
        p.intra_chunk0 = (int)(intra_seg * seg);
        p.state_chunk0 = (int)(state_seg * seg);
        p.ws_intra = half[intra_seg & 1];
        p.ws_state = half[state_seg & 1];
        p.ctr = launch_no++ & 1;
        long long grid = p.has_state ? chains * p.parts : 0;
        if (p.has_intra) {
            const long long items = chains * seg, want = items < sms ? items : sms;
            if (grid < want) grid = want;
        }
        prefill_sp_kernel<<<(unsigned)grid, kThreadsSp, kSmemSp, stream>>>(p);
        return (int)cudaGetLastError();
    };
    if (segs == 0) return launch(-1, 0);  // nothing but empty sequences: their states are copied
    if (overlap) {
        for (long long s = 0; s <= segs; ++s) {
            const int rc = launch(s < segs ? s : -1, s - 1);
            if (rc != 0) return rc;
        }
    } else {
        for (long long s = 0; s < segs; ++s) {
            int rc = launch(s, -1);
            if (rc == 0) rc = launch(-1, s);
            if (rc != 0) return rc;
        }
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// The same two-pass prefill for callers that may not allocate device memory at all.
//
// Some hosts of this library run inside a memory plan that is fixed before the first request: an inference engine
// whose planner has handed every byte of HBM to weights, KV pages and state arenas, or a component called from a
// region of its host where allocation is forbidden (an allocator lock held, a latency-critical loop), where cudaMalloc
// would fail, fragment the plan or stall.  Such a caller cannot produce the workspace
// glm53f_kda_core_prefill_varlen_ws asks for.  For them the library carries its own scratch: a fixed array in the
// library's device image (held by every GPU that has loaded the image until the process exits; with the runtime's
// default lazy loading the image is placed in device memory at the first call below, which is why a host makes one
// small set-up call per device before its memory plan is final), big enough for 64 workspace slots and the item counters.  Nothing in it has to start at zero: the
// intra role writes every byte of a slot that the state role reads, and each call clears the counters itself.  All calls share the one array, so two calls in flight at once (two
// streams, two threads) overwrite each other's slots; the caller serialises them.
constexpr int kStaticSlots = 64;
constexpr long long kStaticScratchBytes = (long long)kStaticSlots * kSlotBytes + kCounterBytes;  // 6,848,768 bytes
static __device__ __align__(256) unsigned char g_prefill_scratch[kStaticScratchBytes];

// The array's name is a host-side handle here, not a device address: the address a kernel can use is asked for once
// per device (with that device current) and remembered.
int core_prefill_static_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len, const glm53f_bf16* q,
                               const glm53f_bf16* k, const glm53f_bf16* v, const float* g, const float* beta, const void* state_in,
                               void* state_out, const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate,
                               const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, cudaStream_t stream) {
    constexpr int kMaxDevices = 64;
    static void* scratch_of[kMaxDevices] = {};
    if ((long long)heads * batch > kStaticSlots) return kInvalid;  // not even one chunk per chain would fit
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return kInvalid;
    if (scratch_of[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_prefill_scratch);
        if (e != cudaSuccess) return (int)e;
        scratch_of[dev] = ptr;
    }
    return core_prefill_sp_launch(heads, batch, cu_seqlens, max_len, q, k, v, g, beta, state_in, state_out, state_off, bf16_state,
                                  gate, norm_w, eps, out, scratch_of[dev], kStaticScratchBytes, stream);
}

}  // namespace kda
