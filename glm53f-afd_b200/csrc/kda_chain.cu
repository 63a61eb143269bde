// The recurrent KDA step on B200 (sm_100a): decode, draft verification, commit replay.
//
// One persistent, warp-specialised block per SM walks a list of units, unit = (request, head) of one layer (or
// (request, layer, head) for the commit replay).  Four roles, connected by mbarrier rings in shared memory:
//
//   mover (1 warp)      bulk-copies (cp.async.bulk) each unit's 128x128 state and each row's raw inputs from global
//                       memory into shared-memory rings, several units ahead of the arithmetic;
//   prologue (2 warps)  turns a row's raw inputs into q, k, v, the decay multipliers, beta and sigmoid(gate)
//                       (short conv + SiLU, L2 norms, gates for the layer entry points; exp(g) for the core ones);
//   recurrence (16 warps) keeps the unit's state in registers across its rows: warp w owns value rows 8w..8w+7,
//                       lane l key columns 4l..4l+3; per row the delta rule and the read-out; afterwards each warp
//                       stores its own 8 rows, a whole contiguous row per instruction;
//   epilogue (1 warp)   gated RMSNorm, bf16 outputs, replay saves.
//
// The state therefore crosses HBM once in each direction -- in as bulk transfers that are always several units deep
// in flight, out as coalesced vector stores from the registers -- and no role ever waits on a global load.
//
// Arithmetic contract (what makes this a drop-in for the reference's kernels/kda.cu): every sum over the 128 key
// channels is formed as the reference forms it -- a lane's four consecutive channels added in order from zero,
// then the five-step xor butterfly over 32 lanes -- and nothing is contracted into an FMA (this file is compiled
// with --fmad=false --ftz=false --prec-div=true --prec-sqrt=true, the reference's build.rs flags).  The butterfly
// is evaluated as a reduce-scatter (kda.cu:30-33 applied to eight rows at once): the same additions in the same
// pairing, so the same bits, with 9 shuffles for eight rows instead of 40.  decode, verify and replay share
// `delta_rule`, so a replayed prefix of a window has the bits of serial single-row steps
// (reference kernels/glm53f_kda.h:111-116, 166-168).
//
// Reference lines restated here: kernels/kda.cu:38-53 (update), 98-210 (chain_kernel), 214-253 (replay_kernel),
// 290-460 (argument checks and entry points).

#include <atomic>
#include <cstdlib>
#include <cstring>
#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"

namespace kda {

__device__ int g_status = 0;
// Host-side settings of the diagnostic hook glm53f_kda_debug_wait_test: the bound of the recurrent kernels' waits, and
// a one-shot request that the next launch's block 0 leaves its first unit's state unfetched.
static unsigned long long g_wait_limit_ns = kWaitLimitNs;
// How glm53f_kda_chain_batch_bf16state runs a verify call (read-only states, saves on): 0 = the exact row-by-row form,
// 1 = the chunked tensor-core form; GLM53F_KDA_VERIFY=chunked makes 1 the default.
static std::atomic<int> g_layer_verify_mode{[] {
    const char* e = getenv("GLM53F_KDA_VERIFY");
    return e != nullptr && strcmp(e, "chunked") == 0 ? 1 : 0;
}()};
// How the bf16-state replays run: 0 = the exact row-by-row form, 1 = chunks of 16 rows on the tensor cores;
// GLM53F_KDA_COMMIT=chunked makes 1 the default.
static std::atomic<int> g_commit_mode{[] {
    const char* e = getenv("GLM53F_KDA_COMMIT");
    return e != nullptr && strcmp(e, "chunked") == 0 ? 1 : 0;
}()};
static int g_skip_first_state = 0;

int sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            n = v;
        else {
            cudaGetLastError();
            return 1;
        }
    }
    return n;
}

namespace {

enum Mode : int { kLayer = 0, kCore = 1, kReplay = 2 };

constexpr int kRecWarps = 16, kRecThreads = kRecWarps * 32;
// Prologue warps per mode.  The layer prologue (conv + SiLU, decay, gate: ~740 warp instructions per row in dependent
// chains of divisions and exponentials) on two warps was the slowest stage of a layer call (measured: decode through
// the layer symbol 0.746 -> 0.657 ms per step with four, the exact verify 24.5 -> 19.1 ms, an exact prefill lane
// 2.05 -> 1.57 ms, the replay 4.97 -> 4.72 ms); the core prologue is a widening and one exponential per channel, and
// there two more warps only take registers and issue slots from the recurrence (0.538 -> 0.566 ms).
template <int MODE>
constexpr int kProWarpsOf = MODE == 1 /* kCore */ ? 2 : 4;
template <int MODE>
constexpr int kProThreadsOf = kProWarpsOf<MODE> * 32;
template <int MODE>
constexpr int kThreadsOf = kRecThreads + kProThreadsOf<MODE> + 64;  // + epilogue warp + mover warp
constexpr int kRowsPerLane = DV / kRecWarps;              // 8
constexpr unsigned FULL = 0xffffffffu;

struct Params {
    int H, layers;
    long long units;
    const int32_t* cu_rows;
    const int32_t* keep;
    int rows1;
    // layer entry points
    const uint16_t* P;
    long long p_stride, b_off;
    const uint16_t* A;
    long long a_stride;
    const uint16_t* G;  // output-gate rows (layer: stride g_stride; core: dense, may be null)
    long long g_stride;
    const uint16_t* conv;
    const long long* conv_off;
    const uint16_t* cw;
    const float* a_log;
    const float* dt_bias;
    const uint16_t* norm_w;
    float eps, lower;
    // core entry points
    const uint16_t *q, *k, *v;
    const float* glog;
    const float* beta;
    int flags;
    // states
    const void* state_in;
    void* state_out;
    long long state_stride;
    const long long* state_off;
    // outputs (for the replay the saves are inputs)
    uint16_t* out;
    long long out_stride;
    float* k_save;
    uint16_t* v_save;
    float* g_save;
    float* b_save;
    long long kv_stride, b_stride;
    unsigned long long neg_zero2;  // two -0.0f: see mul2
    unsigned long long wait_limit_ns;  // bound of every device-side wait (no progress for this long: give up)
    int skip_first_state;  // diagnostic (glm53f_kda_debug_wait_test): block 0 does not fetch its first unit's state
};

// Raw-row slot layouts, byte offsets.
struct RawLayer {
    static constexpr int X = 0;                 // bf16 [4 taps][3 parts][128]
    static constexpr int W = X + 4 * 3 * 256;   // bf16 [3 parts][128][4]
    static constexpr int A = W + 3 * 1024;      // bf16 [128]
    static constexpr int GATE = A + 256;        // bf16 [128]
    static constexpr int DTB = GATE + 256;      // f32 [128]
    static constexpr int B = DTB + 512;         // the 16 aligned bytes that hold the beta logit
    static constexpr int BYTES = B + 16;
};
struct RawCore {
    static constexpr int Q = 0, K = 256, V = 512;  // bf16 [128] each
    static constexpr int GLOG = 768;               // f32 [128]
    static constexpr int GATE = GLOG + 512;        // bf16 [128]
    static constexpr int B = GATE + 256;           // the 16 aligned bytes that hold beta (f32)
    static constexpr int BYTES = B + 16;
};
struct RawReplay {
    static constexpr int K = 0, G = 512;  // f32 [128] each
    static constexpr int V = 1024;        // bf16 [128]
    static constexpr int B = V + 256;     // the 16 aligned bytes that hold beta (f32)
    static constexpr int BYTES = B + 16;
};
template <int MODE>
struct RawOf;
template <>
struct RawOf<kLayer> { using T = RawLayer; };
template <>
struct RawOf<kCore> { using T = RawCore; };
template <>
struct RawOf<kReplay> { using T = RawReplay; };

constexpr int align_up(int x, int a) { return (x + a - 1) / a * a; }

// A cooked row: what the recurrence and the epilogue read.
struct Cooked {
    float q[DK], k[DK], v[DV], g[DK], sg[DV], ys[DV];
    float beta;
    int pad[3];
};

template <typename S, int MODE>
struct Smem {
    static constexpr int kStateBytes = DV * DK * (int)sizeof(S);
    static constexpr int kStateSlots = sizeof(S) == 4 ? 3 : 5;
    static constexpr int kRawSlots = sizeof(S) == 4 ? 3 : 4;  // raw-row ring depth
    static constexpr int kRowSlots = sizeof(S) == 4 ? 3 : 4;  // cooked-row ring depth
    static constexpr int kRawBytes = align_up(RawOf<MODE>::T::BYTES, 128);
    static constexpr int oState = 0;
    static constexpr int oRaw = oState + kStateSlots * kStateBytes;
    static constexpr int oCooked = oRaw + kRawSlots * kRawBytes;
    static constexpr int oScratch = oCooked + kRowSlots * (int)sizeof(Cooked);  // prologue scratch: q, k before norm
    static constexpr int oBars = oScratch + 2 * DK * 4;
    // barriers: st_full[S], st_empty[S], raw_full[R], raw_empty[R], row_full[C], y_full[C], row_empty[C]
    static constexpr int kBars = 2 * kStateSlots + 2 * kRawSlots + 3 * kRowSlots;
    static constexpr int oCtl = oBars + kBars * 8;  // progress, abort
    static constexpr int kBytes = oCtl + 16;
};

struct Unit {
    int b, h, layer, rows;
    long long row0;
    long long s_elem;    // element offset of this head's state inside state_in / state_out
    long long conv_off;  // layer entry points: element offset of the request's conv window
    float a_log;         // layer entry points: A_log of the head
};

// The units of this block, u = blockIdx.x, blockIdx.x + gridDim.x, ...: (request, head) with the head fastest, or
// (request, layer, head) for the replay.  Indices advance by 32-bit arithmetic; the metadata of the next unit
// (row range, state and window offsets: loads from global memory) is fetched while the current one is processed.
template <int MODE>
struct UnitIter {
    unsigned long long u;
    unsigned b, h, layer;
    unsigned step_b, step_h;  // gridDim.x = step_b * H + step_h
    bool ok;
    Unit nxt;

    __device__ __forceinline__ explicit UnitIter(const Params& p) {
        u = blockIdx.x;
        ok = u < (unsigned long long)p.units;
        const unsigned H = (unsigned)p.H, L = (unsigned)p.layers;
        h = blockIdx.x % H;
        step_b = gridDim.x / H;
        step_h = gridDim.x - step_b * H;
        const unsigned q = blockIdx.x / H;
        layer = MODE == kReplay ? q % L : 0u;
        b = MODE == kReplay ? q / L : q;
        if (ok) nxt = fetch(p);
    }
    __device__ __forceinline__ Unit fetch(const Params& p) const {
        Unit x;
        x.b = (int)b;
        x.h = (int)h;
        x.layer = (int)layer;
        if (MODE == kReplay) {
            x.row0 = p.cu_rows ? p.cu_rows[b] : 0;
            x.rows = p.keep ? p.keep[b] : p.rows1;
        } else if (p.cu_rows) {
            const int r0 = p.cu_rows[b];
            x.row0 = r0;
            x.rows = p.cu_rows[b + 1] - r0;
            if (MODE == kLayer && p.keep) {  // a commit by recomputation: only the request's first keep[b] rows
                const int kept = p.keep[b];
                if (kept < x.rows) x.rows = kept;
            }
        } else {
            x.row0 = 0;
            x.rows = p.rows1;
        }
        if (x.rows < 0) x.rows = 0;
        x.s_elem = (long long)layer * p.state_stride + (p.state_off ? p.state_off[b] : 0) + (long long)h * DV * DK;
        x.conv_off = 0;
        x.a_log = 0.0f;
        if (MODE == kLayer) {
            x.conv_off = p.conv_off ? p.conv_off[b] : 0;
            x.a_log = p.a_log[h];
        }
        return x;
    }
    __device__ __forceinline__ bool valid() const { return ok; }
    // The current unit; advances to the next one and starts fetching its metadata.
    __device__ __forceinline__ Unit take(const Params& p) {
        const Unit cur = nxt;
        u += gridDim.x;
        ok = u < (unsigned long long)p.units;
        const unsigned H = (unsigned)p.H;
        if (MODE == kReplay) {
            const unsigned nh = h + gridDim.x, dq = nh / H;
            h = nh - dq * H;
            const unsigned L = (unsigned)p.layers, nl = layer + dq, lq = nl / L;
            layer = nl - lq * L;
            b += lq;
        } else {  // the stride in (request, head) is fixed for the launch: no division per unit
            h += step_h;
            b += step_b;
            if (h >= H) {
                h -= H;
                ++b;
            }
        }
        if (ok) nxt = fetch(p);
        return cur;
    }
};

// Whether a unit without rows still has to move its state (out of place copy).
__device__ __forceinline__ bool copies_state(const Params& p) { return p.state_out != nullptr && p.state_out != p.state_in; }

struct Ring {
    int idx = 0;
    uint32_t phase = 0;
    __device__ __forceinline__ void next(int n) {
        if (++idx == n) {
            idx = 0;
            phase ^= 1u;
        }
    }
};

// ---- packed FP32 pairs -----------------------------------------------------------------------------------------
// sm_100 has two-wide FP32 instructions (mul.f32x2, add.f32x2): each half is an IEEE round-to-nearest operation,
// so a pair gives the bits of two scalar instructions for half the issue slots.  The recurrence is bound by
// instruction issue, not by the FP32 pipe, so the state is held as pairs: pair jp of a lane holds value rows
// 2jp and 2jp+1 of its warp at one key column.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
// The product of two pairs, each half rounded once.  It is written as fma(a, b, -0) with the -0 pair read from the
// kernel's parameters: ptxas contracts a dependent mul.rn.f32x2 / add.rn.f32x2 pair into one FFMA2 even when
// contraction is off (measured: 1-ulp differences against the scalar sequence), which would break the bitwise
// contract; a product that comes out of an FMA with an addend the compiler cannot see through is left alone, and
// x*y + (-0) is x*y for every x*y, signed zeros included.
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b, f32x2 nz) {
    f32x2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(nz));
    return r;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

constexpr int kPairs = kRowsPerLane / 2;  // 4 row pairs per lane

// ---- state registers <-> shared memory -----------------------------------------------------------------------
template <typename S>
__device__ __forceinline__ void load_row(const unsigned char* slot, int row, int lane, float (&x)[4]) {
    if constexpr (sizeof(S) == 4) {
        const float4 v = *reinterpret_cast<const float4*>(slot + ((size_t)row * DK + lane * 4) * 4);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(slot + ((size_t)row * DK + lane * 4) * 2);
        x[0] = __uint_as_float(v.x << 16);
        x[1] = __uint_as_float(v.x & 0xffff0000u);
        x[2] = __uint_as_float(v.y << 16);
        x[3] = __uint_as_float(v.y & 0xffff0000u);
    }
}

template <typename S>
__device__ __forceinline__ void load_rows(const unsigned char* slot, int warp, int lane, f32x2 (&s)[kPairs][4]) {
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        float a[4], b[4];
        load_row<S>(slot, warp * kRowsPerLane + 2 * jp, lane, a);
        load_row<S>(slot, warp * kRowsPerLane + 2 * jp + 1, lane, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) s[jp][i] = pack2(a[i], b[i]);
    }
}

// Two floats rounded to bf16 (nearest even) in one instruction: lo in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <typename S>
__device__ __forceinline__ void store_row(unsigned char* slot, int row, int lane, const float (&x)[4]) {
    if constexpr (sizeof(S) == 4) {
        *reinterpret_cast<float4*>(slot + ((size_t)row * DK + lane * 4) * 4) = make_float4(x[0], x[1], x[2], x[3]);
    } else {
        *reinterpret_cast<uint2*>(slot + ((size_t)row * DK + lane * 4) * 2) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
    }
}

template <typename S>
__device__ __forceinline__ void store_rows(unsigned char* slot, int warp, int lane, const f32x2 (&s)[kPairs][4]) {
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) unpack2(s[jp][i], a[i], b[i]);
        store_row<S>(slot, warp * kRowsPerLane + 2 * jp, lane, a);
        store_row<S>(slot, warp * kRowsPerLane + 2 * jp + 1, lane, b);
    }
}

template <typename S>
__device__ __forceinline__ void store_rows_global(S* head, int warp, int lane, const f32x2 (&s)[kPairs][4]) {
    const bool vec = (reinterpret_cast<uintptr_t>(head) & (4 * sizeof(S) - 1)) == 0;
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        float x[2][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) unpack2(s[jp][i], x[0][i], x[1][i]);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            S* dst = head + (size_t)(warp * kRowsPerLane + 2 * jp + half) * DK + lane * 4;
            if constexpr (sizeof(S) == 4) {
                if (vec) *reinterpret_cast<float4*>(dst) = make_float4(x[half][0], x[half][1], x[half][2], x[half][3]);
                else
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = x[half][i];
            } else {
                const uint32_t lo = pack_bf16x2(x[half][0], x[half][1]), hi = pack_bf16x2(x[half][2], x[half][3]);
                if (vec) *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
                else {
                    uint16_t* d = reinterpret_cast<uint16_t*>(dst);
                    d[0] = (uint16_t)lo; d[1] = (uint16_t)(lo >> 16); d[2] = (uint16_t)hi; d[3] = (uint16_t)(hi >> 16);
                }
            }
        }
    }
}

// A bf16 state's rounding between two rows of a window: every element to bf16 and back.
__device__ __forceinline__ void round_rows(f32x2 (&s)[kPairs][4]) {
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float a, b;
            unpack2(s[jp][i], a, b);
            const uint32_t r = pack_bf16x2(a, b);
            s[jp][i] = pack2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u));
        }
}

// The 32-lane xor butterfly (offsets 16, 8, 4, 2, 1) of eight independent values per lane, evaluated as a
// reduce-scatter.  Lane l returns the butterfly's result for value (l >> 2); the additions and their pairing are
// those of `x += shfl_xor(x, o)` applied to each value, so the bits are the same.
__device__ __forceinline__ float butterfly8(const float (&p)[kRowsPerLane], int lane) {
    float r[4], t[2];
    {
        const bool up = (lane & 16) != 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float mine = up ? p[4 + j] : p[j];
            const float give = up ? p[j] : p[4 + j];
            r[j] = mine + __shfl_xor_sync(FULL, give, 16);
        }
    }
    {
        const bool up = (lane & 8) != 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float mine = up ? r[2 + j] : r[j];
            const float give = up ? r[j] : r[2 + j];
            t[j] = mine + __shfl_xor_sync(FULL, give, 8);
        }
    }
    const bool up = (lane & 4) != 0;
    float x = (up ? t[1] : t[0]) + __shfl_xor_sync(FULL, up ? t[0] : t[1], 4);
    x = x + __shfl_xor_sync(FULL, x, 2);
    x = x + __shfl_xor_sync(FULL, x, 1);
    return x;
}

// Dot products of the lane's eight rows with a key-channel vector x (both halves of x2[i] hold x[i]): per row the
// lane's four channels added in order from zero, then the butterfly.  Lane l gets row (l >> 2).
__device__ __forceinline__ float rows_dot(const f32x2 (&s)[kPairs][4], const f32x2 (&x2)[4], int lane, f32x2 nz) {
    float part[kRowsPerLane];
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        f32x2 acc = pack2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc = add2(acc, mul2(s[jp][i], x2[i], nz));
        unpack2(acc, part[2 * jp], part[2 * jp + 1]);
    }
    return butterfly8(part, lane);
}

// The plain butterfly for one value per lane (norms).
__device__ __forceinline__ float butterfly1(float x) {
#pragma unroll
    for (int o = 16; o; o >>= 1) x = x + __shfl_xor_sync(FULL, x, o);
    return x;
}

// One delta-rule step on a lane's 8 x 4 tile (reference kda.cu:38-53): decay, read with k, correct toward v.
// `v_mine` is v at the value row lane l reduces: row (l >> 2) of the warp's eight.
__device__ __forceinline__ void delta_rule_v(f32x2 (&s)[kPairs][4], const f32x2 (&kk)[4], const f32x2 (&gg)[4], float v_mine, int lane,
                                             float beta, f32x2 nz) {
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[jp][i] = mul2(s[jp][i], gg[i], nz);
    const float kv = rows_dot(s, kk, lane, nz);
    const float mine = (v_mine - kv) * beta;
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        const f32x2 delta = pack2(__shfl_sync(FULL, mine, 8 * jp), __shfl_sync(FULL, mine, 8 * jp + 4));
#pragma unroll
        for (int i = 0; i < 4; ++i) s[jp][i] = add2(s[jp][i], mul2(kk[i], delta, nz));
    }
}
__device__ __forceinline__ void delta_rule(f32x2 (&s)[kPairs][4], const f32x2 (&kk)[4], const f32x2 (&gg)[4],
                                           const float* vrow, int warp, int lane, float beta, f32x2 nz) {
    delta_rule_v(s, kk, gg, vrow[warp * kRowsPerLane + (lane >> 2)], lane, beta, nz);
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- the mover -----------------------------------------------------------------------------------------------
// Calls f(dst_offset, src, bytes, is_scalar_chunk) for every piece of a row's raw inputs.  Pieces are 16-byte
// multiples except the "scalar chunk" (beta or its logit): for that one `src` is the element's own address and the
// mover copies the aligned 16 bytes around it, so the element lands at dst_offset + (address & 15).
template <int MODE, typename F>
__device__ __forceinline__ void for_each_piece(const Params& p, const Unit& u, int r, F&& f) {
    const long long gr = u.row0 + r;
    if constexpr (MODE == kLayer) {
        const long long C = 3LL * p.H * DK;
        const uint16_t* cs = p.conv + u.conv_off;
#pragma unroll
        for (int tap = 0; tap < TAPS; ++tap) {
            const int at = r + tap;
            const uint16_t* src_row = at < WINDOW ? cs + (long long)at * C : p.P + (u.row0 + at - WINDOW) * p.p_stride;
#pragma unroll
            for (int part = 0; part < 3; ++part)
                f(RawLayer::X + (tap * 3 + part) * 256, src_row + ((long long)part * p.H + u.h) * DK, 256, false);
        }
#pragma unroll
        for (int part = 0; part < 3; ++part)
            f(RawLayer::W + part * 1024, p.cw + (((long long)part * p.H + u.h) * DK) * TAPS, 1024, false);
        f(RawLayer::A, p.A + gr * p.a_stride + (long long)u.h * DK, 256, false);
        f(RawLayer::GATE, p.G + gr * p.g_stride + (long long)u.h * DV, 256, false);
        f(RawLayer::DTB, p.dt_bias + (long long)u.h * DK, 512, false);
        f(RawLayer::B, p.P + gr * p.p_stride + p.b_off + u.h, 2, true);
    } else if constexpr (MODE == kCore) {
        const long long at = (gr * p.H + u.h) * DK;
        f(RawCore::Q, p.q + at, 256, false);
        f(RawCore::K, p.k + at, 256, false);
        f(RawCore::V, p.v + at, 256, false);
        f(RawCore::GLOG, p.glog + at, 512, false);
        if (p.G) f(RawCore::GATE, p.G + at, 256, false);
        f(RawCore::B, p.beta + gr * p.H + u.h, 4, true);
    } else {
        const long long at = (gr * p.H + u.h) * DK;
        f(RawReplay::K, p.k_save + u.layer * p.kv_stride + at, 512, false);
        f(RawReplay::G, p.g_save + u.layer * p.kv_stride + at, 512, false);
        f(RawReplay::V, p.v_save + u.layer * p.kv_stride + at, 256, false);
        f(RawReplay::B, p.b_save + u.layer * p.b_stride + gr * p.H + u.h, 4, true);
    }
}

template <typename S, int MODE>
__device__ void mover_role(const Params& p, unsigned char* smem, uint64_t* bars, const WaitCtx& ctx, int lane) {
    using L = Smem<S, MODE>;
    uint64_t* st_full = bars;
    uint64_t* st_empty = st_full + L::kStateSlots;
    uint64_t* raw_full = st_empty + L::kStateSlots;
    uint64_t* raw_empty = raw_full + L::kRawSlots;
    Ring st, raw;
    const bool copy0 = copies_state(p);
    UnitIter<MODE> units(p);
    bool first = true;
    for (; units.valid(); first = false) {
        const Unit un = units.take(p);
        if (un.rows == 0 && !copy0) continue;
        // The unit's state.
        if (!mbar_wait(&st_empty[st.idx], st.phase ^ 1u, ctx, kStatusWaitStateEmpty)) return;
        if (p.skip_first_state && blockIdx.x == 0 && first) {
            // Diagnostic launch: nothing is copied and nobody is told, so the recurrence's wait for this state runs out.
        } else {
            unsigned char* dst = smem + L::oState + st.idx * L::kStateBytes;
            const unsigned char* src = reinterpret_cast<const unsigned char*>(p.state_in) + un.s_elem * (long long)sizeof(S);
            if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&st_full[st.idx], L::kStateBytes);
                    bulk_load(dst, src, L::kStateBytes, &st_full[st.idx]);
                }
            } else {  // a state that is not 16-byte aligned: element-wise copy by the whole warp
                const S* s = reinterpret_cast<const S*>(src);
                S* d = reinterpret_cast<S*>(dst);
                for (int e = lane; e < DV * DK; e += 32) d[e] = s[e];
                __syncwarp();
                if (lane == 0) mbar_arrive(&st_full[st.idx]);
            }
        }
        st.next(L::kStateSlots);
        // Its rows' raw inputs.
        for (int r = 0; r < un.rows; ++r) {
            if (!mbar_wait(&raw_empty[raw.idx], raw.phase ^ 1u, ctx, kStatusWaitRawEmpty)) return;
            unsigned char* dst = smem + L::oRaw + raw.idx * L::kRawBytes;
            uintptr_t low = 0;
            uint32_t bytes = 0;
            for_each_piece<MODE>(p, un, r, [&](int, const void* src, int n, bool scalar) {
                if (!scalar) low |= reinterpret_cast<uintptr_t>(src);
                bytes += scalar ? 16 : n;
            });
            if ((low & 15) == 0) {
                if (lane == 0) {
                    mbar_arrive_expect_tx(&raw_full[raw.idx], bytes);
                    for_each_piece<MODE>(p, un, r, [&](int off, const void* src, int n, bool scalar) {
                        if (scalar)
                            bulk_load(dst + off, reinterpret_cast<const void*>(reinterpret_cast<uintptr_t>(src) & ~uintptr_t(15)), 16,
                                      &raw_full[raw.idx]);
                        else
                            bulk_load(dst + off, src, n, &raw_full[raw.idx]);
                    });
                }
            } else {  // unaligned rows: 2-byte copies by the whole warp
                for_each_piece<MODE>(p, un, r, [&](int off, const void* src, int n, bool scalar) {
                    const uint16_t* s = reinterpret_cast<const uint16_t*>(src);
                    uint16_t* d = reinterpret_cast<uint16_t*>(dst + off + (scalar ? (int)(reinterpret_cast<uintptr_t>(src) & 15) : 0));
                    for (int e = lane; e < n / 2; e += 32) d[e] = s[e];
                });
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_full[raw.idx]);
            }
            raw.next(L::kRawSlots);
            if (lane == 0) atomicAdd(const_cast<uint32_t*>(ctx.progress), 1u);
        }
    }
}

// ---- the prologue --------------------------------------------------------------------------------------------
// L2 norm of scratch[0..127] by one warp in the reference's order (kda.cu:151-165): lane partial over 4
// consecutive channels from zero, butterfly, times 1/sqrt(ss + 1e-6), q also times 128^-0.5.
__device__ __forceinline__ void l2norm_warp(const float* x, float* y, int lane, bool is_q) {
    float v4[4], ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v4[i] = x[lane * 4 + i];
        ss = ss + v4[i] * v4[i];
    }
    ss = butterfly1(ss);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float t = v4[i] * inv;
        if (is_q) t = t * (1.0f / sqrtf((float)DK));
        y[lane * 4 + i] = t;
    }
}

template <typename S, int MODE>
__device__ void prologue_role(const Params& p, unsigned char* smem, uint64_t* bars, const WaitCtx& ctx, int t) {
    using L = Smem<S, MODE>;
    constexpr int kProThreads = kProThreadsOf<MODE>;
    uint64_t* raw_full = bars + 2 * L::kStateSlots;
    uint64_t* raw_empty = raw_full + L::kRawSlots;
    uint64_t* row_full = raw_empty + L::kRawSlots;
    uint64_t* row_empty = row_full + 2 * L::kRowSlots;
    float* scratch = reinterpret_cast<float*>(smem + L::oScratch);
    const int warp = t >> 5, lane = t & 31;
    Ring raw, row;
    const bool copy0 = copies_state(p);
    // Whether the role's threads meet at barriers in every row (the L2 norms go through shared scratch).
    const bool syncs = MODE == kLayer || (MODE == kCore && (p.flags & GLM53F_KDA_CORE_L2NORM) != 0);
    UnitIter<MODE> units(p);
    while (units.valid()) {
        const Unit un = units.take(p);
        if (un.rows == 0 && !copy0) continue;
        float decay_rate = 0.0f;
        if constexpr (MODE == kLayer) decay_rate = expf(un.a_log);
        for (int r = 0; r < un.rows; ++r) {
            // A thread that gave up on a wait may not simply leave when the role synchronises below: the threads that got
            // through would wait for it at the role's barrier for ever.  There the decision is taken by all at that barrier.
            bool ready = mbar_wait(&raw_full[raw.idx], raw.phase, ctx, kStatusWaitRawFull);
            if (ready) ready = mbar_wait(&row_empty[row.idx], row.phase ^ 1u, ctx, kStatusWaitRowEmpty);
            if (!syncs && !ready) return;
            const unsigned char* in = smem + L::oRaw + raw.idx * L::kRawBytes;
            Cooked& ck = *reinterpret_cast<Cooked*>(smem + L::oCooked + row.idx * sizeof(Cooked));
            const long long gr = un.row0 + r;
            bool normalise = true;
            if (!ready) {
                // nothing to read: go to the vote
            } else if constexpr (MODE == kLayer) {
                // Short conv + SiLU, one bf16 rounding (kda.cu:129-142): channel c of q, k and v.
                const uint16_t* x = reinterpret_cast<const uint16_t*>(in + RawLayer::X);
                const uint16_t* w = reinterpret_cast<const uint16_t*>(in + RawLayer::W);
                for (int c = t; c < DK; c += kProThreads) {
#pragma unroll
                    for (int part = 0; part < 3; ++part) {
                        float acc = 0.0f;
#pragma unroll
                        for (int tap = 0; tap < TAPS; ++tap)
                            acc = acc + bf16_bits_to_f32(w[(part * DK + c) * TAPS + tap]) * bf16_bits_to_f32(x[(tap * 3 + part) * DK + c]);
                        const float act = bf16_round(acc / (1.0f + expf(-acc)));
                        if (part == 0) scratch[c] = act;
                        else if (part == 1) scratch[DK + c] = act;
                        else ck.v[c] = act;
                    }
                    // Decay multiplier (kda.cu:143-146) and sigmoid of the output gate (kda.cu:199-200).
                    const float a = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawLayer::A)[c]) +
                                    reinterpret_cast<const float*>(in + RawLayer::DTB)[c];
                    ck.g[c] = expf(p.lower * sigmoidf_(decay_rate * a));
                    ck.sg[c] = sigmoidf_(bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawLayer::GATE)[c]));
                }
                if (t == 0) {
                    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.P + gr * p.p_stride + p.b_off + un.h);
                    const uint16_t logit = *reinterpret_cast<const uint16_t*>(in + RawLayer::B + (addr & 15));
                    ck.beta = bf16_round(sigmoidf_(bf16_bits_to_f32(logit)));  // kda.cu:147-149
                }
            } else if constexpr (MODE == kCore) {
                normalise = (p.flags & GLM53F_KDA_CORE_L2NORM) != 0;
                for (int c = t; c < DK; c += kProThreads) {
                    const float qv = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawCore::Q)[c]);
                    const float kv = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawCore::K)[c]);
                    if (normalise) {
                        scratch[c] = qv;
                        scratch[DK + c] = kv;
                    } else {
                        ck.q[c] = qv;
                        ck.k[c] = kv;
                    }
                    ck.v[c] = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawCore::V)[c]);
                    ck.g[c] = expf(reinterpret_cast<const float*>(in + RawCore::GLOG)[c]);
                    if (p.G) ck.sg[c] = sigmoidf_(bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawCore::GATE)[c]));
                }
                if (t == 0) {
                    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.beta + gr * p.H + un.h);
                    ck.beta = *reinterpret_cast<const float*>(in + RawCore::B + (addr & 15));
                }
            } else {
                normalise = false;
                for (int c = t; c < DK; c += kProThreads) {
                    ck.k[c] = reinterpret_cast<const float*>(in + RawReplay::K)[c];
                    ck.g[c] = reinterpret_cast<const float*>(in + RawReplay::G)[c];
                    ck.v[c] = bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(in + RawReplay::V)[c]);
                }
                if (t == 0) {
                    const uintptr_t addr = reinterpret_cast<uintptr_t>(p.b_save + un.layer * p.b_stride + gr * p.H + un.h);
                    ck.beta = *reinterpret_cast<const float*>(in + RawReplay::B + (addr & 15));
                }
            }
            if (syncs) {
                if (!named_bar_all(1, kProThreads, ready)) return;
                if (warp == 0) l2norm_warp(scratch, ck.q, lane, true);
                else if (warp == 1) l2norm_warp(scratch + DK, ck.k, lane, false);
                named_bar_sync(2, kProThreads);  // scratch may be overwritten by the next row
            }
            mbar_arrive(&row_full[row.idx]);   // one arrival per prologue thread: every thread's writes are released
            mbar_arrive(&raw_empty[raw.idx]);
            raw.next(L::kRawSlots);
            row.next(L::kRowSlots);
        }
    }
}

// ---- the recurrence ------------------------------------------------------------------------------------------
template <typename S, int MODE>
__device__ void recurrence_role(const Params& p, unsigned char* smem, uint64_t* bars, const WaitCtx& ctx, int warp, int lane) {
    using L = Smem<S, MODE>;
    uint64_t* st_full = bars;
    uint64_t* st_empty = st_full + L::kStateSlots;
    uint64_t* row_full = st_empty + L::kStateSlots + 2 * L::kRawSlots;
    uint64_t* y_full = row_full + L::kRowSlots;
    uint64_t* row_empty = y_full + L::kRowSlots;
    Ring st, row;
    const bool copy0 = copies_state(p);
    UnitIter<MODE> units(p);
    while (units.valid()) {
        const Unit un = units.take(p);
        if (un.rows == 0 && !copy0) continue;
        if (!mbar_wait(&st_full[st.idx], st.phase, ctx, kStatusWaitStateFull)) return;
        unsigned char* slot = smem + L::oState + st.idx * L::kStateBytes;
        f32x2 s[kPairs][4];
        load_rows<S>(slot, warp, lane, s);
        const bool writes = p.state_out != nullptr;
        __syncwarp();  // the slot is free as soon as every lane's registers hold the state
        if (lane == 0) mbar_arrive(&st_empty[st.idx]);
        for (int r = 0; r < un.rows; ++r) {
            if (!mbar_wait(&row_full[row.idx], row.phase, ctx, kStatusWaitRowFull)) return;
            Cooked& ck = *reinterpret_cast<Cooked*>(smem + L::oCooked + row.idx * sizeof(Cooked));
            f32x2 kk[4], gg[4];
            {
                const float4 k4 = *reinterpret_cast<const float4*>(&ck.k[lane * 4]);
                const float4 g4 = *reinterpret_cast<const float4*>(&ck.g[lane * 4]);
                kk[0] = pack2(k4.x, k4.x); kk[1] = pack2(k4.y, k4.y); kk[2] = pack2(k4.z, k4.z); kk[3] = pack2(k4.w, k4.w);
                gg[0] = pack2(g4.x, g4.x); gg[1] = pack2(g4.y, g4.y); gg[2] = pack2(g4.z, g4.z); gg[3] = pack2(g4.w, g4.w);
            }
            delta_rule(s, kk, gg, ck.v, warp, lane, ck.beta, p.neg_zero2);
            if constexpr (MODE != kReplay) {
                // Read-out y = S q, rounded to bf16 (kda.cu:172-179).
                const float4 q4 = *reinterpret_cast<const float4*>(&ck.q[lane * 4]);
                const f32x2 qq[4] = {pack2(q4.x, q4.x), pack2(q4.y, q4.y), pack2(q4.z, q4.z), pack2(q4.w, q4.w)};
                const float o = rows_dot(s, qq, lane, p.neg_zero2);
                if ((lane & 3) == 0) ck.ys[warp * kRowsPerLane + (lane >> 2)] = bf16_round(o);
            }
            // A bf16 state is rounded after every row, after its read-out; after the last row the store rounds.
            if constexpr (sizeof(S) == 2) {
                if (r + 1 < un.rows || !writes) round_rows(s);
            }
            __syncwarp();
            if (lane == 0) {
                if (MODE != kReplay) mbar_arrive(&y_full[row.idx]);
                else mbar_arrive(&row_empty[row.idx]);
                if (warp == 0) atomicAdd(const_cast<uint32_t*>(ctx.progress), 1u);
            }
            row.next(L::kRowSlots);
        }
        if (writes) {
            // Straight from the registers: per row a lane stores its 4 consecutive elements (8 or 16 bytes), a warp a
            // whole contiguous row.  Each warp wrote nothing but the rows it read, so in place is safe.
            S* dst = reinterpret_cast<S*>(p.state_out) + un.s_elem;
            store_rows_global<S>(dst, warp, lane, s);
        }
        st.next(L::kStateSlots);
    }
}

// ---- the epilogue --------------------------------------------------------------------------------------------
template <typename S, int MODE>
__device__ void epilogue_role(const Params& p, unsigned char* smem, uint64_t* bars, const WaitCtx& ctx, int lane) {
    using L = Smem<S, MODE>;
    uint64_t* y_full = bars + 2 * L::kStateSlots + 2 * L::kRawSlots + L::kRowSlots;
    uint64_t* row_empty = y_full + L::kRowSlots;
    Ring row;
    const bool copy0 = copies_state(p);
    const bool gated = MODE == kLayer || p.G != nullptr;
    float nw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (gated)
#pragma unroll
        for (int i = 0; i < 4; ++i) nw[i] = bf16_bits_to_f32(p.norm_w[lane * 4 + i]);
    UnitIter<MODE> units(p);
    while (units.valid()) {
        const Unit un = units.take(p);
        if (un.rows == 0 && !copy0) continue;
        for (int r = 0; r < un.rows; ++r) {
            if (!mbar_wait(&y_full[row.idx], row.phase, ctx, kStatusWaitYFull)) return;
            const Cooked& ck = *reinterpret_cast<const Cooked*>(smem + L::oCooked + row.idx * sizeof(Cooked));
            const long long gr = un.row0 + r;
            float y[4];
            {
                const float4 y4 = *reinterpret_cast<const float4*>(&ck.ys[lane * 4]);
                y[0] = y4.x; y[1] = y4.y; y[2] = y4.z; y[3] = y4.w;
            }
            uint16_t o[4];
            if (gated) {  // kda.cu:188-201
                float ss = 0.0f;
#pragma unroll
                for (int i = 0; i < 4; ++i) ss = ss + y[i] * y[i];
                ss = butterfly1(ss);
                const float rinv = 1.0f / sqrtf(ss / (float)DV + p.eps);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float yn = y[i] * rinv;
                    const float yw = nw[i] * yn;
                    o[i] = f32_to_bf16_bits(yw * ck.sg[lane * 4 + i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = f32_to_bf16_bits(y[i]);
            }
            uint16_t* dst = p.out + gr * p.out_stride + (long long)un.h * DV + lane * 4;
            if ((reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
                *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)o[0] | ((uint32_t)o[1] << 16), (uint32_t)o[2] | ((uint32_t)o[3] << 16));
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) dst[i] = o[i];
            }
            if (p.k_save != nullptr) {  // kda.cu:181-186
                const long long base = (gr * p.H + un.h) * DK + lane * 4;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    p.k_save[base + i] = ck.k[lane * 4 + i];
                    p.g_save[base + i] = ck.g[lane * 4 + i];
                    p.v_save[base + i] = f32_to_bf16_bits(ck.v[lane * 4 + i]);
                }
                if (lane == 0) p.b_save[gr * p.H + un.h] = ck.beta;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&row_empty[row.idx]);
            row.next(L::kRowSlots);
        }
    }
}

// ---- the kernel ----------------------------------------------------------------------------------------------
template <typename S, int MODE>
__global__ void __launch_bounds__(kThreadsOf<MODE>, 1) recurrent_kernel(const __grid_constant__ Params p) {
    using L = Smem<S, MODE>;
    constexpr int kProWarps = kProWarpsOf<MODE>, kProThreads = kProThreadsOf<MODE>;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::oBars);
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + L::oCtl);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        uint64_t* b = bars;
        for (int i = 0; i < L::kStateSlots; ++i) mbar_init(b++, 1);                                // st_full
        for (int i = 0; i < L::kStateSlots; ++i) mbar_init(b++, kRecWarps);                        // st_empty
        for (int i = 0; i < L::kRawSlots; ++i) mbar_init(b++, 1);                                     // raw_full
        for (int i = 0; i < L::kRawSlots; ++i) mbar_init(b++, kProThreads);                           // raw_empty
        for (int i = 0; i < L::kRowSlots; ++i) mbar_init(b++, kProThreads);                           // row_full
        for (int i = 0; i < L::kRowSlots; ++i) mbar_init(b++, kRecWarps);                             // y_full
        for (int i = 0; i < L::kRowSlots; ++i) mbar_init(b++, MODE == kReplay ? kRecWarps : 1);       // row_empty
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    __syncthreads();
    // Programmatic dependent launch: let the next kernel of the stream be scheduled onto SMs as this grid's blocks
    // retire (its block set-up then overlaps this grid's tail), and do not touch global memory before every earlier
    // grid of the stream has completed and flushed.  Both are no-ops for a launch without the attribute.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const WaitCtx ctx{ctl, ctl + 1, &g_status, p.wait_limit_ns};
    if (warp < kRecWarps) {
        recurrence_role<S, MODE>(p, smem, bars, ctx, warp, lane);
    } else if (warp < kRecWarps + kProWarps) {
        prologue_role<S, MODE>(p, smem, bars, ctx, tid - kRecThreads);
    } else if (warp == kRecWarps + kProWarps) {
        if (MODE != kReplay) epilogue_role<S, MODE>(p, smem, bars, ctx, lane);
    } else {
        mover_role<S, MODE>(p, smem, bars, ctx, lane);
    }
    // No thread leaves while bulk loads into this block's shared memory may still be in flight: the mover issues a
    // load only after its consumers freed the slot, and every consumer role waits for every load before it ends,
    // except after an abort -- then give outstanding loads a bounded time to land.
    if (ctl[1]) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
    }
    __syncthreads();
}

// ---- the core step on many small blocks ------------------------------------------------------------------------
// The same arithmetic (delta_rule, rows_dot, round_rows: the bits are those of the kernel above and of the reference)
// for the core entry points without fused norms, arranged for few units: a block of four warps owns a QUARTER of a
// unit -- 32 of its 128 value rows, 8 a warp, which never interact with the others -- loads that part of the state
// straight from global memory into registers (a lane's four consecutive key channels of a row are 8 or 16 contiguous
// bytes, a warp's a whole row), cooks each row's inputs itself (128 threads, one channel each: widen q, k, v, exp of
// the log decay, beta), steps through the request's rows and stores its rows of the state back.  No rings, no bulk
// copies: with eight such blocks resident on an SM, and blocks handed out as SMs free up, the loads of some cover the
// arithmetic and stores of others, a launch's last blocks end within one small block's time of each other, and the
// next launch's blocks move in as room appears (programmatic dependent launch).  Used for the exact verify, whose 16
// serial rows a unit want many warps; for single-row decode the persistent kernel above streams faster.  (A variant
// without shared memory, every warp cooking its own lanes' pieces of a row as the replay below does, was slower: the
// sixteen warps of a unit each repeat the row's exponentials -- exact verify 12.0 against 11.1 ms, decode 3,567 GB/s.)
constexpr int kSmallWarps = 4, kSmallThreads = kSmallWarps * 32, kSmallParts = kRecWarps / kSmallWarps;

template <typename S>
__device__ __forceinline__ void load_rows_global(const S* head, int warp, int lane, f32x2 (&s)[kPairs][4]) {
    const bool vec = (reinterpret_cast<uintptr_t>(head) & (4 * sizeof(S) - 1)) == 0;
#pragma unroll
    for (int jp = 0; jp < kPairs; ++jp) {
        float x[2][4];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const S* src = head + (size_t)(warp * kRowsPerLane + 2 * jp + half) * DK + lane * 4;
            if constexpr (sizeof(S) == 4) {
                if (vec) {
                    const float4 v = *reinterpret_cast<const float4*>(src);
                    x[half][0] = v.x; x[half][1] = v.y; x[half][2] = v.z; x[half][3] = v.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) x[half][i] = src[i];
                }
            } else {
                uint32_t lo, hi;
                if (vec) {
                    const uint2 v = *reinterpret_cast<const uint2*>(src);
                    lo = v.x; hi = v.y;
                } else {
                    const uint16_t* u = reinterpret_cast<const uint16_t*>(src);
                    lo = (uint32_t)u[0] | ((uint32_t)u[1] << 16);
                    hi = (uint32_t)u[2] | ((uint32_t)u[3] << 16);
                }
                x[half][0] = __uint_as_float(lo << 16);
                x[half][1] = __uint_as_float(lo & 0xffff0000u);
                x[half][2] = __uint_as_float(hi << 16);
                x[half][3] = __uint_as_float(hi & 0xffff0000u);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) s[jp][i] = pack2(x[0][i], x[1][i]);
    }
}

template <typename S>
__global__ void __launch_bounds__(kSmallThreads, 8) core_small_kernel(const __grid_constant__ Params p) {
    __shared__ __align__(16) float sq[DK], sk[DK], sg[DK], sv[DV];
    __shared__ float sbeta;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const long long unit = blockIdx.x / kSmallParts;
    const int part = blockIdx.x % kSmallParts, uw = part * kSmallWarps + warp;  // this warp's place among the unit's 16
    const int b = (int)(unit / p.H), h = (int)(unit % p.H);
    const int r0 = p.cu_rows[b], rows = max(p.cu_rows[b + 1] - r0, 0);
    const bool writes = p.state_out != nullptr;
    if (rows == 0 && !copies_state(p)) return;
    const long long s_elem = p.state_off[b] + (long long)h * DV * DK;
    f32x2 s[kPairs][4];
    load_rows_global<S>(reinterpret_cast<const S*>(p.state_in) + s_elem, uw, lane, s);
    for (int r = 0; r < rows; ++r) {
        const long long gr = (long long)r0 + r, at = (gr * p.H + h) * DK + t;
        // The row's inputs, one channel a thread (the prologue of the kernel above for the core entry points).
        const float kf = bf16_bits_to_f32(p.k[at]), gf = expf(p.glog[at]);
        const uint16_t vb = p.v[at];
        sq[t] = bf16_bits_to_f32(p.q[at]);
        sk[t] = kf;
        sg[t] = gf;
        sv[t] = bf16_bits_to_f32(vb);
        float bt = 0.0f;
        if (t == 0) sbeta = bt = p.beta[gr * p.H + h];
        if (p.k_save != nullptr && part == 0) {
            p.k_save[at] = kf;
            p.g_save[at] = gf;
            p.v_save[at] = vb;
            if (t == 0) p.b_save[gr * p.H + h] = bt;
        }
        __syncthreads();
        f32x2 kk[4], gg[4];
        {
            const float4 k4 = *reinterpret_cast<const float4*>(&sk[lane * 4]);
            const float4 g4 = *reinterpret_cast<const float4*>(&sg[lane * 4]);
            kk[0] = pack2(k4.x, k4.x); kk[1] = pack2(k4.y, k4.y); kk[2] = pack2(k4.z, k4.z); kk[3] = pack2(k4.w, k4.w);
            gg[0] = pack2(g4.x, g4.x); gg[1] = pack2(g4.y, g4.y); gg[2] = pack2(g4.z, g4.z); gg[3] = pack2(g4.w, g4.w);
        }
        delta_rule(s, kk, gg, sv, uw, lane, sbeta, p.neg_zero2);
        const float4 q4 = *reinterpret_cast<const float4*>(&sq[lane * 4]);
        const f32x2 qq[4] = {pack2(q4.x, q4.x), pack2(q4.y, q4.y), pack2(q4.z, q4.z), pack2(q4.w, q4.w)};
        const float o = rows_dot(s, qq, lane, p.neg_zero2);
        if ((lane & 3) == 0) p.out[gr * p.out_stride + (long long)h * DV + uw * kRowsPerLane + (lane >> 2)] = f32_to_bf16_bits(o);
        if constexpr (sizeof(S) == 2) {
            if (r + 1 < rows || !writes) round_rows(s);
        }
        __syncthreads();  // the cooked row is overwritten by the next one
    }
    if (writes) store_rows_global<S>(reinterpret_cast<S*>(p.state_out) + s_elem, uw, lane, s);
}

template <typename S>
int launch_small(const Params& p, cudaStream_t stream) {
    Params q = p;
    q.neg_zero2 = 0x8000000080000000ull;
    static const bool pdl = [] {
        const char* v = getenv("GLM53F_KDA_PDL");
        return !(v && v[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.units * kSmallParts));
    cfg.blockDim = dim3(kSmallThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, core_small_kernel<S>, q);
}

// ---- the replay on many small blocks ---------------------------------------------------------------------------
// A commit replays keep[b] saved rows onto every (request, layer, head) state: no read-out, no norms, inputs that are
// already cooked.  Eight of a unit's value rows never interact with the others, and what a lane needs of a saved row is
// exactly a 16-byte piece of k and of the decay (its four key channels), one v and beta: so a WARP is the unit of work
// here -- no shared memory, no barrier, the next row's inputs loaded into registers while the current row's delta rule
// runs -- and 32 such warps are resident on an SM where the persistent kernel has one unit's 16.  Same delta_rule, same
// rounding points (a bf16 state is rounded after every row), so the bits are the persistent kernel's and the
// reference's.  Measured at 48 slots x 34 layers, accepted prefixes drawn from 0..16: 3.63 ms a commit against 4.71 ms.
struct ReplayRow {
    float4 k, g;
    float v, beta;
};
__device__ __forceinline__ ReplayRow replay_row(const Params& p, long long kv_base, long long b_base, long long gr, int h, int uw, int lane) {
    ReplayRow x;
    const long long at = kv_base + (gr * p.H + h) * DK;
    x.k = *reinterpret_cast<const float4*>(p.k_save + at + lane * 4);
    x.g = *reinterpret_cast<const float4*>(p.g_save + at + lane * 4);
    x.v = bf16_bits_to_f32(p.v_save[at + uw * kRowsPerLane + (lane >> 2)]);
    x.beta = p.b_save[b_base + gr * p.H + h];
    return x;
}

template <typename S>
__global__ void __launch_bounds__(kSmallThreads, sizeof(S) == 4 ? 6 : 8) replay_small_kernel(const __grid_constant__ Params p) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const long long unit = blockIdx.x / kSmallParts;
    const int uw = (int)(blockIdx.x % kSmallParts) * kSmallWarps + warp;  // this warp's place among the unit's 16
    const int h = (int)(unit % p.H), layer = (int)((unit / p.H) % p.layers), b = (int)(unit / ((long long)p.H * p.layers));
    const long long r0 = p.cu_rows ? p.cu_rows[b] : 0;
    int rows = p.keep ? p.keep[b] : p.rows1;
    if (rows < 0) rows = 0;
    if (rows == 0 && !copies_state(p)) return;
    const long long s_elem = (long long)layer * p.state_stride + (p.state_off ? p.state_off[b] : 0) + (long long)h * DV * DK;
    const long long kv_base = (long long)layer * p.kv_stride, b_base = (long long)layer * p.b_stride;
    f32x2 s[kPairs][4];
    load_rows_global<S>(reinterpret_cast<const S*>(p.state_in) + s_elem, uw, lane, s);
    ReplayRow cur{};
    if (rows > 0) cur = replay_row(p, kv_base, b_base, r0, h, uw, lane);
    for (int r = 0; r < rows; ++r) {
        ReplayRow nxt = cur;
        if (r + 1 < rows) nxt = replay_row(p, kv_base, b_base, r0 + r + 1, h, uw, lane);
        const f32x2 kk[4] = {pack2(cur.k.x, cur.k.x), pack2(cur.k.y, cur.k.y), pack2(cur.k.z, cur.k.z), pack2(cur.k.w, cur.k.w)};
        const f32x2 gg[4] = {pack2(cur.g.x, cur.g.x), pack2(cur.g.y, cur.g.y), pack2(cur.g.z, cur.g.z), pack2(cur.g.w, cur.g.w)};
        delta_rule_v(s, kk, gg, cur.v, lane, cur.beta, p.neg_zero2);
        if constexpr (sizeof(S) == 2) {
            if (r + 1 < rows) round_rows(s);  // the last row's rounding is the store's
        }
        cur = nxt;
    }
    store_rows_global<S>(reinterpret_cast<S*>(p.state_out) + s_elem, uw, lane, s);
}

template <typename S>
int launch_replay_small(const Params& p, cudaStream_t stream) {
    Params q = p;
    q.neg_zero2 = 0x8000000080000000ull;
    static const bool pdl = [] {
        const char* v = getenv("GLM53F_KDA_PDL");
        return !(v && v[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(p.units * kSmallParts));
    cfg.blockDim = dim3(kSmallThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, replay_small_kernel<S>, q);
}

template <typename S, int MODE>
int launch(const Params& p, cudaStream_t stream) {
    using L = Smem<S, MODE>;
    static bool configured = false;  // per process; the attribute is per device, so set it on every device change
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured || configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(recurrent_kernel<S, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
        if (e != cudaSuccess) return (int)e;
        configured = true;
        configured_dev = dev;
    }
    const long long sms = sm_count();
    const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
    Params q = p;
    q.neg_zero2 = 0x8000000080000000ull;
    q.wait_limit_ns = g_wait_limit_ns;
    q.skip_first_state = g_skip_first_state;
    g_skip_first_state = 0;
    // Launched with programmatic stream serialization: the kernel itself waits for its predecessors before its first
    // global access, so ordering is what a plain launch gives.  GLM53F_KDA_PDL=0 selects a plain launch.
    static const bool pdl = [] {
        const char* v = getenv("GLM53F_KDA_PDL");
        return !(v && v[0] == '0');
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreadsOf<MODE>);
    cfg.dynamicSmemBytes = L::kBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, recurrent_kernel<S, MODE>, q);
}

template <int MODE>
int launch_typed(const Params& p, bool bf16_state, cudaStream_t stream) {
    return bf16_state ? launch<__nv_bfloat16, MODE>(p, stream) : launch<float, MODE>(p, stream);
}

bool saves_ok(const void* k, const void* v, const void* g, const void* b) {
    const int n = (k != nullptr) + (v != nullptr) + (g != nullptr) + (b != nullptr);
    return n == 0 || n == 4;
}

// Reference kda.cu:290-299, 310-312, 329-332.
int chain_entry(int32_t heads, int32_t batch, bool batched, const int32_t* cu_rows, const int32_t* keep, int32_t rows, const glm53f_bf16* p,
                int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                int64_t g_stride, const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w,
                const void* state_in, void* state_out, const int64_t* state_off, bool bf16_state, const float* a_log,
                const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower, glm53f_bf16* out,
                int64_t out_stride, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save,
                glm53f_stream_t stream) {
    if (heads < 1 || heads > 65535) return kInvalid;
    if (!p || !a || !g || !conv || !conv_w || !state_in || !a_log || !dt_bias || !norm_w || !out) return kInvalid;
    if (!saves_ok(k_save, v_save, g_save, b_save)) return kInvalid;
    if (batched) {
        if (batch < 1 || batch > 65535 || !cu_rows || !conv_off || !state_off) return kInvalid;
    } else if (rows < 1) {
        return kInvalid;
    }
    if (batched && bf16_state && state_out == nullptr && k_save != nullptr && keep == nullptr && g_layer_verify_mode.load() == 1) {
        // The chunked form of a verify call: eligible when every row the two kernels touch by vector is aligned; any
        // other call runs the exact form below.
        auto al = [](const void* x, int bytes) { return (reinterpret_cast<uintptr_t>(x) & (bytes - 1)) == 0; };
        if (al(p, 8) && al(a, 8) && al(g, 8) && al(conv, 8) && al(conv_w, 16) && al(dt_bias, 16) && al(out, 16) && al(k_save, 16) && al(v_save, 16) &&
            al(g_save, 16) && al(state_in, 16) && p_stride % 4 == 0 && a_stride % 4 == 0 && g_stride % 4 == 0 && out_stride % 8 == 0) {
            cudaStream_t st = (cudaStream_t)stream;
            const int rc = verify_prologue_launch(heads, batch, cu_rows, p, p_stride, b_off, a, a_stride, conv, conv_off, conv_w, a_log, dt_bias,
                                                  lower, out, out_stride, k_save, v_save, g_save, b_save, st);
            if (rc != 0) return rc;
            return layer_verify_tc_launch(heads, batch, cu_rows, state_in, state_off, g, g_stride, norm_w, eps, out, out_stride, k_save, v_save,
                                          g_save, b_save, st);
        }
    }
    Params q{};
    q.H = heads;
    q.layers = 1;
    q.units = (long long)heads * batch;
    q.cu_rows = cu_rows;
    q.keep = keep;
    q.rows1 = rows;
    q.P = p; q.p_stride = p_stride; q.b_off = b_off;
    q.A = a; q.a_stride = a_stride;
    q.G = g; q.g_stride = g_stride;
    q.conv = conv; q.conv_off = reinterpret_cast<const long long*>(conv_off); q.cw = conv_w;
    q.a_log = a_log; q.dt_bias = dt_bias; q.norm_w = norm_w; q.eps = eps; q.lower = lower;
    q.state_in = state_in; q.state_out = state_out; q.state_stride = 0;
    q.state_off = reinterpret_cast<const long long*>(state_off);
    q.out = out; q.out_stride = out_stride;
    q.k_save = k_save; q.v_save = v_save; q.g_save = g_save; q.b_save = b_save;
    return launch_typed<kLayer>(q, bf16_state, (cudaStream_t)stream);
}

// Reference kda.cu:381-383, 412, 424.
int replay_entry(int32_t heads, int32_t layers, int32_t batch, bool batched, const int32_t* cu_rows, const int32_t* keep,
                 int32_t rows, const void* state_in, void* state_out, int64_t state_stride, const int64_t* state_off,
                 bool bf16_state, const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                 const float* b_save, int64_t kv_stride, int64_t b_stride, glm53f_stream_t stream) {
    if (batched && (!cu_rows || !keep || !state_off)) return kInvalid;
    if (heads < 1 || layers < 1 || batch < 1 || batch > 65535 || (long long)heads * layers > 0x7fffffffLL || !state_in ||
        !state_out || !k_save || !v_save || !g_save || !b_save || rows < 0)
        return kInvalid;
    Params q{};
    q.H = heads;
    q.layers = layers;
    q.units = (long long)heads * layers * batch;
    q.cu_rows = cu_rows;
    q.keep = keep;
    q.rows1 = rows;
    q.state_in = state_in; q.state_out = state_out; q.state_stride = state_stride;
    q.state_off = reinterpret_cast<const long long*>(state_off);
    q.k_save = const_cast<float*>(k_save); q.v_save = const_cast<glm53f_bf16*>(v_save);
    q.g_save = const_cast<float*>(g_save); q.b_save = const_cast<float*>(b_save);
    q.kv_stride = kv_stride; q.b_stride = b_stride;
    if (bf16_state && g_commit_mode.load() == 1)
        return commit_tc_launch(heads, layers, batch, cu_rows, keep, rows, state_in, state_out, state_stride, state_off, k_save, v_save, g_save,
                                b_save, kv_stride, b_stride, (cudaStream_t)stream);
    // The warp-per-eight-rows kernel takes aligned saves and grids that fit; GLM53F_KDA_REPLAY=pipeline keeps the
    // persistent kernel.
    static const bool small = [] {
        const char* e = getenv("GLM53F_KDA_REPLAY");
        return !(e != nullptr && strcmp(e, "pipeline") == 0);
    }();
    auto al16 = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (small && al16(k_save) && al16(g_save) && kv_stride % 4 == 0 && q.units * kSmallParts <= 0x7fffffffLL)
        return bf16_state ? launch_replay_small<__nv_bfloat16>(q, (cudaStream_t)stream) : launch_replay_small<float>(q, (cudaStream_t)stream);
    return launch_typed<kReplay>(q, bf16_state, (cudaStream_t)stream);
}

int core_entry(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q, const glm53f_bf16* k,
               const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, void* state_out,
               const int64_t* state_off, int32_t state_bf16, int32_t flags, const glm53f_bf16* gate,
               const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, float* k_save, glm53f_bf16* v_save,
               float* g_save, float* b_save, glm53f_stream_t stream) {
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535) return kInvalid;
    if (!cu_rows || !q || !k || !v || !g || !beta || !state_in || !state_off || !out) return kInvalid;
    if (gate && !norm_w) return kInvalid;
    if (flags & ~(GLM53F_KDA_CORE_L2NORM | GLM53F_KDA_CORE_TENSOR)) return kInvalid;
    if (!saves_ok(k_save, v_save, g_save, b_save)) return kInvalid;
    if (flags & GLM53F_KDA_CORE_TENSOR) {
        // The chunked verify takes read-only bf16 states, inputs as given (no fused norms) and aligned rows; any other
        // call runs the exact form, whose results are always valid.
        auto al = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
        if (state_bf16 != 0 && state_out == nullptr && gate == nullptr && !(flags & GLM53F_KDA_CORE_L2NORM) && al(q) && al(k) && al(v) && al(g))
            return core_verify_tc_launch(heads, batch, cu_rows, q, k, v, g, beta, state_in, state_off, out, k_save, v_save, g_save, b_save,
                                         (cudaStream_t)stream);
        flags &= ~GLM53F_KDA_CORE_TENSOR;
    }
    Params x{};
    x.H = heads;
    x.layers = 1;
    x.units = (long long)heads * batch;
    x.cu_rows = cu_rows;
    x.q = q; x.k = k; x.v = v; x.glog = g; x.beta = beta; x.flags = flags;
    x.G = gate; x.norm_w = norm_w; x.eps = eps;
    x.state_in = state_in; x.state_out = state_out;
    x.state_off = reinterpret_cast<const long long*>(state_off);
    x.out = out; x.out_stride = (long long)heads * DV;
    x.k_save = k_save; x.v_save = v_save; x.g_save = g_save; x.b_save = b_save;
    // The exact verify (saves requested, inputs used as given, no fused output norm) runs on the small-block kernel: 16
    // serial rows a unit are bound by instruction issue, and 32 resident warps an SM issue more than the persistent
    // kernel's 16 (11.1 against 12.3 ms per step of 48 slots x 16 rows x 34 layers).  Single-row decode stays on the
    // persistent kernel, which streams faster (4,263 against 3,500 GB/s at 16 slots: small blocks keep too few bytes in
    // flight).  GLM53F_KDA_DECODE=pipeline / small forces one or the other; the bits are the same either way.
    static const int forced = [] {
        const char* e = getenv("GLM53F_KDA_DECODE");
        return e == nullptr ? 0 : (strcmp(e, "pipeline") == 0 ? 1 : (strcmp(e, "small") == 0 ? 2 : 0));
    }();
    const bool small = forced == 2 || (forced == 0 && k_save != nullptr);
    if (small && flags == 0 && gate == nullptr && x.units * kSmallParts <= 0x7fffffffll)
        return state_bf16 != 0 ? launch_small<__nv_bfloat16>(x, (cudaStream_t)stream) : launch_small<float>(x, (cudaStream_t)stream);
    return launch_typed<kCore>(x, state_bf16 != 0, (cudaStream_t)stream);
}

}  // namespace

int layer_chain_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t rows, const glm53f_bf16* p,
                       int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                       int64_t g_stride, const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w,
                       const void* state_in, void* state_out, const int64_t* state_off, bool bf16_state,
                       const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower,
                       glm53f_bf16* out, int64_t out_stride, cudaStream_t stream) {
    Params q{};
    q.H = heads;
    q.layers = 1;
    q.units = (long long)heads * batch;
    q.cu_rows = cu_rows;
    q.rows1 = rows;
    q.P = p; q.p_stride = p_stride; q.b_off = b_off;
    q.A = a; q.a_stride = a_stride;
    q.G = g; q.g_stride = g_stride;
    q.conv = conv; q.conv_off = reinterpret_cast<const long long*>(conv_off); q.cw = conv_w;
    q.a_log = a_log; q.dt_bias = dt_bias; q.norm_w = norm_w; q.eps = eps; q.lower = lower;
    q.state_in = state_in; q.state_out = state_out;
    q.state_off = reinterpret_cast<const long long*>(state_off);
    q.out = out; q.out_stride = out_stride;
    return launch_typed<kLayer>(q, bf16_state, stream);
}

int core_chain_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q, const glm53f_bf16* k,
                      const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, void* state_out,
                      const int64_t* state_off, bool bf16_state, int32_t flags, const glm53f_bf16* gate,
                      const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, cudaStream_t stream) {
    return core_entry(heads, batch, cu_rows, q, k, v, g, beta, state_in, state_out, state_off, bf16_state ? 1 : 0, flags, gate,
                      norm_w, eps, out, nullptr, nullptr, nullptr, nullptr, (glm53f_stream_t)stream);
}

}  // namespace kda

using namespace kda;

extern "C" int glm53f_kda_chain(int32_t heads, int32_t rows, const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g, int64_t g_stride,
                                const glm53f_bf16* conv, const glm53f_bf16* conv_w, const float* state_in,
                                float* state_out, const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                                float eps, float lower, glm53f_bf16* out, int64_t out_stride, float* k_save,
                                glm53f_bf16* v_save, float* g_save, float* b_save, glm53f_stream_t stream) {
    return chain_entry(heads, 1, false, nullptr, nullptr, rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, nullptr, conv_w,
                       state_in, state_out, nullptr, false, a_log, dt_bias, norm_w, eps, lower, out, out_stride, k_save,
                       v_save, g_save, b_save, stream);
}

extern "C" int glm53f_kda_chain_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* p,
                                      int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride,
                                      const glm53f_bf16* g, int64_t g_stride, const glm53f_bf16* conv,
                                      const int64_t* conv_off, const glm53f_bf16* conv_w, const float* state_in,
                                      float* state_out, const int64_t* state_off, const float* a_log,
                                      const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower,
                                      glm53f_bf16* out, int64_t out_stride, float* k_save, glm53f_bf16* v_save,
                                      float* g_save, float* b_save, glm53f_stream_t stream) {
    return chain_entry(heads, batch, true, cu_rows, nullptr, 0, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off,
                       conv_w, state_in, state_out, state_off, false, a_log, dt_bias, norm_w, eps, lower, out,
                       out_stride, k_save, v_save, g_save, b_save, stream);
}

extern "C" int glm53f_kda_chain_batch_bf16state(int32_t heads, int32_t batch, const int32_t* cu_rows,
                                                const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                                const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                                                int64_t g_stride, const glm53f_bf16* conv, const int64_t* conv_off,
                                                const glm53f_bf16* conv_w, const glm53f_bf16* state_in,
                                                glm53f_bf16* state_out, const int64_t* state_off, const float* a_log,
                                                const float* dt_bias, const glm53f_bf16* norm_w, float eps,
                                                float lower, glm53f_bf16* out, int64_t out_stride, float* k_save,
                                                glm53f_bf16* v_save, float* g_save, float* b_save,
                                                glm53f_stream_t stream) {
    return chain_entry(heads, batch, true, cu_rows, nullptr, 0, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off,
                       conv_w, state_in, state_out, state_off, true, a_log, dt_bias, norm_w, eps, lower, out, out_stride,
                       k_save, v_save, g_save, b_save, stream);
}

extern "C" int glm53f_kda_chain_commit_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, const int32_t* keep,
                                             const glm53f_bf16* p, int64_t p_stride, int64_t b_off, const glm53f_bf16* a,
                                             int64_t a_stride, const glm53f_bf16* g, int64_t g_stride, const glm53f_bf16* conv,
                                             const int64_t* conv_off, const glm53f_bf16* conv_w, void* state,
                                             const int64_t* state_off, int32_t state_bf16, const float* a_log,
                                             const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower,
                                             glm53f_bf16* out, int64_t out_stride, glm53f_stream_t stream) {
    if (!keep || !state) return kInvalid;
    return chain_entry(heads, batch, true, cu_rows, keep, 0, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off, conv_w,
                       state, state, state_off, state_bf16 != 0, a_log, dt_bias, norm_w, eps, lower, out, out_stride, nullptr,
                       nullptr, nullptr, nullptr, stream);
}

extern "C" int glm53f_kda_replay(int32_t heads, int32_t rows, const float* state_in, float* state_out,
                                 const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                                 const float* b_save, glm53f_stream_t stream) {
    return replay_entry(heads, 1, 1, false, nullptr, nullptr, rows, state_in, state_out, 0, nullptr, false, k_save,
                        v_save, g_save, b_save, 0, 0, stream);
}

extern "C" int glm53f_kda_replay_layers(int32_t heads, int32_t layers, int32_t rows, const float* state_in,
                                        float* state_out, int64_t state_stride, const float* k_save,
                                        const glm53f_bf16* v_save, const float* g_save, const float* b_save,
                                        int64_t kv_stride, int64_t b_stride, glm53f_stream_t stream) {
    return replay_entry(heads, layers, 1, false, nullptr, nullptr, rows, state_in, state_out, state_stride, nullptr,
                        false, k_save, v_save, g_save, b_save, kv_stride, b_stride, stream);
}

extern "C" int glm53f_kda_replay_batch(int32_t heads, int32_t layers, int32_t batch, const int32_t* cu_rows,
                                       const int32_t* keep, const float* state_in, float* state_out,
                                       int64_t state_stride, const int64_t* state_off, const float* k_save,
                                       const glm53f_bf16* v_save, const float* g_save, const float* b_save,
                                       int64_t kv_stride, int64_t b_stride, glm53f_stream_t stream) {
    return replay_entry(heads, layers, batch, true, cu_rows, keep, 0, state_in, state_out, state_stride, state_off, false,
                        k_save, v_save, g_save, b_save, kv_stride, b_stride, stream);
}

extern "C" int glm53f_kda_replay_batch_bf16state(int32_t heads, int32_t layers, int32_t batch, const int32_t* cu_rows,
                                                 const int32_t* keep, const glm53f_bf16* state_in,
                                                 glm53f_bf16* state_out, int64_t state_stride,
                                                 const int64_t* state_off, const float* k_save,
                                                 const glm53f_bf16* v_save, const float* g_save, const float* b_save,
                                                 int64_t kv_stride, int64_t b_stride, glm53f_stream_t stream) {
    return replay_entry(heads, layers, batch, true, cu_rows, keep, 0, state_in, state_out, state_stride, state_off, true,
                        k_save, v_save, g_save, b_save, kv_stride, b_stride, stream);
}

extern "C" int glm53f_kda_core_decode_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q,
                                            const glm53f_bf16* k, const glm53f_bf16* v, const float* g,
                                            const float* beta, const void* state_in, void* state_out,
                                            const int64_t* state_off, int32_t state_bf16, int32_t flags,
                                            const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                            glm53f_bf16* out, glm53f_stream_t stream) {
    return core_entry(heads, batch, cu_rows, q, k, v, g, beta, state_in, state_out, state_off, state_bf16, flags, gate,
                      norm_w, eps, out, nullptr, nullptr, nullptr, nullptr, stream);
}

extern "C" int glm53f_kda_core_verify_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q,
                                            const glm53f_bf16* k, const glm53f_bf16* v, const float* g,
                                            const float* beta, const void* state_in, void* state_out,
                                            const int64_t* state_off, int32_t state_bf16, int32_t flags,
                                            const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                            glm53f_bf16* out, float* k_save, glm53f_bf16* v_save, float* g_save,
                                            float* b_save, glm53f_stream_t stream) {
    return core_entry(heads, batch, cu_rows, q, k, v, g, beta, state_in, state_out, state_off, state_bf16, flags, gate,
                      norm_w, eps, out, k_save, v_save, g_save, b_save, stream);
}

extern "C" int glm53f_kda_core_commit_batch(int32_t heads, int32_t layers, int32_t batch, const int32_t* cu_rows,
                                            const int32_t* keep, const void* state_in, void* state_out,
                                            int64_t state_stride, const int64_t* state_off, int32_t state_bf16,
                                            const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                                            const float* b_save, int64_t kv_stride, int64_t b_stride,
                                            glm53f_stream_t stream) {
    return replay_entry(heads, layers, batch, true, cu_rows, keep, 0, state_in, state_out, state_stride, state_off,
                        state_bf16 != 0, k_save, v_save, g_save, b_save, kv_stride, b_stride, stream);
}

int* kda::status_word() {
    int* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

extern "C" int glm53f_kda_device_status(void) {
    int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    e = cudaMemcpyFromSymbol(&v, g_status, sizeof v);
    if (e != cudaSuccess) return (int)e;
    if (v != 0) cudaMemcpyToSymbol(g_status, &zero, sizeof zero);
    return v;
}

extern "C" int32_t glm53f_kda_verify_mode(int32_t mode) {
    const int prev = kda::g_layer_verify_mode.load();
    if (mode == 0 || mode == 1) kda::g_layer_verify_mode.store(mode);
    return prev;
}

extern "C" int32_t glm53f_kda_commit_mode(int32_t mode) {
    const int prev = kda::g_commit_mode.load();
    if (mode == 0 || mode == 1) kda::g_commit_mode.store(mode);
    return prev;
}

extern "C" int glm53f_kda_debug_wait_test(uint64_t wait_limit_ns, int32_t skip_first_state) {
    if (wait_limit_ns != 0 && (wait_limit_ns < 100000ull || wait_limit_ns > 60000000000ull)) return kda::kInvalid;  // 0.1 ms .. 60 s
    kda::g_wait_limit_ns = wait_limit_ns == 0 ? kda::kWaitLimitNs : wait_limit_ns;
    kda::g_skip_first_state = skip_first_state != 0 ? 1 : 0;
    return 0;
}
