// The projections either side of the KDA core as a tcgen05 GEMM: out[g][r][o] = sum_k x[g][r][k] * w[g][o][k], bf16
// operands, f32 accumulation in tensor memory, bf16 or f32 results.
//
// What it stands in for: the reference's Gemm::bf16 (crates/glm53f-forward/src/gemm.rs:212-235), which sends up to 8
// rows to its CUDA-core GEMV (kernels/glm53f_forward.h:19-40) and more rows to cuBLAS, at the call sites of a KDA
// layer (crates/glm53f-forward/src/forward.rs:3494-3542: the fused [q|k|v|b] projection 4096 -> 24,640 and the
// low-rank gate pair 4096 -> 256 -> 2 x 8192; 3772-3790: o_proj 8192 -> 4096).
//
// Shape of the kernel.  The weight is the M operand: a tile is 128 output features x NR activation rows, NR in
// {16, 32, 64, 128, 256} chosen from the row count, so a decode step's 16 rows waste nothing and the weight -- which
// dominates the traffic at few rows (202 MB for the fused projection) -- streams through once.  Both operands are
// K-major in global memory ([o][k] and [r][k]), so tiled tensor copies in the 128-byte swizzle feed tcgen05.mma
// in place: a stage is 64 k of the weight tile (16 KiB) and of the row tile (NR x 128 bytes).  Roles per block:
//   warp 0  producer: tensor copies into a ring of stages, each completing a stage's mbarrier;
//   warp 1  one elected thread issues 4 MMAs (K = 16) per stage and commits the stage back to the producer, and the
//           tile's accumulator to the epilogue when its last stage is in; owns the TMEM allocation;
//   warps 2-5  epilogue: tcgen05.ld of the finished accumulator (lane = feature, column = row), convert, store.
// Two accumulators alternate, so the epilogue of a tile overlaps the MMAs of the next; blocks walk the tile list with
// the row tile fastest (blocks that run together share a weight tile in L2).  With NR <= 128 a block stays under
// 113 KiB of shared memory so that two fit an SM and every tile of a decode-size launch is in flight at once
// (measured for the fused projection at 16 rows, 193 tiles: 38 us so, 48 us with one deeper-ringed block per SM).
//
// A row's result depends on that row's inputs and on (n, k) only -- the accumulation order over k is fixed by the
// stage loop -- never on how many rows the launch has or which NR it picked (tests hold this bitwise).
//
// Few tiles (o_proj at decode: 32 feature tiles of k = 8192) would leave most SMs idle: there the k range of a tile is
// split over the blocks of a thread-block cluster, each with its own accumulator, and rank 0 adds the partial tiles
// in rank order through distributed shared memory (no scratch in global memory, the same bits every run).
//
// Every wait is bounded (codes 130-135 in the device status word); TMEM is freed on every path; every block of a
// cluster reaches the closing cluster barrier on every path.

#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "glm53f_proj.h"
#include "kda_internal.h"
#include "tc.cuh"

namespace kda {

// proj_gemm_pair.cu: 256 x 256 tiles on SM pairs, for launches with many rows.
int proj_gemm_pair_launch(const CUtensorMap& tm_w, int w_swapped, const CUtensorMap& tm_x, int x_swapped, void* out, long long ldo, long long o_gstride,
                          int groups, int rows, int n, int k, int out_f32, int* status, cudaStream_t stream);

namespace {

constexpr int kBM = 128;            // output features per tile (UMMA M)
constexpr int kBK = 64;             // k per stage: one 128-byte swizzle row of bf16
constexpr int kGemmThreads = 192;   // producer, MMA, 4 epilogue warps
constexpr int kEpiThreads = 128;
constexpr int kABytes = kBM * 128;  // a stage's weight tile

enum : int { kStatusGemmEmpty = 130, kStatusGemmFull = 131, kStatusGemmAccFull = 132, kStatusGemmAccEmpty = 133, kStatusGemmRedFull = 134, kStatusGemmRedEmpty = 135 };

template <int NR, bool SPLIT>
struct Cfg {
    static constexpr int kBBytes = NR * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = SPLIT ? (NR == 16 ? 5 : NR == 32 ? 4 : NR == 64 ? 3 : 4) : (NR == 16 ? 6 : NR == 32 ? 5 : NR == 64 ? 4 : NR == 128 ? 3 : 4);
    static constexpr int kTmemCols = 2 * NR < 32 ? 32 : 2 * NR;
    static constexpr int kRedBytes = SPLIT ? kBM * NR * 4 : 0;  // this block's partial tile, f32 [128][NR]
    static constexpr int oRed = kStages * kStageBytes;
    static constexpr int oBars = oRed + kRedBytes;  // full[S], empty[S], acc_full[2], acc_empty[2], red_full, red_empty
    static constexpr int oCtl = oBars + (2 * kStages + 6) * 8;
    static constexpr int kBytes = oCtl + 16 + 1024;      // + slack to align the stages to 1024 bytes
    static constexpr int kBlocksPerSm = (NR <= 64 || (NR == 128 && !SPLIT)) ? 2 : 1;
};

struct GemmParams {
    CUtensorMap tm_w, tm_x;
    void* out;
    long long ldo, o_gstride;
    int rows, n, kblocks, out_f32;
    int n_tiles, r_tiles;
    int w_swapped, x_swapped;  // the map's coordinates are (k, group, row) instead of (k, row, group)
    long long tiles;
    int* status;
};

// ---- thread-block clusters: the K splits of a tile are the blocks of one cluster --------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tensormap(const void* tmap) { asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory"); }
// Programmatic dependent launch: the next kernel of the stream may be scheduled once every block has said so, and a
// block touches nothing an earlier kernel may still write (or read, where this kernel writes) before grid_dependency_wait.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of this block's shared-memory location `local` in block `rank` of the cluster.
__device__ __forceinline__ uint32_t peer_smem(const void* local, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
    return ra;
}
__device__ __forceinline__ void peer_mbar_arrive(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }

__device__ __forceinline__ float4 peer_load4(uint32_t remote_addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote_addr) : "memory");
    return v;
}

// KS = blocks per cluster = K splits of a tile (1: no cluster).
template <int NR, int KS>
__global__ void __launch_bounds__(kGemmThreads, Cfg<NR, (KS > 1)>::kBlocksPerSm) proj_gemm_kernel(const __grid_constant__ GemmParams p) {
    constexpr bool SPLIT = KS > 1;
    using C = Cfg<NR, SPLIT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::oBars);
    uint64_t* empty = full + C::kStages;
    uint64_t* acc_full = empty + C::kStages;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* red_full = acc_empty + 2;   // rank 0: every peer's partial is in its buffer
    uint64_t* red_empty = red_full + 1;   // peers: rank 0 has read the partial
    constexpr uint32_t ks = KS;
    const uint32_t kr = SPLIT ? cluster_rank() : 0u;
    const long long tile0 = blockIdx.x / ks, tile_step = gridDim.x / ks;
    const int kb_n = p.kblocks / (int)ks, kb0 = (int)kr * kb_n;
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + C::oCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < C::kStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], kEpiThreads / 32);
        }
        mbar_init(red_full, ks > 1 ? (ks - 1) * (kEpiThreads / 32) : 1);
        mbar_init(red_empty, kEpiThreads / 32);
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, C::kTmemCols);
    if (tid == 0) {
        prefetch_tensormap(&p.tm_w);
        prefetch_tensormap(&p.tm_x);
    }
    tc::fence_before_sync();
    __syncthreads();
    // Every block's barriers exist before a peer arrives on one: the blocks say so here and check it only before their
    // first remote arrival (the end of their first tile), so nobody stands still at the start.
    if (SPLIT) cluster_arrive();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const WaitCtx ctx{ctl, ctl + 1, p.status};
    launch_dependents();
    bool opened = !SPLIT;  // whether this thread has completed the opening cluster barrier
    grid_dependency_wait();  // before the first global access: an earlier kernel may be writing the weight or the rows

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (long long t = tile0; t < p.tiles; t += tile_step) {
                const int rt = (int)(t % p.r_tiles);
                const long long u = t / p.r_tiles;
                const int nt = (int)(u % p.n_tiles), g = (int)(u / p.n_tiles);
                for (int kb = kb0; kb < kb0 + kb_n; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, ctx, kStatusGemmEmpty)) goto done;
                    unsigned char* st = smem + s * C::kStageBytes;
                    mbar_arrive_expect_tx(&full[s], C::kStageBytes);
                    if (p.w_swapped) tensor_load_3d(st, &p.tm_w, kb * kBK, g, nt * kBM, &full[s]);
                    else tensor_load_3d(st, &p.tm_w, kb * kBK, nt * kBM, g, &full[s]);
                    if (p.x_swapped) tensor_load_3d(st + kABytes, &p.tm_x, kb * kBK, g, rt * NR, &full[s]);
                    else tensor_load_3d(st + kABytes, &p.tm_x, kb * kBK, rt * NR, g, &full[s]);
                    if (++s == C::kStages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16(kBM, NR, 0, 0, 0);
            int s = 0, buf = 0;
            uint32_t ph = 0, acc_ph[2] = {0, 0};
            for (long long t = tile0; t < p.tiles; t += tile_step) {
                if (!mbar_wait(&acc_empty[buf], acc_ph[buf] ^ 1u, ctx, kStatusGemmAccEmpty)) goto done;
                tc::fence_after_sync();
                const uint32_t d = tm + (uint32_t)(buf * NR);
                for (int kb = 0; kb < kb_n; ++kb) {
                    if (!mbar_wait(&full[s], ph, ctx, kStatusGemmFull)) goto done;
                    tc::fence_after_sync();
                    const unsigned char* st = smem + s * C::kStageBytes;
#pragma unroll
                    for (int i = 0; i < kBK / 16; ++i)
                        tc::mma_bf16(d, tc::desc_sw128_kmajor(st, kBM, 16 * i), tc::desc_sw128_kmajor(st + kABytes, NR, 16 * i), idesc, kb > 0 || i > 0);
                    tc::mma_commit(&empty[s]);
                    if (++s == C::kStages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                tc::mma_commit(&acc_full[buf]);
                acc_ph[buf] ^= 1u;
                buf ^= 1;
                ctl[0] = ctl[0] + 1u;
            }
        }
    } else {
        const int q = warp & 3;  // the TMEM lane quarter this warp may read
        int buf = 0;
        uint32_t acc_ph[2] = {0, 0}, red_ph = 0;
        for (long long t = tile0; t < p.tiles; t += tile_step) {
            const int rt = (int)(t % p.r_tiles);
            const long long u = t / p.r_tiles;
            const int nt = (int)(u % p.n_tiles), g = (int)(u / p.n_tiles);
            if (!mbar_wait(&acc_full[buf], acc_ph[buf], ctx, kStatusGemmAccFull)) goto done;
            acc_ph[buf] ^= 1u;
            tc::fence_after_sync();
            const int fl = q * 32 + lane, f = nt * kBM + fl;
            const bool f_ok = f < p.n;
            const long long row0 = (long long)rt * NR;
            unsigned char* base = reinterpret_cast<unsigned char*>(p.out) + ((long long)g * p.o_gstride + f) * (p.out_f32 ? 4 : 2);
            auto store = [&](int c, float v) {
                const long long row = row0 + c;
                if (f_ok && row < p.rows) {
                    if (p.out_f32) *reinterpret_cast<float*>(base + row * p.ldo * 4) = v;
                    else *reinterpret_cast<uint16_t*>(base + row * p.ldo * 2) = f32_to_bf16_bits(v);
                }
            };
            if constexpr (!SPLIT) {
#pragma unroll 1
                for (int c0 = 0; c0 < NR; c0 += 16) {
                    uint32_t r[16];
                    tc::tmem_ld16(tc::tmem_addr(tm, q, buf * NR + c0), r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) store(c0 + j, __uint_as_float(r[j]));
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
            } else {
                // The tile's K splits live in the blocks of this cluster.  Peers park their partial tile in their own
                // shared memory; rank 0 adds them to its own in rank order (a fixed order: the same bits every time)
                // through distributed shared memory, and stores.  32 columns at a time.
                constexpr int CW = NR < 32 ? NR : 32;
                float* red = reinterpret_cast<float*>(smem + C::oRed) + fl * NR;
                if (!opened) {  // the opening cluster barrier: every peer's barriers and buffers exist
                    cluster_wait();
                    opened = true;
                }
                if (kr != 0) {
                    if (!mbar_wait(red_empty, red_ph ^ 1u, ctx, kStatusGemmRedEmpty)) goto done;  // rank 0 is done with the last one
                    fence_cluster();
                } else {
                    if (!mbar_wait(red_full, red_ph, ctx, kStatusGemmRedFull)) goto done;
                    fence_cluster();
                }
#pragma unroll 1
                for (int c0 = 0; c0 < NR; c0 += CW) {
                    float v[CW];
#pragma unroll
                    for (int c1 = 0; c1 < CW; c1 += 16) {
                        uint32_t r[16];
                        tc::tmem_ld16(tc::tmem_addr(tm, q, buf * NR + c0 + c1), r);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[c1 + j] = __uint_as_float(r[j]);
                    }
                    if (kr != 0) {
#pragma unroll
                        for (int j = 0; j < CW; j += 4) *reinterpret_cast<float4*>(red + c0 + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    } else {
#pragma unroll
                        for (uint32_t r = 1; r < ks; ++r) {
                            const uint32_t remote = peer_smem(red + c0, r);
#pragma unroll
                            for (int j = 0; j < CW; j += 4) {
                                const float4 t4 = peer_load4(remote + (uint32_t)j * 4);
                                v[j] = v[j] + t4.x;
                                v[j + 1] = v[j + 1] + t4.y;
                                v[j + 2] = v[j + 2] + t4.z;
                                v[j + 3] = v[j + 3] + t4.w;
                            }
                        }
#pragma unroll
                        for (int j = 0; j < CW; ++j) store(c0 + j, v[j]);
                    }
                }
                tc::fence_before_sync();
                fence_cluster();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&acc_empty[buf]);
                    if (kr != 0) peer_mbar_arrive(peer_smem(red_full, 0));
                    else
                        for (uint32_t r = 1; r < ks; ++r) peer_mbar_arrive(peer_smem(red_empty, r));
                }
                red_ph ^= 1u;
            }
            buf ^= 1;
        }
    }
done:
    // After an abort, copies into this block's shared memory may still be in flight: give them a bounded time.
    if (ctl[1]) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) {
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tm, C::kTmemCols);
    // No block leaves while a peer may still read its partial tile or arrive on its barriers.
    if (SPLIT) {
        if (!opened) cluster_wait();  // the threads that never needed the opening barrier complete it here
        cluster_sync_all();
    }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiled>(f);
    }();
    return fn;
}

// A [groups][rows][k] bf16 matrix (row stride ld, group stride gstride, in elements) as a 3-D map with boxes of
// 64 k x box_rows rows in the 128-byte swizzle; rows past the extent read as zero.  The dimensions are ordered by
// stride -- (k, rows, groups), or (k, groups, rows) when the groups interleave inside a row (`swapped`).
bool matrix_map(CUtensorMap* tm, int* swapped, const void* base, long long k, long long rows, long long groups, long long ld, long long gstride,
                int box_rows) {
    EncodeTiled enc = encode_tiled();
    if (enc == nullptr) return false;
    const long long gs = groups > 1 ? gstride : rows * ld;
    *swapped = groups > 1 && gs < ld;
    if (groups > 1 && !*swapped && gs < rows * ld) return false;  // neither nesting: not a layout the callers have
    const cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)(*swapped ? groups : rows), (cuuint64_t)(*swapped ? rows : groups)};
    const cuuint64_t strides[2] = {(cuuint64_t)(*swapped ? gs : ld) * 2, (cuuint64_t)(*swapped ? ld : gs) * 2};
    const cuuint32_t box[3] = {(cuuint32_t)kBK, *swapped ? 1u : (cuuint32_t)box_rows, *swapped ? (cuuint32_t)box_rows : 1u};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// K splits for a launch of few tiles (little n, deep k: o_proj at decode): the largest of 8, 4, 2 that divides the
// k blocks into runs of at least four and still leaves every block of a one-row-tile launch resident at once.  It is
// a function of (n, k, groups) alone for every launch on row tiles of up to 128 rows (all launches of up to 512 rows), so
// a row's bits do not depend on `rows` there.  Measured for
// o_proj at 16 rows (32 tiles): no split 40.7 us, 2 splits 27.1, 4 splits 20.9, 8 splits (two waves of clusters) 24.7.
int pick_ksplit(long long tiles, int kblocks, long long resident) {
    for (int s = 8; s >= 2; s >>= 1)
        if (kblocks % s == 0 && kblocks / s >= 4 && tiles * s <= resident) return s;
    return 1;
}

template <int NR, int KS>
int launch_one(GemmParams& p, long long clusters, cudaStream_t stream) {
    using C = Cfg<NR, (KS > 1)>;
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(proj_gemm_kernel<NR, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kBytes);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(clusters * KS));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = C::kBytes;
    cfg.stream = stream;
    // Programmatic stream serialization: the kernel waits for its predecessors itself (grid_dependency_wait) before its
    // first global access, so its blocks' set-up (barriers, tensor memory, descriptor fetch) overlaps their tail.
    static const bool pdl = [] {
        const char* v = getenv("GLM53F_KDA_PDL");
        return !(v && v[0] == '0');
    }();
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (KS > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = (unsigned)KS;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, proj_gemm_kernel<NR, KS>, p);
}

template <int NR>
int launch_gemm(GemmParams& p, const void* x, long long ldx, long long x_gstride, int groups, int k, cudaStream_t stream) {
    if (!matrix_map(&p.tm_x, &p.x_swapped, x, k, p.rows, groups, ldx, x_gstride, NR)) return (int)cudaErrorNotSupported;
    p.r_tiles = (p.rows + NR - 1) / NR;
    p.tiles = (long long)groups * p.n_tiles * p.r_tiles;
    const long long cap = (long long)sm_count() * Cfg<NR, false>::kBlocksPerSm;
    if constexpr (NR <= 128) {
        // The split is chosen for ONE row tile, whatever the launch's row count: a row's bits then depend on
        // (groups, n, k) only.  More row tiles than fit at once are walked by the same clusters.
        const int ks = pick_ksplit((long long)groups * p.n_tiles, p.kblocks, sm_count());  // clusters were measured at one block per SM
        const long long fit = cap / ks;
        const long long clusters = p.tiles < fit ? p.tiles : fit;
        if (ks == 8) return launch_one<NR, 8>(p, clusters, stream);
        if (ks == 4) return launch_one<NR, 4>(p, clusters, stream);
        if (ks == 2) return launch_one<NR, 2>(p, clusters, stream);
    }
    return launch_one<NR, 1>(p, p.tiles < cap ? p.tiles : cap, stream);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace kda

extern "C" int32_t glm53f_kda_proj_bf16(const uint16_t* x, int64_t ldx, int64_t x_gstride, const uint16_t* w, int64_t ldw, int64_t w_gstride,
                                        int32_t groups, int32_t rows, int32_t n, int32_t k, void* out, int32_t out_f32, int64_t ldo,
                                        int64_t o_gstride, glm53f_stream_t stream) {
    using namespace kda;
    if (groups < 1 || rows < 0 || n < 1 || k < kBK || k % kBK || n % 8 || ldx % 8 || ldw % 8 || ldx < k || ldw < k || ldo < n) return kInvalid;
    if (groups > 1 && (x_gstride % 8 || w_gstride % 8 || x_gstride < 0 || w_gstride < 0 || o_gstride < 0)) return kInvalid;
    if (rows == 0) return 0;
    if (!x || !w || !out || !aligned16(x) || !aligned16(w) || (reinterpret_cast<uintptr_t>(out) & (out_f32 ? 3 : 1))) return kInvalid;
    GemmParams p{};
    p.out = out;
    p.ldo = ldo;
    p.o_gstride = groups > 1 ? o_gstride : 0;
    p.rows = rows;
    p.n = n;
    p.kblocks = k / kBK;
    p.out_f32 = out_f32 != 0;
    p.n_tiles = (n + kBM - 1) / kBM;
    p.status = status_word();
    if (p.status == nullptr) return (int)cudaErrorUnknown;
    if (!matrix_map(&p.tm_w, &p.w_swapped, w, k, n, groups, ldw, w_gstride, kBM)) return (int)cudaErrorNotSupported;
    if (rows <= 16) return launch_gemm<16>(p, x, ldx, x_gstride, groups, k, stream);
    if (rows <= 32) return launch_gemm<32>(p, x, ldx, x_gstride, groups, k, stream);
    if (rows <= 64) return launch_gemm<64>(p, x, ldx, x_gstride, groups, k, stream);
    if (rows <= 128) return launch_gemm<128>(p, x, ldx, x_gstride, groups, k, stream);
    // Wide row tiles once there are rows enough to fill the GPU with them; otherwise narrower ones, two blocks per SM,
    // which quantise better (measured for n = 24,640: 384 rows 81 us against 96 us, 768 rows 144 us against 141 us).
    if (rows > 512 && (long long)groups * p.n_tiles * ((rows + 255) / 256) >= sm_count()) {
        // Enough 256 x 256 tiles for every SM pair: the two-block kernel (GLM53F_KDA_PROJ_PAIR=0 keeps one block per tile).
        static const bool pair = [] {
            const char* e = getenv("GLM53F_KDA_PROJ_PAIR");
            return e == nullptr || e[0] != '0';
        }();
        if (pair) {
            if (!matrix_map(&p.tm_x, &p.x_swapped, x, k, rows, groups, ldx, x_gstride, 128)) return (int)cudaErrorNotSupported;
            return proj_gemm_pair_launch(p.tm_w, p.w_swapped, p.tm_x, p.x_swapped, out, ldo, o_gstride, groups, rows, n, k, out_f32 != 0, p.status, stream);
        }
        return launch_gemm<256>(p, x, ldx, x_gstride, groups, k, stream);
    }
    return launch_gemm<128>(p, x, ldx, x_gstride, groups, k, stream);
}
