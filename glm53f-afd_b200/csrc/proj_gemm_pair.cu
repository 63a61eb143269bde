// The projection GEMM for many rows on SM pairs: out[g][r][o] = sum_k x[g][r][k] * w[g][o][k] with 256 x 256 tiles
// computed by tcgen05.mma.cta_group::2.
//
// Why a pair.  With one block per tile (proj_gemm.cu) a 128 x 256 tile reads 48 KiB of operands from L2 per 4.2 MFLOP;
// the tensor pipe then waits on the copies a quarter of the time.  Two blocks of a cluster that share a 256 x 256 tile
// read 32 KiB each for the same work: each loads its own 128 weight rows and HALF of the activation rows, and the
// pair's MMA reads the activation halves from both blocks' shared memory.
//
// Protocol (block 0 of the pair leads):
//   producer (warp 0, both blocks)  tensor copies of the block's weight tile and its half of the rows into its own
//                                   ring; the copies of BOTH blocks complete the LEADER's stage barrier;
//   MMA (warp 1 of the leader)      one thread issues the pair's MMAs (M = 256, N = 256, K = 16) and commits each stage
//                                   to both blocks' `empty` barriers, each finished tile to both `acc_full` barriers;
//   epilogue (warps 2-5, both)      each block drains its own 128 features x 256 rows from its tensor memory and
//                                   arrives on the leader's `acc_empty`.
// Tensor memory is allocated by both blocks together (512 columns: two accumulators).  Every wait is bounded (codes
// 140-143); both blocks reach the collective TMEM release and the closing cluster barrier on every path.

#include <cuda.h>

#include "common.cuh"
#include "glm53f_proj.h"
#include "kda_internal.h"
#include "tc.cuh"

namespace kda {
namespace {

constexpr int kPM = 128;           // features per block (256 per pair)
constexpr int kPN = 256;           // rows per tile (128 loaded by each block)
constexpr int kPK = 64;
constexpr int kPairThreads = 192;
constexpr int kPairStages = 6;
constexpr int kPairABytes = kPM * 128, kPairBBytes = (kPN / 2) * 128;
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;  // 32 KiB
constexpr int kPairTmemCols = 512;
constexpr int oPairBars = kPairStages * kPairStageBytes;
constexpr int oPairCtl = oPairBars + (2 * kPairStages + 4) * 8;
constexpr int kPairSmem = oPairCtl + 16 + 1024;

enum : int { kStatusPairEmpty = 140, kStatusPairFull = 141, kStatusPairAccFull = 142, kStatusPairAccEmpty = 143 };

__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void pair_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pair_addr(const void* local, uint32_t rank) {
    uint32_t ra;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
    return ra;
}
__device__ __forceinline__ void pair_mbar_arrive(uint32_t remote_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
// A tiled tensor copy into this block's shared memory whose completion is counted on `bar_addr`, a barrier of this
// block or of its pair (a shared::cluster address).
__device__ __forceinline__ void pair_tensor_load(void* smem_dst, const void* tmap, int x, int y, int z, uint32_t bar_addr) {
    asm volatile("cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_addr), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void pair_tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pair_tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void pair_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// `bar_addr` (a shared::cluster address, this block's or the pair's) completes once the pair's MMAs issued so far have.
__device__ __forceinline__ void pair_commit(uint32_t bar_addr) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}

struct PairParams {
    CUtensorMap tm_w, tm_x;
    void* out;
    long long ldo, o_gstride;
    int rows, n, kblocks, out_f32;
    int n_tiles, r_tiles;
    int w_swapped, x_swapped;
    long long tiles;
    int* status;
};

__global__ void __launch_bounds__(kPairThreads, 1) proj_gemm_pair_kernel(const __grid_constant__ PairParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + oPairBars);   // used in the leader: both blocks' copies
    uint64_t* empty = full + kPairStages;                            // in each block: the pair's MMAs are done with the stage
    uint64_t* acc_full = empty + kPairStages;                        // in each block
    uint64_t* acc_empty = acc_full + 2;                              // used in the leader: both blocks' epilogues
    volatile uint32_t* ctl = reinterpret_cast<volatile uint32_t*>(smem + oPairCtl);
    uint32_t* tmem_slot = const_cast<uint32_t*>(ctl) + 2;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = pair_rank();
    const long long tile0 = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
    if (tid == 0) {
        for (int i = 0; i < kPairStages; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 8);  // four epilogue warps of each block
        }
        ctl[0] = 0u;
        ctl[1] = 0u;
        mbar_init_fence();
    }
    __syncthreads();
    pair_sync_all();  // the pair's barriers exist before either block touches the other's
    if (warp == 1) pair_tmem_alloc(tmem_slot, kPairTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tm = *tmem_slot;
    const WaitCtx ctx{ctl, ctl + 1, p.status};

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            for (long long t = tile0; t < p.tiles; t += tile_step) {
                const int rt = (int)(t % p.r_tiles);
                const long long u = t / p.r_tiles;
                const int nt = (int)(u % p.n_tiles), g = (int)(u / p.n_tiles);
                const int f0 = nt * 2 * kPM + (int)rank * kPM, r0 = rt * kPN + (int)rank * (kPN / 2);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1u, ctx, kStatusPairEmpty)) goto done;
                    unsigned char* st = smem + s * kPairStageBytes;
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * kPairStageBytes);
                    const uint32_t bar = pair_addr(&full[s], 0);
                    if (p.w_swapped) pair_tensor_load(st, &p.tm_w, kb * kPK, g, f0, bar);
                    else pair_tensor_load(st, &p.tm_w, kb * kPK, f0, g, bar);
                    if (p.x_swapped) pair_tensor_load(st + kPairABytes, &p.tm_x, kb * kPK, g, r0, bar);
                    else pair_tensor_load(st + kPairABytes, &p.tm_x, kb * kPK, r0, g, bar);
                    if (++s == kPairStages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = tc::idesc_bf16(2 * kPM, kPN, 0, 0, 0);
            int s = 0, buf = 0;
            uint32_t ph = 0, acc_ph[2] = {0, 0};
            for (long long t = tile0; t < p.tiles; t += tile_step) {
                if (!mbar_wait(&acc_empty[buf], acc_ph[buf] ^ 1u, ctx, kStatusPairAccEmpty)) goto done;
                tc::fence_after_sync();
                const uint32_t d = tm + (uint32_t)(buf * kPN);
                for (int kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(&full[s], ph, ctx, kStatusPairFull)) goto done;
                    tc::fence_after_sync();
                    const unsigned char* st = smem + s * kPairStageBytes;
#pragma unroll
                    for (int i = 0; i < kPK / 16; ++i)
                        pair_mma(d, tc::desc_sw128_kmajor(st, kPM, 16 * i), tc::desc_sw128_kmajor(st + kPairABytes, kPN / 2, 16 * i), idesc, kb > 0 || i > 0);
                    pair_commit(smem_u32(&empty[s]));
                    pair_commit(pair_addr(&empty[s], 1));
                    if (++s == kPairStages) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                pair_commit(smem_u32(&acc_full[buf]));
                pair_commit(pair_addr(&acc_full[buf], 1));
                acc_ph[buf] ^= 1u;
                buf ^= 1;
                ctl[0] = ctl[0] + 1u;
            }
        }
    } else {
        const int q = warp & 3;
        int buf = 0;
        uint32_t acc_ph[2] = {0, 0};
        for (long long t = tile0; t < p.tiles; t += tile_step) {
            const int rt = (int)(t % p.r_tiles);
            const long long u = t / p.r_tiles;
            const int nt = (int)(u % p.n_tiles), g = (int)(u / p.n_tiles);
            if (!mbar_wait(&acc_full[buf], acc_ph[buf], ctx, kStatusPairAccFull)) goto done;
            acc_ph[buf] ^= 1u;
            tc::fence_after_sync();
            const int f = nt * 2 * kPM + (int)rank * kPM + q * 32 + lane;
            const bool f_ok = f < p.n;
            const long long row0 = (long long)rt * kPN;
            unsigned char* base = reinterpret_cast<unsigned char*>(p.out) + ((long long)g * p.o_gstride + f) * (p.out_f32 ? 4 : 2);
#pragma unroll 1
            for (int c0 = 0; c0 < kPN; c0 += 16) {
                uint32_t r[16];
                tc::tmem_ld16(tc::tmem_addr(tm, q, buf * kPN + c0), r);
                tc::tmem_ld_wait();
                if (f_ok) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const long long row = row0 + c0 + j;
                        if (row < p.rows) {
                            if (p.out_f32) *reinterpret_cast<float*>(base + row * p.ldo * 4) = __uint_as_float(r[j]);
                            else *reinterpret_cast<uint16_t*>(base + row * p.ldo * 2) = f32_to_bf16_bits(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(&acc_empty[buf]);
                else pair_mbar_arrive(pair_addr(&acc_empty[buf], 0));
                ctl[0] = ctl[0] + 1u;
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
    pair_sync_all();  // neither block releases tensor memory or leaves while the pair's MMAs or arrivals may still touch it
    if (warp == 1) pair_tmem_dealloc(tm, kPairTmemCols);
    pair_sync_all();
}

}  // namespace

// Declared in kda_internal.h: the tensor maps are built by the caller (proj_gemm.cu), boxes of 128 rows each.
int proj_gemm_pair_launch(const CUtensorMap& tm_w, int w_swapped, const CUtensorMap& tm_x, int x_swapped, void* out, long long ldo, long long o_gstride,
                          int groups, int rows, int n, int k, int out_f32, int* status, cudaStream_t stream) {
    static int configured_dev = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (configured_dev != dev) {
        const cudaError_t e = cudaFuncSetAttribute(proj_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem);
        if (e != cudaSuccess) return (int)e;
        configured_dev = dev;
    }
    PairParams p{};
    p.tm_w = tm_w;
    p.tm_x = tm_x;
    p.w_swapped = w_swapped;
    p.x_swapped = x_swapped;
    p.out = out;
    p.ldo = ldo;
    p.o_gstride = groups > 1 ? o_gstride : 0;
    p.rows = rows;
    p.n = n;
    p.kblocks = k / kPK;
    p.out_f32 = out_f32;
    p.n_tiles = (n + 2 * kPM - 1) / (2 * kPM);
    p.r_tiles = (rows + kPN - 1) / kPN;
    p.tiles = (long long)groups * p.n_tiles * p.r_tiles;
    p.status = status;
    const long long pairs_cap = sm_count() / 2;
    const long long pairs = p.tiles < pairs_cap ? p.tiles : pairs_cap;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)(pairs * 2));
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = kPairSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, proj_gemm_pair_kernel, p);
}

}  // namespace kda
