// Device helpers shared by the sm_100a KDA kernels: mbarrier and bulk-copy PTX, bounded waits, bf16 bits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kda {

constexpr int DK = 128, DV = 128, TAPS = 4, WINDOW = 3;
constexpr int kInvalid = 1;  // cudaErrorInvalidValue

// Status codes a kernel records when a bounded wait runs out (read by glm53f_kda_device_status).
enum : int {
    kStatusOk = 0,
    kStatusWaitStateFull = 101,
    kStatusWaitStateEmpty = 102,
    kStatusWaitRawFull = 103,
    kStatusWaitRawEmpty = 104,
    kStatusWaitRowFull = 105,
    kStatusWaitRowEmpty = 106,
    kStatusWaitYFull = 107,
    kStatusWaitYEmpty = 108,
    kStatusWaitPrefill = 120,
    kStatusPrefillRange = 121,  // eight rows of decay beyond what the tensor-core kernels can factor (or a positive log decay)
    kStatusVerifyWindow = 122,  // the tensor-core verify met a window of more than 16 rows (it computed the first 16)
};

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier (shared::cta) -------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// try_wait with a suspend-time hint: the thread may sleep in hardware until the phase completes or the hint runs
// out, instead of burning issue slots (and shared-memory bandwidth) in a polling loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// A wait that cannot spin forever.  It gives up when neither the barrier flips nor the block's progress
// counter moves for kWaitLimitNs; the caller then records `code`, raises the block's abort flag and returns
// from the kernel.  Every other wait of the block sees the abort flag and returns false at once.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s without any progress in this block

struct WaitCtx {
    volatile uint32_t* progress;  // bumped by every role whenever it finishes a job
    volatile uint32_t* abort;     // set once by the first wait that gives up
    int* status;                  // the library's device status word (global memory)
    uint64_t limit_ns = kWaitLimitNs;  // how long a wait goes without progress before it gives up
};

static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int code) {
    uint64_t t0 = global_timer_ns();
    uint32_t seen = *ctx.progress;
    for (;;) {
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait_hint(bar, parity, 4000u)) return true;
            if (*ctx.abort) return false;
        }
        const uint32_t now_p = *ctx.progress;
        const uint64_t now = global_timer_ns();
        if (now_p != seen) {
            seen = now_p;
            t0 = now;
        } else if (now - t0 > ctx.limit_ns) {
            atomicCAS(ctx.status, 0, code);
            *ctx.abort = 1u;
            return false;
        }
    }
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, ctx, code);
}

// ---- bulk asynchronous copies (1-D, 16-byte aligned, size a multiple of 16) ------------------------------------
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}
// Tiled tensor copy (rank 3) of one box into this block's shared memory; `tmap` points at a CUtensorMap in the kernel's
// parameters.  x (the innermost coordinate) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tensor_load_3d(void* smem_dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
// Tiled tensor copy (rank 3) of one box from this block's shared memory to global memory (a bulk-group operation).
__device__ __forceinline__ void tensor_store_3d(const void* tmap, int x, int y, int z, const void* smem_src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Generic-proxy writes to shared memory made visible to the async proxy (bulk stores read them).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// The same barrier carrying a vote: true when `ok` holds on every one of the `threads` threads.  A role whose threads
// may individually give up on a wait decides at such a barrier whether it goes on, so that either all of its threads
// reach the role's next barrier or none does.
__device__ __forceinline__ bool named_bar_all(int id, int threads, bool ok) {
    uint32_t all;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %3, 0;\n\t"
        "bar.red.and.pred q, %1, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(all)
        : "r"(id), "r"(threads), "r"((uint32_t)ok)
        : "memory");
    return all != 0;
}

}  // namespace kda
