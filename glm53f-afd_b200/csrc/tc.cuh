// tcgen05 / TMEM helpers for sm_100a (cta_group::1), and the shared-memory "cell" layout the kernels write their
// MMA operands in by hand.
//
// Cell layout.  A matrix operand tile is stored as 16-byte cells: cell(c, r) at byte (c * R + r) * 16, where c is
// the 16-byte chunk index along the dimension that is contiguous in the data and r runs over the other dimension
// (R values).  With one lane per r, a warp's 16-byte writes land on 512 contiguous bytes: no bank conflicts.
// The same bytes are a valid un-swizzled tcgen05 operand in either role:
//   contiguous dimension = K  : K-major,  leading byte offset (K-chunk to K-chunk)   = R * 16, stride byte offset
//                                (8-row group to 8-row group) = 128;
//   contiguous dimension = M/N: MN-major, stride byte offset (MN-chunk to MN-chunk)  = R * 16, leading byte offset
//                                (8-k group to 8-k group)     = 128.
// One instruction consumes 32 bytes of K: for bf16, two K-chunks (K-major) or two 8-k groups (MN-major).
// These encodings were checked against a CPU product on the device for M = 64/128, N = 64/128/256, bf16 and tf32
// K-major, bf16 MN-major, negated A and accumulation (tf32 MN-major operands did not give correct products
// un-swizzled, so the kernels use bf16 hi/lo splits where they need more than 8 bits of operand mantissa).
#pragma once

#include "common.cuh"

namespace kda {
namespace tc {

// ---- TMEM allocation (one warp, all lanes) ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- descriptors ------------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, no swizzle: start address, leading / stride byte offsets (all >> 4), version 1.
__device__ __forceinline__ uint64_t smem_desc(const void* smem, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = (uint64_t)((smem_u32(smem) & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}
// Operand tile in the cell layout with R cells per chunk, starting at K offset k0 (elements).
//   K-major : the tile's contiguous dimension is K (elements per cell T = 8 for bf16)
//   MN-major: the tile's contiguous dimension is M or N; k0 counts rows of 16 bytes
__device__ __forceinline__ uint64_t desc_kmajor_bf16(const unsigned char* tile, int R, int row0, int k0) {
    return smem_desc(tile + ((size_t)(k0 / 8) * R + row0) * 16, (uint32_t)R * 16, 128);
}
__device__ __forceinline__ uint64_t desc_mnmajor_bf16(const unsigned char* tile, int R, int mn0, int k0) {
    return smem_desc(tile + ((size_t)(mn0 / 8) * R + k0) * 16, 128, (uint32_t)R * 16);
}
// Operand tiles in the 128-byte swizzle (what a tiled tensor copy with that swizzle writes): boxes of R rows x 128 bytes
// (64 bf16), 1024-byte aligned, the 16-byte piece p of row r stored at piece p ^ (r & 7); a second box follows at R * 128.
//   K-major : rows are M/N indices, the 128 bytes run along K.  One instruction's 16 K elements are 32 bytes of a row.
//   MN-major: rows are K indices, the 128 bytes run along M/N; 64-wide M/N blocks are R * 128 bytes apart (R = K rows).
__device__ __forceinline__ uint64_t desc_sw128_kmajor(const unsigned char* tile, int R, int k0) {
    return smem_desc(tile + (size_t)(k0 / 64) * R * 128 + (k0 % 64) * 2, 16, 1024) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_sw128_mnmajor(const unsigned char* tile, int R, int k0) {
    return smem_desc(tile + (size_t)k0 * 128, (uint32_t)R * 128, 1024) | ((uint64_t)2 << 61);
}
// Instruction descriptor for kind::f16 with bf16 operands and an f32 accumulator.
__device__ __forceinline__ constexpr uint32_t idesc_bf16(int M, int N, int a_mn_major, int b_mn_major, int a_negate) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_negate << 13) | ((uint32_t)a_mn_major << 15) |
           ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], issued by one thread.
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Makes `bar` complete once every MMA issued so far by this thread has finished (implies fence::before_thread_sync).
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- TMEM <-> registers: 32 lanes x 32 columns of 32 bits per warp; thread l of warp w touches lane 32*(w%4)+l -------
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
// 32 lanes x C columns (C = 16 or 32).
template <int C>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[C]) {
    if constexpr (C == 32) tmem_ld32(taddr, r);
    else tmem_ld16(taddr, r);
}
template <int C>
__device__ __forceinline__ void tmem_st(uint32_t taddr, const uint32_t (&r)[C]) {
    if constexpr (C == 32) tmem_st32(taddr, r);
    else tmem_st16(taddr, r);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM lane of accumulator row m: M = 128 accumulators put row m in lane m; M = 64 accumulators put row m in lane
// (m % 16) + 32 * (m / 16), i.e. warp w holds rows 16w .. 16w+15 in its first 16 lanes.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int warp, int col) { return base + ((uint32_t)(warp * 32) << 16) + (uint32_t)col; }

// ---- bf16 packing ----------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi): 16 bits of mantissa in two bf16 operands.
__device__ __forceinline__ void split_bf16(float x, float& hi, float& lo) {
    hi = bf16_round(x);
    lo = x - hi;
}

}  // namespace tc
}  // namespace kda
