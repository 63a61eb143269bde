// Row gather / scatter by an index list, and the one-launch copy of a slot's positional state into pool pages and
// back.  Pure data movement, bound by HBM: every byte is read once and written once.
//
// The reference's kernel (crates/glm53f-forward/kernels/glue.cu:101-110) gives each row one block of 128 threads that
// walks the row 2 KiB at a time; a mark's rows are pool pages of 394,944 bytes, so a launch there is 181-376 blocks
// with one 16-byte load in flight per thread.  Here the (row, 32 KiB tile) pairs of a launch are spread over the
// whole grid and a thread keeps eight independent 16-byte loads in flight before its first store (32 KiB per block
// of 256 threads and iteration, up to eight blocks per SM), with streaming cache hints in both directions: the data
// is not read again soon.  Rows of at most 4 KiB (the token rows other callers of the same entry points move) go one
// warp per row.
//
// Results are the bytes of the reference's kernel: dst[i] = src[idx[i]] (gather) or dst[idx[i]] = src[i] (scatter).

#include "common.cuh"
#include "glm53f_fwd_rows.h"
#include "kda_internal.h"

namespace kda {
namespace {

// Measured on a B200 for a 73 MiB mark (one launch per mark, marks back to back): 256 threads x 8 vectors with at most
// 16 blocks per SM 28.9 us; 4 vectors 31-33 us; 512 or 1024 threads 31-32 us; a device-to-device cudaMemcpyAsync of
// the same bytes 31.1 us.
#ifndef ROWS_THREADS
#define ROWS_THREADS 256
#define ROWS_VECS 8
#define ROWS_BLOCKS_PER_SM 16
#endif
#ifndef ROWS_MIN_BLOCKS
#define ROWS_MIN_BLOCKS 1
#endif
constexpr int kCopyThreads = ROWS_THREADS;
constexpr int kVecs = ROWS_VECS;                       // 16-byte loads in flight per thread
constexpr int kTileChunks = kCopyThreads * kVecs;      // 16-byte chunks per tile: 32 KiB
constexpr int kSmallChunks = 32 * kVecs;               // rows up to 4 KiB: one warp per row

__device__ __forceinline__ uint4 load_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void store_stream(uint4* p, const uint4& v) { __stcs(p, v); }

// Copies chunks [first, first + n * stride) of a row, at most kVecs per caller thread: all loads, then all stores.
__device__ __forceinline__ void copy_vecs(const uint4* __restrict__ s, uint4* __restrict__ d, long long first, int stride, long long chunks) {
    uint4 v[kVecs];
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        const long long c = first + (long long)j * stride;
        if (c < chunks) v[j] = load_stream(s + c);
    }
#pragma unroll
    for (int j = 0; j < kVecs; ++j) {
        const long long c = first + (long long)j * stride;
        if (c < chunks) store_stream(d + c, v[j]);
    }
}

__global__ void __launch_bounds__(kCopyThreads, ROWS_MIN_BLOCKS) rows_tile_kernel(const uint8_t* __restrict__ src, long long src_stride, const int32_t* __restrict__ idx,
                                                                 uint8_t* __restrict__ dst, long long dst_stride, long long chunks, int tiles_per_row,
                                                                 long long units, int scatter) {
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const long long row = u / tiles_per_row;
        const int tile = (int)(u - row * tiles_per_row);
        const long long other = idx[row];
        const long long s_row = scatter ? row : other, d_row = scatter ? other : row;
        const uint4* s = reinterpret_cast<const uint4*>(src + s_row * src_stride);
        uint4* d = reinterpret_cast<uint4*>(dst + d_row * dst_stride);
        copy_vecs(s, d, (long long)tile * kTileChunks + threadIdx.x, kCopyThreads, chunks);
    }
}

__global__ void __launch_bounds__(kCopyThreads) rows_warp_kernel(const uint8_t* __restrict__ src, long long src_stride, const int32_t* __restrict__ idx,
                                                                 uint8_t* __restrict__ dst, long long dst_stride, int chunks, long long rows, int scatter) {
    const int lane = threadIdx.x & 31;
    const long long warps = (long long)gridDim.x * (kCopyThreads / 32);
    for (long long row = (long long)blockIdx.x * (kCopyThreads / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
        const long long other = idx[row];
        const long long s_row = scatter ? row : other, d_row = scatter ? other : row;
        copy_vecs(reinterpret_cast<const uint4*>(src + s_row * src_stride), reinterpret_cast<uint4*>(dst + d_row * dst_stride), lane, 32, chunks);
    }
}

struct MarkParts {
    uint8_t* part[3];         // one mark: the slot's parts; several: the arenas' bases
    long long chunks[3];      // 16-byte chunks of each part
    long long first_unit[4];  // prefix sums of the parts' (page, tile) units; [3] = units of one mark
    int first_page[3];        // the part's first entry of a mark's page list
    long long slot_chunks[3]; // several marks: 16-byte chunks from one slot's part to the next slot's
    const int32_t* slots;     // several marks: the slot of each (device), or null for one mark at part[]
    int mark_pages;           // entries of page_idx per mark
    long long units;          // all marks' units
};

__global__ void __launch_bounds__(kCopyThreads, ROWS_MIN_BLOCKS) mark_copy_kernel(uint8_t* __restrict__ pages, long long page_chunks, int tiles_per_page,
                                                                 const int32_t* __restrict__ page_idx, const MarkParts m, int save) {
    for (long long u0 = blockIdx.x; u0 < m.units; u0 += gridDim.x) {
        const long long mark = u0 / m.first_unit[3], u = u0 - mark * m.first_unit[3];
        const int p = u >= m.first_unit[2] ? 2 : u >= m.first_unit[1] ? 1 : 0;
        const long long v = u - m.first_unit[p];
        const long long page = v / tiles_per_page;
        const int tile = (int)(v - page * tiles_per_page);
        // What this page holds of the part: a whole page, or the part's remainder.
        const long long left = m.chunks[p] - page * page_chunks;
        const long long n = left < page_chunks ? left : page_chunks;
        uint4* in_pool = reinterpret_cast<uint4*>(pages) + (long long)page_idx[mark * m.mark_pages + m.first_page[p] + page] * page_chunks;
        uint4* in_arena = reinterpret_cast<uint4*>(m.part[p]) + (m.slots ? (long long)m.slots[mark] * m.slot_chunks[p] : 0) + page * page_chunks;
        const long long c0 = (long long)tile * kTileChunks + threadIdx.x;
        if (save) copy_vecs(in_arena, in_pool, c0, kCopyThreads, n);
        else copy_vecs(in_pool, in_arena, c0, kCopyThreads, n);
    }
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Blocks for `units` independent tiles: every SM full several times over, never more blocks than tiles.
int grid_for(long long units) {
    const long long cap = (long long)sm_count() * ROWS_BLOCKS_PER_SM;
    return (int)(units < cap ? units : cap);
}

int32_t gather_scatter(const uint8_t* src, int64_t src_stride, const int32_t* idx, uint8_t* dst, int64_t dst_stride, int32_t rows, int64_t bytes,
                       int scatter, cudaStream_t stream) {
    // The reference's checks, in its order (kernels/glue.cu:222-233).
    if (rows < 0 || bytes < 0 || bytes % 16 || src_stride % 16 || dst_stride % 16 || src_stride < bytes || dst_stride < bytes)
        return cudaErrorInvalidValue;
    if (rows == 0 || bytes == 0) return cudaSuccess;
    if (!aligned16(src) || !aligned16(dst) || !idx) return cudaErrorInvalidValue;
    const long long chunks = bytes / 16;
    if (chunks <= kSmallChunks) {
        const long long blocks = ((long long)rows + kCopyThreads / 32 - 1) / (kCopyThreads / 32);
        rows_warp_kernel<<<grid_for(blocks), kCopyThreads, 0, stream>>>(src, src_stride, idx, dst, dst_stride, (int)chunks, rows, scatter);
    } else {
        const long long tiles = (chunks + kTileChunks - 1) / kTileChunks;
        if (tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
        const long long units = tiles * rows;
        rows_tile_kernel<<<grid_for(units), kCopyThreads, 0, stream>>>(src, src_stride, idx, dst, dst_stride, chunks, (int)tiles, units, scatter);
    }
    return cudaGetLastError();
}

}  // namespace
}  // namespace kda

extern "C" int32_t glm53f_fwd_gather_rows(const uint8_t* src, int64_t src_stride, const int32_t* idx, uint8_t* dst, int64_t dst_stride, int32_t rows,
                                          int64_t bytes, glm53f_stream_t stream) {
    return kda::gather_scatter(src, src_stride, idx, dst, dst_stride, rows, bytes, 0, stream);
}

extern "C" int32_t glm53f_fwd_scatter_rows(const uint8_t* src, int64_t src_stride, const int32_t* idx, uint8_t* dst, int64_t dst_stride, int32_t rows,
                                           int64_t bytes, glm53f_stream_t stream) {
    return kda::gather_scatter(src, src_stride, idx, dst, dst_stride, rows, bytes, 1, stream);
}

namespace kda {
namespace {
int32_t mark_copy_launch(uint8_t* pages, int64_t page_bytes, const int32_t* page_idx, uint8_t* const part[3], const int64_t part_bytes[3],
                         const int64_t* slot_stride, const int32_t* slots, int32_t marks, int32_t save, cudaStream_t stream) {
    if (!part || !part_bytes || page_bytes <= 0 || page_bytes % 16 || marks < 0) return cudaErrorInvalidValue;
    MarkParts m{};
    const long long page_chunks = page_bytes / 16;
    const long long tiles = (page_chunks + kTileChunks - 1) / kTileChunks;
    if (tiles > 0x7fffffffLL) return cudaErrorInvalidValue;
    long long unit = 0, page = 0;
    for (int p = 0; p < 3; ++p) {
        if (part_bytes[p] < 0 || part_bytes[p] % 16) return cudaErrorInvalidValue;
        if (part_bytes[p] > 0 && (!part[p] || !aligned16(part[p]))) return cudaErrorInvalidValue;
        if (slot_stride && part_bytes[p] > 0 && (slot_stride[p] % 16 || slot_stride[p] < part_bytes[p])) return cudaErrorInvalidValue;
        const long long n_pages = (part_bytes[p] + page_bytes - 1) / page_bytes;
        m.part[p] = part[p];
        m.chunks[p] = part_bytes[p] / 16;
        m.slot_chunks[p] = slot_stride ? slot_stride[p] / 16 : 0;
        m.first_unit[p] = unit;
        m.first_page[p] = (int)page;
        unit += n_pages * tiles;
        page += n_pages;
        if (page > 0x7fffffffLL) return cudaErrorInvalidValue;
    }
    m.first_unit[3] = unit;
    m.mark_pages = (int)page;
    m.slots = slots;
    m.units = unit * marks;
    if (m.units == 0) return cudaSuccess;
    if (!pages || !aligned16(pages) || !page_idx) return cudaErrorInvalidValue;
    mark_copy_kernel<<<grid_for(m.units), kCopyThreads, 0, stream>>>(pages, page_chunks, (int)tiles, page_idx, m, save != 0);
    return cudaGetLastError();
}
}  // namespace
}  // namespace kda

extern "C" int32_t glm53f_kda_mark_copy(uint8_t* pages, int64_t page_bytes, const int32_t* page_idx, uint8_t* const part[3],
                                        const int64_t part_bytes[3], int32_t save, glm53f_stream_t stream) {
    return kda::mark_copy_launch(pages, page_bytes, page_idx, part, part_bytes, nullptr, nullptr, 1, save, stream);
}

extern "C" int32_t glm53f_kda_mark_copy_slots(uint8_t* pages, int64_t page_bytes, const int32_t* page_idx, uint8_t* const arena[3],
                                              const int64_t part_bytes[3], const int64_t slot_stride[3], const int32_t* slots, int32_t marks,
                                              int32_t save, glm53f_stream_t stream) {
    if (!slot_stride || (marks > 0 && !slots)) return cudaErrorInvalidValue;
    return kda::mark_copy_launch(pages, page_bytes, page_idx, arena, part_bytes, slot_stride, slots, marks, save, stream);
}
