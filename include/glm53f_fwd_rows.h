/* Row gather / scatter and the snapshot ("mark") copy of a slot's positional state, for B200 (sm_100a).
 *
 * What this replaces.  The reference keeps a request's KDA states, conv windows and DSA tails in per-slot arenas and
 * saves them ("marks") into pages of the KV pool, so that a prefix-cache hit, a rewind or a fork can restore the
 * recurrent state at a position (crates/glm53f-forward/src/kv.rs:412-476 copy_mark, 482-509 mark, 511-575 rewind and
 * fork, 623-664 export_state, 692-720 import_state; layout in crates/glm53f-forward/src/kvplan.rs:100-132).  The
 * device side of that is two entry points of the forward crate's CUDA library,
 *
 *     glm53f_fwd_gather_rows   crates/glm53f-forward/kernels/glm53f_forward.h:75-80, kernels/glue.cu:101-110,222-239
 *     glm53f_fwd_scatter_rows  crates/glm53f-forward/kernels/glm53f_forward.h:82-85, kernels/glue.cu:241-244
 *
 * bound by crates/glm53f-forward/src/ffi.rs:75-95.  Part 1 below declares them with the reference's names, argument
 * meaning and error behaviour (cudaError_t values as int32_t, 0 = launched, 1 = cudaErrorInvalidValue before any
 * launch).  Part 2 adds one call that moves a whole mark -- all three parts, partial last pages included -- in one
 * launch, where the reference issues up to three launches and three copies.
 *
 * All calls are asynchronous on `stream`, allocate nothing and keep no state.
 */
#ifndef GLM53F_FWD_ROWS_H
#define GLM53F_FWD_ROWS_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef GLM53F_STREAM_T_DEFINED
#define GLM53F_STREAM_T_DEFINED
typedef struct CUstream_st* glm53f_stream_t; /* cudaStream_t; NULL = the legacy default stream */
#endif

/* ---- Part 1: the reference's symbols ------------------------------------------------------------------------ */

/* dst[i] = src[idx[i]] for i < rows: rows of `bytes` bytes, src rows `src_stride` bytes apart, dst rows `dst_stride`
 * bytes apart.  bytes, strides and pointers are multiples of 16; idx is a device array of `rows` entries.
 * rows == 0 or bytes == 0: nothing is launched, returns 0.  Returns 1 (cudaErrorInvalidValue) when rows < 0,
 * bytes < 0, bytes or a stride is not a multiple of 16, a stride is smaller than bytes, a pointer is not 16-byte
 * aligned, or idx is null. */
int32_t glm53f_fwd_gather_rows(const uint8_t* src, int64_t src_stride, const int32_t* idx, uint8_t* dst,
                               int64_t dst_stride, int32_t rows, int64_t bytes, glm53f_stream_t stream);

/* dst[idx[i]] = src[i] for i < rows (same layout rules; idx entries distinct). */
int32_t glm53f_fwd_scatter_rows(const uint8_t* src, int64_t src_stride, const int32_t* idx, uint8_t* dst,
                                int64_t dst_stride, int32_t rows, int64_t bytes, glm53f_stream_t stream);

/* ---- Part 2: a whole mark in one launch (an addition) -------------------------------------------------------- */

/* Copies a slot's positional state into pool pages (save != 0) or back out of them (save == 0), the job of
 * copy_mark (kv.rs:412-476) in one launch.
 *
 *   pages, page_bytes   the page pool and the bytes of one physical page;
 *   page_idx            device array: the mark's pages, the three parts in order, part p taking
 *                       ceil(part_bytes[p] / page_bytes) entries (kvplan.rs:113-126);
 *   part[p], part_bytes[p]   p = 0..2: the slot's KDA states, conv windows and DSA tails (device pointers into the
 *                       arenas) and their sizes; a part of 0 bytes is skipped and takes no pages.
 *
 * Part p's byte b lives at page page_idx[first_p + b / page_bytes], offset b % page_bytes; the last page of a part
 * is filled only as far as the part reaches, the rest of it is not touched.  page_bytes, part_bytes and all
 * pointers are multiples of 16.  Returns 0 or 1 (cudaErrorInvalidValue) like the calls above. */
int32_t glm53f_kda_mark_copy(uint8_t* pages, int64_t page_bytes, const int32_t* page_idx, uint8_t* const part[3],
                             const int64_t part_bytes[3], int32_t save, glm53f_stream_t stream);

/* The same for several slots in one launch (an addition): mark i (i < marks) saves or restores slot slots[i] (a device
 * array), whose part p lies at arena[p] + slots[i] * slot_stride[p]; its pages are page_idx[i * mark_pages ..] with
 * mark_pages = the sum over p of ceil(part_bytes[p] / page_bytes).  slot_stride[p] is a multiple of 16 and at least
 * part_bytes[p].  The slots are distinct, and so are all pages.  marks == 0 launches nothing. */
int32_t glm53f_kda_mark_copy_slots(uint8_t* pages, int64_t page_bytes, const int32_t* page_idx, uint8_t* const arena[3],
                                   const int64_t part_bytes[3], const int64_t slot_stride[3], const int32_t* slots,
                                   int32_t marks, int32_t save, glm53f_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GLM53F_FWD_ROWS_H */
