/* glm53f_kda.h: C ABI of the B200 (sm_100a) KDA (Kimi delta attention) recurrent core.
 *
 * Part 1 declares the thirteen entry points of the reference crate's kernel header
 * (crates/glm53f-kda/kernels/glm53f_kda.h:73-270, bound by crates/glm53f-kda/src/ffi.rs:16-287) with the
 * same names, argument order, types and meaning, so the reference's Rust `ffi` module links against this
 * library unchanged.  Part 2 adds the "core" entry points the benchmark configurations use (inputs after
 * the short convolution: q, k, v, log decay, beta).
 *
 * Conventions shared by every entry point (reference header lines 5-9, 43-47):
 *   - raw device pointers, strides and offsets in ELEMENTS of the pointed-to type, a CUDA stream;
 *   - the return value is a cudaError_t: 0 = enqueued, 1 (cudaErrorInvalidValue) = rejected on the host
 *     before anything was enqueued, anything else = the launch error;
 *   - launches are asynchronous on `stream`; nothing is allocated, nothing is synchronised;
 *   - device-side metadata arrays (cu_rows, keep, conv_off, state_off) are read on the device only, so a
 *     captured graph can be replayed with new metadata.
 *
 * Geometry: DK = DV = 128, TAPS = 4, any heads H in [1, 65535]; C = 3*H*128 conv channels (q | k | v).
 *
 * Layouts (row-major):
 *   recurrent state   [H][128 (v)][128 (k)], f32 or (the *_bf16state entry points) bf16
 *   conv window       bf16 [3][C], the 3 projection rows before the window's first row, oldest first
 *   conv weight       bf16 [C][4], tap 3 multiplies the current row
 *   replay saves      row r, head h: k (f32, L2-normalised) and exp(g) (f32) at (r*H + h)*128, v (bf16) at the
 *                     same index, beta (f32) at r*H + h
 *
 * Numerics: FP32 arithmetic in the reference kernels' operation order with no multiply-add contraction for
 * everything the chain, the replays and the conv shift compute, so those entry points return the reference
 * kernels' bits.  The chunked prefill agrees with the chain to rounding, as the reference's does.
 */
#ifndef GLM53F_KDA_H
#define GLM53F_KDA_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

struct CUstream_st;
#ifndef GLM53F_STREAM_T_DEFINED
#define GLM53F_STREAM_T_DEFINED
typedef struct CUstream_st* glm53f_stream_t; /* cudaStream_t; NULL = the legacy default stream */
#endif
typedef uint16_t glm53f_bf16;                /* raw bfloat16 bits */

#define GLM53F_KDA_DK 128
#define GLM53F_KDA_DV 128
#define GLM53F_KDA_TAPS 4

/* ===================================================================================================
 * Part 1: the reference's entry points
 * =================================================================================================== */

/* Replaces reference glm53f_kda.h:73-83 (kernels/kda.cu:303-318).
 * One layer, one request, `rows` >= 1 consecutive rows from the committed state.
 *   p        bf16 rows; row r has q|k|v at [0, C) of p + r*p_stride and H beta logits at [b_off, b_off+H)
 *            (b_off may be negative)
 *   a, g     bf16 forget-gate / output-gate rows, [H*128] each, strides a_stride / g_stride
 *   conv     bf16 [3][C] window (read only);  conv_w bf16 [C][4]
 *   state_in f32 [H][128][128];  state_out the state after the last row, may be NULL or == state_in
 *   a_log f32 [H]; dt_bias f32 [H*128]; norm_w bf16 [128]; eps 1e-5; lower -5
 *   out      bf16 rows [H*128] at out + r*out_stride: the gated RMSNorm output
 *   k_save, v_save, g_save, b_save   replay inputs for every row; all NULL or all set */
int glm53f_kda_chain(int32_t heads, int32_t rows,
                     const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                     const glm53f_bf16* a, int64_t a_stride,
                     const glm53f_bf16* g, int64_t g_stride,
                     const glm53f_bf16* conv, const glm53f_bf16* conv_w,
                     const float* state_in, float* state_out,
                     const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                     float eps, float lower,
                     glm53f_bf16* out, int64_t out_stride,
                     float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save,
                     glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:97-108 (kernels/kda.cu:343-354).
 * A batch of requests: request b owns rows [cu_rows[b], cu_rows[b+1]) (device int32 [batch+1]; 0 rows
 * allowed, the state is then copied), its window is conv + conv_off[b], its state state_in + state_off[b]
 * written to state_out + state_off[b] (device int64 [batch] each; regions must not overlap). */
int glm53f_kda_chain_batch(int32_t heads, int32_t batch, const int32_t* cu_rows,
                           const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                           const glm53f_bf16* a, int64_t a_stride,
                           const glm53f_bf16* g, int64_t g_stride,
                           const glm53f_bf16* conv, const int64_t* conv_off,
                           const glm53f_bf16* conv_w,
                           const float* state_in, float* state_out, const int64_t* state_off,
                           const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                           float eps, float lower,
                           glm53f_bf16* out, int64_t out_stride,
                           float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save,
                           glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:118-130 (kernels/kda.cu:356-371).
 * As above with bf16 states (offsets in bf16 elements): FP32 arithmetic on the widened state, rounded to
 * bf16 after every row's read-out, so R rows in one call equal R single-row calls bit for bit. */
int glm53f_kda_chain_batch_bf16state(int32_t heads, int32_t batch, const int32_t* cu_rows,
                                     const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                     const glm53f_bf16* a, int64_t a_stride,
                                     const glm53f_bf16* g, int64_t g_stride,
                                     const glm53f_bf16* conv, const int64_t* conv_off,
                                     const glm53f_bf16* conv_w,
                                     const glm53f_bf16* state_in, glm53f_bf16* state_out,
                                     const int64_t* state_off,
                                     const float* a_log, const float* dt_bias,
                                     const glm53f_bf16* norm_w, float eps, float lower,
                                     glm53f_bf16* out, int64_t out_stride,
                                     float* k_save, glm53f_bf16* v_save, float* g_save,
                                     float* b_save, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:136-138 (kernels/kda.cu:392-397).
 * The state after the first `rows` >= 0 saved rows of a chain; state_out may equal state_in. */
int glm53f_kda_replay(int32_t heads, int32_t rows, const float* state_in, float* state_out,
                      const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                      const float* b_save, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:144-148 (kernels/kda.cu:399-405).
 * Every layer of one request: layer l at state + l*state_stride, saves + l*kv_stride, b_save + l*b_stride. */
int glm53f_kda_replay_layers(int32_t heads, int32_t layers, int32_t rows,
                             const float* state_in, float* state_out, int64_t state_stride,
                             const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                             const float* b_save, int64_t kv_stride, int64_t b_stride,
                             glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:157-163 (kernels/kda.cu:407-415).
 * The commit after a verify round: every layer of every request; request b replays keep[b] rows from its
 * row cu_rows[b], 0 <= keep[b] <= its row count (device int32 [batch]). */
int glm53f_kda_replay_batch(int32_t heads, int32_t layers, int32_t batch,
                            const int32_t* cu_rows, const int32_t* keep,
                            const float* state_in, float* state_out, int64_t state_stride,
                            const int64_t* state_off,
                            const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                            const float* b_save, int64_t kv_stride, int64_t b_stride,
                            glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:170-176 (kernels/kda.cu:417-427).  bf16 states, rounded after every row. */
int glm53f_kda_replay_batch_bf16state(int32_t heads, int32_t layers, int32_t batch,
                                      const int32_t* cu_rows, const int32_t* keep,
                                      const glm53f_bf16* state_in, glm53f_bf16* state_out,
                                      int64_t state_stride, const int64_t* state_off,
                                      const float* k_save, const glm53f_bf16* v_save,
                                      const float* g_save, const float* b_save, int64_t kv_stride,
                                      int64_t b_stride, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:183-184 (kernels/kda.cu:448-451).
 * Window rows j = 0..2 become rows keep+j of [window; new rows], in place; new row r is [0, channels) of
 * p + r*p_stride. */
int glm53f_kda_conv_shift(int32_t channels, int32_t keep, glm53f_bf16* conv,
                          const glm53f_bf16* p, int64_t p_stride, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:191-195 (kernels/kda.cu:453-460).
 * Every layer of every request: window conv + l*conv_stride + conv_off[b], new rows from
 * p + l*p_layer_stride + cu_rows[b]*p_stride, keep[b] rows kept. */
int glm53f_kda_conv_shift_batch(int32_t channels, int32_t layers, int32_t batch,
                                const int32_t* cu_rows, const int32_t* keep,
                                glm53f_bf16* conv, int64_t conv_stride, const int64_t* conv_off,
                                const glm53f_bf16* p, int64_t p_layer_stride, int64_t p_stride,
                                glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:204 (kernels/kda_prefill.cu:695-698).
 * Bytes of workspace for `rows_per_pass` rows of every request per pass; the reference's figure
 * (34,816 B per 16 rows, head and request) is kept so callers' arenas fit.  0 for bad arguments. */
int64_t glm53f_kda_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t rows_per_pass);

/* Replaces reference glm53f_kda.h:223-232 (kernels/kda_prefill.cu:700-710).
 * Prefill of `rows` >= 0 rows from the committed state and window; also advances the window past the rows,
 * in place.  state_out must not be NULL (may equal state_in); lower in [-5.8, 0]; value_blocks in
 * {0, 1, 2, 4}; workspace of at least glm53f_kda_prefill_workspace_bytes(heads, 1, 16) bytes. */
int glm53f_kda_prefill(int32_t heads, int32_t rows,
                       const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                       const glm53f_bf16* a, int64_t a_stride,
                       const glm53f_bf16* g, int64_t g_stride,
                       glm53f_bf16* conv, const glm53f_bf16* conv_w,
                       const float* state_in, float* state_out,
                       const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                       float eps, float lower,
                       glm53f_bf16* out, int64_t out_stride, int32_t value_blocks,
                       float* workspace, int64_t workspace_bytes, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:240-250 (kernels/kda_prefill.cu:712-725).  max_rows (host) >= the longest
 * request's rows. */
int glm53f_kda_prefill_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t max_rows,
                             const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                             const glm53f_bf16* a, int64_t a_stride,
                             const glm53f_bf16* g, int64_t g_stride,
                             glm53f_bf16* conv, const int64_t* conv_off,
                             const glm53f_bf16* conv_w,
                             const float* state_in, float* state_out, const int64_t* state_off,
                             const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                             float eps, float lower,
                             glm53f_bf16* out, int64_t out_stride, int32_t value_blocks,
                             float* workspace, int64_t workspace_bytes, glm53f_stream_t stream);

/* Replaces reference glm53f_kda.h:260-270 (kernels/kda_prefill.cu:727-742).  bf16 states. */
int glm53f_kda_prefill_batch_bf16state(int32_t heads, int32_t batch, const int32_t* cu_rows,
                                       int32_t max_rows, const glm53f_bf16* p, int64_t p_stride,
                                       int64_t b_off, const glm53f_bf16* a, int64_t a_stride,
                                       const glm53f_bf16* g, int64_t g_stride, glm53f_bf16* conv,
                                       const int64_t* conv_off, const glm53f_bf16* conv_w,
                                       const glm53f_bf16* state_in, glm53f_bf16* state_out,
                                       const int64_t* state_off, const float* a_log,
                                       const float* dt_bias, const glm53f_bf16* norm_w, float eps,
                                       float lower, glm53f_bf16* out, int64_t out_stride,
                                       int32_t value_blocks, float* workspace,
                                       int64_t workspace_bytes, glm53f_stream_t stream);

/* ===================================================================================================
 * Part 2: the core entry points (inputs after the short convolution)
 *
 * These take what the reference's CPU definitions of the recurrence take (crates/glm53f-kda/src/cpu.rs:573-610,
 * `literal::step`, and src/chunked.rs:67-75, `head`): per row and head q, k, v (bf16, dense [rows][H][128]),
 * the per-channel LOG decay g (f32 [rows][H][128], <= 0) and beta (f32 [rows][H]).  The reference's kernels
 * have no such entry points; its forward always enters through Part 1.
 *
 * Common arguments:
 *   state_in / state_out, state_off   as in glm53f_kda_chain_batch; state_bf16 != 0 selects bf16 storage
 *                                     (rounded after every row in decode/verify/commit, once per chunk in prefill)
 *   flags    GLM53F_KDA_CORE_L2NORM   q and k are L2-normalised (eps 1e-6 inside the sum) and q is scaled by
 *                                     128^-0.5 in the kernel; without it q, k are used as given
 *   gate, norm_w, eps                 gate != NULL fuses the gated RMSNorm: out = bf16(norm_w * y/rms(y) *
 *                                     sigmoid(gate)), gate bf16 [rows][H][128]; gate == NULL stores bf16(y)
 *   out                               bf16 [rows][H][128]
 * =================================================================================================== */

#define GLM53F_KDA_CORE_L2NORM 1
/* glm53f_kda_core_verify_batch only: compute a verify window's outputs as one 16-row chunk on the tensor cores.  The
 * state is read once instead of being walked row by row; the outputs then agree with the serial steps' to the rounding
 * of bf16 operands (max-abs 2e-2, rel-L2 5e-3) instead of bit for bit, while the replay saves are written exactly as
 * without the flag, so a commit still leaves the states of serial decode steps.  Takes windows of up to 16 rows
 * (a longer one records status 122 and only its first 16 rows are computed), bf16 states, state_out == NULL, no gate and
 * no GLM53F_KDA_CORE_L2NORM; any other call ignores the flag and runs the exact form. */
#define GLM53F_KDA_CORE_TENSOR 2

/* One recurrent step per row, rows of request b run in order from its state (decode: one row per request). */
int glm53f_kda_core_decode_batch(int32_t heads, int32_t batch, const int32_t* cu_rows,
                                 const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                 const float* g, const float* beta,
                                 const void* state_in, void* state_out, const int64_t* state_off,
                                 int32_t state_bf16, int32_t flags,
                                 const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                 glm53f_bf16* out, glm53f_stream_t stream);

/* Draft verification: as decode over each request's window of rows, with the replay saves written
 * (k f32, v bf16, exp(g) f32, beta f32; layout of Part 1) and the state optionally left untouched
 * (state_out == NULL). */
int glm53f_kda_core_verify_batch(int32_t heads, int32_t batch, const int32_t* cu_rows,
                                 const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                 const float* g, const float* beta,
                                 const void* state_in, void* state_out, const int64_t* state_off,
                                 int32_t state_bf16, int32_t flags,
                                 const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                 glm53f_bf16* out,
                                 float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save,
                                 glm53f_stream_t stream);

/* A commit without saved replay inputs (an addition): one layer's states advanced in place over the first
 * keep[b] rows of each request, recomputed from the projection rows the verify round kept -- glm53f_kda_chain_batch
 * (same arguments, same arithmetic, so the bits of keep[b] single-row calls) limited to keep[b] <= rows of each
 * request.  The conv windows must still be the verify round's (shift them afterwards).  A verify round then keeps,
 * per row and layer, the 49,280-byte projection row it keeps anyway (crates/glm53f-forward/src/forward.rs:777-790)
 * and the 16,384-byte decay-gate row instead of 82,176 bytes of k, v, g and beta.  `out` receives the kept rows'
 * outputs again (any [rows][out_stride] buffer); `state_bf16` selects the state type. */
int glm53f_kda_chain_commit_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, const int32_t* keep,
                                  const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                  const glm53f_bf16* a, int64_t a_stride,
                                  const glm53f_bf16* g, int64_t g_stride,
                                  const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w,
                                  void* state, const int64_t* state_off, int32_t state_bf16,
                                  const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w,
                                  float eps, float lower, glm53f_bf16* out, int64_t out_stride,
                                  glm53f_stream_t stream);

/* The commit after a verify round, for every layer at once: glm53f_kda_replay_batch with the state type as
 * an argument.  Keeping keep[b] rows gives the bits of keep[b] single-row decode calls. */
int glm53f_kda_core_commit_batch(int32_t heads, int32_t layers, int32_t batch,
                                 const int32_t* cu_rows, const int32_t* keep,
                                 const void* state_in, void* state_out, int64_t state_stride,
                                 const int64_t* state_off, int32_t state_bf16,
                                 const float* k_save, const glm53f_bf16* v_save, const float* g_save,
                                 const float* b_save, int64_t kv_stride, int64_t b_stride,
                                 glm53f_stream_t stream);

/* Chunked prefill (chunk 64) of variable-length sequences packed along the row axis: sequence b owns rows
 * [cu_seqlens[b], cu_seqlens[b+1]) (device int32 [batch+1]); chunks count from each sequence's first row.
 * max_len (host) >= the longest sequence.  state_out must not be NULL. */
int glm53f_kda_core_prefill_varlen(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                   const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                   const float* g, const float* beta,
                                   const void* state_in, void* state_out, const int64_t* state_off,
                                   int32_t state_bf16, int32_t flags,
                                   const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                   glm53f_bf16* out, glm53f_stream_t stream);

/* The same prefill in two passes over a caller-provided workspace, for launches with few (sequence, head) chains --
 * one long sequence, or one GPU's shard of heads -- where one block per chain would leave most SMs idle: the part
 * of every chunk that does not depend on the recurrent state is computed for many chunks at once on all SMs, then
 * one block per chain runs the short state-dependent part chunk by chunk.  `workspace` (device memory, 16-byte
 * aligned) holds 107,008 bytes per (sequence, head, chunk of 64 rows) in flight plus 256 bytes of counters; its size
 * sets how many chunks of every sequence one launch covers (at least one:
 * glm53f_kda_core_prefill_workspace_bytes(heads, batch, 1)); with room for two or more chunks per chain the state part
 * of one segment runs beside the state-independent part of the next.
 * Results do not depend on the workspace size and agree with glm53f_kda_core_prefill_varlen to rounding.  Inputs must be
 * 16-byte aligned and flags must be 0 (status 1 otherwise).  Not in the reference; its own prefill takes a
 * workspace the same way (reference glm53f_kda.h:198-204, 223-232). */
int64_t glm53f_kda_core_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t chunks_per_pass);
int glm53f_kda_core_prefill_varlen_ws(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                      const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                      const float* g, const float* beta,
                                      const void* state_in, void* state_out, const int64_t* state_off,
                                      int32_t state_bf16, int32_t flags,
                                      const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                      glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                                      glm53f_stream_t stream);

/* glm53f_kda_core_prefill_varlen_ws for a head-sharded launch (heads = this GPU's shard of heads_total heads, starting
 * at head0) with the all-gather of the outputs done by the kernel itself: every output row is stored straight into
 * each of the `ranks` (1..8) full buffers full[r], laid out [rows][heads_total][128] bf16 -- this GPU's own and its
 * peers' (device addresses valid in this process: peer-mapped, IPC-opened or symmetric memory; tiled tensor stores,
 * over NVLink for a peer's buffer; no collective follows the launch).  `full` is a host array, read during the call.
 * `out` (the shard-local [rows][heads][128]) may be NULL.  The caller orders the ranks around the launch: no rank may
 * still read a full buffer when another rank's launch starts writing it, and a rank may read its buffer only after
 * every rank's launch has completed (a barrier on each side).  With more than one rank, 16 or fewer chains, FP32 states
 * and a workspace for every chunk of the call (glm53f_kda_core_prefill_workspace_bytes(heads, batch, chunks + 256) is
 * enough) the call scans the sequence in super-blocks on two streams of its own (made once per device on the first such
 * call: host objects, no device memory), so that one super-block's stores run beside the next one's passes; `stream`
 * waits for both before anything later on it runs, also under stream capture.  Calls of this kind on one device share
 * those two streams and their events: issue them from one host thread at a time.  GLM53F_KDA_PREFILL_SUPERBLOCKS=1
 * keeps everything on `stream`.  Not in the reference, which runs on one GPU. */
int glm53f_kda_core_prefill_varlen_ws_gather(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                             const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                             const float* g, const float* beta,
                                             const void* state_in, void* state_out, const int64_t* state_off,
                                             int32_t state_bf16, int32_t flags,
                                             const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                             glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                                             glm53f_bf16* const* full, int32_t ranks, int32_t heads_total, int32_t head0,
                                             glm53f_stream_t stream);

/* No counterpart in the reference.  glm53f_kda_core_prefill_varlen_ws for callers that cannot call cudaMalloc: an
 * engine whose memory planner has already given every byte of HBM away before the first request, or code that runs
 * where an allocation would fail or stall its host (under an allocator lock, in a latency-critical loop).  It takes
 * no workspace: it runs on a fixed array of 6,848,768 bytes (64 workspace slots and the item counters) that lives in
 * the library's device image, so every GPU that has loaded that image holds that much until the process exits.
 *   - Limit: heads * batch <= 64 (at least one chunk per chain must fit); more is rejected with status 1
 *     (cudaErrorInvalidValue) before anything is enqueued.  A launch covers at most 64 / (heads * batch) chunks of
 *     every sequence, so the entry point suits few chains: one sequence on one GPU's shard of heads.
 *   - The first call on each device is a set-up call: it looks the array's device address up (cudaGetSymbolAddress,
 *     with that device current) and remembers it.  Under the CUDA runtime's default lazy module loading this is also
 *     the moment the library's device image -- the array included -- is placed in device memory, so that one call can
 *     fail with cudaErrorMemoryAllocation on a GPU that is already full.  Make it once per device, early: on any small
 *     shape (one chain of one row will do), before the host's memory plan takes the rest of HBM and outside any
 *     stream capture (or run the process with CUDA_MODULE_LOADING=EAGER, which loads the image when the library is).
 *   - After that set-up call a call allocates and frees nothing.
 *   - All calls on a device share the one array.  Its contents are scratch (every slot is written before it is read,
 *     nothing needs clearing, nothing survives a call), so calls that overlap on the GPU -- different streams,
 *     or different processes' threads on one context -- race; keep calls on one device in stream order.
 * Arguments and results otherwise as glm53f_kda_core_prefill_varlen_ws (bit for bit). */
int glm53f_kda_core_prefill_varlen_static(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                          const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                          const float* g, const float* beta,
                                          const void* state_in, void* state_out, const int64_t* state_off,
                                          int32_t state_bf16, int32_t flags,
                                          const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                          glm53f_bf16* out, glm53f_stream_t stream);

/* Status word of the most recent launches on the current device: 0, or a code recorded by a kernel whose
 * bounded wait ran out (the kernel then returned early instead of spinning).  Reads and clears it;
 * synchronises the device.  Not in the reference (its kernels have no device-side waits). */
int glm53f_kda_device_status(void);

/* The multi-GPU boundary of glm53f_kda_core_prefill_varlen_ws_gather for any host, one process per GPU; no counterpart
 * in the reference, which runs on one GPU.  Each rank allocates its full [rows][heads_total][128] bf16 output buffer
 * (plain cudaMalloc memory, 16-byte aligned), exports a handle, gives the 128 opaque bytes to the other ranks by
 * whatever channel the host has, and opens theirs; the addresses it gets are what `full[]` takes.  CUDA IPC underneath:
 * no collective library, no multicast object.  The kernels only store to a peer's buffer, they never load from it.
 *   glm53f_kda_gather_head_range  heads [head0, head0 + heads) of heads_total for `rank` of `ranks` (1..8; heads_total
 *                                 divisible by ranks)
 *   glm53f_kda_gather_export      handle for the `bytes` bytes at `full`, a buffer inside a device allocation of this
 *                                 process (the handle names the allocation and the buffer's offset in it)
 *   glm53f_kda_gather_open        maps a peer's buffer into this process (its GPU must be able to reach the peer's:
 *                                 peer access is enabled on first use); *full is the address to put in `full[]`;
 *                                 *bytes (may be NULL) the exported size.  Not for a handle exported by this process:
 *                                 a rank lists its own buffer by its own address.
 *   glm53f_kda_gather_close       unmaps what glm53f_kda_gather_open mapped; call it after the last launch that stores
 *                                 into the buffer has completed, and before the exporter frees the allocation.
 * All four return 0, 1 (cudaErrorInvalidValue) for a rejected argument, or another cudaError_t.  The caller still
 * orders the ranks around a launch (a barrier on each side), as glm53f_kda_core_prefill_varlen_ws_gather asks. */
typedef struct glm53f_kda_gather_handle { unsigned char opaque[128]; } glm53f_kda_gather_handle;
int glm53f_kda_gather_head_range(int32_t heads_total, int32_t rank, int32_t ranks, int32_t* head0, int32_t* heads);
int glm53f_kda_gather_export(const void* full, int64_t bytes, glm53f_kda_gather_handle* handle);
int glm53f_kda_gather_open(const glm53f_kda_gather_handle* handle, void** full, int64_t* bytes);
int glm53f_kda_gather_close(const glm53f_kda_gather_handle* handle, void* full);

/* Which form the layer prefill entry points (glm53f_kda_prefill, _batch, _batch_bf16state) run; not in the reference's
 * header, whose forward gates its own chunked kernel with a switch of its own (crates/glm53f-forward/src/forward.rs:210,
 * 3580).
 *   0  exact (the default): the row-by-row recurrence, the chain's results bit for bit
 *   1  chunked: passes of (layer prologue, chunk-64 tensor-core kernel with the gated norm fused) over the caller's
 *      workspace; results agree with the chain to the rounding of bf16 operands (the task's tolerances: bf16 outputs
 *      within 2e-2 max-abs / 5e-3 rel-L2, state within 1e-3 rel-L2) and do not depend on the workspace size or the
 *      batching; `value_blocks` is not used.  Calls the chunked kernels cannot take (output rows that are not dense,
 *      rows not 8-byte aligned, a workspace below 64 rows a pass) run the exact form.
 * Any other value only queries.  Returns the mode that was in force.  The environment variable
 * GLM53F_KDA_PREFILL=chunked makes 1 the initial mode.  Process-wide; set it before the launches it should affect. */
int32_t glm53f_kda_prefill_mode(int32_t mode);

/* Which form glm53f_kda_chain_batch_bf16state runs for a draft-verification call, i.e. one with state_out == NULL and
 * the four replay saves given (crates/glm53f-forward/src/forward.rs:3672-3735 with `saves`); not in the reference's
 * header.  Every other call of the chain entry points is unaffected.
 *   0  exact (the default): the row-by-row recurrence, bit for bit the reference kernel's outputs and saves
 *   1  chunked: each request's window of up to 16 rows is one chunk on the tensor cores.  Two launches, nothing
 *      allocated: the first writes the replay saves (k, v, exp(log decay), beta: the exact form's bits, so a commit
 *      still leaves the states of serial decode steps) and parks q, as fp16, in the output rows; the second reads the
 *      bf16 state once per (request, head) and overwrites the output rows with the gated, normalised outputs, which
 *      agree with the exact form's to the rounding of bf16 operands (the task's tolerances: 2e-2 max-abs, 5e-3 rel-L2
 *      before the norm).  A window longer than 16 rows records status 122 (glm53f_kda_device_status): only its first
 *      16 rows get outputs, while the replay saves are still written for every row.  Calls whose rows are not aligned for vector access (p, a, g, conv 8 bytes; out,
 *      the saves, the state base 16 bytes; strides multiples of 4, out_stride of 8 elements) run the exact form.
 * Any other value only queries.  Returns the mode that was in force.  The environment variable GLM53F_KDA_VERIFY=chunked
 * makes 1 the initial mode.  Process-wide; set it before the launches it should affect. */
int32_t glm53f_kda_verify_mode(int32_t mode);

/* Which form the replays of bf16 states run (glm53f_kda_replay_batch_bf16state, glm53f_kda_core_commit_batch with
 * state_bf16 != 0); not in the reference's header.  Replays of f32 states are unaffected.
 *   0  exact (the default): row by row, the state rounded to bf16 after every row: the bits of serial decode steps
 *      (crates/glm53f-kda/kernels/glm53f_kda.h:111-116)
 *   1  chunked: each request's kept rows in chunks of 16 on the tensor cores, the state read once and written once,
 *      rounded to bf16 once per chunk.  The committed state then agrees with serial decode steps to bf16's own rounding
 *      (rel-L2 of a few 1e-3 between the two; the task's bound on a bf16 state is 2e-2), not bit for bit -- against the
 *      FP32 recurrence it is the closer of the two, since mode 0 rounds after every row -- so a host that relies on
 *      verify + commit(k) == k decode steps EXACTLY keeps mode 0.
 * Any other value only queries.  Returns the mode that was in force.  GLM53F_KDA_COMMIT=chunked makes 1 the initial
 * mode.  Process-wide; set it before the launches it should affect. */
int32_t glm53f_kda_commit_mode(int32_t mode);

/* Diagnostic hook, for tests of the failure path; no counterpart in the reference.  The persistent recurrent kernel
 * (the layer entry points, the replays, and core calls with fused norms or an output gate) bounds every device-side wait: a block whose waits see no progress for the limit (2 s by default) records a
 * status code (101-108, which wait), makes its other waits return, and the kernel ends; the context stays usable and
 * glm53f_kda_device_status reports the code.
 *   wait_limit_ns     the limit for the launches that follow, 100,000 .. 60,000,000,000 ns; 0 restores the default
 *   skip_first_state  != 0: in the NEXT launch of that kernel only, block 0 does not fetch its first unit's
 *                     state and tells nobody, so that this unit's wait runs out.  Nothing is in flight and nothing
 *                     faults; the launch's other units complete, that unit's state and outputs are not written.
 * Host-side settings, not thread safe; returns 0, or 1 for a limit outside the range. */
int glm53f_kda_debug_wait_test(uint64_t wait_limit_ns, int32_t skip_first_state);

#ifdef __cplusplus
}
#endif
#endif /* GLM53F_KDA_H */
