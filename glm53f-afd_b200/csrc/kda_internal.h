// Launchers shared between the translation units of the library (not part of the C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "glm53f_kda.h"

namespace kda {

// The layer chain without the rows >= 1 restriction of glm53f_kda_chain: a request with no rows copies its state.
// cu_rows == nullptr runs one request of `rows` rows (conv_off / state_off may then be nullptr too).
int layer_chain_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t rows, const glm53f_bf16* p,
                       int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                       int64_t g_stride, const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w,
                       const void* state_in, void* state_out, const int64_t* state_off, bool bf16_state,
                       const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower,
                       glm53f_bf16* out, int64_t out_stride, cudaStream_t stream);

// The core chain (row-by-row recurrence) on post-conv inputs; the slow-but-exact fallback of the chunked prefill.
int core_chain_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q, const glm53f_bf16* k,
                      const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, void* state_out,
                      const int64_t* state_off, bool bf16_state, int32_t flags, const glm53f_bf16* gate,
                      const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, cudaStream_t stream);

// Window past `keep` rows for every (layer, request): keep from keep[b], else keep1 if >= 0, else the request's
// whole row count (the prefill's advance).
int conv_shift_launch(int32_t channels, int32_t layers, int32_t batch, const int32_t* cu_rows, const int32_t* keep,
                      int32_t keep1, int32_t rows1, glm53f_bf16* conv, int64_t conv_stride, const int64_t* conv_off,
                      const glm53f_bf16* p, int64_t p_layer_stride, int64_t p_stride, cudaStream_t stream);

// One pass of a layer prefill through the core kernel: sequence b's inputs are rows b * pass_rows .. of q, k, v, g, beta
// (its rows row_shift .. row_shift + pass_rows - 1, as many of them as it has); its outputs and gate rows are rows
// cu[b] + row_shift .. of `out` and `gate`, gate rows gate_stride elements apart.
struct PrefillWindow {
    int pass_rows = 0, row_shift = 0;
    long long gate_stride = 0;
    bool qk_fp16 = false;  // q and k hold fp16 bits (the layer prologue's), not bf16
};

// The chunk-64 tensor-core prefill (kda_prefill_tc.cu).  q, k, v, g, out (and norm_w) must be 16-byte aligned.
int core_prefill_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, const glm53f_bf16* q, const glm53f_bf16* k,
                           const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, void* state_out,
                           const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate, const glm53f_bf16* norm_w,
                           float eps, glm53f_bf16* out, cudaStream_t stream, const PrefillWindow* win = nullptr);

// Draft verification as one 16-row chunk on the tensor cores (kda_verify_tc.cu): bf16 states, read only; outputs to the
// rounding of bf16 operands, replay saves as the exact path writes them.  q, k, v, g must be 16-byte aligned.
int core_verify_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* q, const glm53f_bf16* k,
                          const glm53f_bf16* v, const float* g, const float* beta, const void* state_in, const int64_t* state_off,
                          glm53f_bf16* out, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream);

// The chunked form of a layer verify call (glm53f_kda_verify_mode): verify_prologue_launch cooks every window's rows into
// the call's own buffers (k, v, the decay multiplier, beta into the replay saves with the exact form's bits; q as fp16
// into the output rows), layer_verify_tc_launch, on the same stream, computes the windows' outputs from them with the
// gated norm fused.  Saves and out rows 16-byte aligned, out_stride and gate_stride multiples of 8 elements.
int verify_prologue_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                           const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* conv, const int64_t* conv_off,
                           const glm53f_bf16* conv_w, const float* a_log, const float* dt_bias, float lower, glm53f_bf16* out,
                           int64_t out_stride, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream);
int layer_verify_tc_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, const void* state_in, const int64_t* state_off,
                           const glm53f_bf16* gate, int64_t gate_stride, const glm53f_bf16* norm_w, float eps, glm53f_bf16* out,
                           int64_t out_stride, float* k_save, glm53f_bf16* v_save, float* g_save, float* b_save, cudaStream_t stream);

// The commit as chunks of 16 rows on the tensor cores (kda_verify_tc.cu): bf16 states; the committed state agrees with
// the exact replay to the last bits of bf16, not bit for bit.
int commit_tc_launch(int32_t heads, int32_t layers, int32_t batch, const int32_t* cu_rows, const int32_t* keep, int32_t rows1, const void* state_in,
                     void* state_out, int64_t state_stride, const int64_t* state_off, const float* k_save, const glm53f_bf16* v_save,
                     const float* g_save, const float* b_save, int64_t kv_stride, int64_t b_stride, cudaStream_t stream);

// The layer prologue of a prefill pass (kda_prologue.cu): for rows row_shift .. row_shift + pass_rows - 1 of every request,
// the short convolution + SiLU, the L2 norms, the log decay and beta, with the chain's arithmetic, written as core inputs
// (q, k as fp16 bits, v bf16, g f32 log decay [batch * pass_rows][H][128]; beta f32 [batch * pass_rows][H]).  p, a, conv must be
// 8-byte aligned with strides that are multiples of 4 elements.
int layer_prologue_launch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t pass_rows, int32_t row_shift,
                          const glm53f_bf16* p, int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride,
                          const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w, const float* a_log,
                          const float* dt_bias, float lower, glm53f_bf16* q, glm53f_bf16* k, glm53f_bf16* v, float* g, float* beta,
                          cudaStream_t stream);

// The two-pass tensor-core prefill over a workspace (kda_prefill_sp.cu).
int64_t core_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t chunks_per_pass);
// Where a head-sharded prefill sends its outputs: into every rank's full [rows][heads_total][128] buffer, this
// launch's heads at head0.. (up to 8 buffers; they may be peer GPUs' memory mapped into this process).
struct PrefillScatter {
    int ranks = 0;
    glm53f_bf16* full[8] = {};
    int heads_total = 0, head0 = 0;
};

int core_prefill_sp_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len, const glm53f_bf16* q,
                           const glm53f_bf16* k, const glm53f_bf16* v, const float* g, const float* beta, const void* state_in,
                           void* state_out, const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate,
                           const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                           cudaStream_t stream, const PrefillScatter* scatter = nullptr);

// The two-pass prefill on the library's own fixed scratch array (no workspace argument, nothing allocated).
int core_prefill_static_launch(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len, const glm53f_bf16* q,
                               const glm53f_bf16* k, const glm53f_bf16* v, const float* g, const float* beta, const void* state_in,
                               void* state_out, const int64_t* state_off, bool bf16_state, const glm53f_bf16* gate,
                               const glm53f_bf16* norm_w, float eps, glm53f_bf16* out, cudaStream_t stream);

int sm_count();

// Device address of the status word kernels record a timed-out wait in (current device).
int* status_word();

}  // namespace kda
