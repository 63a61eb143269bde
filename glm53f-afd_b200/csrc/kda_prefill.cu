// Prefill entry points.
//
// glm53f_kda_prefill*, the layer entry points (reference kernels/kda_prefill.cu:630-742): a prompt segment of any
// length from a committed state and conv window; the window is advanced past the segment in place.
// glm53f_kda_core_prefill_varlen: the same recurrence on post-conv inputs with packed variable-length sequences.
//
// The layer entry points run the exact row-by-row recurrence of kda_chain.cu (their results are the chain's, bit
// for bit: the model's gate bound of -5 per row is outside the range the chunk-64 tensor-core scheme covers).  The
// core entry point runs the chunk-64 tcgen05 kernel of kda_prefill_tc.cu.

#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kda_internal.h"

namespace kda {
namespace {

// The reference's workspace figure: 8,704 floats per 16-row chunk, head and request (kda_prefill.cu:40-43).
constexpr int64_t kChunkRows = 16, kChunkBytes = 8704 * 4;

// Reference kda_prefill.cu:638-657.
int prefill_entry(int32_t heads, int32_t batch, bool batched, const int32_t* cu_rows, int32_t rows, int32_t max_rows,
                  const glm53f_bf16* p, int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride,
                  const glm53f_bf16* g, int64_t g_stride, glm53f_bf16* conv, const int64_t* conv_off,
                  const glm53f_bf16* conv_w, const void* state_in, void* state_out, const int64_t* state_off,
                  bool bf16_state, const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w, float eps,
                  float lower, glm53f_bf16* out, int64_t out_stride, int32_t value_blocks, float* workspace,
                  int64_t workspace_bytes, glm53f_stream_t stream) {
    if (batched && (!cu_rows || !conv_off || !state_off)) return kInvalid;
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535 || rows < 0 || max_rows < 0 || !p || !a || !g || !conv ||
        !conv_w || !state_in || !state_out || !a_log || !dt_bias || !norm_w || !out || !workspace)
        return kInvalid;
    if (!(lower >= -5.8f && lower <= 0.0f)) return kInvalid;
    if (workspace_bytes / (kChunkBytes * heads * batch) < 1) return kInvalid;
    if (value_blocks != 0 && value_blocks != 1 && value_blocks != 2 && value_blocks != 4) return kInvalid;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = layer_chain_launch(heads, batch, cu_rows, rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off, conv_w,
                                state_in, state_out, state_off, bf16_state, a_log, dt_bias, norm_w, eps, lower, out, out_stride, st);
    if (rc != 0) return rc;
    // The window past the segment (reference kda_prefill.cu:687-690); stream order puts it after the chain's reads.
    return conv_shift_launch(3 * heads * DK, 1, batch, cu_rows, nullptr, -1, rows, conv, 0, conv_off, p, 0, p_stride, st);
}

}  // namespace
}  // namespace kda

using namespace kda;

extern "C" int64_t glm53f_kda_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t rows_per_pass) {
    if (heads < 1 || batch < 1 || rows_per_pass < 1) return 0;
    return (((int64_t)rows_per_pass + kChunkRows - 1) / kChunkRows) * kChunkBytes * heads * batch;
}

extern "C" int glm53f_kda_prefill(int32_t heads, int32_t rows, const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                  const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g, int64_t g_stride,
                                  glm53f_bf16* conv, const glm53f_bf16* conv_w, const float* state_in, float* state_out,
                                  const float* a_log, const float* dt_bias, const glm53f_bf16* norm_w, float eps,
                                  float lower, glm53f_bf16* out, int64_t out_stride, int32_t value_blocks,
                                  float* workspace, int64_t workspace_bytes, glm53f_stream_t stream) {
    return prefill_entry(heads, 1, false, nullptr, rows, rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, nullptr,
                         conv_w, state_in, state_out, nullptr, false, a_log, dt_bias, norm_w, eps, lower, out, out_stride,
                         value_blocks, workspace, workspace_bytes, stream);
}

extern "C" int glm53f_kda_prefill_batch(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t max_rows,
                                        const glm53f_bf16* p, int64_t p_stride, int64_t b_off, const glm53f_bf16* a,
                                        int64_t a_stride, const glm53f_bf16* g, int64_t g_stride, glm53f_bf16* conv,
                                        const int64_t* conv_off, const glm53f_bf16* conv_w, const float* state_in,
                                        float* state_out, const int64_t* state_off, const float* a_log,
                                        const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower,
                                        glm53f_bf16* out, int64_t out_stride, int32_t value_blocks, float* workspace,
                                        int64_t workspace_bytes, glm53f_stream_t stream) {
    return prefill_entry(heads, batch, true, cu_rows, 0, max_rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off,
                         conv_w, state_in, state_out, state_off, false, a_log, dt_bias, norm_w, eps, lower, out, out_stride,
                         value_blocks, workspace, workspace_bytes, stream);
}

extern "C" int glm53f_kda_prefill_batch_bf16state(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t max_rows,
                                                  const glm53f_bf16* p, int64_t p_stride, int64_t b_off,
                                                  const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                                                  int64_t g_stride, glm53f_bf16* conv, const int64_t* conv_off,
                                                  const glm53f_bf16* conv_w, const glm53f_bf16* state_in,
                                                  glm53f_bf16* state_out, const int64_t* state_off, const float* a_log,
                                                  const float* dt_bias, const glm53f_bf16* norm_w, float eps,
                                                  float lower, glm53f_bf16* out, int64_t out_stride,
                                                  int32_t value_blocks, float* workspace, int64_t workspace_bytes,
                                                  glm53f_stream_t stream) {
    return prefill_entry(heads, batch, true, cu_rows, 0, max_rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off,
                         conv_w, state_in, state_out, state_off, true, a_log, dt_bias, norm_w, eps, lower, out, out_stride,
                         value_blocks, workspace, workspace_bytes, stream);
}

extern "C" int glm53f_kda_core_prefill_varlen(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                              const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                              const float* g, const float* beta, const void* state_in, void* state_out,
                                              const int64_t* state_off, int32_t state_bf16, int32_t flags,
                                              const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                              glm53f_bf16* out, glm53f_stream_t stream) {
    if (max_len < 0 || !state_out) return kInvalid;
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535) return kInvalid;
    if (!cu_seqlens || !q || !k || !v || !g || !beta || !state_in || !state_off || !out) return kInvalid;
    if (gate && !norm_w) return kInvalid;
    if (flags & ~GLM53F_KDA_CORE_L2NORM) return kInvalid;
    // The tensor-core path takes 16-byte-aligned dense rows and inputs that are already normalised; anything else
    // (and GLM53F_KDA_PREFILL=chain, for comparisons) runs the exact row-by-row recurrence.
    auto aligned = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    static const bool force_chain = [] {
        const char* e = getenv("GLM53F_KDA_PREFILL");
        return e != nullptr && strcmp(e, "chain") == 0;
    }();
    if (!force_chain && flags == 0 && aligned(q) && aligned(k) && aligned(v) && aligned(g) && aligned(out) &&
        (!gate || (aligned(gate) && aligned(norm_w))))
        return core_prefill_tc_launch(heads, batch, cu_seqlens, q, k, v, g, beta, state_in, state_out, state_off, state_bf16 != 0,
                                      gate, norm_w, eps, out, (cudaStream_t)stream);
    return core_chain_launch(heads, batch, cu_seqlens, q, k, v, g, beta, state_in, state_out, state_off, state_bf16 != 0, flags,
                             gate, norm_w, eps, out, (cudaStream_t)stream);
}

extern "C" int64_t glm53f_kda_core_prefill_workspace_bytes(int32_t heads, int32_t batch, int32_t chunks_per_pass) {
    return core_prefill_workspace_bytes(heads, batch, chunks_per_pass);
}

extern "C" int glm53f_kda_core_prefill_varlen_ws(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                                 const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                                 const float* g, const float* beta, const void* state_in, void* state_out,
                                                 const int64_t* state_off, int32_t state_bf16, int32_t flags,
                                                 const glm53f_bf16* gate, const glm53f_bf16* norm_w, float eps,
                                                 glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                                                 glm53f_stream_t stream) {
    if (max_len < 0 || !state_out || !workspace) return kInvalid;
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535) return kInvalid;
    if (!cu_seqlens || !q || !k || !v || !g || !beta || !state_in || !state_off || !out) return kInvalid;
    if (gate && !norm_w) return kInvalid;
    if (flags != 0) return kInvalid;
    auto aligned = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (!(aligned(q) && aligned(k) && aligned(v) && aligned(g) && aligned(out) && (!gate || (aligned(gate) && aligned(norm_w)))))
        return kInvalid;
    return core_prefill_sp_launch(heads, batch, cu_seqlens, max_len, q, k, v, g, beta, state_in, state_out, state_off,
                                  state_bf16 != 0, gate, norm_w, eps, out, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int glm53f_kda_core_prefill_varlen_ws_gather(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                                        const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                                        const float* g, const float* beta, const void* state_in,
                                                        void* state_out, const int64_t* state_off, int32_t state_bf16,
                                                        int32_t flags, const glm53f_bf16* gate, const glm53f_bf16* norm_w,
                                                        float eps, glm53f_bf16* out, void* workspace, int64_t workspace_bytes,
                                                        glm53f_bf16* const* full, int32_t ranks, int32_t heads_total,
                                                        int32_t head0, glm53f_stream_t stream) {
    if (max_len < 0 || !state_out || !workspace || !full) return kInvalid;
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535) return kInvalid;
    if (ranks < 1 || ranks > 8 || heads_total < heads || heads_total > 65535 || head0 < 0 || head0 + heads > heads_total) return kInvalid;
    if (!cu_seqlens || !q || !k || !v || !g || !beta || !state_in || !state_off) return kInvalid;
    if (gate && !norm_w) return kInvalid;
    if (flags != 0) return kInvalid;
    auto aligned = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (!(aligned(q) && aligned(k) && aligned(v) && aligned(g) && aligned(out) && (!gate || (aligned(gate) && aligned(norm_w)))))
        return kInvalid;
    PrefillScatter sc;
    sc.ranks = ranks; sc.heads_total = heads_total; sc.head0 = head0;
    for (int r = 0; r < ranks; ++r) {
        if (!full[r] || !aligned(full[r])) return kInvalid;
        sc.full[r] = full[r];
    }
    return core_prefill_sp_launch(heads, batch, cu_seqlens, max_len, q, k, v, g, beta, state_in, state_out, state_off,
                                  state_bf16 != 0, gate, norm_w, eps, out, workspace, workspace_bytes, (cudaStream_t)stream, &sc);
}

extern "C" int glm53f_kda_core_prefill_varlen_static(int32_t heads, int32_t batch, const int32_t* cu_seqlens, int32_t max_len,
                                                     const glm53f_bf16* q, const glm53f_bf16* k, const glm53f_bf16* v,
                                                     const float* g, const float* beta, const void* state_in,
                                                     void* state_out, const int64_t* state_off, int32_t state_bf16,
                                                     int32_t flags, const glm53f_bf16* gate, const glm53f_bf16* norm_w,
                                                     float eps, glm53f_bf16* out, glm53f_stream_t stream) {
    if (max_len < 0 || !state_out) return kInvalid;
    if (heads < 1 || heads > 65535 || batch < 1 || batch > 65535) return kInvalid;
    if (!cu_seqlens || !q || !k || !v || !g || !beta || !state_in || !state_off || !out) return kInvalid;
    if (gate && !norm_w) return kInvalid;
    if (flags != 0) return kInvalid;
    auto aligned = [](const void* x) { return (reinterpret_cast<uintptr_t>(x) & 15) == 0; };
    if (!(aligned(q) && aligned(k) && aligned(v) && aligned(g) && aligned(out) && (!gate || (aligned(gate) && aligned(norm_w)))))
        return kInvalid;
    return core_prefill_static_launch(heads, batch, cu_seqlens, max_len, q, k, v, g, beta, state_in, state_out, state_off,
                                      state_bf16 != 0, gate, norm_w, eps, out, (cudaStream_t)stream);
}
