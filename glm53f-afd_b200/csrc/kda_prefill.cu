// Prefill entry points.
//
// glm53f_kda_prefill*, the layer entry points (reference kernels/kda_prefill.cu:630-742): a prompt segment of any
// length from a committed state and conv window; the window is advanced past the segment in place.
// glm53f_kda_core_prefill_varlen: the same recurrence on post-conv inputs with packed variable-length sequences.
//
// The layer entry points have two forms, chosen by glm53f_kda_prefill_mode (the reference gates its own chunked kernel
// the same way, crates/glm53f-forward/src/forward.rs:210,3580):
//   exact (default)   the row-by-row recurrence of kda_chain.cu: the chain's results bit for bit;
//   chunked           passes of (layer prologue -> chunk-64 tcgen05 kernel of kda_prefill_tc.cu with the gated norm
//                     fused) over the caller's workspace, which holds one pass's core inputs; agrees with the chain
//                     to the rounding of bf16 operands, like every chunked form.  The kernels cover the whole gate
//                     domain of the entry points (lower in [-5.8, 0]).
// The core entry point runs the chunk-64 tcgen05 kernel directly.

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "kda_internal.h"

namespace kda {
namespace {

// The reference's workspace figure: 8,704 floats per 16-row chunk, head and request (kda_prefill.cu:40-43).
constexpr int64_t kChunkRows = 16, kChunkBytes = 8704 * 4;

// 0 = the exact recurrence, 1 = the chunked tensor-core form; GLM53F_KDA_PREFILL=chunked makes 1 the default.
std::atomic<int> g_layer_prefill_mode{[] {
    const char* e = getenv("GLM53F_KDA_PREFILL");
    return e != nullptr && strcmp(e, "chunked") == 0 ? 1 : 0;
}()};

constexpr int kNotEligible = -1;
constexpr int64_t kCoreBytesPerRowHead = 3 * DK * 2 + DK * 4 + 4;  // q, k, v bf16, log decay f32, beta f32

// Batch metadata of a single-request call, written into the workspace (the kernels read metadata on the device).
__global__ void single_request_meta(int32_t* cu, long long* zeros, int32_t rows) {
    cu[0] = 0;
    cu[1] = rows;
    zeros[0] = 0;
}

// The chunked form.  The workspace holds the core inputs of one pass: P rows of every request, P the largest multiple
// of 64 that fits (chunks count from a request's first row, so passes cut at chunk boundaries and the results do not
// depend on the workspace size).  Returns kNotEligible when the call does not meet the kernels' layout requirements
// (dense output rows, aligned rows, room for 64 rows a pass); the caller then runs the exact form.
int chunked_layer_prefill(int32_t heads, int32_t batch, const int32_t* cu_rows, int32_t max_rows, const glm53f_bf16* p,
                          int64_t p_stride, int64_t b_off, const glm53f_bf16* a, int64_t a_stride, const glm53f_bf16* g,
                          int64_t g_stride, const glm53f_bf16* conv, const int64_t* conv_off, const glm53f_bf16* conv_w,
                          const void* state_in, void* state_out, const int64_t* state_off, bool bf16_state, const float* a_log,
                          const float* dt_bias, const glm53f_bf16* norm_w, float eps, float lower, glm53f_bf16* out,
                          int64_t out_stride, float* workspace, int64_t workspace_bytes, cudaStream_t st) {
    auto al = [](const void* x, int n) { return (reinterpret_cast<uintptr_t>(x) & (uintptr_t)(n - 1)) == 0; };
    if (out_stride != (int64_t)heads * DV || !al(out, 16) || !al(workspace, 16) || !al(p, 8) || !al(a, 8) || !al(conv, 8) || !al(conv_w, 16) ||
        !al(dt_bias, 16) || p_stride % 4 || a_stride % 4 || g_stride < (int64_t)heads * DV)
        return kNotEligible;
    constexpr int64_t kMeta = 256;
    int64_t pass = (workspace_bytes - kMeta) / ((int64_t)batch * heads * kCoreBytesPerRowHead) / 64 * 64;
    const int64_t need = ((int64_t)max_rows + 63) / 64 * 64;
    if (pass > need) pass = need;
    if (pass < 64 || (int64_t)batch * pass > 0x7fffffffll) return kNotEligible;
    const int64_t cap = (int64_t)batch * pass * heads;  // (row, head) pairs a pass holds
    unsigned char* w = reinterpret_cast<unsigned char*>(workspace);
    glm53f_bf16* q = reinterpret_cast<glm53f_bf16*>(w);
    glm53f_bf16* k = q + cap * DK;
    glm53f_bf16* v = k + cap * DK;
    float* lg = reinterpret_cast<float*>(v + cap * DK);
    float* beta = lg + cap * DK;
    if (cu_rows == nullptr) {
        int32_t* cu = reinterpret_cast<int32_t*>(beta + cap);
        long long* zeros = reinterpret_cast<long long*>(w + ((reinterpret_cast<unsigned char*>(cu + 2) - w + 15) / 16) * 16);
        single_request_meta<<<1, 1, 0, st>>>(cu, zeros, max_rows);
        cu_rows = cu;
        conv_off = state_off = reinterpret_cast<const int64_t*>(zeros);
    }
    PrefillWindow win;
    win.pass_rows = (int)pass;
    win.gate_stride = g_stride;
    win.qk_fp16 = true;
    for (int64_t shift = 0; shift < max_rows; shift += pass) {
        win.row_shift = (int)shift;
        int rc = layer_prologue_launch(heads, batch, cu_rows, (int)pass, (int)shift, p, p_stride, b_off, a, a_stride, conv, conv_off, conv_w,
                                       a_log, dt_bias, lower, q, k, v, lg, beta, st);
        if (rc != 0) return rc;
        rc = core_prefill_tc_launch(heads, batch, cu_rows, q, k, v, lg, beta, shift == 0 ? state_in : state_out, state_out, state_off,
                                    bf16_state, g, norm_w, eps, out, st, &win);
        if (rc != 0) return rc;
    }
    return 0;
}

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
    if (g_layer_prefill_mode.load() == 1 && (batched ? max_rows : rows) > 0) {
        const int rc = chunked_layer_prefill(heads, batch, cu_rows, batched ? max_rows : rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv,
                                             conv_off, conv_w, state_in, state_out, state_off, bf16_state, a_log, dt_bias, norm_w, eps, lower,
                                             out, out_stride, workspace, workspace_bytes, st);
        if (rc != kNotEligible) {
            if (rc != 0) return rc;
            return conv_shift_launch(3 * heads * DK, 1, batch, cu_rows, nullptr, -1, rows, conv, 0, conv_off, p, 0, p_stride, st);
        }
    }
    int rc = layer_chain_launch(heads, batch, cu_rows, rows, p, p_stride, b_off, a, a_stride, g, g_stride, conv, conv_off, conv_w,
                                state_in, state_out, state_off, bf16_state, a_log, dt_bias, norm_w, eps, lower, out, out_stride, st);
    if (rc != 0) return rc;
    // The window past the segment (reference kda_prefill.cu:687-690); stream order puts it after the chain's reads.
    return conv_shift_launch(3 * heads * DK, 1, batch, cu_rows, nullptr, -1, rows, conv, 0, conv_off, p, 0, p_stride, st);
}

}  // namespace
}  // namespace kda

using namespace kda;

extern "C" int32_t glm53f_kda_prefill_mode(int32_t mode) {
    const int prev = g_layer_prefill_mode.load();
    if (mode == 0 || mode == 1) g_layer_prefill_mode.store(mode);
    return prev;
}

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
