// The conv-window shift: after `keep` rows are accepted, the 3-row window of a (layer, request) becomes rows
// keep .. keep+2 of [old window; new projection rows].  Pure data movement (reference kernels/kda.cu:258-277 for
// the commit's shift, kernels/kda_prefill.cu:574-590 for the prefill's advance past all rows).
//
// One thread moves 8 consecutive channels of all three window rows, as 16-byte vectors when the window and the
// new rows are 16-byte aligned (checked on the device: the per-request offsets live there), else element by
// element; each thread reads its three values before it writes any, so the shift is in place, as the reference's.

#include "common.cuh"
#include "kda_internal.h"

namespace kda {
namespace {

constexpr int kThreadsShift = 256, kVec = 8;  // a thread moves kVec channels of every window row

struct ShiftJob {
    int channels, requests_rows;      // channels per row; rows of the request when there is no row table
    const int32_t* row_table;         // [batch + 1] or null
    const int32_t* kept;              // [batch] or null: then `kept_all` (>= 0), else every row of the request
    int kept_all;
    uint16_t* windows;
    long long window_layer_pitch;
    const long long* window_at;       // [batch] or null
    const uint16_t* fresh;            // the new projection rows
    long long fresh_layer_pitch, fresh_row_pitch;
};

// Where row `pos` of the concatenation [3 old window rows; the request's new rows] lives, at this thread's channels.
__device__ __forceinline__ const uint16_t* stacked_row(const uint16_t* window, const uint16_t* fresh, int pos, int channels, long long fresh_row_pitch,
                                                       long long ch) {
    return pos < WINDOW ? window + (long long)pos * channels + ch : fresh + (long long)(pos - WINDOW) * fresh_row_pitch + ch;
}

__global__ void __launch_bounds__(kThreadsShift) conv_shift_kernel(const ShiftJob job) {
    const long long ch = ((long long)blockIdx.x * kThreadsShift + threadIdx.x) * kVec;
    if (ch >= job.channels) return;
    const int layer = blockIdx.y, req = blockIdx.z;
    long long first_row = 0;
    int n_rows = job.requests_rows;
    if (job.row_table != nullptr) {
        first_row = job.row_table[req];
        n_rows = job.row_table[req + 1] - job.row_table[req];
    }
    const int accepted = job.kept != nullptr ? job.kept[req] : (job.kept_all >= 0 ? job.kept_all : n_rows);
    uint16_t* window = job.windows + layer * job.window_layer_pitch + (job.window_at != nullptr ? job.window_at[req] : 0);
    const uint16_t* fresh = job.fresh + layer * job.fresh_layer_pitch + first_row * job.fresh_row_pitch;
    const bool wide = job.channels % kVec == 0 && job.fresh_row_pitch % kVec == 0 &&
                      ((reinterpret_cast<uintptr_t>(window) | reinterpret_cast<uintptr_t>(fresh)) & 15) == 0;
    // All three source rows are read before the first destination row is written: source and destination overlap.
    if (wide) {
        uint4 held[WINDOW];
#pragma unroll
        for (int w = 0; w < WINDOW; ++w)
            held[w] = *reinterpret_cast<const uint4*>(stacked_row(window, fresh, accepted + w, job.channels, job.fresh_row_pitch, ch));
#pragma unroll
        for (int w = 0; w < WINDOW; ++w) *reinterpret_cast<uint4*>(window + (long long)w * job.channels + ch) = held[w];
    } else {
        const int live = (int)(job.channels - ch < kVec ? job.channels - ch : kVec);
        uint16_t held[WINDOW][kVec];
#pragma unroll
        for (int w = 0; w < WINDOW; ++w) {
            const uint16_t* src = stacked_row(window, fresh, accepted + w, job.channels, job.fresh_row_pitch, ch);
#pragma unroll
            for (int e = 0; e < kVec; ++e) held[w][e] = e < live ? src[e] : (uint16_t)0;
        }
#pragma unroll
        for (int w = 0; w < WINDOW; ++w)
#pragma unroll
            for (int e = 0; e < kVec; ++e)
                if (e < live) window[(long long)w * job.channels + ch + e] = held[w][e];
    }
}

}  // namespace

int conv_shift_launch(int32_t channels, int32_t layers, int32_t batch, const int32_t* cu_rows, const int32_t* keep,
                      int32_t keep1, int32_t rows1, glm53f_bf16* conv, int64_t conv_stride, const int64_t* conv_off,
                      const glm53f_bf16* p, int64_t p_layer_stride, int64_t p_stride, cudaStream_t stream) {
    if (channels < 1 || layers < 1 || layers > 65535 || batch < 1 || batch > 65535 || !conv || !p) return kInvalid;
    ShiftJob job{};
    job.channels = channels; job.requests_rows = rows1;
    job.row_table = cu_rows; job.kept = keep; job.kept_all = keep1;
    job.windows = conv; job.window_layer_pitch = conv_stride; job.window_at = reinterpret_cast<const long long*>(conv_off);
    job.fresh = p; job.fresh_layer_pitch = p_layer_stride; job.fresh_row_pitch = p_stride;
    const dim3 grid(((channels + kVec - 1) / kVec + kThreadsShift - 1) / kThreadsShift, layers, batch);
    conv_shift_kernel<<<grid, kThreadsShift, 0, stream>>>(job);
    return (int)cudaGetLastError();
}

}  // namespace kda

using namespace kda;

// Reference kda.cu:448-451.
extern "C" int glm53f_kda_conv_shift(int32_t channels, int32_t keep, glm53f_bf16* conv, const glm53f_bf16* p,
                                     int64_t p_stride, glm53f_stream_t stream) {
    if (keep < 0) return kInvalid;
    return conv_shift_launch(channels, 1, 1, nullptr, nullptr, keep, 0, conv, 0, nullptr, p, 0, p_stride, (cudaStream_t)stream);
}

// Reference kda.cu:453-460.
extern "C" int glm53f_kda_conv_shift_batch(int32_t channels, int32_t layers, int32_t batch, const int32_t* cu_rows,
                                           const int32_t* keep, glm53f_bf16* conv, int64_t conv_stride,
                                           const int64_t* conv_off, const glm53f_bf16* p, int64_t p_layer_stride,
                                           int64_t p_stride, glm53f_stream_t stream) {
    if (!cu_rows || !keep || !conv_off) return kInvalid;
    return conv_shift_launch(channels, layers, batch, cu_rows, keep, 0, 0, conv, conv_stride, conv_off, p, p_layer_stride, p_stride,
                             (cudaStream_t)stream);
}
