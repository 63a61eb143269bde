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

constexpr int kThreadsShift = 256;

__global__ void __launch_bounds__(kThreadsShift) conv_shift_kernel(int C, const int32_t* __restrict__ cu_rows,
                                                                  const int32_t* __restrict__ keep, int keep1, int rows1,
                                                                  uint16_t* conv, long long conv_stride,
                                                                  const long long* __restrict__ conv_off, const uint16_t* P,
                                                                  long long p_layer_stride, long long p_stride) {
    const long long c = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (c >= C) return;
    const int layer = blockIdx.y, b = blockIdx.z;
    long long row0 = 0;
    int rows = rows1;
    if (cu_rows != nullptr) {
        row0 = cu_rows[b];
        rows = cu_rows[b + 1] - cu_rows[b];
    }
    const int k = keep != nullptr ? keep[b] : (keep1 >= 0 ? keep1 : rows);
    uint16_t* win = conv + (long long)layer * conv_stride + (conv_off != nullptr ? conv_off[b] : 0);
    const uint16_t* new_rows = P + (long long)layer * p_layer_stride + row0 * p_stride;
    const bool vec = C % 8 == 0 && p_stride % 8 == 0 && ((reinterpret_cast<uintptr_t>(win) | reinterpret_cast<uintptr_t>(new_rows)) & 15) == 0;
    if (vec) {
        uint4 v[WINDOW];
#pragma unroll
        for (int j = 0; j < WINDOW; ++j) {
            const int src = k + j;
            const uint16_t* from = src < WINDOW ? win + (long long)src * C + c : new_rows + (long long)(src - WINDOW) * p_stride + c;
            v[j] = *reinterpret_cast<const uint4*>(from);
        }
#pragma unroll
        for (int j = 0; j < WINDOW; ++j) *reinterpret_cast<uint4*>(win + (long long)j * C + c) = v[j];
    } else {
        const int n = (int)(C - c < 8 ? C - c : 8);
        uint16_t v[WINDOW][8];
#pragma unroll
        for (int j = 0; j < WINDOW; ++j) {
            const int src = k + j;
            const uint16_t* from = src < WINDOW ? win + (long long)src * C + c : new_rows + (long long)(src - WINDOW) * p_stride + c;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = i < n ? from[i] : (uint16_t)0;
        }
#pragma unroll
        for (int j = 0; j < WINDOW; ++j)
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < n) win[(long long)j * C + c + i] = v[j][i];
    }
}

}  // namespace

int conv_shift_launch(int32_t channels, int32_t layers, int32_t batch, const int32_t* cu_rows, const int32_t* keep,
                      int32_t keep1, int32_t rows1, glm53f_bf16* conv, int64_t conv_stride, const int64_t* conv_off,
                      const glm53f_bf16* p, int64_t p_layer_stride, int64_t p_stride, cudaStream_t stream) {
    if (channels < 1 || layers < 1 || layers > 65535 || batch < 1 || batch > 65535 || !conv || !p) return kInvalid;
    const dim3 grid(((channels + 7) / 8 + kThreadsShift - 1) / kThreadsShift, layers, batch);
    conv_shift_kernel<<<grid, kThreadsShift, 0, stream>>>(channels, cu_rows, keep, keep1, rows1, conv, conv_stride,
                                                          reinterpret_cast<const long long*>(conv_off), p, p_layer_stride, p_stride);
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
