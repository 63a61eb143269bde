// The multi-GPU boundary of the head-sharded prefill for a host that is not Python: how a rank's full output buffer
// becomes an address in every other rank's process.
//
// glm53f_kda_core_prefill_varlen_ws_gather stores each output row into every rank's full [rows][heads_total][128]
// buffer, so each rank (one process per GPU) needs the device addresses of its peers' buffers in its own address space.
// These four functions do that with CUDA IPC and nothing else: a rank exports a handle for the buffer it allocated
// (glm53f_kda_gather_export), the host carries the 128-byte handle to the other ranks by whatever it already has (a
// pipe, a file, its own RPC), each of them opens it (glm53f_kda_gather_open) and passes the mapped address in
// `full[]`; glm53f_kda_gather_close unmaps.  No collective library, no multicast object, no Python.  The reference has
// no counterpart (it runs on one GPU).
//
// The kernels only ever STORE to a peer's buffer (tiled tensor stores and plain stores); nothing is loaded from it.

#include <cstring>

#include <cuda.h>

#include "common.cuh"
#include "glm53f_kda.h"
#include "kda_internal.h"

namespace kda {
namespace {

constexpr uint32_t kMagic = 0x4b474831u;  // "KGH1"

struct Handle {  // the layout behind glm53f_kda_gather_handle's 128 bytes
    uint32_t magic;
    int32_t device;      // the exporting process's device ordinal (informational)
    int64_t offset;      // of the buffer inside its allocation (IPC handles name whole allocations)
    int64_t bytes;       // of the buffer
    cudaIpcMemHandle_t ipc;
};
static_assert(sizeof(Handle) <= sizeof(glm53f_kda_gather_handle), "handle layout");

using GetRange = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
GetRange address_range() {
    static GetRange fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<GetRange>(f);
    }();
    return fn;
}

}  // namespace
}  // namespace kda

using namespace kda;

extern "C" int glm53f_kda_gather_head_range(int32_t heads_total, int32_t rank, int32_t ranks, int32_t* head0, int32_t* heads) {
    if (!head0 || !heads || ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks || heads_total < ranks || heads_total % ranks != 0) return kInvalid;
    *heads = heads_total / ranks;
    *head0 = rank * *heads;
    return 0;
}

extern "C" int glm53f_kda_gather_export(const void* full, int64_t bytes, glm53f_kda_gather_handle* handle) {
    if (!full || !handle || bytes <= 0 || (reinterpret_cast<uintptr_t>(full) & 15) != 0) return kInvalid;
    GetRange range = address_range();
    if (range == nullptr) return (int)cudaErrorNotSupported;
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, (CUdeviceptr) reinterpret_cast<uintptr_t>(full)) != CUDA_SUCCESS) return kInvalid;  // not a device allocation of this process
    const int64_t offset = (int64_t)(reinterpret_cast<uintptr_t>(full) - (uintptr_t)base);
    if (offset + bytes > (int64_t)size) return kInvalid;
    Handle h{};
    h.magic = kMagic;
    cudaError_t e = cudaGetDevice(&h.device);
    if (e != cudaSuccess) return (int)e;
    h.offset = offset;
    h.bytes = bytes;
    e = cudaIpcGetMemHandle(&h.ipc, reinterpret_cast<void*>((uintptr_t)base));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    std::memset(handle, 0, sizeof *handle);
    std::memcpy(handle, &h, sizeof h);
    return 0;
}

extern "C" int glm53f_kda_gather_open(const glm53f_kda_gather_handle* handle, void** full, int64_t* bytes) {
    if (!handle || !full) return kInvalid;
    Handle h;
    std::memcpy(&h, handle, sizeof h);
    if (h.magic != kMagic || h.offset < 0 || h.bytes <= 0) return kInvalid;
    void* base = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&base, h.ipc, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return (int)e;
    }
    *full = reinterpret_cast<unsigned char*>(base) + h.offset;
    if (bytes) *bytes = h.bytes;
    return 0;
}

extern "C" int glm53f_kda_gather_close(const glm53f_kda_gather_handle* handle, void* full) {
    if (!handle || !full) return kInvalid;
    Handle h;
    std::memcpy(&h, handle, sizeof h);
    if (h.magic != kMagic || h.offset < 0) return kInvalid;
    const cudaError_t e = cudaIpcCloseMemHandle(reinterpret_cast<unsigned char*>(full) - h.offset);
    if (e != cudaSuccess) cudaGetLastError();
    return (int)e;
}
