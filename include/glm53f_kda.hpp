// Checked C++ wrappers over the thirteen reference entry points of glm53f_kda.h: the host API of the reference crate.
//
// A header-only mirror of crates/glm53f-kda/src/kernel.rs (same type and function names, fields, argument meaning and
// error behaviour) and of the parts of src/device.rs it needs.  Each launch checks on the host that every buffer is
// large enough for the geometry it is given, that written regions do not overlap and that the batch metadata is
// consistent, then enqueues the kernel; a rejection throws Error{Invalid} (the reference's Error::Invalid), any other
// non-zero status Error{Cuda} (kernel.rs:127-135).  Launches are asynchronous on the given stream; buffers must
// outlive the stream's work.
//
//   Weights (kernel.rs:15-52)      RowView (55-105)          Saves (138-179)        StateOut (182-190)
//   StateType (193-211)            Chain (223-326)           replay (330-365)       conv_shift (369-394)
//   Request (397-405)              BatchMeta (409-526)       ChainBatch (530-679)   LayerSaves (682-737)
//   replay_layers (741-777)        replay_batch[_bf16_state] (782-905)              conv_shift_batch (912-973)
//   PrefillWorkspace (992-1041)    Prefill (1055-1141)       PrefillBatch (1146-1285)
//   DeviceBuffer, Stream (device.rs:10-286)
//
// With GLM53F_KDA_HOST_ONLY defined, DeviceBuffer keeps its bytes in host memory and needs no CUDA runtime: the
// host-side checks can then be exercised on a machine without a GPU (nothing is launched when a check rejects).
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#ifndef GLM53F_KDA_HOST_ONLY
#include <cuda_runtime_api.h>
#endif

#include "glm53f_kda.h"

namespace glm53f {
namespace kda {

constexpr size_t DK = 128, DV = 128, TAPS = 4, WINDOW = TAPS - 1;
constexpr float PREFILL_LOWER_MIN = -5.8f;  // kernel.rs:977
inline size_t channels(size_t heads) { return 3 * heads * DK; }
inline size_t state_len(size_t heads) { return heads * DV * DK; }

struct Error : std::runtime_error {
    enum Kind { Invalid, Cuda } kind;
    int code;
    Error(Kind k, int c, const std::string& what) : std::runtime_error(what), kind(k), code(c) {}
};
[[noreturn]] inline void invalid(const std::string& what) { throw Error(Error::Invalid, 1, what); }
inline void launched(int code, const char* what) {
    if (code == 0) return;
    if (code == 1) invalid(std::string(what) + ": rejected by the launcher");
    throw Error(Error::Cuda, code, std::string(what) + ": CUDA error " + std::to_string(code));
}
inline int32_t to_i32(size_t x, const char* what) {
    if (x > 0x7fffffffull) invalid(std::string(what) + " = " + std::to_string(x) + " does not fit in 32 bits");
    return (int32_t)x;
}

// Bytes of device memory (device.rs:10-160).
class DeviceBuffer {
   public:
    DeviceBuffer() = default;
    DeviceBuffer(const DeviceBuffer&) = delete;
    DeviceBuffer& operator=(const DeviceBuffer&) = delete;
    DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr, o.n_ = 0; }
    DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
        if (this != &o) { release(); p_ = o.p_, n_ = o.n_, o.p_ = nullptr, o.n_ = 0; }
        return *this;
    }
    ~DeviceBuffer() { release(); }

    static DeviceBuffer alloc(size_t bytes) {
        DeviceBuffer b;
        b.n_ = bytes;
        if (bytes == 0) return b;
#ifdef GLM53F_KDA_HOST_ONLY
        b.p_ = std::malloc(bytes);
        if (!b.p_) throw Error(Error::Cuda, 2, "out of memory");
#else
        const cudaError_t e = cudaMalloc(&b.p_, bytes);
        if (e != cudaSuccess) throw Error(Error::Cuda, (int)e, "cudaMalloc");
#endif
        return b;
    }
    static DeviceBuffer zeroed(size_t bytes) {
        DeviceBuffer b = alloc(bytes);
        if (bytes) {
#ifdef GLM53F_KDA_HOST_ONLY
            std::memset(b.p_, 0, bytes);
#else
            const cudaError_t e = cudaMemset(b.p_, 0, bytes);
            if (e != cudaSuccess) throw Error(Error::Cuda, (int)e, "cudaMemset");
#endif
        }
        return b;
    }
    template <typename T>
    static DeviceBuffer from_slice(const std::vector<T>& v) {
        DeviceBuffer b = alloc(v.size() * sizeof(T));
        b.upload_at(0, v);
        return b;
    }
    size_t bytes() const { return n_; }
    const void* as_ptr() const { return p_; }
    // Address of element `offset` of type T.
    template <typename T = unsigned char>
    T* ptr(size_t offset = 0) const { return reinterpret_cast<T*>(static_cast<unsigned char*>(p_) + offset * sizeof(T)); }
    template <typename T>
    void upload(const std::vector<T>& v) { upload_at(0, v); }
    // Copies v to element `offset` (elements of T); synchronous.
    template <typename T>
    void upload_at(size_t offset, const std::vector<T>& v) {
        const size_t at = offset * sizeof(T), nb = v.size() * sizeof(T);
        if (at + nb > n_) invalid("upload beyond the buffer");
        if (nb == 0) return;
#ifdef GLM53F_KDA_HOST_ONLY
        std::memcpy(static_cast<unsigned char*>(p_) + at, v.data(), nb);
#else
        const cudaError_t e = cudaMemcpy(static_cast<unsigned char*>(p_) + at, v.data(), nb, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) throw Error(Error::Cuda, (int)e, "cudaMemcpy");
#endif
    }
    // The n elements of T from element `offset`, on the host; synchronous.
    template <typename T>
    std::vector<T> download(size_t n, size_t offset = 0) const {
        if ((offset + n) * sizeof(T) > n_) invalid("download beyond the buffer");
        std::vector<T> v(n);
        if (n == 0) return v;
#ifdef GLM53F_KDA_HOST_ONLY
        std::memcpy(v.data(), static_cast<const unsigned char*>(p_) + offset * sizeof(T), n * sizeof(T));
#else
        const cudaError_t e = cudaMemcpy(v.data(), static_cast<const unsigned char*>(p_) + offset * sizeof(T), n * sizeof(T), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) throw Error(Error::Cuda, (int)e, "cudaMemcpy");
#endif
        return v;
    }

   private:
    void release() {
        if (!p_) return;
#ifdef GLM53F_KDA_HOST_ONLY
        std::free(p_);
#else
        cudaFree(p_);
#endif
        p_ = nullptr;
    }
    void* p_ = nullptr;
    size_t n_ = 0;
};

// A CUDA stream (device.rs:163-230); nullptr is the legacy default stream.
struct Stream {
    glm53f_stream_t raw_ = nullptr;
    glm53f_stream_t raw() const { return raw_; }
};

// bf16 <-> f32, round to nearest even (src/bf16.rs:6-23).
inline uint16_t bf16_from_f32(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
inline float bf16_to_f32(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float x;
    std::memcpy(&x, &u, 4);
    return x;
}
inline std::vector<uint16_t> bf16_encode(const std::vector<float>& v) {
    std::vector<uint16_t> o(v.size());
    std::transform(v.begin(), v.end(), o.begin(), bf16_from_f32);
    return o;
}
inline std::vector<float> bf16_decode(const std::vector<uint16_t>& v) {
    std::vector<float> o(v.size());
    std::transform(v.begin(), v.end(), o.begin(), bf16_to_f32);
    return o;
}

// One layer's parameters on the host (src/cpu.rs:86-100).
struct LayerParams {
    size_t heads = 0;
    std::vector<float> conv_w, a_log, dt_bias, norm_w;
    float eps = 1e-5f, lower = -5.0f;
};

// One layer's weights on the device (kernel.rs:15-52).
struct Weights {
    size_t heads = 0;
    DeviceBuffer conv_w, a_log, dt_bias, norm_w;  // bf16 [C][TAPS], f32 [H], f32 [H * DK], bf16 [DV]
    float eps = 1e-5f, lower = -5.0f;
    static Weights upload(const LayerParams& p) {
        if (p.conv_w.size() != channels(p.heads) * TAPS || p.a_log.size() != p.heads || p.dt_bias.size() != p.heads * DK || p.norm_w.size() != DV)
            invalid("layer parameters have the wrong sizes");
        Weights w;
        w.heads = p.heads;
        w.conv_w = DeviceBuffer::from_slice(bf16_encode(p.conv_w));
        w.a_log = DeviceBuffer::from_slice(p.a_log);
        w.dt_bias = DeviceBuffer::from_slice(p.dt_bias);
        w.norm_w = DeviceBuffer::from_slice(bf16_encode(p.norm_w));
        w.eps = p.eps, w.lower = p.lower;
        return w;
    }
};

// Rows in a device buffer: row r starts at element offset + r * stride (kernel.rs:55-105).
struct RowView {
    const DeviceBuffer* buf = nullptr;
    size_t offset = 0, stride = 0;
    static RowView create(const DeviceBuffer& b, size_t offset, size_t stride) { return RowView{&b, offset, stride}; }
    static RowView dense(const DeviceBuffer& b, size_t width) { return RowView{&b, 0, width}; }
    // Rows first .. first + rows have columns [lo, hi) inside the buffer (elements of `size` bytes).
    void check(const char* what, size_t size, size_t first, size_t rows, long long lo, long long hi) const {
        if (rows == 0) return;
        const long long len = (long long)(buf->bytes() / size);
        const long long start = (long long)offset + (long long)first * (long long)stride;
        const long long mn = start + lo, mx = start + (long long)(rows - 1) * (long long)stride + hi;
        if (mn < 0 || mx > len)
            invalid(std::string(what) + ": rows reach elements [" + std::to_string(mn) + ", " + std::to_string(mx) + ") of a buffer of " + std::to_string(len));
    }
    const glm53f_bf16* ptr() const { return buf->ptr<glm53f_bf16>(offset); }
};

inline void check_region(const char* what, const DeviceBuffer& buf, size_t size, size_t offset, size_t n) {
    const size_t len = buf.bytes() / size;
    if (offset + n < offset || offset + n > len)
        invalid(std::string(what) + ": elements [" + std::to_string(offset) + ", " + std::to_string(offset) + " + " + std::to_string(n) + ") exceed a buffer of " + std::to_string(len));
}
inline bool same(const DeviceBuffer& a, const DeviceBuffer& b) { return a.as_ptr() == b.as_ptr() && a.bytes() > 0; }
inline bool coincide_or_disjoint(size_t a, size_t b, size_t n) { return a == b || a + n <= b || b + n <= a; }

// The first rows of a Saves on the host (the reference's cpu::Saves).
struct HostSaves {
    size_t heads = 0, rows = 0;
    std::vector<float> k, v, g, beta;
};

// Per-row replay inputs on the device, for up to `rows` rows of `heads` heads, one layer (kernel.rs:138-179).
struct Saves {
    size_t heads = 0, rows = 0;
    DeviceBuffer k, v, g, b;  // f32 [rows][H][DK], bf16 [rows][H][DV], f32 [rows][H][DK], f32 [rows][H]
    static Saves alloc(size_t heads, size_t rows) {
        Saves s;
        s.heads = heads, s.rows = rows;
        s.k = DeviceBuffer::zeroed(rows * heads * DK * 4);
        s.v = DeviceBuffer::zeroed(rows * heads * DV * 2);
        s.g = DeviceBuffer::zeroed(rows * heads * DK * 4);
        s.b = DeviceBuffer::zeroed(rows * heads * 4);
        return s;
    }
    HostSaves download(size_t n) const {
        return HostSaves{heads, n, k.download<float>(n * heads * DK), bf16_decode(v.download<uint16_t>(n * heads * DV)), g.download<float>(n * heads * DK),
                         b.download<float>(n * heads)};
    }
};

// Where a chain writes the state after its last row (kernel.rs:182-190).
struct StateOut {
    enum Kind { Skip, InPlace, To } kind = InPlace;
    const DeviceBuffer* buf = nullptr;
    size_t offset = 0;
    static StateOut skip() { return StateOut{Skip, nullptr, 0}; }
    static StateOut in_place() { return StateOut{InPlace, nullptr, 0}; }
    static StateOut to(const DeviceBuffer& b, size_t offset = 0) { return StateOut{To, &b, offset}; }
};

// How a batch launch's states are stored (kernel.rs:193-211).
enum class StateType { F32, Bf16 };
inline size_t bytes(StateType t) { return t == StateType::F32 ? 4 : 2; }

namespace detail {
struct SavePtrs {
    float* k = nullptr;
    glm53f_bf16* v = nullptr;
    float* g = nullptr;
    float* b = nullptr;
};
inline SavePtrs check_saves(const Saves* s, size_t heads, size_t rows) {
    if (!s) return SavePtrs{};
    if (s->heads != heads || s->rows < rows) invalid("saves hold " + std::to_string(s->rows) + " rows of " + std::to_string(s->heads) + " heads");
    return SavePtrs{s->k.ptr<float>(), s->v.ptr<glm53f_bf16>(), s->g.ptr<float>(), s->b.ptr<float>()};
}
inline void check_rows(size_t heads, size_t total, const RowView& p, long long b_off, const RowView& a, const RowView& g, const RowView& out) {
    const long long c = (long long)channels(heads);
    p.check("p", 2, 0, total, std::min<long long>(b_off, 0), std::max<long long>(c, b_off + (long long)heads));
    a.check("a", 2, 0, total, 0, (long long)(heads * DK));
    g.check("g", 2, 0, total, 0, (long long)(heads * DV));
    out.check("out", 2, 0, total, 0, (long long)(heads * DV));
    if (total > 1 && out.stride < heads * DV) invalid("out rows overlap");
}
}  // namespace detail

// One layer, one request: `rows` rows from the committed state (glm53f_kda_chain; kernel.rs:223-326).
struct Chain {
    const Weights* weights = nullptr;
    size_t rows = 0;
    RowView p;             // row r: q | k | v in columns [0, C), the beta logits in [b_off, b_off + H)
    long long b_off = 0;
    RowView a, g;          // forget-gate projections [H * DK] per row; output-gate projections [H * DV] per row
    const DeviceBuffer* conv = nullptr;   // the conv window [WINDOW][C] at conv_offset
    size_t conv_offset = 0;
    const DeviceBuffer* state = nullptr;  // the state [H][DV][DK] at state_offset
    size_t state_offset = 0;
    StateOut state_out;
    RowView out;           // outputs, [H * DV] per row
    const Saves* saves = nullptr;

    void launch(const Stream& stream) const {
        const size_t h = weights->heads;
        if (rows == 0) invalid("a chain needs at least one row");
        detail::check_rows(h, rows, p, b_off, a, g, out);
        check_region("conv", *conv, 2, conv_offset, WINDOW * channels(h));
        check_region("state", *state, 4, state_offset, state_len(h));
        float* so = nullptr;
        if (state_out.kind == StateOut::InPlace) so = state->ptr<float>(state_offset);
        else if (state_out.kind == StateOut::To) {
            check_region("state_out", *state_out.buf, 4, state_out.offset, state_len(h));
            if (same(*state_out.buf, *state) && !coincide_or_disjoint(state_out.offset, state_offset, state_len(h))) invalid("state_out partly overlaps the state");
            so = state_out.buf->ptr<float>(state_out.offset);
        }
        const detail::SavePtrs sv = detail::check_saves(saves, h, rows);
        const Weights& w = *weights;
        launched(glm53f_kda_chain(to_i32(h, "heads"), to_i32(rows, "rows"), p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(), (int64_t)g.stride,
                                  conv->ptr<glm53f_bf16>(conv_offset), w.conv_w.ptr<glm53f_bf16>(), state->ptr<float>(state_offset), so, w.a_log.ptr<float>(),
                                  w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(), w.eps, w.lower, out.buf->ptr<glm53f_bf16>(out.offset), (int64_t)out.stride,
                                  sv.k, sv.v, sv.g, sv.b, stream.raw()),
                 "glm53f_kda_chain");
    }
};

// One layer, one request: the state after the first `rows` saved rows (glm53f_kda_replay; kernel.rs:330-365).
inline void replay(size_t heads, size_t rows, const DeviceBuffer& state, size_t state_offset, const DeviceBuffer& state_out, size_t out_offset, const Saves& saves,
                   const Stream& stream) {
    check_region("state", state, 4, state_offset, state_len(heads));
    check_region("state_out", state_out, 4, out_offset, state_len(heads));
    if (same(state, state_out) && !coincide_or_disjoint(state_offset, out_offset, state_len(heads))) invalid("state_out partly overlaps the state");
    if (saves.heads != heads || saves.rows < rows) invalid("saves hold " + std::to_string(saves.rows) + " rows of " + std::to_string(saves.heads) + " heads");
    launched(glm53f_kda_replay(to_i32(heads, "heads"), to_i32(rows, "rows"), state.ptr<float>(state_offset), state_out.ptr<float>(out_offset), saves.k.ptr<float>(),
                               saves.v.ptr<glm53f_bf16>(), saves.g.ptr<float>(), saves.b.ptr<float>(), stream.raw()),
             "glm53f_kda_replay");
}

// Advance one conv window past `keep` kept rows of p, in place (glm53f_kda_conv_shift; kernel.rs:369-394).
inline void conv_shift(size_t heads, size_t keep, const DeviceBuffer& conv, size_t conv_offset, const RowView& p, const Stream& stream) {
    const size_t c = channels(heads);
    check_region("conv", conv, 2, conv_offset, WINDOW * c);
    const size_t first = keep > WINDOW ? keep - WINDOW : 0;  // the shift reads new rows keep - WINDOW .. keep
    p.check("p", 2, first, keep - first, 0, (long long)c);
    launched(glm53f_kda_conv_shift(to_i32(c, "channels"), to_i32(keep, "keep"), conv.ptr<glm53f_bf16>(conv_offset), p.ptr(), (int64_t)p.stride, stream.raw()),
             "glm53f_kda_conv_shift");
}

// One request of a batch (kernel.rs:397-405).
struct Request {
    size_t rows = 0, conv_offset = 0, state_offset = 0;
};

// Batch metadata on the device, with a host copy for the checks (kernel.rs:409-526).
class BatchMeta {
   public:
    explicit BatchMeta(size_t capacity)
        : capacity_(capacity), cu_rows(DeviceBuffer::zeroed((capacity + 1) * 4)), keep_d(DeviceBuffer::zeroed(capacity * 4)),
          conv_off(DeviceBuffer::zeroed(capacity * 8)), state_off(DeviceBuffer::zeroed(capacity * 8)) {}

    // Sets the requests and, for replays and conv shifts, the rows each keeps (nullptr: all).  Copies synchronously.
    void set(const std::vector<Request>& requests, const std::vector<size_t>* keep = nullptr) {
        if (requests.empty() || requests.size() > capacity_) invalid(std::to_string(requests.size()) + " requests for a capacity of " + std::to_string(capacity_));
        std::vector<size_t> kp;
        if (keep) {
            if (keep->size() != requests.size()) invalid("one keep per request");
            kp = *keep;
        } else
            for (const Request& r : requests) kp.push_back(r.rows);
        for (size_t i = 0; i < requests.size(); ++i)
            if (kp[i] > requests[i].rows) invalid("keep " + std::to_string(kp[i]) + " exceeds the request's " + std::to_string(requests[i].rows) + " rows");
        std::vector<int32_t> cu(requests.size() + 1, 0), k32;
        for (size_t i = 0; i < requests.size(); ++i) {
            const long long next = (long long)cu[i] + to_i32(requests[i].rows, "rows");
            if (next > 0x7fffffffll) invalid("total rows do not fit in 32 bits");
            cu[i + 1] = (int32_t)next;
        }
        for (size_t k : kp) k32.push_back(to_i32(k, "keep"));
        std::vector<int64_t> co, so;
        for (const Request& r : requests) co.push_back((int64_t)r.conv_offset), so.push_back((int64_t)r.state_offset);
        cu_rows.upload(cu);
        keep_d.upload(k32);
        conv_off.upload(co);
        state_off.upload(so);
        requests_ = requests;
    }
    const std::vector<Request>& requests() const { return requests_; }
    size_t total_rows() const {
        size_t n = 0;
        for (const Request& r : requests_) n += r.rows;
        return n;
    }
    int32_t batch() const {
        if (requests_.empty()) invalid("batch metadata not set");
        return to_i32(requests_.size(), "batch");
    }
    // Each request's region of n elements at offset(r) inside the buffer, pairwise disjoint when `disjoint`.
    template <typename F>
    void check_regions(const char* what, const DeviceBuffer& buf, size_t size, size_t base, size_t n, bool disjoint, F&& offset) const {
        std::vector<size_t> spans;
        for (const Request& r : requests_) {
            check_region(what, buf, size, base + offset(r), n);
            spans.push_back(offset(r));
        }
        if (disjoint) {
            std::sort(spans.begin(), spans.end());
            for (size_t i = 1; i < spans.size(); ++i)
                if (spans[i] < spans[i - 1] + n) invalid(std::string(what) + ": requests' regions overlap");
        }
    }

   private:
    size_t capacity_;
    std::vector<Request> requests_;

   public:
    DeviceBuffer cu_rows, keep_d, conv_off, state_off;  // int32 [batch + 1], int32 [batch], int64 [batch], int64 [batch]
};

namespace detail {
inline void* batch_state_out(const BatchMeta& meta, const StateOut& so, const DeviceBuffer& state, size_t es, size_t heads, bool allow_skip) {
    if (so.kind == StateOut::Skip) {
        if (!allow_skip) invalid("a prefill always writes its state");
        return nullptr;
    }
    if (so.kind == StateOut::InPlace) return state.ptr<unsigned char>();
    meta.check_regions("state_out", *so.buf, es, 0, state_len(heads), true, [](const Request& r) { return r.state_offset; });
    if (same(*so.buf, state)) invalid("state_out is the state buffer: use InPlace");
    return so.buf->ptr<unsigned char>();
}
}  // namespace detail

// One layer, a batch of requests (glm53f_kda_chain_batch; kernel.rs:530-679).
struct ChainBatch {
    const Weights* weights = nullptr;
    RowView p;
    long long b_off = 0;
    RowView a, g;
    const DeviceBuffer* conv = nullptr;   // conv windows, at each request's conv_offset
    const DeviceBuffer* state = nullptr;  // states, at each request's state_offset
    StateOut state_out;                   // To(buf, _) writes at each request's state_offset in buf
    RowView out;
    const Saves* saves = nullptr;

    void launch(const BatchMeta& meta, const Stream& stream) const { launch_as(meta, stream, StateType::F32); }
    // With bf16 states (glm53f_kda_chain_batch_bf16state): the requests' state_offsets count bf16 elements.
    void launch_bf16_state(const BatchMeta& meta, const Stream& stream) const { launch_as(meta, stream, StateType::Bf16); }

   private:
    void launch_as(const BatchMeta& meta, const Stream& stream, StateType st) const {
        const size_t es = bytes(st), h = weights->heads;
        const int32_t batch = meta.batch();
        const size_t total = meta.total_rows();
        detail::check_rows(h, total, p, b_off, a, g, out);
        meta.check_regions("conv", *conv, 2, 0, WINDOW * channels(h), false, [](const Request& r) { return r.conv_offset; });
        meta.check_regions("state", *state, es, 0, state_len(h), true, [](const Request& r) { return r.state_offset; });
        void* so = detail::batch_state_out(meta, state_out, *state, es, h, true);
        const detail::SavePtrs sv = detail::check_saves(saves, h, total);
        const Weights& w = *weights;
        const int32_t heads = to_i32(h, "heads");
        int code;
        if (st == StateType::F32)
            code = glm53f_kda_chain_batch(heads, batch, meta.cu_rows.ptr<int32_t>(), p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(), (int64_t)g.stride,
                                          conv->ptr<glm53f_bf16>(), meta.conv_off.ptr<int64_t>(), w.conv_w.ptr<glm53f_bf16>(), state->ptr<float>(), static_cast<float*>(so),
                                          meta.state_off.ptr<int64_t>(), w.a_log.ptr<float>(), w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(), w.eps, w.lower,
                                          out.buf->ptr<glm53f_bf16>(out.offset), (int64_t)out.stride, sv.k, sv.v, sv.g, sv.b, stream.raw());
        else
            code = glm53f_kda_chain_batch_bf16state(heads, batch, meta.cu_rows.ptr<int32_t>(), p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(),
                                                    (int64_t)g.stride, conv->ptr<glm53f_bf16>(), meta.conv_off.ptr<int64_t>(), w.conv_w.ptr<glm53f_bf16>(),
                                                    state->ptr<glm53f_bf16>(), static_cast<glm53f_bf16*>(so), meta.state_off.ptr<int64_t>(), w.a_log.ptr<float>(),
                                                    w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(), w.eps, w.lower, out.buf->ptr<glm53f_bf16>(out.offset),
                                                    (int64_t)out.stride, sv.k, sv.v, sv.g, sv.b, stream.raw());
        launched(code, "glm53f_kda_chain_batch");
    }
};

// Saves for several layers in one allocation each: what a commit replays at once (kernel.rs:682-737).
struct LayerSaves {
    size_t layers = 0, heads = 0, rows = 0;
    DeviceBuffer k, v, g, b;
    static LayerSaves alloc(size_t layers, size_t heads, size_t rows) {
        LayerSaves s;
        s.layers = layers, s.heads = heads, s.rows = rows;
        s.k = DeviceBuffer::zeroed(layers * rows * heads * DK * 4);
        s.v = DeviceBuffer::zeroed(layers * rows * heads * DV * 2);
        s.g = DeviceBuffer::zeroed(layers * rows * heads * DK * 4);
        s.b = DeviceBuffer::zeroed(layers * rows * heads * 4);
        return s;
    }
    size_t kv_stride() const { return rows * heads * DK; }
    size_t b_stride() const { return rows * heads; }
    void fill_layer(size_t layer, const Saves& s, size_t n) {
        if (layer >= layers || s.heads != heads || n > std::min(rows, s.rows)) invalid("fill_layer: shape mismatch");
        k.upload_at(layer * kv_stride(), s.k.download<float>(n * heads * DK));
        v.upload_at(layer * kv_stride(), s.v.download<uint16_t>(n * heads * DV));
        g.upload_at(layer * kv_stride(), s.g.download<float>(n * heads * DK));
        b.upload_at(layer * b_stride(), s.b.download<float>(n * heads));
    }
};

// Several layers, one request: layer l's state is at l * state_stride (glm53f_kda_replay_layers; kernel.rs:741-777).
inline void replay_layers(size_t rows, const DeviceBuffer& state, const DeviceBuffer& state_out, size_t state_stride, const LayerSaves& saves, const Stream& stream) {
    const size_t h = saves.heads, l = saves.layers;
    if (l == 0 || rows > saves.rows || state_stride < state_len(h)) invalid("replay_layers: no layers, rows beyond the saves, or overlapping layers");
    check_region("state", state, 4, (l - 1) * state_stride, state_len(h));
    check_region("state", state_out, 4, (l - 1) * state_stride, state_len(h));
    launched(glm53f_kda_replay_layers(to_i32(h, "heads"), to_i32(l, "layers"), to_i32(rows, "rows"), state.ptr<float>(), state_out.ptr<float>(), (int64_t)state_stride,
                                      saves.k.ptr<float>(), saves.v.ptr<glm53f_bf16>(), saves.g.ptr<float>(), saves.b.ptr<float>(), (int64_t)saves.kv_stride(),
                                      (int64_t)saves.b_stride(), stream.raw()),
             "glm53f_kda_replay_layers");
}

namespace detail {
inline void replay_batch_as(const BatchMeta& meta, const DeviceBuffer& state, const DeviceBuffer& state_out, size_t state_stride, const LayerSaves& saves,
                            const Stream& stream, StateType st) {
    const size_t h = saves.heads, l = saves.layers;
    const int32_t batch = meta.batch();
    if (l == 0 || meta.total_rows() > saves.rows) invalid("replay_batch: no layers, or more rows than the saves hold");
    auto off = [](const Request& r) { return r.state_offset; };
    meta.check_regions("state", state, bytes(st), (l - 1) * state_stride, state_len(h), true, off);
    meta.check_regions("state", state_out, bytes(st), (l - 1) * state_stride, state_len(h), true, off);
    if (l > 1) {
        size_t max_off = 0;
        for (const Request& r : meta.requests()) max_off = std::max(max_off, r.state_offset);
        if (state_stride < max_off + state_len(h)) invalid("replay_batch: layers' regions overlap");
    }
    const int32_t heads = to_i32(h, "heads"), layers = to_i32(l, "layers");
    int code;
    if (st == StateType::F32)
        code = glm53f_kda_replay_batch(heads, layers, batch, meta.cu_rows.ptr<int32_t>(), meta.keep_d.ptr<int32_t>(), state.ptr<float>(), state_out.ptr<float>(),
                                       (int64_t)state_stride, meta.state_off.ptr<int64_t>(), saves.k.ptr<float>(), saves.v.ptr<glm53f_bf16>(), saves.g.ptr<float>(),
                                       saves.b.ptr<float>(), (int64_t)saves.kv_stride(), (int64_t)saves.b_stride(), stream.raw());
    else
        code = glm53f_kda_replay_batch_bf16state(heads, layers, batch, meta.cu_rows.ptr<int32_t>(), meta.keep_d.ptr<int32_t>(), state.ptr<glm53f_bf16>(),
                                                 state_out.ptr<glm53f_bf16>(), (int64_t)state_stride, meta.state_off.ptr<int64_t>(), saves.k.ptr<float>(),
                                                 saves.v.ptr<glm53f_bf16>(), saves.g.ptr<float>(), saves.b.ptr<float>(), (int64_t)saves.kv_stride(),
                                                 (int64_t)saves.b_stride(), stream.raw());
    launched(code, "glm53f_kda_replay_batch");
}
}  // namespace detail

// Every (layer, request): the state after the request's first keep[b] saved rows (kernel.rs:782-822).
inline void replay_batch(const BatchMeta& meta, const DeviceBuffer& state, const DeviceBuffer& state_out, size_t state_stride, const LayerSaves& saves, const Stream& s) {
    detail::replay_batch_as(meta, state, state_out, state_stride, saves, s, StateType::F32);
}
inline void replay_batch_bf16_state(const BatchMeta& meta, const DeviceBuffer& state, const DeviceBuffer& state_out, size_t state_stride, const LayerSaves& saves,
                                    const Stream& s) {
    detail::replay_batch_as(meta, state, state_out, state_stride, saves, s, StateType::Bf16);
}

// Every (layer, request): the conv window past the request's kept rows (glm53f_kda_conv_shift_batch; kernel.rs:912-973).
inline void conv_shift_batch(size_t heads, size_t layers, const BatchMeta& meta, const DeviceBuffer& conv, size_t conv_stride, const RowView& p, size_t p_layer_stride,
                             const Stream& stream) {
    const size_t c = channels(heads);
    const int32_t batch = meta.batch();
    if (layers == 0) invalid("conv_shift_batch: no layers");
    size_t max_off = 0;
    for (const Request& r : meta.requests()) max_off = std::max(max_off, r.conv_offset);
    if (layers > 1 && conv_stride < max_off + WINDOW * c) invalid("conv_shift_batch: layers' windows overlap");
    meta.check_regions("conv", conv, 2, (layers - 1) * conv_stride, WINDOW * c, true, [](const Request& r) { return r.conv_offset; });
    for (size_t l : {size_t(0), layers - 1}) RowView{p.buf, p.offset + l * p_layer_stride, p.stride}.check("p", 2, 0, meta.total_rows(), 0, (long long)c);
    launched(glm53f_kda_conv_shift_batch(to_i32(c, "channels"), to_i32(layers, "layers"), batch, meta.cu_rows.ptr<int32_t>(), meta.keep_d.ptr<int32_t>(),
                                         conv.ptr<glm53f_bf16>(), (int64_t)conv_stride, meta.conv_off.ptr<int64_t>(), p.ptr(), (int64_t)p_layer_stride, (int64_t)p.stride,
                                         stream.raw()),
             "glm53f_kda_conv_shift_batch");
}

inline void check_lower(float lower) {
    if (!(lower >= PREFILL_LOWER_MIN && lower <= 0.0f)) invalid("prefill: gate lower bound " + std::to_string(lower) + " outside [-5.8, 0]");
}
inline int32_t check_value_blocks(size_t vb) {
    if (vb != 0 && vb != 1 && vb != 2 && vb != 4) invalid("value_blocks " + std::to_string(vb) + ": 0 (choose), 1, 2 or 4");
    return (int32_t)vb;
}

// Device workspace for the prefill entry points (kernel.rs:992-1041).
struct PrefillWorkspace {
    size_t heads = 0, batch = 0, rows_per_pass = 0;
    DeviceBuffer buf;
    static PrefillWorkspace create(size_t heads, size_t batch, size_t rows_per_pass) {
        const size_t rows = std::max<size_t>(rows_per_pass, 1);
        const int64_t nbytes = glm53f_kda_prefill_workspace_bytes(to_i32(heads, "heads"), to_i32(batch, "batch"), to_i32(rows, "rows_per_pass"));
        PrefillWorkspace w;
        w.heads = heads, w.batch = batch, w.rows_per_pass = (rows + 15) / 16 * 16;
        w.buf = DeviceBuffer::alloc((size_t)nbytes);
        return w;
    }
    // The rows per pass that keep the workspace within `nbytes` (at least one 16-row chunk).
    static PrefillWorkspace within(size_t heads, size_t batch, size_t nbytes) {
        const size_t chunk = (size_t)glm53f_kda_prefill_workspace_bytes(to_i32(heads, "heads"), to_i32(batch, "batch"), 16);
        return create(heads, batch, std::max<size_t>(nbytes / std::max<size_t>(chunk, 1), 1) * 16);
    }
    void args(size_t h, size_t b, float** ws, int64_t* ws_bytes) const {
        if (h != heads || b > batch)
            invalid("workspace for " + std::to_string(heads) + " heads x " + std::to_string(batch) + " requests used for " + std::to_string(h) + " x " + std::to_string(b));
        *ws = buf.ptr<float>();
        *ws_bytes = (int64_t)buf.bytes();
    }
};

// One layer, one request: a prompt segment through the prefill (glm53f_kda_prefill; kernel.rs:1055-1141).  The conv
// window is advanced past the rows in place; the state after the rows goes to state_out (InPlace or To).
struct Prefill {
    const Weights* weights = nullptr;
    size_t rows = 0;
    RowView p;
    long long b_off = 0;
    RowView a, g;
    const DeviceBuffer* conv = nullptr;
    size_t conv_offset = 0;
    const DeviceBuffer* state = nullptr;
    size_t state_offset = 0;
    StateOut state_out;
    RowView out;
    size_t value_blocks = 0;
    const PrefillWorkspace* workspace = nullptr;

    void launch(const Stream& stream) const {
        const size_t h = weights->heads;
        const int32_t vb = check_value_blocks(value_blocks);
        check_lower(weights->lower);
        detail::check_rows(h, rows, p, b_off, a, g, out);
        check_region("conv", *conv, 2, conv_offset, WINDOW * channels(h));
        check_region("state", *state, 4, state_offset, state_len(h));
        float* so = nullptr;
        if (state_out.kind == StateOut::Skip) invalid("a prefill always writes its state");
        if (state_out.kind == StateOut::InPlace) so = state->ptr<float>(state_offset);
        else {
            check_region("state_out", *state_out.buf, 4, state_out.offset, state_len(h));
            if (same(*state_out.buf, *state) && !coincide_or_disjoint(state_out.offset, state_offset, state_len(h))) invalid("state_out partly overlaps the state");
            so = state_out.buf->ptr<float>(state_out.offset);
        }
        float* ws;
        int64_t ws_bytes;
        workspace->args(h, 1, &ws, &ws_bytes);
        const Weights& w = *weights;
        launched(glm53f_kda_prefill(to_i32(h, "heads"), to_i32(rows, "rows"), p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(), (int64_t)g.stride,
                                    conv->ptr<glm53f_bf16>(conv_offset), w.conv_w.ptr<glm53f_bf16>(), state->ptr<float>(state_offset), so, w.a_log.ptr<float>(),
                                    w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(), w.eps, w.lower, out.buf->ptr<glm53f_bf16>(out.offset), (int64_t)out.stride, vb, ws,
                                    ws_bytes, stream.raw()),
                 "glm53f_kda_prefill");
    }
};

// One layer, a batch of prompt segments (glm53f_kda_prefill_batch; kernel.rs:1146-1285).
struct PrefillBatch {
    const Weights* weights = nullptr;
    RowView p;
    long long b_off = 0;
    RowView a, g;
    const DeviceBuffer* conv = nullptr;
    const DeviceBuffer* state = nullptr;
    StateOut state_out;  // InPlace, or To(buf, _): each request's state at its state_offset in buf
    RowView out;
    size_t value_blocks = 0;
    const PrefillWorkspace* workspace = nullptr;

    void launch(const BatchMeta& meta, const Stream& stream) const { launch_as(meta, stream, StateType::F32); }
    void launch_bf16_state(const BatchMeta& meta, const Stream& stream) const { launch_as(meta, stream, StateType::Bf16); }

   private:
    void launch_as(const BatchMeta& meta, const Stream& stream, StateType st) const {
        const size_t es = bytes(st), h = weights->heads;
        const int32_t vb = check_value_blocks(value_blocks);
        check_lower(weights->lower);
        const int32_t batch = meta.batch();
        const size_t total = meta.total_rows();
        detail::check_rows(h, total, p, b_off, a, g, out);
        // The windows are written: they must not overlap.
        meta.check_regions("conv", *conv, 2, 0, WINDOW * channels(h), true, [](const Request& r) { return r.conv_offset; });
        meta.check_regions("state", *state, es, 0, state_len(h), true, [](const Request& r) { return r.state_offset; });
        void* so = detail::batch_state_out(meta, state_out, *state, es, h, false);
        float* ws;
        int64_t ws_bytes;
        workspace->args(h, (size_t)batch, &ws, &ws_bytes);
        size_t max_rows = 0;
        for (const Request& r : meta.requests()) max_rows = std::max(max_rows, r.rows);
        const Weights& w = *weights;
        const int32_t heads = to_i32(h, "heads"), mr = to_i32(max_rows, "max_rows");
        int code;
        if (st == StateType::F32)
            code = glm53f_kda_prefill_batch(heads, batch, meta.cu_rows.ptr<int32_t>(), mr, p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(),
                                            (int64_t)g.stride, conv->ptr<glm53f_bf16>(), meta.conv_off.ptr<int64_t>(), w.conv_w.ptr<glm53f_bf16>(), state->ptr<float>(),
                                            static_cast<float*>(so), meta.state_off.ptr<int64_t>(), w.a_log.ptr<float>(), w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(),
                                            w.eps, w.lower, out.buf->ptr<glm53f_bf16>(out.offset), (int64_t)out.stride, vb, ws, ws_bytes, stream.raw());
        else
            code = glm53f_kda_prefill_batch_bf16state(heads, batch, meta.cu_rows.ptr<int32_t>(), mr, p.ptr(), (int64_t)p.stride, b_off, a.ptr(), (int64_t)a.stride, g.ptr(),
                                                      (int64_t)g.stride, conv->ptr<glm53f_bf16>(), meta.conv_off.ptr<int64_t>(), w.conv_w.ptr<glm53f_bf16>(),
                                                      state->ptr<glm53f_bf16>(), static_cast<glm53f_bf16*>(so), meta.state_off.ptr<int64_t>(), w.a_log.ptr<float>(),
                                                      w.dt_bias.ptr<float>(), w.norm_w.ptr<glm53f_bf16>(), w.eps, w.lower, out.buf->ptr<glm53f_bf16>(out.offset),
                                                      (int64_t)out.stride, vb, ws, ws_bytes, stream.raw());
        launched(code, "glm53f_kda_prefill_batch");
    }
};

// ---- forms of the layer entry points (additions of this library; process-wide switches) -------------------------------
// The exact forms are the defaults and leave the reference kernels' bits; the chunked forms run on the tensor cores and
// agree to the rounding of bf16 operands (glm53f_kda_prefill_mode, glm53f_kda_verify_mode, glm53f_kda_commit_mode in
// glm53f_kda.h say what each changes).  Each setter returns the form that was in force.
enum class Form : int32_t { Exact = 0, Chunked = 1 };
inline Form set_prefill_form(Form f) { return static_cast<Form>(glm53f_kda_prefill_mode(static_cast<int32_t>(f))); }
inline Form set_verify_form(Form f) { return static_cast<Form>(glm53f_kda_verify_mode(static_cast<int32_t>(f))); }
inline Form set_commit_form(Form f) { return static_cast<Form>(glm53f_kda_commit_mode(static_cast<int32_t>(f))); }
inline Form prefill_form() { return static_cast<Form>(glm53f_kda_prefill_mode(-1)); }
inline Form verify_form() { return static_cast<Form>(glm53f_kda_verify_mode(-1)); }
inline Form commit_form() { return static_cast<Form>(glm53f_kda_commit_mode(-1)); }

}  // namespace kda
}  // namespace glm53f
