// CPU oracle for the KDA recurrent core.  TEST INFRASTRUCTURE ONLY: see kda_oracle.h.
//
// Every function names the reference lines it restates (paths inside crates/glm53f-kda).  Build with
// -ffp-contract=off: the reference's Rust never fuses a multiply and an add, and the bitwise identities the
// tests assert (replayed prefix == shorter chain, serial steps == one window) depend on that.

#include "kda_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr int DK = 128, DV = 128, TAPS = 4, WINDOW = 3;
constexpr float L2_EPS = 1e-6f;

inline float round_as(int mode, float x) { return mode == KDAO_F32 ? x : kdao_bf16_round(x); }

}  // namespace

// ---------------------------------------------------------------- src/bf16.rs:6-23, 41-50
uint16_t kdao_bf16_from_f32(float x) {
    uint32_t u;
    std::memcpy(&u, &x, 4);
    if (std::isnan(x)) return (uint16_t)((u >> 16) | 0x0040u);
    const uint32_t lsb = (u >> 16) & 1u;
    return (uint16_t)((u + 0x7fffu + lsb) >> 16);
}

float kdao_bf16_to_f32(uint16_t b) {
    const uint32_t u = (uint32_t)b << 16;
    float x;
    std::memcpy(&x, &u, 4);
    return x;
}

float kdao_bf16_round(float x) { return kdao_bf16_to_f32(kdao_bf16_from_f32(x)); }

uint32_t kdao_bf16_ulp_distance(uint16_t a, uint16_t b) {
    auto ordered = [](uint16_t x) -> int32_t { return (x & 0x8000) ? -(int32_t)(x & 0x7fff) : (int32_t)x; };
    const int32_t d = ordered(a) - ordered(b);
    return (uint32_t)(d < 0 ? -d : d);
}

// ---------------------------------------------------------------- src/synth.rs:10-45
uint64_t kdao_rng_new(uint64_t seed) { return seed ^ 0x6a09e667f3bcc909ull; }

uint64_t kdao_rng_next_u64(uint64_t* state) {
    *state += 0x9e3779b97f4a7c15ull;
    uint64_t z = *state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

void kdao_rng_fill(uint64_t* state, int64_t n, float lo, float hi, int round_bf16, float* out) {
    for (int64_t i = 0; i < n; ++i) {
        const float u = (float)(kdao_rng_next_u64(state) >> 40) / (float)(1ull << 24);
        const float x = lo + (hi - lo) * u;
        out[i] = round_bf16 ? kdao_bf16_round(x) : x;
    }
}

// ---------------------------------------------------------------- src/cpu.rs:203-254
float kdao_sigmoid(float x) { return 1.0f / (1.0f + std::exp(-x)); }
float kdao_silu(float x) { return x / (1.0f + std::exp(-x)); }

// The xor-butterfly of a warp (offsets 16, 8, 4, 2, 1); every lane ends with the same bits.
float kdao_warp_sum(const float* lanes32) {
    float x[32], prev[32];
    std::memcpy(x, lanes32, sizeof x);
    for (int o = 16; o > 0; o >>= 1) {
        std::memcpy(prev, x, sizeof x);
        for (int l = 0; l < 32; ++l) x[l] = prev[l] + prev[l ^ o];
    }
    return x[0];
}

// Lane l sums elements 4l .. 4l+3 in order from zero, then the butterfly.
float kdao_dot128(const float* a, const float* b) {
    float lanes[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int i = 0; i < 4; ++i) acc = acc + a[4 * l + i] * b[4 * l + i];
        lanes[l] = acc;
    }
    return kdao_warp_sum(lanes);
}

float kdao_log_decay(float a, float dt_bias, float a_log, float lower) {
    return lower * kdao_sigmoid(std::exp(a_log) * (a + dt_bias));
}
float kdao_decay(float a, float dt_bias, float decay_rate, float lower) {
    return std::exp(lower * kdao_sigmoid(decay_rate * (a + dt_bias)));
}
float kdao_beta(float b) { return kdao_bf16_round(kdao_sigmoid(b)); }

// ---------------------------------------------------------------- src/cpu.rs:304-376
float kdao_q_scale(void) { return 1.0f / std::sqrt((float)DK); }

void kdao_l2norm(const float* x, int has_scale, float scale, float* y) {
    const float inv = 1.0f / std::sqrt(kdao_dot128(x, x) + L2_EPS);
    for (int i = 0; i < DK; ++i) {
        float t = x[i] * inv;
        if (has_scale) t = t * scale;
        y[i] = t;
    }
}

void kdao_update(float* s, const float* k, const float* g, const float* v, float beta) {
    for (int row = 0; row < DV; ++row) {
        float* sr = s + row * DK;
        float lanes[32];
        for (int l = 0; l < 32; ++l) {
            float kv = 0.0f;
            for (int i = 0; i < 4; ++i) {
                const int c = 4 * l + i;
                sr[c] = sr[c] * g[c];
                kv = kv + sr[c] * k[c];
            }
            lanes[l] = kv;
        }
        const float delta = (v[row] - kdao_warp_sum(lanes)) * beta;
        for (int c = 0; c < DK; ++c) sr[c] = sr[c] + k[c] * delta;
    }
}

void kdao_read_out(const float* s, const float* q, float* y) {
    for (int row = 0; row < DV; ++row) y[row] = kdao_dot128(s + row * DK, q);
}

void kdao_gated_rmsnorm(const float* y, const float* norm_w, const float* gate, float eps, int mode, float* o) {
    const float rinv = 1.0f / std::sqrt(kdao_dot128(y, y) / (float)DV + eps);
    for (int t = 0; t < DV; ++t) {
        const float yn = y[t] * rinv;
        const float yw = norm_w[t] * yn;
        o[t] = round_as(mode, yw * kdao_sigmoid(gate[t]));
    }
}

// ---------------------------------------------------------------- src/cpu.rs:557-568, 618-635
void kdao_literal_l2norm(const float* x, float* y) {
    float ss = 0.0f;
    for (int i = 0; i < DK; ++i) ss = ss + x[i] * x[i];
    const float n = std::sqrt(ss + L2_EPS);
    for (int i = 0; i < DK; ++i) y[i] = x[i] / n;
}

void kdao_literal_gated_rmsnorm(const float* y, const float* norm_w, const float* gate, float eps, int mode,
                                float* o) {
    float ss = 0.0f;
    for (int i = 0; i < DV; ++i) ss = ss + y[i] * y[i];
    const float r = 1.0f / std::sqrt(ss / (float)DV + eps);
    for (int t = 0; t < DV; ++t) o[t] = round_as(mode, norm_w[t] * (y[t] * r) * kdao_sigmoid(gate[t]));
}

// ---------------------------------------------------------------- src/cpu.rs:257-302
namespace {
float conv_channel(int C, const float* conv_w, const float* conv, const float* qkv, int r, int c, int mode) {
    float acc = 0.0f;
    for (int tap = 0; tap < TAPS; ++tap) {
        const int at = r + tap;
        const float x = at < WINDOW ? conv[(size_t)at * C + c] : qkv[(size_t)(at - WINDOW) * C + c];
        acc = acc + conv_w[(size_t)c * TAPS + tap] * x;
    }
    switch (mode) {
        case KDAO_FUSED: return kdao_bf16_round(kdao_silu(acc));
        case KDAO_UNFUSED: return kdao_bf16_round(kdao_silu(kdao_bf16_round(acc)));
        default: return kdao_silu(acc);
    }
}
}  // namespace

void kdao_conv_qkv(int heads, const float* conv_w, const float* conv, const float* qkv, int r, int h, int mode,
                   float* q, float* k, float* v) {
    const int C = 3 * heads * DK, hd = heads * DK;
    for (int i = 0; i < DK; ++i) {
        q[i] = conv_channel(C, conv_w, conv, qkv, r, h * DK + i, mode);
        k[i] = conv_channel(C, conv_w, conv, qkv, r, hd + h * DK + i, mode);
        v[i] = conv_channel(C, conv_w, conv, qkv, r, 2 * hd + h * DK + i, mode);
    }
}

// ---------------------------------------------------------------- src/cpu.rs:531-547
void kdao_transpose_state(const float* s, int64_t n, float* t) {
    const int64_t per = (int64_t)DK * DV;
    for (int64_t h = 0; h < n / per; ++h)
        for (int a = 0; a < DV; ++a)
            for (int b = 0; b < DK; ++b) t[h * per + (int64_t)b * DV + a] = s[h * per + (int64_t)a * DK + b];
}

// ---------------------------------------------------------------- src/cpu.rs:573-610
void kdao_literal_step(float* s, const float* q, const float* k, const float* v, const float* g, float beta,
                       int normalize, float* y) {
    float qs[DK], kn[DK];
    if (normalize) {
        float qn[DK];
        kdao_literal_l2norm(q, qn);
        kdao_literal_l2norm(k, kn);
        const float scale = kdao_q_scale();
        for (int i = 0; i < DK; ++i) qs[i] = qn[i] * scale;
    } else {
        std::memcpy(qs, q, sizeof qs);
        std::memcpy(kn, k, sizeof kn);
    }
    for (int kk = 0; kk < DK; ++kk) {
        const float e = std::exp(g[kk]);
        for (int vv = 0; vv < DV; ++vv) s[kk * DV + vv] = s[kk * DV + vv] * e;
    }
    float delta[DV];
    for (int vv = 0; vv < DV; ++vv) {
        float kv = 0.0f;
        for (int kk = 0; kk < DK; ++kk) kv = kv + s[kk * DV + vv] * kn[kk];
        delta[vv] = (v[vv] - kv) * beta;
    }
    for (int kk = 0; kk < DK; ++kk)
        for (int vv = 0; vv < DV; ++vv) s[kk * DV + vv] = s[kk * DV + vv] + kn[kk] * delta[vv];
    for (int vv = 0; vv < DV; ++vv) {
        float o = 0.0f;
        for (int kk = 0; kk < DK; ++kk) o = o + s[kk * DV + vv] * qs[kk];
        y[vv] = o;
    }
}

// ---------------------------------------------------------------- src/cpu.rs:380-471, 639-685
void kdao_chain(int heads, const float* conv_w, const float* a_log, const float* dt_bias, const float* norm_w,
                float eps, float lower, const float* conv, const float* state, int rows, const float* qkv,
                const float* a, const float* b, const float* gate, int mode, int bf16_state, int literal,
                float* out, float* y_out, float* state_out, float* k_save, float* v_save, float* g_save,
                float* b_save) {
    const size_t per = (size_t)DV * DK;
    std::vector<float> st(state, state + (size_t)heads * per);
    if (literal) {
        std::vector<float> tmp(st.size());
        kdao_transpose_state(st.data(), (int64_t)st.size(), tmp.data());
        st.swap(tmp);
    }
    for (int h = 0; h < heads; ++h) {
        const float decay_rate = std::exp(a_log[h]);
        float* s = st.data() + h * per;
        for (int r = 0; r < rows; ++r) {
            float q[DK], k[DK], v[DV], g[DK], y[DV], o[DV], kn[DK];
            kdao_conv_qkv(heads, conv_w, conv, qkv, r, h, mode, q, k, v);
            const size_t at = ((size_t)r * heads + h) * DK;
            const float bt = round_as(mode, kdao_sigmoid(b[(size_t)r * heads + h]));
            if (!literal) {
                float qn[DK];
                for (int i = 0; i < DK; ++i) g[i] = kdao_decay(a[at + i], dt_bias[h * DK + i], decay_rate, lower);
                kdao_l2norm(q, 1, kdao_q_scale(), qn);
                kdao_l2norm(k, 0, 0.0f, kn);
                kdao_update(s, kn, g, v, bt);
                kdao_read_out(s, qn, y);
                for (int i = 0; i < DV; ++i) y[i] = round_as(mode, y[i]);
                if (bf16_state)
                    for (size_t i = 0; i < per; ++i) s[i] = kdao_bf16_round(s[i]);
                kdao_gated_rmsnorm(y, norm_w, gate + at, eps, mode, o);
            } else {
                float lg[DK];
                for (int i = 0; i < DK; ++i) lg[i] = kdao_log_decay(a[at + i], dt_bias[h * DK + i], a_log[h], lower);
                kdao_literal_step(s, q, k, v, lg, bt, 1, y);
                for (int i = 0; i < DV; ++i) y[i] = round_as(mode, y[i]);
                kdao_literal_gated_rmsnorm(y, norm_w, gate + at, eps, mode, o);
                kdao_literal_l2norm(k, kn);
                for (int i = 0; i < DK; ++i) g[i] = std::exp(lg[i]);
            }
            if (out) std::memcpy(out + at, o, sizeof o);
            if (y_out) std::memcpy(y_out + at, y, sizeof y);
            if (k_save) std::memcpy(k_save + at, kn, sizeof kn);
            if (v_save) std::memcpy(v_save + at, v, sizeof v);
            if (g_save) std::memcpy(g_save + at, g, sizeof g);
            if (b_save) b_save[(size_t)r * heads + h] = bt;
        }
    }
    if (state_out) {
        if (literal) kdao_transpose_state(st.data(), (int64_t)st.size(), state_out);
        else std::memcpy(state_out, st.data(), st.size() * sizeof(float));
    }
}

// ---------------------------------------------------------------- src/cpu.rs:475-508
void kdao_replay(int heads, const float* state, int rows_saved, const float* k_save, const float* v_save,
                 const float* g_save, const float* b_save, int keep, int bf16_state, float* state_out) {
    (void)rows_saved;
    const size_t per = (size_t)DV * DK;
    if (state_out != state) std::memcpy(state_out, state, (size_t)heads * per * sizeof(float));
    for (int h = 0; h < heads; ++h) {
        float* s = state_out + h * per;
        for (int r = 0; r < keep; ++r) {
            const size_t at = ((size_t)r * heads + h) * DK;
            kdao_update(s, k_save + at, g_save + at, v_save + at, b_save[(size_t)r * heads + h]);
            if (bf16_state)
                for (size_t i = 0; i < per; ++i) s[i] = kdao_bf16_round(s[i]);
        }
    }
}

// ---------------------------------------------------------------- src/cpu.rs:512-527
void kdao_conv_shift(int heads, const float* conv, int rows, const float* qkv, int keep, float* out) {
    (void)rows;
    const size_t C = (size_t)3 * heads * DK;
    std::vector<float> w(WINDOW * C);
    for (int j = 0; j < WINDOW; ++j) {
        const int src = keep + j;
        const float* from = src < WINDOW ? conv + src * C : qkv + (size_t)(src - WINDOW) * C;
        std::memcpy(w.data() + j * C, from, C * sizeof(float));
    }
    std::memcpy(out, w.data(), w.size() * sizeof(float));
}

// ---------------------------------------------------------------- src/chunked.rs:67-198
void kdao_chunked_head(int t, const float* q, const float* k, const float* v, const float* g, const float* beta,
                       float* state, int chunk, float* out) {
    const int c = chunk;
    std::vector<float> gc((size_t)c * DK), a((size_t)c * c), u((size_t)c * DV), w((size_t)c * DK),
        vnew((size_t)c * DV), m(c), rowi(c);
    for (int start = 0; start < t; start += c) {
        const int n = std::min(c, t - start);
        auto kq = [&](const float* x, int i, int d) { return x[(size_t)(start + i) * DK + d]; };
        // Cumulative log decay inside the chunk.
        for (int i = 0; i < n; ++i)
            for (int d = 0; d < DK; ++d)
                gc[i * DK + d] = (i == 0 ? 0.0f : gc[(i - 1) * DK + d]) + g[(size_t)(start + i) * DK + d];
        // A (strictly lower) and the forward substitution.
        std::fill(a.begin(), a.end(), 0.0f);
        for (int i = 0; i < n; ++i) {
            const float bi = beta[start + i];
            for (int j = 0; j < i; ++j) {
                float acc = 0.0f;
                for (int d = 0; d < DK; ++d) {
                    const float kb = kq(k, i, d) * bi;
                    acc = acc + kb * kq(k, j, d) * std::exp(gc[i * DK + d] - gc[j * DK + d]);
                }
                a[i * n + j] = -acc;
            }
        }
        for (int i = 1; i < n; ++i) {
            for (int col = 0; col < i; ++col) rowi[col] = a[i * n + col];
            for (int col = 0; col < i; ++col) {
                float acc = 0.0f;
                for (int mm = 0; mm < i; ++mm) acc = acc + rowi[mm] * a[mm * n + col];
                a[i * n + col] = rowi[col] + acc;
            }
        }
        for (int i = 0; i < n; ++i) a[i * n + i] = a[i * n + i] + 1.0f;
        // U = T (beta V), W = T (beta K exp(G)).
        for (int i = 0; i < n; ++i) {
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int j = 0; j < n; ++j) acc = acc + a[i * n + j] * (v[(size_t)(start + j) * DV + vv] * beta[start + j]);
                u[i * DV + vv] = acc;
            }
            for (int d = 0; d < DK; ++d) {
                float acc = 0.0f;
                for (int j = 0; j < n; ++j)
                    acc = acc + a[i * n + j] * (kq(k, j, d) * beta[start + j] * std::exp(gc[j * DK + d]));
                w[i * DK + d] = acc;
            }
        }
        // The chunk against the incoming state.
        for (int i = 0; i < n; ++i)
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int d = 0; d < DK; ++d) acc = acc + w[i * DK + d] * state[d * DV + vv];
                vnew[i * DV + vv] = u[i * DV + vv] - acc;
            }
        for (int i = 0; i < n; ++i) {
            for (int j = 0; j <= i; ++j) {
                float acc = 0.0f;
                for (int d = 0; d < DK; ++d)
                    acc = acc + kq(q, i, d) * kq(k, j, d) * std::exp(gc[i * DK + d] - gc[j * DK + d]);
                m[j] = acc;
            }
            for (int vv = 0; vv < DV; ++vv) {
                float inter = 0.0f;
                for (int d = 0; d < DK; ++d) inter = inter + kq(q, i, d) * std::exp(gc[i * DK + d]) * state[d * DV + vv];
                float intra = 0.0f;
                for (int j = 0; j <= i; ++j) intra = intra + m[j] * vnew[j * DV + vv];
                out[(size_t)(start + i) * DV + vv] = inter + intra;
            }
        }
        const int last = n - 1;
        for (int d = 0; d < DK; ++d) {
            const float decay_all = std::exp(gc[last * DK + d]);
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int i = 0; i < n; ++i)
                    acc = acc + kq(k, i, d) * std::exp(gc[last * DK + d] - gc[i * DK + d]) * vnew[i * DV + vv];
                state[d * DV + vv] = state[d * DV + vv] * decay_all + acc;
            }
        }
    }
}

// ---------------------------------------------------------------- src/chunked.rs:205-254
void kdao_chunked_layer(int heads, int t, const float* q, const float* k, const float* v, const float* g,
                        const float* beta, float* state, int chunk, float* out) {
    std::vector<float> qh((size_t)t * DK), kh((size_t)t * DK), vh((size_t)t * DV), gh((size_t)t * DK), bh(t),
        o((size_t)t * DV);
    const float scale = kdao_q_scale();
    for (int h = 0; h < heads; ++h) {
        for (int r = 0; r < t; ++r) {
            const size_t at = ((size_t)r * heads + h) * DK;
            float n[DK];
            kdao_literal_l2norm(q + at, n);
            for (int i = 0; i < DK; ++i) qh[(size_t)r * DK + i] = n[i] * scale;
            kdao_literal_l2norm(k + at, kh.data() + (size_t)r * DK);
            std::memcpy(vh.data() + (size_t)r * DV, v + at, DV * sizeof(float));
            std::memcpy(gh.data() + (size_t)r * DK, g + at, DK * sizeof(float));
            bh[r] = beta[(size_t)r * heads + h];
        }
        kdao_chunked_head(t, qh.data(), kh.data(), vh.data(), gh.data(), bh.data(), state + (size_t)h * DK * DV, chunk,
                          o.data());
        for (int r = 0; r < t; ++r)
            std::memcpy(out + ((size_t)r * heads + h) * DV, o.data() + (size_t)r * DV, DV * sizeof(float));
    }
}

// ---------------------------------------------------------------- src/chunked.rs:263-400
void kdao_prefill_head(int t, const float* qn, const float* kn, const float* v, const float* d, const float* beta,
                       float* s, float* y) {
    constexpr int CH = 16;
    float lf[CH * DK], hi[DK], lo[DK], d0[DK], last[DK], elast[DK];
    float a[CH * DK], aq[CH * DK], b[CH * DK], l[CH * CH], m[CH * CH], tm[CH * CH];
    float w[CH * DK], u[CH * DV], delta[CH * DV];
    for (int start = 0; start < t; start += CH) {
        const int n = std::min(CH, t - start);
        auto row = [&](int i) { return (size_t)(start + i) * DK; };
        // Decay products from the chunk's first row, carried as an exact two-product (hi, lo) and rounded once.
        for (int k = 0; k < DK; ++k) { hi[k] = 1.0f; lo[k] = 0.0f; lf[k] = 1.0f; }
        for (int i = 1; i < n; ++i)
            for (int k = 0; k < DK; ++k) {
                const float dk = d[row(i) + k];
                const float p = hi[k] * dk;
                lo[k] = std::fma(lo[k], dk, std::fma(hi[k], dk, -p));
                hi[k] = p;
                lf[i * DK + k] = hi[k] + lo[k];
            }
        for (int k = 0; k < DK; ++k) {
            d0[k] = d[row(0) + k];
            last[k] = lf[(n - 1) * DK + k];
            elast[k] = std::fma(d0[k], hi[k], d0[k] * lo[k]);
        }
        for (int i = 0; i < n; ++i)
            for (int k = 0; k < DK; ++k) {
                const float f = lf[i * DK + k];
                a[i * DK + k] = kn[row(i) + k] * f;
                aq[i * DK + k] = qn[row(i) + k] * f;
                b[i * DK + k] = kn[row(i) + k] / f;
            }
        std::fill(l, l + CH * CH, 0.0f);
        std::fill(m, m + CH * CH, 0.0f);
        for (int i = 0; i < n; ++i)
            for (int j = 0; j <= i; ++j) {
                float sl = 0.0f, sm = 0.0f;
                for (int k = 0; k < DK; ++k) {
                    sl = sl + a[i * DK + k] * b[j * DK + k];
                    sm = sm + aq[i * DK + k] * b[j * DK + k];
                }
                m[i * n + j] = sm;
                if (j < i) l[i * n + j] = beta[start + i] * sl;
            }
        // T = (I + L)^-1 by forward substitution, then T' = T diag(beta).
        std::fill(tm, tm + CH * CH, 0.0f);
        for (int i = 0; i < n; ++i) {
            tm[i * n + i] = 1.0f;
            for (int j = 0; j < i; ++j) {
                float acc = l[i * n + j];
                for (int mm = j + 1; mm < i; ++mm) acc = acc + l[i * n + mm] * tm[mm * n + j];
                tm[i * n + j] = -acc;
            }
        }
        for (int i = 0; i < n; ++i)
            for (int j = 0; j <= i; ++j) tm[i * n + j] = tm[i * n + j] * beta[start + j];
        for (int i = 0; i < n; ++i) {
            for (int k = 0; k < DK; ++k) {
                float acc = 0.0f;
                for (int j = 0; j <= i; ++j) acc = acc + tm[i * n + j] * a[j * DK + k];
                w[i * DK + k] = d0[k] * acc;
            }
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int j = 0; j <= i; ++j) acc = acc + tm[i * n + j] * v[(size_t)(start + j) * DV + vv];
                u[i * DV + vv] = acc;
            }
        }
        for (int i = 0; i < n; ++i)
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int k = 0; k < DK; ++k) acc = acc + w[i * DK + k] * s[vv * DK + k];
                delta[i * DV + vv] = u[i * DV + vv] - acc;
            }
        for (int i = 0; i < n; ++i)
            for (int vv = 0; vv < DV; ++vv) {
                float acc = 0.0f;
                for (int k = 0; k < DK; ++k) acc = acc + (aq[i * DK + k] * d0[k]) * s[vv * DK + k];
                for (int j = 0; j <= i; ++j) acc = acc + m[i * n + j] * delta[j * DV + vv];
                y[(size_t)(start + i) * DV + vv] = acc;
            }
        for (int vv = 0; vv < DV; ++vv)
            for (int k = 0; k < DK; ++k) {
                float acc = s[vv * DK + k] * elast[k];
                for (int i = 0; i < n; ++i) acc = acc + (b[i * DK + k] * last[k]) * delta[i * DV + vv];
                s[vv * DK + k] = acc;
            }
    }
}

// ---------------------------------------------------------------- src/chunked.rs:405-467
void kdao_prefill(int heads, const float* conv_w, const float* a_log, const float* dt_bias, const float* norm_w,
                  float eps, float lower, const float* conv, const float* state, int rows, const float* qkv,
                  const float* a, const float* b, const float* gate, int mode, float* out, float* y_out,
                  float* state_out) {
    const size_t per = (size_t)DV * DK;
    std::vector<float> st(state, state + (size_t)heads * per);
    std::vector<float> qn((size_t)rows * DK), kn((size_t)rows * DK), v((size_t)rows * DV), d((size_t)rows * DK),
        beta(rows), y((size_t)rows * DV);
    for (int h = 0; h < heads; ++h) {
        const float decay_rate = std::exp(a_log[h]);
        for (int r = 0; r < rows; ++r) {
            float q[DK], k[DK];
            kdao_conv_qkv(heads, conv_w, conv, qkv, r, h, mode, q, k, v.data() + (size_t)r * DV);
            kdao_l2norm(q, 1, kdao_q_scale(), qn.data() + (size_t)r * DK);
            kdao_l2norm(k, 0, 0.0f, kn.data() + (size_t)r * DK);
            const size_t at = ((size_t)r * heads + h) * DK;
            for (int i = 0; i < DK; ++i)
                d[(size_t)r * DK + i] = kdao_decay(a[at + i], dt_bias[h * DK + i], decay_rate, lower);
            beta[r] = round_as(mode, kdao_sigmoid(b[(size_t)r * heads + h]));
        }
        kdao_prefill_head(rows, qn.data(), kn.data(), v.data(), d.data(), beta.data(), st.data() + h * per, y.data());
        for (int r = 0; r < rows; ++r) {
            float yr[DV], o[DV];
            for (int i = 0; i < DV; ++i) yr[i] = round_as(mode, y[(size_t)r * DV + i]);
            const size_t at = ((size_t)r * heads + h) * DV;
            kdao_gated_rmsnorm(yr, norm_w, gate + at, eps, mode, o);
            if (out) std::memcpy(out + at, o, sizeof o);
            if (y_out) std::memcpy(y_out + at, yr, sizeof yr);
        }
    }
    if (state_out) std::memcpy(state_out, st.data(), st.size() * sizeof(float));
}

// ---------------------------------------------------------------- the benchmark configurations' "core" contract
void kdao_core_forward(int heads, int h0, int h1, int64_t t, const uint16_t* q_bits, const uint16_t* k_bits,
                       const uint16_t* v_bits, const float* g, const float* beta, float* state, int form,
                       int chunk, int bf16_state, int threads, float* y) {
    const size_t per = (size_t)DK * DV;
    auto run_head = [&](int h) {
        // Gather this head's rows and move its state to the literal [k][v] layout.
        std::vector<float> q((size_t)t * DK), k((size_t)t * DK), v((size_t)t * DV), gg((size_t)t * DK), b(t),
            o(y ? (size_t)t * DV : DV), s(per), tmp(per);
        for (int64_t r = 0; r < t; ++r) {
            const size_t at = ((size_t)r * heads + h) * DK;
            for (int i = 0; i < DK; ++i) {
                q[(size_t)r * DK + i] = kdao_bf16_to_f32(q_bits[at + i]);
                k[(size_t)r * DK + i] = kdao_bf16_to_f32(k_bits[at + i]);
                v[(size_t)r * DV + i] = kdao_bf16_to_f32(v_bits[at + i]);
            }
            std::memcpy(gg.data() + (size_t)r * DK, g + at, DK * sizeof(float));
            b[r] = beta[(size_t)r * heads + h];
        }
        kdao_transpose_state(state + (size_t)h * per, (int64_t)per, s.data());
        if (form == 1) {
            if (y) {
                kdao_chunked_head((int)t, q.data(), k.data(), v.data(), gg.data(), b.data(), s.data(), chunk, o.data());
            } else {
                std::vector<float> full((size_t)t * DV);
                kdao_chunked_head((int)t, q.data(), k.data(), v.data(), gg.data(), b.data(), s.data(), chunk, full.data());
            }
        } else {
            for (int64_t r = 0; r < t; ++r) {
                float* yr = y ? o.data() + (size_t)r * DV : o.data();
                kdao_literal_step(s.data(), q.data() + (size_t)r * DK, k.data() + (size_t)r * DK, v.data() + (size_t)r * DV,
                                  gg.data() + (size_t)r * DK, b[r], 0, yr);
                if (bf16_state)
                    for (size_t i = 0; i < per; ++i) s[i] = kdao_bf16_round(s[i]);
            }
        }
        kdao_transpose_state(s.data(), (int64_t)per, tmp.data());
        std::memcpy(state + (size_t)h * per, tmp.data(), per * sizeof(float));
        if (y)
            for (int64_t r = 0; r < t; ++r)
                std::memcpy(y + ((size_t)r * heads + h) * DV, o.data() + (size_t)r * DV, DV * sizeof(float));
    };
    const int nthreads = std::max(1, std::min(threads, h1 - h0));
    if (nthreads == 1) {
        for (int h = h0; h < h1; ++h) run_head(h);
        return;
    }
    std::vector<std::thread> pool;
    for (int w = 0; w < nthreads; ++w)
        pool.emplace_back([&, w]() {
            for (int h = h0 + w; h < h1; h += nthreads) run_head(h);
        });
    for (auto& th : pool) th.join();
}

// ---------------------------------------------------------------- src/cpu.rs:436-453 on post-conv inputs
void kdao_core_step_batch(int heads, int batch, const int32_t* cu_rows, const uint16_t* q_bits, const uint16_t* k_bits,
                          const uint16_t* v_bits, const float* g, const float* beta, float* states,
                          const int64_t* state_off, int bf16_state, int l2norm, int threads, float* y, float* k_save,
                          float* v_save, float* g_save, float* b_save) {
    const size_t per = (size_t)DV * DK;
    const int units = heads * batch;
    auto run_unit = [&](int u) {
        const int b = u / heads, h = u % heads;
        float* s = states + state_off[b] + (size_t)h * per;
        for (int r = cu_rows[b]; r < cu_rows[b + 1]; ++r) {
            const size_t at = ((size_t)r * heads + h) * DK;
            float q[DK], k[DK], v[DV], gm[DK], yr[DV];
            for (int i = 0; i < DK; ++i) {
                q[i] = kdao_bf16_to_f32(q_bits[at + i]);
                k[i] = kdao_bf16_to_f32(k_bits[at + i]);
                v[i] = kdao_bf16_to_f32(v_bits[at + i]);
                gm[i] = std::exp(g[at + i]);
            }
            if (l2norm) {
                float qn[DK], kn[DK];
                kdao_l2norm(q, 1, kdao_q_scale(), qn);
                kdao_l2norm(k, 0, 0.0f, kn);
                std::memcpy(q, qn, sizeof q);
                std::memcpy(k, kn, sizeof k);
            }
            const float bt = beta[(size_t)r * heads + h];
            kdao_update(s, k, gm, v, bt);
            kdao_read_out(s, q, yr);
            if (y)
                for (int i = 0; i < DV; ++i) y[at + i] = kdao_bf16_round(yr[i]);
            if (bf16_state)
                for (size_t i = 0; i < per; ++i) s[i] = kdao_bf16_round(s[i]);
            if (k_save) std::memcpy(k_save + at, k, sizeof k);
            if (v_save) std::memcpy(v_save + at, v, sizeof v);
            if (g_save) std::memcpy(g_save + at, gm, sizeof gm);
            if (b_save) b_save[(size_t)r * heads + h] = bt;
        }
    };
    const int nthreads = std::max(1, std::min(threads, units));
    if (nthreads == 1) {
        for (int u = 0; u < units; ++u) run_unit(u);
        return;
    }
    std::vector<std::thread> pool;
    for (int w = 0; w < nthreads; ++w)
        pool.emplace_back([&, w]() {
            for (int u = w; u < units; u += nthreads) run_unit(u);
        });
    for (auto& th : pool) th.join();
}
