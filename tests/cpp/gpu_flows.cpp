// The reference's flows through the C++ wrappers on a GPU (crates/glm53f-kda/tests/gpu.rs): a chain with saves; the
// replay of all its rows reproduces the chain's state bit for bit and a replayed prefix equals the shorter chain; a
// batch of one equals the single-request entry point; a prefill agrees with the chain; rejections throw before launch.
#include <cmath>
#include <cstdio>

#include "glm53f_kda.hpp"

using namespace glm53f::kda;

static uint64_t rng_state = 0x9e3779b97f4a7c15ull;
static float uniform(float lo, float hi) {  // SplitMix64, 24-bit uniform (the reference's synth.rs)
    uint64_t z = (rng_state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    return lo + (hi - lo) * (float)((z >> 40) * (1.0 / 16777216.0));
}
static std::vector<float> fill(size_t n, float lo, float hi, bool bf16) {
    std::vector<float> v(n);
    for (float& x : v) x = bf16 ? bf16_to_f32(bf16_from_f32(uniform(lo, hi))) : uniform(lo, hi);
    return v;
}
static int failures = 0;
#define CHECK(cond) do { if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } } while (0)
static void sync() { if (cudaDeviceSynchronize() != cudaSuccess) { std::printf("FAIL device\n"); ++failures; } }

int main() {
    const size_t h = 2, rows = 5, c = channels(h);
    LayerParams lp;
    lp.heads = h;
    lp.conv_w = fill(c * TAPS, -0.6f, 0.6f, true), lp.a_log = fill(h, -1.5f, 1.5f, false), lp.dt_bias = fill(h * DK, -1.f, 1.f, false), lp.norm_w = fill(DV, 0.25f, 1.75f, true);
    Weights w = Weights::upload(lp);
    std::vector<float> qkvb = fill(rows * (c + h), -2.f, 2.f, true), a = fill(rows * h * DK, -4.f, 4.f, true), gate = fill(rows * h * DV, -4.f, 4.f, true);
    std::vector<float> window = fill(WINDOW * c, -2.f, 2.f, true), s0 = fill(state_len(h), -0.5f, 0.5f, false);
    DeviceBuffer pb = DeviceBuffer::from_slice(bf16_encode(qkvb)), ab = DeviceBuffer::from_slice(bf16_encode(a)), gb = DeviceBuffer::from_slice(bf16_encode(gate));
    DeviceBuffer conv = DeviceBuffer::from_slice(bf16_encode(window)), state = DeviceBuffer::from_slice(s0);
    DeviceBuffer next = DeviceBuffer::zeroed(state_len(h) * 4), ob = DeviceBuffer::zeroed(rows * h * DV * 2);
    Saves saves = Saves::alloc(h, rows);
    Stream s;
    Chain ch;
    ch.weights = &w, ch.rows = rows, ch.p = RowView::dense(pb, c + h), ch.b_off = (long long)c, ch.a = RowView::dense(ab, h * DK), ch.g = RowView::dense(gb, h * DV);
    ch.conv = &conv, ch.state = &state, ch.state_out = StateOut::to(next), ch.out = RowView::dense(ob, h * DV), ch.saves = &saves;
    ch.launch(s);
    sync();
    CHECK(glm53f_kda_device_status() == 0);
    const std::vector<float> after = next.download<float>(state_len(h));
    const std::vector<uint16_t> out = ob.download<uint16_t>(rows * h * DV);
    CHECK(state.download<float>(state_len(h)) == s0);  // the input state is untouched
    bool finite = true, moved = false;
    for (size_t i = 0; i < after.size(); ++i) finite &= std::isfinite(after[i]), moved |= after[i] != s0[i];
    CHECK(finite && moved);

    // replay of every row == the chain's state; a prefix == the shorter chain
    DeviceBuffer replayed = DeviceBuffer::zeroed(state_len(h) * 4);
    replay(h, rows, state, 0, replayed, 0, saves, s);
    sync();
    CHECK(replayed.download<float>(state_len(h)) == after);
    DeviceBuffer prefix = DeviceBuffer::zeroed(state_len(h) * 4), shorter = DeviceBuffer::zeroed(state_len(h) * 4), o3 = DeviceBuffer::zeroed(3 * h * DV * 2);
    replay(h, 3, state, 0, prefix, 0, saves, s);
    Chain c3 = ch;
    c3.rows = 3, c3.state_out = StateOut::to(shorter), c3.out = RowView::dense(o3, h * DV), c3.saves = nullptr;
    c3.launch(s);
    sync();
    CHECK(prefix.download<float>(state_len(h)) == shorter.download<float>(state_len(h)));
    std::vector<uint16_t> out3 = o3.download<uint16_t>(3 * h * DV);
    CHECK(std::equal(out3.begin(), out3.end(), out.begin()));

    // a batch of one request == the single-request entry point
    BatchMeta meta(1);
    meta.set({Request{rows, 0, 0}});
    DeviceBuffer bstate = DeviceBuffer::zeroed(state_len(h) * 4), bout = DeviceBuffer::zeroed(rows * h * DV * 2);
    ChainBatch cb;
    cb.weights = &w, cb.p = ch.p, cb.b_off = ch.b_off, cb.a = ch.a, cb.g = ch.g, cb.conv = &conv, cb.state = &state, cb.state_out = StateOut::to(bstate);
    cb.out = RowView::dense(bout, h * DV);
    cb.launch(meta, s);
    sync();
    CHECK(bstate.download<float>(state_len(h)) == after && bout.download<uint16_t>(rows * h * DV) == out);

    // the prefill agrees with the chain (state to f32 rounding, outputs within a bf16 ulp), and advances the window
    DeviceBuffer pconv = DeviceBuffer::from_slice(bf16_encode(window)), pstate = DeviceBuffer::zeroed(state_len(h) * 4), pout = DeviceBuffer::zeroed(rows * h * DV * 2);
    PrefillWorkspace ws = PrefillWorkspace::create(h, 1, 64);
    Prefill pf;
    pf.weights = &w, pf.rows = rows, pf.p = ch.p, pf.b_off = ch.b_off, pf.a = ch.a, pf.g = ch.g, pf.conv = &pconv, pf.state = &state, pf.state_out = StateOut::to(pstate);
    pf.out = RowView::dense(pout, h * DV), pf.workspace = &ws;
    pf.launch(s);
    conv_shift(h, rows, conv, 0, ch.p, s);
    sync();
    const std::vector<float> ps = pstate.download<float>(state_len(h));
    float worst = 0.f, ref = 0.f;
    for (size_t i = 0; i < ps.size(); ++i) worst = std::max(worst, std::fabs(ps[i] - after[i])), ref = std::max(ref, std::fabs(after[i]));
    CHECK(worst <= 1e-5f * ref);
    CHECK(pconv.download<uint16_t>(WINDOW * c) == conv.download<uint16_t>(WINDOW * c));
    CHECK(glm53f_kda_device_status() == 0);

    try {
        Chain bad = ch;
        bad.rows = rows + 1;
        bad.launch(s);
        CHECK(!"no error");
    } catch (const Error& e) {
        CHECK(e.kind == Error::Invalid);
    }
    std::printf(failures ? "%d FAILED\n" : "all GPU flows passed\n", failures);
    return failures ? 1 : 0;
}
