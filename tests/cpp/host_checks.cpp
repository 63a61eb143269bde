// Host-side checks of the C++ wrappers (include/glm53f_kda.hpp) without a GPU: every rejection below is one the
// reference's kernel.rs makes on the host before the launcher is called.  Built with GLM53F_KDA_HOST_ONLY, so buffers
// live in host memory; only rejections and bookkeeping are exercised (nothing is launched).
#define GLM53F_KDA_HOST_ONLY
#include <cstdio>
#include <functional>

#include "glm53f_kda.hpp"

using namespace glm53f::kda;

static int failures = 0;
static void expect_invalid(const char* what, const char* needle, const std::function<void()>& f) {
    try {
        f();
        std::printf("FAIL %s: no error\n", what);
        ++failures;
    } catch (const Error& e) {
        if (e.kind != Error::Invalid || std::string(e.what()).find(needle) == std::string::npos) {
            std::printf("FAIL %s: %s\n", what, e.what());
            ++failures;
        }
    }
}
#define CHECK(cond) do { if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++failures; } } while (0)

static Weights weights(size_t h, float lower = -5.0f) {
    LayerParams p;
    p.heads = h;
    p.conv_w.assign(channels(h) * TAPS, 0.0f), p.a_log.assign(h, 0.0f), p.dt_bias.assign(h * DK, 0.0f), p.norm_w.assign(DV, 1.0f);
    p.lower = lower;
    return Weights::upload(p);
}

int main() {
    const size_t h = 2, c = channels(h);
    Stream s;
    expect_invalid("weights", "wrong sizes", [&] { LayerParams p; p.heads = 2; p.conv_w.assign(5, 0.f); Weights::upload(p); });
    Weights w = weights(h);
    CHECK(w.norm_w.download<uint16_t>(DV)[0] == 0x3F80 && bf16_from_f32(1.00390625f) == 0x3F80 && bf16_to_f32(0x4000) == 2.0f);

    DeviceBuffer pb = DeviceBuffer::zeroed(2 * (c + h) * 2), ab = DeviceBuffer::zeroed(2 * h * DK * 2), gb = DeviceBuffer::zeroed(2 * h * DV * 2);
    DeviceBuffer conv = DeviceBuffer::zeroed(2 * WINDOW * c * 2), state = DeviceBuffer::zeroed(2 * state_len(h) * 4), ob = DeviceBuffer::zeroed(2 * h * DV * 2);
    auto chain = [&](size_t rows) {
        Chain ch;
        ch.weights = &w, ch.rows = rows, ch.p = RowView::dense(pb, c + h), ch.b_off = (long long)c, ch.a = RowView::dense(ab, h * DK), ch.g = RowView::dense(gb, h * DV);
        ch.conv = &conv, ch.state = &state, ch.state_out = StateOut::in_place(), ch.out = RowView::dense(ob, h * DV);
        return ch;
    };
    expect_invalid("chain rows", "at least one row", [&] { chain(0).launch(s); });
    expect_invalid("chain p", "p: rows reach", [&] { chain(3).launch(s); });
    expect_invalid("chain out", "out rows overlap", [&] { Chain ch = chain(2); ch.out.stride = h * DV - 1; ch.launch(s); });
    expect_invalid("chain state", "state", [&] { Chain ch = chain(1); ch.state_offset = state_len(h) + 1; ch.launch(s); });
    expect_invalid("chain conv", "conv", [&] { Chain ch = chain(1); ch.conv_offset = WINDOW * c + 8; ch.launch(s); });
    expect_invalid("chain overlap", "partly overlaps", [&] { Chain ch = chain(1); ch.state_out = StateOut::to(state, 16); ch.launch(s); });
    Saves one = Saves::alloc(h, 1);
    expect_invalid("chain saves", "saves hold", [&] { Chain ch = chain(2); ch.saves = &one; ch.launch(s); });
    expect_invalid("replay saves", "saves hold", [&] { replay(h, 2, state, 0, state, 0, one, s); });
    expect_invalid("conv_shift p", "p: rows reach", [&] { DeviceBuffer small = DeviceBuffer::zeroed(c * 2); conv_shift(h, 2, conv, 0, RowView::dense(small, c), s); });

    BatchMeta meta(3);
    expect_invalid("meta unset", "not set", [&] { meta.batch(); });
    expect_invalid("meta empty", "capacity", [&] { meta.set({}); });
    expect_invalid("meta many", "capacity", [&] { meta.set(std::vector<Request>(4, Request{1, 0, 0})); });
    expect_invalid("meta keeps", "one keep per request", [&] { std::vector<size_t> k{1, 1}; meta.set({Request{1, 0, 0}}, &k); });
    expect_invalid("meta keep", "exceeds the request", [&] { std::vector<size_t> k{3}; meta.set({Request{2, 0, 0}}, &k); });
    std::vector<size_t> keep{1, 0};
    meta.set({Request{1, 0, 0}, Request{1, WINDOW * c, state_len(h)}}, &keep);
    CHECK(meta.batch() == 2 && meta.total_rows() == 2);
    CHECK((meta.cu_rows.download<int32_t>(3) == std::vector<int32_t>{0, 1, 2}) && (meta.keep_d.download<int32_t>(2) == std::vector<int32_t>{1, 0}));
    CHECK((meta.state_off.download<int64_t>(2) == std::vector<int64_t>{0, (int64_t)state_len(h)}));
    auto batch = [&] {
        ChainBatch cb;
        cb.weights = &w, cb.p = RowView::dense(pb, c + h), cb.b_off = (long long)c, cb.a = RowView::dense(ab, h * DK), cb.g = RowView::dense(gb, h * DV);
        cb.conv = &conv, cb.state = &state, cb.state_out = StateOut::in_place(), cb.out = RowView::dense(ob, h * DV);
        return cb;
    };
    DeviceBuffer small_state = DeviceBuffer::zeroed(state_len(h) * 4);
    expect_invalid("batch state", "state", [&] { ChainBatch cb = batch(); cb.state = &small_state; cb.launch(meta, s); });
    expect_invalid("batch same", "use InPlace", [&] { ChainBatch cb = batch(); cb.state_out = StateOut::to(state); cb.launch(meta, s); });
    expect_invalid("batch saves", "saves hold", [&] { ChainBatch cb = batch(); cb.saves = &one; cb.launch_bf16_state(meta, s); });
    LayerSaves ls = LayerSaves::alloc(2, h, 2);
    CHECK(ls.kv_stride() == 2 * h * DK && ls.b_stride() == 2 * h);
    expect_invalid("fill_layer", "shape mismatch", [&] { ls.fill_layer(2, one, 1); });
    expect_invalid("replay_layers rows", "replay_layers", [&] { replay_layers(3, state, state, state_len(h), ls, s); });
    expect_invalid("replay_layers stride", "replay_layers", [&] { replay_layers(1, state, state, state_len(h) - 1, ls, s); });
    DeviceBuffer big = DeviceBuffer::zeroed(4 * state_len(h) * 4);
    expect_invalid("replay_batch overlap", "layers' regions overlap", [&] { replay_batch(meta, big, big, state_len(h), ls, s); });
    expect_invalid("conv_shift_batch none", "no layers", [&] { conv_shift_batch(h, 0, meta, conv, 2 * WINDOW * c, RowView::dense(pb, c + h), 0, s); });
    DeviceBuffer conv4 = DeviceBuffer::zeroed(4 * WINDOW * c * 2);
    expect_invalid("conv_shift_batch overlap", "windows overlap", [&] { conv_shift_batch(h, 2, meta, conv4, WINDOW * c, RowView::dense(pb, c + h), 0, s); });

    PrefillWorkspace ws = PrefillWorkspace::create(h, 1, 20);
    CHECK(ws.rows_per_pass == 32 && ws.buf.bytes() == 34816 * h * 2);
    CHECK(PrefillWorkspace::within(h, 1, 3 * 34816 * h + 5).rows_per_pass == 48);
    auto prefill = [&](const Weights& ww) {
        Prefill pf;
        pf.weights = &ww, pf.rows = 1, pf.p = RowView::dense(pb, c + h), pf.b_off = (long long)c, pf.a = RowView::dense(ab, h * DK), pf.g = RowView::dense(gb, h * DV);
        pf.conv = &conv, pf.state = &state, pf.state_out = StateOut::in_place(), pf.out = RowView::dense(ob, h * DV), pf.workspace = &ws;
        return pf;
    };
    expect_invalid("prefill vb", "value_blocks", [&] { Prefill pf = prefill(w); pf.value_blocks = 3; pf.launch(s); });
    Weights steep = weights(h, -6.0f);
    expect_invalid("prefill lower", "lower bound", [&] { prefill(steep).launch(s); });
    expect_invalid("prefill skip", "always writes its state", [&] { Prefill pf = prefill(w); pf.state_out = StateOut::skip(); pf.launch(s); });
    PrefillWorkspace other = PrefillWorkspace::create(h + 1, 1, 16);
    expect_invalid("prefill ws", "workspace for", [&] { Prefill pf = prefill(w); pf.workspace = &other; pf.launch(s); });
    expect_invalid("prefill batch skip", "always writes its state", [&] {
        PrefillBatch pbh;
        pbh.weights = &w, pbh.p = RowView::dense(pb, c + h), pbh.b_off = (long long)c, pbh.a = RowView::dense(ab, h * DK), pbh.g = RowView::dense(gb, h * DV);
        pbh.conv = &conv, pbh.state = &state, pbh.state_out = StateOut::skip(), pbh.out = RowView::dense(ob, h * DV), pbh.workspace = &ws;
        pbh.launch(meta, s);
    });
    // the form switches: exact by default; each setter returns the form that was in force
    CHECK(prefill_form() == Form::Exact && verify_form() == Form::Exact && commit_form() == Form::Exact);
    CHECK(set_verify_form(Form::Chunked) == Form::Exact && verify_form() == Form::Chunked && set_verify_form(Form::Exact) == Form::Chunked);
    CHECK(set_commit_form(Form::Chunked) == Form::Exact && commit_form() == Form::Chunked && set_commit_form(Form::Exact) == Form::Chunked);
    CHECK(set_prefill_form(Form::Chunked) == Form::Exact && prefill_form() == Form::Chunked && set_prefill_form(Form::Exact) == Form::Chunked);
    std::printf(failures ? "%d FAILED\n" : "all host checks passed\n", failures);
    return failures ? 1 : 0;
}
