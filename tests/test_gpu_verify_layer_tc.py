"""The chunked form of draft verification behind the reference's own symbol (glm53f_kda_verify_mode(1)):
glm53f_kda_chain_batch_bf16state with state_out == NULL and the replay saves given runs the verify prologue and the
16-row tensor-core kernel instead of the row-by-row chain.

Held to the exact form of the same call the way the reference holds a verify window to serial steps
(crates/glm53f-kda/tests/gpu_bf16_state.rs:331-382, crates/glm53f-forward/tests/verify_commit.rs:1-8): the replay
saves must be the exact form's bit for bit (so the commit of any prefix leaves serial decode's state), the state must
not be touched, and the outputs (bf16, after the gated norm) must agree within the reference's tier for a chunked
bf16 path, 5e-2 of max|ref| (crates/glm53f-kda/src/goldens.rs:756-761), and within rel-L2 1e-2.  Saturated and mixed
gates as in crates/glm53f-kda/tests/cpu_reference.rs:399-450.
"""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kda_gpu

    kda_gpu.product()
    return kda_gpu


@pytest.fixture()
def chunked(G):
    """The chunked form for the duration of one test; the exact form (the default) again afterwards."""
    lib = G.product()
    prev = lib.glm53f_kda_verify_mode(1)
    yield lib
    lib.glm53f_kda_verify_mode(prev)


def exact(G, lib, *args, **kw):
    prev = lib.glm53f_kda_verify_mode(0)
    try:
        return G.run_chain(lib, *args, **kw)
    finally:
        lib.glm53f_kda_verify_mode(prev)


def same_saves(G, got, want):
    for f in ("k", "v", "g", "beta"):
        assert np.array_equal(G.bits(getattr(got, f)), G.bits(getattr(want, f))), f


def close_outputs(G, got, want):
    assert np.isfinite(got.out).all()
    assert G.max_abs(got.out, want.out) / G.max_abs(want.out) <= 5e-2
    assert G.rel_l2(got.out, want.out) <= 1e-2


@pytest.mark.parametrize("r,gates", [(1, "random"), (2, "random"), (7, "random"), (9, "random"), (16, "random"),
                                     (16, "strongest"), (16, "mixed"), (5, "strongest")])
def test_chunked_verify_agrees_with_the_exact_form(G, oracle, chunked, r, gates):
    o, lib, h = oracle, chunked, 4
    p, conv, s0, rows = o.Layer(h, 80 + r), o.conv_window(h, 80 + r), o.bf16_round_np(o.state(h, 80 + r, 0.5)), o.Rows(h, r, 80 + r)
    if gates == "strongest":   # every channel at the lower bound: each row decays by exp(-5)
        rows.a[:] = 1e4
    elif gates == "mixed":     # strong and no decay alternating by row
        rows.a[:] = np.where((np.arange(rows.a.size) // (h * DK)) % 3 == 0, -1e4, 1e4)
    w = G.Weights(p)
    want = exact(G, lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w)
    got = G.run_chain(lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w)
    assert got.rc == 0
    G.check_status()
    same_saves(G, got, want)
    close_outputs(G, got, want)
    if r > 2:  # the chunked form did run: thousands of outputs through bf16 operands do not all round alike
        assert not np.array_equal(G.bits(got.out), G.bits(want.out))
    assert np.array_equal(G.bits(got.state_in_after), G.bits(s0)) and not got.state.any()
    assert (got.out_raw[r * h * DV:] == 0xFFFF).all()
    # the commit of every prefix from these saves: serial decode's state, bit for bit
    for keep in sorted({0, 1, r // 2, r}):
        want_state = s0 if keep == 0 else exact(G, lib, p, conv, s0, rows.slice(0, keep), bf16_state=True, w=w).state
        assert np.array_equal(G.bits(G.run_replay(lib, h, s0, got, keep, bf16_state=True)), G.bits(want_state)), keep


def test_chunked_verify_batch_with_scattered_slots_and_an_empty_window(G, oracle, chunked):
    o, lib, h = oracle, chunked, 4   # a head count whose rows (3 * h * 128 + h elements) stay 8-byte aligned
    lens, order = [16, 0, 4, 11], [2, 0, 3, 1]
    reqs = [(o.conv_window(h, 31 + i), o.bf16_round_np(o.state(h, 31 + i, 0.5)), o.Rows(h, n, 31 + i)) for i, n in enumerate(lens)]
    p = o.Layer(h, 31)
    w = G.Weights(p)
    c, total = 3 * h * DK, sum(lens)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    allrows = o.Rows(h, total)
    for name in ("qkv", "a", "b", "gate"):
        setattr(allrows, name, np.concatenate([getattr(r[2], name) for r in reqs]))
    pbuf, base, p_stride, b_off = G.pack_rows(allrows)
    slen, clen = h * DV * DK, 3 * c
    pool, cpool = np.zeros(4 * slen, np.float32), np.zeros(4 * clen, np.float32)
    for i, sl in enumerate(order):
        pool[sl * slen:(sl + 1) * slen] = reqs[i][1]
        cpool[sl * clen:(sl + 1) * clen] = reqs[i][0]
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(allrows.a), G.dev_bf16(allrows.gate)
    d_conv, d_pool = G.dev_bf16(cpool), G.dev_bf16(pool)
    out_stride = h * DV + 8   # padded output rows: the gaps must stay untouched
    d_out = torch.full((total * out_stride,), -1, dtype=torch.int16, device="cuda")
    d_k = torch.zeros(total * h * DK, dtype=torch.float32, device="cuda")
    d_v = torch.zeros(total * h * DV, dtype=torch.int16, device="cuda")
    d_gs, d_b = torch.zeros_like(d_k), torch.zeros(total * h, dtype=torch.float32, device="cuda")
    d_cu, d_soff, d_coff = G.dev_i32(cu), G.dev_i64([sl * slen for sl in order]), G.dev_i64([sl * clen for sl in order])
    rc = lib.glm53f_kda_chain_batch_bf16state(h, 4, G.ptr(d_cu), C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK,
                                              G.ptr(d_g), h * DV, G.ptr(d_conv), G.ptr(d_coff), G.ptr(w.conv_w), G.ptr(d_pool), None,
                                              G.ptr(d_soff), G.ptr(w.a_log), G.ptr(w.dt_bias), G.ptr(w.norm_w), w.eps, w.lower,
                                              G.ptr(d_out), out_stride, G.ptr(d_k), G.ptr(d_v), G.ptr(d_gs), G.ptr(d_b), None)
    assert rc == 0
    G.check_status()
    raw = d_out.cpu().numpy().view(np.uint16).reshape(total, out_stride)
    assert (raw[:, h * DV:] == 0xFFFF).all()
    out = G.widen(raw[:, :h * DV].reshape(-1))
    assert np.array_equal(G.bits(G.host_bf16(d_pool)), G.bits(pool)) and np.array_equal(G.host_bf16(d_conv), cpool)
    ks, vs, gs, bs = G.host_f32(d_k), G.host_bf16(d_v), G.host_f32(d_gs), G.host_f32(d_b)
    for i, n in enumerate(lens):
        if n == 0:
            continue
        one = exact(G, lib, p, reqs[i][0], reqs[i][1], reqs[i][2], bf16_state=True, write_state=False, w=w)
        r0 = cu[i]
        got = G.Result()
        got.out = out[r0 * h * DV:(r0 + n) * h * DV]
        close_outputs(G, got, one)
        assert np.array_equal(G.bits(ks[r0 * h * DK:(r0 + n) * h * DK]), G.bits(one.k)), i
        assert np.array_equal(G.bits(vs[r0 * h * DV:(r0 + n) * h * DV]), G.bits(one.v)), i
        assert np.array_equal(G.bits(gs[r0 * h * DK:(r0 + n) * h * DK]), G.bits(one.g)), i
        assert np.array_equal(G.bits(bs[r0 * h:(r0 + n) * h]), G.bits(one.beta)), i
        # the same request alone through the chunked form: the same bits (results do not depend on the batching)
        alone = G.run_chain(lib, p, reqs[i][0], reqs[i][1], reqs[i][2], bf16_state=True, write_state=False, w=w)
        assert np.array_equal(G.bits(alone.out), G.bits(got.out)), i
        assert not np.array_equal(G.bits(got.out), G.bits(one.out)), i   # the chunked form did run


def test_calls_the_chunked_form_cannot_take_run_the_exact_form(G, oracle, chunked):
    o, lib, h, r = oracle, chunked, 4, 6
    p, conv, s0, rows = o.Layer(h, 17), o.conv_window(h, 17), o.bf16_round_np(o.state(h, 17, 0.5)), o.Rows(h, r, 17)
    w = G.Weights(p)
    want = exact(G, lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w)
    # output rows that are not 16-byte aligned, and projection rows that start on an odd element
    for kw in ({"out_stride": h * DV + 4}, {"p_stride": 3 * h * DK + h + 1, "pad_front": 3}):
        got = G.run_chain(lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w, **kw)
        assert np.array_equal(G.bits(got.out), G.bits(want.out)), kw
        same_saves(G, got, want)
    # a call that writes the state is a decode or prefill step, not a verify: exact
    stepped = G.run_chain(lib, p, conv, s0, rows, bf16_state=True, w=w)
    ref = exact(G, lib, p, conv, s0, rows, bf16_state=True, w=w)
    assert np.array_equal(G.bits(stepped.out), G.bits(ref.out)) and np.array_equal(G.bits(stepped.state), G.bits(ref.state))
    G.check_status()


def test_a_window_longer_than_16_rows_is_reported(G, oracle, chunked, pkg):
    import importlib

    core = importlib.import_module("glm53f-afd_b200.core")
    o, lib, h, r = oracle, chunked, 4, 18
    p, conv, s0, rows = o.Layer(h, 23), o.conv_window(h, 23), o.bf16_round_np(o.state(h, 23, 0.5)), o.Rows(h, r, 23)
    w = G.Weights(p)
    want = exact(G, lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w)
    got = G.run_chain(lib, p, conv, s0, rows, bf16_state=True, write_state=False, w=w)
    assert core.device_status() == 122 and core.device_status() == 0
    n = 16 * h * DV
    first = G.Result()
    first.out = got.out[:n]
    ref = G.Result()
    ref.out = want.out[:n]
    close_outputs(G, first, ref)
    # the replay saves cover EVERY row of the over-long window, bit for bit those of the exact form: a commit of any
    # prefix replays real values even though the rows past 16 got no output
    for name in ("k", "g", "v", "beta"):
        assert np.array_equal(G.bits(getattr(got, name)), G.bits(getattr(want, name))), name


def test_the_mode_switch_reports_and_restores(G):
    lib = G.product()
    assert lib.glm53f_kda_verify_mode(-1) == 0   # the default is the exact form
    assert lib.glm53f_kda_verify_mode(1) == 0
    assert lib.glm53f_kda_verify_mode(7) == 1    # any other value only queries
    assert lib.glm53f_kda_verify_mode(0) == 1
    assert lib.glm53f_kda_verify_mode(-1) == 0
