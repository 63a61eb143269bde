"""The chunked form of the layer prefill entry points (glm53f_kda_prefill_mode(1)): the layer prologue followed by the
chunk-64 tensor-core kernel, in passes over the caller's workspace, behind the reference's own three symbols.

Held to the chain (the exact form of the same entry points) the way the reference holds its chunked kernel to its chain
(crates/glm53f-kda/tests/gpu_prefill.rs:250-300, 303-373, 379-411, 419-456): any length, segments and the hand-off to
decode, batches with zero-row requests, both state types, the conv window advance, and the saturated and mixed gates
of crates/glm53f-kda/tests/cpu_reference.rs:399-450.  Bounds: the state within rel-L2 1e-3 of the chain's (the task's
bound on the FP32 state); the outputs (bf16, after the gated norm) within the reference's tier for a chunked bf16
path, 5e-2 of max|ref| (crates/glm53f-kda/src/goldens.rs:756-761), and within rel-L2 1e-2.  Results must not depend
on the workspace size or on the batching, bit for bit.
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
    prev = lib.glm53f_kda_prefill_mode(1)
    yield lib
    lib.glm53f_kda_prefill_mode(prev)


def prefill(G, lib, p, conv, state, rows, w, ws_rows=256, bf16=False):
    """One request through glm53f_kda_prefill_batch[_bf16state] (batch of one)."""
    h, r = rows.heads, rows.rows
    pbuf, base, p_stride, b_off = G.pack_rows(rows)
    pad = np.zeros(8, np.float32)
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(rows.a if r else pad), G.dev_bf16(rows.gate if r else pad)
    d_conv = G.dev_bf16(conv)
    d_out = torch.full((max(r, 1) * h * DV + 64,), -1, dtype=torch.int16, device="cuda")
    d_s = G.dev_bf16(state) if bf16 else G.dev_f32(state)
    nbytes = lib.glm53f_kda_prefill_workspace_bytes(h, 1, ws_rows)
    ws = torch.zeros(max(nbytes // 4, 1), device="cuda")
    fn = lib.glm53f_kda_prefill_batch_bf16state if bf16 else lib.glm53f_kda_prefill_batch
    d_cu, d_zero = G.dev_i32([0, r]), G.dev_i64([0])  # named: the metadata must outlive the launch
    rc = fn(h, 1, G.ptr(d_cu), r, C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK, G.ptr(d_g), h * DV,
            G.ptr(d_conv), G.ptr(d_zero), G.ptr(w.conv_w), G.ptr(d_s), G.ptr(d_s), G.ptr(d_zero), G.ptr(w.a_log),
            G.ptr(w.dt_bias), G.ptr(w.norm_w), w.eps, w.lower, G.ptr(d_out), h * DV, 0, G.ptr(ws), nbytes, None)
    assert rc == 0
    G.check_status()
    res = G.Result()
    res.out = G.host_bf16(d_out)[:r * h * DV]
    assert (d_out[r * h * DV:].cpu().numpy() == -1).all()
    res.state = G.host_bf16(d_s) if bf16 else G.host_f32(d_s)
    res.conv = G.host_bf16(d_conv)
    return res


def close(G, got, want, state_tol=1e-3):
    assert np.isfinite(got.state).all() and np.isfinite(got.out).all()
    assert G.rel_l2(got.state, want.state) <= state_tol
    if want.out.size:
        assert G.max_abs(got.out, want.out) / G.max_abs(want.out) <= 5e-2
        assert G.rel_l2(got.out, want.out) <= 1e-2


@pytest.mark.parametrize("r,gates", [(1, "random"), (17, "random"), (64, "random"), (100, "random"), (257, "random"), (600, "random"),
                                     (48, "strongest"), (48, "mixed"), (200, "strongest"), (200, "mixed")])
def test_chunked_prefill_agrees_with_the_chain(G, oracle, chunked, r, gates):
    o, lib, h = oracle, chunked, 4
    p, conv, s0, rows = o.Layer(h, 60 + r), o.conv_window(h, 60 + r), o.state(h, 60 + r, 0.5), o.Rows(h, r, 60 + r)
    if gates == "strongest":   # every channel at the lower bound: each row decays by exp(-5)
        rows.a[:] = 1e4
    elif gates == "mixed":     # strong and no decay alternating by row
        rows.a[:] = np.where((np.arange(rows.a.size) // (h * DK)) % 3 == 0, -1e4, 1e4)
    w = G.Weights(p)
    ch = G.run_chain(lib, p, conv, s0, rows, w=w, saves=False)
    runs = [prefill(G, lib, p, conv, s0, rows, w, ws_rows=n) for n in (64, 128, 1024)]
    close(G, runs[0], ch)
    for other in runs[1:]:  # the workspace sets the rows per pass, not the results
        assert np.array_equal(G.bits(other.out), G.bits(runs[0].out)) and np.array_equal(G.bits(other.state), G.bits(runs[0].state))
    assert np.array_equal(runs[0].conv, o.conv_shift(conv, rows, r))
    # a workspace below 64 rows a pass cannot hold a chunk's inputs: the call runs the exact form
    small = prefill(G, lib, p, conv, s0, rows, w, ws_rows=16)
    assert np.array_equal(G.bits(small.out), G.bits(ch.out)) and np.array_equal(G.bits(small.state), G.bits(ch.state))


def test_chunked_segments_and_the_hand_off_to_decode(G, oracle, chunked):
    o, lib, h = oracle, chunked, 3
    p, conv, s0, rows = o.Layer(h, 91), o.conv_window(h, 91), o.state(h, 91, 0.5), o.Rows(h, 161, 91)
    w = G.Weights(p)
    a = prefill(G, lib, p, conv, s0, rows.slice(0, 97), w)
    b = prefill(G, lib, p, a.conv, a.state, rows.slice(97, 63), w)
    step = G.run_chain(lib, p, b.conv, b.state, rows.slice(160, 1), w=w, saves=False)
    whole = G.run_chain(lib, p, conv, s0, rows, w=w, saves=False)
    got = G.Result()
    got.state, got.out = step.state, np.concatenate([a.out, b.out, step.out])
    close(G, got, whole)
    empty = prefill(G, lib, p, conv, s0, rows.slice(0, 0), w)
    assert np.array_equal(G.bits(empty.state), G.bits(s0)) and np.array_equal(empty.conv, conv)


@pytest.mark.parametrize("bf16", [False, True])
def test_chunked_batch_equals_single_requests(G, oracle, chunked, bf16):
    o, lib = oracle, chunked
    h, lens = 2, [133, 0, 70, 64]
    nreq, c = len(lens), 3 * h * DK
    p = o.Layer(h, 5)
    w = G.Weights(p)
    reqs = [(o.conv_window(h, 5 + i), o.state(h, 5 + i, 0.5), o.Rows(h, n, 5 + i)) for i, n in enumerate(lens)]
    total = sum(lens)
    allr = o.Rows(h, total)
    for name in ("qkv", "a", "b", "gate"):
        setattr(allr, name, np.concatenate([getattr(r[2], name) for r in reqs]))
    pbuf, base, p_stride, b_off = G.pack_rows(allr)
    states = [o.bf16_round_np(r[1]) if bf16 else r[1] for r in reqs]
    slen = h * DV * DK
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(allr.a), G.dev_bf16(allr.gate)
    d_conv = G.dev_bf16(np.concatenate([r[0] for r in reqs]))
    d_pool = G.dev_bf16(np.concatenate(states)) if bf16 else G.dev_f32(np.concatenate(states))
    d_out = torch.zeros(total * h * DV, dtype=torch.int16, device="cuda")
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    nbytes = lib.glm53f_kda_prefill_workspace_bytes(h, nreq, 64)
    ws = torch.zeros(nbytes // 4, device="cuda")
    fn = lib.glm53f_kda_prefill_batch_bf16state if bf16 else lib.glm53f_kda_prefill_batch
    d_cu, d_coff, d_soff = G.dev_i32(cu), G.dev_i64([i * 3 * c for i in range(nreq)]), G.dev_i64([i * slen for i in range(nreq)])
    rc = fn(h, nreq, G.ptr(d_cu), max(lens), C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK, G.ptr(d_g),
            h * DV, G.ptr(d_conv), G.ptr(d_coff), G.ptr(w.conv_w), G.ptr(d_pool), G.ptr(d_pool),
            G.ptr(d_soff), G.ptr(w.a_log), G.ptr(w.dt_bias), G.ptr(w.norm_w), w.eps, w.lower, G.ptr(d_out),
            h * DV, 1, G.ptr(ws), nbytes, None)
    assert rc == 0
    G.check_status()
    out = G.host_bf16(d_out)
    after = G.host_bf16(d_pool) if bf16 else G.host_f32(d_pool)
    convs = G.host_bf16(d_conv)
    for i, n in enumerate(lens):
        one = prefill(G, lib, p, reqs[i][0], states[i], reqs[i][2], w, bf16=bf16)   # the same request alone: the same bits
        assert np.array_equal(G.bits(after[i * slen:(i + 1) * slen]), G.bits(one.state)), i
        assert np.array_equal(G.bits(out[cu[i] * h * DV:(cu[i] + n) * h * DV]), G.bits(one.out)), i
        assert np.array_equal(convs[i * 3 * c:(i + 1) * 3 * c], o.conv_shift(reqs[i][0], reqs[i][2], n)), i
        if n:
            ch = G.run_chain(lib, p, reqs[i][0], states[i], reqs[i][2], bf16_state=bf16, w=w, saves=False)
            close(G, one, ch, state_tol=2e-2 if bf16 else 1e-3)   # bf16 states: the reference's own prefill bound (gpu_bf16_state.rs:593-656)


def test_the_mode_switch_reports_and_restores(G):
    lib = G.product()
    assert lib.glm53f_kda_prefill_mode(-1) == 0   # the default is the exact form
    assert lib.glm53f_kda_prefill_mode(1) == 0
    assert lib.glm53f_kda_prefill_mode(7) == 1    # any other value only queries
    assert lib.glm53f_kda_prefill_mode(0) == 1
    assert lib.glm53f_kda_prefill_mode(-1) == 0
