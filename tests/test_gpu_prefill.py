"""GPU parity of the layer prefill entry points (glm53f_kda_prefill*), after the reference crate's
tests/gpu_prefill.rs: the prefill against the chain, segments and the prefill -> decode hand-off, the conv
window advance, batches, zero-row requests and the launcher's rejections."""
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


def run_prefill(G, lib, p, conv, state, rows, w=None, value_blocks=0, ws_rows=64, lower=None):
    h, r = rows.heads, rows.rows
    w = w or G.Weights(p)
    pbuf, base, p_stride, b_off = G.pack_rows(rows)
    pad = np.zeros(8, np.float32)  # a request without rows still passes non-null row pointers
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(rows.a if r else pad), G.dev_bf16(rows.gate if r else pad)
    d_conv = G.dev_bf16(conv)
    d_out = torch.full((max(r, 1) * h * DV + 64,), -1, dtype=torch.int16, device="cuda")
    d_sin = G.dev_f32(state)
    d_sout = torch.zeros_like(d_sin)
    nbytes = lib.glm53f_kda_prefill_workspace_bytes(h, 1, ws_rows)
    ws = torch.zeros(max(nbytes // 4, 1), device="cuda")
    rc = lib.glm53f_kda_prefill(h, r, C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK, G.ptr(d_g), h * DV,
                                G.ptr(d_conv), G.ptr(w.conv_w), G.ptr(d_sin), G.ptr(d_sout), G.ptr(w.a_log), G.ptr(w.dt_bias),
                                G.ptr(w.norm_w), w.eps, w.lower if lower is None else lower, G.ptr(d_out), h * DV, value_blocks,
                                G.ptr(ws), nbytes, None)
    torch.cuda.synchronize()
    res = G.Result()
    res.rc = rc
    if rc == 0:
        res.out = G.host_bf16(d_out)[:r * h * DV]
        res.tail = d_out[r * h * DV:].cpu().numpy()
        res.state = G.host_f32(d_sout)
        res.conv = G.host_bf16(d_conv)
    return res


# gpu_prefill.rs:250-300: the prefill against the chain, any length.
@pytest.mark.parametrize("r", [1, 5, 16, 17, 40, 100, 257])
def test_prefill_agrees_with_the_chain(G, oracle, r):
    o = oracle
    h = 4
    p, conv, s0, rows = o.Layer(h, 60 + r), o.conv_window(h, 60 + r), o.state(h, 60 + r, 0.5), o.Rows(h, r, 60 + r)
    lib = G.product()
    w = G.Weights(p)
    pre = run_prefill(G, lib, p, conv, s0, rows, w=w)
    assert pre.rc == 0
    G.check_status()
    ch = G.run_chain(lib, p, conv, s0, rows, w=w, saves=False)
    # the reference's bounds (state to f32 rounding, outputs within a bf16 ulp normwise, few differing)
    assert G.max_abs(pre.state, ch.state) / G.max_abs(ch.state) < 1e-5
    assert G.max_abs(pre.out, ch.out) / G.max_abs(ch.out) < 1.0 / 256.0
    assert G.ulps(pre.out, ch.out)[1] * 1000 <= ch.out.size
    assert (pre.tail == -1).all()
    assert np.array_equal(pre.conv, o.conv_shift(conv, rows, r))
    # and against the oracle's host model of the chunked kernel
    f = o.prefill(p, conv, s0, rows)
    assert G.max_abs(pre.state, f.state) / G.max_abs(f.state) < 1e-3
    assert G.max_abs(pre.out, f.out) / G.max_abs(f.out) < 1.0 / 256.0


# gpu_prefill.rs:379-411: two segments, then a decode step, equal one chain over everything.
def test_segments_and_the_hand_off_to_decode(G, oracle):
    o = oracle
    h = 3
    p, conv, s0, rows = o.Layer(h, 91), o.conv_window(h, 91), o.state(h, 91, 0.5), o.Rows(h, 61, 91)
    lib = G.product()
    w = G.Weights(p)
    a = run_prefill(G, lib, p, conv, s0, rows.slice(0, 37), w=w)
    b = run_prefill(G, lib, p, a.conv, a.state, rows.slice(37, 23), w=w)
    step = G.run_chain(lib, p, b.conv, b.state, rows.slice(60, 1), w=w, saves=False)
    whole = G.run_chain(lib, p, conv, s0, rows, w=w, saves=False)
    assert G.max_abs(step.state, whole.state) / G.max_abs(whole.state) < 1e-5
    got = np.concatenate([a.out, b.out, step.out])
    assert G.max_abs(got, whole.out) / G.max_abs(whole.out) < 1.0 / 256.0
    empty = run_prefill(G, lib, p, conv, s0, rows.slice(0, 0), w=w)
    assert empty.rc == 0 and np.array_equal(G.bits(empty.state), G.bits(s0)) and np.array_equal(empty.conv, conv)
    G.check_status()


# gpu_prefill.rs:303-373: a batch with its own rows, states and windows equals the single requests.
@pytest.mark.parametrize("bf16", [False, True])
def test_batched_prefill_equals_single_requests(G, oracle, bf16):
    o = oracle
    lib = G.product()
    h, lens = 2, [33, 0, 70]
    c = 3 * h * DK
    p = o.Layer(h, 5)
    w = G.Weights(p)
    reqs = [(o.conv_window(h, 5 + i), o.state(h, 5 + i, 0.5), o.Rows(h, n, 5 + i)) for i, n in enumerate(lens)]
    total = sum(lens)
    allr = o.Rows(h, total)
    allr.qkv = np.concatenate([r[2].qkv for r in reqs])
    allr.a = np.concatenate([r[2].a for r in reqs])
    allr.b = np.concatenate([r[2].b for r in reqs])
    allr.gate = np.concatenate([r[2].gate for r in reqs])
    pbuf, base, p_stride, b_off = G.pack_rows(allr)
    states = [o.bf16_round_np(r[1]) if bf16 else r[1] for r in reqs]
    pool = np.concatenate(states)
    slen = h * DV * DK
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(allr.a), G.dev_bf16(allr.gate)
    d_conv = G.dev_bf16(np.concatenate([r[0] for r in reqs]))
    d_pool = G.dev_bf16(pool) if bf16 else G.dev_f32(pool)
    d_out = torch.zeros(total * h * DV, dtype=torch.int16, device="cuda")
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    d_cu, d_soff, d_coff = G.dev_i32(cu), G.dev_i64([i * slen for i in range(3)]), G.dev_i64([i * 3 * c for i in range(3)])
    nbytes = lib.glm53f_kda_prefill_workspace_bytes(h, 3, 32)
    ws = torch.zeros(nbytes // 4, device="cuda")
    fn = lib.glm53f_kda_prefill_batch_bf16state if bf16 else lib.glm53f_kda_prefill_batch
    rc = fn(h, 3, G.ptr(d_cu), max(lens), C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK, G.ptr(d_g),
            h * DV, G.ptr(d_conv), G.ptr(d_coff), G.ptr(w.conv_w), G.ptr(d_pool), G.ptr(d_pool), G.ptr(d_soff), G.ptr(w.a_log),
            G.ptr(w.dt_bias), G.ptr(w.norm_w), w.eps, w.lower, G.ptr(d_out), h * DV, 1, G.ptr(ws), nbytes, None)
    assert rc == 0
    G.check_status()
    out = G.host_bf16(d_out)
    after = G.host_bf16(d_pool) if bf16 else G.host_f32(d_pool)
    convs = G.host_bf16(d_conv)
    for i, n in enumerate(lens):
        ch = G.run_chain(lib, p, reqs[i][0], states[i], reqs[i][2], bf16_state=bf16, w=w, saves=False) if n else None
        want_state = ch.state if n else states[i]
        tol = 2e-2 if bf16 else 1e-5  # the reference's bf16 prefill bound (gpu_bf16_state.rs:593-656)
        assert G.max_abs(after[i * slen:(i + 1) * slen], want_state) / G.max_abs(want_state) <= tol, i
        if n:
            r0 = cu[i]
            got = out[r0 * h * DV:(r0 + n) * h * DV]
            assert G.max_abs(got, ch.out) / G.max_abs(ch.out) <= (1.0 / 32.0 if bf16 else 1.0 / 256.0), i
        assert np.array_equal(convs[i * 3 * c:(i + 1) * 3 * c], o.conv_shift(reqs[i][0], reqs[i][2], n)), i


# gpu_prefill.rs:542-584
def test_prefill_rejections(G, oracle):
    o = oracle
    lib = G.product()
    h = 2
    p, conv, s0, rows = o.Layer(h, 3), o.conv_window(h, 3), o.state(h, 3, 0.5), o.Rows(h, 4, 3)
    assert run_prefill(G, lib, p, conv, s0, rows, value_blocks=3).rc == 1
    assert run_prefill(G, lib, p, conv, s0, rows, lower=-6.0).rc == 1
    assert run_prefill(G, lib, p, conv, s0, rows, lower=0.5).rc == 1
    assert run_prefill(G, lib, p, conv, s0, rows, ws_rows=0).rc == 1  # workspace smaller than one chunk
    assert lib.glm53f_kda_prefill_workspace_bytes(h, 1, 16) == 34816 * h
    assert lib.glm53f_kda_prefill_workspace_bytes(64, 4, 2048) == 128 * 34816 * 64 * 4
    assert lib.glm53f_kda_prefill_workspace_bytes(0, 1, 16) == 0
    for vb in (0, 1, 2, 4):
        assert run_prefill(G, lib, p, conv, s0, rows, value_blocks=vb).rc == 0
