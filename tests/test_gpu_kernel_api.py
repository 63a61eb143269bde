"""The checked wrappers (glm53f-afd_b200/kernel.py, the mirror of the reference's kernel.rs) on the GPU.

The flows are the reference's own (crates/glm53f-kda/tests/gpu.rs: single chain; a verify round over a batch
followed by the commit's replay and conv shift; a batched prefill handing over to decode), written against the
wrapper types so that they read like the reference's tests.  Arithmetic parity is covered by test_gpu_chain.py and
test_gpu_prefill.py through the raw ABI; here the wrappers must reproduce those results and the oracle's bitwise
identities.
"""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    k = importlib.import_module("glm53f-afd_b200.kernel")
    importlib.import_module("glm53f-afd_b200").ffi.load()
    return k


def bits(K, x):
    return K._bf16_encode(x)


def upload_rows(K, rows):
    """Engine layout: p rows [q|k|v|b] of C + H columns, dense a and gate rows."""
    h, r = rows.heads, rows.rows
    c = K.channels(h)
    p = np.zeros((r, c + h), np.float32)
    p[:, :c] = rows.qkv.reshape(r, c)
    p[:, c:] = rows.b.reshape(r, h)
    return (K.RowView.dense(K.DeviceBuffer.from_slice(bits(K, p.reshape(-1))), c + h), c,
            K.RowView.dense(K.DeviceBuffer.from_slice(bits(K, rows.a)), h * DK), K.RowView.dense(K.DeviceBuffer.from_slice(bits(K, rows.gate)), h * DV))


def layer(K, o, heads, seed):
    p = o.Layer(heads, seed)
    return p, K.Weights.upload(K.LayerParams(heads, p.conv_w, p.a_log, p.dt_bias, p.norm_w, p.eps, p.lower))


def status_ok():
    pkg = importlib.import_module("glm53f-afd_b200")
    assert pkg.core.device_status() == 0


def test_chain_then_replay_and_conv_shift(K, oracle):
    o, h, r = oracle, 4, 5
    p, w = layer(K, o, h, 41)
    conv, s0, rows = o.conv_window(h, 41), o.state(h, 41, 0.5), o.Rows(h, r, 41)
    pv, b_off, av, gv = upload_rows(K, rows)
    d_conv, d_state = K.DeviceBuffer.from_slice(bits(K, conv)), K.DeviceBuffer.from_slice(s0)
    d_next = K.DeviceBuffer.zeroed(K.state_len(h) * 4)
    out = K.RowView.dense(K.DeviceBuffer.zeroed(r * h * DV * 2), h * DV)
    saves = K.Saves.alloc(h, r)
    stream = K.Stream()
    K.Chain(w, r, pv, b_off, av, gv, d_conv, 0, d_state, 0, K.StateOut.To(d_next, 0), out, saves).launch(stream)
    stream.synchronize()
    status_ok()
    sv = saves.download(r)
    got = d_next.download(np.float32, K.state_len(h))
    # the recurrence given the kernel's own replay inputs is exact (no transcendental in the update)
    assert np.array_equal(o.replay(s0, sv, r).view(np.uint32), got.view(np.uint32))
    c = o.chain(p, conv, s0, rows)
    y = K._bf16_decode(out.buf.download(np.uint16, r * h * DV))
    assert np.max(np.abs(y - c.out)) / np.max(np.abs(c.out)) <= 1.0 / 256.0
    assert np.array_equal(d_state.download(np.float32, K.state_len(h)), s0)  # the input state is untouched
    # a rollback to 3 rows: replay into a third buffer, and the window past the kept rows in place
    d_roll = K.DeviceBuffer.zeroed(K.state_len(h) * 4)
    K.replay(h, 3, (d_state, 0), (d_roll, 0), saves, stream)
    K.conv_shift(h, 3, d_conv, 0, pv, stream)
    stream.synchronize()
    assert np.array_equal(d_roll.download(np.float32, K.state_len(h)).view(np.uint32), o.replay(s0, sv, 3).view(np.uint32))
    assert np.array_equal(d_conv.download(np.uint16, conv.size), bits(K, o.conv_shift(conv, rows, 3)))
    with pytest.raises(K.Invalid):
        K.replay(h, r + 1, (d_state, 0), (d_roll, 0), saves, stream)


@pytest.mark.parametrize("bf16", [False, True])
def test_verify_round_then_commit_over_a_batch(K, oracle, bf16):
    """ChainBatch with StateOut.Skip and saves (the verify round), then replay_batch and conv_shift_batch with the
    accepted prefixes: every request's state equals the oracle's replay of the kernel's saves, bitwise, and the chain
    over a batch equals the chain over each request alone."""
    o, h, layers = oracle, 4, 2
    reqs, keep = [4, 1, 3], [2, 0, 3]
    es = 2 if bf16 else 4
    c = K.channels(h)
    meta = K.BatchMeta.new(4)
    meta.set([K.Request(n, i * K.WINDOW * c, i * K.state_len(h)) for i, n in enumerate(reqs)], keep)
    total = sum(reqs)
    stream = K.Stream()
    ls = K.LayerSaves.alloc(layers, h, total)
    convs = K.DeviceBuffer.zeroed(layers * len(reqs) * K.WINDOW * c * 2)
    states = K.DeviceBuffer.zeroed(layers * len(reqs) * K.state_len(h) * es)
    p_all = K.DeviceBuffer.zeroed(layers * total * (c + h) * 2)
    host = []
    for l in range(layers):
        p, w = layer(K, o, h, 50 + l)
        rows = o.Rows(h, total, 60 + l)
        pv, b_off, av, gv = upload_rows(K, rows)
        p_all.upload_at(l * total * (c + h), pv.buf.download(np.uint16, total * (c + h)))
        per_req = []
        for i, n in enumerate(reqs):
            conv, s0 = o.conv_window(h, 70 + 10 * l + i), o.state(h, 70 + 10 * l + i, 0.5)
            if bf16:
                s0 = K._bf16_decode(bits(K, s0))
            convs.upload_at((l * len(reqs) + i) * K.WINDOW * c, bits(K, conv))
            states.upload_at((l * len(reqs) + i) * K.state_len(h), bits(K, s0) if bf16 else s0)
            per_req.append((conv, s0))
        host.append((p, rows, per_req))
        # this layer's verify round: states and windows of layer l start at l * (requests' worth)
        view = lambda b, n: K.DeviceBuffer(b.t[l * n:(l + 1) * n])
        l_conv, l_state = view(convs, len(reqs) * K.WINDOW * c * 2), view(states, len(reqs) * K.state_len(h) * es)
        out = K.RowView.dense(K.DeviceBuffer.zeroed(total * h * DV * 2), h * DV)
        saves = K.Saves.alloc(h, total)
        cb = K.ChainBatch(w, pv, b_off, av, gv, l_conv, l_state, K.StateOut.Skip, out, saves)
        (cb.launch_bf16_state if bf16 else cb.launch)(meta, stream)
        stream.synchronize()
        ls.fill_layer(l, saves, total)
        # batch == single: request 0 alone through the one-request entry point (f32 states only there)
        if not bf16:
            single = K.RowView.dense(K.DeviceBuffer.zeroed(reqs[0] * h * DV * 2), h * DV)
            K.Chain(w, reqs[0], pv, b_off, av, gv, l_conv, 0, l_state, 0, K.StateOut.Skip, single, None).launch(stream)
            stream.synchronize()
            assert np.array_equal(single.buf.download(np.uint16, reqs[0] * h * DV), out.buf.download(np.uint16, reqs[0] * h * DV))
    status_ok()
    stride_s, stride_c = len(reqs) * K.state_len(h), len(reqs) * K.WINDOW * c
    (K.replay_batch_bf16_state if bf16 else K.replay_batch)(meta, states, states, stride_s, ls, stream)
    K.conv_shift_batch(h, layers, meta, convs, stride_c, K.RowView.dense(p_all, c + h), total * (c + h), stream)
    stream.synchronize()
    status_ok()
    row0 = np.concatenate([[0], np.cumsum(reqs)])
    for l, (p, rows, per_req) in enumerate(host):
        sv_all = K.HostSaves(h, total, ls.k.download(np.float32, total * h * DK, l * ls.kv_stride()),
                             K._bf16_decode(ls.v.download(np.uint16, total * h * DV, l * ls.kv_stride())),
                             ls.g.download(np.float32, total * h * DK, l * ls.kv_stride()), ls.b.download(np.float32, total * h, l * ls.b_stride()))
        for i, n in enumerate(reqs):
            conv, s0 = per_req[i]
            a, b = row0[i], row0[i] + n
            sv = K.HostSaves(h, n, sv_all.k[a * h * DK:b * h * DK], sv_all.v[a * h * DV:b * h * DV], sv_all.g[a * h * DK:b * h * DK],
                             sv_all.beta[a * h:b * h])
            want = o.replay(s0, sv, keep[i], bf16_state=bf16)
            at = (l * len(reqs) + i) * K.state_len(h)
            got = K._bf16_decode(states.download(np.uint16, K.state_len(h), at)) if bf16 else states.download(np.float32, K.state_len(h), at)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (l, i)
            wconv = o.conv_shift(conv, rows.slice(a, n), keep[i])
            assert np.array_equal(convs.download(np.uint16, K.WINDOW * c, (l * len(reqs) + i) * K.WINDOW * c), bits(K, wconv)), (l, i)


def test_prefill_batch_hands_over_to_decode(K, oracle):
    """PrefillBatch over two prompts, then one decode row each through ChainBatch from the states and windows the
    prefill left: equals the chain over prompt + 1 rows."""
    o, h = oracle, 4
    lens = [37, 80]
    c = K.channels(h)
    p, w = layer(K, o, h, 90)
    stream = K.Stream()
    meta = K.BatchMeta.new(2)
    meta.set([K.Request(n, i * K.WINDOW * c, i * K.state_len(h)) for i, n in enumerate(lens)])
    full = [o.Rows(h, n + 1, 91 + i) for i, n in enumerate(lens)]
    cat = o.Rows(h, sum(lens))
    for f in ("qkv", "a", "b", "gate"):
        setattr(cat, f, np.concatenate([getattr(r.slice(0, n), f) for r, n in zip(full, lens)]))
    pv, b_off, av, gv = upload_rows(K, cat)
    conv0 = [o.conv_window(h, 95 + i) for i in range(2)]
    s0 = [o.state(h, 95 + i, 0.5) for i in range(2)]
    convs = K.DeviceBuffer.from_slice(bits(K, np.concatenate(conv0)))
    states = K.DeviceBuffer.from_slice(np.concatenate(s0))
    out = K.RowView.dense(K.DeviceBuffer.zeroed(sum(lens) * h * DV * 2), h * DV)
    ws = K.PrefillWorkspace.new(h, 2, 32)
    K.PrefillBatch(w, pv, b_off, av, gv, convs, states, K.StateOut.InPlace, out, 0, ws).launch(meta, stream)
    # one decode row per request
    meta1 = K.BatchMeta.new(2)
    meta1.set([K.Request(1, i * K.WINDOW * c, i * K.state_len(h)) for i in range(2)])
    last = o.Rows(h, 2)
    for f in ("qkv", "a", "b", "gate"):
        setattr(last, f, np.concatenate([getattr(r.slice(n, 1), f) for r, n in zip(full, lens)]))
    pv1, _, av1, gv1 = upload_rows(K, last)
    out1 = K.RowView.dense(K.DeviceBuffer.zeroed(2 * h * DV * 2), h * DV)
    K.ChainBatch(w, pv1, b_off, av1, gv1, convs, states, K.StateOut.InPlace, out1, None).launch(meta1, stream)
    stream.synchronize()
    status_ok()
    for i, n in enumerate(lens):
        ref = o.chain(p, conv0[i], s0[i], full[i])
        got_s = states.download(np.float32, K.state_len(h), i * K.state_len(h))
        assert np.linalg.norm(got_s - ref.state) / np.linalg.norm(ref.state) <= 1e-3
        y1 = K._bf16_decode(out1.buf.download(np.uint16, h * DV, i * h * DV))
        assert np.max(np.abs(y1 - ref.out[n * h * DV:])) / np.max(np.abs(ref.out)) <= 1.0 / 256.0
    with pytest.raises(K.Invalid, match="always writes"):
        K.PrefillBatch(w, pv, b_off, av, gv, convs, states, K.StateOut.Skip, out, 0, ws).launch(meta, stream)
