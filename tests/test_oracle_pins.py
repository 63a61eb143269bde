"""Pins the CPU oracle to the reference's own known-answer values and invariants.

Each test restates one test of the reference crate (crates/glm53f-kda/tests/cpu_reference.rs, or the unit
tests of src/bf16.rs), on the reference's own SplitMix64 streams, so the oracle the GPU parity tests lean on
is the reference's arithmetic and not a look-alike.  CPU only.
"""
import math

import numpy as np

DK = DV = 128
WINDOW = 3


def bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def rel_err(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def bf16_diff(o, a, b):
    ua = o.bf16_bits(a).astype(np.int32)
    ub = o.bf16_bits(b).astype(np.int32)
    oa = np.where(ua & 0x8000, -(ua & 0x7FFF), ua)
    ob = np.where(ub & 0x8000, -(ub & 0x7FFF), ub)
    d = np.abs(oa - ob)
    return int(d.max()), int((d != 0).sum())


# src/bf16.rs:52-77
def test_bf16_rounds_to_nearest_even_and_specials(oracle):
    o = oracle
    assert o.bf16_from_f32(1.0) == 0x3F80
    assert o.bf16_from_f32(1.0 + 1.0 / 256.0) == 0x3F80
    assert o.bf16_from_f32(1.0 + 3.0 / 256.0) == 0x3F82
    assert o.bf16_from_f32(float(np.uint32(0x3F808001).view(np.float32))) == 0x3F81
    assert o.bf16_round(-2.5) == -2.5
    assert o.bf16_to_f32(0xC020) == -2.5
    assert o.bf16_from_f32(math.inf) == 0x7F80
    assert o.bf16_from_f32(-math.inf) == 0xFF80
    assert o.bf16_from_f32(float(np.finfo(np.float32).max)) == 0x7F80
    assert math.isnan(o.bf16_to_f32(o.bf16_from_f32(math.nan)))
    assert o.bf16_from_f32(0.0) == 0x0000
    assert o.bf16_from_f32(-0.0) == 0x8000
    assert o.bf16_from_f32(float(np.uint32(0x00018000).view(np.float32))) == 0x0002
    assert o.bf16_ulp_distance(0x3F80, 0x3F81) == 1
    assert o.bf16_ulp_distance(0x0001, 0x8001) == 2
    # The vectorised numpy form used to prepare inputs agrees with the scalar one everywhere it is used.
    x = o.Rng(5).fill(4096, -300.0, 300.0)
    want = np.array([o.bf16_from_f32(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(o.bf16_bits(x), want)


# tests/cpu_reference.rs:36-55
def test_forget_gate_and_beta_hand_values(oracle):
    o = oracle
    assert o.log_decay(0.0, 0.0, 0.0, -5.0) == -2.5
    assert abs(o.decay(0.0, 0.0, 1.0, -5.0) - math.exp(-2.5)) < 1e-8
    assert abs(o.decay(1e4, 0.0, 1.0, -5.0) - math.exp(-5.0)) < 1e-9
    assert o.decay(-1e4, 0.0, 1.0, -5.0) == 1.0
    assert o.log_decay(1.0, -1.0, 3.0, -5.0) == -2.5
    assert o.decay(2.0, -1.0, 0.5, -5.0) == o.decay(0.5, 0.0, 1.0, -5.0)
    assert o.beta(0.0) == 0.5
    assert o.beta(20.0) == 1.0
    assert o.beta(-200.0) == 0.0
    assert o.beta(1.0) == o.bf16_round(0.7310586)


def one_head(o, w):
    p = o.Layer(1, 1)
    p.conv_w = np.tile(np.asarray(w, np.float32), p.channels)
    return p


# tests/cpu_reference.rs:66-100
def test_conv_hand_values(oracle):
    o = oracle
    p = one_head(o, [1.0, 2.0, 3.0, 4.0])
    c = p.channels
    conv = np.repeat(np.arange(1, WINDOW + 1, dtype=np.float32), c)
    rows = o.Rows(1, 2, 2)
    rows.qkv[:c] = 4.0
    rows.qkv[c:] = 5.0
    for r, want in ((0, 30.0), (1, 40.0)):
        q, k, v = o.conv_qkv(p, conv, rows, r, 0)
        assert (q == want).all() and (k == want).all() and (v == want).all()
    rows.qkv[:c] = -11.0
    q, _, _ = o.conv_qkv(p, conv, rows, 0, 0)
    want = o.bf16_round(float(np.float32(-30.0) / (np.float32(1.0) + np.exp(np.float32(30.0)))))
    assert q[0] == np.float32(want)
    assert -1e-11 < q[0] < 0.0
    rows2 = o.Rows(1, 2, 3)
    w1 = o.conv_shift(conv, rows2, 1)
    assert np.array_equal(w1[:c], conv[c:2 * c])
    assert np.array_equal(w1[c:2 * c], conv[2 * c:])
    assert np.array_equal(w1[2 * c:], rows2.qkv[:c])
    w2 = o.conv_shift(conv, rows2, 2)
    assert np.array_equal(w2[:c], conv[2 * c:])
    assert np.array_equal(w2[c:], rows2.qkv)
    assert np.array_equal(o.conv_shift(conv, rows2, 0), conv)


# tests/cpu_reference.rs:102-121
def test_warp_sum_is_the_butterfly(oracle):
    o = oracle
    lanes = np.zeros(32, np.float32)
    lanes[0], lanes[16], lanes[1] = 1e8, -1e8, 1.0
    seq = np.float32(0.0)
    for x in lanes:
        seq = np.float32(seq + x)
    assert seq == 0.0
    assert o.warp_sum(lanes) == 1.0
    lanes = np.zeros(32, np.float32)
    lanes[0], lanes[1], lanes[17] = 1.0, 1e8, -1e8
    assert o.warp_sum(lanes) == 1.0
    assert o.warp_sum(np.arange(32, dtype=np.float32)) == 496.0


# tests/cpu_reference.rs:123-145
def test_l2norm_and_gated_norm_hand_values(oracle):
    o = oracle
    x = np.zeros(DK, np.float32)
    x[5], x[9] = 3.0, 4.0
    y = o.l2norm(x)
    n = np.sqrt(np.float32(25.0) + np.float32(1e-6))
    inv = np.float32(1.0) / n
    assert y[5] == np.float32(3.0) * inv and y[9] == np.float32(4.0) * inv
    yq = o.l2norm(x, o.q_scale())
    assert yq[5] == y[5] * (np.float32(1.0) / np.sqrt(np.float32(128.0)))
    yl = o.literal_l2norm(x)
    assert abs(yl[9] - y[9]) <= np.finfo(np.float32).eps * y[9]
    yc = np.full(DV, 0.5, np.float32)
    w = np.full(DV, 2.0, np.float32)
    gate = np.zeros(DV, np.float32)
    out = o.gated_rmsnorm(yc, w, gate, 1e-5)
    want = o.bf16_round(float(np.float32(2.0) * (np.float32(0.5) * (np.float32(1.0) / np.sqrt(np.float32(0.25) + np.float32(1e-5)))) * np.float32(0.5)))
    assert (out == np.float32(want)).all()
    assert abs(want - 1.0) < 1e-2


# tests/cpu_reference.rs:147-171
def test_delta_rule_writes_the_value_under_its_key(oracle):
    o = oracle
    rng = o.Rng(9)
    s0 = rng.fill(DV * DK, -0.5, 0.5)
    k = np.zeros(DK, np.float32)
    k[3] = 1.0
    g = np.ones(DK, np.float32)
    v = rng.fill(DV, -2.0, 2.0)
    s = o.update(s0, k, g, v, 1.0)
    read = o.read_out(s, k)
    assert np.all(np.abs(read - v) <= 4.0 * np.finfo(np.float32).eps * 2.5)
    keep = np.ones(DK, bool)
    keep[3] = False
    assert np.array_equal(s.reshape(DV, DK)[:, keep], s0.reshape(DV, DK)[:, keep])


# tests/cpu_reference.rs:173-207
def test_gates_saturated(oracle):
    o = oracle
    heads = 2
    p = o.Layer(heads, 4)
    p.a_log[:] = 0.0
    p.dt_bias[:] = 0.0
    conv = o.conv_window(heads, 4)
    s0 = o.state(heads, 4, 0.5)
    rows = o.Rows(heads, 20, 4)
    rows.a[:] = 1e4
    rows.b[:] = -200.0
    r = o.chain(p, conv, s0, rows)
    assert (r.beta == 0.0).all()
    e5 = np.float32(o.decay(1e4, 0.0, 1.0, -5.0))
    assert (r.g == e5).all()
    expect = s0.copy()
    for _ in range(20):
        expect = expect * e5
    assert np.array_equal(r.state, expect)  # as values: +0 == -0
    assert np.abs(r.state).max() < 1e-40
    rows.a[:] = -1e4
    r = o.chain(p, conv, s0, rows)
    assert (r.g == 1.0).all()
    assert np.array_equal(r.state, s0)


# tests/cpu_reference.rs:209-232
def test_replay_of_a_prefix_equals_the_shorter_chain_bitwise(oracle):
    o = oracle
    heads = 4
    p = o.Layer(heads, 11)
    conv = o.conv_window(heads, 11)
    s0 = o.state(heads, 11, 0.5)
    rows = o.Rows(heads, 8, 11)
    full = o.chain(p, conv, s0, rows)
    assert np.array_equal(bits(o.replay(s0, full, 8)), bits(full.state))
    for keep in range(9):
        short = o.chain(p, conv, s0, rows.slice(0, keep))
        assert np.array_equal(bits(o.replay(s0, full, keep)), bits(short.state)), keep
        n = keep * heads * DV
        assert np.array_equal(bits(full.out[:n]), bits(short.out)), keep


# tests/cpu_reference.rs:234-257
def test_serial_steps_equal_one_window_bitwise(oracle):
    o = oracle
    heads = 3
    p = o.Layer(heads, 12)
    conv0 = o.conv_window(heads, 12)
    s0 = o.state(heads, 12, 0.5)
    rows = o.Rows(heads, 8, 12)
    window = o.chain(p, conv0, s0, rows)
    conv, s = conv0.copy(), s0.copy()
    n = heads * DV
    for r in range(8):
        row = rows.slice(r, 1)
        step = o.chain(p, conv, s, row)
        assert np.array_equal(bits(step.out), bits(window.out[r * n:(r + 1) * n])), r
        conv = o.conv_shift(conv, row, 1)
        s = step.state
    assert np.array_equal(bits(s), bits(window.state))
    assert np.array_equal(conv, o.conv_shift(conv0, rows, 8))


# The same two identities for bf16-stored states (src/cpu.rs:390-402, 479-484).
def test_bf16_state_window_equals_serial_steps_and_replay(oracle):
    o = oracle
    heads = 2
    p = o.Layer(heads, 21)
    conv0 = o.conv_window(heads, 21)
    s0 = o.bf16_round_np(o.state(heads, 21, 0.5))
    rows = o.Rows(heads, 6, 21)
    window = o.chain(p, conv0, s0, rows, bf16_state=True)
    conv, s = conv0.copy(), s0.copy()
    for r in range(6):
        row = rows.slice(r, 1)
        step = o.chain(p, conv, s, row, bf16_state=True)
        conv = o.conv_shift(conv, row, 1)
        s = step.state
        assert np.array_equal(bits(o.replay(s0, window, r + 1, bf16_state=True)), bits(s)), r
    assert np.array_equal(bits(s), bits(window.state))
    assert np.array_equal(bits(window.state), bits(o.bf16_round_np(window.state)))


# tests/cpu_reference.rs:259-285
def test_kernel_order_agrees_with_the_literal_formulation(oracle):
    o = oracle
    heads = 4
    p = o.Layer(heads, 13)
    conv = o.conv_window(heads, 13)
    s0 = o.state(heads, 13, 0.5)
    rows = o.Rows(heads, 8, 13)
    a = o.chain(p, conv, s0, rows)
    b = o.chain(p, conv, s0, rows, literal=True)
    assert np.array_equal(bits(a.v), bits(b.v))
    assert np.array_equal(bits(a.beta), bits(b.beta))
    assert rel_err(a.state, b.state) < 1e-5
    assert rel_err(a.k, b.k) < 1e-6 and rel_err(a.g, b.g) < 1e-6
    ulp_y, n_y = bf16_diff(o, a.y, b.y)
    ulp_o, n_o = bf16_diff(o, a.out, b.out)
    assert ulp_y <= 1 and ulp_o <= 1
    assert n_y * 100 <= a.y.size and n_o * 100 <= a.out.size


# tests/cpu_reference.rs:287-319
def test_conv_roundings_differ_slightly(oracle):
    o = oracle
    heads = 2
    p = o.Layer(heads, 14)
    conv = o.conv_window(heads, 14)
    rows = o.Rows(heads, 4, 14)
    differ = total = 0
    for r in range(4):
        for h in range(heads):
            a = np.concatenate(o.conv_qkv(p, conv, rows, r, h, o.FUSED))
            b = np.concatenate(o.conv_qkv(p, conv, rows, r, h, o.UNFUSED))
            assert np.all(np.abs(a - b) <= np.maximum(np.maximum(np.abs(a), np.abs(b)), 1.0) / 64.0)
            differ += bf16_diff(o, a, b)[1]
            total += 3 * DK
    assert 0 < differ and differ * 2 < total


# tests/cpu_reference.rs:321-328
def test_state_layout_transpose(oracle):
    o = oracle
    s = o.state(2, 15, 1.0)
    t = o.transpose_state(s)
    assert t[DV + 3] == s[3 * DK + 1]
    assert t[DK * DV + 7 * DV + 2] == s[DK * DV + 2 * DK + 7]
    assert np.array_equal(o.transpose_state(t), s)


def core_inputs(o, heads, t, seed):
    """tests/cpu_reference.rs:333-345."""
    rng = o.Rng(seed)
    q = rng.fill_bf16(t * heads * DK, -1.0, 1.0)
    k = rng.fill_bf16(t * heads * DK, -1.0, 1.0)
    v = rng.fill_bf16(t * heads * DV, -1.0, 1.0)
    g = np.array([o.log_decay(rng.uniform(-4.0, 4.0), 0.0, 0.0, -5.0) for _ in range(t * heads * DK)], np.float32)
    beta = np.array([o.beta(rng.uniform(-4.0, 4.0)) for _ in range(t * heads)], np.float32)
    return q, k, v, g, beta


# tests/cpu_reference.rs:347-384
def test_chunked_form_matches_the_recurrence(oracle):
    o = oracle
    heads = 2
    for t, chunk in ((1, 64), (7, 64), (64, 64), (65, 64), (150, 64), (40, 16)):
        q, k, v, g, beta = core_inputs(o, heads, t, 16 + t)
        s0 = o.state(heads, t, 0.5)
        s_rec = s0.copy().reshape(heads, DK * DV)
        y_rec = np.zeros(t * heads * DV, np.float32)
        for r in range(t):
            for h in range(heads):
                i = r * heads + h
                s_rec[h], y = o.literal_step(s_rec[h], q[i * DK:(i + 1) * DK], k[i * DK:(i + 1) * DK],
                                             v[i * DV:(i + 1) * DV], g[i * DK:(i + 1) * DK], float(beta[i]))
                y_rec[i * DV:(i + 1) * DV] = y
        y_chunk, s_chunk = o.chunked_layer(heads, q, k, v, g, beta, s0, chunk)
        e_y, e_s = rel_err(y_chunk, y_rec), rel_err(s_chunk, s_rec.reshape(-1))
        assert e_y < 2e-5 and e_s < 2e-5, (t, chunk, e_y, e_s)


# tests/cpu_reference.rs:386-393
def test_rows_slice(oracle):
    o = oracle
    rows = o.Rows(2, 5, 17)
    s = rows.slice(1, 3)
    assert s.rows == 3
    assert np.array_equal(s.b, rows.b[2:8])
    assert np.array_equal(s.slice(2, 1).gate, rows.slice(3, 1).gate)


# tests/cpu_reference.rs:398-450
def test_prefill_form_matches_the_chain(oracle):
    o = oracle
    heads = 2
    for t, gates in ((1, "random"), (5, "random"), (16, "random"), (17, "random"), (40, "random"), (100, "random"),
                     (48, "strongest"), (48, "mixed")):
        p = o.Layer(heads, 60 + t)
        conv = o.conv_window(heads, 60 + t)
        s0 = o.state(heads, 60 + t, 0.5)
        rows = o.Rows(heads, t, 60 + t)
        if gates == "strongest":
            rows.a[:] = 1e4
        elif gates == "mixed":
            idx = np.arange(rows.a.size) // (heads * DK)
            rows.a[:] = np.where(idx % 3 == 0, -1e4, 1e4).astype(np.float32)
        c = o.chain(p, conv, s0, rows)
        f = o.prefill(p, conv, s0, rows)
        assert rel_err(f.state, c.state) < 1e-5, (t, gates)
        assert rel_err(f.y, c.y) < 1.0 / 256.0 and rel_err(f.out, c.out) < 1.0 / 256.0, (t, gates)
        assert bf16_diff(o, f.out, c.out)[1] * 1000 <= c.out.size, (t, gates)
        assert np.isfinite(f.state).all()


# The benchmark configurations' contract: the threaded driver equals the per-head pieces it is made of.
def test_core_forward_equals_its_pieces(oracle):
    o = oracle
    heads, t = 3, 70
    q, k, v, g, beta = core_inputs(o, heads, t, 99)
    qb, kb, vb = o.bf16_bits(q), o.bf16_bits(k), o.bf16_bits(v)
    s0 = o.state(heads, 99, 0.05)
    y_rec, s_rec = o.core_forward(heads, qb, kb, vb, g, beta, s0, form="recurrent", threads=2)
    y_chk, s_chk = o.core_forward(heads, qb, kb, vb, g, beta, s0, form="chunked", chunk=64, threads=3)
    assert rel_err(y_chk, y_rec) < 2e-5 and rel_err(s_chk, s_rec) < 2e-5
    # Head 1 by hand, literal layout, no normalisation.
    s = o.transpose_state(s0)[DK * DV:2 * DK * DV]
    for r in range(t):
        i = r * heads + 1
        s, y = o.literal_step(s, q[i * DK:(i + 1) * DK], k[i * DK:(i + 1) * DK], v[i * DV:(i + 1) * DV],
                              g[i * DK:(i + 1) * DK], float(beta[i]), normalize=False)
        assert np.array_equal(bits(y), bits(y_rec[i * DV:(i + 1) * DV]))
    assert np.array_equal(bits(o.transpose_state(s)), bits(s_rec[DK * DV:2 * DK * DV]))
