"""GPU parity of the recurrent entry points (chain, replay, conv shift) through the C ABI.

The structure follows the reference crate's GPU tests (crates/glm53f-kda/tests/gpu.rs, gpu_bf16_state.rs): the
kernels against the CPU oracle with the reference's stated bounds, the bitwise identities (CPU replay of the
kernel's saves, replayed prefix == shorter chain, serial steps == one window, batch == single), awkward layouts,
and the launchers' rejections.  When the reference's own kernels were compiled (oracle/_ref), every output is
also compared with theirs bit for bit.
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


def case(o, heads, rows, seed, scale=0.5):
    return o.Layer(heads, seed), o.conv_window(heads, seed), o.state(heads, seed, scale), o.Rows(heads, rows, seed)


# gpu.rs:312-368
@pytest.mark.parametrize("r", [1, 2, 3, 5, 8])
def test_chain_matches_the_cpu_oracle(G, oracle, r):
    o = oracle
    h = 64
    p, conv, s0, rows = case(o, h, r, 300 + r)
    g = G.run_chain(G.product(), p, conv, s0, rows)
    assert g.rc == 0
    G.check_status()
    # Bitwise: the recurrence given the kernel's own replay inputs (no transcendental in the update).
    assert np.array_equal(G.bits(o.replay(s0, g, r)), G.bits(g.state))
    c = o.chain(p, conv, s0, rows)
    eg = float(np.max(np.abs(g.g - c.g) / np.abs(c.g)))
    uv, nv = G.ulps(g.v, c.v)
    ub, nb = G.ulps(g.beta, c.beta)
    ek = G.max_abs(g.k, c.k)
    es = G.max_abs(g.state, c.state) / G.max_abs(c.state)
    uo, no = G.ulps(g.out, c.out)
    eo = G.max_abs(g.out, c.out) / G.max_abs(c.out)
    assert eg <= 4e-6
    assert uv <= 1 and ub <= 1
    assert nv * 1000 <= c.v.size and nb * 100 <= max(c.beta.size, 100)
    assert ek <= 1.0 / 256.0
    assert es <= 1e-3
    assert eo <= 1.0 / 256.0 and no * 1000 <= c.out.size
    # Nothing written past the rows (the canaries survive).
    assert (g.out_raw[r * h * DV:] == 0xFFFF).all()


def same_as_reference_kernels(G, a, b, fields):
    for f in fields:
        assert np.array_equal(G.bits(getattr(a, f)), G.bits(getattr(b, f))), f


@pytest.mark.parametrize("heads,r,bf16", [(64, 1, False), (64, 8, False), (3, 5, False), (64, 1, True), (64, 8, True), (5, 16, True)])
def test_chain_equals_the_reference_kernels_bitwise(G, oracle, heads, r, bf16):
    ref = G.reference_kernels()
    if ref is None:
        pytest.skip("reference kernels not built (make -C oracle ref)")
    o = oracle
    p, conv, s0, rows = case(o, heads, r, 700 + r + heads)
    if bf16:
        s0 = o.bf16_round_np(s0)
    mine = G.run_chain(G.product(), p, conv, s0, rows, bf16_state=bf16)
    theirs = G.run_chain(ref, p, conv, s0, rows, bf16_state=bf16)
    assert mine.rc == 0 and theirs.rc == 0
    same_as_reference_kernels(G, mine, theirs, ["out", "state", "k", "v", "g", "beta"])
    for keep in range(r + 1):
        a = G.run_replay(G.product(), heads, s0, mine, keep, bf16_state=bf16)
        b = G.run_replay(ref, heads, s0, theirs, keep, bf16_state=bf16)
        assert np.array_equal(G.bits(a), G.bits(b)), keep
    G.check_status()


@pytest.mark.parametrize("bf16", [False, True])
def test_both_replay_kernels_leave_the_same_bits(G, oracle, bf16):
    """Saves that are 16-byte aligned replay on independent warps, others on the persistent kernel: one result."""
    o, lib, h, r = oracle, G.product(), 3, 7
    p, conv, s0, rows = case(o, h, r, 333)
    if bf16:
        s0 = o.bf16_round_np(s0)
    sv = G.run_chain(lib, p, conv, s0, rows, bf16_state=bf16)
    n = r * h * DK
    k_pad, g_pad = torch.zeros(n + 4, device="cuda"), torch.zeros(n + 4, device="cuda")
    k_pad[1:n + 1] = torch.from_numpy(sv.k).cuda()   # one float in: the rows start 4 bytes off a 16-byte boundary
    g_pad[1:n + 1] = torch.from_numpy(sv.g).cuda()
    d_v, d_b = G.dev_bf16(sv.v), G.dev_f32(sv.beta)
    cu, zoff = G.dev_i32([0, r]), G.dev_i64([0])
    for keep in (0, 1, 4, r):
        want = G.run_replay(lib, h, s0, sv, keep, bf16_state=bf16)
        d_sin = G.dev_bf16(s0) if bf16 else G.dev_f32(s0)
        d_sout = torch.zeros_like(d_sin)
        kp = G.dev_i32([keep])
        fn = lib.glm53f_kda_replay_batch_bf16state if bf16 else lib.glm53f_kda_replay_batch
        rc = fn(h, 1, 1, G.ptr(cu), G.ptr(kp), G.ptr(d_sin), G.ptr(d_sout), 0, G.ptr(zoff), C.c_void_p(k_pad.data_ptr() + 4), G.ptr(d_v),
                C.c_void_p(g_pad.data_ptr() + 4), G.ptr(d_b), 0, 0, None)
        assert rc == 0
        got = G.host_bf16(d_sout) if bf16 else G.host_f32(d_sout)
        assert np.array_equal(G.bits(got), G.bits(want)), keep
    G.check_status()


# gpu.rs:398-474, gpu_bf16_state.rs:331-382
@pytest.mark.parametrize("bf16", [False, True])
def test_prefixes_and_serial_steps_are_bitwise(G, oracle, bf16):
    o = oracle
    h, r = 4, 8
    p, conv0, s0, rows = case(o, h, r, 41)
    if bf16:
        s0 = o.bf16_round_np(s0)
    lib = G.product()
    w = G.Weights(p)
    window = G.run_chain(lib, p, conv0, s0, rows, bf16_state=bf16, w=w)
    # verify without a state write gives the same outputs and saves
    dry = G.run_chain(lib, p, conv0, s0, rows, bf16_state=bf16, write_state=False, w=w)
    same_as_reference_kernels(G, window, dry, ["out", "k", "v", "g", "beta"])
    assert not dry.state.any()
    assert np.array_equal(G.bits(dry.state_in_after), G.bits(s0))
    conv, s = conv0.copy(), s0.copy()
    n = h * DV
    for i in range(r):
        row = rows.slice(i, 1)
        step = G.run_chain(lib, p, conv, s, row, bf16_state=bf16, w=w)
        assert np.array_equal(G.bits(step.out), G.bits(window.out[i * n:(i + 1) * n])), i
        conv = o.conv_shift(conv, row, 1)
        s = step.state
        assert np.array_equal(G.bits(G.run_replay(lib, h, s0, window, i + 1, bf16_state=bf16)), G.bits(s)), i
        # the oracle's replay is a bit-level model of the device's
        assert np.array_equal(G.bits(o.replay(s0, window, i + 1, bf16_state=bf16)), G.bits(s)), i
    assert np.array_equal(G.bits(s), G.bits(window.state))
    assert np.array_equal(G.bits(G.run_replay(lib, h, s0, window, 0, bf16_state=bf16)), G.bits(s0))
    G.check_status()


# gpu.rs:479-549
def test_padded_strides_negative_b_off_in_place_and_unaligned(G, oracle):
    o = oracle
    h, r = 3, 4
    p, conv, s0, rows = case(o, h, r, 52)
    lib = G.product()
    base = G.run_chain(lib, p, conv, s0, rows)
    c = 3 * h * DK
    # wide rows, logits before the row, padded output rows, in place
    alt = G.run_chain(lib, p, conv, s0, rows, p_stride=c + 40, b_off=-24, out_stride=h * DV + 24, in_place=True, pad_front=64)
    for f in ("out", "state", "k", "v", "g", "beta"):
        assert np.array_equal(G.bits(getattr(base, f)), G.bits(getattr(alt, f))), f
    gaps = np.concatenate([alt.out_raw[i * (h * DV + 24) + h * DV:(i + 1) * (h * DV + 24)] for i in range(r)])
    assert (gaps == 0xFFFF).all()
    # rows that start on an odd element: the bulk-copy path cannot be used, the element-wise one must agree
    odd = G.run_chain(lib, p, conv, s0, rows, p_stride=c + h + 1, pad_front=3)
    for f in ("out", "state", "k", "v", "g", "beta"):
        assert np.array_equal(G.bits(getattr(base, f)), G.bits(getattr(odd, f))), f
    G.check_status()


def batch_case(G, o, heads, lens, seed, bf16):
    reqs = [case(o, heads, n, seed + 7 * i) for i, n in enumerate(lens)]
    p = reqs[0][0]
    return p, reqs


# gpu.rs:554-724, gpu_bf16_state.rs:423-587
@pytest.mark.parametrize("bf16", [False, True])
def test_batch_equals_single_requests(G, oracle, bf16):
    o = oracle
    lib = G.product()
    h = 5
    lens = [3, 0, 1, 6]
    p, reqs = batch_case(G, o, h, lens, 61, bf16)
    w = G.Weights(p)
    c = 3 * h * DK
    total = sum(lens)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    qkv = np.concatenate([r[3].qkv for r in reqs])
    a = np.concatenate([r[3].a for r in reqs])
    b = np.concatenate([r[3].b for r in reqs])
    gate = np.concatenate([r[3].gate for r in reqs])
    allrows = o.Rows(h, total)
    allrows.qkv, allrows.a, allrows.b, allrows.gate = qkv, a, b, gate
    pbuf, base, p_stride, b_off = G.pack_rows(allrows)
    states = [o.bf16_round_np(r[2]) if bf16 else r[2] for r in reqs]
    convs = [r[1] for r in reqs]
    # scattered slots: request i lives in slot order[i]
    order = [2, 0, 3, 1]
    slen, clen = h * DV * DK, 3 * c
    pool = np.zeros(4 * slen, np.float32)
    cpool = np.zeros(4 * clen, np.float32)
    for i, sl in enumerate(order):
        pool[sl * slen:(sl + 1) * slen] = states[i]
        cpool[sl * clen:(sl + 1) * clen] = convs[i]
    d_p, d_a, d_g = G.dev_bf16(pbuf), G.dev_bf16(a), G.dev_bf16(gate)
    d_conv = G.dev_bf16(cpool)
    d_pool = G.dev_bf16(pool) if bf16 else G.dev_f32(pool)
    d_out = torch.full((total * h * DV,), -1, dtype=torch.int16, device="cuda")
    d_k = torch.zeros(total * h * DK, dtype=torch.float32, device="cuda")
    d_v = torch.zeros(total * h * DV, dtype=torch.int16, device="cuda")
    d_gs = torch.zeros_like(d_k)
    d_b = torch.zeros(total * h, dtype=torch.float32, device="cuda")
    d_cu = G.dev_i32(cu)
    d_soff = G.dev_i64([sl * slen for sl in order])
    d_coff = G.dev_i64([sl * clen for sl in order])
    fn = lib.glm53f_kda_chain_batch_bf16state if bf16 else lib.glm53f_kda_chain_batch
    rc = fn(h, 4, G.ptr(d_cu), C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, b_off, G.ptr(d_a), h * DK, G.ptr(d_g), h * DV,
            G.ptr(d_conv), G.ptr(d_coff), G.ptr(w.conv_w), G.ptr(d_pool), G.ptr(d_pool), G.ptr(d_soff), G.ptr(w.a_log),
            G.ptr(w.dt_bias), G.ptr(w.norm_w), w.eps, w.lower, G.ptr(d_out), h * DV, G.ptr(d_k), G.ptr(d_v), G.ptr(d_gs),
            G.ptr(d_b), None)
    assert rc == 0
    G.check_status()
    out = G.host_bf16(d_out)
    pool_after = G.host_bf16(d_pool) if bf16 else G.host_f32(d_pool)
    ks = G.host_f32(d_k)
    for i, n in enumerate(lens):
        sl = order[i]
        if n == 0:
            assert np.array_equal(G.bits(pool_after[sl * slen:(sl + 1) * slen]), G.bits(states[i]))
            continue
        single = G.run_chain(lib, p, convs[i], states[i], reqs[i][3], bf16_state=bf16, w=w)
        r0 = cu[i]
        assert np.array_equal(G.bits(out[r0 * h * DV:(r0 + n) * h * DV]), G.bits(single.out)), i
        assert np.array_equal(G.bits(pool_after[sl * slen:(sl + 1) * slen]), G.bits(single.state)), i
        assert np.array_equal(G.bits(ks[r0 * h * DK:(r0 + n) * h * DK]), G.bits(single.k)), i
    # The commit: every request keeps a prefix; layers = 1.
    keeps = [2, 0, 1, 0]
    d_pool2 = G.dev_bf16(pool) if bf16 else G.dev_f32(pool)
    d_keep = G.dev_i32(keeps)
    fn = lib.glm53f_kda_replay_batch_bf16state if bf16 else lib.glm53f_kda_replay_batch
    rc = fn(h, 1, 4, G.ptr(d_cu), G.ptr(d_keep), G.ptr(d_pool2), G.ptr(d_pool2), 0, G.ptr(d_soff), G.ptr(d_k), G.ptr(d_v),
            G.ptr(d_gs), G.ptr(d_b), 0, 0, None)
    assert rc == 0
    G.check_status()
    after = G.host_bf16(d_pool2) if bf16 else G.host_f32(d_pool2)
    for i, n in enumerate(lens):
        sl = order[i]
        if keeps[i] == 0:
            want = states[i]
        else:
            want = G.run_chain(lib, p, convs[i], states[i], reqs[i][3].slice(0, keeps[i]), bf16_state=bf16, w=w).state
        assert np.array_equal(G.bits(after[sl * slen:(sl + 1) * slen]), G.bits(want)), i


def test_conv_shift(G, oracle):
    o = oracle
    lib = G.product()
    h = 2
    c = 3 * h * DK
    for r, keep in ((1, 1), (2, 1), (2, 2), (5, 0), (5, 3), (8, 8)):
        conv = o.conv_window(h, 70 + r)
        rows = o.Rows(h, r, 70 + r)
        pbuf, base, p_stride, b_off = G.pack_rows(rows)
        d_conv, d_p = G.dev_bf16(conv), G.dev_bf16(pbuf)
        rc = lib.glm53f_kda_conv_shift(c, keep, G.ptr(d_conv), C.c_void_p(d_p.data_ptr() + 2 * base), p_stride, None)
        assert rc == 0
        assert np.array_equal(G.host_bf16(d_conv), o.conv_shift(conv, rows, keep)), (r, keep)
    # batch form: 3 layers x 2 requests, device metadata, an odd channel count on the scalar path
    layers, lens, keeps = 3, [4, 2], [3, 0]
    for ch in (c, 100):
        total = sum(lens)
        rng = o.Rng(5 + ch)
        win = rng.fill_bf16(layers * 2 * 3 * ch, -2, 2)
        prow = rng.fill_bf16(layers * total * (ch + 8), -2, 2)
        d_win, d_prow = G.dev_bf16(win), G.dev_bf16(prow)
        cu, d_keep, d_off = G.dev_i32([0, 4, 6]), G.dev_i32(keeps), G.dev_i64([3 * ch, 0])  # held until the sync
        rc = lib.glm53f_kda_conv_shift_batch(ch, layers, 2, G.ptr(cu), G.ptr(d_keep), G.ptr(d_win), 2 * 3 * ch,
                                             G.ptr(d_off), G.ptr(d_prow), total * (ch + 8), ch + 8, None)
        assert rc == 0
        got = G.host_bf16(d_win)
        for l in range(layers):
            for b in range(2):
                off = l * 2 * 3 * ch + (3 * ch if b == 0 else 0)
                old = win[off:off + 3 * ch].reshape(3, ch)
                r0 = [0, 4][b]
                new = prow[l * total * (ch + 8):(l + 1) * total * (ch + 8)].reshape(total, ch + 8)[r0:r0 + lens[b], :ch]
                stack = np.concatenate([old, new])
                assert np.array_equal(got[off:off + 3 * ch].reshape(3, ch), stack[keeps[b]:keeps[b] + 3]), (ch, l, b)


# gpu.rs:728-792
def test_rejections(G, oracle):
    o = oracle
    lib = G.product()
    h = 2
    p, conv, s0, rows = case(o, h, 2, 81)
    ok = G.run_chain(lib, p, conv, s0, rows)
    assert ok.rc == 0
    w = G.Weights(p)
    x = G.dev_bf16(np.zeros(4096, np.float32))
    f = G.dev_f32(np.zeros(h * DV * DK, np.float32))
    P = G.ptr

    def chain(heads=h, nrows=1, pp=x, state=f, out=x, ks=None, vs=None):
        return lib.glm53f_kda_chain(heads, nrows, P(pp), 3 * h * DK + h, 3 * h * DK, P(x), h * DK, P(x), h * DV, P(x),
                                    P(w.conv_w), P(state), None, P(w.a_log), P(w.dt_bias), P(w.norm_w), 1e-5, -5.0, P(out),
                                    h * DV, P(ks), P(vs), None, None, None)

    assert chain(heads=0) == 1
    assert chain(heads=70000) == 1
    assert chain(nrows=0) == 1
    assert chain(pp=None) == 1
    assert chain(state=None) == 1
    assert chain(out=None) == 1
    assert chain(ks=f) == 1  # saves must be all or none
    assert lib.glm53f_kda_replay(h, -1, P(f), P(f), P(f), P(x), P(f), P(f), None) == 1
    assert lib.glm53f_kda_replay(h, 1, P(f), None, P(f), P(x), P(f), P(f), None) == 1
    assert lib.glm53f_kda_replay_batch(h, 1, 1, None, None, P(f), P(f), 0, None, P(f), P(x), P(f), P(f), 0, 0, None) == 1
    assert lib.glm53f_kda_conv_shift(0, 1, P(x), P(x), 8, None) == 1
    assert lib.glm53f_kda_conv_shift(8, -1, P(x), P(x), 8, None) == 1
    assert lib.glm53f_kda_conv_shift_batch(8, 1, 1, None, None, P(x), 0, None, P(x), 0, 8, None) == 1
    torch.cuda.synchronize()
    assert lib.glm53f_kda_device_status() == 0
