"""The verify / commit orchestration over pool slots (glm53f-afd_b200/verify.py, the KDA half of the reference's
Forward::verify and Forward::commit, crates/glm53f-forward/src/forward.rs:1905-2040) on the GPU.

The property is the reference's (crates/glm53f-forward/tests/verify.rs: a verify of n rows committed at k equals k
single steps): states, conv windows and the kept rows' outputs of verify + commit(keep) are the bits of decoding the
kept rows one at a time, over several layers and slots, f32 and bf16 states."""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

H, DK = 64, 128


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    m = {n: importlib.import_module("glm53f-afd_b200." + n) for n in ("kernel", "marks", "verify", "core")}
    importlib.import_module("glm53f-afd_b200").ffi.load()
    return m


def rows_on_device(K, rows):
    h, r = rows.heads, rows.rows
    c = K.channels(h)
    p = np.zeros((r, c + h), np.float32)
    p[:, :c] = rows.qkv.reshape(r, c)
    p[:, c:] = rows.b.reshape(r, h)
    return (K._bf16_encode(p.reshape(-1)), K.RowView.dense(K.DeviceBuffer.from_slice(K._bf16_encode(rows.a)), h * DK),
            K.RowView.dense(K.DeviceBuffer.from_slice(K._bf16_encode(rows.gate)), h * DK))


@pytest.mark.parametrize("bf16,recompute", [(True, False), (False, False), (True, True), (False, True)])
def test_verify_then_commit_equals_serial_decode(mods, oracle, bf16, recompute):
    K, marks, verify = mods["kernel"], mods["marks"], mods["verify"]
    o, layers = oracle, 2
    windows, keep = [5, 8, 1], [3, 8, 1]
    total = sum(windows)
    l = marks.KvLayout.new(layers, 0).with_kda_state_bf16(bf16)
    pools = [marks.KvPool(marks.KvConfig(l, 4, 4)) for _ in range(2)]  # [0]: verify + commit, [1]: serial steps
    params = [o.Layer(H, 300 + j) for j in range(layers)]
    weights = [K.Weights.upload(K.LayerParams(H, p.conv_w, p.a_log, p.dt_bias, p.norm_w, p.eps, p.lower)) for p in params]
    kvs = []
    for pool in pools:
        pool.slot()  # slot 0 stays idle: the round's slots do not start at offset 0
        mine = [pool.slot() for _ in windows]
        g = torch.Generator(device="cuda").manual_seed(9)
        st = (torch.randn(pool.state.t.numel() // l.kda_state_elem_bytes(), device="cuda", generator=g) * 0.3)
        pool.state.t.copy_((st.to(torch.bfloat16) if bf16 else st).view(torch.uint8))
        pool.conv.t.copy_((torch.randn(pool.conv.t.numel() // 2, device="cuda", generator=g) * 0.5).to(torch.bfloat16).view(torch.uint8))
        for kv in mine:
            kv.advance(40)
        kvs.append(mine)
    rows = [o.Rows(H, total, 310 + j) for j in range(layers)]
    dev = [rows_on_device(K, r) for r in rows]

    # ---- pool 0: one verify round over all layers, then the commit
    kv0 = kvs[0]
    vf = verify.KdaVerify(pools[0], weights, 16, 4, recompute=recompute)
    assert vf.v.bytes() == (2 * 16 * (24_640 * 2 + 8192 * 2) + 16 * 8192 * 2 if recompute else 2 * 16 * (24_640 * 2 + 64 * 1_284))
    with pytest.raises(verify.Invalid, match="commit without a verify"):
        vf.commit(kv0, keep)
    with pytest.raises(verify.Invalid, match="1..=8 rows"):
        vf.verify([(kv0[0], 9)])
    with pytest.raises(verify.Invalid, match="no verify is open"):
        vf.layer(0, dev[0][1], dev[0][2], K.RowView.dense(K.DeviceBuffer.zeroed(total * H * DK * 2), H * DK))
    vf.verify(list(zip(kv0, windows)))
    assert [kv.pending for kv in kv0] == windows
    with pytest.raises(verify.Invalid, match="pending"):
        vf.verify(list(zip(kv0, windows)))
    outs = []
    before = pools[0].state.t.clone()
    for j in range(layers):
        vf.v.p.upload_at(j * vf.v.rows * verify.KDA_P_COLS, dev[j][0])
        out = K.RowView.dense(K.DeviceBuffer.zeroed(total * H * DK * 2), H * DK)
        a_rows = dev[j][1]
        if recompute:  # the decay-gate rows are kept in the scratch for the commit
            vf.v.a.upload_at(j * vf.v.rows * H * DK, dev[j][1].buf.download(np.uint16, total * H * DK))
            a_rows = vf.v.a_rows(j)
            with pytest.raises(verify.Invalid, match="decay-gate rows live in scratch"):
                vf.layer(j, dev[j][1], dev[j][2], out)
        vf.layer(j, a_rows, dev[j][2], out)
        outs.append(out)
    pools[0].stream.synchronize()
    assert torch.equal(pools[0].state.t, before)  # a verify reads the states, it does not write them
    with pytest.raises(verify.Invalid, match="commit of 2 slots after a verify of 3"):
        vf.commit(kv0[:2], keep[:2])
    with pytest.raises(verify.Invalid, match="does not match the pending verify"):
        vf.commit(kv0, [3, 9, 1])
    vf.pending = [verify._Req(kv.slot, kv.tokens(), r) for kv, r in zip(kv0, windows)]  # the failed commit consumed the round: reopen it
    vf.commit(kv0, keep)
    pools[0].stream.synchronize()
    assert [kv.tokens() for kv in kv0] == [40 + k for k in keep] and all(kv.pending == 0 for kv in kv0)
    assert mods["core"].device_status() == 0

    # ---- pool 1: the kept rows one at a time, in place
    kv1 = kvs[1]
    row0 = np.concatenate([[0], np.cumsum(windows)])
    sn = l.state_elems_per_layer() * l.kda_state_elem_bytes()
    cn = l.conv_elems_per_layer() * 2
    c = K.channels(H)
    serial_out = {}
    stream = pools[1].stream
    for j in range(layers):
        state_j, conv_j = K.DeviceBuffer(pools[1].state.t[j * sn:]), K.DeviceBuffer(pools[1].conv.t[j * cn:])
        p_buf = K.DeviceBuffer.from_slice(dev[j][0])
        for i, kv in enumerate(kv1):
            for t in range(keep[i]):
                r = int(row0[i]) + t
                meta = K.BatchMeta.new(1)
                meta.set([K.Request(1, kv.conv_elem_offset(), kv.state_elem_offset())])
                out = K.RowView.dense(K.DeviceBuffer.zeroed(H * DK * 2), H * DK)
                cb = K.ChainBatch(weights[j], K.RowView.new(p_buf, r * (c + H), c + H), c, K.RowView.new(dev[j][1].buf, r * H * DK, H * DK),
                                  K.RowView.new(dev[j][2].buf, r * H * DK, H * DK), conv_j, state_j, K.StateOut.InPlace, out, None)
                (cb.launch_bf16_state if bf16 else cb.launch)(meta, stream)
                K.conv_shift_batch(H, 1, meta, conv_j, cn // 2, K.RowView.new(p_buf, r * (c + H), c + H), 0, stream)
                serial_out[(j, r)] = out
    stream.synchronize()
    assert mods["core"].device_status() == 0
    assert torch.equal(pools[0].state.t, pools[1].state.t)
    assert torch.equal(pools[0].conv.t, pools[1].conv.t)
    for (j, r), out in serial_out.items():
        got = outs[j].buf.download(np.uint16, H * DK, r * H * DK)
        assert np.array_equal(got, out.buf.download(np.uint16, H * DK)), (j, r)
