"""Host-side checks of the checked wrappers (glm53f-afd_b200/kernel.py), without a GPU.

The wrappers mirror crates/glm53f-kda/src/kernel.rs: every rejection below is one the reference makes on the host,
before the launcher is called (kernel.rs:85-135, 245-275, 432-459, 507-526, 556-595, 716-720, 749-757, 836-861,
923-953, 980-987, 1019-1053).  Buffers live in host memory here; a check that passes would go on to launch, so only
rejections (and pure bookkeeping) are exercised.
"""
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")


@pytest.fixture()
def K(monkeypatch):
    k = importlib.import_module("glm53f-afd_b200.kernel")
    monkeypatch.setattr(k, "DEVICE", "cpu")
    return k


def weights(K, heads, lower=-5.0):
    p = K.LayerParams(heads, np.zeros(K.channels(heads) * K.TAPS, np.float32), np.zeros(heads, np.float32),
                      np.zeros(heads * K.DK, np.float32), np.ones(K.DV, np.float32), 1e-5, lower)
    return K.Weights.upload(p)


def chain_args(K, h, nrows, **over):
    rows = nrows
    c = K.channels(h)
    a = dict(weights=weights(K, h), rows=rows, p=K.RowView.dense(K.DeviceBuffer.zeroed(rows * (c + h) * 2), c + h), b_off=c,
             a=K.RowView.dense(K.DeviceBuffer.zeroed(rows * h * K.DK * 2), h * K.DK),
             g=K.RowView.dense(K.DeviceBuffer.zeroed(rows * h * K.DV * 2), h * K.DV),
             conv=K.DeviceBuffer.zeroed(K.WINDOW * c * 2), conv_offset=0, state=K.DeviceBuffer.zeroed(K.state_len(h) * 4), state_offset=0,
             state_out=K.StateOut.InPlace, out=K.RowView.dense(K.DeviceBuffer.zeroed(rows * h * K.DV * 2), h * K.DV), saves=None)
    a.update(over)
    return a


def test_weights_sizes_and_bf16_encoding(K):
    with pytest.raises(K.Invalid):
        K.Weights.upload(K.LayerParams(2, np.zeros(5, np.float32), np.zeros(2, np.float32), np.zeros(256, np.float32), np.ones(128, np.float32)))
    w = weights(K, 2)
    assert w.norm_w.download(np.uint16, 128).tolist() == [0x3F80] * 128
    assert K._bf16_encode(np.array([1.00390625, 3.0e38, np.inf], np.float32)).tolist() == [0x3F80, 0x7F62, 0x7F80]
    assert np.array_equal(K._bf16_decode(K._bf16_encode(np.array([0.5, -2.0], np.float32))), np.array([0.5, -2.0], np.float32))


def test_row_view_extents(K):
    buf = K.DeviceBuffer.zeroed(100 * 2)
    K.RowView.new(buf, 0, 10).check("x", 2, 0, 10, 0, 10)
    with pytest.raises(K.Invalid):
        K.RowView.new(buf, 0, 10).check("x", 2, 0, 11, 0, 10)
    with pytest.raises(K.Invalid):
        K.RowView.new(buf, 0, 10).check("x", 2, 0, 1, -1, 10)     # a negative column before the buffer
    K.RowView.new(buf, 5, 10).check("x", 2, 0, 1, -5, 10)          # ... but inside it when the view starts later
    K.RowView.new(buf, 0, 10).check("x", 2, 0, 0, 0, 1000)         # no rows: nothing to check


def test_chain_rejections(K):
    s = K.Stream()
    h = 2
    with pytest.raises(K.Invalid, match="at least one row"):
        K.Chain(**chain_args(K, h, 0)).launch(s)
    with pytest.raises(K.Invalid, match="p: rows reach"):
        K.Chain(**dict(chain_args(K, h, 2), rows=3)).launch(s)
    with pytest.raises(K.Invalid, match="out rows overlap"):
        a = chain_args(K, h, 2)
        a["out"] = K.RowView.new(a["out"].buf, 0, h * K.DV - 1)
        K.Chain(**a).launch(s)
    with pytest.raises(K.Invalid, match="state"):
        K.Chain(**chain_args(K, h, 1, state_offset=1)).launch(s)
    with pytest.raises(K.Invalid, match="conv"):
        K.Chain(**chain_args(K, h, 1, conv_offset=8)).launch(s)
    with pytest.raises(K.Invalid, match="partly overlaps"):
        st = K.DeviceBuffer.zeroed(2 * K.state_len(h) * 4)
        K.Chain(**chain_args(K, h, 1, state=st, state_out=K.StateOut.To(st, 16))).launch(s)
    with pytest.raises(K.Invalid, match="saves hold"):
        K.Chain(**chain_args(K, h, 2, saves=K.Saves.alloc(h, 1))).launch(s)
    with pytest.raises(K.Invalid, match="saves hold"):
        K.Chain(**chain_args(K, h, 1, saves=K.Saves.alloc(h + 1, 4))).launch(s)


def test_batch_meta(K):
    m = K.BatchMeta.new(3)
    with pytest.raises(K.Invalid, match="not set"):
        m.batch()
    with pytest.raises(K.Invalid, match="capacity"):
        m.set([])
    with pytest.raises(K.Invalid, match="capacity"):
        m.set([K.Request(1, 0, 0)] * 4)
    with pytest.raises(K.Invalid, match="one keep per request"):
        m.set([K.Request(1, 0, 0)], keep=[1, 1])
    with pytest.raises(K.Invalid, match="exceeds the request"):
        m.set([K.Request(2, 0, 0)], keep=[3])
    m.set([K.Request(2, 0, 0), K.Request(0, 10, 100), K.Request(5, 20, 200)], keep=[1, 0, 5])
    assert m.batch() == 3 and m.total_rows() == 7
    assert m.cu_rows.download(np.int32, 4).tolist() == [0, 2, 2, 7]
    assert m.keep_d.download(np.int32, 3).tolist() == [1, 0, 5]
    assert m.conv_off.download(np.int64, 3).tolist() == [0, 10, 20]
    assert m.state_off.download(np.int64, 3).tolist() == [0, 100, 200]
    buf = K.DeviceBuffer.zeroed(300 * 4)
    m.check_regions("state", buf, 4, 0, 100, True, lambda r: r.state_offset)
    with pytest.raises(K.Invalid, match="overlap"):
        m.check_regions("state", K.DeviceBuffer.zeroed(400 * 4), 4, 0, 101, True, lambda r: r.state_offset)
    m.check_regions("conv", K.DeviceBuffer.zeroed(400 * 4), 4, 0, 101, False, lambda r: r.state_offset)  # read-only regions may overlap
    with pytest.raises(K.Invalid, match="exceed"):
        m.check_regions("state", buf, 4, 1, 100, True, lambda r: r.state_offset)


def test_batched_rejections(K):
    s, h = K.Stream(), 2
    c = K.channels(h)
    meta = K.BatchMeta.new(2)
    meta.set([K.Request(1, 0, 0), K.Request(1, K.WINDOW * c, K.state_len(h))])
    a = chain_args(K, h, 2)
    for name in ("rows", "conv_offset", "state_offset"):
        a.pop(name)
    a["conv"] = K.DeviceBuffer.zeroed(2 * K.WINDOW * c * 2)
    small_state = dict(a, state=K.DeviceBuffer.zeroed(K.state_len(h) * 4))
    with pytest.raises(K.Invalid, match="state"):
        K.ChainBatch(**small_state).launch(meta, s)
    a["state"] = K.DeviceBuffer.zeroed(2 * K.state_len(h) * 4)
    with pytest.raises(K.Invalid, match="use InPlace"):
        K.ChainBatch(**dict(a, state_out=K.StateOut.To(a["state"], 0))).launch(meta, s)
    # bf16 states: the same buffer holds four requests' worth, offsets count bf16 elements
    with pytest.raises(K.Invalid, match="saves hold"):
        K.ChainBatch(**dict(a, saves=K.Saves.alloc(h, 1))).launch_bf16_state(meta, s)
    ls = K.LayerSaves.alloc(2, h, 2)
    assert ls.kv_stride() == 2 * h * K.DK and ls.b_stride() == 2 * h
    with pytest.raises(K.Invalid, match="shape mismatch"):
        ls.fill_layer(2, K.Saves.alloc(h, 2), 2)
    with pytest.raises(K.Invalid, match="replay_layers"):
        K.replay_layers(3, a["state"], a["state"], K.state_len(h), ls, s)
    with pytest.raises(K.Invalid, match="replay_layers"):
        K.replay_layers(1, a["state"], a["state"], K.state_len(h) - 1, ls, s)
    with pytest.raises(K.Invalid, match="layers' regions overlap"):
        K.replay_batch(meta, K.DeviceBuffer.zeroed(4 * K.state_len(h) * 4), K.DeviceBuffer.zeroed(4 * K.state_len(h) * 4), K.state_len(h), ls, s)
    with pytest.raises(K.Invalid, match="no layers"):
        K.conv_shift_batch(h, 0, meta, a["conv"], 2 * K.WINDOW * c, a["p"], 0, s)
    with pytest.raises(K.Invalid, match="windows overlap"):
        K.conv_shift_batch(h, 2, meta, K.DeviceBuffer.zeroed(4 * K.WINDOW * c * 2), K.WINDOW * c, a["p"], 0, s)
    with pytest.raises(K.Invalid, match="p: rows reach"):
        K.conv_shift(h, 2, a["conv"], 0, K.RowView.dense(K.DeviceBuffer.zeroed(c * 2), c), s)


def test_prefill_rejections(K):
    s, h = K.Stream(), 2
    ws = K.PrefillWorkspace.new(h, 1, 20)
    assert ws.rows_per_pass == 32 and ws.buf.bytes() == 34816 * h * 2
    assert K.PrefillWorkspace.within(h, 1, 3 * 34816 * h + 5).rows_per_pass == 48
    base = chain_args(K, h, 1)
    base.pop("saves")
    with pytest.raises(K.Invalid, match="value_blocks"):
        K.Prefill(**base, value_blocks=3, workspace=ws).launch(s)
    with pytest.raises(K.Invalid, match="lower bound"):
        K.Prefill(**dict(base, weights=weights(K, h, lower=-6.0)), value_blocks=0, workspace=ws).launch(s)
    with pytest.raises(K.Invalid, match="always writes its state"):
        K.Prefill(**dict(base, state_out=K.StateOut.Skip), value_blocks=0, workspace=ws).launch(s)
    with pytest.raises(K.Invalid, match="workspace for"):
        K.Prefill(**base, value_blocks=0, workspace=K.PrefillWorkspace.new(h + 1, 1, 16)).launch(s)


def test_form_switches(K):
    """The process-wide switches between the exact and the chunked forms: exact by default, each setter returns the
    form that was in force (host-side state of the library: no GPU involved)."""
    F = K.Form
    for setter in (K.set_prefill_form, K.set_verify_form, K.set_commit_form):
        assert setter(F.CHUNKED) is F.EXACT
        assert setter(F.EXACT) is F.CHUNKED
        assert setter(F.EXACT) is F.EXACT
