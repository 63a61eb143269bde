"""Host-side checks of the verify / commit orchestration (forward.rs:1905-1956): no launch, no GPU."""
import importlib

import pytest


def test_round_bookkeeping_and_rejections(pkg, monkeypatch):
    kernel = importlib.import_module("glm53f-afd_b200.kernel")
    marks = importlib.import_module("glm53f-afd_b200.marks")
    verify = importlib.import_module("glm53f-afd_b200.verify")
    monkeypatch.setattr(kernel, "DEVICE", "cpu")
    l = marks.KvLayout.new(1, 0).with_kda_state_bf16(True)
    pool, other = marks.KvPool(marks.KvConfig(l, 3, 2)), marks.KvPool(marks.KvConfig(l, 1, 2))
    with pytest.raises(verify.Invalid, match="2 layers of weights"):
        verify.KdaVerify(pool, [None, None], 16, 4)
    vf = verify.KdaVerify(pool, [None], 12, 4)
    assert vf.v.bytes() == 12 * (24_640 * 2 + 64 * 1_284)  # projection rows + 1,284 B of replay inputs per row and head
    assert verify.VerifyScratch(12, 1, recompute=True).bytes() == 12 * (24_640 * 2 + 8_192 * 2) + 12 * 8_192 * 2
    a, b, c = pool.slot(), pool.slot(), pool.slot()
    with pytest.raises(verify.Invalid, match="commit without a verify"):
        vf.commit([a], [1])
    for bad in ([(a, 0)], [(a, 9)], [(a, 3), (b, 12)]):
        with pytest.raises(verify.Invalid, match="1..=8 rows"):
            vf.verify(bad)
    with pytest.raises(verify.Invalid, match="exceed the scratch"):
        vf.verify([(a, 8), (b, 8)])
    with pytest.raises(verify.Invalid, match="another pool"):
        vf.verify([(other.slot(), 2)])
    a.advance(10)
    vf.verify([(a, 4), (b, 8)])
    assert (a.pending, b.pending, c.pending) == (4, 8, 0)
    with pytest.raises(verify.Invalid, match="mark inside an uncommitted verify window"):
        a.mark()
    with pytest.raises(verify.Invalid, match="pending"):
        vf.verify([(c, 1)])
    with pytest.raises(verify.Invalid, match="commit of 1 slots after a verify of 2"):
        vf.commit([a], [1])
    assert vf.pending is not None  # a commit of the wrong size leaves the round open
    for keep in ([0, 8], [5, 8], [4, 9]):
        vf.pending = [verify._Req(a.slot, 10, 4), verify._Req(b.slot, 0, 8)]
        with pytest.raises(verify.Invalid, match="does not match the pending verify"):
            vf.commit([a, b], keep)
    vf.pending = [verify._Req(a.slot, 10, 4), verify._Req(b.slot, 0, 8)]
    with pytest.raises(verify.Invalid, match="does not match the pending verify of slot 1"):
        vf.commit([b, a], [4, 4])  # the verify's order
