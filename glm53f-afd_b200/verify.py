"""The verify / commit orchestration of the KDA layers: what the reference's forward does around the kernels for a
speculative-decoding round.

Mirror of the KDA half of `Forward::verify` and `Forward::commit` (crates/glm53f-forward/src/forward.rs:1905-2040) and
of `VerifyScratch` (forward.rs:777-815), over the slots of `marks.KvPool`:

  verify   every KDA layer runs its chain over the windows' rows with the states read but not written, and keeps the
           layer's projection rows and replay inputs in the scratch (forward.rs:3484-3560 in Mode::Verify);
  commit   with the rows each slot keeps, one launch replays every layer's saves into the states and one moves every
           layer's conv window past the kept rows (forward.rs:1958-2031); the slots' token counts advance.

The checks and their messages are the reference's: windows of 1..=8 rows, no verify while one is pending, a commit
must name the slots of the pending verify in its order with 1..=rows kept rows.  The attention (DSA) layers, the MLPs
and the sampling between `verify` and `commit` belong to the rest of the forward and are not built: the caller hands
each KDA layer its projected rows (`KdaVerify.layer`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

from . import ffi
from . import kernel as K
from . import marks
from .core import Invalid

KDA_HEADS, KDA_DIM = marks.KDA_HEADS, marks.KDA_DIM
KDA_WIDTH = KDA_HEADS * KDA_DIM
KDA_QKV = marks.KDA_QKV
KDA_P_COLS = KDA_QKV + KDA_HEADS
MAX_WINDOW = 8  # forward.rs:1908


class VerifyScratch:
    """Buffers a verify round keeps until its commit (forward.rs:777-815, the KDA layers' part): every layer's
    projection rows (the conv shift reads them) and replay inputs.  With `recompute` the replay inputs (82,176 bytes
    per row and layer) are not kept: the commit recomputes them from the projection rows and the decay-gate rows
    (16,384 bytes per row and layer), which are kept instead."""

    def __init__(self, rows: int, kda_layers: int, recompute: bool = False):
        self.rows, self.layers, self.recompute = rows, kda_layers, recompute
        self.p = K.DeviceBuffer.zeroed(kda_layers * rows * KDA_P_COLS * 2)
        self.saves = None if recompute else K.LayerSaves.alloc(kda_layers, KDA_HEADS, rows)
        self.a = K.DeviceBuffer.zeroed(kda_layers * rows * KDA_WIDTH * 2) if recompute else None
        self.sink = K.DeviceBuffer.zeroed(rows * KDA_WIDTH * 2) if recompute else None  # the recomputed rows' outputs

    def bytes(self) -> int:
        if self.recompute:
            return self.p.bytes() + self.a.bytes() + self.sink.bytes()
        s = self.saves
        return self.p.bytes() + s.k.bytes() + s.v.bytes() + s.g.bytes() + s.b.bytes()

    def a_rows(self, layer: int) -> K.RowView:
        """Layer `layer`'s decay-gate rows [rows][8192] (recompute mode: the caller's gate GEMM writes them here)."""
        return K.RowView.new(self.a, layer * self.rows * KDA_WIDTH, KDA_WIDTH)

    def p_rows(self, layer: int) -> K.RowView:
        """Layer `layer`'s projection rows [rows][24,640]: the caller's projection GEMM writes them here."""
        return K.RowView.new(self.p, layer * self.rows * KDA_P_COLS, KDA_P_COLS)

    def layer_saves(self, layer: int) -> K.Saves:
        s, kv, b = self.saves, self.saves.kv_stride(), self.saves.b_stride()
        view = lambda buf, at, n, size: K.DeviceBuffer(buf.t[at * size:(at + n) * size])
        return K.Saves(KDA_HEADS, self.rows, view(s.k, layer * kv, kv, 4), view(s.v, layer * kv, kv, 2), view(s.g, layer * kv, kv, 4),
                       view(s.b, layer * b, b, 4))


@dataclass
class _Req:
    slot: int
    start: int
    rows: int


class KdaVerify:
    """Verify and commit over the KDA layers of the slots of one pool."""

    def __init__(self, pool: marks.KvPool, weights: Sequence[K.Weights], max_verify_rows: int, max_requests: int, recompute: bool = False):
        l = pool.cfg.layout
        if len(weights) != l.kda_layers:
            raise Invalid(f"{len(weights)} layers of weights for a pool of {l.kda_layers} KDA layers")
        self.pool, self.weights = pool, list(weights)
        self.v = VerifyScratch(max_verify_rows, l.kda_layers, recompute)
        self.meta = K.BatchMeta.new(max_requests)
        self.pending: Optional[list[_Req]] = None
        self._st = K.StateType.Bf16 if l.kda_state_bf16 else K.StateType.F32

    # ---- verify -----------------------------------------------------------------------------------------------
    def verify(self, windows: Sequence[tuple[marks.GlmKv, int]]) -> None:
        """Open a verify round over `windows` = (slot, rows): checks, batch metadata, the slots become pending."""
        if self.pending is not None or any(kv.pending != 0 for kv, _ in windows):
            raise Invalid("a verify is pending: commit it first")
        rows = [r for _, r in windows]
        if any(r == 0 or r > MAX_WINDOW for r in rows):
            raise Invalid(f"verify windows of 1..=8 rows, got {rows}")
        if sum(rows) > self.v.rows:
            raise Invalid(f"{sum(rows)} verify rows exceed the scratch of {self.v.rows}")
        if any(kv.pool is not self.pool for kv, _ in windows):
            raise Invalid("a slot of another pool")
        self.meta.set([K.Request(r, kv.conv_elem_offset(), kv.state_elem_offset()) for kv, r in windows])
        self.pending = [_Req(kv.slot, kv.tokens(), r) for kv, r in windows]
        for kv, r in windows:
            kv.pending = r

    def _layer_views(self, j: int):
        l = self.pool.cfg.layout
        sn, cn = l.state_elems_per_layer() * l.kda_state_elem_bytes(), l.conv_elems_per_layer() * 2
        return K.DeviceBuffer(self.pool.state.t[j * sn:]), K.DeviceBuffer(self.pool.conv.t[j * cn:])

    def layer(self, j: int, a: K.RowView, g: K.RowView, out: K.RowView, stream: Optional[K.Stream] = None) -> None:
        """KDA layer j of the open round: the chain over the windows' rows in `scratch.p_rows(j)`, states read but not
        written, replay inputs saved (forward.rs:3484-3560 in Mode::Verify)."""
        if self.pending is None:
            raise Invalid("no verify is open")
        state, conv = self._layer_views(j)
        if self.v.recompute and not (a.buf is self.v.a and a.offset == self.v.a_rows(j).offset):
            raise Invalid("recompute mode: layer j's decay-gate rows live in scratch.a_rows(j)")
        cb = K.ChainBatch(self.weights[j], self.v.p_rows(j), KDA_QKV, a, g, conv, state, K.StateOut.Skip, out,
                          None if self.v.recompute else self.v.layer_saves(j))
        stream = stream or self.pool.stream
        if self._st is K.StateType.Bf16:
            cb.launch_bf16_state(self.meta, stream)
        else:
            cb.launch(self.meta, stream)

    # ---- commit -----------------------------------------------------------------------------------------------
    def commit(self, slots: Sequence[marks.GlmKv], keep: Sequence[int], stream: Optional[K.Stream] = None) -> None:
        """Keep the first keep[i] pending rows of slots[i] (the slots of the last verify, in its order),
        forward.rs:1934-2031."""
        pending, self.pending = self.pending, None
        if pending is None:
            raise Invalid("commit without a verify")
        if len(slots) != len(pending) or len(keep) != len(slots):
            self.pending = pending
            raise Invalid(f"commit of {len(slots)} slots after a verify of {len(pending)}")
        for kv, req, k in zip(slots, pending, keep):
            if kv.slot != req.slot or kv.pending != req.rows or kv.tokens() != req.start or k == 0 or k > req.rows:
                raise Invalid(f"commit of {k} rows does not match the pending verify of slot {kv.slot}")
        l = self.pool.cfg.layout
        stream = stream or self.pool.stream
        self.meta.set(self.meta.requests(), list(keep))
        # The arenas are slot-major ([slot][layer]...): layer strides of one layer's elements, request offsets of whole
        # slots.  The checked wrappers of kernel.py assume layer-major arenas, so, like the reference's forward, this goes
        # to the entry points directly (forward.rs:1972-2031).
        sn, cn = l.state_elems_per_layer(), l.conv_elems_per_layer()
        sv, m = self.v.saves, self.meta
        if self.v.recompute:
            # No saves: every layer's chain again over the kept rows, in place, from the rows the round kept.  The decay
            # rows stand in for the output-gate rows: the outputs go to a sink.
            for j, w in enumerate(self.weights):
                state, conv = self._layer_views(j)
                pr, ar = self.v.p_rows(j), self.v.a_rows(j)
                K._launched(ffi.glm53f_kda_chain_commit_batch(
                    KDA_HEADS, m.batch(), m.cu_rows.ptr(), m.keep_d.ptr(), pr.ptr(), pr.stride, KDA_QKV, ar.ptr(), ar.stride, ar.ptr(), ar.stride,
                    conv.ptr(), m.conv_off.ptr(), w.conv_w.ptr(), state.ptr(), m.state_off.ptr(), 1 if self._st is K.StateType.Bf16 else 0,
                    w.a_log.ptr(), w.dt_bias.ptr(), w.norm_w.ptr(), w.eps, w.lower, self.v.sink.ptr(), KDA_WIDTH, stream.raw()),
                    "glm53f_kda_chain_commit_batch")
        else:
            fn = ffi.glm53f_kda_replay_batch_bf16state if self._st is K.StateType.Bf16 else ffi.glm53f_kda_replay_batch
            K._launched(fn(KDA_HEADS, l.kda_layers, m.batch(), m.cu_rows.ptr(), m.keep_d.ptr(), self.pool.state.ptr(), self.pool.state.ptr(), sn,
                           m.state_off.ptr(), sv.k.ptr(), sv.v.ptr(), sv.g.ptr(), sv.b.ptr(), sv.kv_stride(), sv.b_stride(), stream.raw()),
                        "glm53f_kda_replay_batch")
        K._launched(ffi.glm53f_kda_conv_shift_batch(KDA_QKV, l.kda_layers, m.batch(), m.cu_rows.ptr(), m.keep_d.ptr(), self.pool.conv.ptr(), cn,
                                                    m.conv_off.ptr(), self.v.p.ptr(), self.v.rows * KDA_P_COLS, KDA_P_COLS, stream.raw()),
                    "glm53f_kda_conv_shift_batch")
        for kv, k in zip(slots, keep):
            kv.advance(k)
            kv.pending = 0
