"""Checked wrappers over the thirteen reference entry points: the host API of the reference crate, in Python.

Mirror of crates/glm53f-kda/src/kernel.rs (names, fields, argument meaning and error behaviour) and of the parts of
src/device.rs it needs, over the C ABI of include/glm53f_kda.h.  Each launch checks on the host that every buffer is
large enough for the geometry it is given, that written regions do not overlap and that the batch metadata is
consistent, then enqueues the kernel; a rejection raises `Invalid` (the reference's Error::Invalid), any other
non-zero status `CudaError` (Error::Cuda), kernel.rs:127-135.  Launches are asynchronous on the given stream.

  Weights (kernel.rs:15-52)        RowView (55-105)          Saves (138-179)        StateOut (182-190)
  StateType (193-211)              Chain (223-326)           replay (330-365)       conv_shift (369-394)
  Request (397-405)                BatchMeta (409-526)       ChainBatch (530-679)   LayerSaves (682-737)
  replay_layers (741-777)          replay_batch[_bf16_state] (782-905)              conv_shift_batch (912-973)
  PrefillWorkspace (992-1041)      Prefill (1055-1141)       PrefillBatch (1146-1285)
  DeviceBuffer, Stream (device.rs:10-286): device memory and streams are torch's here.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import ffi
from .core import CudaError, Invalid

DK = DV = 128
TAPS = 4
WINDOW = TAPS - 1
PREFILL_LOWER_MIN = -5.8  # kernel.rs:977


def channels(heads: int) -> int:
    return 3 * heads * DK


def state_len(heads: int) -> int:
    return heads * DV * DK


# Where DeviceBuffer allocates.  "cuda" for anything that launches; the host-side checks can be exercised without a GPU
# by pointing this at "cpu" (nothing is launched when a check rejects the arguments).
DEVICE = "cuda"


def _torch():
    import torch

    return torch


class DeviceBuffer:
    """Bytes of device memory (device.rs:10-160), held as a torch uint8 CUDA tensor."""

    def __init__(self, tensor):
        self.t = tensor

    @classmethod
    def alloc(cls, nbytes: int) -> "DeviceBuffer":
        torch = _torch()
        return cls(torch.empty(max(int(nbytes), 0), dtype=torch.uint8, device=DEVICE))

    @classmethod
    def zeroed(cls, nbytes: int) -> "DeviceBuffer":
        torch = _torch()
        return cls(torch.zeros(max(int(nbytes), 0), dtype=torch.uint8, device=DEVICE))

    @classmethod
    def from_slice(cls, data) -> "DeviceBuffer":
        torch = _torch()
        a = np.ascontiguousarray(data)
        return cls(torch.from_numpy(a.view(np.uint8).reshape(-1).copy()).to(DEVICE))

    def bytes(self) -> int:
        return int(self.t.numel())

    def as_ptr(self) -> int:
        return int(self.t.data_ptr()) if self.t.numel() else 0

    def ptr(self, offset: int = 0, size: int = 1) -> C.c_void_p:
        """Address of element `offset` for elements of `size` bytes."""
        return C.c_void_p(self.as_ptr() + int(offset) * size)

    def upload(self, data) -> None:
        self.upload_at(0, data)

    def upload_at(self, offset: int, data) -> None:
        """Copy `data` to element `offset` (elements of data's dtype); synchronous."""
        torch = _torch()
        a = np.ascontiguousarray(data)
        raw = a.view(np.uint8).reshape(-1)
        start = int(offset) * a.dtype.itemsize
        if start + raw.size > self.bytes():
            raise Invalid(f"upload of {raw.size} bytes at {start} exceeds a buffer of {self.bytes()}")
        self.t[start:start + raw.size].copy_(torch.from_numpy(raw.copy()))
        if self.t.is_cuda:
            torch.cuda.synchronize()

    def download(self, dtype, n: int, offset: int = 0) -> np.ndarray:
        """The `n` elements of `dtype` from element `offset`, on the host; synchronous."""
        dt = np.dtype(dtype)
        start, stop = int(offset) * dt.itemsize, (int(offset) + int(n)) * dt.itemsize
        if stop > self.bytes():
            raise Invalid(f"download of elements [{offset}, {offset} + {n}) exceeds the buffer")
        return self.t[start:stop].cpu().numpy().view(dt).copy()


class Stream:
    """A CUDA stream (device.rs:163-230): torch's current stream unless one is given."""

    def __init__(self, stream=None):
        self.stream = stream

    def raw(self) -> C.c_void_p:
        torch = _torch()
        s = self.stream if self.stream is not None else torch.cuda.current_stream()
        return C.c_void_p(s.cuda_stream)

    def synchronize(self) -> None:
        torch = _torch()
        (self.stream if self.stream is not None else torch.cuda.current_stream()).synchronize()


def _launched(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 1:
        raise Invalid(f"{what}: rejected by the launcher")
    raise CudaError(code, what)


def _to_i32(x: int, what: str) -> int:
    if not 0 <= int(x) <= 0x7FFFFFFF:
        raise Invalid(f"{what} = {x} does not fit in 32 bits")
    return int(x)


def _check_region(what: str, buf: DeviceBuffer, size: int, offset: int, n: int) -> None:
    length = buf.bytes() // size
    if offset < 0 or offset + n > length:
        raise Invalid(f"{what}: elements [{offset}, {offset} + {n}) exceed a buffer of {length}")


def _same(a: DeviceBuffer, b: DeviceBuffer) -> bool:
    return a.as_ptr() == b.as_ptr() and a.bytes() > 0


def _coincide_or_disjoint(a: int, b: int, n: int) -> bool:
    return a == b or a + n <= b or b + n <= a


@dataclass
class LayerParams:
    """One layer's parameters on the host (the reference's cpu::LayerParams, src/cpu.rs:86-100)."""

    heads: int
    conv_w: np.ndarray   # [C][TAPS], bf16-representable f32
    a_log: np.ndarray    # [H]
    dt_bias: np.ndarray  # [H * DK]
    norm_w: np.ndarray   # [DV], bf16-representable f32
    eps: float = 1e-5
    lower: float = -5.0


def _bf16_encode(x) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even (exact for values that came from bfloat16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
    return r


def _bf16_decode(b) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


class Weights:
    """One layer's weights on the device (kernel.rs:15-52)."""

    def __init__(self, heads, conv_w, a_log, dt_bias, norm_w, eps, lower):
        self.heads, self.conv_w, self.a_log, self.dt_bias, self.norm_w, self.eps, self.lower = heads, conv_w, a_log, dt_bias, norm_w, eps, lower

    @classmethod
    def upload(cls, p: LayerParams) -> "Weights":
        if (np.size(p.conv_w) != channels(p.heads) * TAPS or np.size(p.a_log) != p.heads or np.size(p.dt_bias) != p.heads * DK
                or np.size(p.norm_w) != DV):
            raise Invalid("layer parameters have the wrong sizes")
        return cls(p.heads, DeviceBuffer.from_slice(_bf16_encode(p.conv_w)), DeviceBuffer.from_slice(np.asarray(p.a_log, np.float32)),
                   DeviceBuffer.from_slice(np.asarray(p.dt_bias, np.float32)), DeviceBuffer.from_slice(_bf16_encode(p.norm_w)),
                   float(p.eps), float(p.lower))


@dataclass
class RowView:
    """Rows in a device buffer: row r starts at element `offset + r * stride` (kernel.rs:55-105)."""

    buf: DeviceBuffer
    offset: int
    stride: int

    @classmethod
    def new(cls, buf: DeviceBuffer, offset: int, stride: int) -> "RowView":
        return cls(buf, offset, stride)

    @classmethod
    def dense(cls, buf: DeviceBuffer, width: int) -> "RowView":
        return cls(buf, 0, width)

    def check(self, what: str, size: int, first: int, rows: int, lo: int, hi: int) -> None:
        """Rows first .. first + rows have columns [lo, hi) inside the buffer (elements of `size` bytes)."""
        if rows == 0:
            return
        length = self.buf.bytes() // size
        start = self.offset + first * self.stride
        mn, mx = start + lo, start + (rows - 1) * self.stride + hi
        if mn < 0 or mx > length:
            raise Invalid(f"{what}: rows reach elements [{mn}, {mx}) of a buffer of {length}")

    def ptr(self, size: int = 2) -> C.c_void_p:
        return self.buf.ptr(self.offset, size)


@dataclass
class HostSaves:
    """The first rows of a Saves on the host (the reference's cpu::Saves)."""

    heads: int
    rows: int
    k: np.ndarray
    v: np.ndarray
    g: np.ndarray
    beta: np.ndarray


class Saves:
    """Per-row replay inputs on the device, for up to `rows` rows of `heads` heads, one layer (kernel.rs:138-179):
    k f32 [rows][H][DK], v bf16 [rows][H][DV], g f32 [rows][H][DK], b f32 [rows][H]."""

    def __init__(self, heads: int, rows: int, k, v, g, b):
        self.heads, self.rows, self.k, self.v, self.g, self.b = heads, rows, k, v, g, b

    @classmethod
    def alloc(cls, heads: int, rows: int) -> "Saves":
        return cls(heads, rows, DeviceBuffer.zeroed(rows * heads * DK * 4), DeviceBuffer.zeroed(rows * heads * DV * 2),
                   DeviceBuffer.zeroed(rows * heads * DK * 4), DeviceBuffer.zeroed(rows * heads * 4))

    def download(self, rows: int) -> HostSaves:
        h = self.heads
        return HostSaves(h, rows, self.k.download(np.float32, rows * h * DK), _bf16_decode(self.v.download(np.uint16, rows * h * DV)),
                         self.g.download(np.float32, rows * h * DK), self.b.download(np.float32, rows * h))

    def ptrs(self):
        return self.k.ptr(), self.v.ptr(), self.g.ptr(), self.b.ptr()


_NO_SAVES = (None, None, None, None)


class StateOut:
    """Where a chain writes the state after its last row (kernel.rs:182-190): StateOut.Skip (not written: a verify
    round followed by a replay), StateOut.InPlace (over the input state), StateOut.To(buf, offset)."""

    def __init__(self, kind: str, buf: Optional[DeviceBuffer] = None, offset: int = 0):
        self.kind, self.buf, self.offset = kind, buf, offset

    @classmethod
    def To(cls, buf: DeviceBuffer, offset: int = 0) -> "StateOut":
        return cls("to", buf, offset)

    def __repr__(self):
        return f"StateOut.{self.kind}"


StateOut.Skip = StateOut("skip")
StateOut.InPlace = StateOut("in_place")


class StateType(enum.Enum):
    """How a batch launch's states are stored (kernel.rs:193-211): f32, or bf16 with f32 arithmetic and the state
    rounded after every row (chain, replay) or chunk (prefill)."""

    F32 = 4
    Bf16 = 2

    def bytes(self) -> int:
        return self.value


class Form(enum.IntEnum):
    """Which form a layer entry point runs (additions of this library; process-wide switches of the C library):
    EXACT leaves the reference kernels' bits and is the default, CHUNKED runs on the tensor cores and agrees to the
    rounding of bf16 operands."""

    EXACT = 0
    CHUNKED = 1


def set_prefill_form(form: Form) -> Form:
    """glm53f_kda_prefill_mode: the form of glm53f_kda_prefill*; returns the form that was in force."""
    return Form(ffi.load().glm53f_kda_prefill_mode(int(form)))


def set_verify_form(form: Form) -> Form:
    """glm53f_kda_verify_mode: the form of a verify call of glm53f_kda_chain_batch_bf16state (state not written, saves on)."""
    return Form(ffi.load().glm53f_kda_verify_mode(int(form)))


def set_commit_form(form: Form) -> Form:
    """glm53f_kda_commit_mode: the form of the bf16-state replays."""
    return Form(ffi.load().glm53f_kda_commit_mode(int(form)))


def _check_saves(saves: Optional[Saves], heads: int, rows: int):
    if saves is None:
        return _NO_SAVES
    if saves.heads != heads or saves.rows < rows:
        raise Invalid(f"saves hold {saves.rows} rows of {saves.heads} heads")
    return saves.ptrs()


def _check_rows(heads: int, total: int, p: RowView, b_off: int, a: RowView, g: RowView, out: RowView) -> None:
    c = channels(heads)
    lo, hi = min(b_off, 0), max(c, b_off + heads)
    p.check("p", 2, 0, total, lo, hi)
    a.check("a", 2, 0, total, 0, heads * DK)
    g.check("g", 2, 0, total, 0, heads * DV)
    out.check("out", 2, 0, total, 0, heads * DV)
    if total > 1 and out.stride < heads * DV:
        raise Invalid("out rows overlap")


@dataclass
class Chain:
    """One layer, one request: `rows` rows from the committed state (glm53f_kda_chain; kernel.rs:223-326)."""

    weights: Weights
    rows: int
    p: RowView          # row r: q | k | v in columns [0, C), the beta logits in [b_off, b_off + H)
    b_off: int
    a: RowView          # forget-gate projections, [H * DK] per row
    g: RowView          # output-gate projections, [H * DV] per row
    conv: DeviceBuffer  # the conv window [WINDOW][C] at conv_offset
    conv_offset: int
    state: DeviceBuffer  # the state [H][DV][DK] at state_offset
    state_offset: int
    state_out: StateOut
    out: RowView        # outputs, [H * DV] per row
    saves: Optional[Saves] = None

    def launch(self, stream: Stream) -> None:
        h = self.weights.heads
        if self.rows == 0:
            raise Invalid("a chain needs at least one row")
        _check_rows(h, self.rows, self.p, self.b_off, self.a, self.g, self.out)
        _check_region("conv", self.conv, 2, self.conv_offset, WINDOW * channels(h))
        _check_region("state", self.state, 4, self.state_offset, state_len(h))
        so = self.state_out
        if so.kind == "skip":
            state_out = None
        elif so.kind == "in_place":
            state_out = self.state.ptr(self.state_offset, 4)
        else:
            _check_region("state_out", so.buf, 4, so.offset, state_len(h))
            if _same(so.buf, self.state) and not _coincide_or_disjoint(so.offset, self.state_offset, state_len(h)):
                raise Invalid("state_out partly overlaps the state")
            state_out = so.buf.ptr(so.offset, 4)
        ks, vs, gs, bs = _check_saves(self.saves, h, self.rows)
        w = self.weights
        code = ffi.glm53f_kda_chain(_to_i32(h, "heads"), _to_i32(self.rows, "rows"), self.p.ptr(), self.p.stride, self.b_off, self.a.ptr(),
                                    self.a.stride, self.g.ptr(), self.g.stride, self.conv.ptr(self.conv_offset, 2), w.conv_w.ptr(),
                                    self.state.ptr(self.state_offset, 4), state_out, w.a_log.ptr(), w.dt_bias.ptr(), w.norm_w.ptr(), w.eps,
                                    w.lower, self.out.ptr(), self.out.stride, ks, vs, gs, bs, stream.raw())
        _launched(code, "glm53f_kda_chain")


def replay(heads: int, rows: int, state, state_out, saves: Saves, stream: Stream) -> None:
    """One layer, one request: the state after the first `rows` saved rows (glm53f_kda_replay; kernel.rs:330-365).
    `state` and `state_out` are (buffer, element offset); they may coincide (in place)."""
    _check_region("state", state[0], 4, state[1], state_len(heads))
    _check_region("state_out", state_out[0], 4, state_out[1], state_len(heads))
    if _same(state[0], state_out[0]) and not _coincide_or_disjoint(state[1], state_out[1], state_len(heads)):
        raise Invalid("state_out partly overlaps the state")
    if saves.heads != heads or saves.rows < rows:
        raise Invalid(f"saves hold {saves.rows} rows of {saves.heads} heads")
    ks, vs, gs, bs = saves.ptrs()
    code = ffi.glm53f_kda_replay(_to_i32(heads, "heads"), _to_i32(rows, "rows"), state[0].ptr(state[1], 4), state_out[0].ptr(state_out[1], 4),
                                 ks, vs, gs, bs, stream.raw())
    _launched(code, "glm53f_kda_replay")


def conv_shift(heads: int, keep: int, conv: DeviceBuffer, conv_offset: int, p: RowView, stream: Stream) -> None:
    """Advance one conv window ([WINDOW][C] at conv_offset) past `keep` kept rows of p, in place
    (glm53f_kda_conv_shift; kernel.rs:369-394)."""
    c = channels(heads)
    _check_region("conv", conv, 2, conv_offset, WINDOW * c)
    first = max(keep - WINDOW, 0)  # the shift reads new rows keep - WINDOW .. keep
    p.check("p", 2, first, keep - first, 0, c)
    code = ffi.glm53f_kda_conv_shift(_to_i32(c, "channels"), _to_i32(keep, "keep"), conv.ptr(conv_offset, 2), p.ptr(), p.stride, stream.raw())
    _launched(code, "glm53f_kda_conv_shift")


@dataclass(frozen=True)
class Request:
    """One request of a batch (kernel.rs:397-405): its rows in the window (it owns the next `rows` rows of the shared
    buffers), the element offset of its conv window and of its state (per layer)."""

    rows: int
    conv_offset: int
    state_offset: int


class BatchMeta:
    """Batch metadata on the device -- row ranges, offsets and kept rows -- with a host copy for the checks
    (kernel.rs:409-526)."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self._requests: list[Request] = []
        self.cu_rows = DeviceBuffer.zeroed((capacity + 1) * 4)
        self.keep_d = DeviceBuffer.zeroed(capacity * 4)
        self.conv_off = DeviceBuffer.zeroed(capacity * 8)
        self.state_off = DeviceBuffer.zeroed(capacity * 8)

    @classmethod
    def new(cls, capacity: int) -> "BatchMeta":
        return cls(capacity)

    def set(self, requests: Sequence[Request], keep: Optional[Sequence[int]] = None) -> None:
        """Set the requests and, for replays and conv shifts, the rows each keeps (None: all).  Copies to the device
        synchronously."""
        if len(requests) == 0 or len(requests) > self.capacity:
            raise Invalid(f"{len(requests)} requests for a capacity of {self.capacity}")
        if keep is None:
            keep = [r.rows for r in requests]
        elif len(keep) != len(requests):
            raise Invalid("one keep per request")
        for r, k in zip(requests, keep):
            if k > r.rows:
                raise Invalid(f"keep {k} exceeds the request's {r.rows} rows")
        cu = [0]
        for r in requests:
            nxt = cu[-1] + _to_i32(r.rows, "rows")
            if nxt > 0x7FFFFFFF:
                raise Invalid("total rows do not fit in 32 bits")
            cu.append(nxt)
        keep32 = [_to_i32(k, "keep") for k in keep]
        self.cu_rows.upload(np.asarray(cu, np.int32))
        self.keep_d.upload(np.asarray(keep32, np.int32))
        self.conv_off.upload(np.asarray([r.conv_offset for r in requests], np.int64))
        self.state_off.upload(np.asarray([r.state_offset for r in requests], np.int64))
        self._requests = list(requests)

    def requests(self) -> list[Request]:
        return self._requests

    def device_arrays(self):
        """cu_rows (int32 [batch + 1]), keep (int32 [batch]), conv and state offsets (int64 [batch]) as device
        addresses, for launches through the raw bindings (for example inside a captured graph)."""
        return self.cu_rows.ptr(), self.keep_d.ptr(), self.conv_off.ptr(), self.state_off.ptr()

    def total_rows(self) -> int:
        return sum(r.rows for r in self._requests)

    def batch(self) -> int:
        if not self._requests:
            raise Invalid("batch metadata not set")
        return _to_i32(len(self._requests), "batch")

    def check_regions(self, what: str, buf: DeviceBuffer, size: int, base: int, n: int, disjoint: bool, offset) -> None:
        """Each request's region of n elements at offset(r) inside the buffer, pairwise disjoint when `disjoint`."""
        spans = []
        for r in self._requests:
            _check_region(what, buf, size, base + offset(r), n)
            spans.append(offset(r))
        if disjoint:
            spans.sort()
            if any(b < a + n for a, b in zip(spans, spans[1:])):
                raise Invalid(f"{what}: requests' regions overlap")


def _batch_state_out(meta: BatchMeta, so: StateOut, state: DeviceBuffer, es: int, heads: int, allow_skip: bool):
    if so.kind == "skip":
        if not allow_skip:
            raise Invalid("a prefill always writes its state")
        return None
    if so.kind == "in_place":
        return state.ptr()
    meta.check_regions("state_out", so.buf, es, 0, state_len(heads), True, lambda r: r.state_offset)
    if _same(so.buf, state):
        raise Invalid("state_out is the state buffer: use InPlace")
    return so.buf.ptr()


@dataclass
class ChainBatch:
    """One layer, a batch of requests (glm53f_kda_chain_batch; kernel.rs:530-679).  The requests' rows are
    consecutive in p, a, g, out and the saves, in the order of the metadata."""

    weights: Weights
    p: RowView
    b_off: int
    a: RowView
    g: RowView
    conv: DeviceBuffer    # conv windows, at each request's conv_offset
    state: DeviceBuffer   # states, at each request's state_offset
    state_out: StateOut   # To(buf, _) writes at each request's state_offset in buf (the offset is ignored)
    out: RowView
    saves: Optional[Saves] = None

    def launch(self, meta: BatchMeta, stream: Stream) -> None:
        self._launch_as(meta, stream, StateType.F32)

    def launch_bf16_state(self, meta: BatchMeta, stream: Stream) -> None:
        """With bf16 states (glm53f_kda_chain_batch_bf16state): state and state_out hold bf16 values and the
        requests' state_offsets count bf16 elements."""
        self._launch_as(meta, stream, StateType.Bf16)

    def _launch_as(self, meta: BatchMeta, stream: Stream, st: StateType) -> None:
        es, h = st.bytes(), self.weights.heads
        batch, total = meta.batch(), meta.total_rows()
        _check_rows(h, total, self.p, self.b_off, self.a, self.g, self.out)
        meta.check_regions("conv", self.conv, 2, 0, WINDOW * channels(h), False, lambda r: r.conv_offset)
        meta.check_regions("state", self.state, es, 0, state_len(h), True, lambda r: r.state_offset)
        state_out = _batch_state_out(meta, self.state_out, self.state, es, h, True)
        ks, vs, gs, bs = _check_saves(self.saves, h, total)
        w = self.weights
        fn = ffi.glm53f_kda_chain_batch if st is StateType.F32 else ffi.glm53f_kda_chain_batch_bf16state
        code = fn(_to_i32(h, "heads"), batch, meta.cu_rows.ptr(), self.p.ptr(), self.p.stride, self.b_off, self.a.ptr(), self.a.stride,
                  self.g.ptr(), self.g.stride, self.conv.ptr(), meta.conv_off.ptr(), w.conv_w.ptr(), self.state.ptr(), state_out,
                  meta.state_off.ptr(), w.a_log.ptr(), w.dt_bias.ptr(), w.norm_w.ptr(), w.eps, w.lower, self.out.ptr(), self.out.stride,
                  ks, vs, gs, bs, stream.raw())
        _launched(code, "glm53f_kda_chain_batch")


class LayerSaves:
    """Saves for several layers in one allocation each: what a commit replays at once (kernel.rs:682-737)."""

    def __init__(self, layers: int, heads: int, rows: int):
        self.layers, self.heads, self.rows = layers, heads, rows
        self.k = DeviceBuffer.zeroed(layers * rows * heads * DK * 4)
        self.v = DeviceBuffer.zeroed(layers * rows * heads * DV * 2)
        self.g = DeviceBuffer.zeroed(layers * rows * heads * DK * 4)
        self.b = DeviceBuffer.zeroed(layers * rows * heads * 4)

    @classmethod
    def alloc(cls, layers: int, heads: int, rows: int) -> "LayerSaves":
        return cls(layers, heads, rows)

    def kv_stride(self) -> int:
        return self.rows * self.heads * DK

    def b_stride(self) -> int:
        return self.rows * self.heads

    def fill_layer(self, layer: int, s: Saves, rows: int) -> None:
        if layer >= self.layers or s.heads != self.heads or rows > min(self.rows, s.rows):
            raise Invalid("fill_layer: shape mismatch")
        h = self.heads
        self.k.upload_at(layer * self.kv_stride(), s.k.download(np.float32, rows * h * DK))
        self.v.upload_at(layer * self.kv_stride(), s.v.download(np.uint16, rows * h * DV))
        self.g.upload_at(layer * self.kv_stride(), s.g.download(np.float32, rows * h * DK))
        self.b.upload_at(layer * self.b_stride(), s.b.download(np.float32, rows * h))


def replay_layers(rows: int, state: DeviceBuffer, state_out: DeviceBuffer, state_stride: int, saves: LayerSaves, stream: Stream) -> None:
    """Several layers, one request: layer l's state is at l * state_stride (glm53f_kda_replay_layers;
    kernel.rs:741-777)."""
    h, l = saves.heads, saves.layers
    if l == 0 or rows > saves.rows or state_stride < state_len(h):
        raise Invalid("replay_layers: no layers, rows beyond the saves, or overlapping layers")
    for buf in (state, state_out):
        _check_region("state", buf, 4, (l - 1) * state_stride, state_len(h))
    code = ffi.glm53f_kda_replay_layers(_to_i32(h, "heads"), _to_i32(l, "layers"), _to_i32(rows, "rows"), state.ptr(), state_out.ptr(),
                                        state_stride, saves.k.ptr(), saves.v.ptr(), saves.g.ptr(), saves.b.ptr(), saves.kv_stride(),
                                        saves.b_stride(), stream.raw())
    _launched(code, "glm53f_kda_replay_layers")


def _replay_batch_as(meta: BatchMeta, state: DeviceBuffer, state_out: DeviceBuffer, state_stride: int, saves: LayerSaves, stream: Stream,
                     st: StateType) -> None:
    h, l = saves.heads, saves.layers
    batch = meta.batch()
    if l == 0 or meta.total_rows() > saves.rows:
        raise Invalid("replay_batch: no layers, or more rows than the saves hold")
    for buf in (state, state_out):
        meta.check_regions("state", buf, st.bytes(), (l - 1) * state_stride, state_len(h), True, lambda r: r.state_offset)
    if l > 1:
        max_off = max((r.state_offset for r in meta.requests()), default=0)
        if state_stride < max_off + state_len(h):
            raise Invalid("replay_batch: layers' regions overlap")
    fn = ffi.glm53f_kda_replay_batch if st is StateType.F32 else ffi.glm53f_kda_replay_batch_bf16state
    code = fn(_to_i32(h, "heads"), _to_i32(l, "layers"), batch, meta.cu_rows.ptr(), meta.keep_d.ptr(), state.ptr(), state_out.ptr(),
              state_stride, meta.state_off.ptr(), saves.k.ptr(), saves.v.ptr(), saves.g.ptr(), saves.b.ptr(), saves.kv_stride(),
              saves.b_stride(), stream.raw())
    _launched(code, "glm53f_kda_replay_batch")


def replay_batch(meta, state, state_out, state_stride, saves, stream) -> None:
    """Every (layer, request): the state after the request's first keep[b] saved rows (glm53f_kda_replay_batch;
    kernel.rs:782-801)."""
    _replay_batch_as(meta, state, state_out, state_stride, saves, stream, StateType.F32)


def replay_batch_bf16_state(meta, state, state_out, state_stride, saves, stream) -> None:
    """The same with bf16 states, rounded after every row (glm53f_kda_replay_batch_bf16state; kernel.rs:803-822)."""
    _replay_batch_as(meta, state, state_out, state_stride, saves, stream, StateType.Bf16)


def conv_shift_batch(heads: int, layers: int, meta: BatchMeta, conv: DeviceBuffer, conv_stride: int, p: RowView, p_layer_stride: int,
                     stream: Stream) -> None:
    """Every (layer, request): the conv window past the request's kept rows (glm53f_kda_conv_shift_batch;
    kernel.rs:912-973)."""
    c = channels(heads)
    batch = meta.batch()
    if layers == 0:
        raise Invalid("conv_shift_batch: no layers")
    max_off = max((r.conv_offset for r in meta.requests()), default=0)
    if layers > 1 and conv_stride < max_off + WINDOW * c:
        raise Invalid("conv_shift_batch: layers' windows overlap")
    meta.check_regions("conv", conv, 2, (layers - 1) * conv_stride, WINDOW * c, True, lambda r: r.conv_offset)
    for l in (0, layers - 1):
        RowView(p.buf, p.offset + l * p_layer_stride, p.stride).check("p", 2, 0, meta.total_rows(), 0, c)
    code = ffi.glm53f_kda_conv_shift_batch(_to_i32(c, "channels"), _to_i32(layers, "layers"), batch, meta.cu_rows.ptr(), meta.keep_d.ptr(),
                                           conv.ptr(), conv_stride, meta.conv_off.ptr(), p.ptr(), p_layer_stride, p.stride, stream.raw())
    _launched(code, "glm53f_kda_conv_shift_batch")


def _check_lower(lower: float) -> None:
    if not (PREFILL_LOWER_MIN <= lower <= 0.0):
        raise Invalid(f"prefill: gate lower bound {lower} outside [{PREFILL_LOWER_MIN}, 0]")


def _check_value_blocks(value_blocks: int) -> int:
    if value_blocks not in (0, 1, 2, 4):
        raise Invalid(f"value_blocks {value_blocks}: 0 (choose), 1, 2 or 4")
    return int(value_blocks)


class PrefillWorkspace:
    """Device workspace for the prefill entry points, sized by glm53f_kda_prefill_workspace_bytes for `rows_per_pass`
    rows of every request at a time (kernel.rs:992-1041)."""

    def __init__(self, heads: int, batch: int, rows_per_pass: int):
        nbytes = ffi.glm53f_kda_prefill_workspace_bytes(_to_i32(heads, "heads"), _to_i32(batch, "batch"), _to_i32(max(rows_per_pass, 1), "rows_per_pass"))
        self.heads, self.batch = heads, batch
        self.rows_per_pass = (max(rows_per_pass, 1) + 15) // 16 * 16
        self.buf = DeviceBuffer.alloc(int(nbytes))

    @classmethod
    def new(cls, heads: int, batch: int, rows_per_pass: int) -> "PrefillWorkspace":
        return cls(heads, batch, rows_per_pass)

    @classmethod
    def within(cls, heads: int, batch: int, nbytes: int) -> "PrefillWorkspace":
        """The rows per pass that keep the workspace within `nbytes` (at least one 16-row chunk)."""
        chunk = int(ffi.glm53f_kda_prefill_workspace_bytes(_to_i32(heads, "heads"), _to_i32(batch, "batch"), 16))
        return cls(heads, batch, max(nbytes // max(chunk, 1), 1) * 16)

    def args(self, heads: int, batch: int):
        if heads != self.heads or batch > self.batch:
            raise Invalid(f"workspace for {self.heads} heads x {self.batch} requests used for {heads} x {batch}")
        return self.buf.ptr(), self.buf.bytes()


@dataclass
class Prefill:
    """One layer, one request: a prompt segment through the prefill (glm53f_kda_prefill; kernel.rs:1055-1141), from
    the state and conv window it is given.  The conv window is advanced past the rows in place; the state after the
    rows goes to state_out (InPlace or To: a prefill always writes its state)."""

    weights: Weights
    rows: int
    p: RowView
    b_off: int
    a: RowView
    g: RowView
    conv: DeviceBuffer
    conv_offset: int
    state: DeviceBuffer
    state_offset: int
    state_out: StateOut
    out: RowView
    value_blocks: int
    workspace: PrefillWorkspace

    def launch(self, stream: Stream) -> None:
        h = self.weights.heads
        vb = _check_value_blocks(self.value_blocks)
        _check_lower(self.weights.lower)
        _check_rows(h, self.rows, self.p, self.b_off, self.a, self.g, self.out)
        _check_region("conv", self.conv, 2, self.conv_offset, WINDOW * channels(h))
        _check_region("state", self.state, 4, self.state_offset, state_len(h))
        so = self.state_out
        if so.kind == "skip":
            raise Invalid("a prefill always writes its state")
        if so.kind == "in_place":
            state_out = self.state.ptr(self.state_offset, 4)
        else:
            _check_region("state_out", so.buf, 4, so.offset, state_len(h))
            if _same(so.buf, self.state) and not _coincide_or_disjoint(so.offset, self.state_offset, state_len(h)):
                raise Invalid("state_out partly overlaps the state")
            state_out = so.buf.ptr(so.offset, 4)
        ws, ws_bytes = self.workspace.args(h, 1)
        w = self.weights
        code = ffi.glm53f_kda_prefill(_to_i32(h, "heads"), _to_i32(self.rows, "rows"), self.p.ptr(), self.p.stride, self.b_off, self.a.ptr(),
                                      self.a.stride, self.g.ptr(), self.g.stride, self.conv.ptr(self.conv_offset, 2), w.conv_w.ptr(),
                                      self.state.ptr(self.state_offset, 4), state_out, w.a_log.ptr(), w.dt_bias.ptr(), w.norm_w.ptr(), w.eps,
                                      w.lower, self.out.ptr(), self.out.stride, vb, ws, ws_bytes, stream.raw())
        _launched(code, "glm53f_kda_prefill")


@dataclass
class PrefillBatch:
    """One layer, a batch of prompt segments (glm53f_kda_prefill_batch; kernel.rs:1146-1285): request rows
    consecutive in p, a, g and out in the order of the metadata, each request with its own state and conv window
    (advanced in place)."""

    weights: Weights
    p: RowView
    b_off: int
    a: RowView
    g: RowView
    conv: DeviceBuffer
    state: DeviceBuffer
    state_out: StateOut   # InPlace, or To(buf, _): each request's state at its state_offset in buf
    out: RowView
    value_blocks: int
    workspace: PrefillWorkspace

    def launch(self, meta: BatchMeta, stream: Stream) -> None:
        self._launch_as(meta, stream, StateType.F32)

    def launch_bf16_state(self, meta: BatchMeta, stream: Stream) -> None:
        """With bf16 states (glm53f_kda_prefill_batch_bf16state)."""
        self._launch_as(meta, stream, StateType.Bf16)

    def _launch_as(self, meta: BatchMeta, stream: Stream, st: StateType) -> None:
        es, h = st.bytes(), self.weights.heads
        vb = _check_value_blocks(self.value_blocks)
        _check_lower(self.weights.lower)
        batch, total = meta.batch(), meta.total_rows()
        _check_rows(h, total, self.p, self.b_off, self.a, self.g, self.out)
        # The windows are written: they must not overlap.
        meta.check_regions("conv", self.conv, 2, 0, WINDOW * channels(h), True, lambda r: r.conv_offset)
        meta.check_regions("state", self.state, es, 0, state_len(h), True, lambda r: r.state_offset)
        state_out = _batch_state_out(meta, self.state_out, self.state, es, h, False)
        ws, ws_bytes = self.workspace.args(h, batch)
        max_rows = _to_i32(max((r.rows for r in meta.requests()), default=0), "max_rows")
        cu_rows, _, conv_off, state_off = meta.device_arrays()
        w = self.weights
        fn = ffi.glm53f_kda_prefill_batch if st is StateType.F32 else ffi.glm53f_kda_prefill_batch_bf16state
        code = fn(_to_i32(h, "heads"), batch, cu_rows, max_rows, self.p.ptr(), self.p.stride, self.b_off, self.a.ptr(), self.a.stride,
                  self.g.ptr(), self.g.stride, self.conv.ptr(), conv_off, w.conv_w.ptr(), self.state.ptr(), state_out, state_off,
                  w.a_log.ptr(), w.dt_bias.ptr(), w.norm_w.ptr(), w.eps, w.lower, self.out.ptr(), self.out.stride, vb, ws, ws_bytes,
                  stream.raw())
        _launched(code, "glm53f_kda_prefill_batch")
