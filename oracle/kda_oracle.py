"""ctypes view of the CPU oracle (``libkda_oracle.so``).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the bench's CPU-baseline leg import this module; the product
(the package and its CUDA library) never does.  Every function forwards to the C++ restatement in
``kda_oracle.cpp``, which cites the reference lines it follows.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkda_oracle.so")

DK = DV = 128
TAPS = 4
WINDOW = 3
FUSED, UNFUSED, F32 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (g++ only)."""
    if force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(os.path.join(_HERE, f)) > os.path.getmtime(_LIB_PATH)
        for f in ("kda_oracle.cpp", "kda_oracle.h")
    ):
        subprocess.check_call(["make", "-C", _HERE, "libkda_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None
_f32p = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.kdao_bf16_from_f32.restype = C.c_uint16
        L.kdao_bf16_from_f32.argtypes = [C.c_float]
        L.kdao_bf16_to_f32.restype = C.c_float
        L.kdao_bf16_to_f32.argtypes = [C.c_uint16]
        L.kdao_bf16_round.restype = C.c_float
        L.kdao_bf16_round.argtypes = [C.c_float]
        L.kdao_bf16_ulp_distance.restype = C.c_uint32
        L.kdao_bf16_ulp_distance.argtypes = [C.c_uint16, C.c_uint16]
        L.kdao_rng_new.restype = C.c_uint64
        L.kdao_rng_new.argtypes = [C.c_uint64]
        L.kdao_rng_next_u64.restype = C.c_uint64
        L.kdao_rng_next_u64.argtypes = [C.POINTER(C.c_uint64)]
        L.kdao_rng_fill.restype = None
        for name in ("kdao_sigmoid", "kdao_silu"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.kdao_warp_sum.restype = C.c_float
        L.kdao_dot128.restype = C.c_float
        for name in ("kdao_log_decay", "kdao_decay"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float] * 4
        L.kdao_beta.restype = C.c_float
        L.kdao_beta.argtypes = [C.c_float]
        L.kdao_q_scale.restype = C.c_float
        _lib = L
    return _lib


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(_f32p) if a is not None else None


# ------------------------------------------------------------------ scalars
def bf16_from_f32(x: float) -> int:
    return int(lib().kdao_bf16_from_f32(C.c_float(x)))


def bf16_to_f32(b: int) -> float:
    return float(lib().kdao_bf16_to_f32(C.c_uint16(b)))


def bf16_round(x: float) -> float:
    return float(lib().kdao_bf16_round(C.c_float(x)))


def bf16_ulp_distance(a: int, b: int) -> int:
    return int(lib().kdao_bf16_ulp_distance(a, b))


def sigmoid(x):
    return float(lib().kdao_sigmoid(x))


def silu(x):
    return float(lib().kdao_silu(x))


def log_decay(a, dt_bias, a_log, lower):
    return float(lib().kdao_log_decay(a, dt_bias, a_log, lower))


def decay(a, dt_bias, decay_rate, lower):
    return float(lib().kdao_decay(a, dt_bias, decay_rate, lower))


def beta(b):
    return float(lib().kdao_beta(b))


def q_scale():
    return float(lib().kdao_q_scale())


def warp_sum(lanes) -> float:
    a = _f(lanes)
    assert a.size == 32
    return float(lib().kdao_warp_sum(_p(a)))


def dot128(a, b) -> float:
    a, b = _f(a), _f(b)
    return float(lib().kdao_dot128(_p(a), _p(b)))


# ------------------------------------------------------------------ vector helpers (numpy, exact)
def bf16_bits(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bits, round to nearest even, NaN quieted (src/bf16.rs:6-13), vectorised."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    r = ((u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((u >> np.uint32(16)).astype(np.uint16)) | np.uint16(0x0040), r)
    return r


def bf16_widen(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def bf16_round_np(x: np.ndarray) -> np.ndarray:
    return bf16_widen(bf16_bits(x))


# ------------------------------------------------------------------ the reference's generator
class Rng:
    """SplitMix64 with 24-bit uniforms (src/synth.rs:10-45)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(lib().kdao_rng_new(C.c_uint64(seed & (2**64 - 1))))

    def next_u64(self) -> int:
        return int(lib().kdao_rng_next_u64(C.byref(self.state)))

    def uniform(self, lo: float, hi: float) -> float:
        return float(self.fill(1, lo, hi)[0])

    def fill(self, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().kdao_rng_fill(C.byref(self.state), C.c_int64(n), C.c_float(lo), C.c_float(hi), C.c_int(0), _p(out))
        return out

    def fill_bf16(self, n: int, lo: float, hi: float) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        lib().kdao_rng_fill(C.byref(self.state), C.c_int64(n), C.c_float(lo), C.c_float(hi), C.c_int(1), _p(out))
        return out


_M64 = 2**64 - 1


class Layer:
    """A layer's parameters (src/cpu.rs:84-98), synthesised as src/synth.rs:49-60."""

    def __init__(self, heads: int, seed: int):
        rng = Rng(((seed * 3) & _M64) ^ 0x11)
        self.heads = heads
        self.conv_w = rng.fill_bf16(3 * heads * DK * TAPS, -0.6, 0.6)
        self.a_log = rng.fill(heads, -1.5, 1.5)
        self.dt_bias = rng.fill(heads * DK, -1.0, 1.0)
        self.norm_w = rng.fill_bf16(DV, 0.25, 1.75)
        self.eps = 1e-5
        self.lower = -5.0

    @property
    def channels(self):
        return 3 * self.heads * DK


class Rows:
    """Projection rows (src/cpu.rs:123-135), synthesised as src/synth.rs:63-73."""

    def __init__(self, heads: int, rows: int, seed: int | None = None):
        self.heads, self.rows = heads, rows
        if seed is not None:
            rng = Rng(((seed * 5) & _M64) ^ 0x22)
            self.qkv = rng.fill_bf16(rows * 3 * heads * DK, -2.0, 2.0)
            self.a = rng.fill_bf16(rows * heads * DK, -4.0, 4.0)
            self.b = rng.fill_bf16(rows * heads, -4.0, 4.0)
            self.gate = rng.fill_bf16(rows * heads * DV, -4.0, 4.0)

    def slice(self, start: int, n: int) -> "Rows":
        h, c = self.heads, 3 * self.heads * DK
        r = Rows(h, n)
        r.qkv = self.qkv[start * c:(start + n) * c].copy()
        r.a = self.a[start * h * DK:(start + n) * h * DK].copy()
        r.b = self.b[start * h:(start + n) * h].copy()
        r.gate = self.gate[start * h * DV:(start + n) * h * DV].copy()
        return r


def conv_window(heads: int, seed: int) -> np.ndarray:
    return Rng(((seed * 7) & _M64) ^ 0x33).fill_bf16(WINDOW * 3 * heads * DK, -2.0, 2.0)


def state(heads: int, seed: int, scale: float) -> np.ndarray:
    return Rng(((seed * 11) & _M64) ^ 0x44).fill(heads * DV * DK, -scale, scale)


# ------------------------------------------------------------------ per-head pieces
def l2norm(x, scale=None) -> np.ndarray:
    x = _f(x)
    y = np.empty(DK, np.float32)
    lib().kdao_l2norm(_p(x), C.c_int(scale is not None), C.c_float(scale or 0.0), _p(y))
    return y


def literal_l2norm(x) -> np.ndarray:
    x = _f(x)
    y = np.empty(DK, np.float32)
    lib().kdao_literal_l2norm(_p(x), _p(y))
    return y


def update(s, k, g, v, beta_) -> np.ndarray:
    s = _f(s).copy()
    k, g, v = _f(k), _f(g), _f(v)
    lib().kdao_update(_p(s), _p(k), _p(g), _p(v), C.c_float(beta_))
    return s


def read_out(s, q) -> np.ndarray:
    s, q = _f(s), _f(q)
    y = np.empty(DV, np.float32)
    lib().kdao_read_out(_p(s), _p(q), _p(y))
    return y


def gated_rmsnorm(y, w, gate, eps, mode=FUSED, literal=False) -> np.ndarray:
    y, w, gate = _f(y), _f(w), _f(gate)
    o = np.empty(DV, np.float32)
    fn = lib().kdao_literal_gated_rmsnorm if literal else lib().kdao_gated_rmsnorm
    fn(_p(y), _p(w), _p(gate), C.c_float(eps), C.c_int(mode), _p(o))
    return o


def conv_qkv(p: Layer, conv, rows: Rows, r: int, h: int, mode=FUSED):
    conv = _f(conv)
    q, k, v = (np.empty(DK, np.float32) for _ in range(3))
    lib().kdao_conv_qkv(C.c_int(p.heads), _p(p.conv_w), _p(conv), _p(rows.qkv), C.c_int(r), C.c_int(h),
                        C.c_int(mode), _p(q), _p(k), _p(v))
    return q, k, v


def transpose_state(s) -> np.ndarray:
    s = _f(s)
    t = np.empty_like(s)
    lib().kdao_transpose_state(_p(s), C.c_int64(s.size), _p(t))
    return t


def literal_step(s, q, k, v, g, beta_, normalize=True):
    """Returns (new state [128 (k)][128 (v)], read-out)."""
    s = _f(s).copy()
    q, k, v, g = _f(q), _f(k), _f(v), _f(g)
    y = np.empty(DV, np.float32)
    lib().kdao_literal_step(_p(s), _p(q), _p(k), _p(v), _p(g), C.c_float(beta_), C.c_int(int(normalize)), _p(y))
    return s, y


class ChainOut:
    pass


def chain(p: Layer, conv, state_, rows: Rows, mode=FUSED, bf16_state=False, literal=False) -> ChainOut:
    conv, state_ = _f(conv), _f(state_)
    h, r = p.heads, rows.rows
    o = ChainOut()
    o.out = np.empty(r * h * DV, np.float32)
    o.y = np.empty(r * h * DV, np.float32)
    o.state = np.empty(h * DV * DK, np.float32)
    o.k = np.empty(r * h * DK, np.float32)
    o.v = np.empty(r * h * DV, np.float32)
    o.g = np.empty(r * h * DK, np.float32)
    o.beta = np.empty(r * h, np.float32)
    o.heads, o.rows = h, r
    lib().kdao_chain(C.c_int(h), _p(p.conv_w), _p(p.a_log), _p(p.dt_bias), _p(p.norm_w), C.c_float(p.eps),
                     C.c_float(p.lower), _p(conv), _p(state_), C.c_int(r), _p(rows.qkv), _p(rows.a), _p(rows.b),
                     _p(rows.gate), C.c_int(mode), C.c_int(int(bf16_state)), C.c_int(int(literal)), _p(o.out),
                     _p(o.y), _p(o.state), _p(o.k), _p(o.v), _p(o.g), _p(o.beta))
    return o


def replay(state_, saves: ChainOut, keep: int, bf16_state=False) -> np.ndarray:
    state_ = _f(state_)
    out = np.empty_like(state_)
    lib().kdao_replay(C.c_int(saves.heads), _p(state_), C.c_int(saves.rows), _p(saves.k), _p(saves.v), _p(saves.g),
                      _p(saves.beta), C.c_int(keep), C.c_int(int(bf16_state)), _p(out))
    return out


def conv_shift(conv, rows: Rows, keep: int) -> np.ndarray:
    conv = _f(conv)
    out = np.empty_like(conv)
    lib().kdao_conv_shift(C.c_int(rows.heads), _p(conv), C.c_int(rows.rows), _p(rows.qkv), C.c_int(keep), _p(out))
    return out


def chunked_head(q, k, v, g, beta_, state_, chunk: int):
    """One head, literal-layout state; returns (read-out [t][128], new state)."""
    q, k, v, g, beta_ = _f(q), _f(k), _f(v), _f(g), _f(beta_)
    s = _f(state_).copy()
    t = beta_.size
    out = np.empty(t * DV, np.float32)
    lib().kdao_chunked_head(C.c_int(t), _p(q), _p(k), _p(v), _p(g), _p(beta_), _p(s), C.c_int(chunk), _p(out))
    return out, s


def chunked_layer(heads, q, k, v, g, beta_, state_, chunk: int):
    q, k, v, g, beta_ = _f(q), _f(k), _f(v), _f(g), _f(beta_)
    s = _f(state_).copy()
    t = beta_.size // heads
    out = np.empty(t * heads * DV, np.float32)
    lib().kdao_chunked_layer(C.c_int(heads), C.c_int(t), _p(q), _p(k), _p(v), _p(g), _p(beta_), _p(s),
                             C.c_int(chunk), _p(out))
    return out, s


def prefill(p: Layer, conv, state_, rows: Rows, mode=FUSED) -> ChainOut:
    conv, state_ = _f(conv), _f(state_)
    h, r = p.heads, rows.rows
    o = ChainOut()
    o.out = np.empty(r * h * DV, np.float32)
    o.y = np.empty(r * h * DV, np.float32)
    o.state = np.empty(h * DV * DK, np.float32)
    lib().kdao_prefill(C.c_int(h), _p(p.conv_w), _p(p.a_log), _p(p.dt_bias), _p(p.norm_w), C.c_float(p.eps),
                       C.c_float(p.lower), _p(conv), _p(state_), C.c_int(r), _p(rows.qkv), _p(rows.a), _p(rows.b),
                       _p(rows.gate), C.c_int(mode), _p(o.out), _p(o.y), _p(o.state))
    return o


def core_forward(heads, q_bits, k_bits, v_bits, g, beta_, state_, form="recurrent", chunk=64, bf16_state=False,
                 threads=1, h0=0, h1=None, want_y=True):
    """The benchmark configurations' contract.  q/k/v: uint16 bf16 bits [T][H][128]; g f32 [T][H][128];
    beta f32 [T][H]; state f32 kernel layout [H][128 (v)][128 (k)].  Returns (y or None, new state)."""
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    k_bits = np.ascontiguousarray(k_bits, dtype=np.uint16)
    v_bits = np.ascontiguousarray(v_bits, dtype=np.uint16)
    g, beta_ = _f(g), _f(beta_)
    s = _f(state_).copy()
    t = beta_.size // heads
    y = np.zeros(t * heads * DV, np.float32) if want_y else None
    h1 = heads if h1 is None else h1
    lib().kdao_core_forward(C.c_int(heads), C.c_int(h0), C.c_int(h1), C.c_int64(t),
                            q_bits.ctypes.data_as(_u16p), k_bits.ctypes.data_as(_u16p), v_bits.ctypes.data_as(_u16p),
                            _p(g), _p(beta_), _p(s), C.c_int(1 if form == "chunked" else 0), C.c_int(chunk),
                            C.c_int(int(bf16_state)), C.c_int(threads), _p(y) if want_y else None)
    return y, s


def core_step_batch(heads, cu_rows, q_bits, k_bits, v_bits, g, beta_, states, state_off, bf16_state=False, l2norm=False,
                    threads=1, want_saves=False):
    """The recurrent core in the kernels' operation order; returns (y, states after[, saves])."""
    cu = np.ascontiguousarray(cu_rows, dtype=np.int32)
    so = np.ascontiguousarray(state_off, dtype=np.int64)
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    k_bits = np.ascontiguousarray(k_bits, dtype=np.uint16)
    v_bits = np.ascontiguousarray(v_bits, dtype=np.uint16)
    g, beta_ = _f(g), _f(beta_)
    s = _f(states).copy()
    rows = int(cu[-1])
    y = np.zeros(rows * heads * DV, np.float32)
    sv = ChainOut()
    sv.heads, sv.rows = heads, rows
    if want_saves:
        sv.k = np.zeros(rows * heads * DK, np.float32)
        sv.v = np.zeros(rows * heads * DV, np.float32)
        sv.g = np.zeros(rows * heads * DK, np.float32)
        sv.beta = np.zeros(rows * heads, np.float32)
    i32p, i64p = C.POINTER(C.c_int32), C.POINTER(C.c_int64)
    lib().kdao_core_step_batch(C.c_int(heads), C.c_int(cu.size - 1), cu.ctypes.data_as(i32p),
                               q_bits.ctypes.data_as(_u16p), k_bits.ctypes.data_as(_u16p), v_bits.ctypes.data_as(_u16p),
                               _p(g), _p(beta_), _p(s), so.ctypes.data_as(i64p), C.c_int(int(bf16_state)),
                               C.c_int(int(l2norm)), C.c_int(threads), _p(y),
                               _p(sv.k) if want_saves else None, _p(sv.v) if want_saves else None,
                               _p(sv.g) if want_saves else None, _p(sv.beta) if want_saves else None)
    return (y, s, sv) if want_saves else (y, s)
