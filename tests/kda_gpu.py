"""Helpers for the GPU parity tests: device buffers from numpy, and one function per C-ABI call that runs it on
oracle-style inputs (f32 arrays holding bf16-exact values) and returns numpy results.

`lib` is any library exporting the reference's thirteen symbols: the product (`ffi.load()`), or the reference's
own kernels compiled by `make -C oracle ref`, used as a second checker when present.
"""
from __future__ import annotations

import ctypes as C
import importlib
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DK = DV = 128
REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libglm53f_kda_ref.so")

pkg = importlib.import_module("glm53f-afd_b200")
ffi = pkg.ffi


def product():
    return ffi.load()


_ref = None


def reference_kernels():
    """The reference's own CUDA kernels, or None when they were not built."""
    global _ref
    if _ref is None and os.path.exists(REF_LIB):
        lib = C.CDLL(REF_LIB)
        for name in ffi.REFERENCE_SYMBOLS:
            res, args = ffi.SIGNATURES[name]
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _ref = lib
    return _ref


def bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def widen(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def dev_bf16(x: np.ndarray) -> torch.Tensor:
    """f32 values (bf16-exact or to be rounded) -> device tensor of bf16 bits (int16 storage)."""
    return torch.from_numpy(bf16_bits(x).view(np.int16).copy()).cuda()


def dev_bits(b: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(b, dtype=np.uint16).view(np.int16).copy()).cuda()


def dev_f32(x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32).copy()).cuda()


def dev_i32(x) -> torch.Tensor:
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def dev_i64(x) -> torch.Tensor:
    return torch.tensor(list(x), dtype=torch.int64, device="cuda")


def host_bf16(t: torch.Tensor) -> np.ndarray:
    return widen(t.cpu().numpy().view(np.uint16))


def host_f32(t: torch.Tensor) -> np.ndarray:
    return t.cpu().numpy()


def ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def check_status():
    torch.cuda.synchronize()
    st = ffi.load().glm53f_kda_device_status()
    assert st == 0, f"device status {st}"


class Weights:
    def __init__(self, p):
        self.heads = p.heads
        self.conv_w = dev_bf16(p.conv_w)
        self.a_log = dev_f32(p.a_log)
        self.dt_bias = dev_f32(p.dt_bias)
        self.norm_w = dev_bf16(p.norm_w)
        self.eps, self.lower = p.eps, p.lower


class Result:
    pass


def pack_rows(rows, p_stride=None, b_off=None, pad_front=0):
    """Rows in the engine's layout: p rows [q|k|v|b] (stride p_stride, logits at b_off), a and gate rows."""
    h, r = rows.heads, rows.rows
    c = 3 * h * DK
    p_stride = p_stride or c + h
    b_off = c if b_off is None else b_off
    lo = min(0, b_off)
    buf = np.zeros(pad_front - lo + max(r, 1) * p_stride + h + 8, np.float32)
    base = pad_front - lo
    for i in range(r):
        buf[base + i * p_stride: base + i * p_stride + c] = rows.qkv[i * c:(i + 1) * c]
        buf[base + i * p_stride + b_off: base + i * p_stride + b_off + h] = rows.b[i * h:(i + 1) * h]
    return buf, base, p_stride, b_off


def run_chain(lib, p, conv, state, rows, bf16_state=False, saves=True, write_state=True, in_place=False,
              p_stride=None, b_off=None, out_stride=None, w=None, pad_front=0):
    """glm53f_kda_chain (f32 state) or glm53f_kda_chain_batch_bf16state with a batch of one."""
    h, r = rows.heads, rows.rows
    w = w or Weights(p)
    pbuf, base, p_stride, b_off = pack_rows(rows, p_stride, b_off, pad_front)
    d_p = dev_bf16(pbuf)
    d_a, d_g = dev_bf16(rows.a), dev_bf16(rows.gate)
    d_conv = dev_bf16(conv)
    out_stride = out_stride or h * DV
    d_out = torch.full((max(r, 1) * out_stride + 64,), -1, dtype=torch.int16, device="cuda")  # 0xffff canaries
    d_sin = dev_bf16(state) if bf16_state else dev_f32(state)
    d_sout = d_sin if in_place else torch.zeros_like(d_sin)
    d_k = torch.zeros(r * h * DK, dtype=torch.float32, device="cuda") if saves else None
    d_v = torch.zeros(r * h * DV, dtype=torch.int16, device="cuda") if saves else None
    d_gs = torch.zeros(r * h * DK, dtype=torch.float32, device="cuda") if saves else None
    d_b = torch.zeros(r * h, dtype=torch.float32, device="cuda") if saves else None
    p_ptr = C.c_void_p(d_p.data_ptr() + 2 * base)
    if bf16_state:
        cu, zoff = dev_i32([0, r]), dev_i64([0])
        rc = lib.glm53f_kda_chain_batch_bf16state(h, 1, ptr(cu), p_ptr, p_stride, b_off, ptr(d_a), h * DK, ptr(d_g), h * DV,
                                                  ptr(d_conv), ptr(zoff), ptr(w.conv_w), ptr(d_sin),
                                                  ptr(d_sout) if write_state else None, ptr(zoff), ptr(w.a_log),
                                                  ptr(w.dt_bias), ptr(w.norm_w), w.eps, w.lower, ptr(d_out), out_stride,
                                                  ptr(d_k), ptr(d_v), ptr(d_gs), ptr(d_b), None)
    else:
        rc = lib.glm53f_kda_chain(h, r, p_ptr, p_stride, b_off, ptr(d_a), h * DK, ptr(d_g), h * DV, ptr(d_conv),
                                  ptr(w.conv_w), ptr(d_sin), ptr(d_sout) if write_state else None, ptr(w.a_log),
                                  ptr(w.dt_bias), ptr(w.norm_w), w.eps, w.lower, ptr(d_out), out_stride, ptr(d_k),
                                  ptr(d_v), ptr(d_gs), ptr(d_b), None)
    torch.cuda.synchronize()
    res = Result()
    res.rc = rc
    if rc != 0:
        return res
    raw = host_bf16(d_out)
    res.out_raw = d_out.cpu().numpy().view(np.uint16)
    res.out = np.concatenate([raw[i * out_stride: i * out_stride + h * DV] for i in range(r)]) if r else np.zeros(0, np.float32)
    res.state = host_bf16(d_sout) if bf16_state else host_f32(d_sout)
    res.state_in_after = host_bf16(d_sin) if bf16_state else host_f32(d_sin)
    res.heads, res.rows = h, r
    if saves:
        res.k, res.v, res.g, res.beta = host_f32(d_k), host_bf16(d_v), host_f32(d_gs), host_f32(d_b)
    return res


def run_replay(lib, heads, state, sv, keep, bf16_state=False):
    """glm53f_kda_replay (f32) or glm53f_kda_replay_batch_bf16state with one layer and one request."""
    d_sin = dev_bf16(state) if bf16_state else dev_f32(state)
    d_sout = torch.zeros_like(d_sin)
    d_k, d_v, d_g, d_b = dev_f32(sv.k), dev_bf16(sv.v), dev_f32(sv.g), dev_f32(sv.beta)
    if bf16_state:
        cu, kp, zoff = dev_i32([0, sv.rows]), dev_i32([keep]), dev_i64([0])
        rc = lib.glm53f_kda_replay_batch_bf16state(heads, 1, 1, ptr(cu), ptr(kp), ptr(d_sin), ptr(d_sout), 0, ptr(zoff),
                                                   ptr(d_k), ptr(d_v), ptr(d_g), ptr(d_b), 0, 0, None)
    else:
        rc = lib.glm53f_kda_replay(heads, keep, ptr(d_sin), ptr(d_sout), ptr(d_k), ptr(d_v), ptr(d_g), ptr(d_b), None)
    torch.cuda.synchronize()
    assert rc == 0, rc
    return host_bf16(d_sout) if bf16_state else host_f32(d_sout)


def bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def max_abs(a, b=None):
    a = np.asarray(a, np.float32)
    return float(np.max(np.abs(a - b))) if b is not None else float(np.max(np.abs(a)))


def ulps(a, b):
    ua, ub = bf16_bits(a).astype(np.int32), bf16_bits(b).astype(np.int32)
    oa = np.where(ua & 0x8000, -(ua & 0x7FFF), ua)
    ob = np.where(ub & 0x8000, -(ub & 0x7FFF), ub)
    d = np.abs(oa - ob)
    return int(d.max()) if d.size else 0, int((d != 0).sum())


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.sqrt(np.sum((a - b) ** 2)) / max(np.sqrt(np.sum(b ** 2)), 1e-30))
