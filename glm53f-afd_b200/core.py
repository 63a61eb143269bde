"""Checked host wrappers for the core entry points (post-conv inputs), on torch CUDA tensors.

The calling convention follows the reference crate's checked wrappers (crates/glm53f-kda/src/kernel.rs): extents
are checked on the host against the geometry, a rejected launch raises `Invalid`, a CUDA error raises `CudaError`,
and a launch is asynchronous on the current torch stream.  Tensors are the caller's; nothing is allocated here.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import ffi

DK = DV = 128
L2NORM = 1
TENSOR = 2   # verify only: the window as one 16-row chunk on the tensor cores (outputs to bf16-operand rounding, saves exact)
STATIC_SCRATCH_SLOTS = 64  # chains the library's own scratch array can serve (one chunk per pass each)


class Invalid(ValueError):
    """An argument was rejected before anything was enqueued (launcher status 1)."""


class CudaError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: CUDA error {code}")
        self.code = code


def _launched(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 1:
        raise Invalid(f"{what}: rejected by the launcher")
    raise CudaError(code, what)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, what, dtype, numel):
    if t is None:
        raise Invalid(f"{what} is required")
    if not t.is_cuda or not t.is_contiguous():
        raise Invalid(f"{what} must be a contiguous CUDA tensor")
    if t.dtype not in dtype:
        raise Invalid(f"{what} has dtype {t.dtype}")
    if t.numel() < numel:
        raise Invalid(f"{what} holds {t.numel()} elements, needs {numel}")


_BF = (torch.bfloat16, torch.int16, torch.uint16)


def _state_kind(state):
    if state.dtype == torch.float32:
        return 0
    if state.dtype in _BF:
        return 1
    raise Invalid(f"state has dtype {state.dtype}")


def _check_tokens(heads, rows, q, k, v, g, beta, gate, norm_w, out):
    n = rows * heads * DK
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (out, "out")):
        if t is not None or name != "out":  # only the gathering prefill may go without a local `out`
            _need(t, name, _BF, n)
    _need(g, "g", (torch.float32,), n)
    _need(beta, "beta", (torch.float32,), rows * heads)
    if gate is not None:
        _need(gate, "gate", _BF, n)
        _need(norm_w, "norm_w", _BF, DV)


def decode_batch(heads, rows, cu_rows, q, k, v, g, beta, state, state_off, *, state_out="in_place", flags=0,
                 gate=None, norm_w=None, eps=1e-5, out=None, saves=None, max_state_off=None):
    """glm53f_kda_core_decode_batch / _verify_batch.  `rows` = total rows (host), `cu_rows` int32 [batch+1] and
    `state_off` int64 [batch] on the device.  state_out: "in_place", None (verify: not written) or a tensor.
    saves = (k f32, v bf16, g f32, beta f32) makes it the verify entry point."""
    batch = cu_rows.numel() - 1
    _need(cu_rows, "cu_rows", (torch.int32,), 2)
    _need(state_off, "state_off", (torch.int64,), batch)
    _check_tokens(heads, rows, q, k, v, g, beta, gate, norm_w, out)
    kind = _state_kind(state)
    if max_state_off is not None and state.numel() < max_state_off + heads * DV * DK:
        raise Invalid("state: a request's region exceeds the buffer")
    so = state if isinstance(state_out, str) else state_out
    if so is not None and so is not state:
        if so.dtype != state.dtype or so.numel() < state.numel():
            raise Invalid("state_out must match the state's type and size")
    if saves is not None:
        ks, vs, gs, bs = saves
        _need(ks, "k_save", (torch.float32,), rows * heads * DK)
        _need(vs, "v_save", _BF, rows * heads * DV)
        _need(gs, "g_save", (torch.float32,), rows * heads * DK)
        _need(bs, "b_save", (torch.float32,), rows * heads)
        code = ffi.glm53f_kda_core_verify_batch(heads, batch, _ptr(cu_rows), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta),
                                                _ptr(state), _ptr(so), _ptr(state_off), kind, flags, _ptr(gate),
                                                _ptr(norm_w), eps, _ptr(out), _ptr(ks), _ptr(vs), _ptr(gs), _ptr(bs),
                                                _stream())
        return _launched(code, "glm53f_kda_core_verify_batch")
    code = ffi.glm53f_kda_core_decode_batch(heads, batch, _ptr(cu_rows), _ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta),
                                            _ptr(state), _ptr(so), _ptr(state_off), kind, flags, _ptr(gate), _ptr(norm_w),
                                            eps, _ptr(out), _stream())
    _launched(code, "glm53f_kda_core_decode_batch")


def commit_batch(heads, layers, cu_rows, keep, state, state_stride, state_off, saves, kv_stride, b_stride, *,
                 state_out="in_place"):
    """glm53f_kda_core_commit_batch: every layer of every request keeps keep[b] of its verified rows."""
    batch = keep.numel()
    _need(cu_rows, "cu_rows", (torch.int32,), batch + 1)
    _need(keep, "keep", (torch.int32,), batch)
    _need(state_off, "state_off", (torch.int64,), batch)
    kind = _state_kind(state)
    so = state if isinstance(state_out, str) else state_out
    if so is None:
        raise Invalid("a commit writes the state")
    ks, vs, gs, bs = saves
    code = ffi.glm53f_kda_core_commit_batch(heads, layers, batch, _ptr(cu_rows), _ptr(keep), _ptr(state), _ptr(so),
                                            state_stride, _ptr(state_off), kind, _ptr(ks), _ptr(vs), _ptr(gs), _ptr(bs),
                                            kv_stride, b_stride, _stream())
    _launched(code, "glm53f_kda_core_commit_batch")


def prefill_workspace_bytes(heads, batch, chunks_per_pass):
    return int(ffi.glm53f_kda_core_prefill_workspace_bytes(heads, batch, chunks_per_pass))


def prefill_varlen(heads, rows, cu_seqlens, max_len, q, k, v, g, beta, state, state_off, *, state_out="in_place",
                   flags=0, gate=None, norm_w=None, eps=1e-5, out=None, workspace=None, gather=None):
    """glm53f_kda_core_prefill_varlen: chunked prefill of packed variable-length sequences.  With `workspace` (a
    CUDA uint8 tensor) the two-pass glm53f_kda_core_prefill_varlen_ws runs instead; with workspace="static" the
    two passes run on the library's own fixed scratch array (glm53f_kda_core_prefill_varlen_static: for callers
    that must not allocate; at most 64 (sequence, head) chains).  `gather` = (addresses, heads_total, head0) with a
    workspace runs glm53f_kda_core_prefill_varlen_ws_gather: this launch's heads are heads head0.. of heads_total, and
    every output row is also stored into each [rows][heads_total][128] bf16 buffer whose device address is listed
    (this GPU's and its peers'); `out` may then be None."""
    batch = cu_seqlens.numel() - 1
    _need(cu_seqlens, "cu_seqlens", (torch.int32,), 2)
    _need(state_off, "state_off", (torch.int64,), batch)
    if out is None and gather is None:
        raise Invalid("out is required")
    _check_tokens(heads, rows, q, k, v, g, beta, gate, norm_w, out)
    kind = _state_kind(state)
    so = state if isinstance(state_out, str) else state_out
    if so is None:
        raise Invalid("a prefill writes the state")
    if isinstance(workspace, str):
        if workspace != "static":
            raise Invalid("workspace must be a tensor, None or \"static\"")
        if heads * batch > STATIC_SCRATCH_SLOTS:
            raise Invalid(f"the static scratch holds {STATIC_SCRATCH_SLOTS} (sequence, head) chains, got {heads * batch}")
        code = ffi.glm53f_kda_core_prefill_varlen_static(heads, batch, _ptr(cu_seqlens), max_len, _ptr(q), _ptr(k), _ptr(v),
                                                         _ptr(g), _ptr(beta), _ptr(state), _ptr(so), _ptr(state_off), kind,
                                                         flags, _ptr(gate), _ptr(norm_w), eps, _ptr(out), _stream())
        return _launched(code, "glm53f_kda_core_prefill_varlen_static")
    if gather is not None and (workspace is None or isinstance(workspace, str)):
        raise Invalid("gather needs a workspace tensor")
    if workspace is not None:
        if not workspace.is_cuda or not workspace.is_contiguous():
            raise Invalid("workspace must be a contiguous CUDA tensor")
        nbytes = workspace.numel() * workspace.element_size()
        if gather is not None:
            addrs, heads_total, head0 = gather
            if not 1 <= len(addrs) <= 8:
                raise Invalid(f"1 to 8 full buffers, got {len(addrs)}")
            if head0 < 0 or head0 + heads > heads_total:
                raise Invalid(f"heads [{head0}, {head0 + heads}) outside the {heads_total} of the full buffers")
            arr = (C.c_void_p * len(addrs))(*[int(a) for a in addrs])
            code = ffi.glm53f_kda_core_prefill_varlen_ws_gather(heads, batch, _ptr(cu_seqlens), max_len, _ptr(q), _ptr(k), _ptr(v), _ptr(g),
                                                                _ptr(beta), _ptr(state), _ptr(so), _ptr(state_off), kind, flags,
                                                                _ptr(gate), _ptr(norm_w), eps, _ptr(out), _ptr(workspace), nbytes,
                                                                C.cast(arr, C.c_void_p), len(addrs), heads_total, head0, _stream())
            return _launched(code, "glm53f_kda_core_prefill_varlen_ws_gather")
        code = ffi.glm53f_kda_core_prefill_varlen_ws(heads, batch, _ptr(cu_seqlens), max_len, _ptr(q), _ptr(k), _ptr(v), _ptr(g),
                                                     _ptr(beta), _ptr(state), _ptr(so), _ptr(state_off), kind, flags,
                                                     _ptr(gate), _ptr(norm_w), eps, _ptr(out), _ptr(workspace), nbytes, _stream())
        return _launched(code, "glm53f_kda_core_prefill_varlen_ws")
    code = ffi.glm53f_kda_core_prefill_varlen(heads, batch, _ptr(cu_seqlens), max_len, _ptr(q), _ptr(k), _ptr(v), _ptr(g),
                                              _ptr(beta), _ptr(state), _ptr(so), _ptr(state_off), kind, flags, _ptr(gate),
                                              _ptr(norm_w), eps, _ptr(out), _stream())
    _launched(code, "glm53f_kda_core_prefill_varlen")


def device_status() -> int:
    return int(ffi.glm53f_kda_device_status())
