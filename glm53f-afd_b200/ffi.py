"""Raw bindings of the C ABI (include/glm53f_kda.h, include/glm53f_fwd_rows.h, include/glm53f_proj.h), one Python callable per `extern "C"` symbol.

The counterpart of the reference crate's `ffi` module (crates/glm53f-kda/src/ffi.rs:16-287): no checks, raw device
addresses as integers, the launcher's int status returned as is.  The library must exist: there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

_lib = None

P = C.c_void_p
I32, I64, F32 = C.c_int32, C.c_int64, C.c_float

_CHAIN_TAIL = [P, I64, I64, P, I64, P, I64]  # p, p_stride, b_off, a, a_stride, g, g_stride

SIGNATURES = {
    "glm53f_kda_chain": (C.c_int, [I32, I32, *_CHAIN_TAIL, P, P, P, P, P, P, P, F32, F32, P, I64, P, P, P, P, P]),
    "glm53f_kda_chain_batch": (C.c_int, [I32, I32, P, *_CHAIN_TAIL, P, P, P, P, P, P, P, P, P, F32, F32, P, I64, P, P, P, P, P]),
    "glm53f_kda_chain_batch_bf16state": (C.c_int, [I32, I32, P, *_CHAIN_TAIL, P, P, P, P, P, P, P, P, P, F32, F32, P, I64, P, P, P, P, P]),
    "glm53f_kda_replay": (C.c_int, [I32, I32, P, P, P, P, P, P, P]),
    "glm53f_kda_replay_layers": (C.c_int, [I32, I32, I32, P, P, I64, P, P, P, P, I64, I64, P]),
    "glm53f_kda_replay_batch": (C.c_int, [I32, I32, I32, P, P, P, P, I64, P, P, P, P, P, I64, I64, P]),
    "glm53f_kda_replay_batch_bf16state": (C.c_int, [I32, I32, I32, P, P, P, P, I64, P, P, P, P, P, I64, I64, P]),
    "glm53f_kda_conv_shift": (C.c_int, [I32, I32, P, P, I64, P]),
    "glm53f_kda_conv_shift_batch": (C.c_int, [I32, I32, I32, P, P, P, I64, P, P, I64, I64, P]),
    "glm53f_kda_prefill_workspace_bytes": (I64, [I32, I32, I32]),
    "glm53f_kda_prefill": (C.c_int, [I32, I32, *_CHAIN_TAIL, P, P, P, P, P, P, P, F32, F32, P, I64, I32, P, I64, P]),
    "glm53f_kda_prefill_batch": (C.c_int, [I32, I32, P, I32, *_CHAIN_TAIL, P, P, P, P, P, P, P, P, P, F32, F32, P, I64, I32, P, I64, P]),
    "glm53f_kda_prefill_batch_bf16state": (C.c_int, [I32, I32, P, I32, *_CHAIN_TAIL, P, P, P, P, P, P, P, P, P, F32, F32, P, I64, I32, P, I64, P]),
    "glm53f_kda_chain_commit_batch": (C.c_int, [I32, I32, P, P, *_CHAIN_TAIL, P, P, P, P, P, I32, P, P, P, F32, F32, P, I64, P]),
    "glm53f_kda_core_decode_batch": (C.c_int, [I32, I32, P, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P]),
    "glm53f_kda_core_verify_batch": (C.c_int, [I32, I32, P, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P, P, P, P, P]),
    "glm53f_kda_core_commit_batch": (C.c_int, [I32, I32, I32, P, P, P, P, I64, P, I32, P, P, P, P, I64, I64, P]),
    "glm53f_kda_core_prefill_varlen": (C.c_int, [I32, I32, P, I32, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P]),
    "glm53f_kda_core_prefill_workspace_bytes": (I64, [I32, I32, I32]),
    "glm53f_kda_core_prefill_varlen_ws": (C.c_int, [I32, I32, P, I32, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P, I64, P]),
    "glm53f_kda_core_prefill_varlen_ws_gather": (C.c_int, [I32, I32, P, I32, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P, I64, P, I32, I32, I32, P]),
    "glm53f_kda_core_prefill_varlen_static": (C.c_int, [I32, I32, P, I32, P, P, P, P, P, P, P, P, I32, I32, P, P, F32, P, P]),
    "glm53f_kda_device_status": (C.c_int, []),
    "glm53f_kda_debug_wait_test": (C.c_int, [C.c_uint64, I32]),
    "glm53f_kda_prefill_mode": (I32, [I32]),
    "glm53f_kda_verify_mode": (I32, [I32]),
    "glm53f_kda_commit_mode": (I32, [I32]),
    "glm53f_kda_gather_head_range": (C.c_int, [I32, I32, I32, P, P]),
    "glm53f_kda_gather_export": (C.c_int, [P, I64, P]),
    "glm53f_kda_gather_open": (C.c_int, [P, P, P]),
    "glm53f_kda_gather_close": (C.c_int, [P, P]),
    # include/glm53f_fwd_rows.h: the forward crate's row movers (crates/glm53f-forward/src/ffi.rs:75-95) and the mark copy
    "glm53f_fwd_gather_rows": (I32, [P, I64, P, P, I64, I32, I64, P]),
    "glm53f_fwd_scatter_rows": (I32, [P, I64, P, P, I64, I32, I64, P]),
    "glm53f_kda_mark_copy": (I32, [P, I64, P, P, P, I32, P]),
    "glm53f_kda_mark_copy_slots": (I32, [P, I64, P, P, P, P, P, I32, I32, P]),
    # include/glm53f_proj.h: the projections' GEMM (the arguments of glm53f_fwd_gemv_bf16 without its split-K scratch)
    "glm53f_kda_proj_bf16": (I32, [P, I64, I64, P, I64, I64, I32, I32, I32, I32, P, I32, I64, I64, P]),
}

# The reference's thirteen (crates/glm53f-kda/tests/provenance.rs:41-69 asserts exactly these).
REFERENCE_SYMBOLS = [n for n in SIGNATURES if n.startswith("glm53f_kda_") and "_core_" not in n and "_gather_" not in n and n not in ("glm53f_kda_device_status", "glm53f_kda_debug_wait_test", "glm53f_kda_prefill_mode", "glm53f_kda_verify_mode", "glm53f_kda_commit_mode", "glm53f_kda_mark_copy", "glm53f_kda_mark_copy_slots", "glm53f_kda_proj_bf16", "glm53f_kda_chain_commit_batch")]


def library_path() -> str:
    return _build.LIB


def load(path: str | None = None):
    """dlopen the CUDA library and type its entry points.  Raises if it has not been built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or _build.LIB
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(there is no CPU fallback for the KDA kernels)")
    lib = C.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    if path == _build.LIB:
        _lib = lib
    return lib


def __getattr__(name: str):
    if name in SIGNATURES:
        return getattr(load(), name)
    raise AttributeError(name)
