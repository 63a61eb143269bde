"""B200 (sm_100a) implementation of the KDA recurrent core behind the reference crate's C ABI.

`ffi`     raw bindings of include/glm53f_kda.h (the drop-in boundary);
`kernel`  checked wrappers mirroring the reference crate's host API (crates/glm53f-kda/src/kernel.rs);
`core`    wrappers of the post-conv ("core") entry points; `marks` state snapshot / restore over pool pages;
`proj`    the projections' GEMM; `verify` the verify / commit round over pool slots;
`synth`   seeded synthetic inputs of the benchmark configurations;
`build()` compiles csrc/ into libglm53f_kda.so (nvcc, sm_100a).
"""
from . import _build, ffi, synth  # noqa: F401

DK = DV = 128
TAPS = 4
WINDOW = 3
HEADS = 64
LAYERS = 34
LOWER_BOUND = -5.0
RMS_EPS = 1e-5
L2_EPS = 1e-6


def build(force: bool = False, verbose: bool = False) -> str:
    return _build.build(force=force, verbose=verbose)


def channels(heads: int) -> int:
    return 3 * heads * DK


def state_len(heads: int) -> int:
    return heads * DV * DK
