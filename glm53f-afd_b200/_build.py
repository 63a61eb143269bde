"""Compiles the CUDA sources under csrc/ into libglm53f_kda.so beside this file (nvcc, sm_100a only)."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "libglm53f_kda.so")

# The IEEE flags are the reference's (crates/glm53f-kda/build.rs:63-68): the chain, the replays and the prologue
# must not contract a multiply and an add, or a replayed prefix stops matching serial steps bit for bit.
IEEE = ["--fmad=false", "--ftz=false", "--prec-div=true", "--prec-sqrt=true"]
SOURCES = {
    "kda_chain.cu": IEEE,
    "kda_conv.cu": IEEE,
    "kda_prefill.cu": IEEE,
    "kda_verify_tc.cu": IEEE,  # the chunked verify: its replay saves must carry the exact path's bits (the same expf)
    "kda_prologue.cu": IEEE,  # the layer prologue in front of the chunked prefill: the chain's prologue arithmetic
    "kda_prefill_tc.cu": [],
    "kda_prefill_sp.cu": [],
    "proj_gemm.cu": [],      # the projections: tcgen05 GEMM
    "proj_gemm_pair.cu": [], # the same on SM pairs (cta_group::2) for many rows
    "kda_gather.cu": [],     # host code only: CUDA IPC handles for the full output buffers of a head-sharded prefill
    "fwd_rows.cu": [],       # row gather / scatter and the mark copy: data movement only  # tensor-core prefill: agrees with the chain to rounding, so default FP flags
}


def nvcc() -> str:
    return os.environ.get("GLM53F_NVCC", "/usr/local/cuda/bin/nvcc")


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers += [os.path.join(INCLUDE, "glm53f_kda.h"), os.path.join(INCLUDE, "glm53f_fwd_rows.h"), os.path.join(INCLUDE, "glm53f_proj.h")]
    objs = []
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)
    for src, flags in SOURCES.items():
        path = os.path.join(CSRC, src)
        obj = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        if force or _stale(obj, [path] + headers):
            cmd = [nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", *flags,
                   "-I" + CSRC, "-I" + INCLUDE, "-Xcompiler", "-fPIC", "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            subprocess.check_call(cmd)
        objs.append(obj)
    if force or _stale(LIB, objs):
        subprocess.check_call([nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs])
    return LIB


if __name__ == "__main__":
    print(build(verbose=True))
