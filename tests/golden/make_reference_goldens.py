#!/usr/bin/env python
"""Generates tests/golden/reference_kernels.npz: outputs of the REFERENCE's own CUDA kernels on seeded inputs.

The reference's kernels (crates/glm53f-kda/kernels/kda.cu, kda_prefill.cu) are compiled from the reference tree
where it lies by `make -C oracle ref` into oracle/_ref/ (build output, not committed); this script runs them on a
GPU through their C ABI on the small cases below and stores what they produced.  Inputs are not stored: they are the
oracle's seeded generator streams (the reference's SplitMix64 synthesis, src/synth.rs:10-73), re-created by the test
from the seeds recorded here.  tests/test_golden_reference.py then holds the CPU oracle to these outputs with the
bounds the reference states between its own CPU and GPU code (crates/glm53f-kda/tests/gpu.rs:312-368).

Run on a machine with a GPU, after `python -c "import __graft_entry__ as g; g.build()"` built oracle/_ref where the
reference sources are present:   python tests/golden/make_reference_goldens.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
for d in (ROOT, os.path.dirname(HERE), os.path.join(ROOT, "oracle")):
    sys.path.insert(0, d)

# (name, heads, rows, seed, kind); kinds: chain (f32 state), chain_bf16 (bf16 state), prefill
CASES = [("chain_h1_r1", 1, 1, 901, "chain"), ("chain_h2_r3", 2, 3, 902, "chain"), ("chain_h1_r8", 1, 8, 903, "chain"),
         ("bf16_h1_r5", 1, 5, 904, "chain_bf16"), ("prefill_h1_r40", 1, 40, 905, "prefill"), ("prefill_h2_r17", 2, 17, 906, "prefill")]


def main():
    import kda_gpu as G
    import kda_oracle as o
    import test_gpu_prefill as TP

    lib = G.reference_kernels()
    if lib is None:
        raise SystemExit("oracle/_ref/libglm53f_kda_ref.so is missing: build it where the reference sources are present")
    out = {"cases": np.array([f"{n}|{h}|{r}|{s}|{k}" for n, h, r, s, k in CASES])}
    for name, h, r, seed, kind in CASES:
        p, conv, s0, rows = o.Layer(h, seed), o.conv_window(h, seed), o.state(h, seed, 0.5), o.Rows(h, r, seed)
        if kind == "prefill":
            res = TP.run_prefill(G, lib, p, conv, s0, rows)
            assert res.rc == 0
            out[name + ".out"] = G.bf16_bits(res.out)
            out[name + ".state"] = res.state
            out[name + ".conv"] = G.bf16_bits(res.conv)
            continue
        bf16 = kind == "chain_bf16"
        if bf16:
            s0 = o.bf16_round_np(s0)
        res = G.run_chain(lib, p, conv, s0, rows, bf16_state=bf16)
        assert res.rc == 0
        out[name + ".out"] = G.bf16_bits(res.out)
        out[name + ".state"] = G.bf16_bits(res.state) if bf16 else res.state
        out[name + ".k"], out[name + ".g"], out[name + ".beta"] = res.k, res.g, res.beta
        out[name + ".v"] = G.bf16_bits(res.v)
        keep = max(r // 2, 0)
        out[name + ".replay_keep"] = np.array([keep])
        rs = G.run_replay(lib, h, s0, res, keep, bf16_state=bf16)
        out[name + ".replay_state"] = G.bf16_bits(rs) if bf16 else rs
    # the conv shift of the first chain case, every keep
    name, h, r, seed, _ = CASES[2]
    conv, rows = o.conv_window(h, seed), o.Rows(h, r, seed)
    import torch

    c = 3 * h * 128
    for keep in (0, 1, 2, 3, 8):
        d_conv, d_p = G.dev_bf16(conv), G.dev_bf16(rows.qkv)
        assert lib.glm53f_kda_conv_shift(c, keep, G.ptr(d_conv), G.ptr(d_p), c, None) == 0
        torch.cuda.synchronize()
        out[f"{name}.conv_shift_{keep}"] = G.bf16_bits(G.host_bf16(d_conv))
    path = os.path.join(HERE, "reference_kernels.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
