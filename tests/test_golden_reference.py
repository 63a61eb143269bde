"""The CPU oracle against outputs of the reference's own CUDA kernels.

tests/golden/reference_kernels.npz holds what the reference's kernels (compiled from the reference tree, run on a
B200 by tests/golden/make_reference_goldens.py) produced on seeded inputs.  The oracle is the reference's CPU code
restated; the bounds below are the ones the reference states between its CPU and GPU code
(crates/glm53f-kda/tests/gpu.rs:312-368, gpu_bf16_state.rs, gpu_prefill.rs:250-300): everything but the transcendentals
is bit-exact, so the recurrence replayed from the kernel's own saves must reproduce the kernel's state bit for bit.
"""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_kernels.npz")


@pytest.fixture(scope="module")
def gold():
    if not os.path.exists(GOLDEN):
        pytest.fail("tests/golden/reference_kernels.npz is missing")
    return np.load(GOLDEN)


def cases(gold, kinds):
    for line in gold["cases"]:
        name, h, r, seed, kind = str(line).split("|")
        if kind in kinds:
            yield name, int(h), int(r), int(seed), kind


def bits(x):
    return np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)


def ulps16(o, a_bits, b):
    d = np.abs(a_bits.astype(np.int64) - o.bf16_bits(b).astype(np.int64))
    return int(d.max(initial=0)), int((d > 0).sum())


class Saves:
    pass


def test_chain_and_replay_against_the_reference_kernels(gold, oracle):
    o = oracle
    n = 0
    for name, h, r, seed, kind in cases(gold, ("chain", "chain_bf16")):
        bf16 = kind == "chain_bf16"
        p, conv, s0, rows = o.Layer(h, seed), o.conv_window(h, seed), o.state(h, seed, 0.5), o.Rows(h, r, seed)
        if bf16:
            s0 = o.bf16_round_np(s0)
        sv = Saves()
        sv.heads, sv.rows = h, r
        sv.k, sv.g, sv.beta, sv.v = gold[name + ".k"], gold[name + ".g"], gold[name + ".beta"], o.bf16_widen(gold[name + ".v"])
        g_state = o.bf16_widen(gold[name + ".state"]) if bf16 else gold[name + ".state"]
        # bitwise: the recurrence given the kernel's own replay inputs, all rows and a prefix
        assert np.array_equal(bits(o.replay(s0, sv, r, bf16_state=bf16)), bits(g_state)), name
        keep = int(gold[name + ".replay_keep"][0])
        g_replay = o.bf16_widen(gold[name + ".replay_state"]) if bf16 else gold[name + ".replay_state"]
        assert np.array_equal(bits(o.replay(s0, sv, keep, bf16_state=bf16)), bits(g_replay)), name
        # the transcendental part within the reference's bounds
        c = o.chain(p, conv, s0, rows, bf16_state=bf16)
        assert float(np.max(np.abs(sv.g - c.g) / np.abs(c.g))) <= 4e-6, name
        assert ulps16(o, gold[name + ".v"], c.v)[0] <= 1 and np.max(np.abs(sv.beta - c.beta)) <= 2.0 ** -8, name
        assert np.max(np.abs(sv.k - c.k)) <= 1.0 / 256.0, name
        assert np.max(np.abs(g_state - c.state)) / np.max(np.abs(c.state)) <= (8e-3 if bf16 else 1e-3), name
        out = o.bf16_widen(gold[name + ".out"])
        assert np.max(np.abs(out - c.out)) / np.max(np.abs(c.out)) <= 1.0 / 256.0, name
        assert ulps16(o, gold[name + ".out"], c.out)[1] * 100 <= max(c.out.size, 100) * (4 if bf16 else 1), name
        n += 1
    assert n == 4


def test_conv_shift_against_the_reference_kernel(gold, oracle):
    o = oracle
    name, h, r, seed, _ = [c for c in cases(gold, ("chain",))][2]
    conv, rows = o.conv_window(h, seed), o.Rows(h, r, seed)
    for keep in (0, 1, 2, 3, 8):
        assert np.array_equal(gold[f"{name}.conv_shift_{keep}"], o.bf16_bits(o.conv_shift(conv, rows, keep))), keep


def test_prefill_against_the_reference_kernel(gold, oracle):
    """The reference's 16-row chunked prefill kernel against the oracle's chain (the recurrence it must agree with,
    gpu_prefill.rs:250-300) and against the oracle's restatement of the chunked host model."""
    o = oracle
    n = 0
    for name, h, r, seed, _ in cases(gold, ("prefill",)):
        p, conv, s0, rows = o.Layer(h, seed), o.conv_window(h, seed), o.state(h, seed, 0.5), o.Rows(h, r, seed)
        c = o.chain(p, conv, s0, rows)
        out = o.bf16_widen(gold[name + ".out"])
        assert np.max(np.abs(gold[name + ".state"] - c.state)) / np.max(np.abs(c.state)) <= 1e-3, name
        assert np.max(np.abs(out - c.out)) / np.max(np.abs(c.out)) <= 1.0 / 128.0, name
        assert ulps16(o, gold[name + ".out"], c.out)[1] * 50 <= c.out.size, name
        m = o.prefill(p, conv, s0, rows)
        assert np.max(np.abs(gold[name + ".state"] - m.state)) / np.max(np.abs(m.state)) <= 1e-3, name
        # the window after the segment is the last three rows of [old window; new rows]
        assert np.array_equal(gold[name + ".conv"], o.bf16_bits(o.conv_shift(conv, rows, r))), name
        n += 1
    assert n == 2
