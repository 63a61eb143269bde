"""check_core of the golden-fixture module on the GPU: a fixture set written from the oracle's literal recurrence (the
formulation the reference checks its goldens with, src/cpu.rs:573-610) must pass through the B200 kernels with the
reference's tolerance tiers, for a one-row decode set chained to its prefill set and for a multi-row set with
per-row states; a corrupted expectation must fail."""
import importlib
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128


def literal_rows(o, heads, rows, q, k, v, g, beta, state, step_heads):
    """state: [H][DK][DV] (the model's layout), updated in place; returns outputs and the listed heads' per-row states."""
    y = np.zeros((rows, heads, DV), np.float32)
    steps = []
    for r in range(rows):
        for h in range(heads):
            i = r * heads + h
            s, out = o.literal_step(state[h * DK * DV:(h + 1) * DK * DV], q[i * DK:(i + 1) * DK], k[i * DK:(i + 1) * DK], v[i * DV:(i + 1) * DV],
                                    g[i * DK:(i + 1) * DK], float(beta[i]))
            state[h * DK * DV:(h + 1) * DK * DV] = s
            y[r, h] = out
        steps.append(np.concatenate([state[h * DK * DV:(h + 1) * DK * DV] for h in step_heads]))
    return y.reshape(-1), np.concatenate(steps)


def test_check_core_on_sets_written_from_the_literal_recurrence(oracle, tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    G = importlib.import_module("glm53f-afd_b200.goldens")
    importlib.import_module("glm53f-afd_b200").ffi.load()
    o, heads, rows, layer = oracle, 3, 6, 4
    rng = o.Rng(321)
    n = rows * heads
    q, k, v = rng.fill_bf16(n * DK, -2, 2), rng.fill_bf16(n * DK, -2, 2), rng.fill_bf16(n * DV, -2, 2)
    g = np.log(1.0 / (1.0 + np.exp(-rng.fill(n * DK, 0, 5)))).astype(np.float32)
    beta = rng.fill(n, 0, 1)
    s0 = rng.fill(heads * DK * DV, -0.5, 0.5)
    state = s0.copy()
    y, steps = literal_rows(o, heads, rows, q, k, v, g, beta, state, [2])
    root = str(tmp_path)
    pre = os.path.join(root, f"layer{layer:02d}-prefill")
    G.write_set(pre, [("prefill.kda.q", G.DType.BF16, [1, rows, heads, DK], q), ("prefill.kda.k", G.DType.BF16, [1, rows, heads, DK], k),
                      ("prefill.kda.v", G.DType.BF16, [1, rows, heads, DV], v), ("prefill.kda.g", G.DType.F32, [1, rows, heads, DK], g),
                      ("prefill.kda.beta", G.DType.F32, [1, rows, heads], beta), ("prefill.kda.initial_state", G.DType.F32, [heads, DK, DV], s0),
                      ("prefill.kda.core_out", G.DType.BF16, [1, rows, heads, DV], y), ("prefill.kda.state", G.DType.F32, [heads, DK, DV], state),
                      ("prefill.kda.state_heads", G.DType.F32, [rows, 1, DK, DV], steps),
                      ("prefill.kda.path", G.DType.I32, [1], [1])], notes={"state_heads": [2]})
    s = G.Set.load(pre)
    lf = G.kda_layers(s)[0]
    assert lf.has(G.CORE_ROLES)
    res = G.check_core(s, lf, G.Init())
    assert len(res) == 3 and G.verdict(res), [str(c) for c in res]
    assert all(c.tol == G.TOL_RECURRENT for c in res)        # one tier per set, chosen by the core output's dtype and the path
    assert res[1].max_abs <= 1e-5 and res[2].max_abs <= 1e-5  # the FP32 states agree far inside it

    # the decode set of the same layer: one more row, starting from the prefill set's final state
    q1, k1, v1 = rng.fill_bf16(heads * DK, -2, 2), rng.fill_bf16(heads * DK, -2, 2), rng.fill_bf16(heads * DV, -2, 2)
    g1 = np.log(1.0 / (1.0 + np.exp(-rng.fill(heads * DK, 0, 5)))).astype(np.float32)
    b1 = rng.fill(heads, 0, 1)
    st1 = state.copy()
    y1, _ = literal_rows(o, heads, 1, q1, k1, v1, g1, b1, st1, [0])
    dec = os.path.join(root, f"layer{layer:02d}-decode")
    G.write_set(dec, [("decode.kda.q", G.DType.BF16, [1, 1, heads, DK], q1), ("decode.kda.k", G.DType.BF16, [1, 1, heads, DK], k1),
                      ("decode.kda.v", G.DType.BF16, [1, 1, heads, DV], v1), ("decode.kda.g", G.DType.F32, [1, 1, heads, DK], g1),
                      ("decode.kda.beta", G.DType.F32, [1, 1, heads], b1), ("decode.kda.core_out", G.DType.BF16, [1, 1, heads, DV], y1),
                      ("decode.kda.state", G.DType.F32, [heads, DK, DV], st1)])
    sd = G.Set.load(dec)
    init = G.Init.from_prefill(sd, layer)
    assert init.state is not None and np.array_equal(init.state, state)
    res = G.check_core(sd, G.kda_layers(sd)[0], init)
    assert len(res) == 2 and G.verdict(res), [str(c) for c in res]
    # without the prefill set's state the decode set must fail
    assert not G.verdict(G.check_core(sd, G.kda_layers(sd)[0], G.Init()))
