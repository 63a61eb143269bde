"""Draft verification as one 16-row chunk on the tensor cores (GLM53F_KDA_CORE_TENSOR on glm53f_kda_core_verify_batch).

What the flag may change and what it may not: a window's outputs agree with the exact verify's (which are the serial
decode steps' bits) within the task's tolerance for bf16 outputs (max-abs 2e-2, rel-L2 5e-3); the replay saves are the
exact verify's bit for bit, so the commit leaves the states of serial decode steps; the states are not touched.
Windows of 0..16 rows, scattered slots, the model's strongest gates, configuration 4's shape (48 slots x 16 rows).
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128
OUT_MAX_ABS, OUT_REL_L2 = 2e-2, 5e-3


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import importlib

    import kda_gpu as G

    G.product()
    return G, importlib.import_module("glm53f-afd_b200.core"), importlib.import_module("glm53f-afd_b200")


def verify(G, core, heads, cu, tok, d_state, d_off, flags):
    rows = int(cu[-1])
    q, k, v, g, beta = tok
    dq, dk, dv, dg, db = G.dev_bits(q), G.dev_bits(k), G.dev_bits(v), G.dev_f32(g), G.dev_f32(beta)
    out = torch.full((rows * heads * DV + 32,), -1, dtype=torch.int16, device="cuda")
    sv = (torch.zeros(rows * heads * DK, device="cuda"), torch.zeros(rows * heads * DV, dtype=torch.int16, device="cuda"),
          torch.zeros(rows * heads * DK, device="cuda"), torch.zeros(rows * heads, device="cuda"))
    d_cu = G.dev_i32(cu)
    core.decode_batch(heads, rows, d_cu, dq, dk, dv, dg, db, d_state, d_off, state_out=None, flags=flags, out=out, saves=sv)
    G.check_status()
    assert (out[rows * heads * DV:].cpu().numpy() == -1).all()
    return G.host_bf16(out)[:rows * heads * DV], [x.cpu().numpy() for x in sv]


def compare(G, got, want, saves_got, saves_want):
    assert G.max_abs(got, want) <= OUT_MAX_ABS
    assert G.rel_l2(got, want) <= OUT_REL_L2
    for a, b in zip(saves_got, saves_want):   # k, v, exp(g), beta: the commit's inputs, bit for bit
        assert np.array_equal(a.view(np.uint8), b.view(np.uint8))


@pytest.mark.parametrize("gates", ["benchmark", "strongest", "mixed"])
def test_windows_of_every_length_against_the_exact_verify(env, oracle, gates):
    G, core, pkg = env
    heads, lens = 3, [16, 1, 7, 0, 16, 9]
    slots, per = len(lens), heads * DV * DK
    rows = sum(lens)
    q, k, v, g, beta = pkg.synth.tokens(4, 3, rows, heads)
    if gates == "strongest":
        g = np.full_like(g, -5.8)
    elif gates == "mixed":
        g = (np.where((np.arange(rows) % 3 == 0)[:, None, None], 0.0, -5.0) * np.ones((rows, heads, DK))).astype(np.float32).reshape(-1)
    states = oracle.bf16_round_np(np.concatenate([pkg.synth.state(4, 3, s, heads) for s in range(slots)]))
    cu = np.concatenate([[0], np.cumsum(lens)])
    order = [4, 0, 5, 2, 1, 3]   # slots scattered in the arena
    d_state, d_off = G.dev_bf16(states), G.dev_i64([s * per for s in order])
    before = d_state.clone()
    want, sv_want = verify(G, core, heads, cu, (q, k, v, g, beta), d_state, d_off, 0)
    got, sv_got = verify(G, core, heads, cu, (q, k, v, g, beta), d_state, d_off, core.TENSOR)
    assert torch.equal(d_state, before), "a verify must not touch the states"
    compare(G, got, want, sv_got, sv_want)
    # and against the FP32 recurrence itself, request by request
    st = states.reshape(slots, per)
    for i, n in enumerate(lens):
        if n == 0:
            continue
        part = lambda a, w: a.reshape(rows, heads * w)[cu[i]:cu[i] + n].reshape(-1)
        y, _ = oracle.core_forward(heads, part(q, DK), part(k, DK), part(v, DV), part(g, DK), beta.reshape(rows, heads)[cu[i]:cu[i] + n].reshape(-1),
                                   st[order[i]], form="recurrent", threads=2)
        mine = got.reshape(rows, heads * DV)[cu[i]:cu[i] + n].reshape(-1)
        assert G.max_abs(mine, y) <= OUT_MAX_ABS and G.rel_l2(mine, y) <= OUT_REL_L2, i


def test_configuration_4_shape_and_the_commit(env):
    """48 slots x 16 draft rows x 64 heads, two layers: outputs within tolerance of the exact verify, saves identical, and
    the commit from the tensor-core verify's saves leaves the exact verify's committed states, bit for bit."""
    G, core, pkg = env
    heads, slots, window, layers = 64, 48, 16, 2
    per, rows = heads * DV * DK, slots * window
    gs = torch.Generator(device="cuda").manual_seed(17)
    keeps = torch.tensor(np.random.default_rng(3).integers(0, window + 1, slots), dtype=torch.int32, device="cuda")
    cu = torch.arange(slots + 1, dtype=torch.int32, device="cuda") * window
    off = torch.arange(slots, dtype=torch.int64, device="cuda") * per
    nkv, nb = rows * heads * DK, rows * heads
    n = rows * heads

    def unit(scale):
        x = torch.randn(n, DK, device="cuda", generator=gs)
        return (x * (scale / torch.sqrt((x * x).sum(1, keepdim=True) + 1e-6))).to(torch.bfloat16).reshape(-1)

    arenas, outs = {}, {}
    for flags in (0, core.TENSOR):
        gs.manual_seed(17)
        arena = (torch.randn(layers * slots * per, device="cuda", generator=gs) * 0.05).to(torch.bfloat16)
        ks, gsv = torch.zeros(layers * nkv, device="cuda"), torch.zeros(layers * nkv, device="cuda")
        vs, bs = torch.zeros(layers * nkv, dtype=torch.bfloat16, device="cuda"), torch.zeros(layers * nb, device="cuda")
        out = torch.zeros(layers * rows * heads * DV, dtype=torch.bfloat16, device="cuda")
        for l in range(layers):
            q, k = unit(DK ** -0.5), unit(1.0)
            v = torch.randn(n * DK, device="cuda", generator=gs).to(torch.bfloat16)
            g = torch.nn.functional.logsigmoid(torch.randn(n * DK, device="cuda", generator=gs) + 3.0)
            beta = torch.sigmoid(torch.randn(n, device="cuda", generator=gs))
            core.decode_batch(heads, rows, cu, q, k, v, g, beta, arena[l * slots * per:(l + 1) * slots * per], off, state_out=None, flags=flags,
                              out=out[l * rows * heads * DV:], saves=(ks[l * nkv:], vs[l * nkv:], gsv[l * nkv:], bs[l * nb:]))
        torch.cuda.synchronize()
        assert core.device_status() == 0
        core.commit_batch(heads, layers, cu, keeps, arena, slots * per, off, (ks, vs, gsv, bs), nkv, nb)
        torch.cuda.synchronize()
        assert core.device_status() == 0
        arenas[flags], outs[flags] = arena, out.float()
    assert torch.equal(arenas[0].view(torch.int16), arenas[core.TENSOR].view(torch.int16))
    diff = (outs[core.TENSOR] - outs[0])
    assert float(diff.abs().max()) <= OUT_MAX_ABS
    assert float(diff.norm() / outs[0].norm()) <= OUT_REL_L2


def test_calls_the_chunked_verify_cannot_take_run_the_exact_form(env, oracle):
    """f32 states, a written state or fused norms: the flag is ignored and the results are the exact verify's bits."""
    G, core, pkg = env
    heads, lens = 2, [5, 16]
    rows, per = sum(lens), heads * DV * DK
    tok = pkg.synth.tokens(4, 9, rows, heads)
    states = np.concatenate([pkg.synth.state(4, 9, s, heads) for s in range(2)])
    cu = np.concatenate([[0], np.cumsum(lens)])
    d_off = G.dev_i64([0, per])
    a, sa = verify(G, core, heads, cu, tok, G.dev_f32(states), d_off, 0)
    b, sb = verify(G, core, heads, cu, tok, G.dev_f32(states), d_off, core.TENSOR)   # f32 states
    assert np.array_equal(G.bits(a), G.bits(b)) and all(np.array_equal(x.view(np.uint8), y.view(np.uint8)) for x, y in zip(sa, sb))
