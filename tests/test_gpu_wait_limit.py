"""The failure path of the decode kernel, exercised without a fault: a device-side wait that runs out.

Every wait inside the kernels is bounded; when one sees no progress for the limit, the block records which wait gave
up in the library's status word, makes its other waits return, lets copies in flight land and ends.  The hook
`glm53f_kda_debug_wait_test` shortens the limit to a millisecond and makes block 0 of the next launch leave its first
unit's state unfetched (nothing is issued, nothing is in flight), so that unit's wait must run out.  What is checked:
the launch returns, the status call reports a wait code (101-108) once and then 0, the launch's other units computed
what a clean launch computes, and the context keeps working (the same launch afterwards gives a clean launch's bits).
No trap, no bad address, no endless loop.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(pkg):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import importlib

    import kda_gpu as G

    core = importlib.import_module("glm53f-afd_b200.core")
    lib = pkg.ffi.load()
    heads, slots = 2, 3   # six units on six blocks: block 0 holds unit 0 = (slot 0, head 0) only
    per = heads * DV * DK
    tok = pkg.synth.tokens(1, 5, slots, heads)
    states = np.concatenate([pkg.synth.state(1, 5, s, heads) for s in range(slots)])
    dq, dk, dv = (G.dev_bits(t) for t in tok[:3])
    dg, db = G.dev_f32(tok[3]), G.dev_f32(tok[4])
    cu, off = G.dev_i32(np.arange(slots + 1)), G.dev_i64([s * per for s in range(slots)])

    def launch():
        st = G.dev_f32(states)
        out = torch.zeros(slots * heads * DV, dtype=torch.int16, device="cuda")
        # with the L2 norms fused: that call runs the persistent kernel, the one with device-side waits (and its prologue
        # meets at barriers in every row, so the vote that keeps a role together after a wait gave up is on the path)
        core.decode_batch(heads, slots, cu, dq, dk, dv, dg, db, st, off, out=out, flags=core.L2NORM)
        torch.cuda.synchronize()
        return out.cpu().numpy().reshape(slots * heads, DV), st.cpu().numpy().reshape(slots * heads, DV * DK)

    assert lib.glm53f_kda_debug_wait_test(50_000, 0) == 1          # a limit below 0.1 ms is refused
    clean_out, clean_st = launch()
    assert core.device_status() == 0
    assert lib.glm53f_kda_debug_wait_test(1_000_000, 1) == 0       # 1 ms; the next launch's unit 0 never gets its state
    try:
        out, st = launch()
        code = core.device_status()
        assert 101 <= code <= 108, code
        assert core.device_status() == 0                           # read once, then clear
        # the other five units are a clean launch's; unit 0's state was not written
        assert np.array_equal(out[1:], clean_out[1:]) and np.array_equal(st[1:].view(np.uint32), clean_st[1:].view(np.uint32))
        assert np.array_equal(st[0].view(np.uint32), states.reshape(slots * heads, -1)[0].view(np.uint32))
        # the request was for one launch only: with the short limit still set, a normal launch is clean
        again_out, again_st = launch()
        assert core.device_status() == 0
        assert np.array_equal(again_out, clean_out) and np.array_equal(again_st.view(np.uint32), clean_st.view(np.uint32))
    finally:
        assert lib.glm53f_kda_debug_wait_test(0, 0) == 0           # the default limit again
    final_out, _ = launch()
    assert core.device_status() == 0 and np.array_equal(final_out, clean_out)
