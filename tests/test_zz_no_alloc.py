"""The prefill entry point that allocates nothing, through the C ABI.

`glm53f_kda_core_prefill_varlen_static` exists for hosts that cannot hand the library a workspace because they
cannot allocate one: every byte of device memory was planned away before the first request, or the call sits where
cudaMalloc would fail or disturb the host (an allocator lock held, a latency-critical loop).  It runs the two-pass
prefill on a fixed scratch array inside the library.  The first call on a device is the set-up call (the CUDA runtime
may load the library's device image, the scratch array with it, only then; the array's address is looked up): a host
makes it once, early, on a small shape, before its memory plan is final and outside any stream capture -- as this test
does first.  Then the entry point is called twice in a row on different inputs and must give the bits
of the workspace entry point (same kernels, same arithmetic; only where the scratch lives differs), which in turn
is held to the task's tolerances against the oracle.  The file sorts last so that a `-x` run has run everything else
first; it also passes alone in a fresh process.
"""
import ctypes as C
import importlib

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = 128


def test_static_scratch_prefill_matches_the_workspace_entry_point_twice(oracle):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    pkg = importlib.import_module("glm53f-afd_b200")
    lib = pkg.ffi.load()
    heads, lens = 4, [200, 0, 65, 300]
    batch, rows = len(lens), sum(lens)
    per = heads * DK * DK
    P = lambda t: C.c_void_p(t.data_ptr())
    dev_bits = lambda b: torch.from_numpy(np.ascontiguousarray(b).view(np.int16).copy()).cuda()
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    off = torch.arange(batch, dtype=torch.int64, device="cuda") * per
    # the set-up call a host makes once per device: one chain, one row
    z16, zf = torch.zeros(DK, dtype=torch.int16, device="cuda"), torch.zeros(DK, device="cuda")
    st1, cu1 = torch.zeros(DK * DK, device="cuda"), torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    rc = lib.glm53f_kda_core_prefill_varlen_static(1, 1, P(cu1), 1, P(z16), P(z16), P(z16), P(zf), P(zf), P(st1), P(st1), P(off), 0, 0,
                                                   None, None, 1e-5, P(torch.zeros(DK, dtype=torch.int16, device="cuda")), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert lib.glm53f_kda_device_status() == 0
    for call in range(2):  # two calls in a row share the scratch array: the second must not see the first
        q, k, v, g, beta = pkg.synth.tokens(2, 10 + call, rows, heads)
        s0 = np.concatenate([pkg.synth.state(2, 10 + call, i, heads) for i in range(batch)])
        dq, dk, dv = dev_bits(q), dev_bits(k), dev_bits(v)
        dg, db = torch.from_numpy(g).cuda(), torch.from_numpy(beta).cuda()
        results = []
        for which in ("static", "workspace"):
            st = torch.from_numpy(s0.copy()).cuda()
            out = torch.zeros(rows * heads * DK, dtype=torch.int16, device="cuda")
            if which == "static":
                rc = lib.glm53f_kda_core_prefill_varlen_static(heads, batch, P(cu), max(lens), P(dq), P(dk), P(dv), P(dg), P(db), P(st), P(st),
                                                               P(off), 0, 0, None, None, 1e-5, P(out), None)
            else:
                nbytes = lib.glm53f_kda_core_prefill_workspace_bytes(heads, batch, 3)
                ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
                rc = lib.glm53f_kda_core_prefill_varlen_ws(heads, batch, P(cu), max(lens), P(dq), P(dk), P(dv), P(dg), P(db), P(st), P(st),
                                                           P(off), 0, 0, None, None, 1e-5, P(out), P(ws), nbytes, None)
            assert rc == 0, (which, rc)
            torch.cuda.synchronize()
            assert lib.glm53f_kda_device_status() == 0
            results.append((out.cpu().numpy(), st.cpu().numpy()))
        assert np.array_equal(results[0][0], results[1][0]), f"call {call}: outputs differ"
        assert np.array_equal(results[0][1].view(np.uint32), results[1][1].view(np.uint32)), f"call {call}: states differ"
        # and the result itself is right: the first sequence against the FP32 recurrence, at the task's tolerances
        n = lens[0]
        part = lambda a, w: a.reshape(rows, heads * w)[:n].reshape(-1)
        y, s_ref = oracle.core_forward(heads, part(q, DK), part(k, DK), part(v, DK), part(g, DK), beta.reshape(rows, heads)[:n].reshape(-1),
                                       s0[:per], form="recurrent", threads=4)
        got = oracle.bf16_widen(results[0][0].view(np.uint16)).reshape(rows, heads * DK)[:n].reshape(-1)
        assert np.max(np.abs(got - y)) <= 2e-2
        assert np.linalg.norm(got - y) / np.linalg.norm(y) <= 5e-3
        assert np.linalg.norm(results[0][1][:per] - s_ref) / np.linalg.norm(s_ref) <= 1e-3
    # more chains than the scratch can serve: rejected on the host, nothing enqueued
    big = torch.zeros(8, dtype=torch.int16, device="cuda")
    rc = lib.glm53f_kda_core_prefill_varlen_static(64, 2, P(cu), 1, P(big), P(big), P(big), P(big), P(big), P(big), P(big), P(off), 0, 0,
                                                   None, None, 1e-5, P(big), None)
    assert rc == 1
