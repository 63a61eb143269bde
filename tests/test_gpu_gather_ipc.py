"""The head-sharded prefill with its all-gather done by the kernels, set up through the C ABI alone: two processes (one
rank each), each allocates its full output buffer, exports it (glm53f_kda_gather_export), opens the other's
(glm53f_kda_gather_open) and launches glm53f_kda_core_prefill_varlen_ws_gather on its half of the heads with both
addresses.  Afterwards both full buffers must hold the unsharded run's outputs, bit for bit (heads never interact).
The ranks use different GPUs when the box has two, else they share GPU 0 (the launches do not wait on one another: each
only stores, and the processes meet at host barriers around the launch).
"""
import ctypes as C
import multiprocessing as mp
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DK = 128
HEADS, LENS = 4, [200, 65, 0, 130]


def rank_main(rank, ranks, to_peer, from_peer, barrier, results):
    try:
        sys.path.insert(0, ROOT)
        import importlib

        import torch

        torch.cuda.set_device(rank % torch.cuda.device_count())
        pkg = importlib.import_module("glm53f-afd_b200")
        lib = pkg.ffi.load()
        P = lambda t: C.c_void_p(t.data_ptr())
        rows, batch, per = sum(LENS), len(LENS), HEADS * DK * DK
        q, k, v, g, beta = pkg.synth.tokens(2, 21, rows, HEADS)
        states = np.concatenate([pkg.synth.state(2, 21, i, HEADS) for i in range(batch)])
        bits = lambda b: torch.from_numpy(np.ascontiguousarray(b).view(np.int16).copy()).cuda()
        dq, dk, dv, dg, db = bits(q), bits(k), bits(v), torch.from_numpy(g).cuda(), torch.from_numpy(beta).cuda()
        cu = torch.tensor(np.concatenate([[0], np.cumsum(LENS)]), dtype=torch.int32, device="cuda")
        # the unsharded run, for comparison
        st = torch.from_numpy(states.copy()).cuda()
        off = torch.arange(batch, dtype=torch.int64, device="cuda") * per
        want = torch.zeros(rows * HEADS * DK, dtype=torch.int16, device="cuda")
        nb = lib.glm53f_kda_core_prefill_workspace_bytes(HEADS, batch, 4)
        ws = torch.empty(nb, dtype=torch.uint8, device="cuda")
        assert lib.glm53f_kda_core_prefill_varlen_ws(HEADS, batch, P(cu), max(LENS), P(dq), P(dk), P(dv), P(dg), P(db), P(st), P(st), P(off), 0, 0,
                                                     None, None, 1e-5, P(want), P(ws), nb, None) == 0
        # this rank's shard
        h0, hn = C.c_int32(), C.c_int32()
        assert lib.glm53f_kda_gather_head_range(HEADS, rank, ranks, C.byref(h0), C.byref(hn)) == 0
        h0, hn = h0.value, hn.value
        cut = lambda t, w: t.view(rows, HEADS, w)[:, h0:h0 + hn].contiguous().view(-1)
        sq, sk, sv, sg, sb = cut(dq, DK), cut(dk, DK), cut(dv, DK), cut(dg, DK), cut(db, 1)
        s_state = torch.from_numpy(np.concatenate([states[i * per + h0 * DK * DK: i * per + (h0 + hn) * DK * DK] for i in range(batch)]).copy()).cuda()
        s_off = torch.arange(batch, dtype=torch.int64, device="cuda") * (hn * DK * DK)
        # the full buffer, its handle out, the peer's handle in
        full = torch.full((rows * HEADS * DK + 64,), -1, dtype=torch.int16, device="cuda")
        mine = (C.c_ubyte * 128)()
        assert lib.glm53f_kda_gather_export(P(full), rows * HEADS * DK * 2, mine) == 0
        to_peer.put(bytes(mine))
        theirs = (C.c_ubyte * 128).from_buffer_copy(from_peer.get(timeout=120))
        mapped, nbytes = C.c_void_p(), C.c_int64()
        assert lib.glm53f_kda_gather_open(theirs, C.byref(mapped), C.byref(nbytes)) == 0
        assert nbytes.value == rows * HEADS * DK * 2
        addrs = [None, None]
        addrs[rank], addrs[1 - rank] = full.data_ptr(), mapped.value
        arr = (C.c_void_p * 2)(*addrs)
        torch.cuda.synchronize()
        barrier.wait(timeout=120)   # both buffers exist, are filled with the canary and mapped
        rc = lib.glm53f_kda_core_prefill_varlen_ws_gather(hn, batch, P(cu), max(LENS), P(sq), P(sk), P(sv), P(sg), P(sb), P(s_state), P(s_state), P(s_off),
                                                          0, 0, None, None, 1e-5, None, P(ws), nb, C.cast(arr, C.c_void_p), 2, HEADS, h0, None)
        assert rc == 0
        torch.cuda.synchronize()
        assert lib.glm53f_kda_device_status() == 0
        barrier.wait(timeout=120)   # both ranks' rows have landed everywhere
        ok = bool(torch.equal(full[:rows * HEADS * DK], want)) and bool((full[rows * HEADS * DK:] == -1).all())
        whole = st.view(batch, HEADS, DK * DK)[:, h0:h0 + hn].reshape(-1)
        ok_state = bool(torch.equal(s_state, whole))
        barrier.wait(timeout=120)   # nobody unmaps a buffer another rank may still be comparing... or storing to
        assert lib.glm53f_kda_gather_close(theirs, mapped) == 0
        barrier.wait(timeout=120)   # unmapped everywhere before any exporter frees its allocation
        results.put((rank, ok, ok_state, ""))
    except Exception as e:  # the parent reports it
        import traceback

        results.put((rank, False, False, traceback.format_exc()))
        try:
            barrier.abort()
        except Exception:
            pass


def test_two_processes_gather_through_the_c_abi():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    ctx = mp.get_context("spawn")
    q01, q10, results, barrier = ctx.Queue(), ctx.Queue(), ctx.Queue(), ctx.Barrier(2)
    procs = [ctx.Process(target=rank_main, args=(0, 2, q01, q10, barrier, results)),
             ctx.Process(target=rank_main, args=(1, 2, q10, q01, barrier, results))]
    for p in procs:
        p.start()
    got = [results.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, ok, ok_state, err in sorted(got):
        assert err == "", f"rank {rank}:\n{err}"
        assert ok, f"rank {rank}: its full buffer differs from the unsharded run"
        assert ok_state, f"rank {rank}: its states differ from the unsharded run's"
