"""The multi-GPU host logic on CPU: world_size-2 gloo processes stand in for two GPUs.

Head-sharded prefill (each rank runs its heads with the oracle's chunk-64 form, then the all-gather) must
reproduce the unsharded result bit for bit; slot sharding must partition the slots exactly."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("glm53f-afd_b200")
        par = importlib.import_module("glm53f-afd_b200.parallel")
        import kda_oracle as o

        heads, t, dk = 4, 70, 128
        q, k, v, g, beta = pkg.synth.tokens(0, 3, t, heads)
        s0 = pkg.synth.state(0, 3, 0, heads)
        full_y, full_s = o.core_forward(heads, q, k, v, g, beta, s0, form="chunked", chunk=64)
        lo, hi = par.head_range(heads, rank, world)
        hl = hi - lo
        sh = lambda a, w: par.shard_heads(torch.from_numpy(a.reshape(t, heads, w).copy()), heads, rank, world).numpy().reshape(-1)
        y_loc, s_loc = o.core_forward(hl, sh(q, dk), sh(k, dk), sh(v, dk), sh(g, dk),
                                      par.shard_heads(torch.from_numpy(beta.reshape(t, heads, 1).copy()), heads, rank, world).numpy().reshape(-1),
                                      s0.reshape(heads, -1)[lo:hi].reshape(-1), form="chunked", chunk=64)
        gathered = par.gather_heads(torch.from_numpy(y_loc.reshape(t, hl, dk)), heads)
        ok_y = np.array_equal(gathered.numpy().reshape(-1).view(np.uint32), full_y.view(np.uint32))
        ok_s = np.array_equal(s_loc.view(np.uint32), full_s.reshape(heads, -1)[lo:hi].reshape(-1).view(np.uint32))
        # slot sharding: the ranks' ranges tile [0, slots) exactly
        rng = torch.tensor(list(par.slot_range(5, rank, world)))
        allr = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(allr, rng)
        ok_slots = allr[0][0].item() == 0 and allr[-1][1].item() == 5 and all(allr[i][1] == allr[i + 1][0] for i in range(world - 1))
        ret[rank] = bool(ok_y and ok_s and ok_slots)
    finally:
        dist.destroy_process_group()


def test_head_sharded_prefill_and_slot_ranges_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_shard_ranges():
    par = importlib.import_module("glm53f-afd_b200.parallel")
    assert [par.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert par.head_range(64, 3, 8) == (24, 32)
    with pytest.raises(ValueError):
        par.head_range(64, 0, 3)
    with pytest.raises(ValueError):
        par.shard_range(4, 4, 4)
