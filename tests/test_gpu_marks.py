"""GPU parity of the row movers and of the state snapshot / restore, through the C ABI.

Byte work: every comparison is exact.  Cases follow the reference's tests: the known-answer gather / scatter of
crates/glm53f-forward/tests/gemv.rs:329-358, and the properties of crates/glm53f-forward/tests/snapshot.rs:66-170
(a mark takes pool pages and gives them back; a restore from host images re-exports the same images; a rewound or
forked slot continues bit for bit)."""
import ctypes as C
import importlib

import numpy as np
import pytest

import rows_oracle as ro

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

DK = DV = 128


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kda_gpu

    kda_gpu.product()
    return kda_gpu


@pytest.fixture(scope="module")
def lib(G):
    return importlib.import_module("glm53f-afd_b200.ffi").load()


@pytest.fixture(scope="module")
def marks(G):
    return importlib.import_module("glm53f-afd_b200.marks")


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_reference_known_answer(lib):
    src = np.array([(i * 7 % 251) for i in range(10 * 64)], np.uint8)
    idx = np.array([7, 2, 9], np.int32)
    ds, dix = dev(src), dev(idx)
    dd = torch.zeros(3 * 48, dtype=torch.uint8, device="cuda")
    back = torch.zeros(10 * 64, dtype=torch.uint8, device="cuda")
    assert lib.glm53f_fwd_gather_rows(ds.data_ptr(), 64, dix.data_ptr(), dd.data_ptr(), 48, 3, 48, stream()) == 0
    assert lib.glm53f_fwd_scatter_rows(dd.data_ptr(), 48, dix.data_ptr(), back.data_ptr(), 64, 3, 48, stream()) == 0
    torch.cuda.synchronize()
    g, b = dd.cpu().numpy(), back.cpu().numpy()
    for i, row in enumerate(idx):
        assert (g[i * 48:(i + 1) * 48] == src[row * 64:row * 64 + 48]).all()
        assert (b[row * 64:row * 64 + 48] == src[row * 64:row * 64 + 48]).all()


# (rows, bytes, src_stride, dst_stride, table rows): one-warp rows, the 4 KiB boundary on both sides, a ragged
# last tile, a pool page, a single row, many small rows.
SHAPES = [
    (3, 16, 16, 16, 8),
    (257, 48, 64, 48, 1000),
    (100, 2048, 2048, 4096, 300),
    (100, 2064, 2080, 2064, 300),
    (50, 4096, 4096, 4112, 128),
    (50, 4112, 4112, 4128, 128),
    (21, 32_768 + 48, 32_768 + 64, 32_768 + 48, 64),
    (37, 16_400, 16_416, 16_400, 64),
    (19, 394_944, 394_944, 394_944, 40),
    (1, 35_904, 35_904 + 160, 35_904, 5),
    (200_000, 64, 64, 80, 250_000),
]


@pytest.mark.parametrize("rows,nbytes,ss,ds,table", SHAPES)
def test_gather_and_scatter_match_the_oracle(lib, rows, nbytes, ss, ds, table):
    rng = np.random.default_rng(rows * 31 + nbytes)
    idx = rng.permutation(table)[:rows].astype(np.int32)
    # gather: the table has `table` rows of stride ss, the result `rows` rows of stride ds
    src = rng.integers(0, 256, table * ss, dtype=np.uint8)
    want = np.full(rows * ds, 0xA5, np.uint8)
    ro.gather_rows(src, ss, idx, want, ds, rows, nbytes)
    d_src, d_idx = dev(src), dev(idx)
    d_dst = torch.full((rows * ds,), 0xA5, dtype=torch.uint8, device="cuda")
    assert lib.glm53f_fwd_gather_rows(d_src.data_ptr(), ss, d_idx.data_ptr(), d_dst.data_ptr(), ds, rows, nbytes, stream()) == 0
    torch.cuda.synchronize()
    assert (d_dst.cpu().numpy() == want).all()  # the gaps between rows keep their fill
    # scatter the gathered rows into a table of stride ss
    want2 = np.full(table * ss, 0x5A, np.uint8)
    ro.scatter_rows(want, ds, idx, want2, ss, rows, nbytes)
    d_back = torch.full((table * ss,), 0x5A, dtype=torch.uint8, device="cuda")
    assert lib.glm53f_fwd_scatter_rows(d_dst.data_ptr(), ds, d_idx.data_ptr(), d_back.data_ptr(), ss, rows, nbytes, stream()) == 0
    torch.cuda.synchronize()
    assert (d_back.cpu().numpy() == want2).all()


def test_nothing_to_move_launches_nothing(lib):
    t = torch.zeros(64, dtype=torch.uint8, device="cuda")
    i = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert lib.glm53f_fwd_gather_rows(t.data_ptr(), 16, i.data_ptr(), t.data_ptr(), 16, 0, 16, stream()) == 0
    assert lib.glm53f_fwd_scatter_rows(t.data_ptr(), 16, i.data_ptr(), t.data_ptr(), 16, 4, 0, stream()) == 0
    assert lib.glm53f_fwd_gather_rows(t.data_ptr() + 8, 16, i.data_ptr(), t.data_ptr(), 16, 1, 16, stream()) == 1
    torch.cuda.synchronize()


@pytest.mark.parametrize("layout", [(1, 2, True), (2, 1, False), (1, 0, True)])
def test_mark_copy_matches_the_oracle(lib, marks, layout):
    kda_layers, dsa_layers, bf16 = layout
    l = marks.KvLayout.new(kda_layers, dsa_layers).with_kda_state_bf16(bf16)
    pb = l.page_bytes
    rng = np.random.default_rng(17 + kda_layers)
    sizes = [r[1] for r in l.mark_regions()]
    parts = [rng.integers(0, 256, n, dtype=np.uint8) for n in sizes]
    n_pages = l.mark_pages()
    total = n_pages + 11
    page_list = sorted(rng.permutation(total)[:n_pages].tolist())
    pool = rng.integers(0, 256, total * pb, dtype=np.uint8)
    want_pool = pool.copy()
    ro.copy_mark(want_pool, pb, page_list, parts, True)
    d_pool, d_idx = dev(pool), dev(np.array(page_list, np.int32))
    d_parts = [dev(p) if p.size else torch.zeros(16, dtype=torch.uint8, device="cuda") for p in parts]
    ptrs = (C.c_void_p * 3)(*[t.data_ptr() for t in d_parts])
    nb = (C.c_int64 * 3)(*sizes)
    assert lib.glm53f_kda_mark_copy(d_pool.data_ptr(), pb, d_idx.data_ptr(), ptrs, nb, 1, stream()) == 0
    torch.cuda.synchronize()
    assert (d_pool.cpu().numpy() == want_pool).all()  # pages outside the mark and the rest of partial pages untouched
    # and back out into cleared arenas, each followed by a guard
    d_back = [torch.full((n + 64,), 0x77, dtype=torch.uint8, device="cuda") for n in sizes]
    ptrs = (C.c_void_p * 3)(*[t.data_ptr() for t in d_back])
    assert lib.glm53f_kda_mark_copy(d_pool.data_ptr(), pb, d_idx.data_ptr(), ptrs, nb, 0, stream()) == 0
    torch.cuda.synchronize()
    for t, p in zip(d_back, parts):
        got = t.cpu().numpy()
        assert (got[:p.size] == p).all() and (got[p.size:] == 0x77).all()


@pytest.mark.parametrize("bf16", [True, False])
def test_full_model_mark_rewind_fork_and_host_images(marks, bf16):
    """The whole model's positional state (73 MiB with bf16 states, 141 MiB with f32), fused and as the reference's
    sequence of launches: same pool bytes, same images; pages are taken and given back."""
    l = marks.KvLayout.glm53_flash().with_kda_state_bf16(bf16)
    need = l.mark_pages()
    assert need == (195 if bf16 else 376)
    pools = [marks.KvPool(marks.KvConfig(l, 2, 2 * need + 5), fused=f) for f in (True, False)]
    g = torch.Generator(device="cuda").manual_seed(3)
    images = []
    for pool in pools:
        g.manual_seed(3)
        a = pool.slot()
        for arena, at, n in ((pool.state, a._state_at(), l.kda_state_bytes()), (pool.conv, a._conv_at(), l.conv_bytes()),
                             (pool.tails, a._tails_at(), l.tails_bytes())):
            arena.t[at:at + n] = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda", generator=g)
        # tail counts 0..3 and beyond, little endian in the first 4 bytes of each tail
        for j in range(l.dsa_layers):
            at = a._tails_at() + j * marks.TAIL
            pool.tails.t[at:at + 4] = torch.tensor([j % 5, 0, 0, 0], dtype=torch.uint8, device="cuda")
        a.advance(72)
        free0 = pool.free_pages()
        m = a.mark()
        assert (m.tokens, m.pages(), m.bytes(), pool.free_pages()) == (72, need, l.mark_bytes(), free0 - need)
        before = [arena.t[at:at + n].clone() for arena, at, n in
                  ((pool.state, a._state_at(), l.kda_state_bytes()), (pool.conv, a._conv_at(), l.conv_bytes()),
                   (pool.tails, a._tails_at(), l.tails_bytes()))]
        image = a.export_state(m)
        want = np.concatenate([t.cpu().numpy() for t in before])
        marks.zero_stale_tail_slots(want, l)
        assert (image == want).all()
        assert (image == ro.export_state(pool.pages.t.cpu().numpy(), l.page_bytes, m.page_list(),
                                         [r[1] for r in l.mark_regions()], l.dsa_layers)).all()
        # the slot moves on, then rewinds
        a.advance(3)
        pool.state.t[a._state_at():a._state_at() + l.kda_state_bytes()] ^= 0xFF
        pool.conv.t[a._conv_at():a._conv_at() + l.conv_bytes()].zero_()
        pool.tails.t[a._tails_at():a._tails_at() + l.tails_bytes()].zero_()
        a.rewind(72, m)
        assert a.tokens() == 72
        for t, (arena, at) in zip(before, a._arenas()):
            assert torch.equal(arena.t[at:at + t.numel()], t)
        # a fork and a restore from the host image into the other slot
        b = pool.slot()
        b.fork(a, 72, m)
        assert b.tokens() == 72
        for t, (arena, at) in zip(before, b._arenas()):
            assert torch.equal(arena.t[at:at + t.numel()], t)
        b.reset()
        b.advance(72)
        b.import_state(72, image)
        mb = b.mark()
        assert (b.export_state(mb) == image).all()
        assert (b.download_state(33).view(np.uint32) == a.download_state(33).view(np.uint32)).all()  # as bits: random bytes hold NaNs
        assert (b.download_conv(5) == a.download_conv(5)).all()
        mb.drop()
        m.drop()
        assert pool.free_pages() == free0
        images.append((image, pool.pages.t[:need * l.page_bytes].cpu().numpy()))
    assert (images[0][0] == images[1][0]).all()
    assert (images[0][1] == images[1][1]).all()  # fused and unfused wrote the same pool bytes


def test_a_rewound_slot_continues_bit_for_bit(G, marks):
    """Decode steps on a slot's states in the pool arena, a mark, more steps, a rewind, the same steps again: the
    outputs and the states repeat exactly (snapshot.rs:118-125 on the KDA core)."""
    core = importlib.import_module("glm53f-afd_b200.core")
    synth = importlib.import_module("glm53f-afd_b200.synth")
    H, layers = 64, 2
    l = marks.KvLayout.new(layers, 1).with_kda_state_bf16(True)
    pool = marks.KvPool(marks.KvConfig(l, 2, 2 * l.mark_pages()))
    pool.slot()            # slot 0 stays idle: the test's slot is not at offset 0
    a = pool.slot()
    state = pool.state.t.view(torch.bfloat16)
    per_layer = marks.KvLayout.state_elems_per_layer()
    cu = torch.tensor([0, 1], dtype=torch.int32, device="cuda")

    def step(i):
        outs = []
        for layer in range(layers):
            q, k, v, gl, beta = synth.tokens(1, layer * 100 + i, 1, H)
            off = torch.tensor([a.state_elem_offset() + layer * per_layer], dtype=torch.int64, device="cuda")
            out = torch.zeros(H * DV, dtype=torch.int16, device="cuda")
            core.decode_batch(H, 1, cu, G.dev_bits(q), G.dev_bits(k), G.dev_bits(v), G.dev_f32(gl), G.dev_f32(beta), state, off, out=out)
            outs.append(out)
        a.advance(1)
        return torch.stack(outs)

    for i in range(3):
        step(i)
    m = a.mark()
    first = [step(i) for i in range(3, 6)]
    after = pool.state.t[a._state_at():a._state_at() + l.kda_state_bytes()].clone()
    a.rewind(3, m)
    again = [step(i) for i in range(3, 6)]
    G.check_status()
    assert all(torch.equal(x, y) for x, y in zip(first, again))
    assert torch.equal(pool.state.t[a._state_at():a._state_at() + l.kda_state_bytes()], after)
    assert after.any()


@pytest.mark.parametrize("bf16", [True, False])
def test_marks_of_several_slots_in_one_launch(marks, bf16):
    """mark_many / rewind_many (one launch for all slots) write and restore the bytes of slot-by-slot marks."""
    l = marks.KvLayout.new(2, 3).with_kda_state_bf16(bf16)
    need = l.mark_pages()
    pool = marks.KvPool(marks.KvConfig(l, 5, 8 * need + 3))
    g = torch.Generator(device="cuda").manual_seed(11)
    for arena in (pool.state, pool.conv, pool.tails):
        arena.t.copy_(torch.randint(0, 256, (arena.t.numel(),), dtype=torch.uint8, device="cuda", generator=g))
    kvs = [pool.slot() for _ in range(5)]
    for arena in (pool.state, pool.conv, pool.tails):  # slot() zeroes a slot's state: fill again
        arena.t.copy_(torch.randint(0, 256, (arena.t.numel(),), dtype=torch.uint8, device="cuda", generator=g))
    for i, kv in enumerate(kvs):
        kv.advance(10 + i)
    # interleave allocations so that the marks' pages are scattered, then take marks of slots 4, 1, 3 in one launch
    spare = [pool.alloc.alloc() for _ in range(7)]
    for p in spare[::2]:
        pool.alloc.release(p)
    chosen = [kvs[4], kvs[1], kvs[3]]
    free0 = pool.free_pages()
    batch = pool.mark_many(chosen)
    assert pool.free_pages() == free0 - 3 * need and [m.tokens for m in batch] == [14, 11, 13]
    single = [kv.mark() for kv in chosen]
    pool.stream.synchronize()
    pages = pool.pages.t.cpu().numpy().reshape(-1, l.page_bytes)
    for mb, ms in zip(batch, single):
        sizes = [r[1] for r in l.mark_regions()]
        a = ro.export_state(pages.reshape(-1), l.page_bytes, mb.page_list(), sizes, 0)
        b = ro.export_state(pages.reshape(-1), l.page_bytes, ms.page_list(), sizes, 0)
        assert (a == b).all()
    before = [arena.t.clone() for arena in (pool.state, pool.conv, pool.tails)]
    for kv in chosen:
        kv.advance(2)
        pool.state.t[kv._state_at():kv._state_at() + l.kda_state_bytes()].zero_()
        pool.conv.t[kv._conv_at():kv._conv_at() + l.conv_bytes()] ^= 0x55
        pool.tails.t[kv._tails_at():kv._tails_at() + l.tails_bytes()].zero_()
    pool.rewind_many(chosen, batch)
    pool.stream.synchronize()
    for arena, want in zip((pool.state, pool.conv, pool.tails), before):
        assert torch.equal(arena.t, want)  # the chosen slots are back, the others were never touched
    assert [kv.tokens() for kv in chosen] == [14, 11, 13]
    with pytest.raises(marks.Invalid, match="same slot twice"):
        pool.mark_many([kvs[0], kvs[0]])
    with pytest.raises(marks.OutOfMemory):
        pool.mark_many(kvs)
    assert pool.mark_many([]) == []
