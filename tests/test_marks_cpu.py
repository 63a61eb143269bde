"""Host side of the state snapshot / restore: layout numbers, page accounting, the oracle's pins, error behaviour.

The numbers are the reference's (crates/glm53f-forward/tests/kv_plan.rs:31-97); the row movers' known-answer case is
crates/glm53f-forward/tests/gemv.rs:329-358.  No GPU: nothing here launches."""
import importlib

import numpy as np
import pytest

import rows_oracle as ro


@pytest.fixture(scope="module")
def marks(pkg):
    return importlib.import_module("glm53f-afd_b200.marks")


def test_layout_numbers_of_the_full_model(marks):
    l = marks.KvLayout.glm53_flash()
    assert l.page_bytes == 394_944 == 64 * 6_171
    assert l.kda_state_bytes() == 136 << 20
    assert l.conv_bytes() == 34 * 3 * 24_576 * 2
    assert l.tails_bytes() == 17_072
    assert [r[2] for r in l.mark_regions()] == [362, 13, 1]
    assert [r[0] for r in l.mark_regions()] == [0, l.kda_state_bytes(), l.kda_state_bytes() + l.conv_bytes()]
    assert sum(r[1] for r in l.mark_regions()) == l.mark_bytes()
    assert l.mark_pages() == 376
    assert l.mark_pages() * l.page_bytes >= l.mark_bytes()
    for tokens, pages in [(1, 1), (63, 1), (64, 1), (65, 2), (4096, 64), (1_048_576, 16_384)]:
        assert marks.KvLayout.pages_for(tokens) == pages
        assert l.paged_bytes(tokens) == pages * 394_944
    # the layer prefix of the golden tests: 4 KDA layers and 1 DSA layer
    s5 = marks.KvLayout.new(4, 1)
    assert s5.page_bytes == 35_904
    assert s5.mark_pages() == 468 + 17 + 1


def test_bf16_states_halve_the_state(marks):
    f = marks.KvLayout.glm53_flash()
    b = f.with_kda_state_bf16(True)
    assert (f.kda_state_elem_bytes(), b.kda_state_elem_bytes()) == (4, 2)
    assert b.kda_state_bytes() == 68 << 20
    assert b.conv_bytes() == f.conv_bytes()
    assert b.mark_bytes() == f.mark_bytes() - (68 << 20)
    assert b.slot_fixed_bytes() == f.slot_fixed_bytes() - (68 << 20)
    assert [r[2] for r in b.mark_regions()] == [181, 13, 1]
    assert b.mark_pages() == 195
    # the oracle's regions are the same function
    assert ro.mark_regions(b.kda_state_bytes(), b.conv_bytes(), b.tails_bytes(), b.page_bytes) == b.mark_regions()


def test_page_alloc_hands_out_the_lowest_page_first(marks):
    a = marks.PageAlloc(4)
    assert (a.total(), a.free()) == (4, 4)
    assert [a.alloc(), a.alloc()] == [0, 1]
    a.share(1)
    assert a.refs(1) == 2 and not a.release(1) and a.release(1)
    assert a.alloc() == 1  # the page just freed comes back first
    assert [a.alloc(), a.alloc(), a.alloc()] == [2, 3, None]
    with pytest.raises(AssertionError):
        a.release(0) and a.release(0)


def test_oracle_reproduces_the_reference_known_answer():
    """gemv.rs:329-358."""
    src = np.array([(i * 7 % 251) for i in range(10 * 64)], np.uint8)
    idx = [7, 2, 9]
    assert ro.check(64, 48, 3, 48) == 0
    got = np.zeros(3 * 48, np.uint8)
    ro.gather_rows(src, 64, idx, got, 48, 3, 48)
    back = np.zeros(10 * 64, np.uint8)
    ro.scatter_rows(got, 48, idx, back, 64, 3, 48)
    for i, row in enumerate(idx):
        assert (got[i * 48:(i + 1) * 48] == src[row * 64:row * 64 + 48]).all()
        assert (back[row * 64:row * 64 + 48] == src[row * 64:row * 64 + 48]).all()
    untouched = np.ones(10 * 64, bool)
    for row in idx:
        untouched[row * 64:row * 64 + 48] = False
    assert (back[untouched] == 0).all()
    # first bytes of row 7: (448 + j) * 7 % 251
    assert got[:4].tolist() == [(448 + j) * 7 % 251 for j in range(4)]


def test_oracle_mark_round_trip_and_image(marks):
    l = marks.KvLayout.new(1, 2).with_kda_state_bf16(True)  # small: 2 MiB of state, 2 tails
    pb = l.page_bytes
    rng = np.random.default_rng(5)
    sizes = [r[1] for r in l.mark_regions()]
    parts = [rng.integers(0, 256, n, dtype=np.uint8) for n in sizes]
    # tails: counts 1 and 7 (clamped to 3)
    parts[2][0:4] = np.frombuffer((1).to_bytes(4, "little"), np.uint8)
    parts[2][marks.TAIL:marks.TAIL + 4] = np.frombuffer((7).to_bytes(4, "little"), np.uint8)
    n_pages = l.mark_pages()
    page_list = sorted(rng.permutation(n_pages + 9)[:n_pages].tolist())
    pool = np.zeros((n_pages + 9) * pb, np.uint8)
    ro.copy_mark(pool, pb, page_list, parts, True)
    back = [np.zeros_like(p) for p in parts]
    ro.copy_mark(pool, pb, page_list, back, False)
    assert all((a == b).all() for a, b in zip(parts, back))
    image = ro.export_state(pool, pb, page_list, sizes, l.dsa_layers)
    want = np.concatenate(parts)
    base = sizes[0] + sizes[1]
    want[base + 16 + 512:base + marks.TAIL] = 0  # tail 0 keeps one slot; tail 1's count clamps to 3: all kept
    assert (image == want).all()
    twice = image.copy()
    marks.zero_stale_tail_slots(twice, l)
    assert (twice == image).all()


def test_error_behaviour_needs_no_launch(marks, pkg, monkeypatch):
    kernel = importlib.import_module("glm53f-afd_b200.kernel")
    monkeypatch.setattr(kernel, "DEVICE", "cpu")
    l = marks.KvLayout.new(1, 1).with_kda_state_bf16(True)
    need = l.mark_pages()
    pool = marks.KvPool(marks.KvConfig(l, 2, need - 1))
    other = marks.KvPool(marks.KvConfig(l, 1, 2 * need))
    with pytest.raises(marks.Invalid):
        marks.KvPool(marks.KvConfig(l, 0, 4))
    a, b = pool.slot(), pool.slot()
    assert (a.slot_index(), b.slot_index(), pool.free_slots()) == (0, 1, 0)
    with pytest.raises(marks.OutOfMemory, match="all 2 KV slots"):
        pool.slot()
    with pytest.raises(marks.OutOfMemory, match=f"takes {need} pages"):
        a.mark()
    assert pool.free_pages() == need - 1  # nothing was allocated
    a.pending = 3
    with pytest.raises(marks.Invalid, match="uncommitted verify window"):
        a.mark()
    a.pending = 0
    foreign = marks.KvMark(0, [], other)
    with pytest.raises(marks.Invalid, match="another pool"):
        a.rewind(0, foreign)
    mine = marks.KvMark(5, [], pool)
    with pytest.raises(marks.Invalid, match="rewind to 4 with a mark at 5"):
        a.rewind(4, mine)
    with pytest.raises(marks.Invalid, match="the slot holds 0"):
        a.rewind(5, mine)
    with pytest.raises(marks.Invalid, match="fork across pools"):
        a.fork(other.slot(), 0, foreign)
    with pytest.raises(marks.Invalid, match="fork of 5 tokens"):
        a.fork(b, 5, mine)
    with pytest.raises(marks.Invalid, match="import_state"):
        a.import_state(0, np.zeros(l.mark_bytes() - 16, np.uint8))
    with pytest.raises(marks.Invalid, match="import_state"):
        a.import_state(3, np.zeros(l.mark_bytes(), np.uint8))
    assert a.state_elem_offset() == 0 and b.state_elem_offset() == l.kda_state_bytes() // 2
    assert b.conv_elem_offset() == l.conv_bytes() // 2 and b.tail_row(0) == 1
    b.release()
    assert pool.free_slots() == 1
