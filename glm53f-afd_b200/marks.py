"""Snapshot and restore of a slot's positional state (KDA states, conv windows, DSA tails): what makes prefix caching,
rewind and fork work with a recurrent state.

Mirror of the positional-state half of the reference's device KV, over include/glm53f_fwd_rows.h:

  KvLayout   crates/glm53f-forward/src/kvplan.rs:42-148   byte accounting, a mark's three regions and its pool pages
  PageAlloc  kvplan.rs:150-204                             reference counts and the free list (lowest page first)
  KvConfig   crates/glm53f-forward/src/kv.rs:58-71
  KvPool     kv.rs:85-227                                  the page pool and the per-slot arenas
  KvMark     kv.rs:207-236                                 a saved state: pool pages, given back when dropped
  GlmKv      kv.rs:238-330, 385-575, 623-664, 692-720, 744-783   a slot: mark, rewind, fork, host images, downloads

Names, argument meaning and error behaviour are the reference's (`Invalid` = Error::Invalid, `OutOfMemory` =
Error::OutOfMemory).  The paged half of the KV (page tables, copy-on-write of DSA pages, the drafter's ring) belongs
to the attention layers and is not built: `rewind` and `fork` here move the positional state only, and `tokens`
is advanced by whoever runs the KDA kernels on the slot (`GlmKv.advance`).

A mark is copied by one launch of `glm53f_kda_mark_copy`; `KvPool(fused=False)` issues the reference's sequence
instead (one row scatter or gather per region plus a copy of each partial last page, kv.rs:412-476) - same bytes.
Device memory is torch's; there is no CPU copy path: without the CUDA library every copy raises.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, replace
from typing import Optional

import numpy as np

from . import ffi, kernel
from .core import CudaError, Invalid
from .kernel import DeviceBuffer, Stream

LAYER_PAGE_BYTES = 35_904  # one DSA layer's 64-token block (crates/glm53f-dsa/src/cache.rs:58)
PAGE = 64                  # tokens per page (cache.rs:48)
TAIL = 1_552               # one DSA layer's tail record: 16 + 3 x 512 (cache.rs:64)
KDA_HEADS, KDA_DIM = 64, 128
KDA_QKV = 3 * KDA_HEADS * KDA_DIM  # 24,576 (crates/glm53f-forward/src/shape.rs:23-32)
KDA_WINDOW = 3


class OutOfMemory(RuntimeError):
    """The reference's Error::OutOfMemory: the pool has too few free pages or slots; nothing was allocated."""


@dataclass(frozen=True)
class KvLayout:
    """Byte layout of the device KV for a model shape (kvplan.rs:42-148)."""

    kda_layers: int
    dsa_layers: int
    page_bytes: int
    draft_kv_bytes: int = 0
    kda_state_bf16: bool = False

    @classmethod
    def new(cls, kda_layers: int, dsa_layers: int, draft_kv_bytes: int = 0) -> "KvLayout":
        return cls(kda_layers, dsa_layers, max(dsa_layers, 1) * LAYER_PAGE_BYTES, draft_kv_bytes, False)

    @classmethod
    def glm53_flash(cls) -> "KvLayout":
        """The full model: 34 KDA layers and 11 DSA layers (crates/glm53f-forward/tests/kv_plan.rs:22-68)."""
        return cls.new(34, 11)

    def with_kda_state_bf16(self, bf16: bool) -> "KvLayout":
        return replace(self, kda_state_bf16=bool(bf16))

    @staticmethod
    def state_elems_per_layer() -> int:
        return KDA_HEADS * KDA_DIM * KDA_DIM

    def kda_state_elem_bytes(self) -> int:
        return 2 if self.kda_state_bf16 else 4

    @staticmethod
    def conv_elems_per_layer() -> int:
        return KDA_WINDOW * KDA_QKV

    def kda_state_bytes(self) -> int:
        return self.kda_layers * self.state_elems_per_layer() * self.kda_state_elem_bytes()

    def conv_bytes(self) -> int:
        return self.kda_layers * self.conv_elems_per_layer() * 2

    def tails_bytes(self) -> int:
        return self.dsa_layers * TAIL

    def mark_bytes(self) -> int:
        return self.kda_state_bytes() + self.conv_bytes() + self.tails_bytes()

    def mark_regions(self) -> list[tuple[int, int, int]]:
        """A mark's three parts: (offset in its host image, bytes, pool pages), each part from a page of its own."""
        pb = self.page_bytes
        s, c, t = self.kda_state_bytes(), self.conv_bytes(), self.tails_bytes()
        return [(0, s, -(-s // pb)), (s, c, -(-c // pb)), (s + c, t, -(-t // pb))]

    def mark_pages(self) -> int:
        return sum(r[2] for r in self.mark_regions())

    def slot_fixed_bytes(self) -> int:
        return self.mark_bytes() + self.draft_kv_bytes

    @staticmethod
    def pages_for(tokens: int) -> int:
        return -(-tokens // PAGE)

    def paged_bytes(self, tokens: int) -> int:
        return self.pages_for(tokens) * self.page_bytes


class PageAlloc:
    """Reference counts and the free list of a pool of physical pages (kvplan.rs:150-204)."""

    def __init__(self, pages: int):
        self._free = list(range(pages - 1, -1, -1))  # popped from the end: the lowest page first
        self._refs = [0] * pages

    def total(self) -> int:
        return len(self._refs)

    def free(self) -> int:
        return len(self._free)

    def refs(self, page: int) -> int:
        return self._refs[page]

    def alloc(self) -> Optional[int]:
        if not self._free:
            return None
        p = self._free.pop()
        assert self._refs[p] == 0
        self._refs[p] = 1
        return p

    def share(self, page: int) -> None:
        assert self._refs[page] > 0, "sharing a free page"
        self._refs[page] += 1

    def release(self, page: int) -> bool:
        assert self._refs[page] > 0, "releasing a free page"
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False


@dataclass(frozen=True)
class KvConfig:
    """How big the pool is (kv.rs:58-71; the page-table widths belong to the paged half and are not kept)."""

    layout: KvLayout
    max_slots: int
    pages: int


def _launched(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 1:
        raise Invalid(f"{what}: rejected by the launcher")
    raise CudaError(code, what)


class KvPool:
    """The page pool and the per-slot arenas of the positional state (kv.rs:85-227)."""

    def __init__(self, cfg: KvConfig, stream: Optional[Stream] = None, fused: bool = True):
        if cfg.max_slots <= 0:
            raise Invalid("max_slots must be positive")
        l = cfg.layout
        self.cfg = cfg
        self.stream = stream or Stream()
        self.fused = fused
        self.pages = DeviceBuffer.zeroed(cfg.pages * l.page_bytes)
        self.state = DeviceBuffer.zeroed(cfg.max_slots * l.kda_state_bytes())
        self.conv = DeviceBuffer.zeroed(cfg.max_slots * l.conv_bytes())
        self.tails = DeviceBuffer.zeroed(cfg.max_slots * max(l.tails_bytes(), 16))
        self.mark_index = DeviceBuffer.alloc(max(l.mark_pages(), 1) * 4)
        self.alloc = PageAlloc(cfg.pages)
        self._free_slots = list(range(cfg.max_slots - 1, -1, -1))

    def config(self) -> KvConfig:
        return self.cfg

    def free_pages(self) -> int:
        return self.alloc.free()

    def free_slots(self) -> int:
        return len(self._free_slots)

    def bytes(self) -> int:
        return self.pages.bytes()

    # ---- several slots in one launch (an addition: the reference marks slot by slot) -------------------------------
    def _copy_marks(self, kvs, marks_, save: bool) -> None:
        torch = kernel._torch()
        l = self.cfg.layout
        if any(m._pool is not self or kv.pool is not self for kv, m in zip(kvs, marks_)):
            raise Invalid("a mark or a slot of another pool")
        if len({kv.slot for kv in kvs}) != len(kvs):
            raise Invalid("the same slot twice in one batch")
        n = len(kvs)
        lists = torch.tensor([m._pages for m in marks_], dtype=torch.int32).reshape(-1).to(self.pages.t.device)
        slots = torch.tensor([kv.slot for kv in kvs], dtype=torch.int32).to(self.pages.t.device)
        arenas = (C.c_void_p * 3)(self.state.as_ptr(), self.conv.as_ptr(), self.tails.as_ptr())
        sizes = (C.c_int64 * 3)(*[r[1] for r in l.mark_regions()])
        strides = (C.c_int64 * 3)(l.kda_state_bytes(), l.conv_bytes(), max(l.tails_bytes(), 16))
        _launched(ffi.load().glm53f_kda_mark_copy_slots(self.pages.as_ptr(), l.page_bytes, lists.data_ptr(), arenas, sizes, strides, slots.data_ptr(),
                                                        n, 1 if save else 0, self.stream.raw()), "mark pages")
        self._keep = (lists, slots)  # alive until the next batch: the launch reads them in stream order

    def mark_many(self, kvs) -> list:
        """A mark of every slot of `kvs` (each as GlmKv.mark), copied by one launch; OutOfMemory before anything is
        allocated when the pool has too few free pages for all of them."""
        if any(kv.pending != 0 for kv in kvs):
            raise Invalid("mark inside an uncommitted verify window")
        need = self.cfg.layout.mark_pages()
        if self.alloc.free() < need * len(kvs):
            raise OutOfMemory(f"{len(kvs)} snapshot marks take {need * len(kvs)} pages of the KV pool, {self.alloc.free()} are free")
        out = [KvMark(kv.tokens(), sorted(self.alloc.alloc() for _ in range(need)), self) for kv in kvs]
        if kvs:
            self._copy_marks(kvs, out, True)
        return out

    def rewind_many(self, kvs, marks_) -> None:
        """GlmKv.rewind(mark.tokens, mark) for every (slot, mark), the states restored by one launch."""
        if len(kvs) != len(marks_):
            raise Invalid("one mark per slot")
        for kv, m in zip(kvs, marks_):
            if m.tokens > kv.tokens():
                raise Invalid(f"rewind to {m.tokens} with a mark at {m.tokens} (the slot holds {kv.tokens()})")
        if kvs:
            self._copy_marks(kvs, marks_, False)
        for kv, m in zip(kvs, marks_):
            kv._tokens = m.tokens
            kv.pending = 0

    def slot(self) -> "GlmKv":
        """A new empty slot, or OutOfMemory when every slot is taken (kv.rs:174-200)."""
        if not self._free_slots:
            raise OutOfMemory(f"all {self.cfg.max_slots} KV slots are taken")
        kv = GlmKv(self, self._free_slots.pop())
        kv._clear_state()
        return kv


class KvMark:
    """A slot's positional state at `tokens`, held in pages of the pool (kv.rs:207-236).  `drop()` (or garbage
    collection) gives the pages back."""

    def __init__(self, tokens: int, pages: list[int], pool: KvPool):
        self.tokens = tokens
        self._pages = pages
        self._pool = pool

    def bytes(self) -> int:
        return self._pool.cfg.layout.mark_bytes()

    def pages(self) -> int:
        return len(self._pages)

    def page_list(self) -> list[int]:
        return list(self._pages)

    def drop(self) -> None:
        for p in self._pages:
            self._pool.alloc.release(p)
        self._pages = []

    def __del__(self):
        try:
            self.drop()
        except Exception:
            pass


class GlmKv:
    """One request's positional state on the device (kv.rs:238-330, 385-575, 623-720, 744-783)."""

    def __init__(self, pool: KvPool, slot: int):
        self.pool = pool
        self.slot = slot
        self._tokens = 0
        self.pending = 0  # rows of an uncommitted verify window

    def layout(self) -> KvLayout:
        return self.pool.cfg.layout

    def slot_index(self) -> int:
        return self.slot

    def tokens(self) -> int:
        return self._tokens

    def advance(self, rows: int) -> None:
        """`rows` more tokens were committed into the slot's state by the KDA kernels."""
        self._tokens += int(rows)

    def mark_bytes(self) -> int:
        return self.layout().mark_pages() * self.layout().page_bytes

    def state_bytes(self) -> int:
        return self.layout().mark_bytes()

    def reset(self) -> None:
        self._tokens = 0
        self.pending = 0
        self._clear_state()

    def release(self) -> None:
        """Drop every token and give the slot back to the pool."""
        self.reset()
        self.pool._free_slots.append(self.slot)

    # ---- regions ----------------------------------------------------------------------------------------------
    def _state_at(self) -> int:
        return self.slot * self.layout().kda_state_bytes()

    def _conv_at(self) -> int:
        return self.slot * self.layout().conv_bytes()

    def _tails_at(self) -> int:
        return self.slot * max(self.layout().tails_bytes(), 16)

    def state_elem_offset(self) -> int:
        """Element offset of the slot's KDA states (all layers) in the state arena: what the kernels' `state_off` takes."""
        return self._state_at() // self.layout().kda_state_elem_bytes()

    def conv_elem_offset(self) -> int:
        return self._conv_at() // 2

    def tail_row(self, dsa_layer: int) -> int:
        return self._tails_at() // TAIL + dsa_layer

    def _clear_state(self) -> None:
        l, p = self.layout(), self.pool
        p.state.t[self._state_at():self._state_at() + l.kda_state_bytes()].zero_()
        p.conv.t[self._conv_at():self._conv_at() + l.conv_bytes()].zero_()
        p.tails.t[self._tails_at():self._tails_at() + l.tails_bytes()].zero_()

    def _arenas(self):
        p = self.pool
        return [(p.state, self._state_at()), (p.conv, self._conv_at()), (p.tails, self._tails_at())]

    # ---- the copy ---------------------------------------------------------------------------------------------
    def _copy_mark(self, mark: KvMark, save: bool) -> None:
        """The positional state into `mark`'s pages (`save`) or out of them into the slot (kv.rs:412-476)."""
        if mark._pool is not self.pool:
            raise Invalid("a mark of another pool")
        torch = kernel._torch()
        l, p = self.layout(), self.pool
        pb = l.page_bytes
        n_idx = len(mark._pages)
        # The list buffer is reused in stream order.
        p.mark_index.t[:n_idx * 4].view(torch.int32).copy_(torch.tensor(mark._pages, dtype=torch.int32))
        lib = ffi.load()
        s = p.stream.raw()
        if p.fused:
            parts = (C.c_void_p * 3)(*[a.as_ptr() + at for a, at in self._arenas()])
            sizes = (C.c_int64 * 3)(*[n for _, n, _ in l.mark_regions()])
            _launched(lib.glm53f_kda_mark_copy(p.pages.as_ptr(), pb, p.mark_index.as_ptr(), parts, sizes, 1 if save else 0, s), "mark pages")
            return
        first = 0
        for (arena, at), (_, n, pages) in zip(self._arenas(), l.mark_regions()):
            full, rem = divmod(n, pb)
            if full > 0:
                idx = p.mark_index.as_ptr() + first * 4
                if save:
                    rc = lib.glm53f_fwd_scatter_rows(arena.as_ptr() + at, pb, idx, p.pages.as_ptr(), pb, full, pb, s)
                else:
                    rc = lib.glm53f_fwd_gather_rows(p.pages.as_ptr(), pb, idx, arena.as_ptr() + at, pb, full, pb, s)
                _launched(rc, "mark pages")
            if rem > 0:
                page = mark._pages[first + full] * pb
                if save:
                    p.pages.t[page:page + rem].copy_(arena.t[at + full * pb:at + full * pb + rem])
                else:
                    arena.t[at + full * pb:at + full * pb + rem].copy_(p.pages.t[page:page + rem])
            first += pages

    # ---- marks, rewind, fork ----------------------------------------------------------------------------------
    def mark(self) -> KvMark:
        """Save the positional state at the current position in pages of the pool; OutOfMemory when the pool has too
        few free pages (nothing is allocated then), kv.rs:482-509."""
        if self.pending != 0:
            raise Invalid("mark inside an uncommitted verify window")
        need = self.layout().mark_pages()
        a = self.pool.alloc
        if a.free() < need:
            raise OutOfMemory(f"a snapshot mark takes {need} pages of the KV pool, {a.free()} are free")
        pages = sorted(a.alloc() for _ in range(need))
        mark = KvMark(self._tokens, pages, self.pool)
        self._copy_mark(mark, True)
        return mark

    def rewind(self, to: int, mark: KvMark) -> None:
        """Go back to `to` tokens, where `mark` was taken in this slot's history (kv.rs:511-538)."""
        if mark.tokens != to or to > self._tokens:
            raise Invalid(f"rewind to {to} with a mark at {mark.tokens} (the slot holds {self._tokens})")
        self._copy_mark(mark, False)
        self._tokens = to
        self.pending = 0

    def fork(self, src: "GlmKv", to: int, mark: KvMark) -> None:
        """Become `src`'s first `to` tokens at `mark` (taken by `src` at `to`), kv.rs:541-575."""
        if src.pool is not self.pool:
            raise Invalid("fork across pools")
        if mark.tokens != to or to > src._tokens:
            raise Invalid(f"fork of {to} tokens with a mark at {mark.tokens} from a slot of {src._tokens}")
        self.reset()
        self._copy_mark(mark, False)
        self._tokens = to

    # ---- host images ------------------------------------------------------------------------------------------
    def export_state(self, mark: KvMark) -> np.ndarray:
        """`mark`'s positional state as a host image of `state_bytes()` bytes.  The tail slots past each tail's count
        are zeroed, so the image depends only on the committed tokens (kv.rs:623-664)."""
        if mark._pool is not self.pool:
            raise Invalid(f"state image: the mark holds {mark.bytes()} bytes (or is another pool's)")
        l, p = self.layout(), self.pool
        pb = l.page_bytes
        p.stream.synchronize()
        dst = np.zeros(l.mark_bytes(), np.uint8)
        first = 0
        for off, n, pages in l.mark_regions():
            k = 0
            while k < pages:  # runs of consecutive pages in one copy
                run = 1
                while k + run < pages and mark._pages[first + k + run] == mark._pages[first + k] + run:
                    run += 1
                nbytes = min(n - k * pb, run * pb)
                at = mark._pages[first + k] * pb
                dst[off + k * pb:off + k * pb + nbytes] = p.pages.t[at:at + nbytes].cpu().numpy()
                k += run
            first += pages
        zero_stale_tail_slots(dst, l)
        return dst

    def import_state(self, tokens: int, src) -> None:
        """Finish a restore of `tokens` tokens: load the positional state image (kv.rs:692-720)."""
        l = self.layout()
        src = np.ascontiguousarray(src).view(np.uint8).reshape(-1)
        if tokens != self._tokens or src.size != l.mark_bytes():
            raise Invalid(f"import_state({tokens}) after {self._tokens} imported rows, {src.size} bytes")
        torch = kernel._torch()
        off = 0
        for (arena, at), (_, n, _) in zip(self._arenas(), l.mark_regions()):
            arena.t[at:at + n].copy_(torch.from_numpy(src[off:off + n].copy()))
            off += n

    # ---- downloads (tests) --------------------------------------------------------------------------------------
    def download_state(self, j: int) -> np.ndarray:
        """KDA layer j's state as f32 [64][128 (v)][128 (k)] (a BF16 state widened), kv.rs:761-773."""
        self.pool.stream.synchronize()
        n = KvLayout.state_elems_per_layer()
        at = self.state_elem_offset() + j * n
        if self.layout().kda_state_bf16:
            b = self.pool.state.download(np.uint16, n, at)
            return (b.astype(np.uint32) << 16).view(np.float32)
        return self.pool.state.download(np.float32, n, at)

    def download_conv(self, j: int) -> np.ndarray:
        self.pool.stream.synchronize()
        n = KvLayout.conv_elems_per_layer()
        return self.pool.conv.download(np.uint16, n, self.conv_elem_offset() + j * n)

    def download_tail(self, j: int) -> np.ndarray:
        self.pool.stream.synchronize()
        return self.pool.tails.download(np.uint8, TAIL, self.tail_row(j) * TAIL)


def zero_stale_tail_slots(image: np.ndarray, l: KvLayout) -> None:
    """In a state image, zero each DSA tail's slots past its count (the first 4 bytes, little endian, at most 3):
    keys of a pool that has since completed (kv.rs:653-662)."""
    base = l.kda_state_bytes() + l.conv_bytes()
    for j in range(l.dsa_layers):
        t = image[base + j * TAIL:base + (j + 1) * TAIL]
        n = min(int.from_bytes(t[:4].tobytes(), "little"), 3)
        t[16 + n * 512:] = 0
