"""CPU restatement of the reference's row gather / scatter and of its mark copy and state image.  TEST INFRASTRUCTURE
ONLY: the checker the CUDA row movers are compared with; nothing in the product imports it.

Restated from the reference (numpy on bytes, bit-exact by construction):

  gather_rows / scatter_rows   crates/glm53f-forward/kernels/glue.cu:101-110 (the kernel), 222-244 (checks, entry points)
  copy_mark                    crates/glm53f-forward/src/kv.rs:412-476 (whole pages by index list, the partial last
                               page of each part by a plain copy)
  export_state                 kv.rs:623-664 (page runs into the image; tail slots past each tail's count zeroed)
  mark_regions                 crates/glm53f-forward/src/kvplan.rs:113-126

Pinned by the reference's own known-answer test of the two kernels (crates/glm53f-forward/tests/gemv.rs:329-358:
10 rows of 64 bytes, byte i = i * 7 % 251, rows 7, 2, 9 gathered as 48-byte rows and scattered back) and by the
layout numbers of crates/glm53f-forward/tests/kv_plan.rs:31-97 (tests/test_marks_cpu.py).
"""
import numpy as np

INVALID = 1  # cudaErrorInvalidValue


def check(src_stride, dst_stride, rows, nbytes):
    """The launcher's layout checks (glue.cu:224-227): 0 = go on, 1 = rejected."""
    if rows < 0 or nbytes < 0 or nbytes % 16 or src_stride % 16 or dst_stride % 16 or src_stride < nbytes or dst_stride < nbytes:
        return INVALID
    return 0


def gather_rows(src, src_stride, idx, dst, dst_stride, rows, nbytes):
    """dst[i] = src[idx[i]] for i < rows, on flat uint8 arrays (glue.cu:101-110 with scatter = 0)."""
    for i in range(rows):
        s, d = int(idx[i]) * src_stride, i * dst_stride
        dst[d:d + nbytes] = src[s:s + nbytes]


def scatter_rows(src, src_stride, idx, dst, dst_stride, rows, nbytes):
    """dst[idx[i]] = src[i] for i < rows (glue.cu:101-110 with scatter = 1)."""
    for i in range(rows):
        s, d = i * src_stride, int(idx[i]) * dst_stride
        dst[d:d + nbytes] = src[s:s + nbytes]


def mark_regions(state_bytes, conv_bytes, tails_bytes, page_bytes):
    """(offset in the host image, bytes, pool pages) of a mark's three parts (kvplan.rs:113-126)."""
    out, off = [], 0
    for n in (state_bytes, conv_bytes, tails_bytes):
        out.append((off, n, -(-n // page_bytes)))
        off += n
    return out


def copy_mark(pages, page_bytes, page_list, parts, save):
    """The parts (flat uint8 arrays: a slot's states, windows, tails) into the mark's pages of `pages` or back
    (kv.rs:412-476): per part its whole pages row by row through the index list, then the remainder."""
    first = 0
    for part in parts:
        n = part.size
        full, rem = divmod(n, page_bytes)
        idx = page_list[first:first + full]
        if save:
            scatter_rows(part, page_bytes, idx, pages, page_bytes, full, page_bytes)
        else:
            gather_rows(pages, page_bytes, idx, part, page_bytes, full, page_bytes)
        if rem:
            at = int(page_list[first + full]) * page_bytes
            if save:
                pages[at:at + rem] = part[full * page_bytes:]
            else:
                part[full * page_bytes:] = pages[at:at + rem]
        first += full + (1 if rem else 0)


def export_state(pages, page_bytes, page_list, sizes, dsa_layers, tail_bytes=1552):
    """The host image of a mark (kv.rs:623-664): the three parts back to back, stale tail slots zeroed."""
    image = np.zeros(sum(sizes), np.uint8)
    first = off = 0
    for n in sizes:
        k = 0
        while k * page_bytes < n:
            at = int(page_list[first + k]) * page_bytes
            m = min(page_bytes, n - k * page_bytes)
            image[off + k * page_bytes:off + k * page_bytes + m] = pages[at:at + m]
            k += 1
        first += k
        off += n
    base = sizes[0] + sizes[1]
    for j in range(dsa_layers):
        t = image[base + j * tail_bytes:base + (j + 1) * tail_bytes]
        count = min(int.from_bytes(t[:4].tobytes(), "little"), 3)
        t[16 + count * 512:] = 0
    return image
