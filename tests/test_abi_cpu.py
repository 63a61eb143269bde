"""The C-ABI library loads without a GPU and exports exactly what include/*.h declare (no compute calls).

Mirrors the reference crate's provenance test (crates/glm53f-kda/tests/provenance.rs:41-69): the header and the
bindings must list the same functions, thirteen of them the reference's."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    names = set()
    for header in ("glm53f_kda.h", "glm53f_fwd_rows.h", "glm53f_proj.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(glm53f_(?:kda|fwd)_\w+)\s*\(", text))
    return sorted(names)


def test_header_bindings_and_library_agree(pkg):
    pkg.build()
    names = declared()
    assert sorted(pkg.ffi.SIGNATURES) == names
    assert len(pkg.ffi.REFERENCE_SYMBOLS) == 13
    lib = pkg.ffi.load()
    for n in names:
        assert getattr(lib, n) is not None


def test_host_side_rejections_need_no_gpu(pkg):
    lib = pkg.ffi.load()
    # The launchers validate before they touch the device: status 1 = rejected on the host.
    assert lib.glm53f_kda_prefill_workspace_bytes(64, 1, 16) == 34816 * 64
    assert lib.glm53f_kda_prefill_workspace_bytes(0, 1, 16) == 0
    assert lib.glm53f_kda_conv_shift(0, 0, None, None, 0, None) == 1
    assert lib.glm53f_kda_replay(0, 0, None, None, None, None, None, None, None) == 1
    a = 4096  # a stand-in for a device address: never dereferenced when a check rejects
    args = [a, 24640, 24576, a, 8192, a, 8192, a, a, a, a, a, 1, a, a, a, 1e-5, -5.0, a, 8192, None]
    assert lib.glm53f_kda_chain_commit_batch(64, 2, a, None, *args) == 1   # a commit names the rows each request keeps
    assert lib.glm53f_kda_chain_commit_batch(0, 2, a, a, *args) == 1


def test_row_movers_reject_on_the_host_like_the_reference(pkg):
    """kernels/glue.cu:222-233: layout errors are cudaErrorInvalidValue (1) before any launch; nothing to move is 0."""
    import ctypes as C

    lib = pkg.ffi.load()
    a, b = 4096, 8192  # stand-ins for 16-byte aligned device addresses: never dereferenced on these paths
    for fn in (lib.glm53f_fwd_gather_rows, lib.glm53f_fwd_scatter_rows):
        assert fn(a, 64, a, b, 48, 0, 48, None) == 0       # no rows
        assert fn(a, 64, a, b, 48, 3, 0, None) == 0        # no bytes
        assert fn(a, 64, a, b, 48, -1, 48, None) == 1
        assert fn(a, 64, a, b, 48, 3, -16, None) == 1
        assert fn(a, 64, a, b, 48, 3, 40, None) == 1       # bytes not a multiple of 16
        assert fn(a, 72, a, b, 48, 3, 48, None) == 1       # stride not a multiple of 16
        assert fn(a, 64, a, b, 32, 3, 48, None) == 1       # stride below the row
        assert fn(a + 8, 64, a, b, 48, 3, 48, None) == 1   # pointer not aligned
        assert fn(a, 64, None, b, 48, 3, 48, None) == 1    # no index list
    parts = (C.c_void_p * 3)(a, a, a)
    sizes = (C.c_int64 * 3)(0, 0, 0)
    assert lib.glm53f_kda_mark_copy(a, 1024, a, parts, sizes, 1, None) == 0    # an empty mark
    assert lib.glm53f_kda_mark_copy(a, 1000, a, parts, sizes, 1, None) == 1    # page size not a multiple of 16
    sizes = (C.c_int64 * 3)(32, 8, 0)
    assert lib.glm53f_kda_mark_copy(a, 1024, a, parts, sizes, 1, None) == 1    # part size not a multiple of 16
    sizes = (C.c_int64 * 3)(32, 16, 0)
    assert lib.glm53f_kda_mark_copy(a, 1024, None, parts, sizes, 1, None) == 1  # no page list
    assert lib.glm53f_kda_mark_copy(None, 1024, a, parts, sizes, 1, None) == 1
    strides = (C.c_int64 * 3)(64, 16, 16)
    assert lib.glm53f_kda_mark_copy_slots(a, 1024, a, parts, sizes, strides, a, 0, 1, None) == 0     # no marks
    assert lib.glm53f_kda_mark_copy_slots(a, 1024, a, parts, sizes, None, a, 2, 1, None) == 1        # no strides
    assert lib.glm53f_kda_mark_copy_slots(a, 1024, a, parts, sizes, strides, None, 2, 1, None) == 1  # no slot list
    assert lib.glm53f_kda_mark_copy_slots(a, 1024, a, parts, sizes, (C.c_int64 * 3)(16, 16, 16), a, 2, 1, None) == 1  # slots overlap
    assert lib.glm53f_kda_mark_copy_slots(a, 1024, a, parts, sizes, strides, a, -1, 1, None) == 1


def test_missing_library_fails_loudly(pkg, tmp_path):
    import pytest

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        pkg.ffi.load(str(tmp_path / "libglm53f_kda.so"))


def test_projection_gemm_rejects_on_the_host(pkg):
    lib = pkg.ffi.load()
    a = 4096  # a stand-in for an aligned device address: never dereferenced on these paths
    ok = dict(x=a, ldx=4096, xg=0, w=a, ldw=4096, wg=0, groups=1, rows=0, n=64, k=4096, out=a, f32=0, ldo=64, og=0)

    def call(**kw):
        v = {**ok, **kw}
        return lib.glm53f_kda_proj_bf16(v["x"], v["ldx"], v["xg"], v["w"], v["ldw"], v["wg"], v["groups"], v["rows"], v["n"], v["k"],
                                        v["out"], v["f32"], v["ldo"], v["og"], None)

    assert call() == 0                 # no rows: nothing to do
    assert call(rows=-1) == 1
    assert call(groups=0) == 1
    assert call(k=4000) == 1           # k not a multiple of 64
    assert call(k=0) == 1
    assert call(n=60) == 1             # n not a multiple of 8
    assert call(ldx=4100) == 1 and call(ldw=4100) == 1
    assert call(ldx=2048) == 1         # a row stride below k
    assert call(ldo=32) == 1           # an output stride below n
    assert call(groups=2, xg=12) == 1  # group stride not a multiple of 8
    assert call(rows=4, x=a + 8) == 1 and call(rows=4, w=a + 2) == 1
    assert call(rows=4, x=None) == 1 and call(rows=4, out=None) == 1
