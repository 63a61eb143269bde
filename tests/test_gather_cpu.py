"""The host-side checks of the multi-GPU boundary (glm53f_kda_gather_*): argument rejections and the head ranges need no
GPU (nothing is dereferenced, no CUDA call is made before a rejection)."""
import ctypes as C


def test_head_ranges(pkg):
    lib = pkg.ffi.load()
    h0, n = C.c_int32(-1), C.c_int32(-1)
    for ranks in (1, 2, 4, 8):
        seen = []
        for rank in range(ranks):
            assert lib.glm53f_kda_gather_head_range(64, rank, ranks, C.byref(h0), C.byref(n)) == 0
            seen.append((h0.value, n.value))
        assert seen == [(r * (64 // ranks), 64 // ranks) for r in range(ranks)]   # contiguous, in rank order, all 64 heads
    assert lib.glm53f_kda_gather_head_range(64, 0, 3, C.byref(h0), C.byref(n)) == 1    # 64 heads do not split over 3 ranks
    assert lib.glm53f_kda_gather_head_range(64, 8, 8, C.byref(h0), C.byref(n)) == 1    # rank out of range
    assert lib.glm53f_kda_gather_head_range(64, 0, 16, C.byref(h0), C.byref(n)) == 1   # at most 8 full buffers
    assert lib.glm53f_kda_gather_head_range(64, 0, 2, None, C.byref(n)) == 1


def test_handles_are_checked_before_anything_is_mapped(pkg):
    lib = pkg.ffi.load()
    handle = (C.c_ubyte * 128)()
    mapped, nbytes = C.c_void_p(), C.c_int64()
    assert lib.glm53f_kda_gather_export(None, 1024, handle) == 1
    assert lib.glm53f_kda_gather_export(4096, 0, handle) == 1        # no bytes
    assert lib.glm53f_kda_gather_export(4104, 1024, handle) == 1     # not 16-byte aligned
    assert lib.glm53f_kda_gather_export(4096, 1024, None) == 1
    assert lib.glm53f_kda_gather_open(handle, C.byref(mapped), C.byref(nbytes)) == 1   # 128 zero bytes are not a handle
    assert lib.glm53f_kda_gather_open(None, C.byref(mapped), None) == 1
    assert lib.glm53f_kda_gather_close(handle, 4096) == 1
    assert lib.glm53f_kda_gather_close(handle, None) == 1
