"""The C-ABI library loads without a GPU and exports exactly what include/glm53f_kda.h declares (no compute calls).

Mirrors the reference crate's provenance test (crates/glm53f-kda/tests/provenance.rs:41-69): the header and the
bindings must list the same functions, thirteen of them the reference's."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "glm53f_kda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(glm53f_kda_\w+)\s*\(", text)))


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


def test_missing_library_fails_loudly(pkg, tmp_path):
    import pytest

    with pytest.raises(RuntimeError, match="no CPU fallback"):
        pkg.ffi.load(str(tmp_path / "libglm53f_kda.so"))
