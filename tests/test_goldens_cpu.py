"""The golden-fixture loader (glm53f-afd_b200/goldens.py, the mirror of crates/glm53f-kda/src/goldens.rs) on the CPU:
the name classification cases of the reference's own unit tests (goldens.rs:1316-1370), set loading with digest and
size verification, grouping by layer, the comparison's tolerance rule, and the reference repository's own manifests
(names, shapes and digests are committed there; the payloads are not)."""
import importlib
import os

import numpy as np
import pytest

REFERENCE_GOLDENS = os.path.join(os.environ.get("GLM53F_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference"), "oracle", "goldens")


@pytest.fixture(scope="module")
def G():
    return importlib.import_module("glm53f-afd_b200.goldens")


def test_classifies_names(G):
    R = G.Role
    assert G.classify("layers.4.kda.q", None) == (4, R.Q)
    assert G.classify("model.language_model.layers.4.self_attn.A_log", None) == (4, R.ALog)
    assert G.classify("model.language_model.layers.0.self_attn.forget_gate.dt_bias", None) == (0, R.DtBias)
    assert G.classify("model.language_model.layers.0.self_attn.q_conv1d.weight", None) == (0, R.ConvWQ)
    assert G.classify("L06.kda.core_out", None) == (6, R.CoreOut)
    assert G.classify("prefill.kda.q", 4) == (4, R.Q)            # the oracle's names: the layer comes from the set
    assert G.classify("decode.kda.state", 0) == (0, R.StateOut)
    assert G.classify("decode.s3.kda.q", 0) is None              # per-step tensors are not used
    assert G.classify("layers.3.kda.q", None) is None            # layer 3 is full attention
    assert G.classify("prefill.kda.q", None) is None             # no layer anywhere
    assert G.classify("layers.4.kda.unknown", None) is None
    assert [i for i in range(12) if G.is_kda_layer(i)] == [0, 1, 2, 4, 5, 6, 8, 9, 10] and not G.is_kda_layer(45)


def test_dtype_names(G):
    assert G.DType.parse("torch.bfloat16") is G.DType.BF16 and G.DType.parse("FLOAT") is G.DType.F32 and G.DType.parse("bool") is G.DType.U8
    assert G.DType.parse("complex64") is None
    assert [d.size() for d in (G.DType.F64, G.DType.F32, G.DType.BF16, G.DType.I64, G.DType.U8)] == [8, 4, 2, 8, 1]


def make_set(G, root, name="layer04-prefill"):
    d = os.path.join(root, name)
    rng = np.random.default_rng(5)
    G.write_set(d, [("prefill.kda.q", G.DType.BF16, [3, 2, 128], rng.standard_normal(768)),
                    ("prefill.kda.beta", G.DType.F32, [3, 2], rng.random(6)),
                    ("prefill.kda.state", G.DType.F32, [2, 128, 128], rng.standard_normal(2 * 128 * 128)),
                    ("prefill.tokens", G.DType.I32, [3], [5, 6, 7])], notes={"state_heads": [1]})
    return d


def test_set_round_trip_and_verification(G, tmp_path):
    d = make_set(G, str(tmp_path))
    s = G.Set.load(d)
    assert s.name() == "layer04-prefill" and s.layer_phase() == (4, G.Phase.Prefill) and s.state_heads() == [1]
    s.verify_all()
    q = s.read("prefill.kda.q")
    assert q.dtype is G.DType.BF16 and q.shape == [3, 2, 128] and q.data.dtype == np.float32
    assert np.array_equal(G._f32_to_bf16(q.data), np.frombuffer(s.bytes("prefill.kda.q"), "<u2"))   # widened exactly
    assert s.read("prefill.tokens").data.tolist() == [5.0, 6.0, 7.0]
    lfs = G.kda_layers(s)
    assert len(lfs) == 1 and lfs[0].layer == 4 and lfs[0].phase is G.Phase.Prefill
    assert lfs[0].name(G.Role.Q) == "prefill.kda.q" and lfs[0].name(G.Role.StateOut) == "prefill.kda.state" and not lfs[0].has(G.CORE_ROLES)
    assert G.discover(str(tmp_path)) == [d] and G.discover(os.path.join(str(tmp_path), "nope")) == []
    with pytest.raises(G.GoldenError) as e:
        s.read("prefill.kda.k")
    assert e.value.kind == "missing"
    # a flipped byte, then a truncated payload
    path = os.path.join(d, "prefill.kda.beta.bin")
    raw = bytearray(open(path, "rb").read())
    raw[3] ^= 1
    open(path, "wb").write(bytes(raw))
    with pytest.raises(G.GoldenError) as e:
        s.bytes("prefill.kda.beta")
    assert e.value.kind == "digest"
    open(path, "wb").write(bytes(raw[:-4]))
    with pytest.raises(G.GoldenError) as e:
        s.verify_all()
    assert e.value.kind == "size"


def test_manifest_rejections(G, tmp_path):
    d = str(tmp_path / "bad")
    os.makedirs(d)
    for body, kind in (("[1, 2]", "manifest"), ("{", "json"), ('{"t": {"file": "../x.bin", "dtype": "f32", "shape": [1], "sha256": "00"}}', "manifest"),
                       ('{"t": {"file": "x.bin", "dtype": "q7", "shape": [1], "sha256": "00"}}', "manifest"),
                       ('{"t": {"file": "x.bin", "dtype": "f32", "shape": [-1], "sha256": "00"}}', "manifest")):
        open(os.path.join(d, "manifest.json"), "w").write(body)
        with pytest.raises(G.GoldenError) as e:
            G.Set.load(d)
        assert e.value.kind == kind, body
    with pytest.raises(G.GoldenError) as e:
        G.Set.load(str(tmp_path / "absent"))
    assert e.value.kind == "io"


def test_comparison_rule(G):
    want = np.array([1.0, -2.0, 0.5], np.float32)
    c = G.Comparison.compare("x", want + np.array([0.0, 1e-4, 0.0], np.float32), want, G.TOL_F32)
    assert c.passes() and c.differing == 1 and c.max_ref == 2.0
    assert not G.Comparison.compare("x", want + np.float32(1e-3), want, G.TOL_F32).passes()
    assert G.Comparison.compare("x", want + np.float32(1e-3), want, G.TOL_RECURRENT).passes()
    assert not G.Comparison.compare("x", np.array([np.nan, 0, 0], np.float32), want, 1.0).passes()
    tiny = np.zeros(4, np.float32)
    assert G.Comparison.compare("x", tiny + 5e-8, tiny, G.TOL_F32).passes()       # relative to at least 1e-3
    assert G.Comparison.compare("x", [1.0, 1.0078125], [1.0, 1.0], 1.0).max_ulp == 1
    assert G.tolerance(G.DType.F32, False) == 1e-4 and G.tolerance(G.DType.BF16, True) == 1e-2 and G.tolerance(G.DType.BF16, False) == 5e-2
    ok = G.Comparison.compare("a", want, want, 1e-4)
    bad = G.Comparison.compare("b", want + 1, want, 1e-4)
    assert G.verdict([ok]) and not G.verdict([ok, bad])
    bad.weight = G.Weight.Informational
    assert G.verdict([ok, bad])


@pytest.mark.skipif(not os.path.isdir(REFERENCE_GOLDENS), reason="the reference checkout is not on this machine")
def test_the_reference_repositorys_own_manifests_load(G):
    sets = G.discover(REFERENCE_GOLDENS)
    assert len(sets) >= 6
    seen = 0
    for d in sets:
        s = G.Set.load(d)
        for lf in G.kda_layers(s):
            if lf.has(G.CORE_ROLES):
                seen += 1
                e = s.entry(lf.name(G.Role.Q))
                assert e.shape[-1] == 128 and len(e.sha256) == 64
        if s.entries:
            with pytest.raises(G.GoldenError) as e:   # the payloads are not in the repository
                s.bytes(s.entries[0].name)
            assert e.value.kind == "io"
    assert seen >= 3
