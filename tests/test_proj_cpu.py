"""The projection GEMM's oracle against the reference's own host model of its GEMV, on the reference test's generator
and shapes (crates/glm53f-forward/tests/gemv.rs:20-40, 104-143), and the host mirror's checks.  No GPU."""
import importlib

import numpy as np
import pytest

import gemm_oracle as go


def test_generator_is_splitmix64():
    # SplitMix64 from state 0: the published first outputs
    r = go.Rng(0)
    assert [hex(int(v)) for v in r._next(3)] == ["0xe220a8397b1dcdaf", "0x6e789e6aa1b965f4", "0x6c45d188009454f"]


@pytest.mark.parametrize("n,k,ksplit", [(64, 4096, 4), (40, 1536, 1), (24, 128, 1)])
def test_oracle_agrees_with_the_reference_gemv_model(n, k, ksplit):
    """The exact sum and the GEMV's f32 order (lanes, butterfly, K splits) agree within the bound the reference puts
    between its GEMV and cuBLAS (gemv.rs:199-201)."""
    rng = go.Rng(11)
    w = rng.bf16s(n * k, 0.02).reshape(1, n, k)
    x = rng.bf16s(8 * k, 1.0).reshape(1, 8, k)
    exact = go.gemm(x, w, True)[0]
    model = go.gemv_model(x[0], w[0], ksplit)
    assert go.rel_rms(model, exact) < 1e-5
    assert go.rel_rms(go.gemv_model(x[0], w[0], 1), model) < 1e-5
    # bf16 outputs are the rounded f32 values
    assert (go.gemm(x, w, False)[0] == go.bf16_widen(go.bf16_bits(exact))).all()


def test_bf16_rounding_is_nearest_even():
    f = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38], np.float32)
    assert go.bf16_bits(f).tolist() == [0x3F80, 0x3F80, 0x3F82, 0xC020, 0x7F7F]


def test_host_mirror_rejects_small_buffers(pkg):
    torch = pytest.importorskip("torch")
    proj = importlib.import_module("glm53f-afd_b200.proj")
    w = proj.Bf16Mat.dense(torch.zeros(64, 128, dtype=torch.bfloat16))
    assert (w.n, w.k, w.ld, w.groups, w.bytes()) == (64, 128, 128, 1, 64 * 128 * 2)
    g = proj.Bf16Mat.dense(torch.zeros(2, 64, 128, dtype=torch.bfloat16))
    assert (g.groups, g.gstride) == (2, 64 * 128)
    x = torch.zeros(4, 128, dtype=torch.bfloat16)
    out = torch.zeros(4, 64, dtype=torch.bfloat16)
    proj.bf16(x, 128, 0, w, 0, out, 64, 0)  # no rows: nothing happens, as Gemm::bf16
    with pytest.raises(proj.Invalid, match="smaller"):
        proj.bf16(x, 128, 0, w, 5, out, 64, 0)
    with pytest.raises(proj.Invalid, match="smaller"):
        proj.bf16(x, 128, 0, w, 4, out[:3], 64, 0)
    with pytest.raises(proj.Invalid, match="bf16"):
        proj.bf16(x.float(), 128, 0, w, 4, out, 64, 0)
    assert proj.KDA_P_COLS == 24_640
