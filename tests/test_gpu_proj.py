"""GPU parity of the projections' tcgen05 GEMM through the C ABI.

The bound is the reference's own for a GEMM against its GEMV (crates/glm53f-forward/tests/gemv.rs:199-201): relative
RMS below 1e-5 on f32 outputs; bf16 outputs are the rounded f32 results, so they sit within one bf16 step of the
rounded oracle.  Row independence (gemv.rs:144-170: a row's result never depends on the launch's other rows) is held
bit for bit across every row count up to 128 (one row tile)."""
import importlib

import numpy as np
import pytest

import gemm_oracle as go

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_RMS = 1e-5


@pytest.fixture(scope="module")
def proj():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import kda_gpu

    kda_gpu.product()
    return importlib.import_module("glm53f-afd_b200.proj")


def dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()


def status():
    return importlib.import_module("glm53f-afd_b200.core").device_status()


def run(proj, x, w, rows, f32_out, ldo=None, pad=0):
    """x [groups][rows][k], w [groups][n][k] bf16 bits, dense -> f32 [groups][rows][n]."""
    groups, n, k = w.shape
    ldo = ldo or n
    mat = proj.Bf16Mat(dev(w), n, k, k, groups, n * k)
    out = torch.full((groups * rows * ldo + pad,), 7.0 if f32_out else 0x4141, dtype=torch.float32 if f32_out else torch.int16, device="cuda")
    proj.bf16(dev(x[:, :rows]), k, rows * k, mat, rows, out, ldo, rows * ldo, f32_out)
    torch.cuda.synchronize()
    assert status() == 0
    o = out.cpu().numpy()
    guard = o[groups * rows * ldo:]
    body = o[:groups * rows * ldo].reshape(groups, rows, ldo)
    assert (guard == (7.0 if f32_out else 0x4141)).all() and (body[:, :, n:] == (7.0 if f32_out else 0x4141)).all()
    body = body[:, :, :n]
    return body.copy() if f32_out else go.bf16_widen(body.view(np.uint16))


def bf16_step(wb, want):
    """One bf16 step at the value's exponent (at most), plus the f32 accumulation's share for results that cancel to
    near zero, where a bf16 step is smaller than the sum's own rounding."""
    return np.abs(wb) * 2.0 ** -7 + REL_RMS * np.sqrt(np.mean(np.square(want)))


def check(got, x, w, f32_out):
    want = go.gemm(x[:, :got.shape[1]], w, True)
    if f32_out:
        assert go.rel_rms(got, want) < REL_RMS
    else:
        wb = go.bf16_widen(go.bf16_bits(want))
        assert (np.abs(got - wb) <= bf16_step(wb, want)).all()
        assert (got != wb).mean() < 2e-2  # only results that sit on a rounding boundary move


# The reference test's shapes (gemv.rs:104-110): (groups, n, k, f32 output).
@pytest.mark.parametrize("groups,n,k,f32_out", [(1, 64, 4096, False), (1, 288, 4096, True), (1, 1024, 1536, False), (2, 512, 128, False),
                                                (1, 4096, 4096, True)])
def test_reference_shapes_and_row_independence(proj, groups, n, k, f32_out):
    rng = go.Rng(11)
    w = rng.bf16s(groups * n * k, 0.02).reshape(groups, n, k)
    x = rng.bf16s(8 * groups * k, 1.0).reshape(8, groups, k).transpose(1, 0, 2).copy()
    all8 = run(proj, x, w, 8, f32_out)
    check(all8, x, w, f32_out)
    for rows in range(1, 8):
        part = run(proj, x, w, rows, f32_out)
        assert (part.view(np.uint32) == all8[:, :rows].view(np.uint32)).all(), f"rows of {rows} differ from the same rows of 8"


def test_every_tile_shape_gives_a_row_the_same_bits(proj):
    """Row counts that select each row-tile width (16, 32, 64, 128, 256) and ragged last tiles, n with a partial
    feature tile, output rows wider than n, guards."""
    rng = go.Rng(12)
    groups, n, k, R = 1, 328, 512, 300
    w = rng.bf16s(n * k, 0.05).reshape(1, n, k)
    x = rng.bf16s(R * k, 1.0).reshape(1, R, k)
    full = run(proj, x, w, R, True, ldo=n + 8, pad=64)
    check(full, x, w, True)
    # Up to 128 rows (one row tile) the tile shape and the K split are functions of (n, k) alone: a row's bits never
    # depend on the row count.  (This shape splits k over clusters of 2: 3 feature tiles would leave the GPU idle.)
    small = run(proj, x, w, 128, True, ldo=n + 8, pad=64)
    check(small, x, w, True)
    for rows in (1, 15, 16, 17, 31, 32, 33, 64, 65, 127):
        part = run(proj, x, w, rows, True, ldo=n + 24, pad=32)
        assert (part.view(np.uint32) == small[:, :rows].view(np.uint32)).all(), rows
    for rows in (129, 256, 257):
        check(run(proj, x, w, rows, True, ldo=n + 24, pad=32), x, w, True)
    b = run(proj, x, w, 257, False)
    check(b, x, w, False)
    assert (b == go.bf16_widen(go.bf16_bits(full[:, :257]))).all()  # the bf16 result is the rounded f32 result


@pytest.mark.parametrize("rows", [16, 300])
def test_kda_layer_projections(proj, rows):
    """forward.rs:3494-3542 at the model's widths: [q|k|v|b] 4096 -> 24,640 (a partial last feature tile), the gates'
    4096 -> 256 and the grouped 128 -> 8192 over the interleaved halves of its output."""
    g = torch.Generator(device="cuda").manual_seed(rows)
    mk = lambda *s, sigma: (torch.randn(*s, device="cuda", generator=g) * sigma).to(torch.bfloat16)
    w = proj.KdaProjW(proj.Bf16Mat.dense(mk(proj.KDA_P_COLS, proj.HIDDEN, sigma=0.02)), proj.Bf16Mat.dense(mk(256, proj.HIDDEN, sigma=0.02)),
                      proj.Bf16Mat.dense(mk(2, proj.KDA_WIDTH, 128, sigma=0.05)))
    normed = mk(rows, proj.HIDDEN, sigma=1.0)
    p = torch.zeros(rows, proj.KDA_P_COLS, dtype=torch.bfloat16, device="cuda")
    fga = torch.zeros(rows, 256, dtype=torch.bfloat16, device="cuda")
    ag = torch.zeros(rows, 2 * proj.KDA_WIDTH, dtype=torch.bfloat16, device="cuda")
    proj.kda_input_projections(normed, rows, w, p, fga, ag)
    torch.cuda.synchronize()
    assert status() == 0
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    xb = bits(normed)[None]
    for got, wm, xin in ((p, w.qkvb, xb), (fga, w.fga, xb)):
        want = go.gemm(xin, bits(wm.t).reshape(1, wm.n, wm.k), True)[0]
        assert go.rel_rms(got.float().cpu().numpy(), go.bf16_widen(go.bf16_bits(want))) < 2e-3  # bf16 rounding: 2^-9 rms
        wb = go.bf16_widen(go.bf16_bits(want))
        assert (np.abs(got.float().cpu().numpy() - wb) <= bf16_step(wb, want)).all()
    fb = bits(fga)
    xg = np.stack([fb[:, :128], fb[:, 128:]])
    want = go.gemm(xg, bits(w.fgb.t), True)
    got = ag.float().cpu().numpy().reshape(rows, 2, proj.KDA_WIDTH).transpose(1, 0, 2)
    wb = go.bf16_widen(go.bf16_bits(want))
    assert (np.abs(got - wb) <= bf16_step(wb, want)).all()
    # the library GEMM agrees within the same bound (reported by the reference's test for cuBLAS)
    lib = (normed.float() @ w.qkvb.t.float().T)
    assert go.rel_rms(p.float().cpu().numpy(), lib.to(torch.bfloat16).float().cpu().numpy()) < 2e-3


@pytest.mark.parametrize("f32_out", [True, False])
def test_many_rows_on_sm_pairs(proj, f32_out):
    """Above 512 rows with enough tiles the 256 x 256 tiles run on SM pairs (cta_group::2): ragged features (n not a
    multiple of 128), ragged rows, padded output rows, guards."""
    rng = go.Rng(21)
    groups, n, k, R = 1, 2568, 512, 2050
    w = rng.bf16s(n * k, 0.05).reshape(1, n, k)
    x = rng.bf16s(R * k, 1.0).reshape(1, R, k)
    got = run(proj, x, w, R, f32_out, ldo=n + 8, pad=64)
    check(got, x, w, f32_out)
    # a second launch on the same buffers gives the same bits
    again = run(proj, x, w, R, f32_out, ldo=n + 8, pad=64)
    assert (got.view(np.uint32) == again.view(np.uint32)).all()


def test_wide_weight_mid_range_rows(proj):
    """A wide weight (150 feature tiles) at 65..300 rows (128-row tiles, two blocks per SM): parity, and the rows that
    a 64-row launch also computes have the same bits -- the accumulation over k is the same sequence in every tile
    shape that does not split k."""
    rng = go.Rng(23)
    n, k, R = 19_200, 256, 300
    w = rng.bf16s(n * k, 0.05).reshape(1, n, k)
    x = rng.bf16s(R * k, 1.0).reshape(1, R, k)
    small = run(proj, x, w, 64, True)
    check(small, x, w, True)
    for rows in (65, 128, 129, 300):
        got = run(proj, x, w, rows, True, ldo=n + 8, pad=16)
        check(got, x, w, True)
        assert (got[:, :64].view(np.uint32) == small.view(np.uint32)).all(), rows


def test_split_k_shape_is_row_count_independent(proj):
    """o_proj's shape (32 feature tiles, 128 k blocks: the K range of a tile is split over a cluster) at 129..512
    rows: the split is chosen from (groups, n, k) alone, so the rows a 64-row launch also computes keep its bits."""
    rng = go.Rng(29)
    n, k, R = 4096, 8192, 512
    w = rng.bf16s(n * k, 0.02).reshape(1, n, k)
    x = rng.bf16s(R * k, 1.0).reshape(1, R, k)
    small = run(proj, x, w, 64, True)
    check(small, x, w, True)
    for rows in (129, 256, 384, 512):
        got = run(proj, x, w, rows, True, ldo=n + 8, pad=16)
        assert (got[:, :64].view(np.uint32) == small.view(np.uint32)).all(), rows
    check(got, x, w, True)
