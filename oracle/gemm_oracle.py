"""CPU restatement of the reference's bf16 projection GEMM.  TEST INFRASTRUCTURE ONLY: the checker the tcgen05 GEMM is
compared with; nothing in the product imports it.

  gemm        out[g][m][o] = sum_k x[g][m][k] * w[g][o][k]: the contract of Gemm::bf16 / glm53f_fwd_gemv_bf16
              (crates/glm53f-forward/kernels/glm53f_forward.h:19-24, src/gemm.rs:212-235).  Products of bf16 values
              are exact in f32; the sum is formed in f64 here and rounded once, so this is the value every f32
              accumulation order approximates.
  gemv_model  the reference's host model of its GEMV (crates/glm53f-forward/src/reference.rs, `gemv_bf16`): lane l of
              a warp accumulates fma(x, w, acc) over k = 8 l + 256 i + j in f32, the 32 lane sums are added by the
              xor butterfly, K splits are added in split order.  Used to pin `gemm` against the reference's own
              model on its test shapes (tests/test_proj_cpu.py) within the reference's cuBLAS-vs-GEMV bound.
  rel_rms     crates/glm53f-forward/src/reference.rs:116-124.
  rng         the reference tests' generator (crates/glm53f-forward/tests/gemv.rs:20-40): SplitMix64 + Box-Muller.

Parity bar for the GPU kernel (the reference's, tests/gemv.rs:199-201): relative RMS below 1e-5 on f32 outputs.
"""
import numpy as np


def bf16_widen(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_bits(x):
    u = np.asarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(x, np.float32))
    r[nan] = 0x7FC0
    return r


def gemm(x, w, out_f32=True):
    """x [groups][rows][k], w [groups][n][k] as bf16 bits -> f32 [groups][rows][n] (rounded to bf16 values when
    out_f32 is False)."""
    xs, ws = bf16_widen(x).astype(np.float64), bf16_widen(w).astype(np.float64)
    out = np.einsum("gmk,gok->gmo", xs, ws).astype(np.float32)
    return out if out_f32 else bf16_widen(bf16_bits(out))


def gemv_model(x, w, ksplit=1):
    """The reference GEMV's accumulation order for one group: x [rows][k], w [n][k] bf16 bits -> f32 [rows][n]."""
    xs, ws = bf16_widen(x), bf16_widen(w)
    rows, k = xs.shape
    n = ws.shape[0]
    width = k // ksplit
    out = np.zeros((rows, n), np.float32)
    for s in range(ksplit):
        lo = s * width
        acc = np.zeros((rows, n, 32), np.float32)
        for i in range(0, width, 256):
            for j in range(8):
                cols = lo + i + 8 * np.arange(32) + j
                ok = cols < lo + width
                xv = np.where(ok[None, :], xs[:, np.minimum(cols, k - 1)], 0.0).astype(np.float32)   # [rows][32]
                wv = np.where(ok[None, :], ws[:, np.minimum(cols, k - 1)], 0.0).astype(np.float32)   # [n][32]
                prod = (xv[:, None, :].astype(np.float64) * wv[None, :, :].astype(np.float64) + acc.astype(np.float64))
                acc = prod.astype(np.float32)  # one rounding per fma
        v = acc
        for off in (16, 8, 4, 2, 1):
            v = (v + v[..., np.arange(32) ^ off]).astype(np.float32)
        out = (out + v[..., 0]).astype(np.float32) if s else v[..., 0].copy()
    return out


def rel_rms(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-300)))


class Rng:
    """SplitMix64 and Box-Muller, as the reference's tests draw their matrices."""

    def __init__(self, seed):
        self.s = np.uint64(seed)

    def _next(self, n):
        with np.errstate(over="ignore"):
            idx = np.arange(1, n + 1, dtype=np.uint64)
            z = self.s + idx * np.uint64(0x9E3779B97F4A7C15)
            self.s = z[-1]
            z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
            z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
            return z ^ (z >> np.uint64(31))

    def normal(self, n):
        r = self._next(2 * n)
        u1 = np.maximum((r[0::2] >> np.uint64(11)).astype(np.float64) / float(1 << 53), 1e-12)
        u2 = (r[1::2] >> np.uint64(11)).astype(np.float64) / float(1 << 53)
        return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)

    def bf16s(self, n, sigma):
        return bf16_bits(self.normal(n) * np.float32(sigma))
