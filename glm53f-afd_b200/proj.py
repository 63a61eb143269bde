"""The projections either side of the KDA core: host side of include/glm53f_proj.h.

Mirror of the reference's `Bf16Mat` and `Gemm::bf16` (crates/glm53f-forward/src/gemm.rs:35-48, 212-235) and of the
three GEMMs a KDA layer issues on its normed input (crates/glm53f-forward/src/forward.rs:3494-3542).  Where the
reference picks its CUDA-core GEMV for up to 8 rows and cuBLAS above, every row count goes to the tcgen05 kernel
here.  Tensors are torch CUDA tensors; there is no CPU path.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ffi
from .core import CudaError, Invalid

HIDDEN = 4096
KDA_HEADS, KDA_DIM = 64, 128
KDA_WIDTH = KDA_HEADS * KDA_DIM          # 8192
KDA_QKV = 3 * KDA_WIDTH                  # 24,576
KDA_P_COLS = KDA_QKV + KDA_HEADS         # 24,640: [q | k | v | beta logits] (crates/glm53f-forward/src/shape.rs:23-32)


def _launched(code: int, what: str) -> None:
    if code == 0:
        return
    if code == 1:
        raise Invalid(f"{what}: rejected by the launcher")
    raise CudaError(code, what)


@dataclass
class Bf16Mat:
    """A BF16 weight [groups][n][k] on the device (gemm.rs:35-48): row stride `ld`, group stride `gstride` (elements)."""

    t: torch.Tensor
    n: int
    k: int
    ld: int
    groups: int = 1
    gstride: int = 0

    @classmethod
    def dense(cls, t: torch.Tensor) -> "Bf16Mat":
        if t.dim() == 2:
            return cls(t, t.shape[0], t.shape[1], t.shape[1], 1, 0)
        return cls(t, t.shape[1], t.shape[2], t.shape[2], t.shape[0], t.shape[1] * t.shape[2])

    def bytes(self) -> int:
        return self.groups * self.n * self.k * 2


def bf16(x: torch.Tensor, ldx: int, x_gstride: int, w: Bf16Mat, rows: int, out: torch.Tensor, ldo: int, o_gstride: int,
         out_f32: bool = False, x_offset: int = 0, out_offset: int = 0) -> None:
    """out[g][m][o] = sum_k x[g][m][k] w[g][o][k] (Gemm::bf16, gemm.rs:212-235); offsets in elements of x / out."""
    if rows == 0:
        return
    if x.dtype not in (torch.bfloat16, torch.int16, torch.uint16) or w.t.dtype not in (torch.bfloat16, torch.int16, torch.uint16):
        raise Invalid("x and the weight are bf16")
    if out.dtype != (torch.float32 if out_f32 else x.dtype) and not (not out_f32 and out.element_size() == 2):
        raise Invalid("out is f32 when out_f32, else bf16")
    need_x = x_offset + (w.groups - 1) * x_gstride + (rows - 1) * ldx + w.k
    need_o = out_offset + (w.groups - 1) * o_gstride + (rows - 1) * ldo + w.n
    if x.numel() < need_x or out.numel() < need_o or w.t.numel() < (w.groups - 1) * w.gstride + (w.n - 1) * w.ld + w.k:
        raise Invalid("a buffer is smaller than the shapes named")
    stream = torch.cuda.current_stream().cuda_stream
    code = ffi.glm53f_kda_proj_bf16(x.data_ptr() + 2 * x_offset, ldx, x_gstride, w.t.data_ptr(), w.ld, w.gstride, w.groups, rows, w.n, w.k,
                                    out.data_ptr() + out_offset * out.element_size(), 1 if out_f32 else 0, ldo, o_gstride, stream)
    _launched(code, "glm53f_kda_proj_bf16")


@dataclass
class KdaProjW:
    """The projection weights of one KDA layer (crates/glm53f-forward/src/weights.rs:145-162): the fused [q|k|v|b]
    weight [24,640][4096], the low-rank gates' first factor [256][4096] (f and g stacked) and second factors
    [2][8192][128]."""

    qkvb: Bf16Mat
    fga: Bf16Mat
    fgb: Bf16Mat


def kda_input_projections(normed: torch.Tensor, rows: int, w: KdaProjW, p: torch.Tensor, fga: torch.Tensor, ag: torch.Tensor) -> None:
    """The three GEMMs of a KDA layer's input (forward.rs:3494-3542): p [rows][24,640] = normed . qkvb^T; fga
    [rows][256] = normed . fga^T; ag [rows][2 x 8192] = per group g, fga[:, 128 g : 128 g + 128] . fgb[g]^T."""
    bf16(normed, HIDDEN, 0, w.qkvb, rows, p, KDA_P_COLS, 0)
    bf16(normed, HIDDEN, 0, w.fga, rows, fga, 2 * KDA_DIM, 0)
    bf16(fga, 2 * KDA_DIM, KDA_DIM, w.fgb, rows, ag, 2 * KDA_WIDTH, KDA_WIDTH)
