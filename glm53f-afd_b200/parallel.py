"""Sharding of the KDA core over the GPUs of one box: one process per GPU, torch.distributed for the plumbing.

The recurrence never mixes heads and never mixes slots, so both shardings need no collective on the data path:

  prefill   by head: rank r runs heads [r*H/N, (r+1)*H/N) of every row; the per-head outputs are then all-gathered
            into the full [T, H, 128] tensor (the one exchange step, `gather_heads`);
  decode, verify, commit   by slot: rank r owns slots [r*S/N, (r+1)*S/N) and their states; nothing is exchanged.

The reference has no counterpart (it runs on one GPU).  Everything here works on CPU tensors with the gloo backend
too, which is how the host-side logic is tested.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """[lo, hi) of `total` units owned by `rank`: contiguous blocks, the first total % world ranks one unit larger."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def head_range(heads: int, rank: int, world: int) -> tuple[int, int]:
    if heads % world != 0:
        raise ValueError(f"{heads} heads do not split evenly over {world} ranks")
    return shard_range(heads, rank, world)


def slot_range(slots: int, rank: int, world: int) -> tuple[int, int]:
    return shard_range(slots, rank, world)


def shard_heads(x: torch.Tensor, heads: int, rank: int, world: int) -> torch.Tensor:
    """Rows [T, H, ...] -> this rank's heads [T, H/N, ...], contiguous (what the kernels take)."""
    lo, hi = head_range(heads, rank, world)
    if x.dim() < 2 or x.shape[1] != heads:
        raise ValueError(f"expected [T, {heads}, ...], got {tuple(x.shape)}")
    return x[:, lo:hi].contiguous()


def gather_heads(local: torch.Tensor, heads: int, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather of per-head outputs: local [T, H/N, D] on every rank -> [T, H, D] on every rank.

    The collective lands rank-major ([N, T, H/N, D]) in a local staging buffer; the head-major result is then one
    local transposing copy, so nothing but the collective itself touches another GPU's memory."""
    world = dist.get_world_size(group)
    t, hl, d = local.shape
    if hl * world != heads:
        raise ValueError(f"{world} ranks x {hl} heads != {heads}")
    staged = torch.empty((world * t, hl, d), dtype=local.dtype, device=local.device)  # rank-major concatenation
    dist.all_gather_into_tensor(staged, local.contiguous(), group=group)
    if out is None:
        out = torch.empty((t, heads, d), dtype=local.dtype, device=local.device)
    out.view(t, world, hl, d).copy_(staged.view(world, t, hl, d).permute(1, 0, 2, 3))
    return out


class GatheredOutput:
    """The full [rows][heads][128] bf16 output of a head-sharded prefill on every rank, each rank's buffer mapped into
    every other rank's address space (torch symmetric memory), so that the prefill kernel of each rank can store its
    heads' rows straight into all of them: the all-gather happens inside the kernel, over NVLink, by plain stores.

    `addresses` is what core.prefill_varlen(..., gather=(addresses, heads, head0)) takes.  `barrier()` orders the ranks
    on the current stream; call it before a launch that overwrites the buffers (no rank may still be reading) and
    after it (every rank's rows have landed) before reading `tensor`."""

    def __init__(self, rows: int, heads: int, group=None):
        import torch.distributed._symmetric_memory as symm

        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm.empty((rows, heads, 128), dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.tensor, self.group)
        self.addresses = [int(a) for a in self.handle.buffer_ptrs]
        self._token = torch.zeros(1, device="cuda")

    def barrier(self) -> None:
        # A one-element all-reduce in stream order: every rank's earlier work on its stream is complete before any
        # rank's later work starts.
        dist.all_reduce(self._token, group=self.group)
