"""Multi-GPU execution of the five operators: independent shards, one optional all-gather.

The reference is single-device: ``select_device`` refuses arguments that span
devices (``python/intent/targets/local.py:42-43``) and no collective exists in
its tree.  Every one of the five kernels is parallel over independent units
(``I.parallel`` over rows, M-tiles or batch x head), so N processes — one per
GPU — each run the unmodified single-GPU kernel on a contiguous block of units:

============  =======================================  ==========================
operator      sharded along                            replicated on every rank
============  =======================================  ==========================
softmax       rows of x / y                            —
layer_norm    rows of x / y                            gamma, beta
gemm          rows of A / C                            B
attention     flattened (batch, head) of q/k/v/out     —
csr_spmm      rows of A (offsets re-based) / Y         dense X
============  =======================================  ==========================

There is no exchange during compute.  ``gather`` concatenates the output blocks
with one ``all_gather`` (NCCL over NVLink on GPUs, gloo on CPU in tests) only
when the caller wants the whole result on every rank.  The unit split is the
contiguous split the reference's CPU dispatcher uses for its workers
(``python/intent/runtime/mojo/task_dispatch.c:44-49``).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def unit_range(units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous [begin, end) of `units` owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    chunk, extra = divmod(units, world)
    begin = rank * chunk + min(rank, extra)
    return begin, begin + chunk + (1 if rank < extra else 0)


@dataclass(frozen=True)
class RowShard:
    begin: int
    end: int

    @property
    def rows(self) -> int:
        return self.end - self.begin


def shard_rows(tensor: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    begin, end = unit_range(tensor.shape[dim], rank, world)
    return tensor.narrow(dim, begin, end - begin)


def shard_csr(row_offsets: torch.Tensor, column_indices: torch.Tensor, values: torch.Tensor,
              rank: int, world: int):
    """Row block of a CSR matrix with offsets re-based to the block's first non-zero.
    Index values are copied bit for bit; only the offsets' origin moves."""
    rows = row_offsets.numel() - 1
    begin, end = unit_range(rows, rank, world)
    first = int(row_offsets[begin])
    last = int(row_offsets[end])
    local_offsets = (row_offsets[begin:end + 1] - first).to(torch.int32)
    return local_offsets, column_indices[first:last], values[first:last], RowShard(begin, end)


def shard_heads(tensor: torch.Tensor, rank: int, world: int, group: int = 1) -> torch.Tensor:
    """Block of flattened (batch, head) units of a (B, H, S, D) tensor as (1, units, S, D).
    `group` keeps the query heads of one key/value head on one rank (GQA)."""
    b, h, s, d = tensor.shape
    if h % group:
        raise ValueError("head count must be a multiple of the head group")
    flat = tensor.reshape(1, b * h, s, d)
    begin, end = unit_range(b * h // group, rank, world)
    return flat[:, begin * group:end * group]


def gather(local: torch.Tensor, total_units: int, *, dim: int = 0, group=None) -> torch.Tensor:
    """All-gather of unevenly sized contiguous blocks along `dim` (the only collective)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    sizes = [unit_range(total_units, r, world) for r in range(world)]
    widest = max(end - begin for begin, end in sizes)
    moved = local.movedim(dim, 0).contiguous()
    padded = moved
    if moved.shape[0] < widest:
        padded = torch.zeros((widest, *moved.shape[1:]), dtype=moved.dtype, device=moved.device)
        padded[:moved.shape[0]] = moved
    blocks = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(blocks, padded, group=group)
    joined = torch.cat([block[:end - begin] for block, (begin, end) in zip(blocks, sizes)], dim=0)
    return joined.movedim(0, dim)


def world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1
