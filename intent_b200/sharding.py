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


# --------------------------------------------------------------------------- one call, N ranks
@dataclass(frozen=True)
class Distribution:
    """How one prepared call is spread over the ranks of a process group (one process per GPU).

    Every rank makes the same call with the same FULL operands resident on its own GPU; the
    call computes only this rank's block of units.  With ``gather_output`` the output blocks
    are exchanged by one all-gather, so the full result lands on every rank; without it only
    the rank's own block of the output buffer is defined."""
    rank: int
    world: int
    gather_output: bool = False
    group: object = None


def distribution(gpus, gather_output: bool, device: torch.device) -> Distribution | None:
    """Reads the ``gpus`` / ``gather_output`` backend options.  ``gpus`` is the number of ranks
    or the list of their CUDA ordinals in rank order; None or 1 keeps the call on one GPU."""
    if gpus is None:
        if gather_output:
            raise ValueError("gather_output needs the gpus option")
        return None
    count = gpus if isinstance(gpus, int) and not isinstance(gpus, bool) else len(tuple(gpus))
    if count < 1:
        raise ValueError("gpus must name at least one device")
    if count == 1:
        return None
    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("the gpus option runs one process per GPU: initialise torch.distributed first")
    rank, size = dist.get_rank(), dist.get_world_size()
    if size != count:
        raise ValueError(f"gpus names {count} devices but the process group has {size} ranks")
    if not isinstance(gpus, int) and device.index is not None and int(tuple(gpus)[rank]) != device.index:
        raise ValueError(f"rank {rank} runs on cuda:{device.index}, but gpus[{rank}] is {tuple(gpus)[rank]}")
    return Distribution(rank, size, bool(gather_output))


@dataclass(frozen=True)
class OutputBlock:
    """One declared output: the whole buffer as (units, ...) and the rank's block of it."""
    full: torch.Tensor       # the caller's (or the runtime's) whole output buffer
    flat: torch.Tensor       # a view of it with the sharded units on axis 0
    begin: int               # the rank's rows of `flat`
    end: int
    per_unit: int = 1        # rows of `flat` per unit (query heads per key head for attention)

    @property
    def local(self) -> torch.Tensor:
        return self.flat[self.begin:self.end]


@dataclass(frozen=True)
class Partition:
    arguments: tuple         # per public parameter: the rank's shard (tensors) or the scalar itself
    outputs: tuple           # OutputBlock per declared output, in declaration order
    units: int               # independent units of the whole call
    begin: int
    end: int


def _rows(tensor: torch.Tensor, begin: int, end: int) -> torch.Tensor:
    return tensor[begin:end]


def _flat_heads(tensor: torch.Tensor, name: str) -> torch.Tensor:
    """(B, H, S, D) -> (B*H, S, D) without a copy; the kernels walk (batch, head) by strides,
    so the two leading axes must collapse into one."""
    b, h = tensor.shape[:2]
    if b > 1 and h > 1 and tensor.stride(0) != h * tensor.stride(1):
        raise NotImplementedError(f"{name}: a sharded attention call needs batch and head axes that collapse "
                                  "into one (stride[0] == heads * stride[1])")
    return tensor.as_strided((b * h, *tensor.shape[2:]), (tensor.stride(1) if h > 1 else tensor.stride(0),
                                                           *tensor.stride()[2:]), tensor.storage_offset())


# family -> (positions cut along rows, position of the CSR row offsets, output positions)
_ROW_FAMILIES = {
    "softmax": ((0, 1), None, (1,)),
    "softmax_backward": ((0, 1, 2), None, (2,)),
    "layer_norm": ((0, 3), None, (3,)),
    "gemm": ((0, 2), None, (2,)),
    "csr_spmm": ((4,), 0, (4,)),
    "csr_spmv": ((4,), 0, (4,)),
}


def partition(family: str, ordered: tuple, rank: int, world: int, *, head_group: int = 1) -> Partition:
    """The rank's shard of one call.  `ordered` holds the full operands in public-parameter
    order (outputs included).  Every shard is a view: nothing is copied, so a prepared call
    keeps seeing what the caller writes into the full buffers.

    Rows (softmax, LayerNorm, the M axis of GEMM, CSR rows) and flattened (batch, key head)
    units (attention) are cut by the contiguous split of
    ``python/intent/runtime/mojo/task_dispatch.c:44-49``.  A CSR block keeps the absolute
    offsets of its rows and the whole index / value arrays: the kernel addresses non-zeros by
    offset, so no array is re-based and index values are consumed bit for bit."""
    if family in _ROW_FAMILIES:
        cut, offsets, outputs = _ROW_FAMILIES[family]
        units = ordered[outputs[0]].shape[0]
        begin, end = unit_range(units, rank, world)
        arguments = list(ordered)
        for position in cut:
            arguments[position] = _rows(ordered[position], begin, end)
        if offsets is not None:
            arguments[offsets] = ordered[offsets][begin:end + 1]
        blocks = tuple(OutputBlock(ordered[p], ordered[p], begin, end) for p in outputs)
        return Partition(tuple(arguments), blocks, units, begin, end)
    if family == "flash_attention":
        q, k, v, out = ordered[:4]
        if q.shape[1] != k.shape[1] * head_group:
            raise ValueError("query heads must equal key heads times the head group")
        units = k.shape[0] * k.shape[1]
        begin, end = unit_range(units, rank, world)
        flat_q, flat_k, flat_v, flat_out = (_flat_heads(t, n) for t, n in zip((q, k, v, out), "qkvo"))
        arguments = list(ordered)
        arguments[0] = flat_q[begin * head_group:end * head_group].unsqueeze(0)
        arguments[1] = flat_k[begin:end].unsqueeze(0)
        arguments[2] = flat_v[begin:end].unsqueeze(0)
        arguments[3] = flat_out[begin * head_group:end * head_group].unsqueeze(0)
        block = OutputBlock(out, flat_out, begin * head_group, end * head_group, head_group)
        return Partition(tuple(arguments), (block,), units, begin, end)
    raise NotImplementedError(f"the {family} family has no multi-GPU partition rule")


def gather_blocks(block: OutputBlock, world: int, *, group=None) -> None:
    """The one collective: every rank's block of `block.flat` reaches every rank, in place.
    Equal blocks of a dense buffer travel as one all-gather; otherwise each block is broadcast
    from its owner (block sizes differ by at most one unit)."""
    flat = block.flat
    if flat.shape[0] == 0 or world == 1:
        return
    if not flat.is_contiguous():
        raise NotImplementedError("gather_output needs a dense output buffer")
    units = flat.shape[0] // block.per_unit
    if units % world == 0:
        dist.all_gather_into_tensor(flat, block.local, group=group)
        return
    for owner in range(world):
        begin, end = unit_range(units, owner, world)
        if end > begin:
            source = dist.get_global_rank(group, owner) if group is not None else owner
            dist.broadcast(flat[begin * block.per_unit:end * block.per_unit], src=source, group=group)


def world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1
