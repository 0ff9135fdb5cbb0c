"""Host logic of the multi-GPU path on CPU: two gloo ranks shard the units, compute
their block with the CPU oracle standing in for the device kernel, and the single
optional collective (all-gather of output blocks) reassembles the full result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from intent_b200 import sharding, workloads


def test_unit_range_is_a_contiguous_partition():
    for units in (0, 1, 7, 8, 4096):
        for world in (1, 2, 3, 8):
            ranges = [sharding.unit_range(units, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == units
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.unit_range(4, 2, 2)


def test_csr_shard_rebases_offsets_and_keeps_indices_bit_exact():
    ro, ci, va, _ = workloads.csr_inputs(101, 64, 9, 4, seed=1)
    pieces = [sharding.shard_csr(ro, ci, va, r, 3) for r in range(3)]
    assert torch.equal(torch.cat([p[1] for p in pieces]), ci)
    assert torch.equal(torch.cat([p[2] for p in pieces]), va)
    for offsets, columns, _, rows in pieces:
        assert offsets[0] == 0 and offsets[-1] == columns.numel() and offsets.dtype == torch.int32
        assert torch.equal(offsets, ro[rows.begin:rows.end + 1] - ro[rows.begin])


def test_head_shards_keep_query_groups_together():
    q = torch.arange(2 * 8 * 3 * 4).reshape(2, 8, 3, 4)
    blocks = [sharding.shard_heads(q, r, 3, group=4) for r in range(3)]
    assert [b.shape[1] for b in blocks] == [8, 4, 4]
    assert torch.equal(torch.cat(blocks, dim=1).reshape(2, 8, 3, 4), q)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures):
    try:
        import oracle
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        # softmax: rows
        (x,) = workloads.softmax_inputs(37, 64, seed=2)
        local = oracle.softmax(sharding.shard_rows(x, rank, world).contiguous(), workers=1)
        assert torch.equal(sharding.gather(local, 37), oracle.softmax(x, workers=1))
        # gemm: row blocks of A and C, B replicated
        a, b = workloads.gemm_inputs(45, 24, 32, seed=3)
        local = oracle.gemm(sharding.shard_rows(a, rank, world).contiguous(), b, workers=1)
        assert torch.equal(sharding.gather(local, 45), oracle.gemm(a, b, workers=1))
        # attention: flattened (batch, head) units, GQA groups kept together
        q, k, v, scale = workloads.attention_inputs(1, 6, 40, 64, seed=4, kv_heads=3)
        ql, kl, vl = (sharding.shard_heads(q, rank, world, 2), sharding.shard_heads(k, rank, world),
                      sharding.shard_heads(v, rank, world))
        local = oracle.attention(ql.contiguous(), kl.contiguous(), vl.contiguous(), scale, head_group=2,
                                 chunk=16, workers=1)
        joined = sharding.gather(local.reshape(-1, 2, 40, 64), 3).reshape(1, 6, 40, 64)
        assert torch.equal(joined, oracle.attention(q, k, v, scale, head_group=2, chunk=16, workers=1))
        # csr spmm: row blocks with re-based offsets, X replicated
        ro, ci, va, dense = workloads.csr_inputs(53, 40, 7, 8, seed=5)
        offsets, columns, values, rows = sharding.shard_csr(ro, ci, va, rank, world)
        local = oracle.csr_spmm(offsets.contiguous(), columns.contiguous(), values.contiguous(), dense, workers=1)
        assert local.shape[0] == rows.rows
        assert torch.equal(sharding.gather(local, 53), oracle.csr_spmm(ro, ci, va, dense, workers=1))
        assert sharding.world() == (rank, world)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as error:  # surface the failure in the parent
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
        raise


def test_two_gloo_ranks_shard_and_gather():
    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_worker, args=(rank, 2, port, failures)) for rank in range(2)]
    for process in processes:
        process.start()
    for process in processes:
        process.join(120)
    messages = []
    while not failures.empty():
        messages.append(failures.get())
    assert not messages, messages
    assert all(process.exitcode == 0 for process in processes)
