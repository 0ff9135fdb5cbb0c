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
        _partitioned_calls(oracle, rank, world)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as error:  # surface the failure in the parent
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
        raise


def _partitioned_calls(oracle, rank, world):
    """`partition` + `gather_blocks`: what a prepared call with the gpus / gather_output options
    does, with the CPU oracle standing in for the kernel.  Every rank holds the full operands,
    computes its block in place and the all-gather completes the output on every rank."""
    # rows, uneven split (37 rows over the ranks) -> per-owner broadcast path
    (x,) = workloads.softmax_inputs(37, 64, seed=6)
    y = torch.zeros_like(x)
    part = sharding.partition("softmax", (x, y), rank, world)
    assert part.units == 37 and part.arguments[1].data_ptr() == y[part.begin:].data_ptr()
    part.arguments[1].copy_(oracle.softmax(part.arguments[0].contiguous(), workers=1))
    sharding.gather_blocks(part.outputs[0], world)
    assert torch.equal(y, oracle.softmax(x, workers=1))
    # rows, even split -> one all_gather_into_tensor; gamma and beta are not cut
    x, w, b, inv, eps = workloads.layer_norm_inputs(8 * world, 64, seed=7)
    y = torch.zeros_like(x)
    part = sharding.partition("layer_norm", (x, w, b, y, inv, eps), rank, world)
    assert part.arguments[1] is w and part.arguments[4] == inv
    part.arguments[3].copy_(oracle.layer_norm(part.arguments[0].contiguous(), w, b, inv, eps, workers=1))
    sharding.gather_blocks(part.outputs[0], world)
    assert torch.equal(y, oracle.layer_norm(x, w, b, inv, eps, workers=1))
    # CSR rows: offsets keep their absolute values, index and value arrays are not cut
    ro, ci, va, dense = workloads.csr_inputs(53, 40, 7, 8, seed=8)
    y = torch.zeros(53, 8)
    part = sharding.partition("csr_spmm", (ro, ci, va, dense, y), rank, world)
    offsets = part.arguments[0]
    assert part.arguments[1] is ci and offsets.numel() == part.end - part.begin + 1
    assert torch.equal(offsets, ro[part.begin:part.end + 1])
    first, last = int(offsets[0]), int(offsets[-1])
    local = oracle.csr_spmm((offsets - first).contiguous(), ci[first:last].contiguous(),
                            va[first:last].contiguous(), dense, workers=1)
    part.arguments[4].copy_(local)
    sharding.gather_blocks(part.outputs[0], world)
    assert torch.equal(y, oracle.csr_spmm(ro, ci, va, dense, workers=1))
    # attention: (batch, key head) units, the query heads of a key head stay on one rank
    q, k, v, scale = workloads.attention_inputs(2, 6, 40, 64, seed=9, kv_heads=3)
    out = torch.zeros_like(q)
    part = sharding.partition("flash_attention", (q, k, v, out, scale), rank, world, head_group=2)
    ql, kl, vl, ol = part.arguments[:4]
    assert part.units == 6 and ql.shape[1] == 2 * kl.shape[1] and ol.data_ptr() == part.outputs[0].local.data_ptr()
    ol.copy_(oracle.attention(ql.contiguous(), kl.contiguous(), vl.contiguous(), scale, head_group=2, chunk=16,
                              workers=1))
    sharding.gather_blocks(part.outputs[0], world)
    assert torch.equal(out, oracle.attention(q, k, v, scale, head_group=2, chunk=16, workers=1))
    with pytest.raises(NotImplementedError):
        sharding.partition("layer_norm_backward_rows", (x,), rank, world)


def _absent_rank_worker(rank: int, world: int, port: int, results):
    """Rank 1 never joins the collective: rank 0's all-gather must end with an error after the
    process group's timeout instead of blocking for ever."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    y = torch.zeros(8, 4)
    part = sharding.partition("softmax", (torch.zeros(8, 4), y), rank, world)
    if rank == 0:
        try:
            sharding.gather_blocks(part.outputs[0], world)
            results.put("rank 0: the gather returned although rank 1 never joined")
        except Exception as error:
            results.put(f"timeout:{type(error).__name__}")
    else:
        import time
        time.sleep(12)          # alive, but it never reaches the collective
    os._exit(0)                 # no orderly shutdown: the group is broken on purpose


def test_a_rank_that_never_joins_ends_the_gather_with_an_error():
    context = mp.get_context("spawn")
    results = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_absent_rank_worker, args=(rank, 2, port, results)) for rank in range(2)]
    for process in processes:
        process.start()
    message = results.get(timeout=60)
    for process in processes:
        process.join(30)
    assert message.startswith("timeout:"), message


def test_distribution_reads_the_backend_options():
    assert sharding.distribution(None, False, torch.device("cpu")) is None
    assert sharding.distribution(1, False, torch.device("cpu")) is None
    with pytest.raises(ValueError):
        sharding.distribution(None, True, torch.device("cpu"))
    with pytest.raises(RuntimeError, match="torch.distributed"):
        sharding.distribution([0, 1], False, torch.device("cpu"))


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
