"""The five operators split over two GPUs: one process per GPU under torch.distributed/NCCL,
every rank makes the same prepared call with ``backend_options={"gpus": ..., "gather_output":
True}``, computes its block of rows / M-tiles / (batch, head) units with the CUDA kernel, and
one NCCL all-gather completes the output on every rank.  Checked against the CPU oracle on
every rank (bit-exact for CSR SpMM).  Skipped on a machine with fewer than two GPUs."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two CUDA devices")]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank: int, world: int, port: int, failures):
    try:
        import datetime

        import torch.distributed as dist

        import intent_b200 as b200
        import oracle
        from conftest import relative_error
        from intent_b200 import workloads
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        device = torch.device("cuda", rank)
        torch.cuda.set_device(device)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device,
                                timeout=datetime.timedelta(seconds=120))
        options = {"gpus": list(range(world)), "gather_output": True}

        (x,) = workloads.softmax_inputs(257, 1024, seed=21)                       # uneven row split
        y = b200.jit(b200.kernels.stable_softmax, backend_options=options).run(x.to(device))
        assert relative_error(y, oracle.softmax(x)) <= 1e-5, "softmax"

        x, w, b, inv, eps = workloads.layer_norm_inputs(128, 4096, seed=22)
        kernel = b200.jit(b200.kernels.layer_norm_f16, backend_options=options)
        call = kernel.prepare(x.to(device), w.to(device), b.to(device), inv, eps)
        call.launch()
        assert relative_error(call.result(), oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2, "layer_norm"
        assert call.description[-1][0] == "shard"

        a, bm = workloads.gemm_inputs(512, 512, 256, seed=23)
        kernel = b200.jit(b200.kernels.gemm, constexprs={"ACTIVATION": "NONE"}, backend_options=options)
        call = kernel.prepare(a.to(device), bm.to(device))
        call.launch()
        call.check()
        assert relative_error(call.result(), oracle.gemm(a, bm)) <= 1e-2, "gemm"

        q, k, v, scale = workloads.attention_inputs(1, 6, 256, 128, seed=24, kv_heads=3)   # 3 units over 2 ranks
        kernel = b200.jit(b200.kernels.flash_attention_bf16_fwd, constexprs={"HEAD_GROUP": 2, "CAUSAL": True},
                          backend_options=options)
        out = kernel.run(q.to(device), k.to(device), v.to(device), scale)
        assert relative_error(out, oracle.attention(q, k, v, scale, head_group=2)) <= 1e-2, "attention"

        ro, ci, va, dense = workloads.csr_inputs(8192, 8192, 32, 128, seed=25)
        y = b200.jit(b200.kernels.csr_spmm, backend_options=options).run(
            ro.to(device), ci.to(device), va.to(device), dense.to(device))
        assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci, va, dense)), "csr_spmm is not bit-exact"

        # the same options through the reference's own front door (its option gate and target resolution)
        from conftest import HAS_REFERENCE, REFERENCE_PYTHON
        if HAS_REFERENCE:
            import sys
            import tempfile
            sys.path.insert(0, str(REFERENCE_PYTHON))
            os.environ["INTENT_CACHE_DIR"] = tempfile.mkdtemp(prefix=f"intent-cache-{rank}-")
            os.environ.pop("INTENT_COMPILER", None)
            import intent
            b200.register()
            from intent.examples.kernels.normalization.layer_norm import layer_norm_f16
            x, w, b, inv, eps = workloads.layer_norm_inputs(130, 2048, seed=27)
            kernel = intent.jit(layer_norm_f16, backend="b200", backend_options=options)
            y = kernel.run(x.to(device), w.to(device), b.to(device), inv, eps)
            assert relative_error(y, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2, "layer_norm through intent.jit"
            with pytest.raises(ValueError, match="unsupported local b200 options"):
                intent.jit(layer_norm_f16, backend="b200", backend_options={"ranks": 2}).prepare(
                    x.to(device), w.to(device), b.to(device), inv, eps)

        # without gather_output only the rank's own block is written
        (x,) = workloads.softmax_inputs(64, 512, seed=26)
        out = torch.full((64, 512), -1.0, device=device)
        local = b200.jit(b200.kernels.stable_softmax, backend_options={"gpus": world})
        local(x.to(device), out)
        begin, end = b200.sharding.unit_range(64, rank, world)
        assert relative_error(out[begin:end], oracle.softmax(x)[begin:end]) <= 1e-5
        other = torch.ones(64, dtype=torch.bool)
        other[begin:end] = False
        assert bool((out.cpu()[other] == -1.0).all())
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    except Exception as error:
        failures.put(f"rank {rank}: {type(error).__name__}: {error}")
        raise


def test_five_operators_split_over_two_gpus_match_the_oracle():
    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    processes = [context.Process(target=_rank, args=(rank, 2, port, failures)) for rank in range(2)]
    for process in processes:
        process.start()
    for process in processes:
        process.join(600)
    messages = []
    while not failures.empty():
        messages.append(failures.get())
    assert not messages, messages
    assert all(process.exitcode == 0 for process in processes)
