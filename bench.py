#!/usr/bin/env python
"""Benchmark of the b200 operator hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--op NAME|all] [--impl b200|reference]

One JSON line on stdout.  A "step" is one launch of the operator over one
batch of seeded synthetic input (``intent_b200.workloads``).  The headline
workload is the LayerNorm configuration (f16 16384 x 4096, 268 MB per step, larger
than L2); ``--op all`` (the default) also measures softmax, GEMM, attention, CSR SpMM
and the widened kernels (SpMV, softmax / LayerNorm / attention backward) and reports
them under ``"ops"``.

  value     device-resident throughput: inputs already in HBM, K launches timed with
            CUDA events on the launching stream between two barriers + syncs,
            max over ranks, whole-job aggregate (weak scaling: each rank runs the
            full per-GPU workload, no data-path collective).
  e2e       the same metric through the public API (jit(...).prepare(...), then
            call.enqueue(stream)) with HOST buffers: every step copies its inputs from
            pinned host memory and its result back inside the timed region; the copies
            of neighbouring steps overlap on three streams over two sets of device
            buffers, and the region ends when the last result is in host memory.
  roofline  achieved = algorithmic bytes (or flops) per launch / average launch time,
            against the pod-measured peak in MEASURED_PEAKS.json.
  cpu_baseline  the CPU oracle (a port of the reference's kernel definitions; the
            reference's own compiler and CPU provider cannot be built here) timed on
            this host's cores with the reference's protocol.

``--impl reference`` times that CPU path alone with every host thread.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL = {"hbm": 8000.0, "tensor": 2250.0}

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures
# summarised under profiles/.
NCU_TRAFFIC_BYTES = {"softmax": 16791040, "layer_norm": 216351232, "gemm": 1154501120, "attention": 1057477120,
                     "spmm": 975351808, "softmax_backward": 160885760, "spmv": 8672256,
                     # steps of several kernels: the sum over the step's launches
                     "layer_norm_backward": 74406912 + 2109440, "attention_backward": 274570496 + 847716352}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return FALLBACK_PEAKS, "fallback"


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index, self.samples, self.process = device_index, [], None
        self.windows = []          # (begin, end) wall-clock intervals with the GPU under the timed load

    def window(self):
        sampler = self

        class Window:
            def __enter__(self):
                self.begin = time.time()

            def __exit__(self, *_):
                sampler.windows.append((self.begin, time.time()))

        return Window()

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) >= 9:
                self.samples.append((time.time(), fields))

    def __exit__(self, *_):
        if self.process:
            self.process.terminate()
            try:
                self.process.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.process.kill()

    def summary(self, windows=None) -> dict:
        clocks, reasons, maximum = [], set(), None
        windows = self.windows if windows is None else windows
        for stamp, fields in list(self.samples):
            # nvidia-smi reports the state of the last ~50 ms; keep samples taken inside a load window
            if not any(begin + 0.05 <= stamp <= end + 0.05 for begin, end in windows):
                continue
            try:
                clocks.append(float(fields[1]))
                maximum = float(fields[2])
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   fields[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in clocks if maximum is None or c > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": maximum,
                "reasons": sorted(reasons), "samples": len(clocks),
                "window": "samples taken while the timed graph replays ran (0.25 s of the same load, then the timed pass)"}


# --------------------------------------------------------------------------- operators
class Case:
    """One operator on one device: resident launch, end-to-end launch, CPU sample."""

    name = ""
    launches_per_step = 1      # kernels of ours one step launches

    def __init__(self, device):
        from intent_b200 import workloads
        self.device = device
        self.workloads = workloads
        self._pipeline = None

    @property
    def pipeline(self):
        """The end-to-end pipeline, built on first use: its device buffers and streams do not exist
        while the device-resident figure is being measured."""
        if self._pipeline is None:
            self._pipeline = self.make_pipeline()
        return self._pipeline

    @property
    def h2d(self):
        return self.pipeline.h2d

    @property
    def d2h(self):
        return self.pipeline.d2h

    def rotate(self, step: int):
        """Hook for cases whose working set is smaller than L2: pick a buffer set."""

    def launch(self, step: int) -> None:
        raise NotImplementedError

    def e2e(self, step: int) -> None:
        raise NotImplementedError


def pinned(tensor: torch.Tensor) -> torch.Tensor:
    return tensor.contiguous().pin_memory()


class PipelinedEndToEnd:
    """End-to-end steps through the artifact API with the copies of neighbouring steps overlapped, the
    way a throughput caller uses `B200Call.enqueue(stream)`: step i's host-to-device copy, its launch
    and its device-to-host copy run on three streams, over two sets of device buffers, so the PCIe
    link carries both directions at once.  Every step still copies its own inputs in and its own
    result out; the timed region ends when the last result has landed in pinned host memory."""

    def __init__(self, kernel, host_inputs, scalars, device, adapt=None, build=None):
        """One kernel: `kernel.prepare(*device buffers, *scalars)`, its result travels back.  Several:
        `build(device buffers)` returns the prepared calls in launch order and the tensors that travel back."""
        self.host_in = [pinned(t) for t in host_inputs]
        self.slots = []
        for _ in range(2):
            device_in = [torch.empty_like(t, device=device) for t in host_inputs]
            if build is not None:
                calls, results = build(device_in)
            else:
                call = kernel.prepare(*(adapt(device_in) if adapt else device_in), *scalars)
                calls, results = [call], [call.result()]
            self.slots.append((device_in, calls, results))
        self.host_out = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in self.slots[0][2]]
        self.streams = [torch.cuda.Stream(device=device) for _ in range(3)]   # in, launch, out
        self.copied_in = [torch.cuda.Event() for _ in range(2)]
        self.launched = [torch.cuda.Event() for _ in range(2)]
        self.copied_out = [torch.cuda.Event() for _ in range(2)]
        self.h2d = sum(t.numel() * t.element_size() for t in host_inputs)
        self.d2h = sum(r.numel() * r.element_size() for r in self.slots[0][2])
        self.used = [False, False]

    def step(self, index: int) -> None:
        slot = index % 2
        device_in, calls, results = self.slots[slot]
        copy_in, launch, copy_out = self.streams
        with torch.cuda.stream(copy_in):
            if self.used[slot]:
                copy_in.wait_event(self.launched[slot])      # the launch two steps ago has read these buffers
            for target, source in zip(device_in, self.host_in):
                target.copy_(source, non_blocking=True)
            self.copied_in[slot].record(copy_in)
        launch.wait_event(self.copied_in[slot])
        if self.used[slot]:
            launch.wait_event(self.copied_out[slot])         # its result has left the output buffer
        for call in calls:
            call.enqueue(launch)
        self.launched[slot].record(launch)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(self.launched[slot])
            for target, source in zip(self.host_out, results):
                target.copy_(source, non_blocking=True)
            self.copied_out[slot].record(copy_out)
        self.used[slot] = True

    def begin(self) -> None:
        """After the start event: the three streams start behind the current stream."""
        for stream in self.streams:
            stream.wait_stream(torch.cuda.current_stream())

    def finish(self) -> None:
        """Before the stop event: the current stream waits until the last result is in host memory."""
        for stream in self.streams:
            torch.cuda.current_stream().wait_stream(stream)


class SoftmaxCase(Case):
    name = "softmax"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.softmax_workload()
        (self.host_x,) = self.workloads.softmax_inputs()
        # 32 MB per launch fits L2 (126 MB): rotate over 12 buffer pairs (384 MB) so DRAM is measured
        self.sets = [(self.host_x.to(device) + 0, torch.empty(4096, 1024, device=device)) for _ in range(12)]
        self.flush = "rotating 12 buffer pairs (384 MB > L2)"
        self.kernel = b200.jit(b200.kernels.stable_softmax)
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, [self.host_x], (), device)

    def launch(self, step):
        x, y = self.sets[step % len(self.sets)]
        self.ops.softmax(x, out=y)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        return lambda: oracle.softmax(self.host_x, workers=workers), 1.0, "full workload (4096 rows)"


class LayerNormCase(Case):
    name = "layer_norm"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.layer_norm_workload()
        self.host = self.workloads.layer_norm_inputs()
        x, w, b, self.inv, self.eps = self.host
        self.x, self.w, self.b = x.to(device), w.to(device), b.to(device)
        self.y = torch.empty_like(self.x)
        self.flush = "inputs larger than L2 (268 MB per launch vs 126 MB)"
        self.kernel = b200.jit(b200.kernels.layer_norm_f16)
        # x travels every step; gamma and beta are parameters that stay on the device
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, [x], (self.w, self.b, self.inv, self.eps), device)

    def launch(self, step):
        self.ops.layer_norm(self.x, self.w, self.b, self.inv, self.eps, out=self.y)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        x, w, b, inv, eps = self.host
        return lambda: oracle.layer_norm(x, w, b, inv, eps, workers=workers), 1.0, "full workload (16384 rows)"


class GemmCase(Case):
    name = "gemm"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.gemm_workload()
        a, b = self.workloads.gemm_inputs()
        self.host_a, self.host_b = a, b
        self.a, self.b = a.to(device), b.t().contiguous().to(device).t()
        self.c = torch.empty(8192, 8192, dtype=torch.float16, device=device)
        self.flush = "inputs larger than L2 (403 MB per launch vs 126 MB)"
        self.kernel = b200.jit(b200.kernels.gemm, constexprs={"ACTIVATION": "NONE"})
        # B travels in its column-major storage (the transposed matrix is the contiguous one)
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, [a, b.t().contiguous()], (), device,
                                          adapt=lambda buffers: (buffers[0], buffers[1].t()))

    def launch(self, step):
        self.ops.gemm(self.a, self.b, out=self.c)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        rows = 64
        out = torch.empty(8192, 8192, dtype=torch.float16)
        return (lambda: oracle.gemm(self.host_a, self.host_b, rows=(0, rows), out=out, workers=workers),
                rows / 8192, f"{rows} of 8192 rows of C (full K and N)")


class AttentionCase(Case):
    name = "attention"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.attention_workload()
        q, k, v, self.scale = self.workloads.attention_inputs()
        self.host = (q, k, v)
        self.q, self.k, self.v = q.to(device), k.to(device), v.to(device)
        self.o = torch.empty_like(self.q)
        self.flush = "inputs larger than L2 (1074 MB per launch vs 126 MB)"
        self.kernel = b200.jit(b200.kernels.flash_attention_bf16_fwd, constexprs={"HEAD_GROUP": 1, "CAUSAL": True})
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, [q, k, v], (self.scale,), device)

    def launch(self, step):
        self.ops.flash_attention(self.q, self.k, self.v, self.scale, out=self.o)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        q, k, v = self.host
        units = max(1, workers)
        out = torch.empty_like(q)
        return (lambda: oracle.attention(q, k, v, self.scale, units=(0, units), out=out, workers=workers),
                units / 256, f"{units} of 256 (batch, head) units, full sequence")


class SpmmCase(Case):
    name = "spmm"
    launches_per_step = 2      # two column-block launches at this shape

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.spmm_workload()
        self.host = self.workloads.csr_inputs()
        self.dev = [t.to(device) for t in self.host]
        self.y = torch.empty(262144, 128, device=device)
        self.flush = "inputs larger than L2 (337 MB compulsory per launch vs 126 MB)"
        self.kernel = b200.jit(b200.kernels.csr_spmm_262144)
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, list(self.host), (), device)

    def launch(self, step):
        self.ops.csr_spmm(*self.dev, out=self.y)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        return lambda: oracle.csr_spmm(*self.host, workers=workers), 1.0, "full workload (262144 rows)"


class SoftmaxBackwardCase(Case):
    name = "softmax_backward"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.softmax_backward_workload()
        self.host = self.workloads.softmax_backward_inputs()
        # 201 MB per launch exceeds L2 (126 MB), but a good part of one working set would survive in it
        # between launches: two sets alternate (403 MB), so every launch reads from DRAM
        self.sets = [tuple(t.to(device) + 0 for t in self.host) + (torch.empty(4096, 4097, device=device),)
                     for _ in range(2)]
        self.flush = "alternating two copies of the operands (403 MB > L2)"
        self.kernel = b200.jit(b200.kernels.softmax_backward)
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, list(self.host), (), device)

    def launch(self, step):
        p, u, g = self.sets[step % 2]
        self.ops.softmax_backward(p, u, out=g)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        return lambda: oracle.softmax_backward(*self.host, workers=workers), 1.0, "full workload (4096 rows)"


class SpmvCase(Case):
    name = "spmv"

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.spmv_workload()
        ro, ci, va, x = self.workloads.csr_inputs(32768, 32768, 32, 1)
        self.host = (ro, ci, va, x[:, 0].contiguous())
        # 8.6 MB per launch fits L2: rotate over 20 copies of the matrix (172 MB) so DRAM is measured
        self.sets = [[t.to(device) + 0 for t in self.host] + [torch.empty(32768, device=device)] for _ in range(20)]
        self.flush = "rotating 20 copies of the operands (172 MB > L2)"
        self.kernel = b200.jit(b200.kernels.csr_spmv)
        self.make_pipeline = lambda: PipelinedEndToEnd(self.kernel, list(self.host), (), device)

    def launch(self, step):
        ro, ci, va, x, y = self.sets[step % len(self.sets)]
        self.ops.csr_spmv(ro, ci, va, x, out=y)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        return lambda: oracle.csr_spmv(*self.host, workers=workers), 1.0, "full workload (32768 rows)"


class LayerNormBackwardCase(Case):
    """Row kernel + partial-sum reduction (two launches per step)."""
    name = "layer_norm_backward"
    launches_per_step = 2

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.layer_norm_backward_workload()
        *tensors, self.inverse = self.workloads.layer_norm_backward_inputs()
        self.host = tuple(tensors)
        # 101 MB per step would fit L2: rotate over three copies of the matrices (302 MB) so DRAM is measured
        self.sets = [[t.to(device) + 0 for t in self.host] + [torch.empty(4096, 4096, dtype=torch.bfloat16, device=device)]
                     for _ in range(3)]
        self.dev = self.sets[0][:7]
        self.dw = torch.empty(4096, device=device)
        self.db = torch.empty(4096, device=device)
        self.flush = "rotating three copies of the operands (302 MB > L2)"
        self.rows = b200.jit(b200.kernels.layer_norm_backward_rows)
        self.reduce = b200.jit(b200.kernels.layer_norm_backward_reduce)

        def build(buffers):
            rows_call = self.rows.prepare(*buffers, self.inverse)
            reduce_call = self.reduce.prepare(buffers[5], buffers[6])
            return [rows_call, reduce_call], [rows_call.result(), *reduce_call.result()]
        self.make_pipeline = lambda: PipelinedEndToEnd(None, list(self.host), (), device, build=build)

    def launch(self, step):
        *operands, dx = self.sets[step % len(self.sets)]
        self.ops.layer_norm_backward_rows(*operands, self.inverse, out=dx)
        self.ops.layer_norm_backward_reduce(operands[5], operands[6], dw=self.dw, db=self.db)

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        x, dy, w, mean, rstd, dw_partial, db_partial = self.host

        def run():
            oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, self.inverse, workers=workers)
            oracle.layer_norm_backward_reduce(dw_partial, db_partial, workers=workers)
        return run, 1.0, "full workload (4096 rows, rows + reduce)"


class AttentionBackwardCase(Case):
    """delta, dK/dV and dQ (three launches per step)."""
    name = "attention_backward"
    launches_per_step = 3

    def __init__(self, device):
        super().__init__(device)
        import intent_b200 as b200
        from intent_b200 import ops
        self.ops, self.workload = ops, self.workloads.attention_backward_workload()
        q, k, v, output, grad_output, lse, self.scale = self.workloads.attention_backward_inputs(
            8, 32, 8, 2048, 128, device=device)
        self.host = (q, k, v, output, grad_output, lse)
        self.dev = [t.to(device) for t in self.host]
        self.delta = torch.empty_like(self.dev[5])
        self.grads = [torch.empty_like(self.dev[0]), torch.empty_like(self.dev[1]), torch.empty_like(self.dev[2])]
        self.flush = "inputs larger than L2 (503 MB of operands and gradients per step vs 126 MB)"
        options = {"HEAD_GROUP": 4, "CAUSAL": True}
        kernels = (b200.jit(b200.kernels.attention_backward_delta),
                   b200.jit(b200.kernels.attention_backward_dkdv, constexprs=options),
                   b200.jit(b200.kernels.attention_backward_dq, constexprs=options))

        def build(buffers):
            qd, kd, vd, od, gd, ld = buffers
            delta_call = kernels[0].prepare(od, gd)
            common = (qd, kd, vd, gd, ld, delta_call.result(), self.scale)
            dkdv_call, dq_call = kernels[1].prepare(*common), kernels[2].prepare(*common)
            return [delta_call, dkdv_call, dq_call], [dq_call.result(), *dkdv_call.result()]
        self.make_pipeline = lambda: PipelinedEndToEnd(None, list(self.host), (), device, build=build)

    def launch(self, step):
        q, k, v, output, grad_output, lse = self.dev
        self.ops.attention_backward_delta(output, grad_output, out=self.delta)
        self.ops.attention_backward_dkdv(q, k, v, grad_output, lse, self.delta, self.scale, head_group=4,
                                         grad_k=self.grads[1], grad_v=self.grads[2])
        self.ops.attention_backward_dq(q, k, v, grad_output, lse, self.delta, self.scale, head_group=4,
                                       grad_q=self.grads[0])

    def e2e(self, step):
        self.pipeline.step(step)

    def cpu(self, oracle, workers):
        # batch 0, key head 0 with its four query heads: 1 of the 64 (batch, key head) groups
        q, k, v, output, grad_output, lse = (t[:1, :4] if t.shape[1] == 32 else t[:1, :1] for t in self.host)

        def run():
            delta = oracle.attention_backward_delta(output, grad_output, workers=workers)
            oracle.attention_backward_dkdv(q, k, v, grad_output, lse, delta, self.scale, head_group=4, workers=workers)
            oracle.attention_backward_dq(q, k, v, grad_output, lse, delta, self.scale, head_group=4, workers=workers)
        return run, 1.0 / 64, "1 of 64 (batch, key head) groups (4 query heads), full sequence"


CASES = {"softmax": SoftmaxCase, "layer_norm": LayerNormCase, "gemm": GemmCase, "attention": AttentionCase,
         "spmm": SpmmCase, "softmax_backward": SoftmaxBackwardCase, "spmv": SpmvCase,
         "layer_norm_backward": LayerNormBackwardCase, "attention_backward": AttentionBackwardCase}


# --------------------------------------------------------------------------- timing
def barrier(distributed: bool) -> None:
    if distributed:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, distributed: bool, device) -> float:
    if not distributed:
        return value
    tensor = torch.tensor([value], dtype=torch.float64, device=device)
    torch.distributed.all_reduce(tensor, op=torch.distributed.ReduceOp.MAX)
    return float(tensor.item())


def timed(function, steps: int, warmup: int, distributed: bool, device, begin=None, finish=None) -> float:
    """Milliseconds per step: CUDA events on the current (launching) stream, max over ranks.  A
    function that spreads its work over other streams gives `begin` (run after the start event: its
    streams wait for the current one) and `finish` (run before the stop event: the current stream
    waits for them), so the two events bracket all of it."""
    for step in range(warmup):
        function(step)
    if finish:
        finish()
    barrier(distributed)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    if begin:
        begin()
    for step in range(steps):
        function(warmup + step)
    if finish:
        finish()
    stop.record()
    barrier(distributed)
    return max_over_ranks(start.elapsed_time(stop), distributed, device) / steps


LOAD_SECONDS = 0.25
CLOCKS = None  # the ClockSampler of this run


def timed_graph(function, steps: int, warmup: int, distributed: bool, device) -> float:
    """Like `timed`, with the K launches captured once in a CUDA graph and replayed, so the
    device time of short kernels is not hidden behind Python's launch cost (the reference's
    own tuner times graph replays, python/intent/runtime/triton/cuda.py:18-43)."""
    for step in range(warmup):
        function(step)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for step in range(steps):
            function(warmup + step)
    graph.replay()
    barrier(distributed)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    window = CLOCKS.window() if CLOCKS is not None else None
    if window:
        window.__enter__()
    # The same load runs for LOAD_SECONDS before the timed pass so that the clock samples
    # (one per 50 ms) describe the state the timed pass sees: a kernel inside a long step.
    deadline = time.time() + LOAD_SECONDS
    while time.time() < deadline:
        graph.replay()
        torch.cuda.synchronize()
    barrier(distributed)
    start.record()
    graph.replay()
    stop.record()
    barrier(distributed)
    if window:
        window.__exit__()
    return max_over_ranks(start.elapsed_time(stop), distributed, device) / steps


def cpu_baseline(case, workers: int) -> dict:
    """Reference CPU timing protocol (python/intent/runtime/mojo/program.py:28-34): evict a
    64 MiB buffer outside the interval, repetitions = min(50, max(1, int(10 ms / first))),
    median of 7 samples (fewer when one run is long), scaled from the sample to the workload."""
    import oracle
    function, fraction, sample = case.cpu(oracle, workers)
    eviction = torch.empty(64 * 1024 * 1024, dtype=torch.uint8)

    def once() -> float:
        oracle.evict(eviction)
        begin = oracle.now_ms()
        function()
        return oracle.now_ms() - begin

    first = once()
    repetitions = min(50, max(1, int(10.0 / first)))
    samples = 7 if first < 1500 else 3 if first < 8000 else 1
    measurements = []
    for _ in range(samples):
        measurements.append(sum(once() for _ in range(repetitions)) / repetitions)
    milliseconds = statistics.median(measurements)
    work = case.workload.work * fraction
    scale = 1e6 if case.workload.unit == "GB/s" else 1e9
    return {"value": work / milliseconds / scale, "unit": case.workload.unit, "cores": workers, "kind": "port",
            "sample": f"{sample}; median of {samples} x {repetitions} runs, 64 MiB eviction outside the interval",
            "ms": milliseconds}


def measure_resident(case, steps: int, warmup: int, distributed: bool, world: int, peak_table: dict,
                     peak_kind: str) -> dict:
    """The device-resident figure and its roofline.  Every operator is measured this way before any
    end-to-end pipeline (extra streams, pinned buffers, PCIe traffic) has run in the process."""
    workload = case.workload
    scale = 1e6 if workload.unit == "GB/s" else 1e9      # bytes/ms -> GB/s, flop/ms -> TFLOP/s
    first_window = len(CLOCKS.windows) if CLOCKS is not None else 0
    resident_ms = timed_graph(case.launch, steps, warmup, distributed, case.device)
    time.sleep(0.06)  # let the sampler deliver the sample that covers the end of the window
    own_clocks = CLOCKS.summary(CLOCKS.windows[first_window:]) if CLOCKS is not None else None
    per_gpu = workload.work / resident_ms / scale
    if workload.bound == "hbm":
        peak, peak_name = peak_table["hbm_gbs"], f"{peak_kind} STREAM-style copy"
        burst = peak
    else:  # timed after 0.25 s of the same load: the sustained cuBLAS figure is the like-for-like peak
        peak, peak_name = peak_table["bf16_tflops_sustained"], f"{peak_kind} cuBLAS bf16 sustained"
        burst = peak_table["bf16_tflops"]
    return {
        "op": case.name, "workload": workload.description, "unit": workload.unit,
        "value": per_gpu * world, "ms_per_step": resident_ms,
        "roofline": {"bound": workload.bound, "achieved": per_gpu, "peak": peak, "unit": workload.unit,
                     "frac": per_gpu / peak, "peak_source": peak_name, "frac_of_burst_peak": per_gpu / burst,
                     "frac_of_nominal": per_gpu / NOMINAL[workload.bound],
                     "traffic": NCU_TRAFFIC_BYTES[case.name], "algorithmic": workload.work},
        "l2": case.flush, "clocks": own_clocks,
    }


def measure_end_to_end(case, steps: int, distributed: bool, world: int, with_cpu: bool) -> dict:
    """The same metric through the artifact API with host buffers, then the CPU sample."""
    workload = case.workload
    scale = 1e6 if workload.unit == "GB/s" else 1e9
    pipeline = case.pipeline
    # a two-deep pipeline needs enough steps for its fill and drain not to dominate
    e2e_ms = timed(case.e2e, steps, 2, distributed, case.device, begin=pipeline.begin, finish=pipeline.finish)
    result = {"e2e": {"value": workload.work / e2e_ms / scale * world, "unit": workload.unit, "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": case.h2d, "d2h_bytes_per_step": case.d2h}}
    if with_cpu:
        import oracle
        result["cpu_baseline"] = cpu_baseline(case, oracle.default_workers())
    return result


def run_reference(arguments, rank: int) -> None:
    """The reference's CPU implementation of the path (the oracle port: the reference
    itself cannot be compiled here) on every host thread; rank 0 only."""
    if rank != 0:
        return
    import oracle
    from intent_b200 import workloads

    class HostCase:
        workload = workloads.layer_norm_workload()

        def __init__(self):
            self.host = workloads.layer_norm_inputs()

        def cpu(self, module, workers):
            x, w, b, inv, eps = self.host
            return lambda: module.layer_norm(x, w, b, inv, eps, workers=workers), 1.0, "full workload (16384 rows)"

    workers = len(os.sched_getaffinity(0))
    case = HostCase()
    function, _, sample = case.cpu(oracle, workers)
    for _ in range(arguments.warmup):
        function()
    begin = time.perf_counter()
    for _ in range(arguments.steps):
        function()
    milliseconds = (time.perf_counter() - begin) * 1e3 / arguments.steps
    value = case.workload.work / milliseconds / 1e6
    print(json.dumps({
        "impl": "reference", "metric": "layer_norm throughput (algorithmic bytes / time)",
        "value": value, "unit": "GB/s", "n_gpus": arguments.gpus, "steps": arguments.steps,
        "warmup": arguments.warmup, "ms_per_step": milliseconds, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": case.workload.description, "host_threads": workers},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": workers, "kind": "port",
                         "sample": f"{sample}, {arguments.steps} timed passes"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--op", default="all", choices=["all", *CASES])
    arguments = parser.parse_args()
    arguments.warmup = max(arguments.warmup, 3) if arguments.impl == "b200" else arguments.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if arguments.impl == "reference":
        run_reference(arguments, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: intent_b200 has no CPU execution path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner on stdout at the first collective; stdout carries the
        # one JSON line only, so the banner is sent to stderr.
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            torch.distributed.init_process_group("nccl", device_id=device)
            torch.distributed.barrier()
            torch.cuda.synchronize()
        finally:
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    from intent_b200 import _native
    _native.library()                                     # fail loudly if the CUDA extension is missing
    peak_table, peak_kind = peaks()
    names = list(CASES) if arguments.op == "all" else [arguments.op]
    primary = "layer_norm" if arguments.op == "all" else arguments.op
    names.sort(key=lambda name: name != primary)           # the headline workload runs first
    results, launches = {}, 0
    global CLOCKS
    with ClockSampler(local_rank) as clocks:
        CLOCKS = clocks
        steps, cases = arguments.steps, {}
        for name in names:               # pass 1: device-resident figures of every operator
            try:
                cases[name] = CASES[name](device)
                results[name] = measure_resident(cases[name], steps, arguments.warmup, distributed, world, peak_table,
                                                 peak_kind)
            except Exception as error:  # one failing operator must not hide the others
                if name == primary:
                    raise
                cases.pop(name, None)
                results[name] = {"op": name, "error": f"{type(error).__name__}: {error}"}
        for name in names:               # pass 2: end to end through the artifact API, and the CPU sample
            case = cases.pop(name, None)
            if case is None:
                continue
            try:
                results[name].update(measure_end_to_end(case, steps, distributed, world,
                                                        with_cpu=(rank == 0 and world == 1)))
                # warm-up, the captured pass, the timed replay (the 0.25 s of load replays before it
                # are not counted), then the end-to-end warm-up and steps
                launches += case.launches_per_step * (arguments.warmup + 3 * steps + steps + 2)
            except Exception as error:
                if name == primary:
                    raise
                results[name] = {"op": name, "error": f"{type(error).__name__}: {error}"}
            del case
            gc.collect()
            torch.cuda.empty_cache()
    clock_summary = clocks.summary()
    if distributed:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank != 0:
        return
    head = results[primary]
    line = {
        "metric": f"{head['op']} throughput (algorithmic {'bytes' if head['unit'] == 'GB/s' else 'flops'} / time)",
        "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": arguments.steps,
        "warmup": arguments.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": {"softmax": "f32", "layer_norm": "f16", "gemm": "f16", "attention": "bf16", "spmm": "f32",
                  "softmax_backward": "f32", "spmv": "f32", "layer_norm_backward": "bf16",
                  "attention_backward": "f16"}[primary],
        "data": "synthetic",
        "config": {"workload": head["workload"], "l2": head["l2"],
                   "parallelism": f"{world} independent shard(s), no data-path collective"},
        "roofline": head["roofline"], "e2e": head["e2e"], "gpu_launches": launches,
        "clocks": head.get("clocks") or clock_summary,
        "ops": [results[name] for name in names],
    }
    if "cpu_baseline" in head:
        line["cpu_baseline"] = head["cpu_baseline"]
    print(json.dumps(line))


if __name__ == "__main__":
    main()
