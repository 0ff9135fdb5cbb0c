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
NCU_TRAFFIC_BYTES = {"softmax": 32286000,      # steady state over rotating operand sets (mean of nine launches)
                     "layer_norm": 217463040, "gemm": 1222019160, "attention": 1059586816,
                     "spmm": 983705088, "softmax_backward": 160885760, "spmv": 8672256,
                     # steps of several kernels: the sum over the step's launches
                     "layer_norm_backward": 74406912 + 2109440, "attention_backward": 274570496 + 846483200}


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
L2_BYTES = 126e6
ROTATION_BYTES = 2.6 * L2_BYTES      # buffer sets rotate until one round touches this much per GPU
FLUSH_BYTES = 1.5 * L2_BYTES         # launches on other operand sets that precede the timed replay touch this much


def region_of(flat_rows):
    """A transfer region for HostBuffers: the rank's block [begin, end) of an operand's leading
    axis, or of its flattened (batch, head) axis for attention operands."""
    begin, end, heads = flat_rows

    def cut(tensor):
        if heads:
            from intent_b200.sharding import _flat_heads
            return _flat_heads(tensor, "operand")[begin:end]
        return tensor[begin:end]
    return cut


class Case:
    """One operator on one rank.

    `value`: K launches of prepared calls (`jit(...).prepare(...)`, then `call.launch()`), inputs
    resident in HBM.  With N > 1 ranks every rank holds the full operands and the call is made
    with ``backend_options={"gpus": N}``: each rank computes its block of units (strong scaling);
    the same call with ``gather_output=True`` adds the NCCL all-gather.  Buffer sets rotate so
    that consecutive launches on one GPU never find their operands in L2.
    `e2e`: the same call fed from HOST buffers through `intent_b200.HostBuffers`: every step
    copies the rank's block of the inputs in and its block of the result out."""

    name = ""
    family = ""                 # the partition rule (intent_b200.sharding)
    launches_per_step = 1
    resident = ()               # input positions that are parameters kept on the device end to end
    head_group = 1
    min_sets = 1

    def __init__(self, device, rank: int, world: int):
        import intent_b200 as b200
        from intent_b200 import sharding, workloads
        self.b200, self.sharding, self.workloads = b200, sharding, workloads
        self.device, self.rank, self.world = device, rank, world
        self.setup()
        self.calls = {}

    # -- per operator ---------------------------------------------------------------
    def setup(self):
        """Sets self.workload, self.host (inputs in declaration order, scalars included),
        self.definition, self.constexprs."""
        raise NotImplementedError

    def shard_bytes(self, world: int) -> float:
        """Bytes one launch touches on one GPU when the call is spread over `world` ranks."""
        raise NotImplementedError

    def cpu(self, oracle, workers):
        raise NotImplementedError

    # -- machinery ------------------------------------------------------------------
    def kernel(self, world: int, gather: bool):
        options = {"gpus": world, "gather_output": gather} if world > 1 else None
        return self.b200.jit(self.definition, constexprs=self.constexprs, backend_options=options)

    def to_device(self, value, shared):
        if not isinstance(value, torch.Tensor):
            return value
        if id(value) in shared:
            return shared[id(value)]
        return value.to(self.device)        # keeps the strides of dense tensors (column-major B)

    def prepare(self, world: int, gather: bool = False):
        """Prepared calls over rotating buffer sets for a call spread over `world` ranks."""
        key = (world, gather)
        if key in self.calls:
            return self.calls[key]
        count = min(96, max(self.min_sets, math.ceil(ROTATION_BYTES / self.shard_bytes(world))))
        kernel = self.kernel(world, gather)
        # parameters and operands every rank reads whole are shared between the sets
        shared = {id(self.host[p]): self.host[p].to(self.device) for p in self.replicated(world)}
        sets = self.operand_sets(count, shared)
        prepared = [kernel.prepare(*operands) for operands in sets]
        description = f"rotating {count} operand sets ({count * self.shard_bytes(world) / 1e6:.0f} MB per GPU per round > L2)" \
            if count > 1 else f"operands larger than L2 ({self.shard_bytes(world) / 1e6:.0f} MB per launch per GPU vs 126 MB)"
        self.calls[key] = (prepared, description)
        return self.calls[key]

    _device_sets = None

    def operand_sets(self, count, shared):
        """`count` device copies of the operands; copies are made once and reused by every
        (world, gather) variant, which differ only in how they cut them."""
        if self._device_sets is None:
            self._device_sets = []
        while len(self._device_sets) < count:
            self._device_sets.append(tuple(self.to_device(value, shared) for value in self.host))
        return self._device_sets[:count]

    def replicated(self, world: int):
        """Input positions that are not cut by the partition rule."""
        return self.resident_inputs

    def launcher(self, world: int, gather: bool = False):
        prepared, _ = self.prepare(world, gather)
        return lambda step: prepared[step % len(prepared)].launch()

    def flush_launches(self, world: int) -> int:
        return max(1, math.ceil(FLUSH_BYTES / self.shard_bytes(world)))

    def release(self):
        self.calls.clear()
        self._device_sets = None


class EndToEnd:
    """Steps fed from host memory through `HostBuffers` and `B200Call.enqueue(stream)`: step i's
    host-to-device copies, its launch and its device-to-host copies run on three streams over two
    scopes (two sets of device twins), so the PCIe link carries both directions at once.  Every
    step copies the rank's block of every non-resident input in and its block of the result out;
    the timed region ends when the last result is in page-locked host memory."""

    def __init__(self, case, world: int):
        b200, device = case.b200, case.device
        kernel = case.kernel(world, False)
        self.slots = []
        self.pinned = {}
        self.h2d = self.d2h = 0
        for _ in range(2):
            scope = b200.HostBuffers(device)
            operands = []
            for position, value in enumerate(case.host):
                if not isinstance(value, torch.Tensor):
                    operands.append(value)
                elif position in case.resident:
                    operands.append(value.to(device))
                else:    # the step's inputs travel from page-locked host memory
                    pinned = self.pinned.setdefault(position, b200.HostBuffers.page_locked(value))
                    operands.append(scope.input(pinned, region=case.input_region(position, world)))
            call = kernel.prepare(*operands)
            results = call.result() if isinstance(call.result(), tuple) else (call.result(),)
            for result in results:
                scope.result(result, region=case.output_region(world))
            self.slots.append((scope, call))
            self.h2d, self.d2h = scope.bytes_in, scope.bytes_out
        self.streams = [torch.cuda.Stream(device=device) for _ in range(3)]   # in, launch, out
        self.copied_in = [torch.cuda.Event() for _ in range(2)]
        self.launched = [torch.cuda.Event() for _ in range(2)]
        self.copied_out = [torch.cuda.Event() for _ in range(2)]
        self.used = [False, False]

    def step(self, index: int) -> None:
        slot = index % 2
        scope, call = self.slots[slot]
        copy_in, launch, copy_out = self.streams
        if self.used[slot]:
            copy_in.wait_event(self.launched[slot])          # the launch two steps ago has read these buffers
        scope.stage_in(copy_in)
        self.copied_in[slot].record(copy_in)
        launch.wait_event(self.copied_in[slot])
        if self.used[slot]:
            launch.wait_event(self.copied_out[slot])         # its result has left the output buffer
        call.enqueue(launch)
        self.launched[slot].record(launch)
        copy_out.wait_event(self.launched[slot])
        scope.stage_out(copy_out)
        self.copied_out[slot].record(copy_out)
        self.used[slot] = True

    def begin(self) -> None:
        for stream in self.streams:
            stream.wait_stream(torch.cuda.current_stream())

    def finish(self) -> None:
        for stream in self.streams:
            torch.cuda.current_stream().wait_stream(stream)

    def close(self) -> None:
        torch.cuda.synchronize()
        for scope, _ in self.slots:
            scope.close()
        self.slots.clear()


class RowCase(Case):
    """Operators cut along the rows of their first operand and of their output."""
    cut_inputs = (0,)

    @property
    def resident_inputs(self):
        return tuple(p for p, v in enumerate(self.host) if isinstance(v, torch.Tensor) and p not in self.cut_inputs)

    def rows(self):
        return self.host[self.cut_inputs[0]].shape[0]

    def block(self, world):
        return self.sharding.unit_range(self.rows(), self.rank, world)

    def input_region(self, position, world):
        if world == 1 or position not in self.cut_inputs:
            return None
        return region_of((*self.block(world), 0))

    def output_region(self, world):
        return None if world == 1 else region_of((*self.block(world), 0))


class SoftmaxCase(RowCase):
    name, family = "softmax", "softmax"

    def setup(self):
        self.workload = self.workloads.softmax_workload()
        self.host = self.workloads.softmax_inputs()
        self.definition, self.constexprs = self.b200.kernels.stable_softmax, None

    def shard_bytes(self, world):
        return self.workload.work / world

    def cpu(self, oracle, workers):
        return lambda: oracle.softmax(self.host[0], workers=workers), 1.0, "full workload (4096 rows)"


class LayerNormCase(RowCase):
    name, family = "layer_norm", "layer_norm"
    resident = (1, 2)            # gamma and beta are parameters that stay on the device
    min_sets = 2                 # 268 MB exceeds L2, but part of one set would survive in it between launches

    def setup(self):
        self.workload = self.workloads.layer_norm_workload()
        self.host = self.workloads.layer_norm_inputs()
        self.definition, self.constexprs = self.b200.kernels.layer_norm_f16, None

    def shard_bytes(self, world):
        return self.workload.work / world

    def cpu(self, oracle, workers):
        x, w, b, inv, eps = self.host
        return lambda: oracle.layer_norm(x, w, b, inv, eps, workers=workers), 1.0, "full workload (16384 rows)"


class GemmCase(RowCase):
    name, family = "gemm", "gemm"

    def setup(self):
        self.workload = self.workloads.gemm_workload()
        self.host = self.workloads.gemm_inputs()          # B is the transposed view of a contiguous (N, K)
        self.definition, self.constexprs = self.b200.kernels.gemm, {"ACTIVATION": "NONE"}

    def shard_bytes(self, world):
        return 8192 * 8192 * 2 * (1 + 2 / world)          # all of B, the rank's rows of A and C

    def cpu(self, oracle, workers):
        rows = 64
        out = torch.empty(8192, 8192, dtype=torch.float16)
        a, b = self.host
        return (lambda: oracle.gemm(a, b, rows=(0, rows), out=out, workers=workers),
                rows / 8192, f"{rows} of 8192 rows of C (full K and N)")


class AttentionCase(Case):
    name, family = "attention", "flash_attention"
    resident_inputs = ()

    def setup(self):
        self.workload = self.workloads.attention_workload()
        self.host = self.workloads.attention_inputs()
        self.definition = self.b200.kernels.flash_attention_bf16_fwd
        self.constexprs = {"HEAD_GROUP": 1, "CAUSAL": True}

    def shard_bytes(self, world):
        return 4 * 8 * 32 * 4096 * 128 * 2 / world

    def block(self, world):
        return self.sharding.unit_range(8 * 32, self.rank, world)

    def input_region(self, position, world):
        return None if world == 1 else region_of((*self.block(world), 1))

    def output_region(self, world):
        return None if world == 1 else region_of((*self.block(world), 1))

    def cpu(self, oracle, workers):
        q, k, v, scale = self.host
        units = max(1, workers)
        out = torch.empty_like(q)
        return (lambda: oracle.attention(q, k, v, scale, units=(0, units), out=out, workers=workers),
                units / 256, f"{units} of 256 (batch, head) units, full sequence")


class SpmmCase(RowCase):
    name, family = "spmm", "csr_spmm"
    cut_inputs = (0,)

    def setup(self):
        self.workload = self.workloads.spmm_workload()
        self.host = self.workloads.csr_inputs()
        self.definition, self.constexprs = self.b200.kernels.csr_spmm_262144, None

    def rows(self):
        return self.host[0].numel() - 1

    def shard_bytes(self, world):
        return 262144 * 128 * 4 * (1 + 1 / world) + (262144 * 32 * 8 + 262144 * 4) / world

    @property
    def resident_inputs(self):
        return (3,)               # X is read whole by every rank; the index and value arrays are cut by offset

    def input_region(self, position, world):
        if world == 1 or position == 3:
            return None
        begin, end = self.block(world)
        if position == 0:
            return lambda t: t[begin:end + 1]
        first, last = int(self.host[0][begin]), int(self.host[0][end])
        return lambda t: t[first:last]     # the non-zeros of the rank's rows

    def cpu(self, oracle, workers):
        return lambda: oracle.csr_spmm(*self.host, workers=workers), 1.0, "full workload (262144 rows)"


class SoftmaxBackwardCase(RowCase):
    name, family = "softmax_backward", "softmax_backward"
    cut_inputs = (0, 1)
    min_sets = 2

    def setup(self):
        self.workload = self.workloads.softmax_backward_workload()
        self.host = self.workloads.softmax_backward_inputs()
        self.definition, self.constexprs = self.b200.kernels.softmax_backward, None

    def shard_bytes(self, world):
        return self.workload.work / world

    def cpu(self, oracle, workers):
        return lambda: oracle.softmax_backward(*self.host, workers=workers), 1.0, "full workload (4096 rows)"


class SpmvCase(RowCase):
    name, family = "spmv", "csr_spmv"

    def setup(self):
        self.workload = self.workloads.spmv_workload()
        ro, ci, va, x = self.workloads.csr_inputs(32768, 32768, 32, 1)
        self.host = (ro, ci, va, x[:, 0].contiguous())
        self.definition, self.constexprs = self.b200.kernels.csr_spmv, None

    def rows(self):
        return self.host[0].numel() - 1

    @property
    def resident_inputs(self):
        return ()

    def shard_bytes(self, world):
        return self.workload.work / world

    input_region = SpmmCase.input_region

    def cpu(self, oracle, workers):
        return lambda: oracle.csr_spmv(*self.host, workers=workers), 1.0, "full workload (32768 rows)"


class SequenceCase(Case):
    """Steps of several kernels (the backward pairs): single-GPU figures only."""
    single_gpu_only = True

    def prepare(self, world, gather=False):
        raise NotImplementedError


class LayerNormBackwardCase(SequenceCase):
    """Row kernel + partial-sum reduction (two launches per step)."""
    name = "layer_norm_backward"
    launches_per_step = 2

    def setup(self):
        b200 = self.b200
        self.workload = self.workloads.layer_norm_backward_workload()
        *tensors, self.inverse = self.workloads.layer_norm_backward_inputs()
        self.host = tuple(tensors)
        self.rows_kernel = b200.jit(b200.kernels.layer_norm_backward_rows)
        self.reduce_kernel = b200.jit(b200.kernels.layer_norm_backward_reduce)

    def build(self, buffers):
        rows_call = self.rows_kernel.prepare(*buffers, self.inverse)
        reduce_call = self.reduce_kernel.prepare(buffers[5], buffers[6])
        return [rows_call, reduce_call], [rows_call.result(), *reduce_call.result()]

    def launcher(self, world, gather=False):
        # 101 MB per step would fit L2: rotate over three copies of the matrices (302 MB) so DRAM is measured
        sets = [self.build([t.to(self.device) + 0 for t in self.host])[0] for _ in range(3)]
        self.flush = "rotating three copies of the operands (302 MB > L2)"

        def launch(step):
            for call in sets[step % 3]:
                call.launch()
        return launch

    def cpu(self, oracle, workers):
        x, dy, w, mean, rstd, dw_partial, db_partial = self.host

        def run():
            oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, self.inverse, workers=workers)
            oracle.layer_norm_backward_reduce(dw_partial, db_partial, workers=workers)
        return run, 1.0, "full workload (4096 rows, rows + reduce)"


class AttentionBackwardCase(SequenceCase):
    """delta, dK/dV and dQ (three launches per step)."""
    name = "attention_backward"
    launches_per_step = 3

    def setup(self):
        b200 = self.b200
        self.workload = self.workloads.attention_backward_workload()
        q, k, v, output, grad_output, lse, self.scale = self.workloads.attention_backward_inputs(
            8, 32, 8, 2048, 128, device=self.device)
        self.host = (q, k, v, output, grad_output, lse)
        options = {"HEAD_GROUP": 4, "CAUSAL": True}
        self.kernels = (b200.jit(b200.kernels.attention_backward_delta),
                        b200.jit(b200.kernels.attention_backward_dkdv, constexprs=options),
                        b200.jit(b200.kernels.attention_backward_dq, constexprs=options))

    def build(self, buffers):
        qd, kd, vd, od, gd, ld = buffers
        delta_call = self.kernels[0].prepare(od, gd)
        common = (qd, kd, vd, gd, ld, delta_call.result(), self.scale)
        dkdv_call, dq_call = self.kernels[1].prepare(*common), self.kernels[2].prepare(*common)
        return [delta_call, dkdv_call, dq_call], [dq_call.result(), *dkdv_call.result()]

    def launcher(self, world, gather=False):
        calls, _ = self.build([t.to(self.device) for t in self.host])
        self.flush = "inputs larger than L2 (503 MB of operands and gradients per step vs 126 MB)"

        def launch(step):
            for call in calls:
                call.launch()
        return launch

    def cpu(self, oracle, workers):
        # batch 0, key head 0 with its four query heads: 1 of the 64 (batch, key head) groups
        q, k, v, output, grad_output, lse = (t[:1, :4] if t.shape[1] == 32 else t[:1, :1] for t in self.host)

        def run():
            delta = oracle.attention_backward_delta(output, grad_output, workers=workers)
            oracle.attention_backward_dkdv(q, k, v, grad_output, lse, delta, self.scale, head_group=4, workers=workers)
            oracle.attention_backward_dq(q, k, v, grad_output, lse, delta, self.scale, head_group=4, workers=workers)
        return run, 1.0 / 64, "1 of 64 (batch, key head) groups (4 query heads), full sequence"


class SequenceEndToEnd(EndToEnd):
    """EndToEnd for a step of several prepared calls."""

    def __init__(self, case, world):
        b200, device = case.b200, case.device
        self.slots = []
        for _ in range(2):
            scope = b200.HostBuffers(device)
            self.pinned = getattr(self, "pinned", None) or [b200.HostBuffers.page_locked(t) for t in case.host]
            calls, results = case.build([scope.input(t) for t in self.pinned])
            for result in results:
                scope.result(result)
            sequence = b200.PreparedSequence(calls, outputs=tuple(results), owners=(scope,))
            self.slots.append((scope, sequence))
            self.h2d, self.d2h = scope.bytes_in, scope.bytes_out
        self.streams = [torch.cuda.Stream(device=device) for _ in range(3)]
        self.copied_in = [torch.cuda.Event() for _ in range(2)]
        self.launched = [torch.cuda.Event() for _ in range(2)]
        self.copied_out = [torch.cuda.Event() for _ in range(2)]
        self.used = [False, False]


CASES = {"softmax": SoftmaxCase, "layer_norm": LayerNormCase, "gemm": GemmCase, "attention": AttentionCase,
         "spmm": SpmmCase, "softmax_backward": SoftmaxBackwardCase, "spmv": SpmvCase,
         "layer_norm_backward": LayerNormBackwardCase, "attention_backward": AttentionBackwardCase}
BASELINE_OPS = ("softmax", "layer_norm", "gemm", "attention", "spmm")     # the five configurations of the metric
DTYPES = {"softmax": "f32", "layer_norm": "f16", "gemm": "f16", "attention": "bf16", "spmm": "f32",
          "softmax_backward": "f32", "spmv": "f32", "layer_norm_backward": "bf16", "attention_backward": "f16"}


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


def timed_graph(function, steps: int, warmup: int, distributed: bool, device, flush_launches: int = 1) -> float:
    """Like `timed`, with the K launches captured once in a CUDA graph and replayed, so the
    device time of short kernels is not hidden behind Python's launch cost (the reference's
    own tuner times graph replays, python/intent/runtime/triton/cuda.py:18-43).

    A second graph holds `flush_launches` further launches, which continue the rotation over the
    operand sets and together touch more than L2 holds; it is the last thing that runs before the
    timed replay, so the K timed launches read their operands from DRAM even when K of them alone
    would fit L2."""
    for step in range(warmup):
        function(step)
    torch.cuda.synchronize()
    graph, flush = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for step in range(steps):
            function(warmup + step)
    with torch.cuda.graph(flush):
        for step in range(flush_launches):
            function(warmup + steps + step)
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
        flush.replay()
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


def timed_case(launch, steps, warmup, distributed, device, flush_launches=1) -> tuple[float, dict | None]:
    first_window = len(CLOCKS.windows) if CLOCKS is not None else 0
    milliseconds = timed_graph(launch, steps, warmup, distributed, device, flush_launches)
    time.sleep(0.06)  # let the sampler deliver the sample that covers the end of the window
    clocks = CLOCKS.summary(CLOCKS.windows[first_window:]) if CLOCKS is not None else None
    return milliseconds, clocks


def roofline_of(workload, name: str, per_gpu: float, peak_table: dict, peak_kind: str) -> dict:
    if workload.bound == "hbm":
        peak, peak_name = peak_table["hbm_gbs"], f"{peak_kind} STREAM-style copy"
        burst = peak
    else:  # timed after 0.25 s of the same load: the sustained cuBLAS figure is the like-for-like peak
        peak, peak_name = peak_table["bf16_tflops_sustained"], f"{peak_kind} cuBLAS bf16 sustained"
        burst = peak_table["bf16_tflops"]
    traffic = NCU_TRAFFIC_BYTES.get(name)
    return {"bound": workload.bound, "achieved": per_gpu, "peak": peak, "unit": workload.unit,
            "frac": per_gpu / peak, "peak_source": peak_name, "frac_of_burst_peak": per_gpu / burst,
            "frac_of_nominal": per_gpu / NOMINAL[workload.bound],
            "traffic": traffic, "traffic_ratio": traffic / workload.work if traffic and workload.bound == "hbm" else None,
            "algorithmic": workload.work}


def measure_resident(case, steps: int, warmup: int, distributed: bool, world: int, peak_table: dict,
                     peak_kind: str) -> dict:
    """Device-resident figures.  One GPU: the whole workload per launch.  N GPUs: the workload
    split over the ranks (strong scaling, max over ranks), the same with the final all-gather,
    and every rank running the whole workload by itself (replicas) for comparison.  Every figure
    is taken before any end-to-end pipeline (extra streams, pinned buffers, PCIe traffic) has run."""
    workload = case.workload
    scale = 1e6 if workload.unit == "GB/s" else 1e9      # bytes/ms -> GB/s, flop/ms -> TFLOP/s
    sequence = getattr(case, "single_gpu_only", False)
    split = world if not sequence else 1
    launch = case.launcher(split)
    flush = case.flush if sequence else case.prepare(split)[1]
    flushes = 1 if sequence else case.flush_launches(split)
    resident_ms, own_clocks = timed_case(launch, steps, warmup, distributed, case.device, flushes)
    whole_job = workload.work / resident_ms / scale * (world if sequence else 1)
    result = {
        "op": case.name, "workload": workload.description, "unit": workload.unit,
        "value": whole_job, "ms_per_step": resident_ms, "l2": flush, "clocks": own_clocks,
        "scaling": "weak" if sequence and world > 1 else "strong" if world > 1 else "single",
    }
    if world == 1 or sequence:
        result["roofline"] = roofline_of(workload, case.name, workload.work / resident_ms / scale, peak_table, peak_kind)
        if case.name == "layer_norm":    # one operand set alone: part of it survives in L2 between launches
            prepared = case.prepare(1)[0]
            one_ms, _ = timed_case(lambda step: prepared[0].launch(), steps, warmup, distributed, case.device)
            result["one_operand_set"] = {"ms_per_step": one_ms, "value": workload.work / one_ms / scale,
                                         "note": "the same launch over a single 268 MB operand set"}
        return result
    # ---- N > 1: per-GPU roofline of the shard, the all-gather, the replica figure
    per_gpu = workload.work / world / resident_ms / scale
    result["roofline"] = roofline_of(workload, case.name, per_gpu, peak_table, peak_kind)
    result["roofline"]["note"] = "per GPU, on 1/N of the algorithmic work (replicated operands not recounted)"
    gather_ms, _ = timed_case(case.launcher(world, True), steps, warmup, distributed, case.device, flushes)
    output_bytes = OUTPUT_BYTES[case.name]
    collective_ms = max(gather_ms - resident_ms, 1e-6)
    result["gather"] = {
        "ms_per_step": gather_ms, "value": workload.work / gather_ms / scale, "unit": workload.unit,
        "all_gather_ms": collective_ms, "output_bytes": output_bytes,
        "bus_gbs": output_bytes * (world - 1) / world / collective_ms / 1e6,
        "note": "the same launches followed by the NCCL all-gather of the output blocks (gather_output=True); "
                "all_gather_ms is the difference to the launch alone",
    }
    replica_ms, _ = timed_case(case.launcher(1), steps, warmup, distributed, case.device, case.flush_launches(1))
    result["replicas"] = {"ms_per_step": replica_ms, "value": workload.work / replica_ms / scale * world,
                          "unit": workload.unit, "scaling": "weak",
                          "note": "every rank runs the whole workload by itself, no collective"}
    return result


def gather_ceiling(case, result: dict) -> dict:
    """What bounds the SpMM gathers on this device, measured beside the SpMM figure: the rate of
    random 512-byte row reads (`b200_gather_probe`) out of a table that fits L2 (a quarter of X)
    and out of all of X in one pass.  The SpMM call moves nnz * 512 bytes of such reads, so its time
    cannot go below that volume over the L2-resident rate; a single pass over all of X cannot go
    below the volume over the all-of-X rate."""
    from intent_b200 import ops
    dense = case.host[3].to(case.device)
    gathers = case.host[1].numel()
    volume = gathers * 512.0
    names = {0: "4 loads in flight per lane", 1: "8 loads in flight per lane", 2: "16 loads in flight per lane"}
    rates = {}
    for label, table in (("l2_resident", dense[:65536]), ("all_of_x", dense)):
        best = None
        for variant in (0, 1, 2):
            for hints in (False, True):
                launch = lambda step, v=variant, h=hints, tb=table: ops.gather_probe(tb, gathers, variant=v, hints=h)
                for _ in range(2):
                    launch(0)
                torch.cuda.synchronize()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                for _ in range(3):
                    launch(0)
                stop.record()
                torch.cuda.synchronize()
                rate = volume * 3 / start.elapsed_time(stop) / 1e9          # TB/s
                if best is None or rate > best[0]:
                    best = (rate, f"{names[variant]}, {'evict_last' if hints else 'no'} hint")
        rates[label] = {"tb_per_s": best[0], "form": best[1]}
    ops.workspace_status(case.device)
    floor_ms = volume / rates["l2_resident"]["tb_per_s"] / 1e9
    one_pass_ms = volume / rates["all_of_x"]["tb_per_s"] / 1e9
    return {"gather_bytes_per_call": volume, "probe": rates,
            "spmm_gather_tb_per_s": volume / result["ms_per_step"] / 1e9,
            "floor_ms_at_l2_gather_rate": floor_ms, "spmm_over_floor": result["ms_per_step"] / floor_ms,
            "one_pass_ms_at_all_of_x_rate": one_pass_ms, "spmm_over_one_pass": result["ms_per_step"] / one_pass_ms,
            "note": "floor = the call's nnz x 512 B of row gathers at the probe's L2-resident rate (what column "
                    "blocks that stay in L2 could reach with free Y traffic); one_pass = the same volume at the "
                    "rate a single pass over all of X reaches (X is 134 MB; about 60 MB of randomly gathered data "
                    "is what the 126 MB L2 serves at its full rate)"}


OUTPUT_BYTES = {"softmax": 4096 * 1024 * 4, "layer_norm": 16384 * 4096 * 2, "gemm": 8192 * 8192 * 2,
                "attention": 8 * 32 * 4096 * 128 * 2, "spmm": 262144 * 128 * 4, "softmax_backward": 4096 * 4097 * 4,
                "spmv": 32768 * 4}


def measure_end_to_end(case, steps: int, distributed: bool, world: int, with_cpu: bool) -> dict:
    """The same metric through the artifact API with host buffers, then the CPU sample."""
    workload = case.workload
    scale = 1e6 if workload.unit == "GB/s" else 1e9
    sequence = getattr(case, "single_gpu_only", False)
    pipeline = SequenceEndToEnd(case, 1) if sequence else EndToEnd(case, world)
    try:
        # a two-deep pipeline needs enough steps for its fill and drain not to dominate
        e2e_ms = timed(pipeline.step, steps, 2, distributed, case.device, begin=pipeline.begin, finish=pipeline.finish)
        whole_job = workload.work / e2e_ms / scale * (world if sequence else 1)
        result = {"e2e": {"value": whole_job, "unit": workload.unit, "ms_per_step": e2e_ms,
                          "h2d_bytes_per_step": pipeline.h2d, "d2h_bytes_per_step": pipeline.d2h,
                          "note": "per rank: its block of the inputs in, its block of the result out"
                                  if world > 1 and not sequence else "all inputs in, the result out"}}
    finally:
        pipeline.close()
    if with_cpu:
        import oracle
        result["cpu_baseline"] = cpu_baseline(case, oracle.default_workers())
    return result


def config_of(workload_description: str, world: int, flush: str) -> dict:
    """The same keys in both arms, so that their configurations compare equal."""
    return {"workload": workload_description, "l2": flush,
            "parallelism": "one GPU" if world == 1 else
            f"the workload split over {world} GPUs (rows), one process per GPU, no data-path collective; "
            "the final all-gather is timed separately under gather"}


HEADLINE = "layer_norm"      # BASELINE.json's second configuration


def run_reference(arguments, rank: int, world: int) -> None:
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
    eviction = torch.empty(64 * 1024 * 1024, dtype=torch.uint8)
    for _ in range(arguments.warmup):
        function()
    elapsed = 0.0
    for _ in range(arguments.steps):        # like cpu_baseline: caches evicted outside the timed interval
        oracle.evict(eviction)
        begin = time.perf_counter()
        function()
        elapsed += time.perf_counter() - begin
    milliseconds = elapsed * 1e3 / arguments.steps
    value = case.workload.work / milliseconds / 1e6
    print(json.dumps({
        "impl": "reference", "metric": "layer_norm throughput (algorithmic bytes / time)",
        "value": value, "unit": "GB/s", "n_gpus": arguments.gpus, "steps": arguments.steps,
        "warmup": arguments.warmup, "ms_per_step": milliseconds, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": config_of(case.workload.description, world, flush_description(world)),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": workers, "kind": "port",
                         "sample": f"{sample}, {arguments.steps} timed passes on {workers} host threads, "
                                   "64 MiB eviction outside each timed pass"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def flush_description(world: int) -> str:
    """The rotation the LayerNorm case uses at `world` ranks (computed, so both arms print the same text)."""
    from intent_b200 import workloads
    per_gpu = workloads.layer_norm_workload().work / world
    count = min(96, max(LayerNormCase.min_sets, math.ceil(ROTATION_BYTES / per_gpu)))
    return f"rotating {count} operand sets ({count * per_gpu / 1e6:.0f} MB per GPU per round > L2)"


def compact(entry: dict) -> dict:
    """One operator's row of the per-operator table kept inside `roofline`."""
    if "error" in entry:
        return {"error": entry["error"]}
    roof = entry["roofline"]
    row = {"value": entry["value"], "unit": entry["unit"], "ms": entry["ms_per_step"], "frac": roof["frac"],
           "frac_of_burst_peak": roof["frac_of_burst_peak"], "bound": roof["bound"], "peak": roof["peak"],
           "achieved_per_gpu": roof["achieved"], "traffic_ratio": roof.get("traffic_ratio"), "scaling": entry["scaling"]}
    if "e2e" in entry:
        row["e2e"] = entry["e2e"]["value"]
    if "cpu_baseline" in entry:
        row["cpu_baseline"] = {k: entry["cpu_baseline"][k] for k in ("value", "cores", "kind")}
    if "gather" in entry:
        row["with_gather"] = entry["gather"]["value"]
        row["all_gather_ms"] = entry["gather"]["all_gather_ms"]
        row["all_gather_bus_gbs"] = entry["gather"]["bus_gbs"]
        row["replicas"] = entry["replicas"]["value"]
    if "ceiling" in entry:
        row["ceiling"] = entry["ceiling"]
    return row


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--op", default="all", choices=["all", "baseline", *CASES])
    arguments = parser.parse_args()
    arguments.warmup = max(arguments.warmup, 3) if arguments.impl == "b200" else arguments.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if arguments.impl == "reference":
        run_reference(arguments, rank, world)
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
    if arguments.op == "all":       # the widened kernels are single-GPU figures: N > 1 measures the five configurations
        names = list(CASES) if world == 1 else list(BASELINE_OPS)
    elif arguments.op == "baseline":
        names = list(BASELINE_OPS)
    else:
        names = [arguments.op]
    primary = HEADLINE if HEADLINE in names else names[0]
    names.sort(key=lambda name: name != primary)           # the headline workload runs first
    results, launches = {}, 0
    global CLOCKS
    with ClockSampler(local_rank) as clocks:
        CLOCKS = clocks
        steps, cases = arguments.steps, {}
        for name in names:               # pass 1: device-resident figures of every operator
            try:
                cases[name] = CASES[name](device, rank, world)
                results[name] = measure_resident(cases[name], steps, arguments.warmup, distributed, world, peak_table,
                                                 peak_kind)
                if name == "spmm" and world == 1:
                    results[name]["ceiling"] = gather_ceiling(cases[name], results[name])
            except Exception as error:  # one failing operator must not hide the others
                if name == primary:
                    raise
                cases.pop(name, None)
                results[name] = {"op": name, "error": f"{type(error).__name__}: {error}"}
            finally:
                if name in cases:
                    cases[name].release()
                gc.collect()
                torch.cuda.empty_cache()
        for name in names:               # pass 2: end to end through the artifact API, and the CPU sample
            case = cases.pop(name, None)
            if case is None:
                continue
            try:
                results[name].update(measure_end_to_end(case, steps, distributed, world,
                                                        with_cpu=(rank == 0 and world == 1)))
                # warm-up, the captured pass and the timed replay of every resident figure (the 0.25 s
                # of load replays before each are not counted), then the end-to-end warm-up and steps
                figures = 1 if world == 1 or getattr(case, "single_gpu_only", False) else 3
                figures += 1 if name == "layer_norm" and world == 1 else 0
                launches += case.launches_per_step * (figures * (arguments.warmup + 2 * steps) + steps + 2)
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
    per_op = {name: compact(results[name]) for name in names}
    measured = {name: row["frac"] for name, row in per_op.items() if "frac" in row and name in BASELINE_OPS}
    roofline = dict(head["roofline"])
    roofline["per_op"] = per_op
    roofline["per_op_note"] = ("the metric is per operator: this line's value is the LayerNorm configuration, per_op holds "
                               "every configuration measured in this run, min_frac the lowest roofline fraction of the five")
    if measured:
        roofline["min_frac_op"] = min(measured, key=measured.get)
        roofline["min_frac"] = measured[roofline["min_frac_op"]]
    line = {
        "metric": f"{head['op']} throughput (algorithmic {'bytes' if head['unit'] == 'GB/s' else 'flops'} / time)",
        "value": head["value"], "unit": head["unit"], "n_gpus": world, "steps": arguments.steps,
        "warmup": arguments.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": DTYPES[primary], "data": "synthetic",
        "config": config_of(head["workload"], world, head["l2"]),
        "roofline": roofline, "e2e": head["e2e"], "gpu_launches": launches,
        "clocks": head.get("clocks") or clock_summary,
        "ops": [results[name] for name in names],
    }
    for key in ("gather", "replicas", "one_operand_set"):
        if key in head:
            line[key] = head[key]
    if "cpu_baseline" in head:
        line["cpu_baseline"] = head["cpu_baseline"]
    print(json.dumps(line))


if __name__ == "__main__":
    main()
