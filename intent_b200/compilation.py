"""``jit`` / ``generate`` for the b200 provider when the reference package is absent.

With the reference installed, ``intent.jit(kernel, backend="b200")`` lowers the
author's ``@intent.kernel`` with the reference frontend and hands the kernel IR
to ``b200-compile`` (see ``intent_b200.provider``).  On a machine that has only
this package, the same kernels are available here by name: their kernel IR was
produced once by that frontend (``intent_b200/kir/make_kir.py``) and is compiled
by the very same native step, so both routes execute one binder and one C ABI.

The classes mirror ``python/intent/jit/kernel.py:14-133`` (``JITKernel``, ``jit``)
and ``python/intent/compiler/artifact.py:41-185`` (``GeneratedProgram``).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
import subprocess
import tempfile
from dataclasses import dataclass, field
from pathlib import Path
from threading import RLock

import torch

from . import _native
from .runtime import Artifact, B200Program, ViewParameter

PACKAGE = Path(__file__).resolve().parent
COMPILER = PACKAGE / "bin" / "b200-compile"
KIR_DIRECTORY = PACKAGE / "kir"

FAILURE_STAGES = {1: "compiler_invocation", 2: "kernel_ir", 3: "physical_program", 4: "shared_pipeline",
                  5: "provider_program", 6: "provider_pipeline", 7: "terminal_translation", 8: "compiler_output"}


class CompilationStageError(RuntimeError):
    """Same shape as the reference's error (python/intent/compiler/toolchain.py:17-26)."""

    def __init__(self, stage: str, message: str, *, cache_directory=None):
        super().__init__(message)
        self.stage = stage
        self.cache_directory = cache_directory


@dataclass(frozen=True)
class CompileOptions:
    """python/intent/compiler/options.py:9-61, without optional transformations (b200 registers none)."""
    numerics: str = "source"
    optimizations: dict = field(default_factory=dict)
    optimization_remarks: bool = False

    @property
    def compiler_arguments(self) -> tuple:
        return (f"--numerics={self.numerics}", f"--optimization-remarks={str(self.optimization_remarks).lower()}",
                *(f"--optimization={n}={str(e).lower()}" for n, e in sorted(self.optimizations.items())))

    def metadata(self) -> dict:
        return {"numerics": self.numerics, "optimizations": dict(self.optimizations),
                "optimization_remarks": self.optimization_remarks}


@dataclass(frozen=True)
class KernelDefinition:
    """A kernel known by name, with its pre-lowered kernel IR.

    ``variants`` maps a frozen constexpr binding to the IR file lowered with it;
    ``head_group`` marks kernels whose HEAD_GROUP constexpr is a free integer:
    it only appears as one integer constant in the IR and is substituted there.
    """
    name: str
    variants: tuple
    constexprs: tuple = ()
    head_group: bool = False

    def __call__(self, *arguments, **keywords):
        raise TypeError(f"{self.name} is a kernel definition; compile it with intent_b200.jit(...)")

    def kir(self, constexprs: dict | None) -> str:
        bound = dict(constexprs or {})
        unknown = set(bound) - set(self.constexprs)
        if unknown:
            raise TypeError(f"{self.name} has no constexpr named {sorted(unknown)}")
        missing = set(self.constexprs) - set(bound)
        if missing:
            raise TypeError(f"{self.name} requires constexprs {sorted(missing)}")
        head_group = int(bound.pop("HEAD_GROUP")) if self.head_group else None
        key = tuple(sorted((name, _plain(value)) for name, value in bound.items()))
        for binding, filename in self.variants:
            if binding == key:
                text = (KIR_DIRECTORY / filename).read_text(encoding="utf-8")
                return text if head_group is None else _substitute_head_group(text, head_group)
        raise NotImplementedError(f"{self.name} was not lowered for constexprs {dict(key)}; add the case to "
                                  "intent_b200/kir/make_kir.py or use the reference frontend")


def _plain(value):
    return getattr(value, "name", value) if not isinstance(value, (bool, int, str)) else value


def _substitute_head_group(text: str, head_group: int) -> str:
    if head_group < 1:
        raise ValueError("HEAD_GROUP must be a positive integer")
    divide = re.search(r'"intent\.binary"\((%v\d+), (%v\d+)\) \{[^\n]*binary_operator<floor_divide>', text)
    if divide is None:
        raise ValueError("kernel IR has no HEAD_GROUP division")
    pattern = re.compile(rf'({re.escape(divide.group(2))} = "intent\.constant"\(\) \{{[^\n]*value = )\d+( : i64)')
    text, count = pattern.subn(rf"\g<1>{head_group}\g<2>", text)
    if count != 1:
        raise ValueError("kernel IR does not hold HEAD_GROUP as a single integer constant")
    return text


class kernels:
    """The kernel definitions of the five operator families, by the reference's names
    (python/intent/examples/kernels/{normalization,contraction,streaming,sparse})."""
    stable_softmax = KernelDefinition("stable_softmax", (((), "stable_softmax.mlir"),))
    stable_softmax_f16 = KernelDefinition("stable_softmax_f16", (((), "stable_softmax_f16.mlir"),))
    chunked_softmax_bf16 = KernelDefinition("chunked_softmax_bf16", (((), "chunked_softmax_bf16.mlir"),))
    layer_norm_f16 = KernelDefinition("layer_norm_f16", (((), "layer_norm_f16.mlir"),))
    layer_norm_bf16 = KernelDefinition("layer_norm_bf16", (((), "layer_norm_bf16.mlir"),))
    weighted_layer_norm = KernelDefinition("weighted_layer_norm", (((), "weighted_layer_norm.mlir"),))
    gemm = KernelDefinition("gemm", (((("ACTIVATION", "NONE"),), "gemm.mlir"),
                                     ((("ACTIVATION", "RELU"),), "gemm_relu.mlir")), ("ACTIVATION",))
    bf16_gemm = KernelDefinition("bf16_gemm", (((), "bf16_gemm.mlir"),))
    flash_attention_bf16_fwd = KernelDefinition(
        "flash_attention_bf16_fwd", (((("CAUSAL", True),), "flash_attention_bf16_fwd.mlir"),),
        ("HEAD_GROUP", "CAUSAL"), head_group=True)
    flash_attention_fwd = KernelDefinition(
        "flash_attention_fwd", (((("CAUSAL", True),), "flash_attention_fwd.mlir"),
                                ((("CAUSAL", False),), "flash_attention_fwd_noncausal.mlir")), ("CAUSAL",))
    flash_gqa_attention_fwd = KernelDefinition(
        "flash_gqa_attention_fwd", (((("CAUSAL", True),), "flash_gqa_attention_fwd.mlir"),),
        ("HEAD_GROUP", "CAUSAL"), head_group=True)
    csr_spmv = KernelDefinition("csr_spmv", (((), "csr_spmv.mlir"),))
    softmax_backward = KernelDefinition("softmax_backward", (((), "softmax_backward.mlir"),))
    layer_norm_backward_rows = KernelDefinition("layer_norm_backward_rows", (((), "layer_norm_backward_rows.mlir"),))
    layer_norm_backward_reduce = KernelDefinition("layer_norm_backward_reduce",
                                                  (((), "layer_norm_backward_reduce.mlir"),))
    attention_backward_delta = KernelDefinition("attention_backward_delta", (((), "attention_backward_delta.mlir"),))
    attention_backward_dkdv = KernelDefinition(
        "attention_backward_dkdv", (((("CAUSAL", True), ("HEAD_GROUP", 4)), "attention_backward_dkdv.mlir"),
                                    ((("CAUSAL", False), ("HEAD_GROUP", 1)), "attention_backward_dkdv_noncausal.mlir")),
        ("HEAD_GROUP", "CAUSAL"))
    attention_backward_dq = KernelDefinition(
        "attention_backward_dq", (((("CAUSAL", True), ("HEAD_GROUP", 4)), "attention_backward_dq.mlir"),
                                  ((("CAUSAL", False), ("HEAD_GROUP", 1)), "attention_backward_dq_noncausal.mlir")),
        ("HEAD_GROUP", "CAUSAL"))
    csr_spmm = KernelDefinition("csr_spmm", (((), "csr_spmm.mlir"),))
    csr_spmm_262144 = KernelDefinition("csr_spmm", (((), "csr_spmm_262144.mlir"),))


# --------------------------------------------------------------------------- target facts
CAPABILITY_FIELDS = ("compute_units", "shared_memory_per_unit", "max_dynamic_shared_memory_per_block",
                     "registers_per_unit", "max_threads_per_block", "compute_capability_major",
                     "compute_capability_minor", "single_to_double_precision_perf_ratio")

# What a B200 reports; used only to generate programs without a device (stage "source").
B200_CAPABILITIES = {
    "compute_units": 148, "shared_memory_per_unit": 233472, "max_dynamic_shared_memory_per_block": 232448,
    "registers_per_unit": 65536, "max_threads_per_block": 1024, "compute_capability_major": 10,
    "compute_capability_minor": 0, "single_to_double_precision_perf_ratio": 2, "matrix_units": True,
    "dynamic_vector_width": False,
}


def device_capabilities(device: int) -> dict:
    """The ten NVIDIA capability facts of python/intent/targets/nvidia/device.py:6-59."""
    import ctypes
    facts = (ctypes.c_int64 * 8)()
    _native.check("b200_device_capabilities", _native.entry("b200_device_capabilities")(int(device), facts))
    values = dict(zip(CAPABILITY_FIELDS, (int(v) for v in facts)))
    values["matrix_units"] = values["compute_capability_major"] >= 7
    values["dynamic_vector_width"] = False
    return values


# --------------------------------------------------------------------------- compile step
def compiler_path(compiler=None) -> Path:
    selected = Path(compiler or os.environ.get("INTENT_B200_COMPILER") or COMPILER)
    if not selected.is_file() or not os.access(selected, os.X_OK):
        raise CompilationStageError("compiler_invocation",
                                    f"{selected} is not an executable; build it with `python -m intent_b200.build`")
    return selected


def run_compiler(kir: str, capabilities: dict, options: CompileOptions | None = None, *, compiler=None,
                 directory: Path | None = None):
    """One subprocess call with the reference's argv and stdin protocol
    (python/intent/compiler/toolchain.py:212-219). Returns (ir, source, metadata)."""
    executable = compiler_path(compiler)
    arguments = ["--target=b200", f"--target-options={json.dumps(capabilities)}"]
    if options is not None:
        arguments += list(options.compiler_arguments)
    owner = tempfile.TemporaryDirectory(prefix="intent_b200-") if directory is None else None
    base = Path(owner.name) if owner else Path(directory)
    try:
        command = [str(executable), *arguments, f"--ir-output={base / 'kernel.mlir'}",
                   f"--source-output={base / 'kernel.source'}", f"--metadata-output={base / 'artifact.json'}", "-"]
        completed = subprocess.run(command, input=kir, text=True, capture_output=True, check=False)
        if completed.returncode:
            raise CompilationStageError(
                FAILURE_STAGES.get(completed.returncode, "compiler_process"),
                f"b200-compile failed with exit code {completed.returncode}:\n{completed.stderr}{completed.stdout}")
        outputs = [base / name for name in ("kernel.mlir", "kernel.source", "artifact.json")]
        if any(not path.is_file() or path.stat().st_size == 0 for path in outputs):
            raise CompilationStageError("compiler_output", "b200-compile did not produce complete outputs")
        return (outputs[0].read_text(encoding="utf-8"), outputs[1].read_text(encoding="utf-8"),
                json.loads(outputs[2].read_text(encoding="utf-8")))
    finally:
        if owner:
            owner.cleanup()


@dataclass(frozen=True)
class GeneratedProgram:
    """Provider source, IR and metadata; ``save``/``load`` use the compiler's own
    three-file layout (python/intent/compiler/artifact.py:105-157)."""
    source: str
    ir: str
    metadata: dict
    entry_name: str

    def save(self, directory) -> Path:
        path = Path(directory).expanduser().absolute()
        if path.exists():
            raise CompilationStageError("generated_program_export", f"destination already exists: {path}")
        path.mkdir(parents=True)
        (path / "kernel.source").write_text(self.source, encoding="utf-8")
        (path / "kernel.mlir").write_text(self.ir, encoding="utf-8")
        (path / "artifact.json").write_text(json.dumps(self.metadata, indent=2) + "\n", encoding="utf-8")
        return path

    @classmethod
    def load(cls, directory, *, name: str | None = None) -> "GeneratedProgram":
        path = Path(directory).expanduser().absolute()
        try:
            source = (path / "kernel.source").read_text(encoding="utf-8")
            ir = (path / "kernel.mlir").read_text(encoding="utf-8")
            metadata = json.loads((path / "artifact.json").read_text(encoding="utf-8"))
            if not source.strip() or not ir.strip() or not isinstance(metadata, dict):
                raise ValueError("generated program requires nonempty source, IR and object metadata")
            return cls(source, ir, metadata, name or metadata["entry_name"])
        except (OSError, ValueError, KeyError) as error:
            raise CompilationStageError("generated_program_loading", str(error), cache_directory=path) from error

    def materialize(self, *, device: int = 0, gpus=None, gather_output: bool = False) -> Artifact:
        """Bind to a device; refuses a device whose facts differ from the compiled ones
        (python/intent/targets/nvidia/target.py:25-31)."""
        _native.check("b200_device_check", _native.entry("b200_device_check")(int(device)))
        current = device_capabilities(device)
        if self.metadata["target"]["capabilities"] != current:
            raise CompilationStageError(
                "generated_source_materialization",
                f"generated target {self.metadata['target']['capabilities']} does not match the selected "
                f"runtime target {current}")
        return Artifact(self.source, self.ir, device,
                        B200Program(self.metadata, device, gpus=gpus, gather_output=gather_output))


_generated: dict[str, GeneratedProgram] = {}
_generated_lock = RLock()


def generate(definition: KernelDefinition, *, capabilities: dict | None = None, constexprs=None,
             options: CompileOptions | None = None, compiler=None) -> GeneratedProgram:
    kir = definition.kir(constexprs)
    facts = dict(capabilities or B200_CAPABILITIES)
    key = hashlib.sha256(json.dumps([kir, facts, options.metadata() if options else None,
                                     str(compiler)], sort_keys=True).encode()).hexdigest()
    with _generated_lock:
        if key not in _generated:
            ir, source, metadata = run_compiler(kir, facts, options, compiler=compiler)
            if options is not None and metadata["compile_options"] != options.metadata():
                raise CompilationStageError("compiler_output",
                                            "compiler output does not preserve the requested compile options")
            _generated[key] = GeneratedProgram(source, ir, metadata, definition.name)
        return _generated[key]


# --------------------------------------------------------------------------- JIT
_BACKEND_OPTIONS = frozenset({"gpus", "gather_output"})


def _cuda_ordinal(device) -> int | None:
    if device is None:
        return None
    return device if isinstance(device, int) else torch.device(device).index


def _ordinal_of_call(tensors, requested) -> int:
    """The one CUDA ordinal a call runs on: every tensor argument must live there, and an
    explicit ``device=`` must agree with them."""
    seen = []
    for tensor in tensors:
        if not isinstance(tensor, torch.Tensor):
            continue
        if tensor.device.type != "cuda":
            raise ValueError(f"backend 'b200' executes on cuda, but arguments select {tensor.device}")
        if tensor.device.index not in seen:
            seen.append(tensor.device.index)
    if len(seen) > 1:
        raise ValueError(f"JIT arguments span different devices: {sorted(seen)}")
    chosen = _cuda_ordinal(requested)
    if chosen is None:
        if not seen:
            raise ValueError("JIT requires a device-bearing input or an explicit local device")
        return seen[0]
    if seen and seen[0] != chosen:
        raise ValueError(f"explicit device cuda:{chosen} conflicts with the input device cuda:{seen[0]}")
    return chosen


class JITKernel:
    """A kernel definition plus the artifacts compiled from it, one per CUDA device, made on
    first use.  Same surface as the reference's JIT object (``python/intent/jit/kernel.py``):
    ``prepare`` / ``run`` / call with explicit outputs / ``as_torch_op`` / ``close``.

    ``backend_options`` takes ``gpus`` (number of ranks, or their CUDA ordinals in rank order)
    and ``gather_output``: one process per GPU makes the same call with the same full operands,
    each computes its block of rows / M-tiles / (batch, head) units, and with ``gather_output``
    one all-gather completes the output on every rank (``intent_b200.sharding``)."""

    def __init__(self, definition, *, backend, device=None, compiler=None, constexprs=None, options=None,
                 backend_options=None):
        if not isinstance(definition, KernelDefinition):
            raise TypeError("intent_b200.jit requires one of intent_b200.kernels.*")
        if backend != "b200":
            raise ValueError(f"Unknown backend {backend!r}; choose from b200")
        unknown = set(backend_options or {}) - _BACKEND_OPTIONS
        if unknown:
            raise ValueError(f"unsupported local b200 options: {sorted(unknown)}")
        self.definition, self.backend, self.device = definition, backend, device
        self.compiler, self.options = compiler, options
        self.constexprs = dict(constexprs or {})
        self.backend_options = dict(backend_options or {})
        self.__name__ = definition.name
        self._guard = RLock()
        self._per_device: dict[int, Artifact] | None = {}      # None once closed

    # -- what has been compiled so far -----------------------------------------------
    @property
    def artifacts(self) -> tuple:
        with self._guard:
            return tuple((self._per_device or {}).values())

    def _only_artifact(self, purpose: str) -> Artifact:
        compiled = self.artifacts
        if len(compiled) != 1:
            raise ValueError(f"prepare one {purpose}")
        return compiled[0]

    @property
    def interface(self):
        return self._only_artifact("local specialization before inspecting its interface").interface

    def as_torch_op(self, name):
        return self._only_artifact(
            "device specialization before registering its PyTorch operator").as_torch_op(name)

    # -- compile on demand -----------------------------------------------------------
    def _program(self, capabilities=None) -> GeneratedProgram:
        return generate(self.definition, capabilities=capabilities, constexprs=self.constexprs,
                        options=self.options, compiler=self.compiler)

    def _artifact_for(self, tensors) -> Artifact:
        ordinal = _ordinal_of_call(tensors, self.device)
        with self._guard:
            if self._per_device is None:
                raise RuntimeError("JIT kernel is closed")
            artifact = self._per_device.get(ordinal)
            if artifact is None:
                artifact = self._program(device_capabilities(ordinal)).materialize(device=ordinal,
                                                                                   **self.backend_options)
                self._per_device[ordinal] = artifact
            return artifact

    # -- calls -------------------------------------------------------------------------
    def prepare(self, *arguments, outputs=None):
        if outputs is not None and not isinstance(outputs, tuple):
            raise TypeError("outputs must be a tuple in declared Out order")
        artifact = self._artifact_for(arguments if outputs is None else (*arguments, *outputs))
        return artifact.prepare(*arguments, outputs=outputs)

    def run(self, *arguments):
        prepared = self.prepare(*arguments)
        prepared.launch()
        return prepared.result()

    def __call__(self, *arguments):
        """All runtime parameters in declaration order, output buffers included."""
        from .runtime import Interface
        declared = Interface.read(self._program().metadata["interface"]).parameters
        if len(arguments) != len(declared):
            raise TypeError(f"expected {len(declared)} runtime arguments, got {len(arguments)}")
        is_output = [isinstance(parameter, ViewParameter) and parameter.output for parameter in declared]
        supplied = tuple(value for value, out in zip(arguments, is_output) if not out)
        buffers = tuple(value for value, out in zip(arguments, is_output) if out)
        self.prepare(*supplied, outputs=buffers).launch()

    # -- lifetime ------------------------------------------------------------------------
    def close(self):
        with self._guard:
            for artifact in (self._per_device or {}).values():
                artifact.runtime.close()
            self._per_device = None

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()


def jit(definition, *, backend="b200", device=None, compiler=None, constexprs=None, options=None,
        backend_options=None):
    return JITKernel(definition, backend=backend, device=device, compiler=compiler,
                     constexprs=constexprs, options=options, backend_options=backend_options)
