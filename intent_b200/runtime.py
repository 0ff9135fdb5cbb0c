"""Host runtime of the b200 provider: artifact.json -> binder -> prepared call -> C ABI.

This module mirrors the part of the reference runtime that sits between a
compiled program and its native entry, with the same names, argument meaning
and error behaviour, but without importing the reference:

===========================  =====================================================
here                         reference
===========================  =====================================================
``Interface.read``           ``PublicInterface.read``   runtime/interface.py:110-150
``Interface.relations``      ``binding_relations``      runtime/interface.py:187-245
``NativeLayout.read``        ``NativeABI.read``         runtime/native.py:77-130
``Requirements``             ``NativeRequirements``     runtime/native_requirements.py:21-91
``B200Program``              ``NativePreparedRuntime``  runtime/native.py:240-273
``B200Call``                 ``PreparedCall``           runtime/artifact.py:23-55
``Artifact``                 ``CompiledArtifact``       runtime/artifact.py:94-218
``register_operator``        same name                  integrations/torch.py:27-93
===========================  =====================================================

A launch is one ``ctypes`` call on torch's current CUDA stream and never
synchronises; ``result()`` returns the output containers as they are
(``doc/getting-started/usage.en.md:53-55``).  There is no fallback: if the CUDA
library is missing or refuses the call, the error propagates.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from inspect import Parameter, Signature
from threading import RLock

import torch

from . import _native, sharding

IN, OUT, INOUT = 0, 1, 2

TORCH_DTYPES = {
    "index": torch.int64, "bool": torch.bool, "i8": torch.int8, "i16": torch.int16, "i32": torch.int32,
    "i64": torch.int64, "u8": torch.uint8, "f16": torch.float16, "bf16": torch.bfloat16,
    "f32": torch.float32, "f64": torch.float64,
}
_DTYPE_BYTES = {"bool": 1, "i8": 1, "u8": 1, "i16": 2, "f16": 2, "bf16": 2, "i32": 4, "f32": 4,
                "i64": 8, "f64": 8, "index": 8}
_CARRIERS = {"ptr": ctypes.c_void_p, "bool": ctypes.c_bool, "i8": ctypes.c_int8, "i16": ctypes.c_int16,
             "i32": ctypes.c_int32, "i64": ctypes.c_int64, "f32": ctypes.c_float, "f64": ctypes.c_double}


# --------------------------------------------------------------------------- interface
@dataclass(frozen=True)
class ScalarParameter:
    position: int
    name: str
    dtype: str


@dataclass(frozen=True)
class StrideSymbol:
    name: str


@dataclass(frozen=True)
class ViewParameter:
    position: int
    name: str
    dtype: str
    shape: tuple
    dimensions: tuple
    strides: tuple
    access: int
    alias: str
    noalias: bool

    @property
    def writable(self) -> bool:
        return self.access != IN

    @property
    def output(self) -> bool:
        return self.access == OUT


@dataclass(frozen=True)
class ViewFacts:
    """What one binding observed of a tensor (runtime/invocation.py:11-24)."""
    shape: tuple
    strides: tuple
    pointer: int | None
    allocation: tuple | None      # (begin, end) of the whole storage
    span: tuple | None            # (begin, end) of the bytes this view can touch
    identity: object


def _byte_span(pointer: int, shape, strides, size: int) -> tuple[int, int]:
    if any(extent == 0 for extent in shape):
        return pointer, pointer
    low = high = 0
    for extent, stride in zip(shape, strides):
        displacement = (extent - 1) * stride
        low += min(0, displacement)
        high += max(0, displacement)
    return pointer + low * size, pointer + (high + 1) * size


def _overlap(lhs, rhs) -> bool:
    return lhs[0] < lhs[1] and rhs[0] < rhs[1] and lhs[0] < rhs[1] and rhs[0] < lhs[1]


def _stride_rule(rule):
    """One entry of a view's "strides" list: free (None), a fixed element stride, or a named
    symbol that several axes must agree on."""
    if rule is None or type(rule) is int:
        return rule
    if isinstance(rule, dict) and rule.get("kind") == "stride_symbol":
        return StrideSymbol(rule["symbol"])
    raise ValueError(f"interface: cannot interpret the stride rule {rule!r}")


def _view_parameter(position: int, record: dict) -> ViewParameter:
    name = record["name"]
    extents = tuple(record["shape"])
    identities = tuple(record["dimensions"])
    rules = tuple(_stride_rule(rule) for rule in record["strides"])
    for extent in extents:
        if type(extent) is not int or extent < -1:
            raise ValueError(f"interface: {name} has the extent {extent!r}; extents are integers, -1 when dynamic")
    if not len(extents) == len(identities) == len(rules):
        raise ValueError(f"interface: {name} lists {len(extents)} extents, {len(identities)} dimension ids "
                         f"and {len(rules)} stride rules; the three must have the view's rank")
    if record["access"] not in (IN, OUT, INOUT):
        raise ValueError(f"interface: {name} has the access code {record['access']!r} (0 In, 1 Out, 2 InOut)")
    if record["alias"] and record["noalias"]:
        raise ValueError(f"interface: {name} names an alias group and is noalias at once")
    return ViewParameter(position, name, record["dtype"], extents, identities, rules, record["access"],
                         record["alias"], record["noalias"])


@dataclass(frozen=True)
class Interface:
    """The author's ordered runtime parameters, independent of the device ABI
    (the "interface" object of artifact.json)."""
    parameters: tuple

    @classmethod
    def read(cls, metadata: dict) -> "Interface":
        records = metadata["parameters"]
        names = [record["name"] for record in records]
        if any(not isinstance(name, str) or not name for name in names) or len(set(names)) != len(names):
            raise ValueError(f"interface: parameter names {names!r} are not distinct non-empty strings")
        parsed = []
        for position, record in enumerate(records):
            if record["dtype"] not in _DTYPE_BYTES:
                raise NotImplementedError(f"element type {record['dtype']!r} is not supported by b200")
            kind = record["kind"]
            if kind == "view":
                parsed.append(_view_parameter(position, record))
            elif kind == "scalar":
                parsed.append(ScalarParameter(position, record["name"], record["dtype"]))
            else:
                raise ValueError(f"interface: {record['name']} is a {kind!r}; only views and scalars cross the ABI")
        return cls(tuple(parsed))

    def _select(self, keep) -> tuple:
        return tuple(parameter for parameter in self.parameters if keep(parameter))

    @property
    def views(self):
        return self._select(lambda parameter: isinstance(parameter, ViewParameter))

    @property
    def outputs(self):
        return self._select(lambda parameter: isinstance(parameter, ViewParameter) and parameter.output)

    @property
    def inputs(self):
        """What a caller supplies when the runtime allocates the outputs: scalars and every
        view that is not a pure output."""
        declared_outputs = self.outputs
        return self._select(lambda parameter: parameter not in declared_outputs)

    def explicit_arguments(self, arguments: tuple, outputs: tuple) -> tuple:
        """Merges inputs and caller-owned output buffers back into declaration order."""
        wanted_inputs, wanted_outputs = len(self.inputs), len(self.outputs)
        if len(arguments) != wanted_inputs:
            raise TypeError(f"expected {wanted_inputs} input arguments, got {len(arguments)}")
        if len(outputs) != wanted_outputs:
            raise TypeError(f"expected {wanted_outputs} explicit output buffers, got {len(outputs)}")
        pending = {True: list(reversed(outputs)), False: list(reversed(arguments))}
        merged = []
        for parameter in self.parameters:
            merged.append(pending[isinstance(parameter, ViewParameter) and parameter.output].pop())
        return tuple(merged)


# --------------------------------------------------------------------------- native layout
@dataclass(frozen=True)
class Workspace:
    position: int
    dtype: str
    shape: tuple


@dataclass(frozen=True)
class Slot:
    parameter: int
    role: str          # pointer | extent | stride | scalar
    carrier: str
    axis: int | None = None


@dataclass(frozen=True)
class ViewRequirement:
    layout: str
    alignment: int


@dataclass(frozen=True)
class Requirements:
    views: dict
    disjoint: frozenset

    @classmethod
    def read(cls, metadata: dict, interface: Interface) -> "Requirements":
        try:
            requirements = metadata["native"]["requirements"]
        except KeyError as error:
            raise ValueError("native artifact lacks explicit entry requirements") from error
        views = {}
        for entry in requirements["views"]:
            position = entry["parameter"]
            if (type(position) is not int or not 0 <= position < len(interface.parameters)
                    or not isinstance(interface.parameters[position], ViewParameter) or position in views):
                raise ValueError("native view requirement references an unknown or repeated public view")
            if entry["layout"] not in {"strided", "contiguous"}:
                raise ValueError("native entry has an unknown view layout requirement")
            if type(entry["alignment"]) is not int or entry["alignment"] <= 0:
                raise ValueError("native entry alignment must be a positive byte count")
            views[position] = ViewRequirement(entry["layout"], entry["alignment"])
        if any(view.position not in views for view in interface.views):
            raise ValueError("native entry must declare requirements for every public view")
        disjoint = set()
        for entry in requirements["disjoint"]:
            left, right = entry["left"], entry["right"]
            if not (type(left) is int and type(right) is int and left < right and left in views and right in views):
                raise ValueError("native disjointness requirement must name two ordered public views")
            disjoint.add((left, right))
        return cls(views, frozenset(disjoint))


@dataclass(frozen=True)
class NativeLayout:
    interface: Interface
    slots: tuple
    workspaces: tuple
    requirements: Requirements

    @classmethod
    def read(cls, metadata: dict) -> "NativeLayout":
        interface = Interface.read(metadata["interface"])
        workspaces = []
        for entry in metadata["native"]["workspaces"]:
            if entry["position"] != len(interface.parameters) + len(workspaces):
                raise ValueError("native workspaces must follow the public arguments in declaration order")
            workspaces.append(Workspace(entry["position"], entry["dtype"], tuple(entry["shape"])))
        count = len(interface.parameters) + len(workspaces)
        slots, seen = [], set()
        for entry in metadata["native"]["slots"]:
            position, role, carrier = entry["parameter"], entry["role"], entry["carrier"]
            if type(position) is not int or not 0 <= position < count:
                raise ValueError("native slot references an unknown entry parameter")
            if carrier not in _CARRIERS:
                raise NotImplementedError(f"native scalar carrier {carrier!r} is unsupported")
            if role not in {"pointer", "extent", "stride", "scalar"}:
                raise ValueError("unknown native slot role")
            axis = entry.get("axis")
            if (axis is not None) != (role in {"extent", "stride"}):
                raise ValueError("native slot fields disagree with its role")
            if (position, role, axis) in seen:
                raise ValueError("native ABI has duplicate parameter slots")
            seen.add((position, role, axis))
            slots.append(Slot(position, role, carrier, axis))
        for parameter in interface.parameters:
            view = isinstance(parameter, ViewParameter)
            if (parameter.position, "pointer" if view else "scalar", None) not in seen:
                raise ValueError("native ABI does not bind every public parameter")
            if view:
                for axis in range(len(parameter.shape)):
                    if any((parameter.position, role, axis) not in seen for role in ("extent", "stride")):
                        raise ValueError("native ABI must bind the extent and stride of every view axis")
        return cls(interface, tuple(slots), tuple(workspaces), Requirements.read(metadata, interface))


@dataclass(frozen=True)
class B200Facts:
    """Provider-private section of artifact.json written by b200-compile."""
    family: str
    entry: str
    tail: tuple          # ((name, carrier, value), ...)

    @classmethod
    def read(cls, metadata: dict) -> "B200Facts":
        section = metadata["b200"]
        if section.get("abi_version") != 1:
            raise ValueError("artifact was produced for another intent_b200 ABI version")
        if section["entry"] not in _native.SIGNATURES:
            raise ValueError(f"artifact names an unknown entry {section['entry']!r}")
        tail = tuple((item["name"], item["carrier"], item["value"]) for item in section["tail"])
        return cls(section["family"], section["entry"], tail)


@dataclass(frozen=True)
class Observation:
    """Per-call facts, the b200 analogue of the reference's NativeObservation
    (runtime/diagnostics.py:22-144)."""
    provider: str
    family: str
    entry: str
    constants: tuple
    stage: str
    arguments: tuple


# --------------------------------------------------------------------------- binding
class _Abstract:
    """Marker: bind shapes only (FakeTensor / meta tracing), never addresses."""


def _relation(actual, expected, message: str, abstract: bool) -> None:
    if abstract:
        torch._check(actual == expected, lambda: message)
    elif actual != expected:
        raise ValueError(message)


class B200Program:
    """Binds torch tensors to one native entry; mirrors NativePreparedRuntime."""

    device_type = "cuda"

    def __init__(self, metadata: dict, device: int | torch.device, *, gpus=None, gather_output: bool = False):
        if metadata.get("provider") != "b200":
            raise ValueError("not a b200 program")
        self.metadata = metadata
        self.layout = NativeLayout.read(metadata)
        self.interface = self.layout.interface
        self.facts = B200Facts.read(metadata)
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        # the gpus / gather_output backend options: this rank's place among the processes that
        # share the call, or None for a call that stays on one GPU
        self.distribution = sharding.distribution(gpus, gather_output, self.device)
        self._observation: Observation | None = None
        self._lock = RLock()
        self._function = None
        signature = _native.SIGNATURES[self.facts.entry]
        expected = [_CARRIERS[slot.carrier] for slot in self.layout.slots]
        expected += [_CARRIERS[carrier] for _, carrier, _ in self.facts.tail] + [ctypes.c_void_p]
        if list(signature) != expected:
            raise ValueError(f"artifact slots do not match the signature of {self.facts.entry}")

    # -- observation ---------------------------------------------------------
    @property
    def observation(self) -> Observation | None:
        return self._observation

    @property
    def configuration_descriptions(self):
        return ({"family": self.facts.family, "entry": self.facts.entry,
                 **{name: value for name, _, value in self.facts.tail}},)

    def inspect_configurations(self):
        return self.configuration_descriptions

    # -- binder ----------------------------------------------------------------
    def _observe(self, parameter: ViewParameter, value, abstract: bool) -> ViewFacts:
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{parameter.name} must be a torch.Tensor")
        expected = TORCH_DTYPES[parameter.dtype]
        if value.dtype != expected:
            raise TypeError(f"{parameter.name} must have dtype {expected}, got {value.dtype}")
        if not abstract and value.device != self.device:
            raise ValueError(f"{parameter.name} must be on {self.device}, got {value.device}")
        shape, strides = tuple(value.shape), tuple(value.stride())
        if len(shape) != len(parameter.shape):
            raise ValueError(f"{parameter.name} must have rank {len(parameter.shape)}, got {len(shape)}")
        if abstract:
            return ViewFacts(shape, strides, None, None, None, None)
        storage = value.untyped_storage()
        begin, size = storage.data_ptr(), storage.nbytes()
        pointer = value.data_ptr()
        identity = (value.device, begin) if size else (value.device, "empty", storage._cdata)
        return ViewFacts(shape, strides, pointer, (begin, begin + size),
                         _byte_span(pointer, shape, strides, value.element_size()), identity)

    def _bind(self, arguments: tuple, explicit_outputs: bool, abstract: bool = False):
        interface = self.interface
        supplied = interface.parameters if explicit_outputs else interface.inputs
        if len(arguments) != len(supplied):
            raise TypeError(f"expected {len(supplied)} runtime arguments, got {len(arguments)}")
        values: dict[int, object] = {}
        facts: dict[int, ViewFacts] = {}
        dimensions: dict[int, int] = {}
        symbols: dict[str, int] = {}
        static = {}
        for view in interface.views:
            for extent, identity in zip(view.shape, view.dimensions):
                if extent >= 0 and identity > 0:
                    known = static.setdefault(identity, extent)
                    if known != extent and not explicit_outputs:
                        raise NotImplementedError(
                            f"Cannot allocate the declared outputs: dimension {identity} has conflicting "
                            f"static extents {known} and {extent}. Provide explicit output buffers with "
                            "prepare(..., outputs=(...)) or launch(...).")

        def check(parameter: ViewParameter, observed: ViewFacts, allocated: bool) -> None:
            for axis, (extent, identity) in enumerate(zip(parameter.shape, parameter.dimensions)):
                message = f"{parameter.name}.shape[{axis}] violates the declared interface relation"
                known = extent if extent >= 0 else static.get(identity)
                if known is not None:
                    _relation(observed.shape[axis], known, message, abstract)
                if identity > 0:
                    if identity in dimensions:
                        _relation(observed.shape[axis], dimensions[identity], message, abstract)
                    else:
                        dimensions[identity] = observed.shape[axis]
            for axis, constraint in enumerate(parameter.strides):
                message = f"{parameter.name}.strides[{axis}] violates the declared interface relation"
                if allocated:
                    message += "; provide explicit output buffers with the required layout"
                if isinstance(constraint, StrideSymbol):
                    if constraint.name in symbols:
                        _relation(observed.strides[axis], symbols[constraint.name], message, abstract)
                    else:
                        symbols[constraint.name] = observed.strides[axis]
                elif constraint is not None:
                    _relation(observed.strides[axis], constraint, message, abstract)
            requirement = self.layout.requirements.views[parameter.position]
            if requirement.layout == "contiguous":
                expected = 1
                for extent, stride in zip(reversed(observed.shape), reversed(observed.strides)):
                    if abstract:
                        torch._check(stride == expected, lambda: f"{parameter.name}: native entry requires "
                                                                 "canonical contiguous element strides")
                    elif stride != expected:
                        raise NotImplementedError(
                            f"{parameter.name}: native entry requires canonical contiguous element strides")
                    expected *= extent
            if not abstract and observed.pointer % requirement.alignment:
                raise ValueError(
                    f"{parameter.name}: native entry requires {requirement.alignment}-byte pointer alignment")

        for position, parameter in enumerate(supplied):
            values[parameter.position] = arguments[position]
            if isinstance(parameter, ViewParameter):
                facts[parameter.position] = self._observe(parameter, arguments[position], abstract)
                check(parameter, facts[parameter.position], False)
            elif isinstance(arguments[position], torch.Tensor):
                raise TypeError(f"{parameter.name} is a scalar parameter, got a tensor")
        if not explicit_outputs:
            for parameter in interface.outputs:
                shape = []
                for axis, (extent, identity) in enumerate(zip(parameter.shape, parameter.dimensions)):
                    known = extent if extent >= 0 else static.get(identity, dimensions.get(identity))
                    if known is None:
                        raise NotImplementedError(
                            f"Cannot allocate the declared outputs: {parameter.name}.shape[{axis}] has no extent "
                            "supplied by inputs or fixed by the public shape declarations. Provide explicit "
                            "output buffers with prepare(..., outputs=(...)) or launch(...).")
                    shape.append(known)
                device = "meta" if abstract and not any(
                    isinstance(v, torch.Tensor) for v in arguments) else (
                    next(v.device for v in arguments if isinstance(v, torch.Tensor)) if abstract else self.device)
                tensor = torch.empty(tuple(shape), dtype=TORCH_DTYPES[parameter.dtype], device=device)
                values[parameter.position] = tensor
                facts[parameter.position] = self._observe(parameter, tensor, abstract)
                check(parameter, facts[parameter.position], True)
        if not abstract:
            views = interface.views
            for index, left in enumerate(views):
                for right in views[index + 1:]:
                    lf, rf = facts[left.position], facts[right.position]
                    names = f"{left.name} and {right.name}"
                    if (left.noalias or right.noalias) and _overlap(lf.allocation, rf.allocation):
                        raise ValueError(f"{names} violate an author noalias allocation constraint")
                    if left.alias and left.alias == right.alias and lf.identity != rf.identity:
                        raise ValueError(f"{names} violate an author named allocation-alias constraint")
                    if ((left.position, right.position) in self.layout.requirements.disjoint
                            and _overlap(lf.span, rf.span)):
                        raise NotImplementedError(
                            f"{names}: native entry requires nonoverlapping accessed byte spans")
        ordered = tuple(values[p.position] for p in interface.parameters)
        outputs = tuple(values[p.position] for p in interface.outputs)
        return ordered, outputs, facts

    def _native_arguments(self, ordered: tuple, facts: dict, workspaces: dict) -> tuple:
        packed = []
        for slot in self.layout.slots:
            if slot.role == "scalar":
                value = ordered[slot.parameter]
                packed.append(float(value) if slot.carrier in {"f32", "f64"} else int(value))
                continue
            observed = facts[slot.parameter] if slot.parameter in facts else workspaces[slot.parameter]
            if slot.role == "pointer":
                packed.append(observed.pointer)
            elif slot.role == "extent":
                packed.append(observed.shape[slot.axis])
            else:
                packed.append(observed.strides[slot.axis])
        packed.extend(value for _, _, value in self.facts.tail)
        return tuple(packed)

    # -- public preparation API --------------------------------------------------
    def prepare(self, arguments: tuple, *, explicit_outputs: bool = False) -> "B200Call":
        ordered, outputs, facts = self._bind(tuple(arguments), explicit_outputs)
        owners, workspace_facts = [], {}
        for workspace in self.layout.workspaces:
            # invocation-owned, like the reference's workspaces (runtime/native.py:207-209)
            tensor = torch.zeros(workspace.shape, dtype=TORCH_DTYPES[workspace.dtype], device=self.device)
            owners.append(tensor)
            workspace_facts[workspace.position] = ViewFacts(
                tuple(tensor.shape), tuple(tensor.stride()), tensor.data_ptr(), None, None, None)
        description = tuple(
            (p.name, facts[p.position].shape, facts[p.position].strides) if isinstance(p, ViewParameter)
            else (p.name, ordered[p.position]) for p in self.interface.parameters)
        blocks = ()
        if self.distribution is not None:
            # The full operands were validated above.  The native call now receives this rank's
            # block of them (views into the same buffers), and the output blocks are remembered
            # for the optional all-gather after the launch.
            constants = {name: value for name, _, value in self.facts.tail}
            part = sharding.partition(self.facts.family, ordered, self.distribution.rank, self.distribution.world,
                                      head_group=int(constants.get("head_group", 1)))
            blocks = part.outputs
            launched = part.arguments
            facts = {p.position: ViewFacts(tuple(launched[p.position].shape), tuple(launched[p.position].stride()),
                                           launched[p.position].data_ptr(), None, None, None)
                     for p in self.interface.views}
            description += (("shard", (part.begin, part.end), part.units),)
            owners.extend(t for t in launched if isinstance(t, torch.Tensor))
        else:
            launched = ordered
        return B200Call(self, ordered, self._native_arguments(launched, facts, workspace_facts), outputs,
                        tuple(owners[:len(self.layout.workspaces)]), description, tuple(owners), blocks)

    def prepare_call(self, arguments: tuple, *, outputs: tuple | None = None) -> "B200Call":
        if outputs is None:
            return self.prepare(arguments)
        return self.prepare(self.interface.explicit_arguments(arguments, outputs), explicit_outputs=True)

    def run(self, *arguments):
        call = self.prepare(arguments)
        call.launch()
        return call.result()

    def launch(self, *arguments) -> None:
        self.prepare(arguments, explicit_outputs=True).launch()

    def infer_outputs(self, arguments: tuple):
        """Output containers for abstract (fake / meta) inputs; never touches addresses."""
        _, outputs, _ = self._bind(tuple(arguments), False, abstract=True)
        return None if not outputs else outputs[0] if len(outputs) == 1 else outputs

    def function(self):
        with self._lock:
            if self._function is None:
                self._function = _native.entry(self.facts.entry)
            return self._function

    def close(self) -> None:
        self._function = None


@dataclass
class B200Call:
    """Invocation-owned arguments and outputs (PreparedCall, runtime/artifact.py:23-55)."""
    program: B200Program
    arguments: tuple
    native_arguments: tuple
    outputs: tuple
    workspaces: tuple
    description: tuple
    owners: tuple = ()            # tensors the native arguments point into (workspaces, shard views)
    blocks: tuple = ()            # output blocks of a call that is spread over several GPUs
    _observation: Observation | None = field(default=None, repr=False)

    def compile(self) -> None:
        """Nothing is JIT-compiled: validate that the AOT library holds the entry."""
        self.program.function()
        self._record("compiled")

    def _record(self, stage: str) -> None:
        facts = self.program.facts
        self._observation = Observation("b200", facts.family, facts.entry, facts.tail, stage, self.description)
        self.program._observation = self._observation

    def launch(self) -> None:
        function = self.program.function()
        device = self.program.device
        with torch.cuda.device(device):
            stream = torch.cuda.current_stream(device).cuda_stream
            status = function(*self.native_arguments, stream)
        if status != _native.OK:
            self._record("failed")
            _native.check(self.program.facts.entry, status)
        self.gather()
        self._record("launched")

    def gather(self) -> None:
        """The final all-gather of a call spread over several GPUs (`gather_output`): every
        rank's output block reaches every rank, in place, ordered after the kernel on torch's
        current stream.  A call on one GPU, or without `gather_output`, does nothing here."""
        distribution = self.program.distribution
        if distribution is None or not distribution.gather_output:
            return
        with torch.cuda.device(self.program.device):
            for block in self.blocks:
                sharding.gather_blocks(block, distribution.world, group=distribution.group)

    def enqueue(self, queue) -> None:
        """Submit on a caller-owned CUDA stream (a ``torch.cuda.Stream`` or a raw handle)
        instead of torch's current one (PreparedSequence.enqueue, runtime/sequence.py:66-69)."""
        handle = queue.cuda_stream if hasattr(queue, "cuda_stream") else int(queue)
        with torch.cuda.device(self.program.device):
            status = self.program.function()(*self.native_arguments, handle)
        if status != _native.OK:
            self._record("failed")
            _native.check(self.program.facts.entry, status)
        if self.blocks and self.program.distribution.gather_output:
            if not hasattr(queue, "cuda_stream"):
                raise NotImplementedError("gather_output on a caller-owned stream needs a torch.cuda.Stream")
            with torch.cuda.stream(queue):
                self.gather()
        self._record("launched")

    def result(self):
        if not self.outputs:
            return None
        return self.outputs[0] if len(self.outputs) == 1 else self.outputs

    def check(self) -> None:
        """Synchronise and raise if a bounded device-side wait gave up (tensor-core entries)."""
        for workspace in self.workspaces:
            detail = ctypes.c_int32(0)
            with torch.cuda.device(self.program.device):
                stream = torch.cuda.current_stream(self.program.device).cuda_stream
                status = _native.entry("b200_workspace_status")(workspace.data_ptr(), ctypes.byref(detail), stream)
            _native.check("b200_workspace_status", status)

    @property
    def observation(self) -> Observation | None:
        return self._observation

    def inspect_configurations(self):
        return self.program.inspect_configurations()


class PreparedSequence:
    """An ordered sequence of already-bound calls (runtime/sequence.py:39-104): construction
    and compile never launch; launch runs the members in order on the current stream."""

    def __init__(self, calls, *, outputs, owners=()):
        self.calls = tuple(calls)
        if not self.calls:
            raise ValueError("a prepared sequence requires at least one invocation")
        self._outputs = outputs
        self._owners = tuple(owners)

    def compile(self):
        for call in self.calls:
            call.compile()

    def launch(self):
        for call in self.calls:
            call.launch()

    def enqueue(self, queue):
        for call in self.calls:
            call.enqueue(queue)

    def result(self):
        return self._outputs

    @property
    def kernel_count(self):
        return sum(call.kernel_count if isinstance(call, PreparedSequence) else 1 for call in self.calls)

    @property
    def observations(self):
        return tuple(item for call in self.calls
                     for item in (call.observations if isinstance(call, PreparedSequence)
                                  else (call.observation,)) if item is not None)


@dataclass
class Artifact:
    """What materialising a generated program yields (CompiledArtifact)."""
    source: str
    mlir: str
    device: int
    runtime: B200Program
    device_type: str = "cuda"
    cache_directory: object = None

    @property
    def interface(self) -> Interface:
        return self.runtime.interface

    @property
    def observation(self):
        return self.runtime.observation

    @property
    def ir(self) -> dict:
        return {"intent": self.mlir}

    def run(self, *arguments):
        return self.runtime.run(*arguments)

    def prepare(self, *arguments, outputs: tuple | None = None) -> B200Call:
        return self.runtime.prepare_call(arguments, outputs=outputs)

    def launch(self, *arguments) -> None:
        self.runtime.launch(*arguments)

    __call__ = launch

    def inspect_configurations(self, *arguments, outputs: tuple | None = None):
        return self.prepare(*arguments, outputs=outputs).inspect_configurations()

    def as_torch_op(self, name: str):
        return register_operator(self, name)


# --------------------------------------------------------------------------- torch custom op
def register_operator(artifact, name: str):
    """Expose the artifact as a ``torch.library`` custom operator: schema from the
    public inputs, fake implementation from ``infer_outputs`` (no execution)."""
    interface = artifact.interface
    inputs = interface.inputs
    views = tuple((index, p) for index, p in enumerate(inputs) if isinstance(p, ViewParameter))
    if not views:
        raise NotImplementedError("PyTorch registration requires an input tensor to determine device dispatch")
    pieces = name.split("::")
    if len(pieces) != 2 or not all(piece.isidentifier() for piece in pieces):
        raise ValueError("operator name must be 'your_namespace::your_operator'")
    mutable = tuple(f"arg{index}" for index, p in views if p.writable)
    parameters = []
    for index, p in enumerate(inputs):
        if isinstance(p, ViewParameter):
            kind = f"Tensor(a{index}!)" if p.writable else "Tensor"
        elif p.dtype == "bool":
            kind = "bool"
        elif p.dtype in {"f16", "bf16", "f32", "f64"}:
            kind = "float"
        else:
            kind = "SymInt"
        parameters.append(f"{kind} arg{index}")
    returns = "Tensor" if len(interface.outputs) == 1 else "(" + ", ".join("Tensor" for _ in interface.outputs) + ")"
    schema = f"({', '.join(parameters)}) -> {returns}"
    signature = Signature(Parameter(f"arg{i}", Parameter.POSITIONAL_OR_KEYWORD) for i in range(len(parameters)))

    def adapt(invoke):
        def operator(*arguments, **keywords):
            return invoke(*signature.bind(*arguments, **keywords).args)
        return operator

    operator = torch.library.custom_op(name, adapt(artifact.run), mutates_args=mutable,
                                       device_types=artifact.device_type, schema=schema)
    operator.register_fake(adapt(lambda *arguments: artifact.runtime.infer_outputs(arguments)))
    return operator
