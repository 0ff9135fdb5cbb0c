"""The ``b200`` provider declaration for the reference's registry.

Importing this module needs the reference package (``import intent``).  It is
what ``intent.targets.provider.provider("b200")`` loads after
``intent_b200.register()`` has added the name to the component catalog
(``python/intent/targets/components.json``, looked up lazily at
``python/intent/targets/provider.py:51-56``).  The declaration has the shape of
the reference's own GPU providers (``python/intent/targets/triton.py:10-51``):

* family ``"gpu"`` so target facts travel as ``NVIDIACompilationTarget``
  (``python/intent/targets/nvidia/specification.py:32-57``);
* execution model ``"b200_native"`` (anything but ``"block"``), so the contract
  reader parses the NativeABI flavour of artifact.json
  (``python/intent/runtime/contract.py:109-113``);
* ``bind`` wraps the b200 host runtime in a ``CompiledArtifact``; launches go
  to ``libintent_b200.so`` on torch's current stream.  No Triton / cuTile / Mojo
  lowering and no other provider is ever consulted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import ClassVar

from intent.runtime import CompiledArtifact
from intent.runtime.native import NativePreparedRuntime
from intent.targets.execution import indexed_key, torch_storage
from intent.targets.nvidia import NVIDIATarget
from intent.targets.nvidia.specification import read_nvidia_target
from intent.targets.nvidia.target import ResolvedNVIDIATarget
from intent.targets.provider import EnvironmentCheck, LocalExecution, Provider

from . import _native
from .runtime import B200Facts, B200Program

INSTALLATION = {
    "modules": ("torch",), "requirements": (), "torch": "2.11.0+cu128",
    "torch_index": "https://download.pytorch.org/whl/cu128", "python_max": (3, 12),
    "toolchain": "NVIDIA B200 (sm_100a), driver with CUDA 12.8+, libintent_b200.so built by nvcc 12.8+",
}


@dataclass(frozen=True, slots=True)
class B200Target(NVIDIATarget):
    provider: ClassVar[str] = "b200"


class B200Runtime(NativePreparedRuntime):
    """The reference-facing face of ``B200Program``: same binder and launch, with
    the reference's typed ``PublicInterface`` exposed for ``as_torch_op``
    (``python/intent/integrations/torch.py:27-93``)."""

    def __init__(self, program: B200Program, interface) -> None:
        self._program = program
        self.interface = interface

    @property
    def observation(self):
        return self._program.observation

    @property
    def configuration_descriptions(self):
        return self._program.configuration_descriptions

    def inspect_configurations(self):
        return self._program.inspect_configurations()

    def prepare(self, arguments: tuple, *, explicit_outputs: bool = False):
        return self._program.prepare(arguments, explicit_outputs=explicit_outputs)

    def infer_outputs(self, arguments: tuple):
        return self._program.infer_outputs(arguments)

    def close(self) -> None:
        self._program.close()


def _read_facts(source, metadata, abi):
    return B200Facts.read(metadata)


@dataclass(frozen=True, slots=True)
class ResolvedB200Target(ResolvedNVIDIATarget):
    """A resolved device plus the two local options of this provider.  ``gpus`` (number of
    ranks, or their CUDA ordinals in rank order) and ``gather_output`` spread one call over
    the processes of a ``torch.distributed`` group, one per GPU (``intent_b200.sharding``);
    the reference's own providers are single-device
    (``python/intent/targets/local.py:36-45``)."""
    gpus: object = None
    gather_output: bool = False


def _resolve(device, *, workers, gpus=None, gather_output=False):
    """``LocalExecution.resolve`` (called from ``python/intent/targets/local.py:60-67`` with the
    whitelisted ``backend_options`` as keywords)."""
    if workers is not None:
        raise ValueError("workers is a CPU execution budget")
    plain = B200Target(device=device.index).resolve()
    frozen = tuple(gpus) if isinstance(gpus, (list, tuple)) else gpus
    return ResolvedB200Target(plain.compilation, plain.device, frozen, bool(gather_output))


def _bind(program, target):
    _native.check("b200_device_check", _native.entry("b200_device_check")(int(target.device)))
    program_runtime = B200Program(program.metadata, target.device, gpus=getattr(target, "gpus", None),
                                  gather_output=getattr(target, "gather_output", False))
    runtime = B200Runtime(program_runtime, program.interface)
    return CompiledArtifact(program.source, program.ir, target.device, runtime, None, device_type="cuda")


def _environment_checks(target):
    def native_library():
        handle = _native.library()
        return {"path": str(_native.LIBRARY_PATH), "abi_version": handle.b200_abi_version()}

    def device():
        if target is None:
            raise RuntimeError("the b200 device check requires a resolved local GPU")
        _native.check("b200_device_check", _native.entry("b200_device_check")(int(target.device)))
        return {"device": target.device, "architecture": "sm_100a"}

    return (EnvironmentCheck("intent_b200 CUDA library", "provider_toolchain", native_library),
            EnvironmentCheck("B200 device", "provider_device", device))


PROVIDER = Provider(
    "gpu", B200Target, _read_facts, _bind, _environment_checks,
    LocalExecution("cuda", True, frozenset({"gpus", "gather_output"}), _resolve, indexed_key, torch_storage),
    "b200_native", read_nvidia_target)
