"""intent_b200 — a B200-native (sm_100a) provider for IntentDSL's operator hot path.

Five operator families — row softmax, LayerNorm, dense GEMM, causal
flash-attention, CSR SpMM — and the kernels that pair with them (CSR SpMV, softmax
backward, the LayerNorm backward pair, the attention backward trio) run as
hand-written CUDA kernels behind a C ABI (``include/intent_b200.h``).  Two front
doors reach them:

* with the reference installed: ``intent_b200.register()`` then
  ``intent.jit(kernel, backend="b200", compiler=intent_b200.COMPILER)``;
* stand-alone: ``intent_b200.jit(intent_b200.kernels.stable_softmax)``.

Both run the same compile step (``b200-compile``), the same binder
(``intent_b200.runtime``) and the same kernels; there is no other execution path.
``python -m intent_b200 describe|doctor`` reports the interface and the environment.
"""
from __future__ import annotations

import os

from . import _native, ops, sharding
from .compilation import (COMPILER, CompilationStageError, CompileOptions, GeneratedProgram, JITKernel,
                  device_capabilities, generate, jit, kernels)
from .host_buffers import HostBuffers
from .runtime import Artifact, B200Call, B200Program, Interface, PreparedSequence, register_operator

__all__ = ["register", "jit", "generate", "kernels", "COMPILER", "CompileOptions", "GeneratedProgram",
           "JITKernel", "Artifact", "PreparedSequence", "B200Program", "B200Call", "Interface", "CompilationStageError",
           "device_capabilities", "register_operator", "ops", "sharding", "HostBuffers"]


def register(*, set_compiler: bool = True) -> None:
    """Add ``"b200"`` to the reference's provider catalog.

    Call before importing ``intent.examples.__main__`` or ``intent.tools.cli``:
    they snapshot the backend names at import
    (``python/intent/targets/registry.py:6``).  With ``set_compiler`` the
    ``INTENT_COMPILER`` variable is pointed at ``b200-compile`` unless the
    caller already chose a compiler
    (``python/intent/compiler/toolchain.py:29-54``); other providers need the
    reference's own ``intent-compile`` and can be given it per call with
    ``intent.jit(..., compiler=...)``.
    """
    from intent.targets.components import COMPONENTS

    COMPONENTS["b200"] = "intent_b200.provider"
    if set_compiler:
        os.environ.setdefault("INTENT_COMPILER", str(COMPILER))
