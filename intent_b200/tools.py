"""``describe`` and ``doctor`` for the b200 backend, with the reference tools' result shape
(``python/intent/tools/compilation.py:125-153`` and ``:343-455``): plain dictionaries with a
``status``, a ``scope`` sentence and ``tool_invoked_kernel: False``.  Neither compiles nor runs a
kernel.  ``python -m intent_b200 describe|doctor`` prints them as JSON.
"""
from __future__ import annotations

import ctypes
import importlib
import inspect
import json
import subprocess

from . import _native, compilation


def _declaration(item) -> str:
    try:
        return f"{getattr(item, '__name__', type(item).__name__)}{inspect.signature(item)}"
    except (TypeError, ValueError):
        return getattr(item, "__name__", repr(item))


def _failure(entry: dict, error: Exception, category: str) -> None:
    entry.update(status="unavailable", category=category,
                 error={"type": type(error).__name__, "message": str(error)})


def describe() -> dict:
    """Public call signatures, kernel definitions and C entries; nothing is probed."""
    import intent_b200

    result = {"target": "b200", "tool_invoked_kernel": False}
    try:
        result["backends"] = {"b200": {
            "toolchain": {"compiler": str(compilation.COMPILER), "library": str(_native.LIBRARY_PATH)},
            "target": {"family": "b200_native", "capability_fields": list(compilation.CAPABILITY_FIELDS)},
            "execution_model": "one process per GPU; entries enqueue on the caller's CUDA stream",
            "local_device": {"kind": "cuda", "indexed": True},
            "local_options": []}}
        result["api"] = {name: _declaration(getattr(intent_b200, name)) for name in (
            "jit", "JITKernel", "generate", "GeneratedProgram", "CompileOptions", "PreparedSequence", "Artifact",
            "register")}
        result["kernels"] = sorted(name for name, value in vars(compilation.kernels).items()
                                   if isinstance(value, compilation.KernelDefinition))
        result["entries"] = sorted(_native.SIGNATURES)
        result["tools"] = {"describe": _declaration(describe), "environment": _declaration(doctor)}
        result.update(status="described",
                      scope="Declarations only; compiler availability and device support are not checked")
    except Exception as error:  # the reference tools report, they do not raise
        _failure(result, error, "interface_discovery")
    return result


def doctor(device: int | None = 0, *, compiler=None) -> dict:
    """Compiler start-up, the native library and its symbols, and (unless ``device`` is None) the
    CUDA device's suitability.  No kernel is compiled or executed."""
    checks: list[dict] = []
    result = {"target": "b200", "checks": checks, "tool_invoked_kernel": False,
              "scope": "Dependency and target resolution only; no kernel compilation or execution"}

    def check(name, category, action):
        entry = {"name": name, "category": category}
        try:
            entry.update(status="available", detail=action())
        except Exception as error:
            _failure(entry, error, category)
        checks.append(entry)
        return entry.get("detail")

    def compiler_information():
        path = compilation.compiler_path(compiler)
        done = subprocess.run([str(path), "--compiler-info"], capture_output=True, text=True, timeout=30)
        if done.returncode != 0:
            raise RuntimeError(f"{path} --compiler-info exited with {done.returncode}: {done.stderr.strip()}")
        facts = json.loads(done.stdout)
        if "b200" not in facts.get("providers", {}):
            raise NotImplementedError("the compile step does not list the b200 provider")
        return facts

    def native_library():
        handle = _native.library()
        missing = [name for name in _native.SIGNATURES if not hasattr(handle, name)]
        if missing:
            raise ImportError(f"{_native.LIBRARY_PATH} lacks {missing}")
        return {"path": str(_native.LIBRARY_PATH), "abi_version": int(handle.b200_abi_version()),
                "entries": len(_native.SIGNATURES)}

    def python_module(name):
        module = importlib.import_module(name)
        return {"path": getattr(module, "__file__", None), "version": str(getattr(module, "__version__", "not declared"))}

    def target():
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible to this process")
        status = _native.entry("b200_device_check")(ctypes.c_int(device))
        _native.check("b200_device_check", status)
        return {"device": device, "name": torch.cuda.get_device_name(device),
                "capabilities": compilation.device_capabilities(device)}

    check("b200 compile step", "compiler", compiler_information)
    check("native library", "compiler_resources", native_library)
    check("torch", "python_package", lambda: python_module("torch"))
    if device is None:
        result["scope"] = "Compiler and library only; the runtime device was not checked"
    else:
        check("target", "target_resolution", target)
    result["status"] = "available" if all(item["status"] == "available" for item in checks) else "unavailable"
    return result


def main(arguments=None) -> int:
    import argparse
    parser = argparse.ArgumentParser(prog="python -m intent_b200")
    parser.add_argument("command", choices=["describe", "doctor"])
    parser.add_argument("--device", default="0", help="CUDA device index, or 'none' to skip the device check")
    parsed = parser.parse_args(arguments)
    if parsed.command == "describe":
        report = describe()
    else:
        report = doctor(None if parsed.device == "none" else int(parsed.device))
    print(json.dumps(report, indent=2, default=str))
    return 0 if report["status"] in ("described", "available") else 1
