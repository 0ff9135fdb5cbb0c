"""ctypes binding of ``libintent_b200.so`` (the C ABI declared in ``include/intent_b200.h``).

The library is loaded from the package directory only, and loading fails
loudly: there is no CPU or PyTorch fallback behind these entries, matching the
reference's rule that a failing backend never switches provider
(``doc/getting-started/usage.en.md:21``).
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from threading import Lock

# INTENT_B200_CHECKED=1 selects the build with device-side index checks (python -m intent_b200.build
# compiles both); it is slower and meant for debugging a caller's CSR arrays, not for production.
_CHECKED = os.environ.get("INTENT_B200_CHECKED", "") not in ("", "0")
LIBRARY_PATH = Path(__file__).resolve().parent / "lib" / ("libintent_b200_checked.so" if _CHECKED else "libintent_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_UNSUPPORTED_LAYOUT = 2
ERR_CUDA = 3
ERR_DEVICE = 4
ERR_DEVICE_TIMEOUT = 5

DTYPE_CODES = {"f32": 0, "f16": 1, "bf16": 2}
WORKSPACE_WORDS = 64

_P, _I64, _I32, _F32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float


def _view(rank: int) -> list:
    return [_P] + [_I64] * (2 * rank)


# entry -> argument types, exactly the declaration order of include/intent_b200.h
SIGNATURES = {
    "b200_softmax": _view(2) + _view(2) + [_I32, _P],
    "b200_layer_norm": _view(2) + _view(1) + _view(1) + _view(2) + [_F32, _F32, _I32, _I32, _P],
    "b200_gemm": _view(2) + _view(2) + _view(2) + _view(1) + [_I32, _I32, _P],
    "b200_gemm_static_scratch": _view(2) + _view(2) + _view(2) + [_I32, _I32, _I32, _P],
    "b200_flash_attention": _view(4) * 4 + [_F32] + _view(1) + [_I32, _I32, _I32, _P],
    "b200_csr_spmm": _view(1) * 3 + _view(2) * 2 + _view(1) + [_P],
    "b200_csr_spmv": _view(1) * 5 + [_P],
    "b200_softmax_backward": _view(2) * 3 + [_I32, _P],
    "b200_layer_norm_backward_rows": _view(2) * 2 + _view(1) * 3 + _view(2) * 3 + [_F32, _P],
    "b200_layer_norm_backward_reduce": _view(2) * 2 + _view(1) * 2 + [_P],
    "b200_attention_backward_delta": _view(4) * 2 + _view(3) + [_I32, _P],
    "b200_attention_backward_dkdv": _view(4) * 4 + _view(3) * 2 + _view(4) * 2 + [_F32] + _view(1) + [_I32, _I32, _I32, _P],
    "b200_attention_backward_dq": _view(4) * 4 + _view(3) * 2 + _view(4) + [_F32] + _view(1) + [_I32, _I32, _I32, _P],
    "b200_csr_validate": [_P, _I64, _P, _I64, _I64, ctypes.POINTER(_I64), _P],
    "b200_gather_probe": [_P, _I64, _I64, _I32, _I32, _P, _P, _P],
    "b200_workspace_status": [_P, ctypes.POINTER(_I32), _P],
    "b200_selftest_bounded_wait": _view(1) + [_I64, _P],
    "b200_device_check": [ctypes.c_int],
    "b200_device_capabilities": [ctypes.c_int, ctypes.POINTER(_I64)],
    "b200_abi_version": [],
    "b200_last_error": [ctypes.c_char_p, _I64],
}

_lock = Lock()
_library = None


class NativeLibraryMissing(RuntimeError):
    """The CUDA extension has not been built; nothing else can run the kernels."""


class NativeCallError(RuntimeError):
    def __init__(self, entry: str, status: int, message: str):
        super().__init__(f"{entry} failed with status {status} ({message})")
        self.entry, self.status = entry, status


def library() -> ctypes.CDLL:
    global _library
    with _lock:
        if _library is None:
            if not LIBRARY_PATH.exists():
                raise NativeLibraryMissing(
                    f"{LIBRARY_PATH} is missing: build it with `python -m intent_b200.build` "
                    "(nvcc, sm_100a). intent_b200 has no fallback execution path.")
            handle = ctypes.CDLL(str(LIBRARY_PATH))
            for name, argtypes in SIGNATURES.items():
                function = getattr(handle, name)  # AttributeError: the build is stale
                function.argtypes = argtypes
                function.restype = ctypes.c_int
            handle.b200_status_string.argtypes = [ctypes.c_int]
            handle.b200_status_string.restype = ctypes.c_char_p
            _library = handle
    return _library


def entry(name: str):
    if name not in SIGNATURES:
        raise KeyError(f"{name} is not an entry of the intent_b200 C ABI")
    return getattr(library(), name)


def last_error() -> str:
    buffer = ctypes.create_string_buffer(512)
    library().b200_last_error(buffer, 512)
    return buffer.value.decode(errors="replace")


def check(name: str, status: int) -> None:
    """Map a non-zero status onto the exception the reference's binders raise for
    the same condition (``python/intent/runtime/native_requirements.py:66-91``)."""
    if status == OK:
        return
    message = last_error() or library().b200_status_string(status).decode()
    if status == ERR_INVALID_ARGUMENT:
        raise ValueError(f"{name}: {message}")
    if status == ERR_UNSUPPORTED_LAYOUT:
        raise NotImplementedError(f"{name}: {message}")
    raise NativeCallError(name, status, message)
