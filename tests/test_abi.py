"""The C-ABI library loads and exports every symbol include/intent_b200.h declares."""
import ctypes
import re
from pathlib import Path

from intent_b200 import _native

HEADER = Path(__file__).resolve().parents[1] / "include" / "intent_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    found = {}
    for match in re.finditer(r"\b(?:int|const char \*)\s*(b200_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        arguments = match.group(2).strip()
        found[match.group(1)] = 0 if arguments in {"", "void"} else len(arguments.split(","))
    return found


def test_header_declares_the_operator_entries():
    names = declared_functions()
    for entry in ("b200_softmax", "b200_layer_norm", "b200_gemm", "b200_flash_attention", "b200_csr_spmm",
                  "b200_csr_validate", "b200_workspace_status", "b200_device_check", "b200_abi_version"):
        assert entry in names


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(str(_native.LIBRARY_PATH))
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is declared but not exported"


def test_checked_build_exports_the_same_symbols():
    """The variant with device-side index checks (-DB200_CHECKED) is built beside the regular
    library and is a drop-in for it."""
    from intent_b200 import build
    handle = ctypes.CDLL(str(build.CHECKED_LIBRARY))
    for name in declared_functions():
        assert hasattr(handle, name), f"{name} is missing from the checked build"


def test_python_signatures_match_header_arity():
    declared = declared_functions()
    for name, argtypes in _native.SIGNATURES.items():
        assert name in declared, name
        assert len(argtypes) == declared[name], name


def test_abi_version_and_status_strings():
    library = _native.library()
    assert library.b200_abi_version() == 1
    assert library.b200_status_string(0) == b"ok"
    assert b"layout" in library.b200_status_string(_native.ERR_UNSUPPORTED_LAYOUT)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import pytest
    monkeypatch.setattr(_native, "_library", None)
    monkeypatch.setattr(_native, "LIBRARY_PATH", tmp_path / "libintent_b200.so")
    with pytest.raises(_native.NativeLibraryMissing):
        _native.library()
