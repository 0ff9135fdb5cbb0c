"""In-tree build of the native parts: the CUDA library and the compile step.

``python -m intent_b200.build`` compiles

* ``intent_b200/csrc/*.cu``  -> ``intent_b200/lib/libintent_b200.so``  (nvcc, sm_100a only)
* ``intent_b200/compiler/b200_compile.cpp`` -> ``intent_b200/bin/b200-compile`` (g++)

nvcc cross-compiles without a GPU, so this runs anywhere the CUDA toolkit is
installed.  Objects are cached under ``build/`` and reused while their sources
(and the shared headers) are older.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "lib" / "libintent_b200.so"
COMPILER = PACKAGE / "bin" / "b200-compile"
OBJECTS = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc was not found; the CUDA toolkit is required to build intent_b200")
    return found


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(source.stat().st_mtime > stamp for source in sources)


def _run(command: list[str]) -> str:
    completed = subprocess.run(command, capture_output=True, text=True)
    if completed.returncode:
        raise RuntimeError(f"{' '.join(command)}\n{completed.stdout}{completed.stderr}")
    return completed.stdout + completed.stderr


CHECKED_LIBRARY = PACKAGE / "lib" / "libintent_b200_checked.so"


def build_library(*, force: bool = False, verbose: bool = False, resource_usage: bool = False,
                  checked: bool = False) -> Path:
    """``checked=True`` builds the variant with device-side index checks (-DB200_CHECKED) as
    ``libintent_b200_checked.so``; ``INTENT_B200_CHECKED=1`` makes the package load it."""
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "intent_b200.h"]
    objects_directory = ROOT / "build" / "obj_checked" if checked else OBJECTS
    library = CHECKED_LIBRARY if checked else LIBRARY
    objects_directory.mkdir(parents=True, exist_ok=True)
    library.parent.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(source: Path) -> tuple[Path, str]:
        target = objects_directory / (source.stem + ".o")
        log = ""
        if force or resource_usage or _stale(target, [source, *headers]):
            flags = NVCC_FLAGS + (["-Xptxas", "-v"] if resource_usage else []) + (["-DB200_CHECKED"] if checked else [])
            log = _run([nvcc, *flags, "-c", str(source), "-o", str(target)])
        return target, log

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as pool:
        results = list(pool.map(compile_one, sources))
    objects = [target for target, _ in results]
    if verbose or resource_usage:
        for _, log in results:
            if log.strip():
                print(log)
    if force or _stale(library, objects):
        _run([nvcc, "-shared", "-o", str(library), *map(str, objects), "-gencode",
              "arch=compute_100a,code=sm_100a"])
    return library


STRUCTURES = PACKAGE / "compiler" / "structures.inc"


def build_compiler(*, force: bool = False) -> Path:
    source = PACKAGE / "compiler" / "b200_compile.cpp"
    COMPILER.parent.mkdir(parents=True, exist_ok=True)
    if force or _stale(COMPILER, [source, STRUCTURES]):
        _run([os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-Wall", "-Wextra", "-o",
              str(COMPILER), str(source)])
    return COMPILER


def structure_table() -> str:
    """The table the compile step checks programs against: family and canonical-structure hash
    of every packaged kernel IR (``intent_b200/kir/*.mlir``), as ``b200-compile --structure``
    reports them.  Kernels the provider refuses (the f32 GEMM fixture) are left out."""
    lines = []
    for path in sorted((PACKAGE / "kir").glob("*.mlir")):
        completed = subprocess.run([str(COMPILER), "--structure", "-"], input=path.read_text(encoding="utf-8"),
                                   capture_output=True, text=True)
        if completed.returncode:
            continue
        family, digest = completed.stdout.split()
        lines.append(f'    {{"{family}", 0x{digest}ull, "{path.name}"}},\n')
    return "".join(lines)


def refresh_structures() -> bool:
    """Regenerates structures.inc after the packaged kernel IR changed; returns True when the
    file changed (the compile step is rebuilt with the new table)."""
    build_compiler()
    table = structure_table()
    if STRUCTURES.exists() and STRUCTURES.read_text() == table:
        return False
    STRUCTURES.write_text(table)
    build_compiler(force=True)
    return True


REFERENCE_INSTALL = ROOT / "baseline" / "_ref"


def reference_checkout() -> Path | None:
    """The reference checkout, when this machine has one: named by INTENT_REFERENCE, else a
    ``reference`` directory beside this repository."""
    candidate = Path(os.environ.get("INTENT_REFERENCE", ROOT.parent / "reference"))
    return candidate if (candidate / "python" / "intent" / "__init__.py").is_file() else None


def install_reference() -> Path | None:
    """Installs the reference's pure-Python package (and its example scripts) from the
    checkout into ``baseline/_ref``, which is kept out of version control.  The provider is
    tested through the unmodified reference from there on machines without the checkout.
    (``pip install`` of the checkout is not possible offline: its build backend needs
    setuptools-scm and the LLVM/MLIR 20 SDK; the Python package itself needs neither.)"""
    checkout = reference_checkout()
    if checkout is None:
        return REFERENCE_INSTALL if (REFERENCE_INSTALL / "intent" / "__init__.py").is_file() else None
    stamp = REFERENCE_INSTALL / ".installed-from"
    newest = max(path.stat().st_mtime for path in (checkout / "python" / "intent").rglob("*.py"))
    if stamp.is_file() and stamp.stat().st_mtime >= newest and stamp.read_text() == str(checkout):
        return REFERENCE_INSTALL
    if REFERENCE_INSTALL.exists():
        shutil.rmtree(REFERENCE_INSTALL)
    ignore = shutil.ignore_patterns("__pycache__", "*.pyc")
    shutil.copytree(checkout / "python" / "intent", REFERENCE_INSTALL / "intent", ignore=ignore)
    if (checkout / "examples").is_dir():
        shutil.copytree(checkout / "examples", REFERENCE_INSTALL / "examples", ignore=ignore)
    stamp.write_text(str(checkout))
    return REFERENCE_INSTALL


def build_all(*, force: bool = False, verbose: bool = False) -> None:
    build_library(force=force, verbose=verbose)
    build_library(force=force, verbose=verbose, checked=True)
    build_compiler(force=force)
    install_reference()


if __name__ == "__main__":
    arguments = set(sys.argv[1:])
    if "--resource-usage" in arguments:
        build_library(force=True, resource_usage=True)
    elif "--structures" in arguments:
        print("structures.inc", "updated" if refresh_structures() else "is current")
    else:
        build_all(force="--force" in arguments, verbose=True)
    print(LIBRARY)
