"""Host-side native code under AddressSanitizer and UndefinedBehaviorSanitizer (gcc): the
compile step over every packaged kernel IR and over malformed inputs, and the CPU oracle over
small cases of every operator.  A sanitizer report fails the run (the sanitized binaries exit
non-zero with a report on stderr)."""
import os
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
KIR = ROOT / "intent_b200" / "kir"
FLAGS = ["-g", "-O1", "-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"]

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="needs gcc")


@pytest.fixture(scope="module")
def sanitized_compiler(tmp_path_factory):
    target = tmp_path_factory.mktemp("sanitized") / "b200-compile"
    subprocess.run(["g++", "-std=c++17", *FLAGS, "-o", str(target), str(ROOT / "intent_b200" / "compiler" / "b200_compile.cpp")],
                   check=True, capture_output=True, text=True)
    return target


def run(executable, text, directory, *extra):
    command = [str(executable), "--target=b200", '--target-options={"compute_capability_major": 10}', *extra,
               f"--ir-output={directory / 'k.mlir'}", f"--source-output={directory / 'k.source'}",
               f"--metadata-output={directory / 'a.json'}", "-"]
    return subprocess.run(command, input=text, capture_output=True, text=True,
                          env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1", UBSAN_OPTIONS="print_stacktrace=1"))


def test_compile_step_is_clean_on_every_packaged_kernel(sanitized_compiler, tmp_path):
    for path in sorted(KIR.glob("*.mlir")):
        done = run(sanitized_compiler, path.read_text(), tmp_path)
        assert "Sanitizer" not in done.stderr and "runtime error" not in done.stderr, (path.name, done.stderr[-2000:])
        assert done.returncode in (0, 6), (path.name, done.returncode, done.stderr[-500:])   # 6: refused by design (f32 GEMM)


def test_compile_step_is_clean_on_malformed_input(sanitized_compiler, tmp_path):
    text = (KIR / "flash_attention_bf16_fwd.mlir").read_text()
    cases = ["", "module {}", text[: len(text) // 2], text.replace("(", "", 5), text.replace(">", "", 7),
             text.replace("tensor<", "tensor", 3), "func.func @f(" + "%v0: " * 50, text.replace('"', "", 9),
             'func.func @f(%v0: !intent.view<tensor<?xf32>>) {intent.parameter = #intent.parameter<"x", 0>}']
    for case in cases:
        done = run(sanitized_compiler, case, tmp_path)
        assert "Sanitizer" not in done.stderr and "runtime error" not in done.stderr, done.stderr[-2000:]
        assert done.returncode != 0


def test_oracle_is_clean_under_the_sanitizers(tmp_path):
    """oracle.c compiled with the sanitizers into an executable of its own (oracle/selfcheck.c
    drives every operator on small shapes, ragged and empty rows included)."""
    target = tmp_path / "oracle_selfcheck"
    subprocess.run(["gcc", "-std=c11", *FLAGS, "-fopenmp", "-o", str(target), str(ROOT / "oracle" / "selfcheck.c"),
                    str(ROOT / "oracle" / "oracle.c"), "-lm", "-lpthread"], check=True, capture_output=True, text=True)
    done = subprocess.run([str(target)], capture_output=True, text=True,
                          env=dict(os.environ, ASAN_OPTIONS="detect_leaks=1"))
    assert done.returncode == 0 and "selfcheck ok" in done.stdout, done.stderr[-3000:]
    assert "Sanitizer" not in done.stderr and "runtime error" not in done.stderr
