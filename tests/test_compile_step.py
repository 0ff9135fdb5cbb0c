"""b200-compile honours the reference compiler's CLI contract
(tools/intent-compile/intent-compile.cpp:37-178) and classifies kernel IR by structure."""
import json
import subprocess

import pytest

from intent_b200 import compilation as b200
from intent_b200.runtime import B200Facts, NativeLayout

KIR = b200.KIR_DIRECTORY

EXPECTED = {
    "stable_softmax": ("softmax", {"dtype": 0}),
    "stable_softmax_f16": ("softmax", {"dtype": 1}),
    "chunked_softmax_bf16": ("softmax", {"dtype": 2}),
    "layer_norm_f16": ("layer_norm", {"dtype": 1, "centered": 1}),
    "layer_norm_bf16": ("layer_norm", {"dtype": 2, "centered": 1}),
    "weighted_layer_norm": ("layer_norm", {"dtype": 0, "centered": 0}),
    "gemm": ("gemm", {"dtype": 1, "relu": 0}),
    "gemm_relu": ("gemm", {"dtype": 1, "relu": 1}),
    "bf16_gemm": ("gemm", {"dtype": 2, "relu": 0}),
    "flash_attention_bf16_fwd": ("flash_attention", {"dtype": 2, "head_group": 1, "causal": 1}),
    "flash_attention_fwd": ("flash_attention", {"dtype": 1, "head_group": 1, "causal": 1}),
    "flash_attention_fwd_noncausal": ("flash_attention", {"dtype": 1, "head_group": 1, "causal": 0}),
    "flash_gqa_attention_fwd": ("flash_attention", {"dtype": 1, "head_group": 4, "causal": 1}),
    "csr_spmm": ("csr_spmm", {}),
    "csr_spmv": ("csr_spmv", {}),
    "softmax_backward": ("softmax_backward", {"dtype": 0}),
    "layer_norm_backward_rows": ("layer_norm_backward_rows", {}),
    "attention_backward_delta": ("attention_backward_delta", {"dtype": 1}),
    "attention_backward_dkdv": ("attention_backward_dkdv", {"dtype": 1, "head_group": 4, "causal": 1}),
    "attention_backward_dkdv_noncausal": ("attention_backward_dkdv", {"dtype": 1, "head_group": 1, "causal": 0}),
    "attention_backward_dq": ("attention_backward_dq", {"dtype": 1, "head_group": 4, "causal": 1}),
    "attention_backward_dq_noncausal": ("attention_backward_dq", {"dtype": 1, "head_group": 1, "causal": 0}),
    "layer_norm_backward_reduce": ("layer_norm_backward_reduce", {}),
    "csr_spmm_262144": ("csr_spmm", {}),
}


def compile_text(text, *extra):
    return b200.run_compiler(text, b200.B200_CAPABILITIES, *extra)


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_classification_and_metadata(name):
    ir, source, metadata = compile_text((KIR / f"{name}.mlir").read_text())
    family, tail = EXPECTED[name]
    facts = B200Facts.read(metadata)
    assert facts.family == family
    assert {n: v for n, _, v in facts.tail} == tail
    assert ir == (KIR / f"{name}.mlir").read_text()          # IR is echoed
    assert f"family {family}" in source
    layout = NativeLayout.read(metadata)                         # the NativeABI flavour parses
    assert metadata["target"] == {"family": "b200_native", "capabilities": b200.B200_CAPABILITIES}
    assert metadata["compile_options"] == {"numerics": "source", "optimizations": {}, "optimization_remarks": False}
    assert bool(layout.workspaces) == (family in {"gemm", "flash_attention", "attention_backward_dkdv", "attention_backward_dq",
                                                 "csr_spmm"})


def test_interface_of_softmax_keeps_author_constraints():
    _, _, metadata = compile_text((KIR / "stable_softmax.mlir").read_text())
    x, y = metadata["interface"]["parameters"]
    assert x == {"kind": "view", "name": "x", "dtype": "f32", "shape": [-1, -1], "dimensions": [2, 1],
                 "strides": [None, 1], "access": 0, "alias": "", "noalias": True}
    assert y["access"] == 1 and y["dimensions"] == [2, 1]
    roles = [(s["role"], s["parameter"], s.get("axis")) for s in metadata["native"]["slots"]]
    assert roles[:5] == [("pointer", 0, None), ("extent", 0, 0), ("extent", 0, 1), ("stride", 0, 0), ("stride", 0, 1)]


def test_static_extents_survive():
    _, _, metadata = compile_text((KIR / "csr_spmm_262144.mlir").read_text())
    shapes = [p["shape"] for p in metadata["interface"]["parameters"]]
    assert shapes == [[262145], [8388608], [8388608], [262144, 128], [262144, 128]]


def test_head_group_substitution():
    text = b200.kernels.flash_attention_bf16_fwd.kir({"HEAD_GROUP": 8, "CAUSAL": True})
    _, _, metadata = compile_text(text)
    assert {n: v for n, _, v in B200Facts.read(metadata).tail}["head_group"] == 8


def test_unsupported_kernel_is_refused_without_fallback():
    with pytest.raises(b200.CompilationStageError) as error:
        compile_text((KIR / "gemm_f32.mlir").read_text())
    assert error.value.stage == "provider_pipeline"


def test_compile_options_are_echoed():
    options = b200.CompileOptions(numerics="relaxed_normalization", optimization_remarks=True)
    _, _, metadata = compile_text((KIR / "gemm.mlir").read_text(), options)
    assert metadata["compile_options"] == options.metadata()


def run(*arguments, text=None):
    return subprocess.run([str(b200.COMPILER), *arguments], input=text, text=True, capture_output=True)


def test_compiler_info_has_the_validated_shape():
    info = json.loads(run("--compiler-info").stdout)
    assert info["providers"] == {"b200": {"family": "b200_native", "available": True, "profiles": []}}
    assert info["stages"] == ["kir", "shared", "provider"]
    assert set(info["outputs"]) == set(info["stages"])
    assert info["failure_stages"]["6"] == "provider_pipeline"


def test_exit_codes(tmp_path):
    text = (KIR / "gemm.mlir").read_text()
    facts = json.dumps(b200.B200_CAPABILITIES)
    outputs = [f"--ir-output={tmp_path / 'k.mlir'}", f"--source-output={tmp_path / 'k.src'}",
               f"--metadata-output={tmp_path / 'a.json'}"]
    assert run("--compiler-info", "--target=b200").returncode == 1
    assert run("--target=triton", f"--target-options={facts}", *outputs, "-", text=text).returncode == 1
    assert run(*outputs, "-", text=text).returncode == 1                      # no --target
    assert run("--target=b200", f"--target-options={facts}", "-", text=text).returncode == 8  # no outputs
    assert run("--target=b200", f"--target-options={facts}", *outputs, "-", text="garbage").returncode == 2
    other = dict(b200.B200_CAPABILITIES, compute_capability_major=9)
    assert run("--target=b200", f"--target-options={json.dumps(other)}", *outputs, "-", text=text).returncode == 6
    assert run("--stop-after-kir", outputs[0], "-", text=text).returncode == 0
    assert (tmp_path / "k.mlir").read_text() == text


def test_generated_program_round_trip(tmp_path):
    program = b200.generate(b200.kernels.layer_norm_f16)
    saved = program.save(tmp_path / "program")
    loaded = b200.GeneratedProgram.load(saved)
    assert loaded.metadata == program.metadata and loaded.source == program.source and loaded.ir == program.ir
    with pytest.raises(b200.CompilationStageError):
        program.save(saved)


def _refused(text):
    with pytest.raises(b200.CompilationStageError) as error:
        compile_text(text)
    assert error.value.stage == "provider_pipeline"
    return str(error.value)


def test_programs_that_only_look_like_a_family_are_refused():
    """The operation counts shortlist a family; the operation graph must then be one of the
    structures the provider implements.  Near misses get the pipeline error, never another kernel."""
    relu = (KIR / "gemm_relu.mlir").read_text()
    assert "value = 0x0000000000000000 : f64" in relu
    # maximum(acc, 1.0) has the counts of the ReLU epilogue, but is not ReLU
    message = _refused(relu.replace("value = 0x0000000000000000 : f64", "value = 0x3FF0000000000000 : f64"))
    assert "gemm" in message and "differ" in message
    softmax = (KIR / "stable_softmax.mlir").read_text()
    # exp(max - x) instead of exp(x - max): same counts, operands of the subtract swapped
    assert '"intent.binary"(%v8, %v15)' in softmax
    _refused(softmax.replace('"intent.binary"(%v8, %v15)', '"intent.binary"(%v15, %v8)'))
    # d / 1.0 instead of 1.0 / d
    assert '"intent.binary"(%v23, %v22)' in softmax
    _refused(softmax.replace('"intent.binary"(%v23, %v22)', '"intent.binary"(%v22, %v23)'))
    # an approximate exponential is another numerics contract
    norm = (KIR / "layer_norm_f16.mlir").read_text()
    assert "unary_operator<rsqrt>" in norm
    _refused(norm.replace("unary_operator<rsqrt>", "unary_operator<sqrt>"))


def test_what_an_author_may_rename_does_not_change_the_structure():
    """Function, parameter, value and local names, source locations and static extents are not
    part of a program's structure: the two CSR instances (8192 and 262144 rows) are one kernel."""
    import re
    import subprocess
    from intent_b200.build import STRUCTURES, structure_table

    def structure(text):
        done = subprocess.run([str(b200.COMPILER), "--structure", "-"], input=text, capture_output=True, text=True)
        assert done.returncode == 0, done.stderr
        return done.stdout.split()

    small, large = (structure((KIR / name).read_text()) for name in ("csr_spmm.mlir", "csr_spmm_262144.mlir"))
    assert small == large and small[0] == "csr_spmm"
    text = (KIR / "stable_softmax.mlir").read_text()
    renamed = re.sub(r'loc\("[^"]*":\d+:\d+\)', 'loc("elsewhere.py":1:1)', text)
    renamed = renamed.replace("@stable_softmax", "@my_kernel").replace('"x", 0', '"inputs", 0')
    renamed = re.sub(r"%v(\d+)", lambda m: f"%t{int(m.group(1)) + 100}", renamed)
    assert structure(renamed) == structure(text)
    compile_text(renamed)                                          # and it still compiles to the softmax entry
    attention = (KIR / "flash_attention_bf16_fwd.mlir").read_text()
    grouped = b200.kernels.flash_attention_bf16_fwd.kir({"HEAD_GROUP": 8, "CAUSAL": True})
    assert grouped != attention and structure(grouped) == structure(attention)
    assert STRUCTURES.read_text() == structure_table(), "run `python -m intent_b200.build --structures`"
