"""Drop-in boundary against the UNMODIFIED reference package (the copy installed under
baseline/_ref): registration beside the existing providers, the reference's own compiler
driver running b200-compile, its contract parser accepting the artifact, and its example
runner compiling the registered programs for the b200 backend.  Nothing here needs a GPU."""
import sys

import pytest

from conftest import HAS_REFERENCE, REFERENCE_PYTHON

pytestmark = pytest.mark.skipif(not HAS_REFERENCE, reason="reference package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def intent(tmp_path_factory):
    import os
    sys.path.insert(0, str(REFERENCE_PYTHON))
    os.environ["INTENT_CACHE_DIR"] = str(tmp_path_factory.mktemp("intent-cache"))
    os.environ.pop("INTENT_COMPILER", None)
    import intent
    import intent_b200
    intent_b200.register()
    yield intent
    sys.path.remove(str(REFERENCE_PYTHON))


def explicit_target():
    from intent.targets.nvidia.specification import NVIDIACapabilities, NVIDIACompilationTarget
    from intent_b200.compilation import B200_CAPABILITIES
    return NVIDIACompilationTarget("b200", NVIDIACapabilities(**B200_CAPABILITIES))


def test_provider_is_registered_beside_the_existing_ones(intent):
    from intent.targets.components import COMPONENTS
    from intent.targets.provider import provider
    assert {"triton", "cutile", "mojo", "b200"} <= set(COMPONENTS)
    declared = provider("b200")
    assert declared.family == "gpu" and declared.execution_model == "b200_native"
    assert declared.local.device_kind == "cuda" and declared.local.indexed
    import intent_b200.provider as module
    assert isinstance(module.INSTALLATION, dict)
    from intent.targets.registry import make_target
    assert make_target("b200", {"device": 1}).device == 1


def test_reference_driver_compiles_the_five_kernels(intent):
    from intent.examples.kernels.contraction.gemm import Activation, gemm
    from intent.examples.kernels.normalization.layer_norm import layer_norm_f16
    from intent.examples.kernels.normalization.softmax import stable_softmax
    from intent.examples.kernels.sparse.csr_spmm import csr_spmm
    from intent.examples.kernels.streaming.attention import flash_attention_bf16_fwd
    cases = [(stable_softmax, None, "softmax"), (layer_norm_f16, None, "layer_norm"),
             (gemm, {"ACTIVATION": Activation.NONE}, "gemm"),
             (flash_attention_bf16_fwd, {"HEAD_GROUP": 1, "CAUSAL": True}, "flash_attention"),
             (csr_spmm, None, "csr_spmm")]
    for definition, constexprs, family in cases:
        program = intent.generate(definition, target=explicit_target(), constexprs=constexprs)
        assert program.metadata["b200"]["family"] == family
        assert program.target == explicit_target()
        names = [p.name for p in program.interface.parameters]
        assert names and program.interface.outputs
        from intent.runtime.native import NativeABI
        assert isinstance(program._contract.abi, NativeABI)
        assert len(program._contract.abi.argument_types()) == len(program.metadata["native"]["slots"])


def test_reference_driver_reports_refusal_as_a_stage_error(intent):
    from intent.examples.kernels.contraction.gemm import gemm_f32
    from intent.compiler.toolchain import CompilationStageError
    with pytest.raises(CompilationStageError) as error:
        intent.generate(gemm_f32, target=explicit_target())
    assert error.value.stage == "provider_pipeline"


def test_compile_options_survive_the_round_trip(intent):
    from intent.examples.kernels.normalization.softmax import stable_softmax
    options = intent.CompileOptions(numerics="relaxed_normalization", optimization_remarks=True)
    program = intent.generate(stable_softmax, target=explicit_target(), options=options)
    assert program.compile_options == options


def test_packaged_kernel_ir_is_what_the_frontend_emits_today(intent):
    """intent_b200/kir/*.mlir are current outputs of the reference frontend."""
    from pathlib import Path
    import intent as package
    from intent.examples.kernels.normalization.softmax import stable_softmax
    from intent.examples.kernels.contraction.gemm import Activation, gemm
    from intent_b200.compilation import KIR_DIRECTORY
    # source locations are recorded relative to the reference's root, where the package is python/intent
    root = str(Path(package.__file__).resolve().parent) + "/"
    for definition, constexprs, name in [(stable_softmax, None, "stable_softmax"),
                                         (gemm, {"ACTIVATION": Activation.RELU}, "gemm_relu")]:
        text = package.lower_to_mlir(definition, constexprs=constexprs).replace(root, "python/intent/")
        assert text == (KIR_DIRECTORY / f"{name}.mlir").read_text()


def test_runtime_binding_through_the_reference_artifact(intent):
    """bind() wraps the b200 runtime in the reference's CompiledArtifact; abstract
    binding (what FakeTensor tracing uses) works without a device."""
    import torch
    from intent.examples.kernels.normalization.softmax import stable_softmax
    from intent.runtime import CompiledArtifact
    from intent_b200.provider import B200Runtime
    from intent_b200.runtime import B200Program
    program = intent.generate(stable_softmax, target=explicit_target())
    runtime = B200Runtime(B200Program(program.metadata, 0), program.interface)
    artifact = CompiledArtifact(program.source, program.ir, 0, runtime, None, device_type="cuda")
    assert artifact.interface is program.interface
    out = runtime.infer_outputs((torch.empty(3, 5, device="meta"),))
    assert out.shape == (3, 5)
    op = artifact.as_torch_op("b200_test::reference_softmax")
    assert "Tensor arg0" in str(op._opoverload._schema)
