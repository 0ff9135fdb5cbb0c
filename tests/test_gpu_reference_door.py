"""The reference's own front door launching b200 kernels on a device.

``intent_b200.register()`` adds the provider to the UNMODIFIED reference package (the copy
under baseline/_ref); every call below then goes through the reference's classes:
``intent.jit`` -> ``JITKernel._artifact`` -> ``resolve_local`` -> ``generate`` (its compiler
driver runs b200-compile) -> ``program.materialize()`` -> the provider's ``bind`` ->
``CompiledArtifact.prepare / launch / as_torch_op`` (python/intent/jit/kernel.py:47-109,
python/intent/runtime/artifact.py:125-202), ``PreparedSequence``
(python/intent/runtime/sequence.py:39-104), ``HostBuffers``
(python/intent/runtime/host_buffers.py:53-149) and the example runner
(python/intent/examples/__main__.py:8-50).  Results are checked against the CPU oracle.
"""
import dataclasses
import json
import os
import subprocess
import sys

import pytest
import torch

import oracle
from conftest import HAS_REFERENCE, REFERENCE_PYTHON, ROOT, relative_error
from intent_b200 import workloads

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not HAS_REFERENCE, reason="reference package not installed under baseline/_ref")]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def intent(tmp_path_factory):
    sys.path.insert(0, str(REFERENCE_PYTHON))
    os.environ["INTENT_CACHE_DIR"] = str(tmp_path_factory.mktemp("intent-cache"))
    os.environ.pop("INTENT_COMPILER", None)
    import intent
    import intent_b200
    intent_b200.register()
    yield intent
    sys.path.remove(str(REFERENCE_PYTHON))


def test_softmax_run_explicit_outputs_and_prepared_launch(intent):
    from intent.examples.kernels.normalization.softmax import stable_softmax
    from intent.runtime import CompiledArtifact
    (x,) = workloads.softmax_inputs(256, 1024, seed=11)
    expected = oracle.softmax(x)
    kernel = intent.jit(stable_softmax, backend="b200")
    xd = x.to(DEV)
    y = kernel.run(xd)
    assert relative_error(y, expected) <= 1e-5
    assert isinstance(kernel.artifacts[0], CompiledArtifact)
    assert any("libintent_b200.so" in line for line in open("/proc/self/maps"))
    out = torch.empty_like(xd)
    kernel(xd, out)                                             # JITKernel.__call__, explicit Out
    assert torch.equal(out, y)
    out.zero_()
    kernel.artifacts[0](xd, out)                                # CompiledArtifact.__call__
    assert torch.equal(out, y)
    out.zero_()
    call = kernel.prepare(xd, outputs=(out,))                   # examples/softmax.py --prepared
    call.compile()
    call.launch()
    assert call.result() is out and torch.equal(out, y)
    observed = kernel.artifacts[-1].observation                 # examples/softmax.py --inspect-native
    assert json.loads(json.dumps(dataclasses.asdict(observed), default=str))["family"] == "softmax"
    with pytest.raises(ValueError, match="noalias"):
        kernel(xd, xd)
    kernel.close()


def test_the_five_kernels_against_the_oracle(intent):
    from intent.examples.kernels.contraction.gemm import Activation, gemm
    from intent.examples.kernels.normalization.layer_norm import layer_norm_f16
    from intent.examples.kernels.sparse.csr_spmm import csr_spmm
    from intent.examples.kernels.streaming.attention import flash_attention_bf16_fwd

    x, w, b, inv, eps = workloads.layer_norm_inputs(96, 4096, seed=12)
    y = intent.jit(layer_norm_f16, backend="b200").run(x.to(DEV), w.to(DEV), b.to(DEV), inv, eps)
    assert relative_error(y, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2

    a, bm = workloads.gemm_inputs(384, 512, 320, seed=13)
    kernel = intent.jit(gemm, backend="b200", constexprs={"ACTIVATION": Activation.NONE})
    call = kernel.prepare(a.to(DEV), bm.to(DEV))
    call.launch()
    assert relative_error(call.result(), oracle.gemm(a, bm)) <= 1e-2

    q, k, v, scale = workloads.attention_inputs(1, 4, 384, 128, seed=14, kv_heads=2)
    kernel = intent.jit(flash_attention_bf16_fwd, backend="b200", constexprs={"HEAD_GROUP": 2, "CAUSAL": True})
    out = kernel.run(q.to(DEV), k.to(DEV), v.to(DEV), scale)
    assert relative_error(out, oracle.attention(q, k, v, scale, head_group=2)) <= 1e-2

    ro, ci, va, dense = workloads.csr_inputs(8192, 8192, 32, 128, seed=15)
    y = intent.jit(csr_spmm, backend="b200").run(ro.to(DEV), ci.to(DEV), va.to(DEV), dense.to(DEV))
    assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci, va, dense))     # bit-exact


def test_as_torch_op_under_torch_compile(intent):
    """examples/softmax.py --torch-compile: prepare, register, call once, then capture."""
    from intent.examples.kernels.normalization.softmax import stable_softmax_f16
    x = torch.randn(512, 2048, device=DEV, dtype=torch.float16)
    softmax = intent.jit(stable_softmax_f16, backend="b200")
    softmax.prepare(x)
    operation = softmax.as_torch_op("b200_reference_door::softmax")
    operation(x)

    def apply(value):
        return operation(value)

    y = torch.compile(apply, fullgraph=True)(x)
    assert relative_error(y, oracle.softmax(x.cpu())) <= 1e-2


def test_forward_backward_example_registers_with_autograd(intent):
    """examples/softmax_forward_backward.py:11-29, its own make_softmax with backend b200."""
    sys.path.insert(0, str(REFERENCE_PYTHON / "examples"))
    try:
        import softmax_forward_backward as example
    finally:
        sys.path.remove(str(REFERENCE_PYTHON / "examples"))
    x = torch.randn((example.ROWS, example.COLUMNS), dtype=torch.float32, device=DEV, requires_grad=True)
    upstream = torch.randn_like(x)
    operation, _, kernels = example.make_softmax("b200", x, upstream)
    probabilities = operation(x)
    probabilities.backward(upstream)
    reference = x.detach().double().requires_grad_(True)
    torch.softmax(reference, 1).backward(upstream.double())
    assert relative_error(probabilities, torch.softmax(reference, 1)) <= 1e-5
    assert relative_error(x.grad[:256], reference.grad[:256]) <= 1e-4
    for kernel in kernels:
        kernel.close()


def test_prepared_sequence_and_host_buffers_of_the_reference(intent):
    """The reference's PreparedSequence over two b200 calls, fed through its HostBuffers
    transfer scope (host arrays in, host result out)."""
    from intent.examples.kernels.normalization.layer_norm import layer_norm_f16
    from intent.examples.kernels.normalization.softmax import stable_softmax_f16
    from intent.runtime.host_buffers import HostBuffers
    from intent.runtime.sequence import PreparedSequence
    x, w, b, inv, eps = workloads.layer_norm_inputs(64, 1024, seed=16)
    buffers = HostBuffers("b200", DEV)
    buffers.begin()
    import numpy
    # NumPy arrays are what the scope stages (it passes torch tensors through as native storage)
    staged = [buffers.input(numpy.array(t.numpy()), element="f16") for t in (x, w, b)]
    assert all(t.device.type == "cuda" for t in staged)
    norm = intent.jit(layer_norm_f16, backend="b200")
    soft = intent.jit(stable_softmax_f16, backend="b200")
    first = norm.prepare(*staged, inv, eps)
    second = soft.prepare(first.result())
    sequence = PreparedSequence((first, second), outputs=second.result(), owners=(buffers,))
    sequence.compile()
    assert sequence.kernel_count == 2
    sequence.launch()
    buffers.finish()
    expected = oracle.softmax(oracle.layer_norm(x, w, b, inv, eps))
    assert relative_error(sequence.result(), expected) <= 1e-2
    assert len(sequence.observations) == 2
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    sequence.enqueue(stream)
    stream.synchronize()
    assert relative_error(sequence.result(), expected) <= 1e-2
    buffers.close()


@pytest.mark.parametrize("program", ["softmax", "layer_norm", "gemm", "attention", "csr_spmv"])
@pytest.mark.parametrize("prepared", [False, True])
def test_example_runner_of_the_reference(program, prepared, tmp_path):
    """python -m intent.examples <program> --backend b200 (python/intent/examples/__main__.py):
    the registered author programs with the registry's own inputs, through ExampleContext."""
    script = ("import sys, intent_b200; intent_b200.register(); "
              "from intent.examples.__main__ import main; "
              f"sys.argv = ['intent.examples', {program!r}, '--backend', 'b200'"
              + (", '--prepared'" if prepared else "") + "]; main()")
    environment = dict(os.environ, PYTHONPATH=f"{ROOT}{os.pathsep}{REFERENCE_PYTHON}",
                       INTENT_CACHE_DIR=str(tmp_path))
    environment.pop("INTENT_COMPILER", None)
    completed = subprocess.run([sys.executable, "-c", script], env=environment, capture_output=True, text=True,
                               timeout=300)
    assert completed.returncode == 0, completed.stderr[-2000:]
    assert "result" in completed.stdout and "shape=" in completed.stdout
