"""Binder behaviour that needs no device: abstract binding and the error contract
(python/intent/runtime/torch_views.py:32-43, runtime/invocation.py:42-53)."""
import pytest
import torch

import intent_b200 as b200
from intent_b200.runtime import B200Program


def program(definition, **constexprs):
    return B200Program(b200.generate(definition, constexprs=constexprs or None).metadata, 0)


def test_infer_outputs_on_meta_tensors():
    softmax = program(b200.kernels.stable_softmax)
    out = softmax.infer_outputs((torch.empty(7, 33, device="meta"),))
    assert out.shape == (7, 33) and out.dtype == torch.float32
    gemm = program(b200.kernels.gemm, ACTIVATION="NONE")
    out = gemm.infer_outputs((torch.empty(5, 16, dtype=torch.float16, device="meta"),
                              torch.empty(16, 9, dtype=torch.float16, device="meta")))
    assert out.shape == (5, 9)
    attention = program(b200.kernels.flash_attention_bf16_fwd, HEAD_GROUP=2, CAUSAL=True)
    q = torch.empty(2, 4, 64, 128, dtype=torch.bfloat16, device="meta")
    kv = torch.empty(2, 2, 96, 128, dtype=torch.bfloat16, device="meta")
    assert attention.infer_outputs((q, kv, kv, 0.1)).shape == (2, 4, 64, 128)


def test_binder_errors_match_the_reference_contract():
    softmax = program(b200.kernels.stable_softmax)
    with pytest.raises(TypeError, match="expected 1 runtime arguments"):
        softmax.infer_outputs(())
    with pytest.raises(TypeError, match="must be a torch.Tensor"):
        softmax.infer_outputs(([1.0, 2.0],))
    with pytest.raises(TypeError, match="must have dtype"):
        softmax.infer_outputs((torch.empty(2, 2, dtype=torch.float16, device="meta"),))
    with pytest.raises(ValueError, match="must have rank 2"):
        softmax.infer_outputs((torch.empty(2, device="meta"),))
    with pytest.raises(RuntimeError, match="strides"):      # author constraint strides=(None, 1)
        softmax.infer_outputs((torch.empty(4, 4, device="meta").t(),))
    gemm = program(b200.kernels.gemm, ACTIVATION="NONE")
    with pytest.raises(RuntimeError, match="shape"):        # K mismatch between a and b
        gemm.infer_outputs((torch.empty(5, 16, dtype=torch.float16, device="meta"),
                            torch.empty(17, 9, dtype=torch.float16, device="meta")))


def test_concrete_binding_rejects_the_wrong_device():
    softmax = program(b200.kernels.stable_softmax)
    with pytest.raises(ValueError, match="must be on cuda:0"):
        softmax.prepare((torch.empty(2, 2),))


def test_static_shapes_are_enforced():
    spmm = program(b200.kernels.csr_spmm)
    good = (torch.empty(8193, dtype=torch.int32, device="meta"), torch.empty(262144, dtype=torch.int32, device="meta"),
            torch.empty(262144, device="meta"), torch.empty(8192, 128, device="meta"))
    assert spmm.infer_outputs(good).shape == (8192, 128)
    bad = (torch.empty(100, dtype=torch.int32, device="meta"),) + good[1:]
    with pytest.raises(RuntimeError, match="shape"):
        spmm.infer_outputs(bad)


def test_definitions_cannot_be_called_directly():
    with pytest.raises(TypeError):
        b200.kernels.stable_softmax(torch.empty(1, 1))
    with pytest.raises(TypeError, match="requires constexprs"):
        b200.generate(b200.kernels.gemm)
    with pytest.raises(ValueError, match="Unknown backend"):
        b200.jit(b200.kernels.stable_softmax, backend="triton")


def test_torch_op_schema_and_fake_kernel():
    artifact = b200.Artifact("source", "mlir", 0, program(b200.kernels.layer_norm_f16))
    op = artifact.as_torch_op("b200_test::layer_norm_cpu_schema")
    assert str(op._opoverload._schema).endswith(
        "(Tensor arg0, Tensor arg1, Tensor arg2, float arg3, float arg4) -> Tensor")
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(6, 32, dtype=torch.float16)
        w = torch.empty(32, dtype=torch.float16)
        out = op(x, w, w, 1 / 32, 1e-5)
        assert out.shape == (6, 32) and out.dtype == torch.float16


def test_describe_and_doctor_views():
    """The b200 views of the reference's `describe` and `doctor` tools
    (python/intent/tools/compilation.py:125-153, 343-455): dictionaries, nothing compiled or run."""
    from intent_b200 import tools
    described = tools.describe()
    assert described["status"] == "described" and described["tool_invoked_kernel"] is False
    assert "b200_flash_attention" in described["entries"] and "attention_backward_dq" in described["kernels"]
    assert described["backends"]["b200"]["local_device"] == {"kind": "cuda", "indexed": True}
    report = tools.doctor(None)                       # compiler and library only: no device here
    assert report["status"] == "available" and report["tool_invoked_kernel"] is False
    assert [item["name"] for item in report["checks"]] == ["b200 compile step", "native library", "torch"]
    missing = tools.doctor(None, compiler="/nonexistent/b200-compile")
    assert missing["status"] == "unavailable" and missing["checks"][0]["status"] == "unavailable"
    assert tools.main(["describe"]) == 0


def test_direct_operator_calls_validate_before_the_foreign_call(monkeypatch):
    """`intent_b200.ops` checks element types and extents itself: the kernels trust them, so a
    wrong index type or a short output buffer must raise here and never reach the library."""
    from intent_b200 import ops

    def launched(*_):
        raise AssertionError("the foreign call was reached")
    monkeypatch.setattr(ops, "_call", launched)
    monkeypatch.setattr(ops, "_require_cuda", lambda *tensors: tensors[0].device)
    x = torch.zeros(4, 8)
    with pytest.raises(TypeError, match="out must have dtype"):
        ops.softmax(x, out=torch.zeros(4, 8, dtype=torch.float16))
    with pytest.raises(ValueError, match="out must have shape"):
        ops.softmax(x, out=torch.zeros(4, 4))
    with pytest.raises(TypeError, match="weight must have dtype"):
        ops.layer_norm(x.half(), torch.ones(8), torch.ones(8).half(), 1 / 8, 1e-5)
    with pytest.raises(TypeError, match="b must have dtype"):
        ops.gemm(torch.zeros(4, 8, dtype=torch.float16), torch.zeros(8, 4, dtype=torch.bfloat16))
    with pytest.raises(TypeError, match="a must be one of"):
        ops.gemm(torch.zeros(4, 8), torch.zeros(8, 4))
    offsets, columns, values = torch.tensor([0, 1, 2]), torch.tensor([0, 1]), torch.ones(2)
    with pytest.raises(TypeError, match="row_offsets must have dtype torch.int32"):
        ops.csr_spmm(offsets, columns.int(), values, torch.zeros(2, 4))       # torch's default int64
    with pytest.raises(TypeError, match="column_indices must have dtype torch.int32"):
        ops.csr_spmv(offsets.int(), columns, values, torch.zeros(2))
    with pytest.raises(ValueError, match="out must have shape"):
        ops.csr_spmm(offsets.int(), columns.int(), values, torch.zeros(2, 4), out=torch.zeros(3, 4))
    q = torch.zeros(1, 2, 8, 64, dtype=torch.bfloat16)
    with pytest.raises(TypeError, match="k must have dtype"):
        ops.flash_attention(q, q.half(), q, 0.1)
    with pytest.raises(ValueError, match="out must have shape"):
        ops.flash_attention(q, q, q, 0.1, out=torch.zeros(1, 2, 8, 32, dtype=torch.bfloat16))
