"""The public API on a device: jit(...).run(), artifact(...) with explicit outputs,
prepared calls and artifact.as_torch_op(), all through b200-compile + the C ABI."""
import pytest
import torch

import intent_b200 as b200
import oracle
from conftest import relative_error
from intent_b200 import workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_native_library_is_the_one_in_tree():
    from intent_b200 import _native
    assert _native.LIBRARY_PATH.exists()
    _native.library()
    assert any("libintent_b200.so" in line for line in open("/proc/self/maps"))


def test_jit_run_and_explicit_outputs_softmax():
    (x,) = workloads.softmax_inputs(256, 1024, seed=1)
    kernel = b200.jit(b200.kernels.stable_softmax)
    y = kernel.run(x.to(DEV))
    expected = oracle.softmax(x)
    assert relative_error(y, expected) <= 1e-5
    out = torch.empty_like(y)
    kernel(x.to(DEV), out)                                   # JITKernel.__call__: explicit Out buffer
    assert torch.equal(out, y)
    artifact = kernel.artifacts[0]
    out.zero_()
    artifact(x.to(DEV), out)                                 # CompiledArtifact.__call__ == launch
    assert torch.equal(out, y)
    assert kernel.interface.outputs[0].name == "y"
    assert artifact.observation.stage == "launched" and artifact.observation.family == "softmax"


def test_prepared_call_replays_without_rebinding():
    x, w, b, inv, eps = workloads.layer_norm_inputs(64, 4096, seed=2)
    kernel = b200.jit(b200.kernels.layer_norm_f16)
    xd = x.to(DEV)
    call = kernel.prepare(xd, w.to(DEV), b.to(DEV), inv, eps)
    call.compile()
    call.launch()
    first = call.result().clone()
    xd.mul_(2)
    call.launch()                                            # same bound buffers, new contents
    assert relative_error(first, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2
    assert relative_error(call.result(), oracle.layer_norm(x * 2, w, b, inv, eps)) <= 1e-2


def test_author_noalias_and_native_requirements():
    kernel = b200.jit(b200.kernels.stable_softmax)
    x = torch.randn(8, 64, device=DEV)
    with pytest.raises(ValueError, match="noalias"):
        kernel(x, x)
    kernel_ln = b200.jit(b200.kernels.layer_norm_f16)
    xh = torch.randn(4, 64, device=DEV).half()
    w = torch.ones(64, device=DEV).half()
    with pytest.raises(NotImplementedError, match="nonoverlapping"):
        kernel_ln(xh, w, w, xh, 1 / 64, 1e-5)
    with pytest.raises(ValueError, match="executes on cuda"):
        b200.jit(b200.kernels.stable_softmax, device=0).prepare(torch.randn(2, 2))


def test_gemm_and_attention_and_spmm_through_jit():
    a, bmat = workloads.gemm_inputs(256, 512, 256, seed=3)
    kernel = b200.jit(b200.kernels.gemm, constexprs={"ACTIVATION": "RELU"})
    call = kernel.prepare(a.to(DEV), bmat.to(DEV))
    call.launch()
    call.check()
    assert relative_error(call.result(), oracle.gemm(a, bmat, relu=True)) <= 1e-2
    q, k, v, scale = workloads.attention_inputs(1, 4, 256, 128, seed=4, kv_heads=2)
    attention = b200.jit(b200.kernels.flash_attention_bf16_fwd, constexprs={"HEAD_GROUP": 2, "CAUSAL": True})
    out = attention.run(q.to(DEV), k.to(DEV), v.to(DEV), scale)
    assert relative_error(out, oracle.attention(q, k, v, scale, head_group=2)) <= 1e-2
    ro, ci, va, x = workloads.csr_inputs(8192, 8192, 32, 128, seed=5)
    spmm = b200.jit(b200.kernels.csr_spmm)
    y = spmm.run(ro.to(DEV), ci.to(DEV), va.to(DEV), x.to(DEV))
    assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci, va, x))


def test_as_torch_op_eager_and_compiled():
    (x,) = workloads.softmax_inputs(128, 512, seed=6)
    kernel = b200.jit(b200.kernels.stable_softmax)
    kernel.prepare(x.to(DEV))
    op = kernel.as_torch_op("b200_test::softmax_gpu")
    y = op(x.to(DEV))
    assert relative_error(y, oracle.softmax(x)) <= 1e-5

    @torch.compile(fullgraph=True)
    def twice(t):
        return op(t) * 2

    assert relative_error(twice(x.to(DEV)), oracle.softmax(x) * 2) <= 1e-5


def test_backward_pair_registers_with_autograd():
    """The reference's own recipe (examples/softmax_forward_backward.py:11-29): forward and
    backward artifacts become torch operators and the backward is registered for autograd."""
    forward = b200.jit(b200.kernels.stable_softmax)
    backward = b200.jit(b200.kernels.softmax_backward)
    x = torch.randn(4096, 4097, device=DEV)
    forward.prepare(x)
    backward.prepare(x, x)
    forward_op = forward.as_torch_op("b200_test::softmax_fwd")
    backward_op = backward.as_torch_op("b200_test::softmax_bwd")

    def setup_context(ctx, inputs, output):
        ctx.save_for_backward(output)

    def backward_rule(ctx, upstream):
        (probabilities,) = ctx.saved_tensors
        return backward_op(probabilities, upstream.contiguous())

    forward_op.register_autograd(backward_rule, setup_context=setup_context)
    leaf = x[:64].clone().requires_grad_(True)
    reference = leaf.detach().double().requires_grad_(True)
    weights = torch.randn(64, 4097, device=DEV)
    # the static kernel shape is 4096 x 4097, so run the full matrix and compare a slice
    full = x.clone().requires_grad_(True)
    (forward_op(full) * torch.nn.functional.pad(weights, (0, 0, 0, 4032))).sum().backward()
    (torch.softmax(reference, 1) * weights.double()).sum().backward()
    assert relative_error(full.grad[:64], reference.grad) <= 1e-4


def test_layer_norm_backward_pair_through_the_artifact_api():
    """The InOut partial sums are supplied by the caller and updated in place; dx, dw, db are
    allocated by the runtime (kernels/backward/layer_norm.py:12-90)."""
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(256, 1024, 128, seed=5)
    device = [t.to(DEV) for t in (x, dy, w, mean, rstd, dw_partial, db_partial)]
    rows = b200.jit(b200.kernels.layer_norm_backward_rows).prepare(*device, inv)
    reduce = b200.jit(b200.kernels.layer_norm_backward_reduce).prepare(device[5], device[6])
    sequence = b200.PreparedSequence([rows, reduce], outputs=(rows.result(), *reduce.result()))
    sequence.compile()
    sequence.launch()
    torch.cuda.synchronize()
    dx, dw, db = sequence.result()
    expected_dx = oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, inv)
    expected_dw, expected_db = oracle.layer_norm_backward_reduce(dw_partial, db_partial)
    assert relative_error(dx, expected_dx) <= 1e-2
    assert torch.equal(device[5].cpu(), dw_partial) and torch.equal(device[6].cpu(), db_partial)
    assert torch.equal(dw.cpu(), expected_dw) and torch.equal(db.cpu(), expected_db)


def test_attention_backward_program():
    """The reference's three-kernel recipe (examples/programs/attention_backward.py:19-41): delta,
    dK/dV and dQ bound once, run as one prepared sequence that yields dQ, dK, dV."""
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(2, 8, 2, 512, 64, seed=13)
    options = {"HEAD_GROUP": 4, "CAUSAL": True}
    delta_kernel = b200.jit(b200.kernels.attention_backward_delta)
    dkdv_kernel = b200.jit(b200.kernels.attention_backward_dkdv, constexprs=options)
    dq_kernel = b200.jit(b200.kernels.attention_backward_dq, constexprs=options)
    device = [t.to(DEV) for t in (q, k, v, output, grad_output, lse)]
    delta = delta_kernel.prepare(device[3], device[4])
    common = (device[0], device[1], device[2], device[4], device[5], delta.result(), scale)
    dkdv = dkdv_kernel.prepare(*common)
    dq = dq_kernel.prepare(*common)
    sequence = b200.PreparedSequence((delta, dkdv, dq), outputs=(dq.result(), *dkdv.result()))
    sequence.compile()
    sequence.launch()
    torch.cuda.synchronize()
    dkdv.check()
    dq.check()
    grad_q, grad_k, grad_v = sequence.result()
    expected_delta = oracle.attention_backward_delta(output, grad_output)
    expected_k, expected_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, expected_delta, scale, head_group=4)
    expected_q = oracle.attention_backward_dq(q, k, v, grad_output, lse, expected_delta, scale, head_group=4)
    assert relative_error(grad_q, expected_q) <= 1e-2
    assert relative_error(grad_k, expected_k) <= 1e-2
    assert relative_error(grad_v, expected_v) <= 1e-2
    assert sequence.kernel_count == 3


def test_prepared_sequence_and_explicit_stream():
    (x,) = workloads.softmax_inputs(4096, 4097, seed=8)
    xd = x.to(DEV)
    forward = b200.jit(b200.kernels.stable_softmax).prepare(xd)
    upstream = torch.randn(4096, 4097, device=DEV)
    backward = b200.jit(b200.kernels.softmax_backward).prepare(forward.result(), upstream)
    sequence = b200.PreparedSequence([forward, backward], outputs=backward.result())
    sequence.compile()
    assert sequence.kernel_count == 2 and not sequence.observations[0].stage == "launched"
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    sequence.enqueue(side)                                   # caller-owned queue
    side.synchronize()
    expected = oracle.softmax_backward(oracle.softmax(x[:32]), upstream[:32].cpu())
    assert relative_error(sequence.result()[:32], expected) <= 1e-4
    assert [o.stage for o in sequence.observations] == ["launched", "launched"]


def test_doctor_resolves_the_device():
    from intent_b200 import tools
    report = tools.doctor(0)
    assert report["status"] == "available", report
    target = report["checks"][-1]
    assert target["name"] == "target" and target["detail"]["capabilities"]["compute_capability_major"] == 10


def test_host_buffers_stage_inputs_and_bring_results_back():
    """The stand-alone transfer scope: host arrays in (NumPy or CPU tensors, page-locked in
    place), the bound device views keep shape and strides, results land in page-locked host
    memory at finish(); a region narrows the transfers to a block of rows."""
    import numpy
    x, w, b, inv, eps = workloads.layer_norm_inputs(64, 1024, seed=31)
    kernel = b200.jit(b200.kernels.layer_norm_f16)
    with b200.HostBuffers(DEV) as scope:
        staged = (scope.input(x.numpy()), scope.input(w), scope.input(b200.HostBuffers.page_locked(b)))
        assert all(t.device.type == "cuda" and t.shape == h.shape for t, h in zip(staged, (x, w, b)))
        call = kernel.prepare(*staged, inv, eps)
        host_result = scope.result(call.result())
        stream = torch.cuda.Stream()
        scope.stage_in(stream)
        call.enqueue(stream)
        scope.finish(stream)
        assert host_result.is_pinned() and scope.bytes_in == x.numel() * 2 + 2 * 1024 * 2
        assert relative_error(host_result, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2
        # the same call again after the host array changed: stage_in copies the new contents
        x.mul_(2)
        scope.stage_in(stream)
        call.enqueue(stream)
        scope.finish(stream)
        assert relative_error(host_result, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2
    # a transposed host view shares its allocation's device twin and keeps its strides
    a, bm = workloads.gemm_inputs(256, 384, 128, seed=32)
    with b200.HostBuffers(DEV) as scope:
        ad, bd = scope.input(a), scope.input(bm)
        assert bd.stride() == bm.stride() and bd.shape == bm.shape
        call = b200.jit(b200.kernels.gemm, constexprs={"ACTIVATION": "NONE"}).prepare(ad, bd)
        out = scope.result(call.result(), region=lambda t: t[64:128])
        out.zero_()
        scope.stage_in()
        call.launch()
        scope.finish()
        expected = oracle.gemm(a, bm)
        assert relative_error(out[64:128], expected[64:128]) <= 1e-2 and not out[:64].any() and not out[128:].any()
        assert scope.bytes_out == 64 * 384 * 2
    with pytest.raises(TypeError):
        b200.HostBuffers(DEV).input([1.0, 2.0])
    with pytest.raises(ValueError):
        b200.HostBuffers("cpu")
