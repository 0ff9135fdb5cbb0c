"""The CPU oracle against float64 restatements of the same kernel definitions and
against the committed vectors (tests/golden/oracle_vectors.pt).  The reference
holds no golden vectors for these operators; parity is unpinned."""
import math
from pathlib import Path

import pytest
import torch

import oracle
from conftest import relative_error
from intent_b200 import workloads

GOLDEN = Path(__file__).resolve().parent / "golden" / "oracle_vectors.pt"


def test_softmax_f32_against_float64():
    (x,) = workloads.softmax_inputs(64, 1024, seed=3)
    assert relative_error(oracle.softmax(x), torch.softmax(x.double(), 1)) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_softmax_16bit(dtype):
    x = torch.randn(9, 257, generator=torch.Generator().manual_seed(1)).to(dtype)
    assert relative_error(oracle.softmax(x), torch.softmax(x.double(), 1)) <= 1e-2


def test_softmax_nan_and_infinities():
    x = torch.tensor([[1.0, float("nan"), 2.0], [float("-inf"), 0.0, 1.0]])
    y = oracle.softmax(x)
    assert torch.isnan(y[0]).all()                     # NaN reaches every output through the sum
    assert y[1, 0] == 0 and abs(float(y[1].sum()) - 1) < 1e-6


def test_layer_norm_against_float64():
    x, w, b, inv, eps = workloads.layer_norm_inputs(32, 4096, seed=5)
    expected = torch.nn.functional.layer_norm(x.double(), (4096,), w.double(), b.double(), eps)
    assert relative_error(oracle.layer_norm(x, w, b, inv, eps), expected) <= 1e-2
    xf = torch.randn(8, 100, generator=torch.Generator().manual_seed(2))
    wf, bf = torch.rand(100) + 0.5, torch.rand(100) - 0.5
    expected = torch.nn.functional.layer_norm(xf.double(), (100,), wf.double(), bf.double(), 1e-5)
    assert relative_error(oracle.layer_norm(xf, wf, bf, 1 / 100, 1e-5), expected) <= 1e-4


def test_gemm_against_float64_and_row_sampling():
    a, b = workloads.gemm_inputs(96, 130, 200, seed=7)
    c = oracle.gemm(a, b)
    assert relative_error(c, a.double() @ b.double()) <= 2e-3
    part = torch.zeros_like(c)
    oracle.gemm(a, b, rows=(32, 16), out=part)
    assert torch.equal(part[32:48], c[32:48]) and not part[:32].any()
    relu = oracle.gemm(a, b, relu=True)
    assert torch.equal(relu, torch.clamp_min(c.float(), 0).half()) or relative_error(relu, c.clamp_min(0)) == 0


def attention_float64(q, k, v, scale, head_group=1, causal=True):
    q, k, v = q.double(), k.double(), v.double()
    k = k.repeat_interleave(head_group, dim=1)
    v = v.repeat_interleave(head_group, dim=1)
    s = q @ k.transpose(-1, -2) * scale
    if causal:
        mask = torch.arange(q.shape[2])[:, None] >= torch.arange(k.shape[2])[None, :]
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, -1).nan_to_num(0.0)
    return p @ v


@pytest.mark.parametrize("chunk", [16, 64, 128, 10_000])
def test_attention_against_float64_for_any_slicing(chunk):
    q, k, v, scale = workloads.attention_inputs(1, 4, 160, 64, seed=11, kv_heads=2)
    out = oracle.attention(q, k, v, scale, head_group=2, chunk=chunk)
    assert relative_error(out, attention_float64(q, k, v, scale, 2)) <= 1e-2


def test_attention_rows_without_a_valid_key_are_zero():
    q, k, v, scale = workloads.attention_inputs(1, 1, 8, 64, seed=1)
    out = oracle.attention(q, k[:, :, :0], v[:, :, :0], scale)
    assert not out.any()
    non_causal = oracle.attention(q, k, v, scale, causal=False)
    assert relative_error(non_causal, attention_float64(q, k, v, scale, causal=False)) <= 1e-2


def test_csr_spmm_is_the_sequential_sum_and_validates():
    ro, ci, va, x = workloads.csr_inputs(200, 300, 17, 24, seed=13)
    y = oracle.csr_spmm(ro, ci, va, x)
    expected = torch.zeros(200, 24)
    for r in range(200):
        acc = torch.zeros(24)
        for nz in range(int(ro[r]), int(ro[r + 1])):
            acc = acc + va[nz] * x[int(ci[nz])]
        expected[r] = acc
    assert torch.equal(y, expected)                       # bit-exact: same order, no fused multiply-add
    oracle.csr_validate(ro, ci, 300)
    broken = ci.clone()
    broken[5] = 300
    with pytest.raises(ValueError):
        oracle.csr_validate(ro, broken, 300)


def test_csr_spmv_and_softmax_backward():
    ro, ci, va, x = workloads.csr_inputs(300, 500, 40, 1, seed=17)
    vector = x[:, 0].contiguous()
    y = oracle.csr_spmv(ro, ci, va, vector)
    assert torch.equal(y, oracle.csr_spmm(ro, ci, va, x)[:, 0])        # a single-feature SpMM
    g = torch.Generator().manual_seed(19)
    probabilities = torch.softmax(torch.randn(33, 4097, generator=g), dim=1)
    upstream = torch.randn(33, 4097, generator=g)
    expected = probabilities.double() * (upstream.double() - (probabilities.double() * upstream.double()).sum(1, keepdim=True))
    assert relative_error(oracle.softmax_backward(probabilities, upstream), expected) <= 1e-5


def test_layer_norm_backward_against_autograd():
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(256, 512, 128, seed=23)
    dx = oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, inv)
    dw, db = oracle.layer_norm_backward_reduce(dw_partial, db_partial)
    xd = x.double().requires_grad_(True)
    wd = w.double().requires_grad_(True)
    bd = torch.zeros(512, dtype=torch.double, requires_grad=True)
    torch.nn.functional.layer_norm(xd, (512,), wd, bd, 1e-5).backward(dy.double())
    assert relative_error(dx, xd.grad) <= 1e-2            # one bf16 rounding of the result
    assert relative_error(dw, wd.grad) <= 2e-2            # two bf16-rounded updates per group
    assert relative_error(db, bd.grad) <= 2e-2
    # the partial sums are InOut: a second call accumulates on top of the first, and the team size
    # does not change the result (the update order is fixed per group)
    again_w, again_b = dw_partial.clone(), db_partial.clone()
    oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, again_w, again_b, inv, workers=3)
    fresh_w, fresh_b = torch.zeros_like(again_w), torch.zeros_like(again_b)
    oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, fresh_w, fresh_b, inv, workers=1)
    assert torch.equal(fresh_w, dw_partial) and torch.equal(fresh_b, db_partial)
    assert not torch.equal(again_w, dw_partial)


def test_attention_backward_against_autograd():
    b, hq, hk, s, d = 1, 4, 2, 96, 64
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(b, hq, hk, s, d, seed=29)
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qd, kd.repeat_interleave(2, dim=1)) * scale
    scores = scores.masked_fill(~torch.ones(s, s, dtype=torch.bool).tril(), float("-inf"))
    torch.einsum("bhqk,bhkd->bhqd", torch.softmax(scores, -1), vd.repeat_interleave(2, dim=1)).backward(grad_output.double())
    delta = oracle.attention_backward_delta(output, grad_output)
    assert relative_error(delta, (output.double() * grad_output.double()).sum(-1)) <= 1e-5
    grad_k, grad_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale, head_group=2)
    grad_q = oracle.attention_backward_dq(q, k, v, grad_output, lse, delta, scale, head_group=2)
    assert relative_error(grad_q, qd.grad) <= 1e-2
    assert relative_error(grad_k, kd.grad) <= 1e-2
    assert relative_error(grad_v, vd.grad) <= 1e-2
    # the team size does not change the result (units are independent)
    again_k, again_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale, head_group=2, workers=3)
    assert torch.equal(again_k, grad_k) and torch.equal(again_v, grad_v)


def test_committed_vectors():
    vectors = torch.load(GOLDEN)
    (x,) = workloads.softmax_inputs(4, 16, seed=100)
    assert torch.equal(oracle.softmax(x), vectors["softmax"])
    x, w, b, inv, eps = workloads.layer_norm_inputs(4, 64, seed=101)
    assert torch.equal(oracle.layer_norm(x, w, b, inv, eps), vectors["layer_norm"])
    a, b = workloads.gemm_inputs(8, 16, 32, seed=102)
    assert torch.equal(oracle.gemm(a, b), vectors["gemm"])
    q, k, v, scale = workloads.attention_inputs(1, 2, 32, 64, seed=103)
    assert torch.equal(oracle.attention(q, k, v, scale, chunk=16), vectors["attention"])
    ro, ci, va, x = workloads.csr_inputs(8, 32, 4, 16, seed=104)
    assert torch.equal(oracle.csr_spmm(ro, ci, va, x), vectors["csr_spmm"])
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(8, 32, 4, seed=105)
    assert torch.equal(oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, inv),
                       vectors["layer_norm_backward_dx"])
    assert torch.equal(dw_partial, vectors["layer_norm_backward_dw_partial"])
    assert torch.equal(db_partial, vectors["layer_norm_backward_db_partial"])
    dw, db = oracle.layer_norm_backward_reduce(dw_partial, db_partial)
    assert torch.equal(dw, vectors["layer_norm_backward_dw"]) and torch.equal(db, vectors["layer_norm_backward_db"])
    p, u = workloads.softmax_backward_inputs(4, 20, seed=106)
    assert torch.equal(oracle.softmax_backward(p, u), vectors["softmax_backward"])
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 2, 1, 24, 64, seed=107)
    delta = oracle.attention_backward_delta(output, grad_output)
    assert torch.equal(delta, vectors["attention_backward_delta"])
    grad_k, grad_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale, head_group=2)
    assert torch.equal(grad_k, vectors["attention_backward_grad_k"]) and torch.equal(grad_v, vectors["attention_backward_grad_v"])
    assert torch.equal(oracle.attention_backward_dq(q, k, v, grad_output, lse, delta, scale, head_group=2),
                       vectors["attention_backward_grad_q"])
