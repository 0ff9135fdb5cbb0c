"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on seeded
inputs at sizes the oracle finishes in seconds.  Tolerances are the stated ones:
fp32 softmax rel <= 1e-5; fp32-accumulated GEMM <= 2e-3 before the narrowing cast
(<= 1e-2 on the f16/bf16 output); 16-bit outputs <= 1e-2; CSR SpMM bit-exact."""
import math

import pytest
import torch

import oracle
from conftest import relative_error
from intent_b200 import ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def cuda(*tensors):
    return [t.to(DEV) if isinstance(t, torch.Tensor) else t for t in tensors]


# ------------------------------------------------------------------ softmax
@pytest.mark.parametrize("m,n", [(4096, 1024), (37, 1000), (5, 7), (1, 1), (3, 4097), (2, 40000), (8, 65536),
                                 (130, 20), (16, 2048)])
def test_softmax_f32(m, n):
    (x,) = workloads.softmax_inputs(m, n, seed=m + n)
    y = ops.softmax(x.to(DEV))
    assert relative_error(y, oracle.softmax(x)) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n", [(64, 1024), (7, 333), (4, 8200)])
def test_softmax_16bit(dtype, m, n):
    x = workloads.softmax_inputs(m, n, seed=1)[0].to(dtype)
    assert relative_error(ops.softmax(x.to(DEV)), oracle.softmax(x)) <= 1e-2


def test_softmax_row_pitch_and_edge_values():
    (x,) = workloads.softmax_inputs(33, 1100, seed=2)
    xd = x.to(DEV)
    view, out = xd[:, 12:1036], torch.zeros(33, 2048, device=DEV)
    ops.softmax(view, out=out[:, 512:1536])                     # free row pitch, offset base
    assert relative_error(out[:, 512:1536], oracle.softmax(x[:, 12:1036].contiguous())) <= 1e-5
    assert not out[:, :512].any() and not out[:, 1536:].any()
    special = torch.tensor([[1.0, float("nan"), 2.0, 0.0], [float("-inf"), 0.0, 1.0, -1.0]])
    y = ops.softmax(special.to(DEV)).cpu()
    assert torch.isnan(y[0]).all() and y[1, 0] == 0
    assert ops.softmax(torch.empty(0, 8, device=DEV)).shape == (0, 8)
    with pytest.raises(NotImplementedError):
        ops.softmax(xd.t())                                        # inner stride != 1
    with pytest.raises(ValueError):
        ops.softmax(xd, out=torch.empty(3, 3, device=DEV))


# --------------------------------------------------------------- layer norm
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n", [(512, 4096), (33, 1000), (7, 8), (3, 50000), (5, 1001), (64, 16384)])
def test_layer_norm_16bit(dtype, m, n):
    x, w, b, inv, eps = workloads.layer_norm_inputs(m, n, seed=n, dtype=dtype)
    y = ops.layer_norm(*cuda(x, w, b), inv, eps)
    assert relative_error(y, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2


@pytest.mark.parametrize("m,n", [(64, 1024), (9, 100), (4, 40000)])
def test_weighted_layer_norm_f32(m, n):
    x, w, b, inv, eps = workloads.layer_norm_inputs(m, n, seed=3, dtype=torch.float32)
    y = ops.layer_norm(*cuda(x, w, b), inv, eps)
    assert relative_error(y, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-4


def test_layer_norm_strided_parameters():
    x, w, b, inv, eps = workloads.layer_norm_inputs(17, 512, seed=4)
    wide_w, wide_b = torch.zeros(512, 2, dtype=w.dtype), torch.zeros(512, 2, dtype=b.dtype)
    wide_w[:, 0], wide_b[:, 0] = w, b
    y = ops.layer_norm(x.to(DEV), wide_w.to(DEV)[:, 0], wide_b.to(DEV)[:, 0], inv, eps)
    assert relative_error(y, oracle.layer_norm(x, w, b, inv, eps)) <= 1e-2


# --------------------------------------------------------------------- gemm
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 128), (100, 200, 72), (1, 8, 8), (300, 520, 1000),
                                   (1024, 1024, 1024), (129, 257, 65 * 8), (640, 128, 4096)])
def test_gemm(dtype, m, n, k):
    a, b = workloads.gemm_inputs(m, n, k, seed=m + k, dtype=dtype)
    c = ops.gemm(*cuda(a, b))
    ops.workspace_status(DEV)
    expected = oracle.gemm(a, b)
    assert relative_error(c, expected) <= 1e-2
    # the f32 accumulators agree to 2e-3 wherever the narrowing cast did not land on a tie
    assert (c.cpu() == expected).float().mean() > 0.98


def test_gemm_relu_empty_k_and_layout_errors():
    a, b = workloads.gemm_inputs(130, 96, 256, seed=9)
    c = ops.gemm(*cuda(a, b), relu=True)
    assert relative_error(c, oracle.gemm(a, b, relu=True)) <= 1e-2 and (c >= 0).all()
    empty = ops.gemm(torch.empty(8, 0, dtype=torch.float16, device=DEV),
                     torch.empty(0, 16, dtype=torch.float16, device=DEV))
    assert empty.shape == (8, 16) and not empty.any()
    with pytest.raises(NotImplementedError):
        ops.gemm(a.to(DEV).t().contiguous().t(), b.to(DEV))        # A must be K-major
    with pytest.raises(ValueError):
        ops.gemm(a.to(DEV), b[:-8].to(DEV))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(128, 192, 256), (300, 520, 1000), (64, 8, 64), (1024, 1024, 512)])
def test_gemm_row_major_b(dtype, m, n, k):
    """b given as a plain contiguous (K, N) tensor, the layout of the reference's own gemm program
    (python/intent/examples/programs/matrix.py:14-18)."""
    a, b = workloads.gemm_inputs(m, n, k, seed=n, dtype=dtype)
    b = b.contiguous()
    c = ops.gemm(a.to(DEV), b.to(DEV))
    ops.workspace_status(DEV)
    assert relative_error(c, oracle.gemm(a, b)) <= 1e-2


def test_gemm_is_linear_in_a():
    a, b = workloads.gemm_inputs(256, 256, 512, seed=5)
    ad, bd = cuda(a, b)
    c1 = ops.gemm(ad, bd).float()
    c2 = ops.gemm((ad * 2).contiguous(), bd).float()               # scaling by 2 is exact in f16
    assert torch.equal(c2, c1 * 2)


# ---------------------------------------------------------------- attention
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,h,s,d", [(1, 2, 256, 128), (2, 3, 300, 128), (1, 1, 128, 128), (1, 2, 1000, 128),
                                     (1, 1, 17, 128), (1, 2, 4096, 128)])
def test_flash_attention_causal(dtype, b, h, s, d):
    q, k, v, scale = workloads.attention_inputs(b, h, s, d, seed=s, dtype=dtype)
    out = ops.flash_attention(*cuda(q, k, v), scale)
    ops.workspace_status(DEV)
    assert relative_error(out, oracle.attention(q, k, v, scale)) <= 1e-2


def test_flash_attention_gqa_noncausal_and_rectangular():
    q, k, v, scale = workloads.attention_inputs(2, 8, 200, 128, seed=21, kv_heads=2)
    out = ops.flash_attention(*cuda(q, k, v), scale, head_group=4)
    assert relative_error(out, oracle.attention(q, k, v, scale, head_group=4)) <= 1e-2
    out = ops.flash_attention(*cuda(q, k, v), scale, head_group=4, causal=False)
    assert relative_error(out, oracle.attention(q, k, v, scale, head_group=4, causal=False)) <= 1e-2
    # more queries than keys: rows past the last key see every key; fewer queries than keys
    short = ops.flash_attention(*cuda(q, k[:, :, :77], v[:, :, :77]), scale, head_group=4)
    assert relative_error(short, oracle.attention(q, k[:, :, :77].contiguous(), v[:, :, :77].contiguous(),
                                                  scale, head_group=4)) <= 1e-2
    few = ops.flash_attention(*cuda(q[:, :, :50], k, v), scale, head_group=4)
    assert relative_error(few, oracle.attention(q[:, :, :50].contiguous(), k, v, scale, head_group=4)) <= 1e-2
    ops.workspace_status(DEV)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_flash_attention_head_dimension_64(dtype):
    """The shape of the reference's registered attention program
    (python/intent/examples/programs/streaming.py:15-21): bf16, GQA 4, causal, D = 64."""
    q, k, v, scale = workloads.attention_inputs(2, 8, 256, 64, seed=3, dtype=dtype, kv_heads=2)
    out = ops.flash_attention(*cuda(q, k, v), scale, head_group=4)
    ops.workspace_status(DEV)
    assert relative_error(out, oracle.attention(q, k, v, scale, head_group=4)) <= 1e-2
    q, k, v, scale = workloads.attention_inputs(1, 2, 700, 64, seed=4, dtype=dtype)
    out = ops.flash_attention(*cuda(q, k, v), scale, causal=False)
    assert relative_error(out, oracle.attention(q, k, v, scale, causal=False)) <= 1e-2


def test_flash_attention_refuses_other_head_dimensions():
    q, k, v, scale = workloads.attention_inputs(1, 2, 64, 32, seed=3)
    with pytest.raises(NotImplementedError, match="head dimensions"):
        ops.flash_attention(*cuda(q, k, v), scale)


def test_flash_attention_strided_heads():
    """(B, S, H, D) storage viewed as (B, H, S, D): only the innermost stride must be 1."""
    q, k, v, scale = workloads.attention_inputs(1, 4, 192, 128, seed=23)
    packed = [t.permute(0, 2, 1, 3).contiguous().to(DEV).permute(0, 2, 1, 3) for t in (q, k, v)]
    out = ops.flash_attention(*packed, scale)
    assert relative_error(out, oracle.attention(q, k, v, scale)) <= 1e-2


# --------------------------------------------------------------------- spmm
@pytest.mark.parametrize("rows,columns,per_row,features", [(1024, 1024, 32, 128), (100, 50, 32, 32), (64, 64, 9, 130),
                                                           (64, 64, 5, 7), (2048, 4096, 32, 256), (1, 1, 1, 1),
                                                           (4096, 300, 33, 128)])
def test_csr_spmm_bit_exact(rows, columns, per_row, features):
    ro, ci, va, x = workloads.csr_inputs(rows, columns, per_row, features, seed=rows)
    y = ops.csr_spmm(*cuda(ro, ci, va, x))
    assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci, va, x))
    ops.csr_validate(ro.to(DEV), ci.to(DEV), columns)


def test_csr_spmm_ragged_rows_and_validation():
    ro = torch.tensor([0, 0, 3, 3, 40, 41, 41], dtype=torch.int32)
    g = torch.Generator().manual_seed(5)
    ci = torch.randint(0, 64, (41,), dtype=torch.int32, generator=g)   # unsorted, repeated columns are legal
    va, x = torch.randn(41, generator=g), torch.randn(64, 128, generator=g)
    y = ops.csr_spmm(*cuda(ro, ci, va, x))
    assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci, va, x))
    assert not y[0].any() and not y[2].any() and not y[5].any()        # empty rows give zeros
    bad = ci.clone()
    bad[5] = 64
    with pytest.raises(ValueError, match="column_indices"):
        ops.csr_validate(ro.to(DEV), bad.to(DEV), 64)
    bad_offsets = ro.clone()
    bad_offsets[3] = 50
    with pytest.raises(ValueError, match="row_offsets"):
        ops.csr_validate(bad_offsets.to(DEV), ci.to(DEV), 64)


# ------------------------------------------------- spmv and softmax backward
@pytest.mark.parametrize("rows,columns,per_row", [(32768, 32768, 32), (1000, 77, 40), (5, 3, 2), (4096, 100000, 7)])
def test_csr_spmv_bit_exact(rows, columns, per_row):
    ro, ci, va, x = workloads.csr_inputs(rows, columns, per_row, 1, seed=rows)
    vector = x[:, 0].contiguous()
    y = ops.csr_spmv(*cuda(ro, ci, va, vector))
    assert torch.equal(y.cpu(), oracle.csr_spmv(ro, ci, va, vector))
    wide = torch.zeros(columns, 3)
    wide[:, 1] = vector                                                # strided x
    assert torch.equal(ops.csr_spmv(*cuda(ro, ci, va), wide.to(DEV)[:, 1]).cpu(), y.cpu())


@pytest.mark.parametrize("rows,longest", [(1003, 100), (7, 3), (130, 33)])
def test_csr_spmv_ragged_rows(rows, longest):
    """Row lengths from 0 to `longest` (empty rows, rows longer than one batch of 32), a row count
    that is not a multiple of the rows a warp takes."""
    g = torch.Generator().manual_seed(rows)
    columns = 500
    lengths = torch.randint(0, longest + 1, (rows,), generator=g)
    lengths[::5] = 0
    ro = torch.zeros(rows + 1, dtype=torch.int32)
    ro[1:] = torch.cumsum(lengths, 0).to(torch.int32)
    nnz = int(ro[-1])
    ci = torch.cat([torch.sort(torch.randperm(columns, generator=g)[:int(n)]).values for n in lengths]
                   + [torch.zeros(0, dtype=torch.int64)]).to(torch.int32)
    va = torch.randn(nnz, generator=g)
    vector = torch.randn(columns, generator=g)
    y = ops.csr_spmv(*cuda(ro, ci, va, vector))
    assert torch.equal(y.cpu(), oracle.csr_spmv(ro, ci, va, vector))


@pytest.mark.parametrize("m,n", [(64, 4097), (7, 5), (130, 1024), (3, 30000)])
def test_softmax_backward(m, n):
    g = torch.Generator().manual_seed(m + n)
    probabilities = torch.softmax(torch.randn(m, n, generator=g), dim=1)
    upstream = torch.randn(m, n, generator=g)
    gradient = ops.softmax_backward(*cuda(probabilities, upstream))
    assert relative_error(gradient, oracle.softmax_backward(probabilities, upstream)) <= 1e-5
    # it is the vector-Jacobian product of the forward kernel
    x = torch.randn(m, n, generator=g, dtype=torch.float64, requires_grad=True)
    y = torch.softmax(x, dim=1)
    (expected,) = torch.autograd.grad(y, x, upstream.double())
    ours = ops.softmax_backward(ops.softmax(x.detach().float().to(DEV)), upstream.to(DEV))
    assert relative_error(ours, expected) <= 1e-4


@pytest.mark.parametrize("m,n,groups", [(256, 512, 128), (130, 4096, 128), (77, 8192, 16), (5, 40, 3), (300, 1000, 128),
                                         (2100, 2048, 300), (1000, 4096, 7), (700, 8192, 40), (3, 64, 8), (40, 128, 600)])
def test_layer_norm_backward(m, n, groups):
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(m, n, groups, seed=m + n)
    # InOut: start from non-zero partial sums
    g = torch.Generator().manual_seed(groups)
    dw_partial = torch.randn(groups, n, generator=g).to(torch.bfloat16)
    db_partial = torch.randn(groups, n, generator=g).to(torch.bfloat16)
    ours_w, ours_b = dw_partial.to(DEV), db_partial.to(DEV)
    dx = ops.layer_norm_backward_rows(*cuda(x, dy, w, mean, rstd), ours_w, ours_b, inv)
    expected_dx = oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, inv)
    assert relative_error(dx, expected_dx) <= 1e-2
    # the partial sums do not depend on the row reductions: same update order, same roundings
    assert torch.equal(ours_w.cpu(), dw_partial) and torch.equal(ours_b.cpu(), db_partial)
    dw, db = ops.layer_norm_backward_reduce(ours_w, ours_b)
    expected_dw, expected_db = oracle.layer_norm_backward_reduce(dw_partial, db_partial)
    assert torch.equal(dw.cpu(), expected_dw) and torch.equal(db.cpu(), expected_db)


def test_layer_norm_backward_layout_errors():
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(8, 36, 4, seed=1)
    with pytest.raises(NotImplementedError):                       # N is not a multiple of 8
        ops.layer_norm_backward_rows(*cuda(x, dy, w, mean, rstd, dw_partial, db_partial), inv)
    x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(8, 64, 4, seed=1)
    with pytest.raises(ValueError):                                # group counts disagree
        ops.layer_norm_backward_rows(*cuda(x, dy, w, mean, rstd, dw_partial, db_partial[:2]), inv)


@pytest.mark.parametrize("b,hq,hk,s,d,causal,dtype", [
    (1, 2, 1, 128, 64, True, torch.float16),
    (1, 4, 2, 256, 64, True, torch.float16),
    (1, 2, 2, 200, 64, False, torch.float16),      # ragged last tile, no mask
    (2, 8, 2, 1024, 64, True, torch.float16),      # the reference kernels' shape
    (1, 2, 1, 300, 128, True, torch.bfloat16),
    (1, 1, 1, 1, 64, True, torch.float16),
])
def test_attention_backward(b, hq, hk, s, d, causal, dtype):
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(b, hq, hk, s, d, seed=s + d,
                                                                                   dtype=dtype, causal=causal)
    group = hq // hk
    delta = ops.attention_backward_delta(*cuda(output, grad_output))
    expected_delta = oracle.attention_backward_delta(output, grad_output)
    assert relative_error(delta, expected_delta) <= 1e-5
    device = cuda(q, k, v, grad_output, lse)
    grad_k, grad_v = ops.attention_backward_dkdv(*device, delta, scale, head_group=group, causal=causal)
    grad_q = ops.attention_backward_dq(*device, delta, scale, head_group=group, causal=causal)
    ops.workspace_status(DEV)
    expected_k, expected_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, expected_delta, scale,
                                                            head_group=group, causal=causal)
    expected_q = oracle.attention_backward_dq(q, k, v, grad_output, lse, expected_delta, scale, head_group=group,
                                              causal=causal)
    assert relative_error(grad_q, expected_q) <= 1e-2
    assert relative_error(grad_k, expected_k) <= 1e-2
    assert relative_error(grad_v, expected_v) <= 1e-2


def test_attention_backward_matches_autograd_of_the_forward_kernel():
    """dQ, dK, dV of the forward kernel's own output: the trio is its vector-Jacobian product."""
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 4, 1, 384, 64, seed=41)
    device = cuda(q, k, v, grad_output, lse)
    ours = ops.flash_attention(*device[:3], scale, head_group=4, causal=True)
    delta = ops.attention_backward_delta(ours, device[3])
    grad_k, grad_v = ops.attention_backward_dkdv(*device, delta, scale, head_group=4)
    grad_q = ops.attention_backward_dq(*device, delta, scale, head_group=4)
    qd, kd, vd = (t.double().requires_grad_(True) for t in (q, k, v))
    scores = torch.einsum("bhqd,bhkd->bhqk", qd, kd.repeat_interleave(4, dim=1)) * scale
    scores = scores.masked_fill(~torch.ones(384, 384, dtype=torch.bool).tril(), float("-inf"))
    torch.einsum("bhqk,bhkd->bhqd", torch.softmax(scores, -1), vd.repeat_interleave(4, dim=1)).backward(grad_output.double())
    assert relative_error(grad_q, qd.grad) <= 1e-2
    assert relative_error(grad_k, kd.grad) <= 1e-2
    assert relative_error(grad_v, vd.grad) <= 1e-2


def test_attention_backward_argument_errors():
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 2, 1, 64, 32, seed=2)
    delta = ops.attention_backward_delta(*cuda(output, grad_output))          # any head dimension
    with pytest.raises(NotImplementedError):                                   # gradients: head dim 64 or 128
        ops.attention_backward_dq(*cuda(q, k, v, grad_output, lse), delta, scale, head_group=2)
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 2, 1, 64, 64, seed=2)
    with pytest.raises(ValueError):                                            # HQ != HK * head_group
        ops.attention_backward_dkdv(*cuda(q, k, v, grad_output, lse), delta, scale, head_group=1)


def test_backward_kernels_accept_empty_operands():
    """Zero-sized operands are not errors anywhere in the reference's binders; nothing is launched."""
    empty = torch.empty((0, 64), dtype=torch.bfloat16, device=DEV)
    partial = torch.ones((4, 64), dtype=torch.bfloat16, device=DEV)
    stats = torch.empty((0,), device=DEV)
    dx = ops.layer_norm_backward_rows(empty, empty, torch.ones(64, dtype=torch.bfloat16, device=DEV), stats, stats,
                                      partial, partial.clone(), 1.0 / 64)
    assert dx.shape == (0, 64) and torch.equal(partial, torch.ones_like(partial))
    none = torch.empty((0, 8), dtype=torch.bfloat16, device=DEV)
    dw, db = ops.layer_norm_backward_reduce(none, none)
    assert torch.equal(dw, torch.zeros(8, device=DEV)) and torch.equal(db, torch.zeros(8, device=DEV))
    q = torch.empty((0, 2, 16, 64), dtype=torch.float16, device=DEV)
    k = torch.empty((0, 1, 16, 64), dtype=torch.float16, device=DEV)
    rows = torch.empty((0, 2, 16), device=DEV)
    assert ops.attention_backward_delta(q, q).shape == (0, 2, 16)
    assert ops.attention_backward_dq(q, k, k, q, rows, rows, 0.125, head_group=2).shape == q.shape
    grad_k, grad_v = ops.attention_backward_dkdv(q, k, k, q, rows, rows, 0.125, head_group=2)
    assert grad_k.shape == k.shape and grad_v.shape == k.shape
    assert ops.softmax_backward(torch.empty((0, 5), device=DEV), torch.empty((0, 5), device=DEV)).shape == (0, 5)
    # keys but no query: the key/value gradients are zero
    q = torch.empty((1, 2, 0, 64), dtype=torch.float16, device=DEV)
    k = torch.randn((1, 1, 40, 64), device=DEV).half()
    rows = torch.empty((1, 2, 0), device=DEV)
    grad_k, grad_v = ops.attention_backward_dkdv(q, k, k, q, rows, rows, 0.125, head_group=2)
    assert not grad_k.any() and not grad_v.any()


def test_attention_backward_keys_shorter_than_queries():
    """Causal tiles past the last key are skipped; query tiles past the last query write zeros."""
    q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 2, 1, 300, 64, seed=9, keys=140)
    delta = ops.attention_backward_delta(*cuda(output, grad_output))
    device = cuda(q, k, v, grad_output, lse)
    grad_k, grad_v = ops.attention_backward_dkdv(*device, delta, scale, head_group=2)
    grad_q = ops.attention_backward_dq(*device, delta, scale, head_group=2)
    expected_delta = oracle.attention_backward_delta(output, grad_output)
    expected_k, expected_v = oracle.attention_backward_dkdv(q, k, v, grad_output, lse, expected_delta, scale, head_group=2)
    expected_q = oracle.attention_backward_dq(q, k, v, grad_output, lse, expected_delta, scale, head_group=2)
    assert relative_error(grad_q, expected_q) <= 1e-2
    assert relative_error(grad_k, expected_k) <= 1e-2
    assert relative_error(grad_v, expected_v) <= 1e-2


def _shuffled_rows(ci, va, rows, per_row, seed):
    g = torch.Generator().manual_seed(seed)
    order = torch.argsort(torch.rand(rows, per_row, generator=g), dim=1)
    return (torch.gather(ci.view(rows, per_row), 1, order).reshape(-1).contiguous(),
            torch.gather(va.view(rows, per_row), 1, order).reshape(-1).contiguous())


@pytest.mark.parametrize("phases", ["1", "2", "5"])
def test_csr_spmm_column_blocks_keep_storage_order(monkeypatch, phases):
    """Large X is processed in column blocks (several launches accumulating into Y); the block
    count is forced here (the entry reads the override at every call) so that small matrices
    take that path too.  Ascending rows and rows in shuffled storage order must both equal the
    sequential left-to-right sum bit for bit."""
    monkeypatch.setenv("INTENT_B200_SPMM_PHASES", phases)
    ro, ci, va, x = workloads.csr_inputs(3000, 5000, 40, 128, seed=7)          # rows span two batches of 32
    d = cuda(ro, ci, va, x)
    assert torch.equal(ops.csr_spmm(*d).cpu(), oracle.csr_spmm(ro, ci, va, x)), "ascending rows"
    ci2, va2 = _shuffled_rows(ci, va, 3000, 40, 3)
    y = ops.csr_spmm(d[0], ci2.to(DEV), va2.to(DEV), d[3])
    assert torch.equal(y.cpu(), oracle.csr_spmm(ro, ci2, va2, x)), "shuffled rows keep storage order"


def test_csr_spmm_calls_on_two_streams_do_not_share_state(monkeypatch):
    """A call keeps its "rows ascend" word in its own workspace.  An
    ascending and a shuffled matrix run concurrently on two streams, in column blocks, many
    times over: neither may see the other's flag, so both stay bit-exact."""
    monkeypatch.setenv("INTENT_B200_SPMM_PHASES", "4")
    rows, per_row = 6000, 48
    ro, ci, va, x = workloads.csr_inputs(rows, 9000, per_row, 128, seed=31)
    ci2, va2 = _shuffled_rows(ci, va, rows, per_row, 5)
    expected_sorted, expected_shuffled = oracle.csr_spmm(ro, ci, va, x), oracle.csr_spmm(ro, ci2, va2, x)
    d = cuda(ro, ci, va, x)
    ci2d, va2d = ci2.to(DEV), va2.to(DEV)
    states = [torch.zeros(64, dtype=torch.int32, device=DEV) for _ in range(2)]
    outs = [torch.empty(rows, 128, device=DEV) for _ in range(2)]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    torch.cuda.synchronize()
    for iteration in range(40):
        with torch.cuda.stream(streams[0]):
            ops.csr_spmm(*d, out=outs[0], state=states[0])
        with torch.cuda.stream(streams[1]):
            ops.csr_spmm(d[0], ci2d, va2d, d[3], out=outs[1], state=states[1])
        if iteration % 8 == 7:
            torch.cuda.synchronize()
            assert torch.equal(outs[0].cpu(), expected_sorted), f"ascending matrix, iteration {iteration}"
            assert torch.equal(outs[1].cpu(), expected_shuffled), f"shuffled matrix, iteration {iteration}"
            outs[0].zero_()
            outs[1].zero_()
    assert int(states[0][2]) == 1 and int(states[1][2]) == 0      # word 2: "every row ascends"


def test_a_bounded_wait_that_runs_out_is_reported_and_the_workspace_recovers():
    """Failure detection without a fault: a wait on a barrier that nothing arrives on gives up
    after a short limit, the kernel returns, the host reads B200_ERR_DEVICE_TIMEOUT with the site
    of the wait, and after clearing the words the same workspace serves an ordinary call."""
    import ctypes
    from intent_b200 import _native
    space = torch.zeros(64, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream(DEV).cuda_stream
    with torch.cuda.device(DEV):
        status = _native.entry("b200_selftest_bounded_wait")(space.data_ptr(), 64, 1, 2_000_000, stream)
        assert status == _native.OK
        detail = ctypes.c_int32(0)
        status = _native.entry("b200_workspace_status")(space.data_ptr(), ctypes.byref(detail), stream)
    assert status == _native.ERR_DEVICE_TIMEOUT and detail.value == 9          # site of the self-test wait
    with pytest.raises(_native.NativeCallError, match="bounded device-side wait gave up"):
        _native.check("b200_workspace_status", status)
    words = space.cpu()
    assert words[0] == 1 and words[8] == 0 and words[9] == 1     # did not arrive; the other warp saw the abort flag
    space.zero_()
    a, b = workloads.gemm_inputs(256, 256, 128, seed=77)
    c = torch.empty(256, 256, dtype=torch.float16, device=DEV)
    bd = b.t().contiguous().to(DEV).t()
    ad = a.to(DEV)
    with torch.cuda.device(DEV):
        status = _native.entry("b200_gemm")(ad.data_ptr(), *ad.shape, *ad.stride(), bd.data_ptr(), *bd.shape, *bd.stride(),
                                            c.data_ptr(), *c.shape, *c.stride(), space.data_ptr(), 64, 1, 1, 0, stream)
        assert status == _native.OK
        assert _native.entry("b200_workspace_status")(space.data_ptr(), ctypes.byref(detail), stream) == _native.OK
    assert relative_error(c, oracle.gemm(a, b)) <= 1e-2
    with pytest.raises(ValueError):
        _native.check("b200_selftest_bounded_wait",
                      _native.entry("b200_selftest_bounded_wait")(space.data_ptr(), 64, 1, 10, stream))   # limit too small


CHECKED_SCRIPT = """
import sys, torch
sys.path.insert(0, %r)
import oracle
from intent_b200 import _native, ops, workloads
assert _native.LIBRARY_PATH.name == "libintent_b200_checked.so"
ro, ci, va, x = workloads.csr_inputs(4096, 4096, 32, 128, seed=9)
d = [t.to("cuda:0") for t in (ro, ci, va, x)]
assert torch.equal(ops.csr_spmm(*d).cpu(), oracle.csr_spmm(ro, ci, va, x)), "the checked build computes the same product"
ops.workspace_status("cuda:0")
bad = ci.clone()
bad[32 * 1000 + 5] = 4096            # one column past the last row of X, in row 1000
y = ops.csr_spmm(d[0], bad.to("cuda:0"), d[2], d[3])
try:
    ops.workspace_status("cuda:0")
    print("not reported")
except ValueError as error:
    assert "row 1000" in str(error), str(error)
    print("reported")
expected = oracle.csr_spmm(ro, ci, va, x)
assert torch.equal(y.cpu()[:1000], expected[:1000]) and torch.equal(y.cpu()[1001:], expected[1001:])
"""


def test_checked_build_reports_an_out_of_range_column_instead_of_loading_it():
    """The -DB200_CHECKED variant of the library (INTENT_B200_CHECKED=1): an index outside X is
    recorded in the workspace with its row and the term is skipped, so nothing is read out of
    bounds; every other row is unaffected."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = str(Path(__file__).resolve().parents[1])
    done = subprocess.run([sys.executable, "-c", CHECKED_SCRIPT % root], env=dict(os.environ, INTENT_B200_CHECKED="1"),
                          capture_output=True, text=True)
    assert done.returncode == 0 and "reported" in done.stdout and "not reported" not in done.stdout, done.stderr[-2000:]
