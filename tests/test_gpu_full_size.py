"""The benchmark configurations at full size, checked through size-independent
properties plus a bounded sample against the CPU oracle."""
import pytest
import torch

import oracle
from conftest import relative_error
from intent_b200 import ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_softmax_4096x1024():
    (x,) = workloads.softmax_inputs()
    xd = x.to(DEV)
    y = ops.softmax(xd)
    assert relative_error(y, oracle.softmax(x)) <= 1e-5
    sums = y.double().sum(dim=1)
    assert (sums - 1).abs().max() < 1e-5                              # rows are distributions
    assert relative_error(ops.softmax(xd + 3.0), y) <= 2e-6           # shift invariance
    assert torch.equal(y.argmax(dim=1), xd.argmax(dim=1))             # order preserved


def test_layer_norm_16384x4096():
    x, w, b, inv, eps = workloads.layer_norm_inputs()
    xd, wd, bd = x.to(DEV), w.to(DEV), b.to(DEV)
    y = ops.layer_norm(xd, wd, bd, inv, eps)
    sample = slice(0, 1024)
    assert relative_error(y[sample], oracle.layer_norm(x[sample], w, b, inv, eps)) <= 1e-2
    # un-doing the affine part must leave rows with zero mean and unit variance
    z = (y.double() - bd.double()) / wd.double()
    assert z.mean(dim=1).abs().max() < 5e-3
    assert (z.var(dim=1, unbiased=False) - 1).abs().max() < 2e-2
    # a row's result does not depend on the other rows: permuting rows permutes the output
    order = torch.randperm(16384, device=DEV, generator=torch.Generator(DEV).manual_seed(0))
    assert torch.equal(ops.layer_norm(xd[order].contiguous(), wd, bd, inv, eps), y[order])


def test_gemm_8192_cubed():
    a, b = workloads.gemm_inputs()
    ad, bd = a.to(DEV), b.t().contiguous().to(DEV).t()
    c = ops.gemm(ad, bd)
    ops.workspace_status(DEV)
    rows = (4000, 32)
    expected = torch.empty(8192, 8192, dtype=torch.float16)
    oracle.gemm(a, b, rows=rows, out=expected)
    block = slice(rows[0], rows[0] + rows[1])
    assert relative_error(c[block], expected[block]) <= 1e-2
    # linearity in exact arithmetic: doubling A doubles C bit for bit (a power-of-two scale commutes
    # with f16 rounding except where C is subnormal in f16)
    doubled = ops.gemm((ad * 2).contiguous(), bd).float()
    normal = c.float().abs() >= 2.0 ** -13
    assert torch.equal(doubled[normal], c.float()[normal] * 2)
    assert (doubled[~normal] - c.float()[~normal] * 2).abs().max() <= 2.0 ** -23
    # checksum of checksums: sum_n C[m, n] == A[m, :] . sum_n B[:, n] within accumulation tolerance
    column_sums = bd.double().sum(dim=1)
    assert relative_error(c.double().sum(dim=1), ad.double() @ column_sums) <= 2e-3


def test_attention_8x32x4096x128():
    q, k, v, scale = workloads.attention_inputs()
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    out = ops.flash_attention(qd, kd, vd, scale)
    ops.workspace_status(DEV)
    units = (37, 2)
    expected = torch.empty_like(q)
    oracle.attention(q, k, v, scale, units=units, out=expected)
    flat, flat_expected = out.reshape(256, 4096, 128), expected.reshape(256, 4096, 128)
    assert relative_error(flat[37:39], flat_expected[37:39]) <= 1e-2
    # causality: the first query row attends to key 0 only, so its output is V[.., 0, :]
    assert torch.equal(out[:, :, 0], vd[:, :, 0])
    # outputs are convex combinations of the values seen so far
    running_max = vd.float().cummax(dim=2).values
    running_min = vd.float().cummin(dim=2).values
    assert (out.float() <= running_max + 2e-2).all() and (out.float() >= running_min - 2e-2).all()
    # changing future keys / values leaves earlier rows untouched
    kd2, vd2 = kd.clone(), vd.clone()
    kd2[:, :, 2048:] = 0
    vd2[:, :, 2048:] = 1
    assert torch.equal(ops.flash_attention(qd, kd2, vd2, scale)[:, :, :2048], out[:, :, :2048])


def test_csr_spmm_262144():
    ro, ci, va, x = workloads.csr_inputs()
    d = [t.to(DEV) for t in (ro, ci, va, x)]
    ops.csr_validate(d[0], d[1], 262144)
    y = ops.csr_spmm(*d)
    rows = (100000, 8192)
    expected = torch.zeros(262144, 128)
    oracle.csr_spmm(ro, ci, va, x, rows=rows, out=expected)
    block = slice(rows[0], rows[0] + rows[1])
    assert torch.equal(y[block].cpu(), expected[block])               # bit-exact on the sample
    # linearity in the values with an exact scale, and idempotence of a repeated launch
    assert torch.equal(ops.csr_spmm(d[0], d[1], d[2] * 2, d[3]), y * 2)
    assert torch.equal(ops.csr_spmm(*d), y)
    # checksum: sum_f Y[r, f] == sum_nz a * (sum_f X[c, f]) within fp32 accumulation tolerance
    feature_sums = d[3].double().sum(dim=1)
    per_row = (d[2].double() * feature_sums[d[1].long()]).reshape(262144, 32).sum(dim=1)
    assert relative_error(y.double().sum(dim=1), per_row) <= 2e-3
