"""Seeded synthetic inputs of the five benchmark workloads.

The reference's example inputs are ``numpy.random.default_rng(seed)`` draws in
fp32 followed by a round-to-nearest cast to the storage type
(``python/intent/examples/programs/inputs.py:16-27, 99-112``); these generators
keep that order.  No public dataset or benchmark suite is involved: shapes and
value distributions are the ones the workload descriptions state.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch


@dataclass(frozen=True)
class Workload:
    name: str
    unit: str              # "GB/s" or "TFLOP/s"
    bound: str             # "hbm" or "tensor"
    work: float            # algorithmic bytes (hbm) or flops (tensor) per launch
    description: str


def _f32(array) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32))


def softmax_inputs(m: int = 4096, n: int = 1024, seed: int = 0):
    rng = np.random.default_rng(seed)
    return (_f32(rng.standard_normal((m, n), dtype=np.float32)),)


def layer_norm_inputs(m: int = 16384, n: int = 4096, seed: int = 0, dtype=torch.float16):
    rng = np.random.default_rng(seed)
    x = _f32(rng.standard_normal((m, n), dtype=np.float32)).to(dtype)
    gamma = _f32(0.5 + rng.random((n,), dtype=np.float32)).to(dtype)
    beta = _f32(-0.1 + 0.2 * rng.random((n,), dtype=np.float32)).to(dtype)
    return x, gamma, beta, float(np.float32(1.0 / n)), float(np.float32(1e-5))


def gemm_inputs(m: int = 8192, n: int = 8192, k: int = 8192, seed: int = 0, dtype=torch.float16):
    """A row-major (M,K); B column-major (K,N), i.e. the transpose view of a contiguous (N,K)."""
    rng = np.random.default_rng(seed)
    a = _f32(2.0 * rng.random((m, k), dtype=np.float32) - 1.0).to(dtype)
    bt = _f32(2.0 * rng.random((n, k), dtype=np.float32) - 1.0).to(dtype)
    return a, bt.t()


def attention_inputs(b: int = 8, h: int = 32, s: int = 4096, d: int = 128, seed: int = 0,
                     dtype=torch.bfloat16, kv_heads: int | None = None):
    rng = np.random.default_rng(seed)
    hk = h if kv_heads is None else kv_heads
    q = _f32(0.5 * rng.standard_normal((b, h, s, d), dtype=np.float32)).to(dtype)
    k = _f32(0.5 * rng.standard_normal((b, hk, s, d), dtype=np.float32)).to(dtype)
    v = _f32(0.5 * rng.standard_normal((b, hk, s, d), dtype=np.float32)).to(dtype)
    return q, k, v, float(np.float32(1.0 / math.sqrt(d)))


def attention_backward_inputs(b: int = 2, hq: int = 8, hk: int = 2, s: int = 1024, d: int = 64, seed: int = 0,
                              dtype=torch.float16, causal: bool = True, keys: int | None = None, device=None):
    """q, k, v, output, grad_output, lse (natural log), scale for the backward trio.  The forward
    pass that yields output and lse is evaluated head by head on the rounded operands, in f64 on the
    host, or in f32 on ``device`` when one is given (the large benchmark shape).  Defaults are the
    reference kernels' shape (kernels/backward/attention.py:7-13)."""
    rng = np.random.default_rng(seed)
    sk = s if keys is None else keys
    q = _f32(0.5 * rng.standard_normal((b, hq, s, d), dtype=np.float32)).to(dtype)
    k = _f32(0.5 * rng.standard_normal((b, hk, sk, d), dtype=np.float32)).to(dtype)
    v = _f32(0.5 * rng.standard_normal((b, hk, sk, d), dtype=np.float32)).to(dtype)
    grad_output = _f32(0.5 * rng.standard_normal((b, hq, s, d), dtype=np.float32)).to(dtype)
    scale = float(np.float32(1.0 / math.sqrt(d)))
    group = hq // hk
    wide = torch.float64 if device is None else torch.float32
    where = torch.device("cpu") if device is None else torch.device(device)
    allowed = (torch.arange(sk, device=where)[None, :] <= torch.arange(s, device=where)[:, None]) if causal else None
    output = torch.empty((b, hq, s, d), dtype=dtype)
    lse = torch.empty((b, hq, s), dtype=torch.float32)
    for batch in range(b):
        for head in range(hq):
            scores = (q[batch, head].to(where, wide) @ k[batch, head // group].to(where, wide).T) * scale
            if causal:
                scores = scores.masked_fill(~allowed, float("-inf"))
            row_lse = torch.logsumexp(scores, dim=-1)
            output[batch, head] = (torch.exp(scores - row_lse[:, None]) @ v[batch, head // group].to(where, wide)).to(dtype).cpu()
            lse[batch, head] = row_lse.float().cpu()
    return q, k, v, output, grad_output, lse, scale


def attention_backward_workload(b=8, hq=32, hk=8, s=2048, d=128) -> Workload:
    """delta + dK/dV + dQ: seven S x S x D products per query head over the causal half
    (K.Q^T, V.dO^T, P^T.dO, dS^T.Q; Q.K^T, dO.V^T, dS.K)."""
    flops = 7.0 * 2.0 * b * hq * (s * (s + 1) / 2) * d
    return Workload("attention_backward", "TFLOP/s", "tensor", flops,
                    f"causal attention backward f16 B={b} HQ={hq} HK={hk} S={s} D={d} (delta, dK/dV, dQ)")


def csr_inputs(rows: int = 262144, columns: int = 262144, per_row: int = 32, features: int = 128,
               seed: int = 0):
    """`per_row` distinct, ascending, uniformly drawn column indices per row."""
    rng = np.random.default_rng(seed)
    per_row = min(per_row, columns)
    column_indices = np.empty((rows, per_row), dtype=np.int32)
    pending = np.arange(rows)
    extra = max(8, per_row // 4)
    while pending.size:
        if columns <= 4 * per_row:  # dense-ish: exact sampling without replacement
            block = np.argsort(rng.random((pending.size, columns)), axis=1)[:, :per_row]
            column_indices[pending] = np.sort(block, axis=1).astype(np.int32)
            break
        draw = rng.integers(0, columns, size=(pending.size, per_row + extra), dtype=np.int64)
        order = np.argsort(draw, axis=1, kind="stable")
        ranked = np.take_along_axis(draw, order, axis=1)
        repeated_ranked = np.zeros_like(ranked, dtype=bool)
        repeated_ranked[:, 1:] = ranked[:, 1:] == ranked[:, :-1]
        repeated = np.empty_like(repeated_ranked)
        np.put_along_axis(repeated, order, repeated_ranked, axis=1)  # later occurrences, in draw order
        enough = (~repeated).sum(axis=1) >= per_row
        good = np.nonzero(enough)[0]
        if good.size:
            # the first per_row distinct draws in draw order (exchangeable, hence uniform), then sorted
            first = np.argsort(repeated[good], axis=1, kind="stable")[:, :per_row]
            chosen = np.take_along_axis(draw[good], first, axis=1)
            column_indices[pending[good]] = np.sort(chosen, axis=1).astype(np.int32)
        pending = pending[~enough]
    row_offsets = np.arange(0, rows * per_row + 1, per_row, dtype=np.int32)
    values = (2.0 * rng.random(rows * per_row, dtype=np.float32) - 1.0).astype(np.float32)
    dense = rng.standard_normal((columns, features), dtype=np.float32)
    return (torch.from_numpy(row_offsets), torch.from_numpy(column_indices.reshape(-1)),
            torch.from_numpy(values), torch.from_numpy(dense))


def softmax_workload(m=4096, n=1024) -> Workload:
    return Workload("softmax", "GB/s", "hbm", 2.0 * m * n * 4, f"row softmax fp32 {m}x{n}")


def layer_norm_workload(m=16384, n=4096) -> Workload:
    return Workload("layer_norm", "GB/s", "hbm", 2.0 * m * n * 2 + 2.0 * n * 2,
                    f"LayerNorm f16 {m}x{n}, fp32 statistics")


def gemm_workload(m=8192, n=8192, k=8192) -> Workload:
    return Workload("gemm", "TFLOP/s", "tensor", 2.0 * m * n * k,
                    f"GEMM f16 {m}x{n}x{k}, row-major A, column-major B, fp32 accumulate")


def attention_workload(b=8, h=32, s=4096, d=128) -> Workload:
    return Workload("attention", "TFLOP/s", "tensor", 4.0 * b * h * d * s * (s + 1) / 2,
                    f"causal flash-attention bf16 B={b} H={h} S={s} D={d}")


def spmm_workload(rows=262144, columns=262144, per_row=32, features=128) -> Workload:
    nnz = rows * per_row
    compulsory = (rows + 1) * 4 + nnz * 8 + columns * features * 4 + rows * features * 4
    return Workload("spmm", "GB/s", "hbm", float(compulsory),
                    f"CSR SpMM fp32 {rows}x{columns}, {per_row} nnz/row, X {columns}x{features}")


def softmax_backward_inputs(m: int = 4096, n: int = 4097, seed: int = 0):
    """Probabilities of a seeded N(0,1) score matrix and an N(0,1) upstream gradient; the
    shape is the reference kernel's static one (kernels/backward/softmax.py:5-6)."""
    rng = np.random.default_rng(seed)
    scores = _f32(rng.standard_normal((m, n), dtype=np.float32))
    upstream = _f32(rng.standard_normal((m, n), dtype=np.float32))
    return torch.softmax(scores, dim=1), upstream


def softmax_backward_workload(m=4096, n=4097) -> Workload:
    return Workload("softmax_backward", "GB/s", "hbm", 3.0 * m * n * 4, f"softmax backward fp32 {m}x{n}")


def layer_norm_backward_inputs(m: int = 4096, n: int = 4096, groups: int = 128, seed: int = 0):
    """bf16 x, dy, weight with the f32 row statistics of x (epsilon 1e-5) and zeroed bf16
    partial-sum matrices; the shape is the reference kernel's (kernels/backward/layer_norm.py:5-7)."""
    rng = np.random.default_rng(seed)
    x = _f32(rng.standard_normal((m, n), dtype=np.float32)).to(torch.bfloat16)
    dy = _f32(rng.standard_normal((m, n), dtype=np.float32)).to(torch.bfloat16)
    weight = _f32(1.0 + 0.1 * rng.standard_normal(n, dtype=np.float32)).to(torch.bfloat16)
    values = x.float()
    mean = values.mean(dim=1)
    rstd = torch.rsqrt(values.var(dim=1, unbiased=False) + 1e-5)
    dw_partial = torch.zeros((groups, n), dtype=torch.bfloat16)
    db_partial = torch.zeros((groups, n), dtype=torch.bfloat16)
    return x, dy, weight, mean, rstd, dw_partial, db_partial, float(np.float32(1.0 / n))


def layer_norm_backward_workload(m=4096, n=4096, groups=128) -> Workload:
    """Row kernel plus the reduction of its partial sums."""
    rows_kernel = 3.0 * m * n * 2 + 4.0 * groups * n * 2 + n * 2 + m * 8
    reduce_kernel = 2.0 * groups * n * 2 + 2.0 * n * 4
    return Workload("layer_norm_backward", "GB/s", "hbm", rows_kernel + reduce_kernel,
                    f"LayerNorm backward bf16 {m}x{n}, {groups} partial-sum groups (rows + reduce)")


def spmv_workload(rows=32768, columns=32768, per_row=32) -> Workload:
    nnz = rows * per_row
    return Workload("spmv", "GB/s", "hbm", float((rows + 1) * 4 + nnz * 8 + columns * 4 + rows * 4),
                    f"CSR SpMV fp32 {rows}x{columns}, {per_row} nnz/row")
