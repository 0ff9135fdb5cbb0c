"""Writes tests/golden/oracle_vectors.pt: outputs of the CPU oracle on small seeded
inputs.  They pin the oracle against accidental change; they are NOT reference
outputs (the reference's compiler and CPU provider cannot run here, and it ships
no vectors of its own).  Run from the repository root: python tests/golden/make_vectors.py"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import oracle  # noqa: E402
from intent_b200 import workloads  # noqa: E402

vectors = {}
(x,) = workloads.softmax_inputs(4, 16, seed=100)
vectors["softmax"] = oracle.softmax(x)
x, w, b, inv, eps = workloads.layer_norm_inputs(4, 64, seed=101)
vectors["layer_norm"] = oracle.layer_norm(x, w, b, inv, eps)
a, b = workloads.gemm_inputs(8, 16, 32, seed=102)
vectors["gemm"] = oracle.gemm(a, b)
q, k, v, scale = workloads.attention_inputs(1, 2, 32, 64, seed=103)
vectors["attention"] = oracle.attention(q, k, v, scale, chunk=16)
ro, ci, va, x = workloads.csr_inputs(8, 32, 4, 16, seed=104)
vectors["csr_spmm"] = oracle.csr_spmm(ro, ci, va, x)
x, dy, w, mean, rstd, dw_partial, db_partial, inv = workloads.layer_norm_backward_inputs(8, 32, 4, seed=105)
vectors["layer_norm_backward_dx"] = oracle.layer_norm_backward_rows(x, dy, w, mean, rstd, dw_partial, db_partial, inv)
vectors["layer_norm_backward_dw_partial"], vectors["layer_norm_backward_db_partial"] = dw_partial, db_partial
vectors["layer_norm_backward_dw"], vectors["layer_norm_backward_db"] = oracle.layer_norm_backward_reduce(dw_partial, db_partial)
p, u = workloads.softmax_backward_inputs(4, 20, seed=106)
vectors["softmax_backward"] = oracle.softmax_backward(p, u)
q, k, v, output, grad_output, lse, scale = workloads.attention_backward_inputs(1, 2, 1, 24, 64, seed=107)
delta = oracle.attention_backward_delta(output, grad_output)
vectors["attention_backward_delta"] = delta
vectors["attention_backward_grad_k"], vectors["attention_backward_grad_v"] = oracle.attention_backward_dkdv(
    q, k, v, grad_output, lse, delta, scale, head_group=2)
vectors["attention_backward_grad_q"] = oracle.attention_backward_dq(q, k, v, grad_output, lse, delta, scale, head_group=2)
torch.save(vectors, Path(__file__).resolve().parent / "oracle_vectors.pt")
print({k: tuple(v.shape) for k, v in vectors.items()})
