"""TEST INFRASTRUCTURE: Python face of the CPU oracle in ``oracle.c``.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this
package; the shipped ``intent_b200`` package never does.  Parity is unpinned:
the reference holds no golden vectors for these operators (see ``oracle.c``).

Every function takes CPU ``torch`` tensors (any strides), allocates the output
the way the reference runtime does (contiguous ``torch.empty``,
``python/intent/runtime/torch_views.py:59-82``) and returns it.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB = None

_DTYPES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def build(force: bool = False) -> Path:
    """Compile ``oracle.c`` with the committed Makefile (gcc only)."""
    target = _HERE / "liboracle.so"
    source = _HERE / "oracle.c"
    if force or not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True,
                       capture_output=True, text=True)
    return target


def library() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        target = _HERE / "liboracle.so"
        if not target.exists():
            build()
        lib = ctypes.CDLL(str(target))
        lib.oracle_now_ms.restype = ctypes.c_double
        lib.oracle_max_workers.restype = ctypes.c_int
        _LIB = lib
    return _LIB


def default_workers() -> int:
    """The reference CPU provider's default team: min(8, allowed CPUs)
    (``python/intent/targets/execution.py:20-26``)."""
    return min(8, len(os.sched_getaffinity(0)))


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _i64(v) -> ctypes.c_int64:
    return ctypes.c_int64(int(v))


def _strides4(t: torch.Tensor):
    return (ctypes.c_int64 * 4)(*t.stride())


def _check_cpu(*tensors):
    for t in tensors:
        if t.device.type != "cpu":
            raise ValueError("the oracle runs on CPU tensors only")


def softmax(x: torch.Tensor, *, workers: int | None = None) -> torch.Tensor:
    _check_cpu(x)
    y = torch.empty(x.shape, dtype=x.dtype)
    m, n = x.shape
    library().oracle_softmax(_ptr(x), _ptr(y), _i64(m), _i64(n), _i64(x.stride(0)), _i64(x.stride(1)),
                             _i64(y.stride(0)), _i64(y.stride(1)), _DTYPES[x.dtype],
                             _i64(workers or default_workers()))
    return y


def layer_norm(x, weight, bias, inverse_features: float, epsilon: float, *, workers=None):
    _check_cpu(x, weight, bias)
    y = torch.empty(x.shape, dtype=x.dtype)
    m, n = x.shape
    library().oracle_layer_norm(
        _ptr(x), _ptr(weight), _ptr(bias), _ptr(y), _i64(m), _i64(n), _i64(x.stride(0)),
        _i64(x.stride(1)), _i64(weight.stride(0)), _i64(bias.stride(0)), _i64(y.stride(0)),
        _i64(y.stride(1)), ctypes.c_float(inverse_features), ctypes.c_float(epsilon),
        _DTYPES[x.dtype], _i64(workers or default_workers()))
    return y


def gemm(a, b, *, relu: bool = False, rows: tuple[int, int] | None = None, out=None, workers=None):
    """``rows=(begin, count)`` computes only that block of C (a bounded sample)."""
    _check_cpu(a, b)
    m, k = a.shape
    n = b.shape[1]
    c = torch.empty((m, n), dtype=a.dtype) if out is None else out
    begin, count = rows if rows is not None else (0, m)
    library().oracle_gemm(
        _ptr(a), _ptr(b), _ptr(c), _i64(begin), _i64(count), _i64(n), _i64(k), _i64(a.stride(0)),
        _i64(a.stride(1)), _i64(b.stride(0)), _i64(b.stride(1)), _i64(c.stride(0)), _i64(c.stride(1)),
        _DTYPES[a.dtype], int(relu), _i64(workers or default_workers()))
    return c


def attention(q, k, v, scale: float, *, head_group: int = 1, causal: bool = True, chunk: int = 128,
              units: tuple[int, int] | None = None, out=None, workers=None):
    """``units=(begin, count)`` computes only those flattened (batch, head) units."""
    _check_cpu(q, k, v)
    b, hq, sq, d = q.shape
    hk, sk, dv = k.shape[1], k.shape[2], v.shape[3]
    o = torch.empty((b, hq, sq, dv), dtype=q.dtype) if out is None else out
    begin, count = units if units is not None else (0, b * hq)
    status = library().oracle_attention(
        _ptr(q), _ptr(k), _ptr(v), _ptr(o), _i64(b), _i64(hq), _i64(hk), _i64(sq), _i64(sk), _i64(d),
        _i64(dv), _strides4(q), _strides4(k), _strides4(v), _strides4(o), ctypes.c_float(scale),
        _i64(head_group), int(causal), _DTYPES[q.dtype], _i64(chunk), _i64(begin), _i64(count),
        _i64(workers or default_workers()))
    if status:
        raise ValueError("oracle_attention rejected its arguments")
    return o


def csr_validate(row_offsets, column_indices, columns: int) -> None:
    where = ctypes.c_int64(-1)
    status = library().oracle_csr_validate(
        _ptr(row_offsets), _ptr(column_indices), _i64(row_offsets.numel() - 1),
        _i64(column_indices.numel()), _i64(columns), ctypes.byref(where))
    if status:
        raise ValueError(f"CSR structure is invalid at position {where.value}")


def csr_spmm(row_offsets, column_indices, values, dense, *, rows: tuple[int, int] | None = None,
             out=None, workers=None):
    _check_cpu(row_offsets, column_indices, values, dense)
    total = row_offsets.numel() - 1
    features = dense.shape[1]
    y = torch.empty((total, features), dtype=torch.float32) if out is None else out
    begin, count = rows if rows is not None else (0, total)
    library().oracle_csr_spmm(
        _ptr(row_offsets), _ptr(column_indices), _ptr(values), _ptr(dense), _ptr(y), _i64(begin),
        _i64(count), _i64(features), _i64(dense.stride(0)), _i64(dense.stride(1)), _i64(y.stride(0)),
        _i64(y.stride(1)), _i64(workers or default_workers()))
    return y


def csr_spmv(row_offsets, column_indices, values, vector, *, workers=None):
    _check_cpu(row_offsets, column_indices, values, vector)
    rows = row_offsets.numel() - 1
    y = torch.empty((rows,), dtype=torch.float32)
    library().oracle_csr_spmv(_ptr(row_offsets), _ptr(column_indices), _ptr(values), _ptr(vector), _ptr(y),
                              _i64(rows), _i64(vector.stride(0)), _i64(1), _i64(workers or default_workers()))
    return y


def softmax_backward(probabilities, upstream, *, workers=None):
    _check_cpu(probabilities, upstream)
    if probabilities.stride(1) != 1 or upstream.stride(1) != 1:
        raise ValueError("the oracle takes unit inner strides here")
    g = torch.empty(probabilities.shape, dtype=torch.float32)
    m, n = probabilities.shape
    library().oracle_softmax_backward(_ptr(probabilities), _ptr(upstream), _ptr(g), _i64(m), _i64(n),
                                      _i64(probabilities.stride(0)), _i64(upstream.stride(0)), _i64(g.stride(0)),
                                      _i64(workers or default_workers()))
    return g


def now_ms() -> float:
    return library().oracle_now_ms()


def evict(buffer: torch.Tensor) -> None:
    library().oracle_evict(_ptr(buffer), _i64(buffer.numel() * buffer.element_size()))


def layer_norm_backward_rows(x, dy, weight, mean, rstd, dw_partial, db_partial, inverse_features: float, *,
                             workers=None):
    """Returns dx; accumulates into ``dw_partial`` / ``db_partial`` in place (they are InOut)."""
    _check_cpu(x, dy, weight, mean, rstd, dw_partial, db_partial)
    for t in (x, dy, dw_partial, db_partial):
        if t.dtype != torch.bfloat16 or t.stride(1) != 1:
            raise ValueError("the oracle takes bf16 matrices with unit inner strides here")
    m, n = x.shape
    dx = torch.empty((m, n), dtype=torch.bfloat16)
    status = library().oracle_layer_norm_backward_rows(
        _ptr(x), _ptr(dy), _ptr(weight.contiguous()), _ptr(mean.contiguous()), _ptr(rstd.contiguous()), _ptr(dx),
        _ptr(dw_partial), _ptr(db_partial), _i64(m), _i64(n), _i64(dw_partial.shape[0]), _i64(x.stride(0)),
        _i64(dy.stride(0)), _i64(dx.stride(0)), _i64(dw_partial.stride(0)), _i64(db_partial.stride(0)),
        ctypes.c_float(inverse_features), _i64(workers or default_workers()))
    if status:
        raise ValueError("oracle_layer_norm_backward_rows rejected its arguments")
    return dx


def layer_norm_backward_reduce(dw_partial, db_partial, *, workers=None):
    _check_cpu(dw_partial, db_partial)
    groups, n = dw_partial.shape
    dw = torch.empty((n,), dtype=torch.float32)
    db = torch.empty((n,), dtype=torch.float32)
    library().oracle_layer_norm_backward_reduce(
        _ptr(dw_partial), _ptr(db_partial), _ptr(dw), _ptr(db), _i64(groups), _i64(n),
        _i64(dw_partial.stride(0)), _i64(db_partial.stride(0)), _i64(workers or default_workers()))
    return dw, db


def _strides3(t: torch.Tensor):
    return list(t.stride()[:3])


def attention_backward_delta(output, grad_output, *, workers=None):
    _check_cpu(output, grad_output)
    b, hq, sq, d = output.shape
    delta = torch.empty((b, hq, sq), dtype=torch.float32)
    library().oracle_attention_backward_delta(
        _ptr(output), _ptr(grad_output), _ptr(delta), _i64(b), _i64(hq), _i64(sq), _i64(d),
        (ctypes.c_int64 * 3)(*_strides3(output)), (ctypes.c_int64 * 3)(*_strides3(grad_output)),
        (ctypes.c_int64 * 3)(*delta.stride()), _DTYPES[output.dtype], _i64(workers or default_workers()))
    return delta


def _attention_backward(which, q, k, v, grad_output, lse, delta, scale, head_group, causal, workers):
    _check_cpu(q, k, v, grad_output, lse, delta)
    for t in (q, k, v, grad_output):
        if t.stride(3) != 1:
            raise ValueError("the oracle takes unit inner strides here")
    b, hq, sq, d = q.shape
    hk, sk = k.shape[1], k.shape[2]
    gq = torch.empty((b, hq, sq, d), dtype=q.dtype)
    gk = torch.empty((b, hk, sk, d), dtype=q.dtype)
    gv = torch.empty((b, hk, sk, d), dtype=q.dtype)
    strides = []
    for t in (q, k, v, grad_output, lse, delta, gq, gk, gv):
        strides += _strides3(t)
    status = library().oracle_attention_backward(
        which, _ptr(q), _ptr(k), _ptr(v), _ptr(grad_output), _ptr(lse), _ptr(delta), _ptr(gq), _ptr(gk), _ptr(gv),
        _i64(b), _i64(hq), _i64(hk), _i64(sq), _i64(sk), _i64(d), (ctypes.c_int64 * 27)(*strides),
        ctypes.c_float(scale), _i64(head_group), int(causal), _DTYPES[q.dtype], _i64(workers or default_workers()))
    if status:
        raise ValueError("oracle_attention_backward rejected its arguments")
    return gq, gk, gv


def attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                            causal: bool = True, workers=None):
    _, gk, gv = _attention_backward(0, q, k, v, grad_output, lse, delta, scale, head_group, causal, workers)
    return gk, gv


def attention_backward_dq(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                          causal: bool = True, workers=None):
    gq, _, _ = _attention_backward(1, q, k, v, grad_output, lse, delta, scale, head_group, causal, workers)
    return gq
