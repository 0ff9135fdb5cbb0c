"""Direct operator calls over CUDA ``torch`` tensors.

Each function packs its tensors into the flat slot list of the C ABI
(pointer, extents, element strides per view — the layout
``lib/Serialization/NativeABI.cpp:80-118`` defines), appends the private tail
and the current CUDA stream, and makes ONE foreign call.  Nothing here computes
on the host and nothing synchronises: like the reference's GPU launches the work
is enqueued on torch's current stream (``doc/getting-started/usage.en.md:53-55``).
Outputs are allocated the way the reference runtime allocates omitted ``Out``
buffers: contiguous ``torch.empty`` on the argument device
(``python/intent/runtime/torch_views.py:59-82``).
"""
from __future__ import annotations

import ctypes

import torch

from . import _native

_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _slots(tensor: torch.Tensor) -> list:
    return [tensor.data_ptr(), *tensor.shape, *tensor.stride()]


def _stream(tensor: torch.Tensor) -> int:
    return torch.cuda.current_stream(tensor.device).cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    device = tensors[0].device
    for tensor in tensors:
        if not isinstance(tensor, torch.Tensor):
            raise TypeError("intent_b200 operators take torch.Tensor arguments")
        if tensor.device.type != "cuda":
            raise ValueError(f"intent_b200 executes on cuda, but an argument is on {tensor.device}")
        if tensor.device != device:
            raise ValueError("arguments span different devices")
    return device


def _expect(name: str, tensor: torch.Tensor, dtype: torch.dtype, shape=None) -> None:
    """What the runtime binder checks for a bound view (``B200Program._observe``), for callers
    that come straight here: a wrong element type or extent must never reach the kernel, which
    trusts them (an int64 index array read as int32, or an output buffer of half the size, would
    send loads and stores out of bounds)."""
    if tensor.dtype != dtype:
        raise TypeError(f"{name} must have dtype {dtype}, got {tensor.dtype}")
    if shape is not None and tuple(tensor.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(tensor.shape)}")


def _float_type(name: str, tensor: torch.Tensor, allowed=(torch.float32, torch.float16, torch.bfloat16)) -> torch.dtype:
    if tensor.dtype not in allowed:
        raise TypeError(f"{name} must be one of {', '.join(str(d) for d in allowed)}, got {tensor.dtype}")
    return tensor.dtype


def _call(name: str, device: torch.device, *arguments) -> None:
    with torch.cuda.device(device):
        _native.check(name, _native.entry(name)(*arguments))


_workspaces: dict[torch.device, torch.Tensor] = {}


def workspace(device: torch.device) -> torch.Tensor:
    """The zero-initialised int32 status/workspace view the tensor-core entries take."""
    device = torch.device(device)
    if device not in _workspaces:
        _workspaces[device] = torch.zeros(_native.WORKSPACE_WORDS, dtype=torch.int32, device=device)
    return _workspaces[device]


def workspace_status(device: torch.device) -> None:
    """Synchronise and raise if a bounded device-side wait gave up."""
    ws = workspace(device)
    detail = ctypes.c_int32(0)
    with torch.cuda.device(ws.device):
        status = _native.entry("b200_workspace_status")(ws.data_ptr(), ctypes.byref(detail), _stream(ws))
    if status != _native.OK:
        ws.zero_()
    _native.check("b200_workspace_status", status)


def softmax(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    device = _require_cuda(x) if out is None else _require_cuda(x, out)
    _float_type("x", x)
    if x.dim() != 2:
        raise ValueError("softmax takes a matrix")
    y = torch.empty(x.shape, dtype=x.dtype, device=device) if out is None else out
    _expect("out", y, x.dtype, x.shape)
    _call("b200_softmax", device, *_slots(x), *_slots(y), _CODES[x.dtype], _stream(x))
    return y


def layer_norm(x, weight, bias, inverse_features: float, epsilon: float, out=None, *, centered=None):
    device = _require_cuda(x, weight, bias) if out is None else _require_cuda(x, weight, bias, out)
    _float_type("x", x)
    if x.dim() != 2:
        raise ValueError("layer_norm takes a matrix")
    _expect("weight", weight, x.dtype, (x.shape[1],))
    _expect("bias", bias, x.dtype, (x.shape[1],))
    y = torch.empty(x.shape, dtype=x.dtype, device=device) if out is None else out
    _expect("out", y, x.dtype, x.shape)
    if centered is None:  # the f32 kernel of the reference is the uncentred one
        centered = x.dtype != torch.float32
    _call("b200_layer_norm", device, *_slots(x), *_slots(weight), *_slots(bias), *_slots(y),
          float(inverse_features), float(epsilon), _CODES[x.dtype], int(centered), _stream(x))
    return y


def gemm(a, b, out=None, *, relu: bool = False):
    device = _require_cuda(a, b) if out is None else _require_cuda(a, b, out)
    _float_type("a", a, (torch.float16, torch.bfloat16))
    if a.dim() != 2 or b.dim() != 2:
        raise ValueError("gemm takes two matrices")
    _expect("b", b, a.dtype, (a.shape[1], b.shape[1]))
    c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=device) if out is None else out
    _expect("out", c, a.dtype, (a.shape[0], b.shape[1]))
    _call("b200_gemm", device, *_slots(a), *_slots(b), *_slots(c), *_slots(workspace(device)),
          _CODES[a.dtype], int(relu), _stream(a))
    return c


def flash_attention(q, k, v, scale: float, out=None, *, head_group: int = 1, causal: bool = True):
    device = _require_cuda(q, k, v) if out is None else _require_cuda(q, k, v, out)
    _float_type("q", q, (torch.float16, torch.bfloat16))
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("flash_attention takes (batch, heads, sequence, head_dim) tensors")
    _expect("k", k, q.dtype, (q.shape[0], k.shape[1], k.shape[2], q.shape[3]))
    _expect("v", v, q.dtype, (q.shape[0], k.shape[1], k.shape[2], v.shape[3]))
    if out is None:
        out = torch.empty((*q.shape[:3], v.shape[3]), dtype=q.dtype, device=device)
    _expect("out", out, q.dtype, (*q.shape[:3], v.shape[3]))
    _call("b200_flash_attention", device, *_slots(q), *_slots(k), *_slots(v), *_slots(out),
          float(scale), *_slots(workspace(device)), _CODES[q.dtype], int(head_group), int(causal),
          _stream(q))
    return out


def _csr_operands(row_offsets, column_indices, values) -> None:
    _expect("row_offsets", row_offsets, torch.int32)
    _expect("column_indices", column_indices, torch.int32)
    _expect("values", values, torch.float32, column_indices.shape)
    if row_offsets.dim() != 1 or column_indices.dim() != 1 or row_offsets.numel() < 1:
        raise ValueError("CSR arrays have one axis and row_offsets holds rows + 1 entries")


def csr_spmm(row_offsets, column_indices, values, dense, out=None, *, state=None):
    """`state`: the call's int32 workspace (``workspace(device)`` by default); calls that may overlap
    on different streams need one each."""
    device = _require_cuda(row_offsets, column_indices, values, dense, *(() if out is None else (out,)))
    _csr_operands(row_offsets, column_indices, values)
    if dense.dim() != 2:
        raise ValueError("dense must be a matrix")
    _expect("dense", dense, torch.float32)
    if out is None:
        out = torch.empty((row_offsets.numel() - 1, dense.shape[1]), dtype=torch.float32, device=device)
    _expect("out", out, torch.float32, (row_offsets.numel() - 1, dense.shape[1]))
    if state is not None:
        _expect("state", state, torch.int32)
    _call("b200_csr_spmm", device, *_slots(row_offsets), *_slots(column_indices), *_slots(values),
          *_slots(dense), *_slots(out), *_slots(workspace(device) if state is None else state), _stream(dense))
    return out


def csr_spmv(row_offsets, column_indices, values, vector, out=None):
    device = _require_cuda(row_offsets, column_indices, values, vector, *(() if out is None else (out,)))
    _csr_operands(row_offsets, column_indices, values)
    _expect("vector", vector, torch.float32)
    if vector.dim() != 1:
        raise ValueError("vector must have one axis")
    if out is None:
        out = torch.empty((row_offsets.numel() - 1,), dtype=torch.float32, device=device)
    _expect("out", out, torch.float32, (row_offsets.numel() - 1,))
    _call("b200_csr_spmv", device, *_slots(row_offsets), *_slots(column_indices), *_slots(values),
          *_slots(vector), *_slots(out), _stream(vector))
    return out


def softmax_backward(probabilities, upstream, out=None):
    device = _require_cuda(probabilities, upstream, *(() if out is None else (out,)))
    _expect("probabilities", probabilities, torch.float32)
    _expect("upstream", upstream, torch.float32, probabilities.shape)
    if out is None:
        out = torch.empty(probabilities.shape, dtype=probabilities.dtype, device=device)
    _expect("out", out, torch.float32, probabilities.shape)
    _call("b200_softmax_backward", device, *_slots(probabilities), *_slots(upstream), *_slots(out),
          _CODES[probabilities.dtype], _stream(probabilities))
    return out


def layer_norm_backward_rows(x, dy, weight, mean, rstd, dw_partial, db_partial, inverse_features: float, out=None):
    """Returns dx; accumulates into ``dw_partial`` / ``db_partial`` (InOut) in place."""
    device = _require_cuda(x, dy, weight, mean, rstd, dw_partial, db_partial, *(() if out is None else (out,)))
    _expect("x", x, torch.bfloat16)
    if x.dim() != 2 or dw_partial.dim() != 2:
        raise ValueError("layer_norm_backward_rows takes matrices")
    _expect("dy", dy, torch.bfloat16, x.shape)
    _expect("weight", weight, torch.bfloat16, (x.shape[1],))
    _expect("mean", mean, torch.float32, (x.shape[0],))
    _expect("rstd", rstd, torch.float32, (x.shape[0],))
    _expect("dw_partial", dw_partial, torch.bfloat16, (dw_partial.shape[0], x.shape[1]))
    _expect("db_partial", db_partial, torch.bfloat16, dw_partial.shape)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=device)
    _expect("out", out, torch.bfloat16, x.shape)
    _call("b200_layer_norm_backward_rows", device, *_slots(x), *_slots(dy), *_slots(weight), *_slots(mean),
          *_slots(rstd), *_slots(out), *_slots(dw_partial), *_slots(db_partial), float(inverse_features), _stream(x))
    return out


def layer_norm_backward_reduce(dw_partial, db_partial, dw=None, db=None):
    device = _require_cuda(dw_partial, db_partial, *(t for t in (dw, db) if t is not None))
    _expect("dw_partial", dw_partial, torch.bfloat16)
    if dw_partial.dim() != 2:
        raise ValueError("the partial sums are matrices")
    _expect("db_partial", db_partial, torch.bfloat16, dw_partial.shape)
    columns = dw_partial.shape[1]
    for name, tensor in (("dw", dw), ("db", db)):
        if tensor is not None:
            _expect(name, tensor, torch.float32, (columns,))
    if dw is None:
        dw = torch.empty((columns,), dtype=torch.float32, device=device)
    if db is None:
        db = torch.empty((columns,), dtype=torch.float32, device=device)
    _call("b200_layer_norm_backward_reduce", device, *_slots(dw_partial), *_slots(db_partial), *_slots(dw), *_slots(db),
          _stream(dw_partial))
    return dw, db


def attention_backward_delta(output, grad_output, out=None):
    device = _require_cuda(output, grad_output, *(() if out is None else (out,)))
    _float_type("output", output, (torch.float16, torch.bfloat16))
    if output.dim() != 4:
        raise ValueError("attention_backward_delta takes (batch, heads, sequence, head_dim) tensors")
    _expect("grad_output", grad_output, output.dtype, output.shape)
    if out is None:
        out = torch.empty(output.shape[:3], dtype=torch.float32, device=device)
    _expect("out", out, torch.float32, output.shape[:3])
    _call("b200_attention_backward_delta", device, *_slots(output), *_slots(grad_output), *_slots(out),
          _CODES[output.dtype], _stream(output))
    return out


def _attention_backward_operands(q, k, v, grad_output, lse, delta) -> None:
    _float_type("q", q, (torch.float16, torch.bfloat16))
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("attention backward takes (batch, heads, sequence, head_dim) tensors")
    _expect("k", k, q.dtype, (q.shape[0], k.shape[1], k.shape[2], q.shape[3]))
    _expect("v", v, q.dtype, k.shape)
    _expect("grad_output", grad_output, q.dtype, q.shape)
    _expect("lse", lse, torch.float32, q.shape[:3])
    _expect("delta", delta, torch.float32, q.shape[:3])


def attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                            causal: bool = True, grad_k=None, grad_v=None):
    device = _require_cuda(q, k, v, grad_output, lse, delta, *(t for t in (grad_k, grad_v) if t is not None))
    _attention_backward_operands(q, k, v, grad_output, lse, delta)
    grad_k = torch.empty(k.shape, dtype=k.dtype, device=device) if grad_k is None else grad_k
    grad_v = torch.empty(v.shape, dtype=v.dtype, device=device) if grad_v is None else grad_v
    _expect("grad_k", grad_k, q.dtype, k.shape)
    _expect("grad_v", grad_v, q.dtype, v.shape)
    space = workspace(device)
    _call("b200_attention_backward_dkdv", device, *_slots(q), *_slots(k), *_slots(v), *_slots(grad_output),
          *_slots(lse), *_slots(delta), *_slots(grad_k), *_slots(grad_v), float(scale), *_slots(space),
          _CODES[q.dtype], int(head_group), int(causal), _stream(q))
    return grad_k, grad_v


def attention_backward_dq(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                          causal: bool = True, grad_q=None):
    device = _require_cuda(q, k, v, grad_output, lse, delta, *(() if grad_q is None else (grad_q,)))
    _attention_backward_operands(q, k, v, grad_output, lse, delta)
    grad_q = torch.empty(q.shape, dtype=q.dtype, device=device) if grad_q is None else grad_q
    _expect("grad_q", grad_q, q.dtype, q.shape)
    space = workspace(device)
    _call("b200_attention_backward_dq", device, *_slots(q), *_slots(k), *_slots(v), *_slots(grad_output),
          *_slots(lse), *_slots(delta), *_slots(grad_q), float(scale), *_slots(space), _CODES[q.dtype],
          int(head_group), int(causal), _stream(q))
    return grad_q


def gather_probe(table: torch.Tensor, gathers: int, *, variant: int = 1, hints: bool = True) -> None:
    """Enqueues the gather-rate probe over `table` (rows of 128 f32)."""
    device = _require_cuda(table)
    if table.dtype != torch.float32 or table.dim() != 2 or table.shape[1] != 128 or not table.is_contiguous():
        raise ValueError("gather_probe takes a contiguous f32 table of 128 columns")
    sink = _probe_sinks.get(device)
    if sink is None:
        sink = _probe_sinks[device] = torch.zeros(148 * 64 * 128 * 4, dtype=torch.float32, device=device)
    _call("b200_gather_probe", device, table.data_ptr(), table.shape[0], int(gathers), int(variant), int(hints),
          sink.data_ptr(), workspace(device).data_ptr(), _stream(table))


_probe_sinks: dict[torch.device, torch.Tensor] = {}


def csr_validate(row_offsets, column_indices, columns: int) -> None:
    device = _require_cuda(row_offsets, column_indices)
    where = ctypes.c_int64(-1)
    _call("b200_csr_validate", device, row_offsets.data_ptr(), row_offsets.numel() - 1,
          column_indices.data_ptr(), column_indices.numel(), int(columns), ctypes.byref(where),
          _stream(row_offsets))
