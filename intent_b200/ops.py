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
    device = _require_cuda(x)
    y = torch.empty(x.shape, dtype=x.dtype, device=device) if out is None else out
    _call("b200_softmax", device, *_slots(x), *_slots(y), _CODES[x.dtype], _stream(x))
    return y


def layer_norm(x, weight, bias, inverse_features: float, epsilon: float, out=None, *, centered=None):
    device = _require_cuda(x, weight, bias)
    y = torch.empty(x.shape, dtype=x.dtype, device=device) if out is None else out
    if centered is None:  # the f32 kernel of the reference is the uncentred one
        centered = x.dtype != torch.float32
    _call("b200_layer_norm", device, *_slots(x), *_slots(weight), *_slots(bias), *_slots(y),
          float(inverse_features), float(epsilon), _CODES[x.dtype], int(centered), _stream(x))
    return y


def gemm(a, b, out=None, *, relu: bool = False):
    device = _require_cuda(a, b)
    c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=device) if out is None else out
    _call("b200_gemm", device, *_slots(a), *_slots(b), *_slots(c), *_slots(workspace(device)),
          _CODES[a.dtype], int(relu), _stream(a))
    return c


def flash_attention(q, k, v, scale: float, out=None, *, head_group: int = 1, causal: bool = True):
    device = _require_cuda(q, k, v)
    if out is None:
        out = torch.empty((*q.shape[:3], v.shape[3]), dtype=q.dtype, device=device)
    _call("b200_flash_attention", device, *_slots(q), *_slots(k), *_slots(v), *_slots(out),
          float(scale), *_slots(workspace(device)), _CODES[q.dtype], int(head_group), int(causal),
          _stream(q))
    return out


def csr_spmm(row_offsets, column_indices, values, dense, out=None, *, state=None):
    """`state`: the call's int32 workspace (``workspace(device)`` by default); calls that may overlap
    on different streams need one each."""
    device = _require_cuda(row_offsets, column_indices, values, dense)
    if out is None:
        out = torch.empty((row_offsets.numel() - 1, dense.shape[1]), dtype=torch.float32, device=device)
    _call("b200_csr_spmm", device, *_slots(row_offsets), *_slots(column_indices), *_slots(values),
          *_slots(dense), *_slots(out), *_slots(workspace(device) if state is None else state), _stream(dense))
    return out


def csr_spmv(row_offsets, column_indices, values, vector, out=None):
    device = _require_cuda(row_offsets, column_indices, values, vector)
    if out is None:
        out = torch.empty((row_offsets.numel() - 1,), dtype=torch.float32, device=device)
    _call("b200_csr_spmv", device, *_slots(row_offsets), *_slots(column_indices), *_slots(values),
          *_slots(vector), *_slots(out), _stream(vector))
    return out


def softmax_backward(probabilities, upstream, out=None):
    device = _require_cuda(probabilities, upstream)
    if out is None:
        out = torch.empty(probabilities.shape, dtype=probabilities.dtype, device=device)
    _call("b200_softmax_backward", device, *_slots(probabilities), *_slots(upstream), *_slots(out),
          _CODES[probabilities.dtype], _stream(probabilities))
    return out


def layer_norm_backward_rows(x, dy, weight, mean, rstd, dw_partial, db_partial, inverse_features: float, out=None):
    """Returns dx; accumulates into ``dw_partial`` / ``db_partial`` (InOut) in place."""
    device = _require_cuda(x, dy, weight, mean, rstd, dw_partial, db_partial)
    if out is None:
        out = torch.empty(x.shape, dtype=x.dtype, device=device)
    _call("b200_layer_norm_backward_rows", device, *_slots(x), *_slots(dy), *_slots(weight), *_slots(mean),
          *_slots(rstd), *_slots(out), *_slots(dw_partial), *_slots(db_partial), float(inverse_features), _stream(x))
    return out


def layer_norm_backward_reduce(dw_partial, db_partial, dw=None, db=None):
    device = _require_cuda(dw_partial, db_partial)
    columns = dw_partial.shape[1]
    if dw is None:
        dw = torch.empty((columns,), dtype=torch.float32, device=device)
    if db is None:
        db = torch.empty((columns,), dtype=torch.float32, device=device)
    _call("b200_layer_norm_backward_reduce", device, *_slots(dw_partial), *_slots(db_partial), *_slots(dw), *_slots(db),
          _stream(dw_partial))
    return dw, db


def attention_backward_delta(output, grad_output, out=None):
    device = _require_cuda(output, grad_output)
    if out is None:
        out = torch.empty(output.shape[:3], dtype=torch.float32, device=device)
    _call("b200_attention_backward_delta", device, *_slots(output), *_slots(grad_output), *_slots(out),
          _CODES[output.dtype], _stream(output))
    return out


def attention_backward_dkdv(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                            causal: bool = True, grad_k=None, grad_v=None):
    device = _require_cuda(q, k, v, grad_output, lse, delta)
    grad_k = torch.empty(k.shape, dtype=k.dtype, device=device) if grad_k is None else grad_k
    grad_v = torch.empty(v.shape, dtype=v.dtype, device=device) if grad_v is None else grad_v
    space = workspace(device)
    _call("b200_attention_backward_dkdv", device, *_slots(q), *_slots(k), *_slots(v), *_slots(grad_output),
          *_slots(lse), *_slots(delta), *_slots(grad_k), *_slots(grad_v), float(scale), *_slots(space),
          _CODES[q.dtype], int(head_group), int(causal), _stream(q))
    return grad_k, grad_v


def attention_backward_dq(q, k, v, grad_output, lse, delta, scale: float, *, head_group: int = 1,
                          causal: bool = True, grad_q=None):
    device = _require_cuda(q, k, v, grad_output, lse, delta)
    grad_q = torch.empty(q.shape, dtype=q.dtype, device=device) if grad_q is None else grad_q
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
