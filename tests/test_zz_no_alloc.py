"""b200_gemm_static_scratch: the GEMM entry for callers that must not allocate.

Some users of this library run where device allocation is forbidden — inside a
region whose memory was fixed at start-up, or as a plugin that receives buffers
but no allocator — so they cannot supply b200_gemm's workspace view.  This entry
keeps that scratch in a device array inside the library.  The test calls it
through the C ABI twice in a row (the array is shared and keeps the previous
call's contents) and compares each result with b200_gemm's on the same operands.
It is collected last so a run that stops at the first failure has already run
every other test, and it passes on its own in a fresh process as well.
"""
import pytest
import torch

from intent_b200 import _native, ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_scratch_gemm(a, b, *, relu=False, check=1):
    c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=a.device)
    code = {torch.float16: 1, torch.bfloat16: 2}[a.dtype]
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        status = _native.entry("b200_gemm_static_scratch")(
            a.data_ptr(), *a.shape, *a.stride(), b.data_ptr(), *b.shape, *b.stride(),
            c.data_ptr(), *c.shape, *c.stride(), code, int(relu), int(check), stream)
    _native.check("b200_gemm_static_scratch", status)
    return c


def test_two_calls_in_a_row_match_the_allocating_entry():
    for seed, (m, n, k), dtype, relu in [(1, (384, 512, 320), torch.float16, False),
                                         (2, (130, 264, 1024), torch.bfloat16, True)]:
        a, b = workloads.gemm_inputs(m, n, k, seed=seed, dtype=dtype)
        a, b = a.to(DEV), b.t().contiguous().to(DEV).t()
        expected = ops.gemm(a, b, relu=relu)
        ops.workspace_status(DEV)
        first = static_scratch_gemm(a, b, relu=relu)
        second = static_scratch_gemm(a, b, relu=relu, check=0)
        torch.cuda.synchronize()
        # same kernel, same operands: the tolerance of the GEMM parity tests is 1e-2,
        # and in fact the results are identical
        assert torch.equal(first, expected)
        assert torch.equal(second, expected)


def test_it_validates_like_the_allocating_entry():
    a, b = workloads.gemm_inputs(64, 64, 64, seed=3)
    a, b = a.to(DEV), b.t().contiguous().to(DEV).t()
    with pytest.raises(NotImplementedError):
        static_scratch_gemm(a, b.contiguous())               # this entry takes K-major B only
    with pytest.raises(ValueError):
        static_scratch_gemm(a, b[:-8])                       # K mismatch
    empty = static_scratch_gemm(a[:, :0], b[:0])
    assert empty.shape == (64, 64) and not empty.any()
