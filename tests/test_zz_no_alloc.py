"""b200_gemm_static_scratch: the GEMM entry for callers that must not allocate.

Some users of this library run where device allocation is forbidden — inside a
region whose memory was fixed at start-up, or as a plugin that receives buffers
but no allocator — so they cannot supply b200_gemm's workspace view.  This entry
keeps that scratch in a device array inside the library.  The test calls it
through the C ABI twice in a row (the array is shared and keeps the previous
call's contents) and compares each result with b200_gemm's on the same operands
and with the CPU oracle, and checks that the device's free memory and torch's
allocator statistics do not move across the calls.  It is collected last so a run that stops at the first failure has already run
every other test, and it passes on its own in a fresh process as well.
"""
import pytest
import torch

import oracle
from conftest import relative_error
from intent_b200 import _native, ops, workloads

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_scratch_gemm(a, b, *, relu=False, check=1, out=None):
    c = torch.empty((a.shape[0], b.shape[1]), dtype=a.dtype, device=a.device) if out is None else out
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
        host_a, host_b = workloads.gemm_inputs(m, n, k, seed=seed, dtype=dtype)
        a, b = host_a.to(DEV), host_b.t().contiguous().to(DEV).t()
        expected = ops.gemm(a, b, relu=relu)
        ops.workspace_status(DEV)
        outputs = [torch.empty((m, n), dtype=dtype, device=DEV) for _ in range(2)]
        static_scratch_gemm(a, b, relu=relu, out=torch.empty((m, n), dtype=dtype, device=DEV))   # first use on the device
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(DEV)
        reserved_before = torch.cuda.memory_stats(DEV)["reserved_bytes.all.current"]
        requests_before = torch.cuda.memory_stats(DEV)["allocation.all.allocated"]
        first = static_scratch_gemm(a, b, relu=relu, out=outputs[0])
        second = static_scratch_gemm(a, b, relu=relu, check=0, out=outputs[1])
        torch.cuda.synchronize()
        # the entry exists for callers that cannot allocate: neither the driver's free memory nor
        # torch's allocator may have moved across the two calls
        assert torch.cuda.mem_get_info(DEV)[0] == free_before
        assert torch.cuda.memory_stats(DEV)["reserved_bytes.all.current"] == reserved_before
        assert torch.cuda.memory_stats(DEV)["allocation.all.allocated"] == requests_before
        # same kernel, same operands as the allocating entry: identical results, and both within
        # the GEMM parity tolerance (1e-2 on the narrowed output) of the CPU oracle
        assert torch.equal(first, expected)
        assert torch.equal(second, expected)
        assert relative_error(first, oracle.gemm(host_a, host_b, relu=relu)) <= 1e-2


def test_it_validates_like_the_allocating_entry():
    a, b = workloads.gemm_inputs(64, 64, 64, seed=3)
    a, b = a.to(DEV), b.t().contiguous().to(DEV).t()
    with pytest.raises(NotImplementedError):
        static_scratch_gemm(a, b.contiguous())               # this entry takes K-major B only
    with pytest.raises(ValueError):
        static_scratch_gemm(a, b[:-8])                       # K mismatch
    empty = static_scratch_gemm(a[:, :0], b[:0])
    assert empty.shape == (64, 64) and not empty.any()
