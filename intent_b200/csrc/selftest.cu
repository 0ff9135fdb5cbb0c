// A check of the bounded-wait path the tensor-core kernels rely on, for use by tests.
//
// Every mbarrier wait in the GEMM and attention kernels gives up after a cycle limit: it raises
// the CTA's abort flag, publishes {1, site} in the call's workspace and returns, so a lost
// arrival ends as an error status the host reads, never as a hung GPU.  That path cannot be
// reached through the operators without breaking one of them, so this entry runs it directly:
// one CTA initialises a barrier that nothing will ever arrive on and waits for it with a SHORT
// limit.  The kernel neither faults nor spins for long; it returns after `limit_cycles`.
#include "tc.cuh"

namespace b200 {
namespace {

__global__ void bounded_wait_selftest_kernel(int *status, long long limit_cycles, int *observed) {
  __shared__ uint64_t never_completed;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&never_completed, 1);
    abort_flag = 0;
    tc::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool arrived = tc::mbar_wait(&never_completed, 0, &abort_flag, status, tc::kSiteSelfTest, limit_cycles);
    observed[0] = arrived ? 1 : 0;
  }
  __syncthreads();
  // what the other roles of a kernel do once a wait has given up: see the flag and leave
  if (threadIdx.x == 32) observed[1] = abort_flag;
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_selftest_bounded_wait(void *workspace, int64_t ws_d0, int64_t ws_s0, int64_t limit_cycles,
                                          void *stream) {
  if (!workspace || ws_d0 < B200_WORKSPACE_WORDS || (ws_d0 > 1 && ws_s0 != 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "selftest_bounded_wait: workspace must hold %d contiguous int32 words",
                B200_WORKSPACE_WORDS);
  if (limit_cycles < 1000 || limit_cycles > 200000000)
    return fail(B200_ERR_INVALID_ARGUMENT, "selftest_bounded_wait: the limit must lie between 1e3 and 2e8 cycles");
  int *words = static_cast<int *>(workspace);
  // words 0-1: the status report; words 8-9: what the kernel observed (arrived?, abort flag seen by another warp)
  bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(words, limit_cycles, words + 8);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
