// CSR SpMM  Y = A . X  (i32 indices, f32 values).
//
// One warp owns one output row.  The 32 lanes cover 128 features with one
// float4 each, so a gathered row of X is one coalesced 512-byte read; column
// indices and values are fetched 32 at a time (coalesced) and broadcast with
// shuffles.  Terms are added strictly in storage order with a separately
// rounded multiply and add, so the result equals a sequential left-to-right
// evaluation bit for bit.  Algorithmic (compulsory) traffic per launch:
// (rows+1)*4 + nnz*8 + columns*F*4 + rows*F*4 bytes; the gathers of X are
// served by L2 where they hit.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kGatherDepth = 8;  // independent X-row loads in flight per lane

template <bool VECTOR>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
csr_spmm_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                const float *__restrict__ values, const float *__restrict__ dense,
                float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                int64_t output_pitch) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int start = row_offsets[row];
  const int stop = row_offsets[row + 1];
  constexpr int kWidth = VECTOR ? 4 : 1;
  for (int feature0 = 0; feature0 < features; feature0 += 32 * kWidth) {
    const int feature = feature0 + lane * kWidth;
    const bool active = feature < features;
    float acc[kWidth];
#pragma unroll
    for (int i = 0; i < kWidth; ++i) acc[i] = 0.0f;
    for (int base = start; base < stop; base += 32) {
      const int count = min(32, stop - base);
      int my_column = 0;
      float my_value = 0.0f;
      if (lane < count) {
        my_column = __ldcs(column_indices + base + lane);
        my_value = __ldcs(values + base + lane);
      }
      for (int j0 = 0; j0 < count; j0 += kGatherDepth) {
        float gathered[kGatherDepth][kWidth];
        float weight[kGatherDepth];
#pragma unroll
        for (int j = 0; j < kGatherDepth; ++j) {
          // lanes past `count` hold column 0 / value 0 and are skipped below
          const int column = __shfl_sync(0xffffffffu, my_column, (j0 + j) & 31);
          weight[j] = __shfl_sync(0xffffffffu, my_value, (j0 + j) & 31);
          if (active && j0 + j < count) {
            const float *source = dense + (int64_t)column * dense_pitch + feature;
            if (VECTOR) {
              const float4 v = __ldg(reinterpret_cast<const float4 *>(source));
              gathered[j][0] = v.x;
              if (kWidth > 1) { gathered[j][1 % kWidth] = v.y; gathered[j][2 % kWidth] = v.z; gathered[j][3 % kWidth] = v.w; }
            } else {
              gathered[j][0] = __ldg(source);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < kGatherDepth; ++j) {
          if (active && j0 + j < count) {
#pragma unroll
            for (int i = 0; i < kWidth; ++i)
              acc[i] = __fadd_rn(acc[i], __fmul_rn(weight[j], gathered[j][i]));
          }
        }
      }
    }
    if (active) {
      float *destination = output + row * output_pitch + feature;
      if (VECTOR) {
        float4 v;
        v.x = acc[0]; v.y = acc[1 % kWidth]; v.z = acc[2 % kWidth]; v.w = acc[3 % kWidth];
        __stcs(reinterpret_cast<float4 *>(destination), v);
      } else {
        destination[0] = acc[0];
      }
    }
  }
}

// result[0] = first bad position + 1 (0 = valid); atomicMin over positions.
__global__ void csr_validate_kernel(const int32_t *__restrict__ row_offsets, int64_t rows,
                                    const int32_t *__restrict__ column_indices, int64_t nnz,
                                    int64_t columns, unsigned long long *first_bad) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t r = tid; r < rows; r += stride) {
    const int32_t lo = row_offsets[r], hi = row_offsets[r + 1];
    if (lo < 0 || hi < lo || hi > nnz) atomicMin(first_bad, (unsigned long long)(r + 1));
  }
  const int64_t begin = rows > 0 ? row_offsets[0] : 0;
  const int64_t end = rows > 0 ? row_offsets[rows] : 0;
  if (begin >= 0 && end <= nnz)
    for (int64_t i = begin + tid; i < end; i += stride) {
      const int32_t c = column_indices[i];
      if (c < 0 || c >= columns) atomicMin(first_bad, (unsigned long long)(rows + 1 + i));
    }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_csr_spmm(const void *row_offsets, int64_t ro_d0, int64_t ro_s0,
                             const void *column_indices, int64_t ci_d0, int64_t ci_s0,
                             const void *values, int64_t va_d0, int64_t va_s0,
                             const void *dense, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                             void *output, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                             void *stream) {
  const int64_t rows = ro_d0 - 1;
  if (ro_d0 < 1 || ci_d0 < 0 || va_d0 != ci_d0 || x_d0 < 0 || x_d1 < 0 || y_d0 != rows || y_d1 != x_d1)
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm: inconsistent extents");
  if (rows == 0 || x_d1 == 0) return B200_OK;
  if (!row_offsets || !output || (ci_d0 > 0 && (!column_indices || !values || !dense)))
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm: null buffer");
  if ((ro_d0 > 1 && ro_s0 != 1) || (ci_d0 > 1 && (ci_s0 != 1 || va_s0 != 1)) ||
      (x_d1 > 1 && (x_s1 != 1 || y_s1 != 1)) || x_s0 < 0 || y_s0 < 0)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: index/value arrays must be contiguous and X, Y unit-stride in features");
  if (x_d1 > INT32_MAX || ci_d0 > INT32_MAX)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: i32 index space exceeded");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t ctas = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  if (ctas > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: too many rows");
  const bool vector = x_d1 % 4 == 0 && x_s0 % 4 == 0 && y_s0 % 4 == 0 && aligned16(dense) && aligned16(output);
  if (vector)
    csr_spmm_kernel<true><<<(unsigned)ctas, kWarpsPerCta * 32, 0, s>>>(
        (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
        (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0);
  else
    csr_spmm_kernel<false><<<(unsigned)ctas, kWarpsPerCta * 32, 0, s>>>(
        (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
        (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_csr_validate(const void *row_offsets, int64_t rows, const void *column_indices,
                                 int64_t nnz, int64_t columns, int64_t *where, void *stream) {
  if (rows < 0 || nnz < 0 || !row_offsets || (nnz > 0 && !column_indices))
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_validate: bad arguments");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned long long *flag = nullptr;
  B200_CUDA_TRY(cudaMallocAsync(&flag, sizeof *flag, s));
  B200_CUDA_TRY(cudaMemsetAsync(flag, 0xff, sizeof *flag, s));
  csr_validate_kernel<<<sm_count() * 4, 256, 0, s>>>((const int32_t *)row_offsets, rows,
                                                     (const int32_t *)column_indices, nnz, columns, flag);
  unsigned long long host = 0;
  cudaError_t launch = cudaGetLastError();
  cudaError_t copy = cudaMemcpyAsync(&host, flag, sizeof host, cudaMemcpyDeviceToHost, s);
  cudaError_t sync = cudaStreamSynchronize(s);
  cudaFreeAsync(flag, s);
  B200_CUDA_TRY(launch);
  B200_CUDA_TRY(copy);
  B200_CUDA_TRY(sync);
  if (host != ~0ull) {
    // positions 1..rows name row_offsets entries, later ones name column_indices entries
    const int64_t position = host <= (unsigned long long)rows ? (int64_t)host : (int64_t)host - rows - 1;
    if (where) *where = position;
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_validate: %s[%lld] is out of range",
                host <= (unsigned long long)rows ? "row_offsets" : "column_indices", (long long)position);
  }
  return B200_OK;
}
