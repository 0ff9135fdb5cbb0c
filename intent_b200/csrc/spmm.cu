// CSR SpMM  Y = A . X  (i32 indices, f32 values).
//
// One warp owns one output row at a time and walks over rows in a persistent
// loop.  The 32 lanes cover 128 features with one float4 each, so a gathered
// row of X is one coalesced 512-byte read; column indices and values are
// fetched 32 at a time (coalesced) and broadcast with shuffles.  The kernel is
// bound by memory latency, not bandwidth, so it keeps as many gathers in flight
// as the register file allows: all (up to) 32 gathers of a batch are issued
// before the first is consumed, and the next row's offsets, indices and values
// are requested while they are in flight.  Terms are added strictly in storage
// order with a separately rounded multiply and add, so the result equals a
// sequential left-to-right evaluation bit for bit.  Algorithmic (compulsory) traffic per launch:
// (rows+1)*4 + nnz*8 + columns*F*4 + rows*F*4 bytes; the gathers of X are
// served by L2 where they hit.
#include <mutex>

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

// ---------------------------------------------------------------------------
// Vector path.  The gathers are latency-bound, so they are handed to the copy
// engine instead of being held in registers: lane j of the warp that owns a row
// issues ONE bulk asynchronous copy (cp.async.bulk, global -> shared, 512 bytes
// for 128 features) for the j-th non-zero's row of X; the up-to-32 copies of a
// batch complete on one mbarrier.  Every warp owns kStages staging buffers of
// 32 x 512 bytes and requests batch i+1 while it folds batch i, so an SM keeps
// kWarps x kStages x 16 KB (224 KB) of gathers in flight with no register cost.
// The fold reads the staged rows back in storage order (lane l takes features
// 4l..4l+3, conflict-free) and keeps the separately rounded multiply and add.
// ---------------------------------------------------------------------------
constexpr int kBulkWarps = 7;
constexpr int kBulkStages = 2;
constexpr int kBulkRowBytes = 512;                       // 128 features
constexpr int kBulkStageBytes = 32 * kBulkRowBytes;      // one batch of 32 non-zeros
constexpr size_t kBulkSmemBytes = (size_t)kBulkWarps * kBulkStages * kBulkStageBytes + kBulkWarps * kBulkStages * 8 + 16;
constexpr long long kBulkWaitCycles = 4000000000ll;      // ~2 s: a copy that has not landed by then never will

__device__ int spmm_status[2];  // {sticky flag, row that gave up}

__device__ __forceinline__ uint32_t shared_address(const void *pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

struct Batch {
  int column;     // this lane's column index (lane j <-> j-th non-zero of the batch)
  float value;
  int count;      // non-zeros in the batch (0..32)
};

__global__ void __launch_bounds__(kBulkWarps * 32, 1)
csr_spmm_bulk_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                     const float *__restrict__ values, const float *__restrict__ dense,
                     float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                     int64_t output_pitch) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int feature0 = blockIdx.y * 128;
  const int width = min(128, features - feature0);         // features of this chunk
  const uint32_t row_bytes = (uint32_t)width * 4;
  const bool active = lane * 4 < width;
  unsigned char *stage_base = bulk_smem + (size_t)warp * kBulkStages * kBulkStageBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(bulk_smem + (size_t)kBulkWarps * kBulkStages * kBulkStageBytes) +
                   warp * kBulkStages;
  if (lane == 0) {
    for (int s = 0; s < kBulkStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(shared_address(bars + s)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int64_t warps = (int64_t)gridDim.x * kBulkWarps;
  int64_t row = (int64_t)blockIdx.x * kBulkWarps + warp;
  if (row >= rows) return;
  const float *source = dense + feature0;

  // Requests the gathers of one batch into `stage`; lane j copies non-zero j's row of X.
  auto request = [&](int stage, int base, int stop) -> Batch {
    Batch batch;
    batch.count = max(0, min(32, stop - base));
    batch.column = 0;
    batch.value = 0.0f;
    if (lane < batch.count) {
      batch.column = __ldcs(column_indices + base + lane);
      batch.value = __ldcs(values + base + lane);
    }
    const uint32_t bar = shared_address(bars + stage);
    if (lane == 0 && batch.count > 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(batch.count * row_bytes)
                   : "memory");
    __syncwarp();
    if (lane < batch.count) {
      const float *from = source + (int64_t)batch.column * dense_pitch;
      const uint32_t to = shared_address(stage_base + stage * kBulkStageBytes + lane * kBulkRowBytes);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(to), "l"(from), "r"(row_bytes), "r"(bar)
                   : "memory");
    }
    return batch;
  };

  int start = __ldg(row_offsets + row), stop = __ldg(row_offsets + row + 1);
  int stage = 0;
  uint32_t parity[kBulkStages];
#pragma unroll
  for (int s = 0; s < kBulkStages; ++s) parity[s] = 0;
  int base = start;
  Batch current = request(stage, base, stop);
  bool alive = true;
  while (alive) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    int64_t next_row = row + warps;
    while (true) {
      // what comes after the current batch: the rest of this row, or the first batch of the next row
      const bool more_in_row = base + 32 < stop;
      int following_start = 0, following_stop = 0;
      const bool has_following = more_in_row || next_row < rows;
      if (more_in_row) {
        following_start = base + 32;
        following_stop = stop;
      } else if (next_row < rows) {
        following_start = __ldg(row_offsets + next_row);
        following_stop = __ldg(row_offsets + next_row + 1);
      }
      const int other = (stage + 1) % kBulkStages;
      Batch following;
      following.count = 0; following.column = 0; following.value = 0.0f;
      if (has_following) following = request(other, following_start, following_stop);

      if (current.count > 0) {
        const uint32_t bar = shared_address(bars + stage);
        uint32_t done = 0;
        const long long begin = clock64();
        while (true) {
          asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                       : "=r"(done) : "r"(bar), "r"(parity[stage]) : "memory");
          if (done) break;
          if (clock64() - begin > kBulkWaitCycles) break;
        }
        if (!done) {  // give up: flag the failure, leave the row unwritten and stop this warp
          if (lane == 0 && atomicCAS(&spmm_status[0], 0, 1) == 0) spmm_status[1] = (int)row;
          if (following.count > 0) {  // let the batch already requested land before the buffers go away
            const uint32_t other_bar = shared_address(bars + other);
            const long long drain = clock64();
            uint32_t landed = 0;
            while (!landed && clock64() - drain < kBulkWaitCycles / 8)
              asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                           : "=r"(landed) : "r"(other_bar), "r"(parity[other]) : "memory");
          }
          alive = false;
          break;
        }
        parity[stage] ^= 1;
        const unsigned char *staged = stage_base + stage * kBulkStageBytes + lane * 16;
#pragma unroll 8
        for (int j = 0; j < 32; ++j) {
          const float weight = __shfl_sync(0xffffffffu, current.value, j);
          if (active && j < current.count) {
            const float4 x = *reinterpret_cast<const float4 *>(staged + j * kBulkRowBytes);
            acc.x = __fadd_rn(acc.x, __fmul_rn(weight, x.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(weight, x.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(weight, x.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(weight, x.w));
          }
        }
        __syncwarp();  // every lane has read the stage before it is requested again
      }
      stage = other;
      current = following;
      if (more_in_row) {
        base += 32;
        continue;
      }
      if (active) __stcs(reinterpret_cast<float4 *>(output + row * output_pitch + feature0 + lane * 4), acc);
      if (next_row >= rows) alive = false;
      row = next_row;
      start = following_start;
      stop = following_stop;
      base = start;
      break;
    }
  }
  // No copy is left in flight here on the normal path: every requested batch was waited for.
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
  if (vector) {
    static std::once_flag configured;
    static cudaError_t attribute_error = cudaSuccess;
    std::call_once(configured, [] {
      attribute_error = cudaFuncSetAttribute(csr_spmm_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kBulkSmemBytes);
    });
    B200_CUDA_TRY(attribute_error);
    const int64_t wanted = (rows + kBulkWarps - 1) / kBulkWarps;
    const int64_t resident = sm_count();
    const dim3 grid((unsigned)(wanted < resident ? wanted : resident), (unsigned)((x_d1 + 127) / 128));
    csr_spmm_bulk_kernel<<<grid, kBulkWarps * 32, kBulkSmemBytes, s>>>(
        (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
        (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0);
  } else
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

extern "C" int b200_csr_spmm_status(int64_t *row, void *stream) {
  int words[2] = {0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_CUDA_TRY(cudaMemcpyFromSymbolAsync(words, spmm_status, sizeof words, 0, cudaMemcpyDeviceToHost, s));
  B200_CUDA_TRY(cudaStreamSynchronize(s));
  if (row) *row = words[1];
  if (words[0] != 0) {
    const int zero[2] = {0, 0};
    cudaMemcpyToSymbolAsync(spmm_status, zero, sizeof zero, 0, cudaMemcpyHostToDevice, s);
    return fail(B200_ERR_DEVICE_TIMEOUT, "csr_spmm: a staged gather did not arrive (row %d left unwritten)", words[1]);
  }
  return B200_OK;
}
