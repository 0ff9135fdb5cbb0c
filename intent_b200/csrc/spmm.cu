// CSR SpMM  Y = A . X  (i32 indices, f32 values).
//
// One warp owns one output row; its 32 lanes cover 128 features with one float4
// each, so a gathered row of X is one coalesced 512-byte read.  Column indices
// and values are fetched 32 at a time (coalesced) and broadcast with shuffles.
// Terms are added strictly in storage order with a separately rounded multiply
// and add, so the result equals a sequential left-to-right evaluation bit for
// bit.  Three kernels share that scheme:
//   csr_spmm_bulk_kernel   X fits L2 (one launch): gathers are staged through
//                          shared memory by the copy engine (cp.async.bulk),
//                          224 KB in flight per SM, software-pipelined rows
//   csr_spmm_block_kernel  X larger than L2: the call is cut into column blocks,
//                          one launch each, accumulating into Y; gathers in
//                          registers, many warps
//   csr_spmm_kernel        any feature count / alignment (scalar fallback)
// Algorithmic (compulsory) traffic per call: (rows+1)*4 + nnz*8 + columns*F*4 +
// rows*F*4 bytes; the gathers touch nnz*F*4 bytes and are served by L2 where they hit.
#include <stdlib.h>

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


// Column-blocked execution.  X (columns x F x 4 bytes) is larger than L2 for the
// benchmark shape, and random 512-byte gathers that miss L2 run at a fraction of
// HBM's streaming rate.  So one call is split into launches that each cover a
// block of columns small enough to (mostly) stay in L2: launch p adds the terms whose
// column lies in block p to Y (read-modify-write, streamed).  With ascending
// columns inside every row the blocks are visited in storage order, so the sum
// of a row is still accumulated strictly left to right.  Launch 0 reads every
// column index anyway, so it also checks that rows ascend and clears `spmm_sorted`
// if one does not; launch 1 then recomputes Y from scratch over all columns (in
// storage order) and the remaining launches return at once.
__device__ int spmm_sorted;

__global__ void spmm_assume_sorted_kernel() { spmm_sorted = 1; }


__global__ void __launch_bounds__(kBulkWarps * 32, 1)
csr_spmm_bulk_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                     const float *__restrict__ values, const float *__restrict__ dense,
                     float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                     int64_t output_pitch, int column_lo, int column_hi, int phase, int phases) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const bool accumulate = phase > 0;
  if (phases > 1 && !spmm_sorted) {  // some row is not ascending: do everything in launch 0
    if (phase > 0) return;
    column_lo = INT32_MIN;
    column_hi = INT32_MAX;
  }
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

  // This warp's rows are first_row, first_row + warps, ...; `count` of them.
  const int64_t warps = (int64_t)gridDim.x * kBulkWarps;
  const int64_t first_row = (int64_t)blockIdx.x * kBulkWarps + warp;
  if (first_row >= rows) return;
  const int64_t count = (rows - first_row + warps - 1) / warps;
  const float *source = dense + feature0;

  // A batch is up to 32 consecutive non-zeros of one row.  The walk over batches is a
  // three-deep software pipeline, so no memory round trip sits on the critical path:
  //   offsets   of 32 of this warp's rows at a time (lane k holds the k-th of them),
  //   indices   (column, value) of the batch after the next one,
  //   copies    of the next batch, while the current one is folded.
  struct Cursor {
    int64_t ordinal;   // which of this warp's rows
    int base, stop;    // batch = non-zeros [base, min(base + 32, stop))
  };
  int cached_start = 0, cached_stop = 0;  // lane k: offsets of row ordinal (cache_block * 32 + k)
  int64_t cache_block = -1;
  auto offsets_of = [&](int64_t ordinal, int *start, int *stop) {
    if (ordinal / 32 != cache_block) {
      cache_block = ordinal / 32;
      const int64_t mine = cache_block * 32 + lane;
      cached_start = cached_stop = 0;
      if (mine < count) {
        const int64_t r = first_row + mine * warps;
        cached_start = __ldg(row_offsets + r);
        cached_stop = __ldg(row_offsets + r + 1);
      }
    }
    *start = __shfl_sync(0xffffffffu, cached_start, (int)(ordinal % 32));
    *stop = __shfl_sync(0xffffffffu, cached_stop, (int)(ordinal % 32));
  };
  struct Batch {
    int column;        // lane j <-> j-th non-zero of the batch
    float value;
    int64_t row;       // -1: no batch (past the end)
    int base, stop;
    bool first, last;  // first / last batch of its row
  };
  auto advance = [&](Cursor &c) -> bool {   // false when the warp's rows are exhausted
    if (c.base + 32 < c.stop) { c.base += 32; return true; }
    if (++c.ordinal >= count) return false;
    offsets_of(c.ordinal, &c.base, &c.stop);
    return true;
  };
  auto fetch = [&](const Cursor &c, bool valid, bool first) -> Batch {
    Batch b;
    b.row = valid ? first_row + c.ordinal * warps : -1;
    b.base = c.base; b.stop = c.stop; b.first = first; b.last = c.base + 32 >= c.stop;
    b.column = 0; b.value = 0.0f;
    if (valid && c.base + lane < c.stop) {
      b.column = __ldcs(column_indices + c.base + lane);
      b.value = __ldcs(values + c.base + lane);
    }
    return b;
  };
  // Requests the gathers of one batch into `stage`; returns the lanes that take part.
  auto request = [&](const Batch &b, int stage) -> unsigned {
    const bool mine = b.row >= 0 && b.base + lane < b.stop && b.column >= column_lo && b.column < column_hi;
    const unsigned mask = __ballot_sync(0xffffffffu, mine);
    const uint32_t bar = shared_address(bars + stage);
    if (lane == 0 && mask != 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(__popc(mask) * row_bytes)
                   : "memory");
    __syncwarp();
    if (mine) {
      const float *from = source + (int64_t)b.column * dense_pitch;
      const uint32_t to = shared_address(stage_base + stage * kBulkStageBytes + lane * kBulkRowBytes);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(to), "l"(from), "r"(row_bytes), "r"(bar)
                   : "memory");
    }
    return mask;
  };
  auto try_wait = [&](int stage, uint32_t parity) -> bool {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(shared_address(bars + stage)), "r"(parity) : "memory");
    return done != 0;
  };

  Cursor cursor{0, 0, 0};
  offsets_of(0, &cursor.base, &cursor.stop);
  Batch current = fetch(cursor, true, true);
  bool more = true;
  bool crossed;
  { const int64_t before = cursor.ordinal; more = advance(cursor); crossed = cursor.ordinal != before; }
  Batch next = fetch(cursor, more, crossed);
  uint32_t parity0 = 0, parity1 = 0;
  int stage = 0;
  unsigned current_mask = request(current, stage);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  while (current.row >= 0) {
    // indices of the batch after next, then the copies of the next batch
    Batch after;
    {
      const int64_t before = cursor.ordinal;
      if (more) more = advance(cursor);
      after = fetch(cursor, more, cursor.ordinal != before);
    }
    const unsigned next_mask = request(next, stage ^ 1);

    if (current.first) {
      acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (accumulate && active)  // partial sums of the earlier column blocks
        acc = __ldcs(reinterpret_cast<const float4 *>(output + current.row * output_pitch + feature0 + lane * 4));
    }
    if (current_mask != 0) {
      const uint32_t parity = stage ? parity1 : parity0;
      const long long begin = clock64();
      bool landed = try_wait(stage, parity);
      while (!landed && clock64() - begin < kBulkWaitCycles) landed = try_wait(stage, parity);
      if (!landed) {  // give up: flag the failure, leave the row unwritten and stop this warp
        if (lane == 0 && atomicCAS(&spmm_status[0], 0, 1) == 0) spmm_status[1] = (int)current.row;
        if (next_mask != 0) {  // let the batch already requested land before the buffers go away
          const long long drain = clock64();
          const uint32_t other_parity = stage ? parity0 : parity1;
          while (!try_wait(stage ^ 1, other_parity) && clock64() - drain < kBulkWaitCycles / 8) {}
        }
        return;
      }
      if (stage) parity1 ^= 1; else parity0 ^= 1;
      const unsigned char *staged = stage_base + stage * kBulkStageBytes + lane * 16;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) {
        const float weight = __shfl_sync(0xffffffffu, current.value, j);
        if (active && ((current_mask >> j) & 1u)) {
          const float4 x = *reinterpret_cast<const float4 *>(staged + j * kBulkRowBytes);
          acc.x = __fadd_rn(acc.x, __fmul_rn(weight, x.x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(weight, x.y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(weight, x.z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(weight, x.w));
        }
      }
      __syncwarp();  // every lane has read the stage before it is requested again
    }
    if (current.last && active)
      __stcs(reinterpret_cast<float4 *>(output + current.row * output_pitch + feature0 + lane * 4), acc);
    stage ^= 1;
    current = next;
    current_mask = next_mask;
    next = after;
  }
  // No copy is left in flight here: every requested batch was waited for.
}

// Column-blocked launches see only a few non-zeros per row and mostly hit L2, where
// round trips are short: there the gathers are kept in registers (eight in flight per
// lane) and rows are spread over many warps instead of being staged through shared memory.
constexpr int kBlockWarps = 8;

__global__ void __launch_bounds__(kBlockWarps * 32)
csr_spmm_block_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                      const float *__restrict__ values, const float *__restrict__ dense,
                      float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                      int64_t output_pitch, int column_lo, int column_hi, int phase) {
  bool accumulate = phase > 0;
  if (phase > 0 && !spmm_sorted) {  // launch 0 met a row that does not ascend
    if (phase > 1) return;
    column_lo = INT32_MIN;          // launch 1 redoes the whole product in storage order
    column_hi = INT32_MAX;
    accumulate = false;
  }
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kBlockWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int feature = blockIdx.y * 128 + lane * 4;
  const bool active = feature < features;
  const int start = __ldg(row_offsets + row), stop = __ldg(row_offsets + row + 1);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float *destination = output + row * output_pitch + feature;
  if (accumulate && active) acc = __ldcs(reinterpret_cast<const float4 *>(destination));
  const float *source = dense + feature;
  bool touched = !accumulate;  // a launch that starts from zero always writes
  int previous = INT32_MIN;    // last column of the batch before (ascending check of launch 0)
  for (int base = start; base < stop; base += 32) {
    int column = 0;
    float value = 0.0f;
    bool mine = false;
    if (base + lane < stop) {
      column = __ldcs(column_indices + base + lane);
      value = __ldcs(values + base + lane);
      mine = column >= column_lo && column < column_hi;
    }
    if (phase == 0) {
      const int before = __shfl_up_sync(0xffffffffu, column, 1);
      const bool descends = base + lane < stop && column < (lane == 0 ? previous : before);
      if (__any_sync(0xffffffffu, descends) && lane == 0) spmm_sorted = 0;
      previous = __shfl_sync(0xffffffffu, column, 31);
    }
    unsigned mask = __ballot_sync(0xffffffffu, mine);
    touched |= mask != 0;
    while (mask != 0) {  // eight gathers at a time, in storage order
      int lanes[8];
      float4 gathered[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        lanes[u] = mask ? __ffs(mask) - 1 : -1;
        if (mask) mask &= mask - 1;
        const int c = __shfl_sync(0xffffffffu, column, lanes[u] < 0 ? 0 : lanes[u]);
        if (active && lanes[u] >= 0)
          gathered[u] = __ldg(reinterpret_cast<const float4 *>(source + (int64_t)c * dense_pitch));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float weight = __shfl_sync(0xffffffffu, value, lanes[u] < 0 ? 0 : lanes[u]);
        if (active && lanes[u] >= 0) {
          acc.x = __fadd_rn(acc.x, __fmul_rn(weight, gathered[u].x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(weight, gathered[u].y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(weight, gathered[u].z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(weight, gathered[u].w));
        }
      }
    }
  }
  if (active && touched) __stcs(reinterpret_cast<float4 *>(destination), acc);
}

// CSR SpMV  y = A . x  (csr_spmm with a single feature).  A warp takes kSpmvRows consecutive rows.
// Batch by batch (32 stored elements of every row): the indices and values of all its rows are
// requested before any is used, then all the gathers, and the products (separately rounded) are
// staged in shared memory; then lane r adds row r's products to its carry one by one in storage
// order, so every sum is the sequential left-to-right one and costs one shared-memory read and
// one add per element for 16 rows at a time, not a shuffle per element per row.
constexpr int kSpmvRows = 16, kSpmvWarps = 4;

__global__ void __launch_bounds__(kSpmvWarps * 32)
csr_spmv_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                const float *__restrict__ values, const float *__restrict__ vector, float *__restrict__ output,
                int64_t rows, int64_t vector_stride, int64_t output_stride) {
  __shared__ float staged[kSpmvWarps][kSpmvRows][33];            // 33: lane r walks row r without bank conflicts
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row0 = ((int64_t)blockIdx.x * kSpmvWarps + warp) * kSpmvRows;
  if (row0 >= rows) return;                                      // whole warps leave; no CTA barrier below
  const int here = (int)min((int64_t)kSpmvRows, rows - row0);
  const int offset = lane <= here ? __ldg(row_offsets + row0 + lane) : 0;
  const int next_offset = __shfl_down_sync(0xffffffffu, offset, 1);
  const int length = lane < here ? next_offset - offset : 0;      // of row `lane`
  int longest = length;
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, step));
  float acc = 0.0f;
  for (int base = 0; base < longest; base += 32) {
    int column[kSpmvRows];
    float value[kSpmvRows];
#pragma unroll
    for (int r = 0; r < kSpmvRows; ++r) {
      const int at = __shfl_sync(0xffffffffu, offset, r) + base + lane, stop = __shfl_sync(0xffffffffu, offset, r + 1);
      const bool stored = r < here && at < stop;
      column[r] = stored ? __ldcs(column_indices + at) : -1;
      value[r] = stored ? __ldcs(values + at) : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < kSpmvRows; ++r)
      staged[warp][r][lane] = column[r] >= 0 ? __fmul_rn(value[r], __ldg(vector + (int64_t)column[r] * vector_stride)) : 0.0f;
    __syncwarp();
    const int count = min(32, length - base);                    // <= 0 once this lane's row is finished
#pragma unroll 8
    for (int j = 0; j < count; ++j) acc = __fadd_rn(acc, staged[warp][lane & (kSpmvRows - 1)][j]);
    __syncwarp();
  }
  if (lane < here) output[(row0 + lane) * output_stride] = acc;
}

// Number of column blocks: X is cut into slices of at most kBlockBytes so that a slice
// stays resident in L2 (126 MB, shared with the streamed index, value and Y traffic).
constexpr int64_t kBlockBytes = 72ll << 20;
int column_phases(int64_t columns, int64_t features) {
  static const int forced = [] {
    const char *text = getenv("INTENT_B200_SPMM_PHASES");  // tuning override, 1..16
    const int value = text ? atoi(text) : 0;
    return value >= 1 && value <= 16 ? value : 0;
  }();
  if (forced) return forced;
  const int64_t bytes = columns * features * 4;
  const int64_t phases = (bytes + kBlockBytes - 1) / kBlockBytes;
  return (int)(phases < 1 ? 1 : phases > 8 ? 8 : phases);
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
    const int phases = column_phases(x_d0, x_d1);
    if (phases > 1) spmm_assume_sorted_kernel<<<1, 1, 0, s>>>();
    const int64_t block = (x_d0 + phases - 1) / phases;
    const dim3 block_grid((unsigned)((rows + kBlockWarps - 1) / kBlockWarps), grid.y);
    for (int phase = 0; phase < phases; ++phase) {
      const int64_t lo = phase * block, hi = (phase + 1 == phases) ? (int64_t)INT32_MAX : (phase + 1) * block;
      if (phases > 1) {
        csr_spmm_block_kernel<<<block_grid, kBlockWarps * 32, 0, s>>>(
            (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
            (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0, (int)lo, (int)hi, phase);
        continue;
      }
      csr_spmm_bulk_kernel<<<grid, kBulkWarps * 32, kBulkSmemBytes, s>>>(
          (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
          (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0,
          phases > 1 ? (int)lo : INT32_MIN, phases > 1 ? (int)hi : INT32_MAX, phase, phases);
    }
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

extern "C" int b200_csr_spmv(const void *row_offsets, int64_t ro_d0, int64_t ro_s0,
                             const void *column_indices, int64_t ci_d0, int64_t ci_s0,
                             const void *values, int64_t va_d0, int64_t va_s0,
                             const void *vector, int64_t x_d0, int64_t x_s0,
                             void *output, int64_t y_d0, int64_t y_s0, void *stream) {
  const int64_t rows = ro_d0 - 1;
  if (ro_d0 < 1 || ci_d0 < 0 || va_d0 != ci_d0 || x_d0 < 0 || y_d0 != rows)
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmv: inconsistent extents");
  if (rows == 0) return B200_OK;
  if (!row_offsets || !output || (ci_d0 > 0 && (!column_indices || !values || !vector)))
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmv: null buffer");
  if ((ro_d0 > 1 && ro_s0 != 1) || (ci_d0 > 1 && (ci_s0 != 1 || va_s0 != 1)))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmv: index/value arrays must be contiguous");
  if (ci_d0 > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmv: i32 index space exceeded");
  const int64_t ctas = (rows + kSpmvWarps * kSpmvRows - 1) / (kSpmvWarps * kSpmvRows);
  if (ctas > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmv: too many rows");
  csr_spmv_kernel<<<(unsigned)ctas, kSpmvWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values, (const float *)vector,
      (float *)output, rows, x_s0, y_s0);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
