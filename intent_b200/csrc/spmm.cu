// CSR SpMM  Y = A . X  (i32 indices, f32 values).
//
// One warp owns one output row at a time; its 32 lanes cover 128 features with one float4
// each, so a gathered row of X is one coalesced 512-byte read.  Terms are added strictly in
// storage order with a separately rounded multiply and add, so the result equals a sequential
// left-to-right evaluation bit for bit.  Kernels:
//   csr_spmm_rows_kernel    16-byte aligned rows: persistent warps, one row ahead, the selected
//                           terms of a row compacted in shared memory; an X larger than L2 is
//                           processed in column blocks, one launch each, accumulating into Y
//   csr_spmm_scalar_kernel  any feature count / alignment
//   csr_spmv_kernel         a single feature
//   gather_probe_kernel     measures the gather rate that bounds the above on this device
// Algorithmic (compulsory) traffic per call: (rows+1)*4 + nnz*8 + columns*F*4 +
// rows*F*4 bytes; the gathers touch nnz*F*4 bytes and are served by L2 where they hit.
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kGatherDepth = 8;  // independent X-row loads in flight per lane

// Any feature count / alignment: scalar lanes, 32 features at a time.
__global__ void __launch_bounds__(kWarpsPerCta * 32)
csr_spmm_scalar_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                       const float *__restrict__ values, const float *__restrict__ dense,
                       float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                       int64_t output_pitch) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int start = row_offsets[row];
  const int stop = row_offsets[row + 1];
  for (int feature0 = 0; feature0 < features; feature0 += 32) {
    const int feature = feature0 + lane;
    const bool active = feature < features;
    float acc = 0.0f;
    for (int base = start; base < stop; base += 32) {
      const int count = min(32, stop - base);
      int my_column = 0;
      float my_value = 0.0f;
      if (lane < count) {
        my_column = __ldcs(column_indices + base + lane);
        my_value = __ldcs(values + base + lane);
      }
      for (int j0 = 0; j0 < count; j0 += kGatherDepth) {
        float gathered[kGatherDepth];
        float weight[kGatherDepth];
#pragma unroll
        for (int j = 0; j < kGatherDepth; ++j) {
          // lanes past `count` hold column 0 / value 0 and are skipped below
          const int column = __shfl_sync(0xffffffffu, my_column, (j0 + j) & 31);
          weight[j] = __shfl_sync(0xffffffffu, my_value, (j0 + j) & 31);
          if (active && j0 + j < count) gathered[j] = __ldg(dense + (int64_t)column * dense_pitch + feature);
        }
#pragma unroll
        for (int j = 0; j < kGatherDepth; ++j)
          if (active && j0 + j < count) acc = __fadd_rn(acc, __fmul_rn(weight[j], gathered[j]));
      }
    }
    if (active) output[row * output_pitch + feature] = acc;
  }
}

// ---- per-call state and L2 eviction priorities --------------------------------
// Word of the caller's int32 workspace (one workspace per prepared call, zeroed once by the
// caller) that carries "every row seen so far ascends" from the first launch of a call, which
// sets it and clears it on meeting a descending row, to the later launches of the same call.
// Nothing of a call lives in library-global device memory, so calls on different streams
// cannot see one another's flag.  (Words 0 and 1 are the status report b200_workspace_status
// reads: this operator has no bounded wait and writes them only in the checked build, as
// {2, row} when it met an offset or a column outside its array.)
constexpr int kStateSorted = 2;

__global__ void spmm_begin_kernel(int *state) { state[kStateSorted] = 1; }

// X is gathered about 32 times per element while the index, value and Y streams are touched
// once: gathers ask L2 to keep their lines (evict_last) and skip L1, where they are never reused.
__device__ __forceinline__ uint64_t policy_keep() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ float4 load_keep(const float *address, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(address), "l"(policy));
  return v;
}

// ---------------------------------------------------------------------------
// Column-blocked execution.  X (columns x F x 4 bytes) is larger than L2 for the
// benchmark shape, and random 512-byte gathers that miss L2 run at a fraction of
// HBM's streaming rate.  So one call is split into launches that each cover a
// block of columns small enough to stay in L2: launch p adds the terms whose
// column lies in block p to Y (read-modify-write, streamed).  With ascending
// columns inside every row the blocks are visited in storage order, so the sum
// of a row is still accumulated strictly left to right.  Launch 0 reads every
// column index anyway, so it also checks that rows ascend and clears the call's
// "sorted" word if one does not; launch 1 then recomputes Y from scratch over
// all columns (in storage order) and the remaining launches return at once.
// ---------------------------------------------------------------------------
struct Block {
  int lo, hi;        // columns of this launch: [lo, hi)
  bool accumulate;   // start from the partial sums already in Y
  bool skip;         // nothing left to do in this launch
};

__device__ __forceinline__ Block block_of_launch(const int *state, int column_lo, int column_hi, int phase) {
  Block b{column_lo, column_hi, phase > 0, false};
  if (phase > 0 && !state[kStateSorted]) {  // launch 0 met a row that does not ascend
    b.skip = phase > 1;
    b.lo = INT32_MIN;                       // launch 1 redoes the whole product in storage order
    b.hi = INT32_MAX;
    b.accumulate = false;
  }
  return b;
}

// ---------------------------------------------------------------------------
// Persistent rows kernel.  What the profiler showed of a one-row-per-warp kernel with eight
// gathers in flight per lane: the issue slots 66 % busy at 40 % occupancy, about 42 instructions
// per gathered row of X, most of them spent finding the next selected non-zero (ballot,
// find-first-set, two shuffles), on top of the offsets -> indices -> gathers chain.  Here
//   * a warp owns rows w, w + W, w + 2W, ...; while it gathers for one row, the indices and
//     values of the next row and the next row's partial sums are already requested, and row
//     offsets are fetched 32 rows at a time, so the only round trips it waits for are gathers;
//   * the non-zeros of a batch that fall into the launch's column block are compacted into
//     shared memory once (offset of the X row in 16-byte units, value); the inner loop reads
//     one broadcast pair per term, forms the address with one multiply-add and issues the load:
//     about 15 instructions per gathered row, eight of them the unfused multiply and add;
//   * gathers are issued kWindow at a time and the adds stay in storage order.  Measured on the
//     262144 x 262144 / 32 per row / 128 feature case (two column blocks): windows of 2 and 4
//     with four CTAs per SM take 365-380 us, windows of 8, 12, 16 take 450-700 us whatever the
//     occupancy, and more than four CTAs per SM (fewer registers) is slower again.
// ---------------------------------------------------------------------------
constexpr int kRowsWarps = 8;
constexpr int kRowsCtas = 4;    // CTAs per SM the kernel is compiled for (64 registers per thread)
constexpr int kWindow = 4;      // gathers a lane issues before it folds them

template <bool ACCUMULATE>
__global__ void __launch_bounds__(kRowsWarps * 32, kRowsCtas)
csr_spmm_rows_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                     const float *__restrict__ values, const float *__restrict__ dense,
                     float *__restrict__ output, int rows, int features, uint32_t dense_pitch16,
                     uint32_t output_pitch16, int column_lo, int column_hi, int phase, int *state, int columns,
                     int stored_elements) {
  struct __align__(8) Term { uint32_t offset; float value; };   // offset of the X row in 16-byte units
  __shared__ Term terms[kRowsWarps][32];
  // ACCUMULATE is false only for launch 0, which never reads partial sums; a later launch decides here
  // whether it accumulates its block or redoes the product (see block_of_launch).
  const bool check_order = phase == 0 && (column_lo != INT32_MIN || column_hi != INT32_MAX);
  bool accumulate = ACCUMULATE;
  if (ACCUMULATE) {
    const Block block = block_of_launch(state, column_lo, column_hi, phase);
    if (block.skip) return;
    column_lo = block.lo; column_hi = block.hi; accumulate = block.accumulate;
  }
  const uint64_t keep = policy_keep();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int stride = gridDim.x * kRowsWarps;
  int row = blockIdx.x * kRowsWarps + warp;
  if (row >= rows) return;
  const int feature16 = blockIdx.y * 32 + lane;                 // this lane's 16-byte piece of a row
  const bool active = feature16 * 4 < features;
  const float4 *source = reinterpret_cast<const float4 *>(dense) + (active ? feature16 : 0);
  float4 *result = reinterpret_cast<float4 *>(output) + (active ? feature16 : 0);
  const unsigned below = (1u << lane) - 1u;
  Term *mine_terms = terms[warp];

#ifdef B200_CHECKED
  auto index_of = [&](int at) { return at >= 0 && at < stored_elements ? __ldcs(column_indices + at) : -1; };
  auto value_of = [&](int at) { return at >= 0 && at < stored_elements ? __ldcs(values + at) : 0.0f; };
#else
  auto index_of = [&](int at) { return __ldcs(column_indices + at); };
  auto value_of = [&](int at) { return __ldcs(values + at); };
#endif
  auto partial_of = [&](int r) { return __ldcs(result + (uint64_t)r * output_pitch16); };
  const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);

  // Offsets of 32 of this warp's rows at a time: lane k holds those of the k-th row from `cached`.
  int cached = row, cached_start = 0, cached_stop = 0;
  auto refill = [&](int first) {
    cached = first;
    const int64_t mine = (int64_t)first + (int64_t)lane * stride;
    cached_start = cached_stop = 0;
    if (mine < rows) { cached_start = __ldg(row_offsets + mine); cached_stop = __ldg(row_offsets + mine + 1); }
  };
  refill(row);
  int start = __shfl_sync(0xffffffffu, cached_start, 0), stop = __shfl_sync(0xffffffffu, cached_stop, 0);
  int column = 0, next_column = 0;
  float value = 0.0f, next_value = 0.0f;
  if (start + lane < stop) { column = index_of(start + lane); value = value_of(start + lane); }
  float4 acc = ACCUMULATE && accumulate && active ? partial_of(row) : zero, next_acc = zero;
  int ordinal = 0;                                   // of `row` within the cached block of 32

  for (; row < rows; row += stride) {
    // requests for the next row, before this row's gathers
    int next_start = 0, next_stop = 0;
    const int64_t next_row = (int64_t)row + stride;
    if (next_row < rows) {
      if (++ordinal == 32) { refill((int)next_row); ordinal = 0; }
      next_start = __shfl_sync(0xffffffffu, cached_start, ordinal);
      next_stop = __shfl_sync(0xffffffffu, cached_stop, ordinal);
      next_column = 0; next_value = 0.0f;
      if (next_start + lane < next_stop) { next_column = index_of(next_start + lane); next_value = value_of(next_start + lane); }
      if (ACCUMULATE && accumulate && active) next_acc = partial_of((int)next_row);
    }
    bool touched = !accumulate;        // a launch that starts from zero always writes
    int previous = INT32_MIN;          // last column of the batch before (ascending check of launch 0)
    for (int base = start; base < stop; base += 32) {
      if (base != start) {             // rows longer than one batch fetch their later batches in place
        column = 0; value = 0.0f;
        if (base + lane < stop) { column = index_of(base + lane); value = value_of(base + lane); }
      }
      bool stored = base + lane < stop;
#ifdef B200_CHECKED
      // Checked build: the kernel trusts the CSR arrays (the definition's assume_in_bounds); here an
      // offset or a column outside its array is recorded in the workspace ({2, row}) and the term is
      // dropped instead of being loaded, so a corrupted matrix ends as an error status, not a fault.
      const bool bad = stored && (base + lane >= stored_elements || column < 0 || column >= columns);
      if (__any_sync(0xffffffffu, bad || stop < start) && lane == 0 && atomicCAS(&state[0], 0, 2) == 0) state[1] = row;
      stored = stored && !bad && stop >= start;
#endif
      if (check_order) {
        const int before = __shfl_up_sync(0xffffffffu, column, 1);
        const bool descends = stored && column < (lane == 0 ? previous : before);
        if (__any_sync(0xffffffffu, descends) && lane == 0) state[kStateSorted] = 0;
        previous = __shfl_sync(0xffffffffu, column, 31);
      }
      const bool selected = stored && column >= column_lo && column < column_hi;
      const unsigned mask = __ballot_sync(0xffffffffu, selected);
      if (mask == 0) continue;
      touched = true;
      if (selected) mine_terms[__popc(mask & below)] = Term{(uint32_t)column * dense_pitch16, value};
      __syncwarp();
      const int count = __popc(mask);
      int j = 0;
      for (; j + kWindow <= count; j += kWindow) {   // full windows: no per-term predicate
        float4 x[kWindow];
#pragma unroll
        for (int u = 0; u < kWindow; ++u) {
          const float4 *from = source + mine_terms[j + u].offset;
          x[u] = load_keep(reinterpret_cast<const float *>(from), keep);
        }
#pragma unroll
        for (int u = 0; u < kWindow; ++u) {
          const float weight = mine_terms[j + u].value;
          acc.x = __fadd_rn(acc.x, __fmul_rn(weight, x[u].x));
          acc.y = __fadd_rn(acc.y, __fmul_rn(weight, x[u].y));
          acc.z = __fadd_rn(acc.z, __fmul_rn(weight, x[u].z));
          acc.w = __fadd_rn(acc.w, __fmul_rn(weight, x[u].w));
        }
      }
      if (j < count) {                                // the last, partial window
        float4 x[kWindow];
#pragma unroll
        for (int u = 0; u < kWindow; ++u) {
          if (j + u < count) {
            const float4 *from = source + mine_terms[j + u].offset;
            x[u] = load_keep(reinterpret_cast<const float *>(from), keep);
          }
        }
#pragma unroll
        for (int u = 0; u < kWindow; ++u) {
          if (j + u < count) {
            const float weight = mine_terms[j + u].value;
            acc.x = __fadd_rn(acc.x, __fmul_rn(weight, x[u].x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(weight, x[u].y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(weight, x[u].z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(weight, x[u].w));
          }
        }
      }
      __syncwarp();                                   // every lane has read the terms before the next batch overwrites them
    }
    if (active && touched) {
      float4 *destination = result + (uint64_t)row * output_pitch16;
      __stcs(destination, acc);
    }
    start = next_start; stop = next_stop;
    column = next_column; value = next_value;
    acc = next_acc;
  }
}

// ---------------------------------------------------------------------------
// Gather-rate probe: the ceiling the SpMM gathers can reach on this device.  Every warp reads
// `per_warp` rows of 512 bytes at pseudo-random positions of `table` (a multiplicative walk
// over the row index, so neighbouring warps touch unrelated rows) with DEPTH loads in flight
// per lane, and folds them into one float4 that is written at the end so the loads are kept.
// With a table that fits L2 this measures the L2-to-SM gather rate; with a larger one, the
// mix of hits and DRAM misses a single pass over X sees.
// ---------------------------------------------------------------------------
template <int DEPTH, bool HINTS>
__global__ void __launch_bounds__(256)
gather_probe_kernel(const float *__restrict__ table, int64_t table_rows, int64_t per_warp, float *__restrict__ sink) {
  const uint64_t keep = policy_keep();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  uint32_t position = (uint32_t)(warp + 1) * 2654435761u;
  const float4 *source = reinterpret_cast<const float4 *>(table) + lane;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int64_t done = 0; done < per_warp; done += DEPTH) {
    float4 got[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      position = position * 1664525u + 1013904223u;
      const uint32_t row = __umulhi(position, (uint32_t)table_rows);   // uniform in [0, table_rows)
      const float4 *from = source + row * 32u;
      got[d] = HINTS ? load_keep(reinterpret_cast<const float *>(from), keep) : __ldg(from);
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) { acc.x += got[d].x; acc.y += got[d].y; acc.z += got[d].z; acc.w += got[d].w; }
  }
  if (acc.x == 12345.678f) sink[warp * 128 + lane * 4] = acc.y + acc.z + acc.w;  // never true in practice
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
// CTAs of `kernel` one SM holds (registers decide), per device and kernel.
int resident_blocks(const void *kernel, int threads) {
  static std::mutex lock;
  static std::map<std::pair<const void *, int>, int> known;
  int device = 0;
  cudaGetDevice(&device);
  std::lock_guard<std::mutex> guard(lock);
  auto found = known.find({kernel, device});
  if (found != known.end()) return found->second;
  int blocks = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, threads, 0) != cudaSuccess || blocks < 1) blocks = 1;
  known[{kernel, device}] = blocks;
  return blocks;
}

// INTENT_B200_SPMM_PHASES (1..16) overrides the number of column blocks; it is read at every
// call so that one process can sweep it (and tests can force the blocked path on small inputs).
int tuning_integer(const char *name, int low, int high, int otherwise) {
  const char *text = getenv(name);
  const int value = text ? atoi(text) : otherwise;
  return text && value >= low && value <= high ? value : otherwise;
}

int column_phases(int64_t columns, int64_t features) {
  const int forced = tuning_integer("INTENT_B200_SPMM_PHASES", 1, 16, 0);
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
                             void *workspace, int64_t ws_d0, int64_t ws_s0,
                             void *stream) {
  const int64_t rows = ro_d0 - 1;
  if (ro_d0 < 1 || ci_d0 < 0 || va_d0 != ci_d0 || x_d0 < 0 || x_d1 < 0 || y_d0 != rows || y_d1 != x_d1)
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm: inconsistent extents");
  if (!workspace || ws_d0 < B200_WORKSPACE_WORDS || (ws_d0 > 1 && ws_s0 != 1))
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm: workspace must hold %d contiguous int32 words", B200_WORKSPACE_WORDS);
  if (rows == 0 || x_d1 == 0) return B200_OK;
  if (!row_offsets || !output || (ci_d0 > 0 && (!column_indices || !values || !dense)))
    return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm: null buffer");
  if ((ro_d0 > 1 && ro_s0 != 1) || (ci_d0 > 1 && (ci_s0 != 1 || va_s0 != 1)) ||
      (x_d1 > 1 && (x_s1 != 1 || y_s1 != 1)) || x_s0 < 0 || y_s0 < 0)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: index/value arrays must be contiguous and X, Y unit-stride in features");
  if (x_d1 > INT32_MAX || ci_d0 > INT32_MAX)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: i32 index space exceeded");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int *state = static_cast<int *>(workspace);
  const int64_t ctas = (rows + kWarpsPerCta - 1) / kWarpsPerCta;
  if (ctas > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "csr_spmm: too many rows");
  // vector path: 16-byte aligned rows whose offsets (in 16-byte units) fit 32 bits
  const bool vector = x_d1 % 4 == 0 && x_s0 % 4 == 0 && y_s0 % 4 == 0 && aligned16(dense) && aligned16(output) &&
                      (x_d0 == 0 || (x_d0 - 1) * (x_s0 / 4) + (x_d1 + 3) / 4 <= (int64_t)UINT32_MAX) &&
                      x_s0 / 4 <= (int64_t)UINT32_MAX && y_s0 / 4 <= (int64_t)UINT32_MAX && rows <= INT32_MAX - 64 * 1024 * 1024;
  if (!vector) {
    csr_spmm_scalar_kernel<<<(unsigned)ctas, kWarpsPerCta * 32, 0, s>>>(
        (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
        (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  const int phases = column_phases(x_d0, x_d1);
  const unsigned chunks = (unsigned)((x_d1 + 127) / 128);
  if (phases > 1) spmm_begin_kernel<<<1, 1, 0, s>>>(state);
  const int64_t span = (x_d0 + phases - 1) / phases;
  for (int phase = 0; phase < phases; ++phase) {
    const int lo = phases > 1 ? (int)(phase * span) : INT32_MIN;
    const int hi = phases > 1 && phase + 1 < phases ? (int)((phase + 1) * span) : INT32_MAX;
    auto launch = [&](auto kernel) {
      const int per_sm = resident_blocks(reinterpret_cast<const void *>(kernel), kRowsWarps * 32);
      const int64_t wanted = (rows + kRowsWarps - 1) / kRowsWarps, resident = (int64_t)sm_count() * per_sm;
      const dim3 grid((unsigned)(wanted < resident ? wanted : resident), chunks);
      kernel<<<grid, kRowsWarps * 32, 0, s>>>((const int32_t *)row_offsets, (const int32_t *)column_indices,
                                               (const float *)values, (const float *)dense, (float *)output, (int)rows,
                                               (int)x_d1, (uint32_t)(x_s0 / 4), (uint32_t)(y_s0 / 4), lo, hi, phase, state,
                                               (int)(x_d0 > INT32_MAX ? INT32_MAX : x_d0), (int)ci_d0);
    };
    if (phase == 0) launch(csr_spmm_rows_kernel<false>);
    else launch(csr_spmm_rows_kernel<true>);
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// Gather-rate probe (see gather_probe_kernel).  `variant`: 0..3 = 4, 8, 16, 32 loads in flight
// per lane.  `hints` selects the evict_last priority on the gathers.  Writes nothing.
extern "C" int b200_gather_probe(const void *table, int64_t table_rows, int64_t gathers, int32_t variant,
                                 int32_t hints, void *sink, void *workspace, void *stream) {
  if (!table || !sink || !workspace || table_rows < 1 || table_rows > (1 << 26) || gathers < 1 || variant < 0 ||
      variant > 3)
    return fail(B200_ERR_INVALID_ARGUMENT, "gather_probe: bad arguments");
  if (!aligned16(table)) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gather_probe: table must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float *t = static_cast<const float *>(table);
  float *out = static_cast<float *>(sink);
  {
    const int64_t ctas = (int64_t)sm_count() * 8;          // 64 warps per SM
    const int64_t per_warp = (gathers + ctas * 8 - 1) / (ctas * 8);
#define B200_PROBE(D) \
    (hints ? gather_probe_kernel<D, true><<<(unsigned)ctas, 256, 0, s>>>(t, table_rows, per_warp, out) \
           : gather_probe_kernel<D, false><<<(unsigned)ctas, 256, 0, s>>>(t, table_rows, per_warp, out))
    switch (variant) {
    case 0: B200_PROBE(4); break;
    case 1: B200_PROBE(8); break;
    case 2: B200_PROBE(16); break;
    default: B200_PROBE(32); break;
    }
#undef B200_PROBE
  }
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
