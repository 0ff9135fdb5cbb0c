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
#include <string.h>

#include <mutex>

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
// Words of the caller's int32 workspace (one per prepared call, zeroed once by the caller):
//   [0] sticky: a bounded wait on a staged gather gave up   [1] the row that was left unwritten
//   [2] "every row seen so far ascends": set by the first launch of a call, cleared by a
//       launch that meets a descending row, read by the later launches of the same call.
// Nothing of a call lives in library-global device memory, so calls on different streams
// cannot see one another's flags.
constexpr int kStateTimeout = 0, kStateRow = 1, kStateSorted = 2;

__global__ void spmm_begin_kernel(int *state) { state[kStateSorted] = 1; }

// X is gathered about 32 times per element while the index, value and Y streams are touched
// once: gathers ask L2 to keep their lines (evict_last), the streams ask to be dropped first.
__device__ __forceinline__ uint64_t policy_keep() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t policy_stream() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ float4 load_keep(const float *address, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(address), "l"(policy));
  return v;
}
template <typename T>
__device__ __forceinline__ T load_stream(const T *address, uint64_t policy) {
  uint32_t bits;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;" : "=r"(bits) : "l"(address), "l"(policy));
  T value;
  memcpy(&value, &bits, 4);
  return value;
}
__device__ __forceinline__ float4 load_stream4(const float *address, uint64_t policy) {
  float4 v;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(address), "l"(policy));
  return v;
}
__device__ __forceinline__ void store_stream4(float *address, float4 v, uint64_t policy) {
  asm volatile("st.global.L1::no_allocate.L2::cache_hint.v4.f32 [%0], {%1, %2, %3, %4}, %5;"
               ::"l"(address), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(policy) : "memory");
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
// Staged gathers.  The gathers are latency-bound, so they are handed to the copy
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

__device__ __forceinline__ uint32_t shared_address(const void *pointer) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(pointer));
}

template <bool HINTS>
__global__ void __launch_bounds__(kBulkWarps * 32, 1)
csr_spmm_bulk_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                     const float *__restrict__ values, const float *__restrict__ dense,
                     float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                     int64_t output_pitch, int column_lo, int column_hi, int phase, int *state) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const Block block = block_of_launch(state, column_lo, column_hi, phase);
  if (block.skip) return;
  const bool check_order = phase == 0 && (column_lo != INT32_MIN || column_hi != INT32_MAX);
  const uint64_t keep = policy_keep(), stream = policy_stream();
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
  int previous = INT32_MIN;                 // last column of the batch before, within one row
  auto fetch = [&](const Cursor &c, bool valid, bool first) -> Batch {
    Batch b;
    b.row = valid ? first_row + c.ordinal * warps : -1;
    b.base = c.base; b.stop = c.stop; b.first = first; b.last = c.base + 32 >= c.stop;
    b.column = 0; b.value = 0.0f;
    const bool stored = valid && c.base + lane < c.stop;
    if (stored) {
      if (HINTS) {
        b.column = load_stream<int>(column_indices + c.base + lane, stream);
        b.value = load_stream<float>(values + c.base + lane, stream);
      } else {
        b.column = __ldcs(column_indices + c.base + lane);
        b.value = __ldcs(values + c.base + lane);
      }
    }
    if (check_order && valid) {
      if (first) previous = INT32_MIN;
      const int before = __shfl_up_sync(0xffffffffu, b.column, 1);
      const bool descends = stored && b.column < (lane == 0 ? previous : before);
      if (__any_sync(0xffffffffu, descends) && lane == 0) state[kStateSorted] = 0;
      previous = __shfl_sync(0xffffffffu, b.column, 31);
    }
    return b;
  };
  // Requests the gathers of one batch into `stage`; returns the lanes that take part.
  auto request = [&](const Batch &b, int stage) -> unsigned {
    const bool mine = b.row >= 0 && b.base + lane < b.stop && b.column >= block.lo && b.column < block.hi;
    const unsigned mask = __ballot_sync(0xffffffffu, mine);
    const uint32_t bar = shared_address(bars + stage);
    if (lane == 0 && mask != 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(__popc(mask) * row_bytes)
                   : "memory");
    __syncwarp();
    if (mine) {
      const float *from = source + (int64_t)b.column * dense_pitch;
      const uint32_t to = shared_address(stage_base + stage * kBulkStageBytes + lane * kBulkRowBytes);
      if (HINTS)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                     ::"r"(to), "l"(from), "r"(row_bytes), "r"(bar), "l"(keep)
                     : "memory");
      else
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
  bool touched = false;
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
      touched = !block.accumulate;   // a launch that starts from zero always writes
      if (block.accumulate && active) {  // partial sums of the earlier column blocks
        const float *partial = output + current.row * output_pitch + feature0 + lane * 4;
        acc = HINTS ? load_stream4(partial, stream) : __ldcs(reinterpret_cast<const float4 *>(partial));
      }
    }
    if (current_mask != 0) {
      touched = true;
      const uint32_t parity = stage ? parity1 : parity0;
      const long long begin = clock64();
      bool landed = try_wait(stage, parity);
      while (!landed && clock64() - begin < kBulkWaitCycles) landed = try_wait(stage, parity);
      if (!landed) {  // give up: flag the failure, leave the row unwritten and stop this warp
        if (lane == 0 && atomicCAS(&state[kStateTimeout], 0, 1) == 0) state[kStateRow] = (int)current.row;
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
    if (current.last && active && touched) {
      float *destination = output + current.row * output_pitch + feature0 + lane * 4;
      if (HINTS) store_stream4(destination, acc, stream);
      else __stcs(reinterpret_cast<float4 *>(destination), acc);
    }
    stage ^= 1;
    current = next;
    current_mask = next_mask;
    next = after;
  }
  // No copy is left in flight here: every requested batch was waited for.
}

// Gathers held in registers (eight in flight per lane), one row per warp, many warps: the
// alternative to staging for launches that see only a few non-zeros of every row.
constexpr int kBlockWarps = 8;

template <bool HINTS>
__global__ void __launch_bounds__(kBlockWarps * 32)
csr_spmm_block_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ column_indices,
                      const float *__restrict__ values, const float *__restrict__ dense,
                      float *__restrict__ output, int64_t rows, int features, int64_t dense_pitch,
                      int64_t output_pitch, int column_lo, int column_hi, int phase, int *state) {
  const Block block = block_of_launch(state, column_lo, column_hi, phase);
  if (block.skip) return;
  const uint64_t keep = policy_keep(), stream = policy_stream();
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kBlockWarps + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int feature = blockIdx.y * 128 + lane * 4;
  const bool active = feature < features;
  const int start = __ldg(row_offsets + row), stop = __ldg(row_offsets + row + 1);
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float *destination = output + row * output_pitch + feature;
  if (block.accumulate && active)
    acc = HINTS ? load_stream4(destination, stream) : __ldcs(reinterpret_cast<const float4 *>(destination));
  const float *source = dense + feature;
  bool touched = !block.accumulate;  // a launch that starts from zero always writes
  int previous = INT32_MIN;          // last column of the batch before (ascending check of launch 0)
  for (int base = start; base < stop; base += 32) {
    int column = 0;
    float value = 0.0f;
    bool mine = false;
    if (base + lane < stop) {
      if (HINTS) {
        column = load_stream<int>(column_indices + base + lane, stream);
        value = load_stream<float>(values + base + lane, stream);
      } else {
        column = __ldcs(column_indices + base + lane);
        value = __ldcs(values + base + lane);
      }
      mine = column >= block.lo && column < block.hi;
    }
    if (phase == 0) {
      const int before = __shfl_up_sync(0xffffffffu, column, 1);
      const bool descends = base + lane < stop && column < (lane == 0 ? previous : before);
      if (__any_sync(0xffffffffu, descends) && lane == 0) state[kStateSorted] = 0;
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
        if (active && lanes[u] >= 0) {
          const float *from = source + (int64_t)c * dense_pitch;
          gathered[u] = HINTS ? load_keep(from, keep) : __ldg(reinterpret_cast<const float4 *>(from));
        }
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
  if (active && touched) {
    if (HINTS) store_stream4(destination, acc, stream);
    else __stcs(reinterpret_cast<float4 *>(destination), acc);
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
  uint64_t position = (uint64_t)(warp + 1) * 0x9E3779B97F4A7C15ull;
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  for (int64_t done = 0; done < per_warp; done += DEPTH) {
    float4 got[DEPTH];
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) {
      position = position * 6364136223846793005ull + 1442695040888963407ull;
      const int64_t row = (int64_t)((position >> 33) % (uint64_t)table_rows);
      const float *from = table + row * 128 + lane * 4;
      got[d] = HINTS ? load_keep(from, keep) : __ldg(reinterpret_cast<const float4 *>(from));
    }
#pragma unroll
    for (int d = 0; d < DEPTH; ++d) { acc.x += got[d].x; acc.y += got[d].y; acc.z += got[d].z; acc.w += got[d].w; }
  }
  if (acc.x == 12345.678f) sink[warp * 128 + lane * 4] = acc.y + acc.z + acc.w;  // never true in practice
}

// The same walk with the copy engine: every lane requests one 512-byte row into the warp's
// staging buffer (two stages of 32 rows), as the staged SpMM kernel does.
template <bool HINTS>
__global__ void __launch_bounds__(kBulkWarps * 32, 1)
gather_probe_bulk_kernel(const float *__restrict__ table, int64_t table_rows, int64_t per_warp, float *__restrict__ sink,
                         int *state) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  const uint64_t keep = policy_keep();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned char *stage_base = bulk_smem + (size_t)warp * kBulkStages * kBulkStageBytes;
  uint64_t *bars = reinterpret_cast<uint64_t *>(bulk_smem + (size_t)kBulkWarps * kBulkStages * kBulkStageBytes) +
                   warp * kBulkStages;
  if (lane == 0) {
    for (int s = 0; s < kBulkStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(shared_address(bars + s)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const int64_t global_warp = (int64_t)blockIdx.x * kBulkWarps + warp;
  uint64_t position = (uint64_t)(global_warp * 32 + lane + 1) * 0x9E3779B97F4A7C15ull;
  auto request = [&](int stage) {
    const uint32_t bar = shared_address(bars + stage);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(32 * kBulkRowBytes) : "memory");
    __syncwarp();
    position = position * 6364136223846793005ull + 1442695040888963407ull;
    const float *from = table + (int64_t)((position >> 33) % (uint64_t)table_rows) * 128;
    const uint32_t to = shared_address(stage_base + stage * kBulkStageBytes + lane * kBulkRowBytes);
    if (HINTS)
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                   ::"r"(to), "l"(from), "r"(kBulkRowBytes), "r"(bar), "l"(keep) : "memory");
    else
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(to), "l"(from), "r"(kBulkRowBytes), "r"(bar) : "memory");
  };
  auto try_wait = [&](int stage, uint32_t parity) -> bool {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(shared_address(bars + stage)), "r"(parity) : "memory");
    return done != 0;
  };
  const int64_t batches = (per_warp + 31) / 32;
  uint32_t parity[2] = {0, 0};
  float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  request(0);
  for (int64_t batch = 0; batch < batches; ++batch) {
    const int stage = (int)(batch & 1);
    if (batch + 1 < batches) request(stage ^ 1);
    const long long begin = clock64();
    bool landed = try_wait(stage, parity[stage]);
    while (!landed && clock64() - begin < kBulkWaitCycles) landed = try_wait(stage, parity[stage]);
    if (!landed) {
      if (lane == 0 && atomicCAS(&state[kStateTimeout], 0, 1) == 0) state[kStateRow] = (int)batch;
      if (batch + 1 < batches) {
        const long long drain = clock64();
        while (!try_wait(stage ^ 1, parity[stage ^ 1]) && clock64() - drain < kBulkWaitCycles / 8) {}
      }
      return;
    }
    parity[stage] ^= 1;
    const unsigned char *staged = stage_base + stage * kBulkStageBytes + lane * 16;
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const float4 x = *reinterpret_cast<const float4 *>(staged + j * kBulkRowBytes);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
    __syncwarp();
  }
  if (acc.x == 12345.678f) sink[global_warp * 128 + lane * 4] = acc.y + acc.z + acc.w;
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
constexpr bool kColumnBlocksStaged = false;   // column blocks run on the register kernel unless overridden

// Tuning overrides, read at every call so that one process can sweep them:
//   INTENT_B200_SPMM_PHASES  1..16   number of column blocks
//   INTENT_B200_SPMM_KERNEL  staged | registers   which kernel runs the column blocks
//   INTENT_B200_SPMM_HINTS   0 | 1   L2 eviction priorities on the loads and stores
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
  const bool vector = x_d1 % 4 == 0 && x_s0 % 4 == 0 && y_s0 % 4 == 0 && aligned16(dense) && aligned16(output);
  if (!vector) {
    csr_spmm_scalar_kernel<<<(unsigned)ctas, kWarpsPerCta * 32, 0, s>>>(
        (const int32_t *)row_offsets, (const int32_t *)column_indices, (const float *)values,
        (const float *)dense, (float *)output, rows, (int)x_d1, x_s0, y_s0);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  const int phases = column_phases(x_d0, x_d1);
  const bool hints = tuning_integer("INTENT_B200_SPMM_HINTS", 0, 1, 1) != 0;
  const char *choice = getenv("INTENT_B200_SPMM_KERNEL");
  const bool staged = phases == 1 || (choice ? strcmp(choice, "staged") == 0 : kColumnBlocksStaged);
  const unsigned chunks = (unsigned)((x_d1 + 127) / 128);
  if (staged) {
    B200_CUDA_TRY(opt_in_dynamic_smem(csr_spmm_bulk_kernel<true>, kBulkSmemBytes));
    B200_CUDA_TRY(opt_in_dynamic_smem(csr_spmm_bulk_kernel<false>, kBulkSmemBytes));
  }
  if (phases > 1) spmm_begin_kernel<<<1, 1, 0, s>>>(state);
  const int64_t wanted = (rows + kBulkWarps - 1) / kBulkWarps;
  const int64_t resident = sm_count();
  const dim3 staged_grid((unsigned)(wanted < resident ? wanted : resident), chunks);
  const dim3 register_grid((unsigned)((rows + kBlockWarps - 1) / kBlockWarps), chunks);
  const int64_t span = (x_d0 + phases - 1) / phases;
  for (int phase = 0; phase < phases; ++phase) {
    const int lo = phases > 1 ? (int)(phase * span) : INT32_MIN;
    const int hi = phases > 1 && phase + 1 < phases ? (int)((phase + 1) * span) : INT32_MAX;
    auto launch = [&](auto kernel, dim3 grid, int threads, size_t smem) {
      kernel<<<grid, threads, smem, s>>>((const int32_t *)row_offsets, (const int32_t *)column_indices,
                                         (const float *)values, (const float *)dense, (float *)output, rows,
                                         (int)x_d1, x_s0, y_s0, lo, hi, phase, state);
    };
    if (staged) {
      if (hints) launch(csr_spmm_bulk_kernel<true>, staged_grid, kBulkWarps * 32, kBulkSmemBytes);
      else launch(csr_spmm_bulk_kernel<false>, staged_grid, kBulkWarps * 32, kBulkSmemBytes);
    } else {
      if (hints) launch(csr_spmm_block_kernel<true>, register_grid, kBlockWarps * 32, 0);
      else launch(csr_spmm_block_kernel<false>, register_grid, kBlockWarps * 32, 0);
    }
  }
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// Gather-rate probe (see gather_probe_kernel).  `variant`: 0..3 = 4, 8, 16, 32 register loads
// in flight per lane; 4 = staged through shared memory by the copy engine.  `hints` selects
// the evict_last priority on the gathers.  Reads table_rows x 512 bytes; writes nothing.
extern "C" int b200_gather_probe(const void *table, int64_t table_rows, int64_t gathers, int32_t variant,
                                 int32_t hints, void *sink, void *workspace, void *stream) {
  if (!table || !sink || !workspace || table_rows < 1 || gathers < 1 || variant < 0 || variant > 4)
    return fail(B200_ERR_INVALID_ARGUMENT, "gather_probe: bad arguments");
  if (!aligned16(table)) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "gather_probe: table must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float *t = static_cast<const float *>(table);
  float *out = static_cast<float *>(sink);
  if (variant == 4) {
    const int64_t warps = (int64_t)sm_count() * kBulkWarps;
    const int64_t per_warp = (gathers + warps - 1) / warps;
    B200_CUDA_TRY(opt_in_dynamic_smem(gather_probe_bulk_kernel<true>, kBulkSmemBytes));
    B200_CUDA_TRY(opt_in_dynamic_smem(gather_probe_bulk_kernel<false>, kBulkSmemBytes));
    if (hints)
      gather_probe_bulk_kernel<true><<<sm_count(), kBulkWarps * 32, kBulkSmemBytes, s>>>(t, table_rows, per_warp, out, (int *)workspace);
    else
      gather_probe_bulk_kernel<false><<<sm_count(), kBulkWarps * 32, kBulkSmemBytes, s>>>(t, table_rows, per_warp, out, (int *)workspace);
  } else {
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

extern "C" int b200_csr_spmm_status(const void *workspace, int64_t *row, void *stream) {
  if (!workspace) return fail(B200_ERR_INVALID_ARGUMENT, "csr_spmm_status: null workspace");
  int words[2] = {0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_CUDA_TRY(cudaMemcpyAsync(words, workspace, sizeof words, cudaMemcpyDeviceToHost, s));
  B200_CUDA_TRY(cudaStreamSynchronize(s));
  if (row) *row = words[1];
  if (words[0] != 0) {
    cudaMemsetAsync(const_cast<void *>(workspace), 0, sizeof words, s);   // the report is delivered once
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
