// LayerNorm backward (bf16 operands, f32 arithmetic): the row kernel's two halves and the
// reduction of its partial sums.
//
// The reference's row kernel does two things per row: dx, which needs two sums over the row,
// and the scatter-reduction of dy*xhat and dy into partial-sum row `row % G`, which needs no
// row sum (xhat only takes the mean and rstd operands) but collides across rows.  They are
// two launches here:
//
//   dx kernel        row-parallel: a group of 1..8 warps owns a row (up to 4 vectors of 8 bf16 per
//                    thread, weight kept in registers), one named-barrier reduction of the pair
//                    (sum w*dy, sum w*dy*xhat), dx written with streaming stores.  x and dy are
//                    read with the default policy so that they stay in L2 for
//   partials kernel  column-parallel: a thread owns 8 columns of one partial-sum row and walks that
//                    group's rows g, g+G, ... in ascending order with loads four rows ahead, every
//                    update rounded to bf16 (the typed combine): a fixed order, so the same result
//                    on every run, and no atomics.
//
// Algorithmic bytes: 3*M*N*2 (x, dy, dx) + 4*G*N*2 (partials read and written) + N*2 + M*8;
// the second read of x and dy is not counted (67 MB at the reference shape, mostly from L2).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kVec = 8;          // bf16 per 128-bit access
constexpr int kMaxVectors = 4;   // vectors per thread in the dx kernel
constexpr int kDxThreads = 256;
constexpr int kPrefetch = 4;     // rows in flight per thread in the partials kernel

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

template <int WARPS>
__global__ void __launch_bounds__(kDxThreads)
layer_norm_backward_dx_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ dy,
                              const __nv_bfloat16 *__restrict__ weight, const float *__restrict__ mean,
                              const float *__restrict__ rstd, __nv_bfloat16 *__restrict__ dx, int64_t rows,
                              int columns, int64_t x_pitch, int64_t dy_pitch, int64_t dx_pitch,
                              int64_t mean_stride, int64_t rstd_stride, float inverse_features) {
  constexpr int kGroups = kDxThreads / 32 / WARPS;   // rows a CTA works on at once
  __shared__ float scratch[2][kGroups][2][WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp / WARPS, warp_in_group = warp % WARPS;
  const int first = (warp_in_group * 32 + lane) * kVec;        // vector v: + v * WARPS * 32 * kVec
  constexpr int kStride = WARPS * 32 * kVec;

  float w[kMaxVectors][kVec];
#pragma unroll
  for (int v = 0; v < kMaxVectors; ++v) {
#pragma unroll
    for (int i = 0; i < kVec; ++i) w[v][i] = 0.0f;
    if (first + v * kStride < columns) load_vector(weight + first + v * kStride, w[v]);
  }
  int parity = 0;
  for (int64_t row = (int64_t)blockIdx.x * kGroups + group; row < rows; row += (int64_t)gridDim.x * kGroups) {
    const float row_mean = mean[row * mean_stride], row_rstd = rstd[row * rstd_stride];
    uint4 x_raw[kMaxVectors], dy_raw[kMaxVectors];
#pragma unroll
    for (int v = 0; v < kMaxVectors; ++v) {
      x_raw[v] = dy_raw[v] = make_uint4(0, 0, 0, 0);
      if (first + v * kStride < columns) {
        x_raw[v] = *reinterpret_cast<const uint4 *>(x + row * x_pitch + first + v * kStride);
        dy_raw[v] = *reinterpret_cast<const uint4 *>(dy + row * dy_pitch + first + v * kStride);
      }
    }
    float sum = 0.0f, sum_normalized = 0.0f;
#pragma unroll
    for (int v = 0; v < kMaxVectors; ++v) {
      const __nv_bfloat16 *x_lanes = reinterpret_cast<const __nv_bfloat16 *>(&x_raw[v]);
      const __nv_bfloat16 *dy_lanes = reinterpret_cast<const __nv_bfloat16 *>(&dy_raw[v]);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float normalized = __fmul_rn(__fsub_rn(__bfloat162float(x_lanes[i]), row_mean), row_rstd);
        const float weighted_dy = __fmul_rn(w[v][i], __bfloat162float(dy_lanes[i]));
        sum += weighted_dy;
        sum_normalized += __fmul_rn(weighted_dy, normalized);
      }
    }
    sum = warp_sum(sum);
    sum_normalized = warp_sum(sum_normalized);
    if (WARPS > 1) {
      if (lane == 0) { scratch[parity][group][0][warp_in_group] = sum; scratch[parity][group][1][warp_in_group] = sum_normalized; }
      asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(WARPS * 32) : "memory");
      sum = sum_normalized = 0.0f;
#pragma unroll
      for (int other = 0; other < WARPS; ++other) {
        sum += scratch[parity][group][0][other];
        sum_normalized += scratch[parity][group][1][other];
      }
      parity ^= 1;   // the other slot is free again once the group has passed the next barrier
    }
    const float mean_weighted_dy = sum * inverse_features;
    const float mean_weighted_dy_normalized = sum_normalized * inverse_features;
#pragma unroll
    for (int v = 0; v < kMaxVectors; ++v) {
      if (first + v * kStride >= columns) continue;
      const __nv_bfloat16 *x_lanes = reinterpret_cast<const __nv_bfloat16 *>(&x_raw[v]);
      const __nv_bfloat16 *dy_lanes = reinterpret_cast<const __nv_bfloat16 *>(&dy_raw[v]);
      uint4 raw;
      __nv_bfloat16 *lanes = reinterpret_cast<__nv_bfloat16 *>(&raw);
#pragma unroll
      for (int i = 0; i < kVec; ++i) {
        const float normalized = __fmul_rn(__fsub_rn(__bfloat162float(x_lanes[i]), row_mean), row_rstd);
        const float weighted_dy = __fmul_rn(w[v][i], __bfloat162float(dy_lanes[i]));
        lanes[i] = __float2bfloat16_rn((weighted_dy - mean_weighted_dy - normalized * mean_weighted_dy_normalized) * row_rstd);
      }
      __stcs(reinterpret_cast<uint4 *>(dx + row * dx_pitch + first + v * kStride), raw);
    }
  }
}

__global__ void __launch_bounds__(256)
layer_norm_backward_partials_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ dy,
                                    const float *__restrict__ mean, const float *__restrict__ rstd,
                                    __nv_bfloat16 *__restrict__ dw_partial, __nv_bfloat16 *__restrict__ db_partial,
                                    int64_t rows, int vectors, int groups, int64_t x_pitch, int64_t dy_pitch,
                                    int64_t dw_pitch, int64_t db_pitch, int64_t mean_stride, int64_t rstd_stride) {
  const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= (int64_t)groups * vectors) return;
  const int group = (int)(index / vectors), column = (int)(index % vectors) * kVec;
  float dw[kVec], db[kVec];
  load_vector(dw_partial + group * dw_pitch + column, dw);
  load_vector(db_partial + group * db_pitch + column, db);

  // rows of this group: group, group + groups, ...
  const int64_t count = rows > group ? (rows - group + groups - 1) / groups : 0;
  uint4 x_next[kPrefetch], dy_next[kPrefetch];
  float mean_next[kPrefetch], rstd_next[kPrefetch];
#pragma unroll
  for (int stage = 0; stage < kPrefetch; ++stage) {
    x_next[stage] = dy_next[stage] = make_uint4(0, 0, 0, 0);
    mean_next[stage] = rstd_next[stage] = 0.0f;
    if (stage < count) {
      const int64_t row = group + (int64_t)stage * groups;
      mean_next[stage] = mean[row * mean_stride];
      rstd_next[stage] = rstd[row * rstd_stride];
      x_next[stage] = *reinterpret_cast<const uint4 *>(x + row * x_pitch + column);
      dy_next[stage] = *reinterpret_cast<const uint4 *>(dy + row * dy_pitch + column);
    }
  }
  for (int64_t step = 0; step < count; ++step) {
    const uint4 x_raw = x_next[0], dy_raw = dy_next[0];
    const float row_mean = mean_next[0], row_rstd = rstd_next[0];
#pragma unroll
    for (int stage = 0; stage + 1 < kPrefetch; ++stage) {
      x_next[stage] = x_next[stage + 1];
      dy_next[stage] = dy_next[stage + 1];
      mean_next[stage] = mean_next[stage + 1];
      rstd_next[stage] = rstd_next[stage + 1];
    }
    if (step + kPrefetch < count) {
      const int64_t ahead = group + (step + kPrefetch) * groups;
      mean_next[kPrefetch - 1] = mean[ahead * mean_stride];
      rstd_next[kPrefetch - 1] = rstd[ahead * rstd_stride];
      x_next[kPrefetch - 1] = *reinterpret_cast<const uint4 *>(x + ahead * x_pitch + column);
      dy_next[kPrefetch - 1] = *reinterpret_cast<const uint4 *>(dy + ahead * dy_pitch + column);
    }
    const __nv_bfloat16 *x_lanes = reinterpret_cast<const __nv_bfloat16 *>(&x_raw);
    const __nv_bfloat16 *dy_lanes = reinterpret_cast<const __nv_bfloat16 *>(&dy_raw);
#pragma unroll
    for (int i = 0; i < kVec; ++i) {
      const float dy_value = __bfloat162float(dy_lanes[i]);
      // unfused, in the reference's order: these values take no part in the row sums
      const float normalized = __fmul_rn(__fsub_rn(__bfloat162float(x_lanes[i]), row_mean), row_rstd);
      dw[i] = round_bf16(dw[i] + round_bf16(__fmul_rn(dy_value, normalized)));
      db[i] = round_bf16(db[i] + dy_value);
    }
  }
  store_vector(dw_partial + group * dw_pitch + column, dw);
  store_vector(db_partial + group * db_pitch + column, db);
}

// dw[n] = sum over groups (ascending) of f32(dw_partial[g, n]); likewise db.  A CTA owns 32 columns:
// all threads stage up to 128 group rows of both matrices in shared memory at once (so every load of
// the tile is in flight together), then one thread per (matrix, column) adds them in group order.
constexpr int kReduceColumns = 32, kReduceGroups = 128, kReduceThreads = 128;

__global__ void __launch_bounds__(kReduceThreads)
layer_norm_backward_reduce_kernel(const __nv_bfloat16 *__restrict__ dw_partial,
                                  const __nv_bfloat16 *__restrict__ db_partial, float *__restrict__ dw,
                                  float *__restrict__ db, int groups, int columns, int64_t dw_pitch,
                                  int64_t db_pitch, int64_t dw_stride, int64_t db_stride, int paired) {
  constexpr int kPairs = kReduceColumns / 2;
  __shared__ __align__(16) __nv_bfloat16 tile[2][kReduceGroups][kReduceColumns];
  const int column0 = blockIdx.x * kReduceColumns;
  const int which = threadIdx.x / kReduceColumns, mine = threadIdx.x % kReduceColumns;  // threads 0..63 add
  const int pair = threadIdx.x % kPairs, first_group = threadIdx.x / kPairs;            // staging role
  constexpr int kGroupStep = kReduceThreads / kPairs;
  const int column = column0 + 2 * pair;
  float total = 0.0f;
  for (int group0 = 0; group0 < groups; group0 += kReduceGroups) {
    const int here = min(kReduceGroups, groups - group0);
    if (group0) __syncthreads();
#pragma unroll
    for (int matrix = 0; matrix < 2; ++matrix) {
      const __nv_bfloat16 *base = matrix ? db_partial : dw_partial;
      const int64_t pitch = matrix ? db_pitch : dw_pitch;
#pragma unroll 8
      for (int g = first_group; g < here; g += kGroupStep) {
        const __nv_bfloat16 *source = base + (group0 + g) * pitch + column;
        __nv_bfloat162 value = __floats2bfloat162_rn(0.0f, 0.0f);
        if (paired && column + 1 < columns) {
          value = *reinterpret_cast<const __nv_bfloat162 *>(source);
        } else {
          if (column < columns) value.x = source[0];
          if (column + 1 < columns) value.y = source[1];
        }
        *reinterpret_cast<__nv_bfloat162 *>(&tile[matrix][g][2 * pair]) = value;
      }
    }
    __syncthreads();
    if (which < 2) {
#pragma unroll 16
      for (int g = 0; g < here; ++g) total += __bfloat162float(tile[which][g][mine]);
    }
  }
  if (which < 2 && column0 + mine < columns) {
    if (which == 0) dw[(column0 + mine) * dw_stride] = total;
    else db[(column0 + mine) * db_stride] = total;
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_layer_norm_backward_rows(
    const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1, const void *dy, int64_t dy_d0,
    int64_t dy_d1, int64_t dy_s0, int64_t dy_s1, const void *weight, int64_t w_d0, int64_t w_s0, const void *mean,
    int64_t mean_d0, int64_t mean_s0, const void *rstd, int64_t rstd_d0, int64_t rstd_s0, void *dx, int64_t dx_d0,
    int64_t dx_d1, int64_t dx_s0, int64_t dx_s1, void *dw_partial, int64_t dw_d0, int64_t dw_d1, int64_t dw_s0,
    int64_t dw_s1, void *db_partial, int64_t db_d0, int64_t db_d1, int64_t db_s0, int64_t db_s1,
    float inverse_features, void *stream) {
  const int64_t m = x_d0, n = x_d1;
  if (m < 0 || n < 0 || dy_d0 != m || dy_d1 != n || dx_d0 != m || dx_d1 != n || w_d0 != n || mean_d0 != m ||
      rstd_d0 != m || dw_d1 != n || db_d1 != n || db_d0 != dw_d0)
    return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm_backward_rows: operand shapes disagree");
  if (m == 0 || n == 0) return B200_OK;
  if (dw_d0 <= 0) return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm_backward_rows: no partial-sum groups");
  if (!x || !dy || !weight || !mean || !rstd || !dx || !dw_partial || !db_partial)
    return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm_backward_rows: null buffer");
  if (n > 1 && (x_s1 != 1 || dy_s1 != 1 || dx_s1 != 1 || dw_s1 != 1 || db_s1 != 1 || w_s0 != 1))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_rows: inner strides must be 1");
  if (n % kVec != 0 || n > 1024 * kVec)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_rows: N = %lld must be a multiple of 8, at most 8192",
                (long long)n);
  if (!aligned16(x) || !aligned16(dy) || !aligned16(dx) || !aligned16(dw_partial) || !aligned16(db_partial) ||
      !aligned16(weight) || x_s0 % kVec || dy_s0 % kVec || dx_s0 % kVec || dw_s0 % kVec || db_s0 % kVec)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_rows: rows must be 16-byte aligned");
  if (dw_d0 > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_rows: too many groups");
  cudaStream_t queue = static_cast<cudaStream_t>(stream);
  const int vectors = (int)(n / kVec);
  const int warps = vectors <= 128 ? 1 : vectors <= 256 ? 2 : vectors <= 512 ? 4 : 8;   // <= 4 vectors per thread
  auto launch_dx = [&](auto kernel, int rows_per_cta) {
    const int64_t wanted = (m + rows_per_cta - 1) / rows_per_cta;
    const int64_t limit = (int64_t)sm_count() * 8;
    kernel<<<(unsigned)(wanted < limit ? wanted : limit), kDxThreads, 0, queue>>>(
        (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)dy, (const __nv_bfloat16 *)weight, (const float *)mean,
        (const float *)rstd, (__nv_bfloat16 *)dx, m, (int)n, x_s0, dy_s0, dx_s0, mean_s0, rstd_s0, inverse_features);
  };
  switch (warps) {
  case 1: launch_dx(layer_norm_backward_dx_kernel<1>, 8); break;
  case 2: launch_dx(layer_norm_backward_dx_kernel<2>, 4); break;
  case 4: launch_dx(layer_norm_backward_dx_kernel<4>, 2); break;
  default: launch_dx(layer_norm_backward_dx_kernel<8>, 1); break;
  }
  B200_CUDA_TRY(cudaGetLastError());
  const int64_t threads = dw_d0 * vectors;
  layer_norm_backward_partials_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, queue>>>(
      (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)dy, (const float *)mean, (const float *)rstd,
      (__nv_bfloat16 *)dw_partial, (__nv_bfloat16 *)db_partial, m, vectors, (int)dw_d0, x_s0, dy_s0, dw_s0, db_s0,
      mean_s0, rstd_s0);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_layer_norm_backward_reduce(const void *dw_partial, int64_t dw_d0, int64_t dw_d1, int64_t dw_s0,
                                               int64_t dw_s1, const void *db_partial, int64_t db_d0, int64_t db_d1,
                                               int64_t db_s0, int64_t db_s1, void *dw, int64_t o_d0, int64_t o_s0,
                                               void *db, int64_t b_d0, int64_t b_s0, void *stream) {
  const int64_t groups = dw_d0, n = dw_d1;
  if (groups < 0 || n < 0 || db_d0 != groups || db_d1 != n || o_d0 != n || b_d0 != n)
    return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm_backward_reduce: operand shapes disagree");
  if (n == 0) return B200_OK;
  if (!dw || !db || (groups > 0 && (!dw_partial || !db_partial)))
    return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm_backward_reduce: null buffer");
  if (n > 1 && (dw_s1 != 1 || db_s1 != 1))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_reduce: inner strides must be 1");
  if (n > INT32_MAX || groups > INT32_MAX)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_reduce: extent too large");
  const int paired = (reinterpret_cast<uintptr_t>(dw_partial) % 4 == 0) && (reinterpret_cast<uintptr_t>(db_partial) % 4 == 0) &&
                     dw_s0 % 2 == 0 && db_s0 % 2 == 0;
  layer_norm_backward_reduce_kernel<<<(unsigned)((n + kReduceColumns - 1) / kReduceColumns), kReduceThreads, 0,
                                      static_cast<cudaStream_t>(stream)>>>(
      (const __nv_bfloat16 *)dw_partial, (const __nv_bfloat16 *)db_partial, (float *)dw, (float *)db, (int)groups,
      (int)n, dw_s0, db_s0, o_s0, b_s0, paired);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
