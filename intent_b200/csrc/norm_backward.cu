// LayerNorm backward (bf16 operands, f32 arithmetic): the row kernel and the reduction of its
// partial sums.
//
// Row kernel.  The scatter-reduction into partial-sum row `row % G` collides across the rows of a
// group; the reference promises no order for colliding updates, so this file fixes one that maps
// onto a thread-block cluster (every add is the typed bf16 add):
//   the group's rows g, g+G, g+2G, ... are dealt round-robin to 8 lanes; each lane folds its rows
//   in ascending order from zero; the lane sums are combined as ((s0+s1)+(s2+s3))+((s4+s5)+(s6+s7));
//   the total is added to the element's previous contents.
// A cluster of 8 CTAs takes one group at a time and CTA l is lane l; the grid is as many clusters as
// the device holds at once and a cluster walks the groups c, c + clusters, ...  A CTA (8 warps) walks
// its lane's rows: a thread owns 1, 2 or 4 vectors of 8 columns (N <= 2048, 4096, 8192) and keeps the
// weight vector and its lane sums in registers.  Three rows of x and dy are in flight towards a
// four-slot ring in shared memory, across group boundaries (asynchronous copies; each thread copies the
// vectors it reads, so no barrier guards the ring).  Per row: the two row sums (packed f32x2 arithmetic,
// one CTA barrier, double-buffered scratch), then dx, written with streaming stores.  After a group's
// last row the lane sums go to shared memory (two buffers alternate between groups); the cluster
// barrier is split around that row's dx, and then CTA l reads the eight lanes' sums of its eighth of
// the columns through distributed shared memory, combines them in the fixed tree, and updates the
// partial-sum rows.  x and dy are read once, dx written once: no atomics, no scratch in global memory,
// and the same result on every run.
// Algorithmic bytes: 3*M*N*2 (x, dy, dx) + 4*G*N*2 (partials read and written) + N*2 + M*8.
#include <cooperative_groups.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace b200 {
namespace {

namespace cg = cooperative_groups;

constexpr int kVec = 8;             // bf16 per 128-bit access
constexpr int kLanes = 8;           // CTAs per cluster = lanes of the update order

// The typed combine, two elements at a time.  A packed bf16 add rounds the exact sum once; that is
// the value bf16(f32(a) + f32(b)) of the definition: the f32 sum of two bf16 numbers is exact unless
// their exponents lie more than 16 apart, and then both roundings return the larger operand.
__device__ __forceinline__ __nv_bfloat162 combine(__nv_bfloat162 a, __nv_bfloat162 b) { return __hadd2(a, b); }
// A 128-bit load the compiler may not sink to its first use: issued here, it is in flight while the
// statements that follow (a barrier wait) run.
__device__ __forceinline__ uint4 load_now(const void *pointer) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(pointer));
  return v;
}
// Asynchronous copies global -> shared memory.  A thread only ever reads what it copied itself (or,
// for the row statistics, what a lane of its own warp copied), so completion needs no mbarrier and
// no spin: `wait_group` blocks the thread until its own groups have landed.
__device__ __forceinline__ void copy_async_16(void *shared, const void *global) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(shared)), "l"(global)
               : "memory");
}
__device__ __forceinline__ void copy_async_4(void *shared, const void *global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(shared)), "l"(global)
               : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING> __device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}
// The cluster barrier in two halves.  The releasing arrival waits for the thread's earlier writes (its
// streaming stores of dx among them) to be performed, so it is issued before the last row's dx is
// written; the relaxed form orders execution only.
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
constexpr int kRing = 4;            // rows of x and dy a CTA keeps in flight or in use

// Both halves of a bf16 pair as f32; the arithmetic below works on such pairs with the packed f32x2
// instructions.  Each rounds to nearest per half like its scalar form, with one caveat measured on
// B200: a packed product that feeds a packed sum is contracted into one packed fma by the assembler,
// explicit rounding modifiers or not.  The values that must match the typed definition bit for bit
// (xhat = (x - mean) * rstd, dy * xhat, and the bf16 sums) contain no product feeding a sum; the f32
// row sums and dx, which are compared within a tolerance, may be contracted.
__device__ __forceinline__ float2 widen(uint32_t pair) {
  return make_float2(__uint_as_float(pair << 16), __uint_as_float(pair & 0xffff0000u));
}

template <int kRowThreads, int VECTORS>
__global__ void __cluster_dims__(kLanes, 1, 1) __launch_bounds__(kRowThreads, VECTORS > 2 ? 1 : 2)
layer_norm_backward_rows_kernel(const __nv_bfloat16 *__restrict__ x, const __nv_bfloat16 *__restrict__ dy,
                                const __nv_bfloat16 *__restrict__ weight, const float *__restrict__ mean,
                                const float *__restrict__ rstd, __nv_bfloat16 *__restrict__ dx,
                                __nv_bfloat16 *__restrict__ dw_partial, __nv_bfloat16 *__restrict__ db_partial,
                                int64_t rows, int columns, int groups, int64_t x_pitch, int64_t dy_pitch,
                                int64_t dx_pitch, int64_t dw_pitch, int64_t db_pitch, int64_t mean_stride,
                                int64_t rstd_stride, float inverse_features) {
  constexpr int kRowStride = kRowThreads * kVec;   // columns between a thread's vectors
  // [2 rounds][dw | db][columns] lane sums, then the ring [kRing][x | dy][columns]
  extern __shared__ __align__(16) __nv_bfloat16 lane_sums[];
  __shared__ float scratch[2][kRowThreads / 32][2];
  __shared__ float statistics[kRing][kRowThreads / 32][2];
  __nv_bfloat16 *ring = lane_sums + 4 * columns;
  cg::cluster_group cluster = cg::this_cluster();
  const int lane = (int)cluster.block_rank();
  const int clusters = gridDim.x / kLanes, first_group = blockIdx.x / kLanes;
  const int warp = threadIdx.x >> 5, thread_lane = threadIdx.x & 31;
  const int first = threadIdx.x * kVec;

  // rows of up to 4096 columns: the weight vector is kept widened and a row's g = w * dy and xhat stay
  // in registers between the two passes; wider rows keep it packed and read the row from the ring again
  constexpr bool kHold = VECTORS <= 2;
  uint4 w_packed[kHold ? 1 : VECTORS];
  float2 w_wide[kHold ? VECTORS : 1][kVec / 2];
#pragma unroll
  for (int v = 0; v < VECTORS; ++v) {
    uint4 loaded = make_uint4(0, 0, 0, 0);
    if (first + v * kRowStride < columns) loaded = *reinterpret_cast<const uint4 *>(weight + first + v * kRowStride);
#pragma unroll
    for (int i = 0; i < kVec / 2; ++i)
      if (kHold) w_wide[v][i] = widen(reinterpret_cast<const uint32_t *>(&loaded)[i]);
    if (!kHold) w_packed[v] = loaded;
  }
  auto weight_pair = [&](int v, int i) {
    return kHold ? w_wide[v][i] : widen(reinterpret_cast<const uint32_t *>(&w_packed[v])[i]);
  };
  // CTA `lane` combines its eighth of the columns of every group (N <= 8192: at most one vector per thread)
  const int vectors = columns / kVec, share = (vectors + kLanes - 1) / kLanes;
  const int combine_index = lane * share + threadIdx.x;
  const bool combines = threadIdx.x < share && combine_index < vectors;
  // The cluster walks the groups first_group, first_group + clusters, ...  Of group g's rows g + j * groups
  // (j < count) this CTA takes j = lane, lane + 8, ...: `rows_of(g)` of them.
  auto rows_of = [&](int group) -> int64_t {
    const int64_t count = rows > group ? (rows - group + groups - 1) / groups : 0;
    return count > lane ? (count - lane + kLanes - 1) / kLanes : 0;
  };
  // Rows travel through a ring of kRing slots in shared memory, kRing - 1 rows requested ahead of the one
  // in use, across group boundaries.  A thread copies exactly the vectors it will read; lane 0 of a warp
  // copies the row's mean and rstd for its warp.  One copy group is committed per request, empty once
  // the CTA's last row has been requested.  The n-th row requested and the n-th row used are the same
  // row, and both sides take slot n % kRing.
  int ahead_group = first_group;
  int64_t ahead_step = 0, ahead_rows = first_group < groups ? rows_of(first_group) : 0;
  uint32_t requested = 0;
  auto request = [&]() {
    while (ahead_group < groups && ahead_step >= ahead_rows) {
      ahead_group += clusters;
      ahead_step = 0;
      if (ahead_group < groups) ahead_rows = rows_of(ahead_group);
    }
    if (ahead_group < groups) {
      const int64_t row = ahead_group + (lane + ahead_step * kLanes) * (int64_t)groups;
      __nv_bfloat16 *slot = ring + (size_t)(requested % kRing) * 2 * columns;
#pragma unroll
      for (int v = 0; v < VECTORS; ++v) {
        const int column = first + v * kRowStride;
        if (column < columns) {
          copy_async_16(slot + column, x + row * x_pitch + column);
          copy_async_16(slot + columns + column, dy + row * dy_pitch + column);
        }
      }
      if (thread_lane == 0) {
        copy_async_4(&statistics[requested % kRing][warp][0], mean + row * mean_stride);
        copy_async_4(&statistics[requested % kRing][warp][1], rstd + row * rstd_stride);
      }
      ++ahead_step;
      ++requested;
    }
    copy_async_commit();
  };
#pragma unroll
  for (int ahead = 0; ahead < kRing - 1; ++ahead) request();
  uint32_t used = 0;                                            // rows consumed so far (all groups)
  int round = 0;
  for (int group = first_group; group < groups; group += clusters, ++round) {
    const int64_t mine = rows_of(group);
    __nv_bfloat16 *round_sums = lane_sums + (size_t)(round & 1) * 2 * columns;
    __nv_bfloat162 dw[VECTORS][kVec / 2], db[VECTORS][kVec / 2];   // this lane's sums for the group, packed
#pragma unroll
    for (int v = 0; v < VECTORS; ++v)
#pragma unroll
      for (int i = 0; i < kVec / 2; ++i) dw[v][i] = db[v][i] = __floats2bfloat162_rn(0.0f, 0.0f);
    // This lane's sums, for the whole cluster to read: final once the group's last row has been added,
    // which is before that row's dx is formed.  Two buffers alternate between rounds: a CTA writes
    // buffer r & 1 again only after the cluster barrier of round r + 1, which every CTA reaches after
    // its reads of round r.
    auto publish = [&]() {
#pragma unroll
      for (int v = 0; v < VECTORS; ++v) {
        const int column = first + v * kRowStride;
        if (column >= columns) continue;
        *reinterpret_cast<uint4 *>(round_sums + column) = *reinterpret_cast<const uint4 *>(dw[v]);
        *reinterpret_cast<uint4 *>(round_sums + columns + column) = *reinterpret_cast<const uint4 *>(db[v]);
      }
      cluster_arrive_release();
    };
    if (mine == 0) publish();
    for (int64_t step = 0; step < mine; ++step, ++used) {
      const int64_t row = group + (lane + step * kLanes) * (int64_t)groups;
      // the slot of the row before this one is free: every thread finished with it before that row's barrier
      request();
      copy_async_wait<kRing - 1>();
      __syncwarp();                                               // lane 0's copy of the statistics, for the warp
      const __nv_bfloat16 *current = ring + (size_t)(used % kRing) * 2 * columns;
      const float row_mean = statistics[used % kRing][warp][0], row_rstd = statistics[used % kRing][warp][1];
      uint4 x_raw[VECTORS], dy_raw[VECTORS];
#pragma unroll
      for (int v = 0; v < VECTORS; ++v) {
        const int column = first + v * kRowStride;
        x_raw[v] = dy_raw[v] = make_uint4(0, 0, 0, 0);
        if (column < columns) {
          x_raw[v] = *reinterpret_cast<const uint4 *>(current + column);
          dy_raw[v] = *reinterpret_cast<const uint4 *>(current + columns + column);
        }
      }
      const float2 minus_mean = make_float2(-row_mean, -row_mean), rstd_pair = make_float2(row_rstd, row_rstd);
      float2 sums = make_float2(0.0f, 0.0f), sums_normalized = make_float2(0.0f, 0.0f);
      float2 g_kept[kHold ? VECTORS : 1][kVec / 2], n_kept[kHold ? VECTORS : 1][kVec / 2];
#pragma unroll
      for (int v = 0; v < VECTORS; ++v) {
        const uint32_t *x_pairs = reinterpret_cast<const uint32_t *>(&x_raw[v]);
        const uint32_t *dy_pairs = reinterpret_cast<const uint32_t *>(&dy_raw[v]);
#pragma unroll
        for (int i = 0; i < kVec / 2; ++i) {
          // xhat = (x - mean) * rstd and dy * xhat: a sum feeding a product, and a bare product, so
          // nothing here can be contracted and the lane sums are those of the typed definition
          const float2 d = widen(dy_pairs[i]);
          const float2 n = __fmul2_rn(__fadd2_rn(widen(x_pairs[i]), minus_mean), rstd_pair);
          const float2 g = __fmul2_rn(weight_pair(v, i), d);
          sums = __fadd2_rn(sums, g);
          sums_normalized = __ffma2_rn(g, n, sums_normalized);
          dw[v][i] = combine(dw[v][i], __float22bfloat162_rn(__fmul2_rn(d, n)));
          db[v][i] = combine(db[v][i], *reinterpret_cast<const __nv_bfloat162 *>(&dy_pairs[i]));
          if (kHold) { g_kept[v][i] = g; n_kept[v][i] = n; }
        }
      }
      const float sum = warp_sum(sums.x + sums.y);
      const float sum_normalized = warp_sum(sums_normalized.x + sums_normalized.y);
      float (*slot)[2] = scratch[used & 1];
      if (thread_lane == 0) { slot[warp][0] = sum; slot[warp][1] = sum_normalized; }
      __syncthreads();   // the other parity's slots are free again once every thread is past this point
      if (step == mine - 1) publish();
      float total = 0.0f, total_normalized = 0.0f;
#pragma unroll
      for (int other = 0; other < kRowThreads / 32; ++other) { total += slot[other][0]; total_normalized += slot[other][1]; }
      const float mean_weighted_dy = total * inverse_features;
      const float mean_weighted_dy_normalized = total_normalized * inverse_features;
      const float2 minus_a = make_float2(-mean_weighted_dy, -mean_weighted_dy);
      const float2 minus_b = make_float2(-mean_weighted_dy_normalized, -mean_weighted_dy_normalized);
#pragma unroll
      for (int v = 0; v < VECTORS; ++v) {
        if (first + v * kRowStride >= columns) continue;
        uint4 x_again, dy_again;                                  // wide rows: read again from the ring, not held
        if (!kHold) {
          x_again = *reinterpret_cast<const uint4 *>(current + first + v * kRowStride);
          dy_again = *reinterpret_cast<const uint4 *>(current + columns + first + v * kRowStride);
        }
        uint4 raw;
        __nv_bfloat162 *pairs = reinterpret_cast<__nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < kVec / 2; ++i) {
          float2 g, n;
          if (kHold) {
            g = g_kept[v][i];
            n = n_kept[v][i];
          } else {
            n = __fmul2_rn(__fadd2_rn(widen(reinterpret_cast<const uint32_t *>(&x_again)[i]), minus_mean), rstd_pair);
            g = __fmul2_rn(weight_pair(v, i), widen(reinterpret_cast<const uint32_t *>(&dy_again)[i]));
          }
          // (g - mean(g) - xhat * mean(g * xhat)) * rstd
          pairs[i] = __float22bfloat162_rn(__fmul2_rn(__ffma2_rn(n, minus_b, __fadd2_rn(g, minus_a)), rstd_pair));
        }
        __stcs(reinterpret_cast<uint4 *>(dx + row * dx_pitch + first + v * kRowStride), raw);
      }
    }
    // the previous contents of this CTA's share of the group's partial sums, requested before the barrier
    uint4 old_sums[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    if (combines) {
      old_sums[0] = load_now(dw_partial + group * dw_pitch + combine_index * kVec);
      old_sums[1] = load_now(db_partial + group * db_pitch + combine_index * kVec);
    }
    cluster_wait_acquire();
    if (combines) {
      const int column = combine_index * kVec;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16 *destination = (which ? db_partial + group * db_pitch : dw_partial + group * dw_pitch) + column;
        uint4 level[kLanes];
#pragma unroll
        for (int l = 0; l < kLanes; ++l)
          level[l] = *reinterpret_cast<const uint4 *>(cluster.map_shared_rank(round_sums, l) + which * columns + column);
#pragma unroll
        for (int width = 1; width < kLanes; width <<= 1)
#pragma unroll
          for (int l = 0; l < kLanes; l += 2 * width) {
            __nv_bfloat162 *into = reinterpret_cast<__nv_bfloat162 *>(&level[l]);
            const __nv_bfloat162 *from = reinterpret_cast<const __nv_bfloat162 *>(&level[l + width]);
#pragma unroll
            for (int i = 0; i < kVec / 2; ++i) into[i] = combine(into[i], from[i]);
          }
        uint4 old = old_sums[which];
        __nv_bfloat162 *result = reinterpret_cast<__nv_bfloat162 *>(&old);
        const __nv_bfloat162 *total = reinterpret_cast<const __nv_bfloat162 *>(&level[0]);
#pragma unroll
        for (int i = 0; i < kVec / 2; ++i) result[i] = combine(result[i], total[i]);
        *reinterpret_cast<uint4 *>(destination) = old;
      }
    }
  }
  copy_async_wait<0>();
  cluster_arrive_relaxed();   // no CTA may leave while another still reads its shared memory
  cluster_wait_acquire();
}

// dw[n] = sum over groups (ascending) of f32(dw_partial[g, n]); likewise db.  A CTA owns 16 columns:
// all threads stage up to 128 group rows of both matrices in shared memory at once (so every load of
// the tile is in flight together), then one thread per (matrix, column) adds them in group order.
constexpr int kReduceColumns = 16, kReduceGroups = 128, kReduceThreads = 256;

__global__ void __launch_bounds__(kReduceThreads)
layer_norm_backward_reduce_kernel(const __nv_bfloat16 *__restrict__ dw_partial,
                                  const __nv_bfloat16 *__restrict__ db_partial, float *__restrict__ dw,
                                  float *__restrict__ db, int groups, int columns, int64_t dw_pitch,
                                  int64_t db_pitch, int64_t dw_stride, int64_t db_stride, int paired) {
  constexpr int kPairs = kReduceColumns / 2;
  __shared__ __align__(16) __nv_bfloat16 tile[2][kReduceGroups][kReduceColumns];
  const int column0 = blockIdx.x * kReduceColumns;
  const int which = threadIdx.x / kReduceColumns, mine = threadIdx.x % kReduceColumns;  // threads 0..31 add
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
#pragma unroll 4
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

// Clusters of kLanes CTAs of `kernel` the current device holds at once; 0 if the query fails.  Cached
// per (kernel, shared memory, device): the entry is called once per step.
int resident_clusters(const void *kernel, int threads, size_t smem) {
  struct Key { const void *kernel; size_t smem; int device; int clusters; };
  static std::mutex guard;
  static std::vector<Key> known;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return 0; }
  std::lock_guard<std::mutex> lock(guard);
  for (const Key &key : known)
    if (key.kernel == kernel && key.smem == smem && key.device == device) return key.clusters;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = kLanes;
  attribute.val.clusterDim.y = attribute.val.clusterDim.z = 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(kLanes);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = smem;
  config.attrs = &attribute;
  config.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess) { cudaGetLastError(); clusters = 0; }
  known.push_back({kernel, smem, device, clusters});
  return clusters;
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
  if (dw_d0 > INT32_MAX / kLanes) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm_backward_rows: too many groups");
  cudaStream_t queue = static_cast<cudaStream_t>(stream);
  // two rounds of lane sums, then the ring
  const size_t smem = (4 + 2 * kRing) * (size_t)n * sizeof(__nv_bfloat16);
  auto launch = [&](auto kernel, int threads) -> cudaError_t {
    if (smem + 1024 > 48 * 1024) {                                // the static arrays count towards the 48 KB
      const cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (error != cudaSuccess) return error;
    }
    // As many clusters as the device holds at once, each walking an equal number of groups (the last
    // round may be short); one cluster per group if the device will not say.
    const int64_t resident = resident_clusters(reinterpret_cast<const void *>(kernel), threads, smem);
    const int64_t rounds = resident > 0 ? (dw_d0 + resident - 1) / resident : 1;
    const int64_t clusters = (dw_d0 + rounds - 1) / rounds;
    kernel<<<(unsigned)(clusters * kLanes), threads, smem, queue>>>(
        (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)dy, (const __nv_bfloat16 *)weight, (const float *)mean,
        (const float *)rstd, (__nv_bfloat16 *)dx, (__nv_bfloat16 *)dw_partial, (__nv_bfloat16 *)db_partial, m, (int)n,
        (int)dw_d0, x_s0, dy_s0, dx_s0, dw_s0, db_s0, mean_s0, rstd_s0, inverse_features);
    return cudaGetLastError();
  };
  // 8 warps per row; 1, 2 or 4 vectors of 8 columns per thread
  if (n <= 256 * kVec) B200_CUDA_TRY(launch(layer_norm_backward_rows_kernel<256, 1>, 256));
  else if (n <= 512 * kVec) B200_CUDA_TRY(launch(layer_norm_backward_rows_kernel<256, 2>, 256));
  else B200_CUDA_TRY(launch(layer_norm_backward_rows_kernel<256, 4>, 256));
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
