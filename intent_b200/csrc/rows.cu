// Row-parallel, HBM-bound operators: softmax and LayerNorm.
//
// Layout: a row is owned by a "row group" of WARPS warps; each thread keeps
// ITERS 128-bit vectors of the row in registers, so every element is read
// from HBM once and written once (8 B/element for f32 softmax, 4 B/element
// for 16-bit LayerNorm).  Reductions are warp shuffles plus, when a row spans
// several warps, one named barrier per reduction.  Row groups stride over the
// rows (persistent grid sized from the SM count) so LayerNorm's gamma/beta are
// staged in shared memory once per CTA.
#include <mutex>

#include "common.cuh"

namespace b200 {
namespace {

constexpr int kCtaWarps = 8;

// CTA_WARPS: warps per CTA when a row needs fewer.  Softmax uses small CTAs so
// that a few thousand rows still spread evenly over 148 SMs.
template <int WARPS, int CTA_WARPS = kCtaWarps> struct GroupShape {
  static constexpr int kCtaThreads = (WARPS > CTA_WARPS ? WARPS : CTA_WARPS) * 32;
  static constexpr int kGroups = kCtaThreads / (WARPS * 32);
};

// ------------------------------------------------------------------ softmax
constexpr int kSoftmaxCtaWarps = 4;
template <int WARPS> using SoftmaxShape = GroupShape<WARPS, kSoftmaxCtaWarps>;

template <typename T, int WARPS, int ITERS>
__global__ void __launch_bounds__(SoftmaxShape<WARPS>::kCtaThreads)
softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int columns,
                    int64_t x_pitch, int64_t y_pitch) {
  constexpr int kVec = Element<T>::kVec;
  constexpr int kGroups = SoftmaxShape<WARPS>::kGroups;
  constexpr int kRowThreads = WARPS * 32;
  __shared__ float scratch[kGroups][2][WARPS];
  const int group = threadIdx.x / kRowThreads;
  const int lane_in_row = threadIdx.x % kRowThreads;
  const int warp_in_group = lane_in_row >> 5;
  const int barrier_id = 1 + group;

  for (int64_t row = (int64_t)blockIdx.x * kGroups + group; row < rows;
       row += (int64_t)gridDim.x * kGroups) {
    const T *source = x + row * x_pitch;
    float value[ITERS][kVec];
    float maximum = -INFINITY;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int column = (it * kRowThreads + lane_in_row) * kVec;
      if (column < columns) {
        load_vector<T>(source + column, value[it]);
#pragma unroll
        for (int i = 0; i < kVec; ++i) maximum = maximum_num(maximum, value[it][i]);
      }
    }
    maximum = group_reduce<WARPS, true>(maximum, scratch[group][0], warp_in_group, barrier_id);
    float sum = 0.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int column = (it * kRowThreads + lane_in_row) * kVec;
      if (column < columns) {
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          value[it][i] = expf(value[it][i] - maximum);
          sum += value[it][i];
        }
      }
    }
    sum = group_reduce<WARPS, false>(sum, scratch[group][1], warp_in_group, barrier_id);
    T *destination = y + row * y_pitch;
    if (sizeof(T) == 4) {
      const float inverse = __fdiv_rn(1.0f, sum);  // multiply by the reciprocal (f32 kernel)
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int column = (it * kRowThreads + lane_in_row) * kVec;
        if (column < columns) {
#pragma unroll
          for (int i = 0; i < kVec; ++i) value[it][i] = __fmul_rn(value[it][i], inverse);
          store_vector<T>(destination + column, value[it]);
        }
      }
    } else {
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int column = (it * kRowThreads + lane_in_row) * kVec;
        if (column < columns) {
#pragma unroll
          for (int i = 0; i < kVec; ++i) value[it][i] = __fdiv_rn(value[it][i], sum);
          store_vector<T>(destination + column, value[it]);
        }
      }
    }
    if (WARPS > 1)  // scratch is reused by the next row of this group
      asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(kRowThreads) : "memory");
  }
}

// Any row length / alignment: one CTA per row, three passes over global memory.
template <typename T>
__global__ void __launch_bounds__(256)
softmax_generic_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int64_t columns,
                       int64_t x_pitch, int64_t y_pitch) {
  __shared__ float scratch[2][8];
  const int warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *source = x + row * x_pitch;
    T *destination = y + row * y_pitch;
    float maximum = -INFINITY;
    for (int64_t c = threadIdx.x; c < columns; c += 256)
      maximum = maximum_num(maximum, Element<T>::widen(source[c]));
    maximum = group_reduce<8, true>(maximum, scratch[0], warp, 1);
    float sum = 0.0f;
    for (int64_t c = threadIdx.x; c < columns; c += 256)
      sum += expf(Element<T>::widen(source[c]) - maximum);
    sum = group_reduce<8, false>(sum, scratch[1], warp, 1);
    const float inverse = __fdiv_rn(1.0f, sum);
    for (int64_t c = threadIdx.x; c < columns; c += 256) {
      const float e = expf(Element<T>::widen(source[c]) - maximum);
      destination[c] = Element<T>::narrow(sizeof(T) == 4 ? __fmul_rn(e, inverse) : __fdiv_rn(e, sum));
    }
    __syncthreads();
  }
}

// --------------------------------------------------------- softmax backward
// gradient = p * (dy - sum(p * dy)) per row.  The reference instance has 4097 columns, so
// rows are not 16-byte aligned: both input rows are staged in shared memory with coalesced
// scalar loads (each element is read from HBM once), reduced, and written back.
__global__ void __launch_bounds__(256)
softmax_backward_kernel(const float *__restrict__ probabilities, const float *__restrict__ upstream,
                        float *__restrict__ gradient, int64_t rows, int columns, int64_t p_pitch,
                        int64_t u_pitch, int64_t g_pitch, int staged) {
  extern __shared__ __align__(16) unsigned char dynamic_smem[];
  float *p_row = reinterpret_cast<float *>(dynamic_smem);
  float *u_row = p_row + columns;
  __shared__ float scratch[8];
  const int warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *p = probabilities + row * p_pitch, *u = upstream + row * u_pitch;
    float partial = 0.0f;
    for (int c = threadIdx.x; c < columns; c += 256) {
      const float pv = __ldcs(p + c), uv = __ldcs(u + c);
      if (staged) { p_row[c] = pv; u_row[c] = uv; }
      partial += __fmul_rn(pv, uv);
    }
    const float projection = group_reduce<8, false>(partial, scratch, warp, 1);
    float *g = gradient + row * g_pitch;
    for (int c = threadIdx.x; c < columns; c += 256) {
      const float pv = staged ? p_row[c] : p[c], uv = staged ? u_row[c] : u[c];
      __stcs(g + c, __fmul_rn(pv, __fsub_rn(uv, projection)));
    }
    __syncthreads();  // scratch and the staged rows are reused by the next row
  }
}

// The same operator for rows of up to 8 * 1024 columns whose three matrices share one alignment
// row by row: each row is peeled to its first 16-byte boundary (0..3 leading and 0..3 trailing
// scalars, one per thread) and the body moves as 128-bit vectors that stay in registers between the
// reduction and the write, so nothing is staged in shared memory.
template <int VECTORS>
__global__ void __launch_bounds__(256)
softmax_backward_vector_kernel(const float *__restrict__ probabilities, const float *__restrict__ upstream,
                               float *__restrict__ gradient, int64_t rows, int columns, int64_t p_pitch,
                               int64_t u_pitch, int64_t g_pitch) {
  __shared__ float scratch[2][8];
  const int warp = threadIdx.x >> 5;
  int parity = 0;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const float *p = probabilities + row * p_pitch, *u = upstream + row * u_pitch;
    float *g = gradient + row * g_pitch;
    const int lead = min(columns, (int)(((16 - (reinterpret_cast<uintptr_t>(p) & 15)) & 15) >> 2));
    const int vectors = (columns - lead) >> 2, tail = columns - lead - 4 * vectors;
    const float4 *p4 = reinterpret_cast<const float4 *>(p + lead), *u4 = reinterpret_cast<const float4 *>(u + lead);
    float4 pv[VECTORS], uv[VECTORS];
#pragma unroll
    for (int v = 0; v < VECTORS; ++v) {
      const int index = threadIdx.x + v * 256;
      pv[v] = uv[v] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (index < vectors) { pv[v] = __ldcs(p4 + index); uv[v] = __ldcs(u4 + index); }
    }
    // the peeled scalars: thread e takes leading element e, or trailing element e - lead
    const int edge = (int)threadIdx.x < lead ? (int)threadIdx.x
                   : (int)threadIdx.x < lead + tail ? lead + 4 * vectors + ((int)threadIdx.x - lead) : -1;
    float pe = 0.0f, ue = 0.0f;
    if (edge >= 0) { pe = p[edge]; ue = u[edge]; }
    float partial = __fmul_rn(pe, ue);
#pragma unroll
    for (int v = 0; v < VECTORS; ++v)
      partial += __fmul_rn(pv[v].x, uv[v].x) + __fmul_rn(pv[v].y, uv[v].y) + __fmul_rn(pv[v].z, uv[v].z) +
                 __fmul_rn(pv[v].w, uv[v].w);
    const float projection = group_reduce<8, false>(partial, scratch[parity], warp, 1);
    parity ^= 1;   // the next row's partial sums go to the other slot: one barrier per row is enough
    float4 *g4 = reinterpret_cast<float4 *>(g + lead);
#pragma unroll
    for (int v = 0; v < VECTORS; ++v) {
      const int index = threadIdx.x + v * 256;
      if (index < vectors)
        __stcs(g4 + index, make_float4(__fmul_rn(pv[v].x, __fsub_rn(uv[v].x, projection)),
                                       __fmul_rn(pv[v].y, __fsub_rn(uv[v].y, projection)),
                                       __fmul_rn(pv[v].z, __fsub_rn(uv[v].z, projection)),
                                       __fmul_rn(pv[v].w, __fsub_rn(uv[v].w, projection))));
    }
    if (edge >= 0) g[edge] = __fmul_rn(pe, __fsub_rn(ue, projection));
  }
}

// --------------------------------------------------------------- layer norm
template <typename T, int WARPS, int ITERS, bool CENTERED>
__global__ void __launch_bounds__(GroupShape<WARPS>::kCtaThreads)
layer_norm_rows_kernel(const T *__restrict__ x, const T *__restrict__ weight,
                       const T *__restrict__ bias, T *__restrict__ y, int64_t rows, int columns,
                       int64_t x_pitch, int64_t y_pitch, float inverse_features, float epsilon,
                       int stage_parameters) {
  constexpr int kVec = Element<T>::kVec;
  constexpr int kGroups = GroupShape<WARPS>::kGroups;
  constexpr int kRowThreads = WARPS * 32;
  constexpr int kCtaThreads = GroupShape<WARPS>::kCtaThreads;
  extern __shared__ __align__(16) unsigned char dynamic_smem[];
  __shared__ float scratch[kGroups][2][WARPS];
  const int group = threadIdx.x / kRowThreads;
  const int lane_in_row = threadIdx.x % kRowThreads;
  const int warp_in_group = lane_in_row >> 5;
  const int barrier_id = 1 + group;

  // gamma / beta: staged once per CTA when they fit, else read through L2.
  const T *gamma = weight, *beta = bias;
  if (stage_parameters) {
    T *staged = reinterpret_cast<T *>(dynamic_smem);
    for (int c = threadIdx.x * kVec; c < columns; c += kCtaThreads * kVec) {
      *reinterpret_cast<uint4 *>(staged + c) = *reinterpret_cast<const uint4 *>(weight + c);
      *reinterpret_cast<uint4 *>(staged + columns + c) = *reinterpret_cast<const uint4 *>(bias + c);
    }
    __syncthreads();
    gamma = staged;
    beta = staged + columns;
  }

  // the next row of this group is requested (raw, 128 bits per vector) before the current one is reduced
  const int64_t row_step = (int64_t)gridDim.x * kGroups;
  uint4 ahead[ITERS];
  auto request = [&](int64_t row) {
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int column = (it * kRowThreads + lane_in_row) * kVec;
      ahead[it] = make_uint4(0, 0, 0, 0);
      if (row < rows && column < columns) ahead[it] = *reinterpret_cast<const uint4 *>(x + row * x_pitch + column);
    }
  };
  request((int64_t)blockIdx.x * kGroups + group);
  for (int64_t row = (int64_t)blockIdx.x * kGroups + group; row < rows; row += row_step) {
    float value[ITERS][kVec];
    float sum = 0.0f, squares = 0.0f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const T *lanes = reinterpret_cast<const T *>(&ahead[it]);
#pragma unroll
      for (int i = 0; i < kVec; ++i) value[it][i] = Element<T>::widen(lanes[i]);
    }
    request(row + row_step);
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int column = (it * kRowThreads + lane_in_row) * kVec;
      if (column < columns) {
#pragma unroll
        for (int i = 0; i < kVec; ++i) {
          sum += value[it][i];
          if (!CENTERED) squares += value[it][i] * value[it][i];
        }
      }
    }
    sum = group_reduce<WARPS, false>(sum, scratch[group][0], warp_in_group, barrier_id);
    const float mean = __fmul_rn(sum, inverse_features);
    float variance;
    if (CENTERED) {
#pragma unroll
      for (int it = 0; it < ITERS; ++it) {
        const int column = (it * kRowThreads + lane_in_row) * kVec;
        if (column < columns) {
#pragma unroll
          for (int i = 0; i < kVec; ++i) {
            value[it][i] = value[it][i] - mean;
            squares += value[it][i] * value[it][i];
          }
        }
      }
      squares = group_reduce<WARPS, false>(squares, scratch[group][1], warp_in_group, barrier_id);
      variance = __fmul_rn(squares, inverse_features);
    } else {
      squares = group_reduce<WARPS, false>(squares, scratch[group][1], warp_in_group, barrier_id);
      variance = __fsub_rn(__fmul_rn(squares, inverse_features), __fmul_rn(mean, mean));
#pragma unroll
      for (int it = 0; it < ITERS; ++it)
#pragma unroll
        for (int i = 0; i < kVec; ++i) value[it][i] = value[it][i] - mean;
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, epsilon)));
    T *destination = y + row * y_pitch;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int column = (it * kRowThreads + lane_in_row) * kVec;
      if (column < columns) {
        float w[kVec], b[kVec];
        load_vector<T>(gamma + column, w);
        load_vector<T>(beta + column, b);
#pragma unroll
        for (int i = 0; i < kVec; ++i)  // left to right, separately rounded like the CPU provider
          value[it][i] = __fadd_rn(__fmul_rn(__fmul_rn(value[it][i], scale), w[i]), b[i]);
        store_vector<T>(destination + column, value[it]);
      }
    }
    if (WARPS > 1)
      asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(kRowThreads) : "memory");
  }
}

template <typename T, bool CENTERED>
__global__ void __launch_bounds__(256)
layer_norm_generic_kernel(const T *__restrict__ x, const T *__restrict__ weight, int64_t w_stride,
                          const T *__restrict__ bias, int64_t b_stride, T *__restrict__ y,
                          int64_t rows, int64_t columns, int64_t x_pitch, int64_t y_pitch,
                          float inverse_features, float epsilon) {
  __shared__ float scratch[2][8];
  const int warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T *source = x + row * x_pitch;
    T *destination = y + row * y_pitch;
    float sum = 0.0f, squares = 0.0f;
    for (int64_t c = threadIdx.x; c < columns; c += 256) {
      const float v = Element<T>::widen(source[c]);
      sum += v;
      if (!CENTERED) squares += v * v;
    }
    sum = group_reduce<8, false>(sum, scratch[0], warp, 1);
    const float mean = __fmul_rn(sum, inverse_features);
    if (CENTERED)
      for (int64_t c = threadIdx.x; c < columns; c += 256) {
        const float v = Element<T>::widen(source[c]) - mean;
        squares += v * v;
      }
    squares = group_reduce<8, false>(squares, scratch[1], warp, 1);
    const float variance = CENTERED
        ? __fmul_rn(squares, inverse_features)
        : __fsub_rn(__fmul_rn(squares, inverse_features), __fmul_rn(mean, mean));
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, epsilon)));
    for (int64_t c = threadIdx.x; c < columns; c += 256) {
      const float v = Element<T>::widen(source[c]) - mean;
      const float w = Element<T>::widen(weight[c * w_stride]), b = Element<T>::widen(bias[c * b_stride]);
      destination[c] = Element<T>::narrow(__fadd_rn(__fmul_rn(__fmul_rn(v, scale), w), b));
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------- dispatch
// Picks the smallest row group that keeps a row in registers with at most
// kMaxIters vectors per thread; returns false when the row is too long.
struct RowPlan { int warps, iters; };

template <typename T> bool plan_row(int64_t columns, RowPlan *plan) {
  constexpr int kVec = Element<T>::kVec;
  constexpr int kMaxIters = 32 / kVec;  // 32 f32 values per thread
  if (columns % kVec) return false;
  const int64_t vectors = columns / kVec;
  for (int warps = 1; warps <= 32; warps *= 2) {
    const int64_t iters = (vectors + warps * 32 - 1) / (warps * 32);
    if (iters <= kMaxIters) {
      int rounded = 1;
      while (rounded < iters) rounded *= 2;
      *plan = {warps, rounded};
      return true;
    }
  }
  return false;
}

// CTAs of `kernel` that are resident per SM (register, thread and shared-memory limits),
// so the persistent grid is exactly one wave.  The last answer is cached per thread, keyed by the
// kernel's address (instantiations that differ only in integer parameters share one function
// type, so a cache per template instance of this helper would mix them up), the CTA size, the
// shared-memory size and the device.
template <typename Kernel>
int resident_ctas(Kernel kernel, int threads, size_t smem) {
  struct Key {
    const void *kernel;
    int threads, device;
    size_t smem;
  };
  static thread_local Key cached_key = {nullptr, 0, -1, 0};
  static thread_local int cached = 0;
  int device = 0;
  cudaGetDevice(&device);
  const void *address = reinterpret_cast<const void *>(kernel);
  if (cached_key.kernel != address || cached_key.threads != threads || cached_key.smem != smem || cached_key.device != device) {
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kernel, threads, smem) != cudaSuccess || blocks < 1)
      blocks = 1;
    cached = blocks;
    cached_key = {address, threads, device, smem};
  }
  return cached;
}

int grid_for(int64_t rows, int groups_per_cta, int ctas_per_sm) {
  const int64_t wanted = (rows + groups_per_cta - 1) / groups_per_cta;
  const int64_t resident = (int64_t)sm_count() * ctas_per_sm;
  return (int)(wanted < resident ? wanted : resident);
}

template <typename T, int WARPS, int ITERS>
int launch_softmax_rows(const T *x, T *y, int64_t rows, int64_t columns, int64_t xp, int64_t yp,
                        cudaStream_t stream) {
  using Shape = SoftmaxShape<WARPS>;
  const int grid = grid_for(rows, Shape::kGroups,
                            resident_ctas(softmax_rows_kernel<T, WARPS, ITERS>, Shape::kCtaThreads, 0));
  softmax_rows_kernel<T, WARPS, ITERS><<<grid, Shape::kCtaThreads, 0, stream>>>(
      x, y, rows, (int)columns, xp, yp);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <typename T, int WARPS>
int softmax_pick_iters(int iters, const T *x, T *y, int64_t rows, int64_t columns, int64_t xp,
                       int64_t yp, cudaStream_t stream) {
  constexpr int kMaxIters = 32 / Element<T>::kVec;
  switch (iters) {
  case 1: return launch_softmax_rows<T, WARPS, 1>(x, y, rows, columns, xp, yp, stream);
  case 2: return launch_softmax_rows<T, WARPS, 2>(x, y, rows, columns, xp, yp, stream);
  case 4: return launch_softmax_rows<T, WARPS, 4>(x, y, rows, columns, xp, yp, stream);
  default:
    return launch_softmax_rows<T, WARPS, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  }
}

template <typename T>
int softmax_typed(const T *x, T *y, int64_t rows, int64_t columns, int64_t xp, int64_t yp,
                  cudaStream_t stream) {
  RowPlan plan;
  const bool vector_ok = aligned16(x) && aligned16(y) && xp % Element<T>::kVec == 0 &&
                         yp % Element<T>::kVec == 0 && plan_row<T>(columns, &plan);
  if (!vector_ok) {
    const int grid = (int)(rows < (int64_t)sm_count() * 8 ? rows : (int64_t)sm_count() * 8);
    softmax_generic_kernel<T><<<grid, 256, 0, stream>>>(x, y, rows, columns, xp, yp);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  constexpr int kMaxIters = 32 / Element<T>::kVec;
  if (plan.warps == 1) return softmax_pick_iters<T, 1>(plan.iters, x, y, rows, columns, xp, yp, stream);
  // wider groups always run with the full register tile
  switch (plan.warps) {
  case 2: return launch_softmax_rows<T, 2, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  case 4: return launch_softmax_rows<T, 4, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  case 8: return launch_softmax_rows<T, 8, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  case 16: return launch_softmax_rows<T, 16, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  default: return launch_softmax_rows<T, 32, kMaxIters>(x, y, rows, columns, xp, yp, stream);
  }
}

constexpr int kMaxStagedParameterBytes = 64 * 1024;

template <typename T, int WARPS, int ITERS, bool CENTERED>
int launch_layer_norm_rows(const T *x, const T *w, const T *b, T *y, int64_t rows, int64_t columns,
                           int64_t xp, int64_t yp, float inverse_features, float epsilon,
                           cudaStream_t stream) {
  using Shape = GroupShape<WARPS>;
  auto kernel = layer_norm_rows_kernel<T, WARPS, ITERS, CENTERED>;
  const size_t parameter_bytes = 2 * (size_t)columns * sizeof(T);
  const int stage = parameter_bytes <= (size_t)kMaxStagedParameterBytes;
  const size_t smem = stage ? parameter_bytes : 0;
  if (smem > 48 * 1024) B200_CUDA_TRY(opt_in_dynamic_smem(kernel, kMaxStagedParameterBytes));
  const int grid = grid_for(rows, Shape::kGroups, resident_ctas(kernel, Shape::kCtaThreads, smem));
  kernel<<<grid, Shape::kCtaThreads, smem, stream>>>(x, w, b, y, rows, (int)columns, xp, yp,
                                                     inverse_features, epsilon, stage);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

template <typename T, int WARPS, bool CENTERED>
int layer_norm_pick_iters(int iters, const T *x, const T *w, const T *b, T *y, int64_t rows,
                          int64_t columns, int64_t xp, int64_t yp, float inv, float eps,
                          cudaStream_t stream) {
  constexpr int kMaxIters = 32 / Element<T>::kVec;
  switch (iters) {
  case 1: return launch_layer_norm_rows<T, WARPS, 1, CENTERED>(x, w, b, y, rows, columns, xp, yp, inv, eps, stream);
  case 2: return launch_layer_norm_rows<T, WARPS, 2, CENTERED>(x, w, b, y, rows, columns, xp, yp, inv, eps, stream);
  case 4: return launch_layer_norm_rows<T, WARPS, 4, CENTERED>(x, w, b, y, rows, columns, xp, yp, inv, eps, stream);
  default:
    return launch_layer_norm_rows<T, WARPS, kMaxIters, CENTERED>(x, w, b, y, rows, columns, xp, yp, inv, eps, stream);
  }
}

template <typename T, bool CENTERED>
int layer_norm_typed(const T *x, const T *w, int64_t ws, const T *b, int64_t bs, T *y, int64_t rows,
                     int64_t columns, int64_t xp, int64_t yp, float inv, float eps,
                     cudaStream_t stream) {
  RowPlan plan;
  const bool vector_ok = aligned16(x) && aligned16(y) && aligned16(w) && aligned16(b) && ws == 1 &&
                         bs == 1 && xp % Element<T>::kVec == 0 && yp % Element<T>::kVec == 0 &&
                         plan_row<T>(columns, &plan);
  if (!vector_ok) {
    const int grid = (int)(rows < (int64_t)sm_count() * 8 ? rows : (int64_t)sm_count() * 8);
    layer_norm_generic_kernel<T, CENTERED><<<grid, 256, 0, stream>>>(
        x, w, ws, b, bs, y, rows, columns, xp, yp, inv, eps);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  constexpr int kMaxIters = 32 / Element<T>::kVec;
#define B200_LN(W) launch_layer_norm_rows<T, W, kMaxIters, CENTERED>(x, w, b, y, rows, columns, xp, yp, inv, eps, stream)
  switch (plan.warps) {
  case 1: return layer_norm_pick_iters<T, 1, CENTERED>(plan.iters, x, w, b, y, rows, columns, xp, yp, inv, eps, stream);
  case 2: return B200_LN(2);
  case 4: return B200_LN(4);
  case 8: return B200_LN(8);
  case 16: return B200_LN(16);
  default: return B200_LN(32);
  }
#undef B200_LN
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" int b200_softmax(const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                            void *y, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                            int32_t dtype, void *stream) {
  if (x_d0 < 0 || x_d1 < 0 || x_d0 != y_d0 || x_d1 != y_d1)
    return fail(B200_ERR_INVALID_ARGUMENT, "softmax: x is %lldx%lld but y is %lldx%lld",
                (long long)x_d0, (long long)x_d1, (long long)y_d0, (long long)y_d1);
  if (x_d0 == 0 || x_d1 == 0) return B200_OK;
  if (!x || !y) return fail(B200_ERR_INVALID_ARGUMENT, "softmax: null buffer");
  if ((x_d1 > 1 && (x_s1 != 1 || y_s1 != 1)) || x_s0 < 0 || y_s0 < 0)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "softmax: inner strides must be 1 (got %lld, %lld)",
                (long long)x_s1, (long long)y_s1);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
  case B200_F32: return softmax_typed<float>((const float *)x, (float *)y, x_d0, x_d1, x_s0, y_s0, s);
  case B200_F16: return softmax_typed<__half>((const __half *)x, (__half *)y, x_d0, x_d1, x_s0, y_s0, s);
  case B200_BF16:
    return softmax_typed<__nv_bfloat16>((const __nv_bfloat16 *)x, (__nv_bfloat16 *)y, x_d0, x_d1, x_s0, y_s0, s);
  default: return fail(B200_ERR_INVALID_ARGUMENT, "softmax: unknown element type %d", dtype);
  }
}

extern "C" int b200_layer_norm(const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                               const void *weight, int64_t w_d0, int64_t w_s0,
                               const void *bias, int64_t b_d0, int64_t b_s0,
                               void *y, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                               float inverse_features, float epsilon,
                               int32_t dtype, int32_t centered, void *stream) {
  if (x_d0 < 0 || x_d1 < 0 || x_d0 != y_d0 || x_d1 != y_d1 || w_d0 != x_d1 || b_d0 != x_d1)
    return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm: inconsistent extents");
  if (x_d0 == 0 || x_d1 == 0) return B200_OK;
  if (!x || !y || !weight || !bias) return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm: null buffer");
  if ((x_d1 > 1 && (x_s1 != 1 || y_s1 != 1)) || x_s0 < 0 || y_s0 < 0)
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "layer_norm: inner strides of x and y must be 1");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200_LN_CALL(T, C)                                                                       \
  layer_norm_typed<T, C>((const T *)x, (const T *)weight, w_s0, (const T *)bias, b_s0, (T *)y,   \
                         x_d0, x_d1, x_s0, y_s0, inverse_features, epsilon, s)
  switch (dtype) {
  case B200_F32: return centered ? B200_LN_CALL(float, true) : B200_LN_CALL(float, false);
  case B200_F16: return centered ? B200_LN_CALL(__half, true) : B200_LN_CALL(__half, false);
  case B200_BF16: return centered ? B200_LN_CALL(__nv_bfloat16, true) : B200_LN_CALL(__nv_bfloat16, false);
  default: return fail(B200_ERR_INVALID_ARGUMENT, "layer_norm: unknown element type %d", dtype);
  }
#undef B200_LN_CALL
}

extern "C" int b200_softmax_backward(const void *p, int64_t p_d0, int64_t p_d1, int64_t p_s0, int64_t p_s1,
                                     const void *dy, int64_t u_d0, int64_t u_d1, int64_t u_s0, int64_t u_s1,
                                     void *dx, int64_t g_d0, int64_t g_d1, int64_t g_s0, int64_t g_s1,
                                     int32_t dtype, void *stream) {
  if (p_d0 < 0 || p_d1 < 0 || u_d0 != p_d0 || u_d1 != p_d1 || g_d0 != p_d0 || g_d1 != p_d1)
    return fail(B200_ERR_INVALID_ARGUMENT, "softmax_backward: probabilities, upstream and gradient must share one shape");
  if (p_d0 == 0 || p_d1 == 0) return B200_OK;
  if (!p || !dy || !dx) return fail(B200_ERR_INVALID_ARGUMENT, "softmax_backward: null buffer");
  if (dtype != B200_F32) return fail(B200_ERR_INVALID_ARGUMENT, "softmax_backward: element type %d is not f32", dtype);
  if (p_d1 > 1 && (p_s1 != 1 || u_s1 != 1 || g_s1 != 1))
    return fail(B200_ERR_UNSUPPORTED_LAYOUT, "softmax_backward: inner strides must be 1");
  if (p_d1 > INT32_MAX) return fail(B200_ERR_UNSUPPORTED_LAYOUT, "softmax_backward: row too long");
  cudaStream_t queue = static_cast<cudaStream_t>(stream);
  const uintptr_t pa = reinterpret_cast<uintptr_t>(p), ua = reinterpret_cast<uintptr_t>(dy), ga = reinterpret_cast<uintptr_t>(dx);
  const bool same_alignment = (pa & 3) == 0 && (pa & 15) == (ua & 15) && (pa & 15) == (ga & 15) &&
                              (p_s0 - u_s0) % 4 == 0 && (p_s0 - g_s0) % 4 == 0;
  if (same_alignment && p_d1 <= 8 * 1024) {
    const int per_thread = (int)((p_d1 / 4 + 255) / 256);
    auto launch = [&](auto kernel) {
      const int64_t limit = (int64_t)sm_count() * resident_ctas(kernel, 256, 0);
      kernel<<<(unsigned)(p_d0 < limit ? p_d0 : limit), 256, 0, queue>>>((const float *)p, (const float *)dy, (float *)dx,
                                                                        p_d0, (int)p_d1, p_s0, u_s0, g_s0);
    };
    if (per_thread <= 1) launch(softmax_backward_vector_kernel<1>);
    else if (per_thread <= 2) launch(softmax_backward_vector_kernel<2>);
    else if (per_thread <= 4) launch(softmax_backward_vector_kernel<4>);
    else launch(softmax_backward_vector_kernel<8>);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
  }
  const size_t row_bytes = 2 * (size_t)p_d1 * sizeof(float);
  const int staged = row_bytes <= 96 * 1024;
  const size_t smem = staged ? row_bytes : 0;
  if (smem > 48 * 1024) B200_CUDA_TRY(opt_in_dynamic_smem(softmax_backward_kernel, 96 * 1024));
  const int resident = resident_ctas(softmax_backward_kernel, 256, smem);
  const int64_t wanted = p_d0, limit = (int64_t)sm_count() * resident;
  softmax_backward_kernel<<<(unsigned)(wanted < limit ? wanted : limit), 256, smem, static_cast<cudaStream_t>(stream)>>>(
      (const float *)p, (const float *)dy, (float *)dx, p_d0, (int)p_d1, p_s0, u_s0, g_s0, staged);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}
