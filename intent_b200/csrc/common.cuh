// Shared host/device helpers of the intent_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/intent_b200.h"

namespace b200 {

// ---- host side: status + last-error text --------------------------------
int fail(int status, const char *format, ...);
int cuda_fail(cudaError_t error, const char *what);
int sm_count();  // multiprocessors of the current device (cached per device)
// Opts `kernel` into `bytes` of dynamic shared memory on the CURRENT device.  The attribute is
// per device and per function, so the answer is remembered per (function, device); an error is
// returned on every call that meets it, not only on the first.
cudaError_t opt_in_dynamic_smem(const void *kernel, size_t bytes);
template <typename Kernel> cudaError_t opt_in_dynamic_smem(Kernel kernel, size_t bytes) {
  return opt_in_dynamic_smem(reinterpret_cast<const void *>(kernel), bytes);
}

#define B200_CUDA_TRY(expression)                                   \
  do {                                                              \
    cudaError_t error_ = (expression);                              \
    if (error_ != cudaSuccess) return ::b200::cuda_fail(error_, #expression); \
  } while (0)

inline bool aligned16(const void *pointer) { return (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0; }

// ---- device side ---------------------------------------------------------
template <typename T> struct Element;
template <> struct Element<float> {
  static constexpr int kVec = 4;  // elements per 128-bit access
  __device__ static float widen(float v) { return v; }
  __device__ static float narrow(float v) { return v; }
};
template <> struct Element<__half> {
  static constexpr int kVec = 8;
  __device__ static float widen(__half v) { return __half2float(v); }
  __device__ static __half narrow(float v) { return __float2half_rn(v); }
};
template <> struct Element<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 narrow(float v) { return __float2bfloat16_rn(v); }
};

// One 128-bit global load / store of kVec elements, widened to f32.
template <typename T>
__device__ __forceinline__ void load_vector(const T *pointer, float (&out)[Element<T>::kVec]) {
  const uint4 raw = *reinterpret_cast<const uint4 *>(pointer);
  const T *lanes = reinterpret_cast<const T *>(&raw);
#pragma unroll
  for (int i = 0; i < Element<T>::kVec; ++i) out[i] = Element<T>::widen(lanes[i]);
}
template <typename T>
__device__ __forceinline__ void store_vector(T *pointer, const float (&in)[Element<T>::kVec]) {
  uint4 raw;
  T *lanes = reinterpret_cast<T *>(&raw);
#pragma unroll
  for (int i = 0; i < Element<T>::kVec; ++i) lanes[i] = Element<T>::narrow(in[i]);
  *reinterpret_cast<uint4 *>(pointer) = raw;
}

// maximum_num: a one-sided NaN is ignored (fmaxf does exactly that).
__device__ __forceinline__ float maximum_num(float a, float b) { return fmaxf(a, b); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = maximum_num(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Reduction over the WARPS warps that share one row (WARPS == 1: shuffles only).
// `scratch` holds WARPS floats per row group; every call uses a fresh slot so
// one __syncthreads-free named barrier per reduction is enough.
template <int WARPS, bool IS_MAX>
__device__ __forceinline__ float group_reduce(float v, float *scratch, int warp_in_group, int barrier_id) {
  v = IS_MAX ? warp_max(v) : warp_sum(v);
  if (WARPS == 1) return v;
  if ((threadIdx.x & 31) == 0) scratch[warp_in_group] = v;
  asm volatile("bar.sync %0, %1;" ::"r"(barrier_id), "r"(WARPS * 32) : "memory");
  float total = scratch[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) total = IS_MAX ? maximum_num(total, scratch[w]) : total + scratch[w];
  return total;
}

}  // namespace b200
