// Host-side plumbing shared by every entry point: status text, last-error
// buffer, device facts.  No kernel lives here.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace b200 {

static thread_local char last_error[512];

int fail(int status, const char *format, ...) {
  va_list arguments;
  va_start(arguments, format);
  vsnprintf(last_error, sizeof last_error, format, arguments);
  va_end(arguments);
  return status;
}

int cuda_fail(cudaError_t error, const char *what) {
  snprintf(last_error, sizeof last_error, "%s: %s (%s)", what, cudaGetErrorString(error),
           cudaGetErrorName(error));
  return B200_ERR_CUDA;
}

cudaError_t opt_in_dynamic_smem(const void *kernel, size_t bytes) {
  static std::mutex lock;
  static std::map<std::pair<const void *, int>, size_t> granted;
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return error;
  std::lock_guard<std::mutex> guard(lock);
  auto found = granted.find({kernel, device});
  if (found != granted.end() && found->second >= bytes) return cudaSuccess;
  error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (error == cudaSuccess) granted[{kernel, device}] = bytes;
  return error;
}

int sm_count() {
  static int cached[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
  if (cached[device] == 0) {
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    cached[device] = count;
  }
  return cached[device];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" const char *b200_status_string(int status) {
  switch (status) {
  case B200_OK: return "ok";
  case B200_ERR_INVALID_ARGUMENT: return "invalid argument";
  case B200_ERR_UNSUPPORTED_LAYOUT: return "unsupported layout";
  case B200_ERR_CUDA: return "CUDA error";
  case B200_ERR_DEVICE: return "device is not sm_100";
  case B200_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
  default: return "unknown status";
  }
}

extern "C" int b200_last_error(char *buffer, int64_t capacity) {
  if (!buffer || capacity <= 0) return B200_ERR_INVALID_ARGUMENT;
  strncpy(buffer, last_error, (size_t)capacity - 1);
  buffer[capacity - 1] = 0;
  return B200_OK;
}

extern "C" int b200_device_check(int device) {
  int major = 0, minor = 0;
  B200_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  B200_CUDA_TRY(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device));
  if (major != 10 || minor != 0)
    return fail(B200_ERR_DEVICE, "device %d has compute capability %d.%d; this library holds sm_100a code only",
                device, major, minor);
  return B200_OK;
}

extern "C" int b200_workspace_status(const void *workspace, int32_t *detail, void *stream) {
  if (!workspace) return fail(B200_ERR_INVALID_ARGUMENT, "workspace_status: null workspace");
  int32_t words[2] = {0, 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_CUDA_TRY(cudaMemcpyAsync(words, workspace, sizeof words, cudaMemcpyDeviceToHost, s));
  B200_CUDA_TRY(cudaStreamSynchronize(s));
  if (detail) *detail = words[1];
  if (words[0] == 2)   // only the checked build (-DB200_CHECKED) writes this
    return fail(B200_ERR_INVALID_ARGUMENT, "checked build: an index or offset was outside its array (row %d)", words[1]);
  if (words[0] != 0)
    return fail(B200_ERR_DEVICE_TIMEOUT, "a bounded device-side wait gave up (site %d)", words[1]);
  return B200_OK;
}

extern "C" int b200_device_capabilities(int device, int64_t *facts) {
  if (!facts) return fail(B200_ERR_INVALID_ARGUMENT, "device_capabilities: null output");
  const cudaDeviceAttr attributes[8] = {
      cudaDevAttrMultiProcessorCount, cudaDevAttrMaxSharedMemoryPerMultiprocessor,
      cudaDevAttrMaxSharedMemoryPerBlockOptin, cudaDevAttrMaxRegistersPerMultiprocessor,
      cudaDevAttrMaxThreadsPerBlock, cudaDevAttrComputeCapabilityMajor,
      cudaDevAttrComputeCapabilityMinor, cudaDevAttrSingleToDoublePrecisionPerfRatio};
  for (int i = 0; i < 8; ++i) {
    int value = 0;
    B200_CUDA_TRY(cudaDeviceGetAttribute(&value, attributes[i], device));
    facts[i] = value;
  }
  return B200_OK;
}
