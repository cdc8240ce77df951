// Shared internals of libmtfc: status codes, the thread-local error string,
// dtype helpers and launch-geometry helpers.  Nothing here is exported.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mtfc.h"

namespace mtfc {

// Records a message retrievable through mtfc_last_error() and returns `code`.
int fail(int code, const char* fmt, ...);

// Per-device status word written by kernels whose bounded waits ran out.
// Allocated on first use for the current device; returns nullptr on failure.
int* device_status_word();

// Number of SMs of the current device (cached per device).
int sm_count();

// Adds `n` to the process-wide count of kernels this library has launched.
void count_launch(int n);

inline int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return MTFC_OK;
  return fail(MTFC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define MTFC_CUDA(call)                                        \
  do {                                                         \
    int _rc = ::mtfc::check_cuda((call), #call);               \
    if (_rc != MTFC_OK) return _rc;                            \
  } while (0)

#define MTFC_LAUNCH_CHECK(name)                                \
  do {                                                         \
    int _rc = ::mtfc::check_cuda(cudaGetLastError(), name);    \
    if (_rc != MTFC_OK) return _rc;                            \
  } while (0)

inline size_t dtype_size(int dtype) {
  switch (dtype) {
    case MTFC_F32: return 4;
    case MTFC_BF16: return 2;
    case MTFC_I32: return 4;
    default: return 0;
  }
}

// Grid size for a grid-stride kernel: enough blocks to cover `n` items at
// `per_block` items each, capped at `waves` resident waves over all SMs.
inline unsigned grid_for(long long n, int per_block, int blocks_per_sm = 8) {
  long long need = (n + per_block - 1) / per_block;
  long long cap = (long long)sm_count() * blocks_per_sm;
  if (need < 1) need = 1;
  return (unsigned)(need < cap ? need : cap);
}

// ---- device-side scalar load/store in fp32 regardless of storage type ----
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ float to_f32<int>(int v) { return (float)v; }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ int from_f32<int>(float v) { return (int)v; }

}  // namespace mtfc
