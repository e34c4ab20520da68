// Shared helpers of the sm_100a kernels: element types, float conversion, warp and block
// reductions with a fixed order, and the status codes the C entry points return.
//
// Every entry point is `extern "C"`, takes raw device pointers plus a CUDA stream, launches on
// that stream and returns 0, a positive cudaError_t, or one of the negative codes below.  The
// Python side turns a non-zero code into an exception; nothing falls back to another backend.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define MLR_OK 0
#define MLR_BAD_DTYPE (-1)
#define MLR_BAD_SIZE (-2)
#define MLR_BAD_ALIGNMENT (-3)
#define MLR_TOO_LARGE (-4)
#define MLR_DEVICE_FLAG (-5)

// dtype codes shared with ops/library.py
#define MLR_F32 0
#define MLR_BF16 1

#define MLR_EXPORT extern "C" __attribute__((visibility("default")))

namespace mlr {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a whole block; every thread gets the result.  `scratch` holds 32 floats.
// The order of additions depends only on blockDim, never on the data.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : 0.f;
  total = warp_sum(total);
  return total;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int warps = (blockDim.x + 31) >> 5;
  float total = (lane < warps) ? scratch[lane] : -INFINITY;
  total = warp_max(total);
  return total;
}

inline int launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? MLR_OK : (int)err;
}

}  // namespace mlr
