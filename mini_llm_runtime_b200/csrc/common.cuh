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

// dtype codes shared with ops/cuda_ops.py
#define MLR_F32 0
#define MLR_BF16 1

#define MLR_EXPORT extern "C" __attribute__((visibility("default")))

namespace mlr {

typedef __nv_bfloat16 bf16;

// What the device keeps of one live request, indexed by the request's slot: eight 32-bit words, so
// that the host can scatter whole records with the same kernel that scatters block-table rows.
// `length` is the number of tokens the cache holds (= the position of the request's next token);
// `counter` is the index of the token the request samples next (the counter of its random stream).
struct SlotState {
  int length;
  int last_token;
  int counter;
  float temperature;
  unsigned int seed_low, seed_high;
  int spare[2];
};
static_assert(sizeof(SlotState) == 32, "the host packs slot records as eight 32-bit words");

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

// Programmatic dependent launch.  Every kernel of this package is launched with the attribute that
// lets it start while the kernel before it on the stream is still running; it then does whatever
// does not depend on that kernel (barrier set-up, tensor-memory allocation, weight loads) and calls
// pdl_wait() before its first access to memory an earlier kernel wrote and before its own first
// write.  pdl_wait() returns once the preceding kernel has completed and its writes are visible;
// since every kernel waits before it finishes, completion is transitive along the stream.
// pdl_trigger() tells the scheduler that the next kernel may be brought in.  Launched without the
// attribute both are no-ops.
// Because a kernel may begin before its input exists, inputs written by earlier kernels are never
// read through the read-only (non-coherent) path: their pointers carry no __restrict__, and
// explicit loads use __ldcg, not __ldg.  Weights and the step's metadata may.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool& pdl_enabled() {
  static bool enabled = true;
  return enabled;
}

// silu(gate) * up in the float32 epilogues of the bfloat16 products: exponential and division by the
// hardware's approximate instructions (about 2 ulp of float32, far inside the bfloat16 rounding that
// follows).  The IEEE division cost 110 cycles per output in the tcgen05 GEMM's epilogue: 4.6 us of
// the 14 us a CTA of the 0.5B gate/up product lives.  The clamp keeps 1 + e inside the range where
// the approximate division is defined; below -80 the result is below 1e-33 in magnitude either way.
__device__ __forceinline__ float silu_times(float gate, float up) {
  const float e = __expf(fminf(-gate, 80.f));
  return __fdividef(gate * up, 1.f + e);
}

// One rotate-half pair: (x1, x2) turned by the angle whose sine and cosine are given.  Written with
// explicit roundings so that every kernel that rotates gets the same bits.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float sine, float cosine, float* y1, float* y2) {
  *y1 = __fsub_rn(__fmul_rn(x1, cosine), __fmul_rn(x2, sine));
  *y2 = __fadd_rn(__fmul_rn(x2, cosine), __fmul_rn(x1, sine));
}

template <typename... KernelArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared, cudaStream_t stream,
                          Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// The same for a grid of thread-block clusters of `cluster_x` CTAs along x (grid.x a multiple of it).
// `balanced`: the blocks of a cluster may go wherever the hardware finds room for them, instead of
// being spread one per SM: large clusters then find room sooner beside the kernel before them (the
// decode attention's clusters of 16 in a step of 8 requests: 646 -> 633 us per step).  Not for
// kernels whose CTAs must sit on the two SMs of a pair.
template <typename... KernelArgs, typename... Args>
inline void launch_clustered(bool balanced, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                             cudaStream_t stream, int cluster_x, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[3];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = (unsigned)cluster_x;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  int count = 1;
  if (balanced) {
    attribute[count].id = cudaLaunchAttributeClusterSchedulingPolicyPreference;
    attribute[count].val.clusterSchedulingPolicyPreference = cudaClusterSchedulingPolicyLoadBalancing;
    ++count;
  }
  if (pdl_enabled()) {
    attribute[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
  }
  config.attrs = attribute;
  config.numAttrs = count;
  cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}
template <typename... KernelArgs, typename... Args>
inline void launch_kernel_clustered(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                                    cudaStream_t stream, int cluster_x, Args&&... args) {
  launch_clustered(false, kernel, grid, block, shared, stream, cluster_x, static_cast<Args&&>(args)...);
}
template <typename... KernelArgs, typename... Args>
inline void launch_kernel_clustered_balanced(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                                             cudaStream_t stream, int cluster_x, Args&&... args) {
  launch_clustered(true, kernel, grid, block, shared, stream, cluster_x, static_cast<Args&&>(args)...);
}

// One switch per library (each .cu is its own shared object).
#define MLR_DEFINE_PDL_SWITCH \
  MLR_EXPORT void mlr_set_pdl(int enabled) { mlr::pdl_enabled() = enabled != 0; }

// Streaming multiprocessors of the current device, asked once per process and device; planners
// size grids and split counts from it.
inline int sm_count() {
  static int cached[64] = {0};
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

inline int launch_status() {
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? MLR_OK : (int)err;
}

}  // namespace mlr
