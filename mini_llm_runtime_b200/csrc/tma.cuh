// Shared by the kernels that move tiles with the tensor memory accelerator: mbarrier helpers with
// bounded waits, the 2-D tile load, and the host-side tensor-map encoder (fetched from the driver
// at run time, so that the libraries link against the runtime only).
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT_NS it stores a code into the caller's
// error word (host-visible memory) and returns false; the caller stops issuing work and returns.
// Loads use no cluster multicast.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>

#include "common.cuh"

namespace mlr {

constexpr unsigned long long WAIT_LIMIT_NS = 1000000000ull;   // a wait gives up after one second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false (and an error code in *error_word) if the phase does not complete in time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* error_word, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_timer_ns();
  do {
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
  } while (global_timer_ns() - start < WAIT_LIMIT_NS);
  *((volatile int*)error_word) = code;
  __threadfence_system();
  return false;
}

__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

}  // namespace mlr

// ---------------------------------------------------------------- host side
namespace mlr {

static inline PFN_cuTensorMapEncodeTiled_v12000 encode_tiled() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)ptr;
  }
  return fn;
}

// rows x K bfloat16, row-major; box = [box_rows x 64], 128-byte swizzle, out-of-range reads give zero.
static inline bool make_tile_map(CUtensorMap* map, const void* base, long long rows, int K, int box_rows) {
  auto encode = encode_tiled();
  if (encode == nullptr) return false;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same through a cache: encoding a map costs a few microseconds on the host, and a model step
// asks for the same maps (weights, cache pools, activation buffers the allocator hands out again)
// over and over.  A direct-mapped table keyed by everything the map depends on; an entry that
// another key hashes onto is simply encoded again.  The map is copied out to the caller, so that a
// later lookup can never change a map that an earlier lookup returned.  Not thread-safe: the
// kernels are launched from one host thread.
struct TileMapKey {
  const void* base;
  long long rows;
  long long width;
  int box_rows;
  bool operator==(const TileMapKey& other) const {
    return base == other.base && rows == other.rows && width == other.width && box_rows == other.box_rows;
  }
};

static inline bool cached_tile_map(CUtensorMap* out, const void* base, long long rows, long long width, int box_rows) {
  constexpr int SLOTS = 4096;
  static TileMapKey keys[SLOTS];
  static CUtensorMap maps[SLOTS];
  const TileMapKey key{base, rows, width, box_rows};
  unsigned long long h = (unsigned long long)(uintptr_t)base * 0x9E3779B97F4A7C15ull;
  h ^= (unsigned long long)rows * 0xBF58476D1CE4E5B9ull + (unsigned long long)width * 0x94D049BB133111EBull +
       (unsigned long long)box_rows;
  const int slot = (int)((h >> 40) % SLOTS);
  if (!(keys[slot] == key) || base == nullptr) {
    auto encode = encode_tiled();
    if (encode == nullptr) return false;
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)width * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t element_strides[2] = {1, 1};
    keys[slot] = TileMapKey{nullptr, 0, 0, 0};
    if (encode(&maps[slot], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
               element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
    keys[slot] = key;
  }
  *out = maps[slot];
  return true;
}

}  // namespace mlr
