// Decode attention: one new token per request over its paged bfloat16 K/V cache, split over the
// keys (split-KV) and shared across the query heads of a kv head (GQA).
//
// The reference's kernel gives one CTA to each (request, query head), walks the keys serially and
// so re-reads every key and value once per query head of the group (csrc/paged_attention_cuda.cu:
// 25-106); its experimental split variant cuts the keys into S partitions per call and merges
// them in a second kernel (csrc/paged_attention_split_cuda.cu:18-88).  Here a CTA owns
// (request, kv head, chunk of keys): every key and value is read once for the whole group of query
// heads, chunks are `chunk` keys long and aligned to absolute positions, and the CTA that finishes
// last for a (request, kv head) merges the chunks' (max, sum, accumulator) states in chunk order,
// so no second launch and no CTA ever waits for another.
//
// Per warp and 32 keys: each lane scores one key against all query heads of the group (float32
// dot products, query pre-scaled by head_dim^-0.5), the online-softmax recurrence of the reference
// (m' = max(m, s); l = l e^{m-m'} + e^{s-m'}; acc likewise) runs per head across the warp, then
// the lanes switch to owning output dimensions and add probability x value rows.
// head_dim 64 or 128, up to 8 query heads per kv head; other sizes use the generic kernel.
#include "common.cuh"

#pragma GCC visibility push(default)
#include "attention_decode_static.h"
#pragma GCC visibility pop

namespace mlr {

constexpr int GROUP_MAX = 8;
constexpr int DECODE_WARPS = 4;

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 two = __bfloat1622float2(pairs[i]);
    f[2 * i] = two.x;
    f[2 * i + 1] = two.y;
  }
}

template <int D>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
decode_attention_kernel(const bf16* q, const bf16* k_pool,
                        const bf16* v_pool, bf16* __restrict__ out,
                        const int* __restrict__ decode_seg, const int* __restrict__ seg_q_start,
                        const int* __restrict__ seg_pos0, const int* __restrict__ block_table, const int* __restrict__ seg_slot,
                        int table_width, int heads, int kv_heads, int page_size, int window, float scale,
                        int chunk, float* __restrict__ scratch, int* __restrict__ counters, int max_splits) {
  pdl_trigger();
  pdl_wait();
  constexpr int PER_LANE = D / 32;            // output dimensions each lane owns
  constexpr int STATE = D + 2;                // floats per partial state: max, sum, accumulator
  __shared__ float q_s[GROUP_MAX][D];
  __shared__ float p_s[DECODE_WARPS][GROUP_MAX][32];
  __shared__ float m_s[DECODE_WARPS][GROUP_MAX], l_s[DECODE_WARPS][GROUP_MAX];
  __shared__ float acc_s[DECODE_WARPS][GROUP_MAX][D];
  __shared__ int last_flag;

  const int group = heads / kv_heads;
  const int split = blockIdx.x, kv_head = blockIdx.y, index = blockIdx.z;
  const int seg = decode_seg[index];
  const int row = seg_q_start[seg];
  const int position = seg_pos0[seg];                       // the row's own position; it sees keys <= position
  const int lowest = window > 0 ? max(0, position - window + 1) : 0;
  const int first_chunk = lowest / chunk;
  // A context that needs more chunks than the grid has CTAs for it (position >= max_splits *
  // chunk) is still covered: the last CTA walks on to the row's own position.
  const int splits = min(position / chunk - first_chunk + 1, max_splits);
  if (split >= splits) return;
  const int k_begin = max(lowest, (first_chunk + split) * chunk);
  const int k_end = split == splits - 1 ? position + 1 : (first_chunk + split + 1) * chunk;
  const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i < group * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    q_s[g][d] = to_float(q[((size_t)row * heads + kv_head * group + g) * D + d]) * scale;
  }
  __syncthreads();

  float m[GROUP_MAX], l[GROUP_MAX], acc[GROUP_MAX][PER_LANE];
#pragma unroll
  for (int g = 0; g < GROUP_MAX; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) acc[g][i] = 0.f;
  }

  for (int base = k_begin + warp * 32; base < k_end; base += DECODE_WARPS * 32) {
    const int key = base + lane;
    const bool valid = key < k_end;
    long long row_offset = 0;
    if (valid) {
      const int page = table[key / page_size];
      row_offset = (((long long)page * kv_heads + kv_head) * page_size + key % page_size) * D;
    }
    // ---- scores of this lane's key against every query head of the group
    float s[GROUP_MAX];
#pragma unroll
    for (int g = 0; g < GROUP_MAX; ++g) s[g] = 0.f;
    if (valid) {
      const uint4* k_row = reinterpret_cast<const uint4*>(k_pool + row_offset);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        float kf[8];
        unpack8(__ldcg(k_row + c), kf);
#pragma unroll
        for (int g = 0; g < GROUP_MAX; ++g) {
          if (g < group) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][c * 8]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][c * 8 + 4]);
            s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] +
                    qb.x * kf[4] + qb.y * kf[5] + qb.z * kf[6] + qb.w * kf[7];
          }
        }
      }
    }
    // ---- online softmax per head across the warp's 32 keys
    float alpha[GROUP_MAX];
#pragma unroll
    for (int g = 0; g < GROUP_MAX; ++g) {
      alpha[g] = 1.f;
      if (g < group) {
        const float score = valid ? s[g] : -INFINITY;
        const float m_new = fmaxf(m[g], warp_max(score));   // finite: lane 0's key is always valid
        alpha[g] = __expf(m[g] - m_new);
        const float prob = valid ? __expf(score - m_new) : 0.f;
        l[g] = l[g] * alpha[g] + warp_sum(prob);
        m[g] = m_new;
        p_s[warp][g][lane] = prob;
      }
    }
    __syncwarp();
    // ---- probability x value: lanes now own output dimensions
#pragma unroll
    for (int g = 0; g < GROUP_MAX; ++g)
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) acc[g][i] *= alpha[g];
    const int count = min(32, k_end - base);
    for (int j0 = 0; j0 < count; j0 += 4) {
      float v[4][PER_LANE];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const long long offset = __shfl_sync(0xffffffffu, row_offset, (j0 + jj) & 31);
        if (j0 + jj < count) {
          if constexpr (PER_LANE == 2) {
            const float2 two = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(v_pool + offset + lane * 2));
            v[jj][0] = two.x;
            v[jj][1] = two.y;
          } else {
            const uint2 raw = *reinterpret_cast<const uint2*>(v_pool + offset + lane * 4);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            v[jj][0] = a.x; v[jj][1] = a.y; v[jj][PER_LANE - 2] = b.x; v[jj][PER_LANE - 1] = b.y;
          }
        } else {
#pragma unroll
          for (int i = 0; i < PER_LANE; ++i) v[jj][i] = 0.f;
        }
      }
#pragma unroll
      for (int g = 0; g < GROUP_MAX; ++g) {
        if (g < group) {
          const float4 pr = *reinterpret_cast<const float4*>(&p_s[warp][g][j0]);
#pragma unroll
          for (int i = 0; i < PER_LANE; ++i)
            acc[g][i] += pr.x * v[0][i] + pr.y * v[1][i] + pr.z * v[2][i] + pr.w * v[3][i];
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the four warps of this CTA
#pragma unroll
  for (int g = 0; g < GROUP_MAX; ++g) {
    if (g < group) {
      if (lane == 0) { m_s[warp][g] = m[g]; l_s[warp][g] = l[g]; }
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i) acc_s[warp][g][lane * PER_LANE + i] = acc[g][i];
    }
  }
  __syncthreads();
  const size_t state_base = ((size_t)index * heads + kv_head * group) * max_splits;   // + g*max_splits + split
  for (int item = threadIdx.x; item < group * D; item += blockDim.x) {
    const int g = item / D, d = item - g * D;
    float m_all = m_s[0][g];
#pragma unroll
    for (int w = 1; w < DECODE_WARPS; ++w) m_all = fmaxf(m_all, m_s[w][g]);
    float l_all = 0.f, a_all = 0.f;
#pragma unroll
    for (int w = 0; w < DECODE_WARPS; ++w) {
      const float factor = __expf(m_s[w][g] - m_all);     // a warp without keys has m = -inf: factor 0
      l_all += l_s[w][g] * factor;
      a_all += acc_s[w][g][d] * factor;
    }
    if (splits == 1) {
      out[((size_t)row * heads + kv_head * group + g) * D + d] = __float2bfloat16_rn(a_all / l_all);
    } else {
      float* state = scratch + (state_base + (size_t)g * max_splits + split) * STATE;
      state[2 + d] = a_all;
      if (d == 0) { state[0] = m_all; state[1] = l_all; }
    }
  }
  if (splits == 1) return;

  // ---- the CTA that arrives last for this (request, kv head) merges all chunks, in chunk order
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_flag = (atomicAdd(&counters[index * kv_heads + kv_head], 1) == splits - 1);
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  for (int item = threadIdx.x; item < group * D; item += blockDim.x) {
    const int g = item / D, d = item - g * D;
    const float* states = scratch + (state_base + (size_t)g * max_splits) * STATE;
    float m_all = -INFINITY;
    for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, __ldcg(&states[(size_t)s * STATE]));
    float l_all = 0.f, a_all = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float factor = __expf(__ldcg(&states[(size_t)s * STATE]) - m_all);
      l_all += __ldcg(&states[(size_t)s * STATE + 1]) * factor;
      a_all += __ldcg(&states[(size_t)s * STATE + 2 + d]) * factor;
    }
    out[((size_t)row * heads + kv_head * group + g) * D + d] = __float2bfloat16_rn(a_all / l_all);
  }
  if (threadIdx.x == 0) counters[index * kv_heads + kv_head] = 0;   // ready for the next launch
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// Bytes of scratch for `rows` decode rows (float32 partial states).
MLR_EXPORT long long mlr_attention_decode_scratch(int rows, int heads, int head_dim, int max_splits) {
  return (long long)rows * heads * max_splits * (head_dim + 2) * 4;
}

// q, out: [all rows of the step, heads, head_dim] bfloat16; decode_seg: the segments (of one row
// each) this launch handles; max_splits sizes the grid: with max_splits >= ceil(longest context /
// chunk) every chunk has its own CTA; beyond that the last CTA of a row takes the rest.
static int decode_arguments_status(int rows, int heads, int kv_heads, int head_dim, int page_size, int chunk,
                                   int max_splits, int table_width) {
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || chunk <= 0 ||
      chunk % 32 != 0 || max_splits <= 0 || table_width <= 0)
    return MLR_BAD_SIZE;
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  if (heads / kv_heads > GROUP_MAX || rows > 65535 || kv_heads > 65535) return MLR_TOO_LARGE;
  return MLR_OK;
}

MLR_EXPORT int mlr_attention_decode(const void* q, const void* k_pool, const void* v_pool, void* out,
                                    const int* decode_seg, const int* seg_q_start, const int* seg_pos0,
                                    const int* block_table, const int* seg_slot, int table_width, int rows, int heads, int kv_heads,
                                    int head_dim, int page_size, int window, float scale, int chunk,
                                    int max_splits, void* scratch, int* counters, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  const int refused = decode_arguments_status(rows, heads, kv_heads, head_dim, page_size, chunk, max_splits, table_width);
  if (refused != MLR_OK) return refused;
  dim3 grid(max_splits, kv_heads, rows);
  if (head_dim == 64)
    launch_kernel(decode_attention_kernel<64>, dim3(grid), dim3(DECODE_WARPS * 32), 0, stream, 
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, decode_seg, seg_q_start, seg_pos0,
        block_table, seg_slot, table_width, heads, kv_heads, page_size, window, scale, chunk, (float*)scratch, counters,
        max_splits);
  else
    launch_kernel(decode_attention_kernel<128>, dim3(grid), dim3(DECODE_WARPS * 32), 0, stream, 
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, decode_seg, seg_q_start, seg_pos0,
        block_table, seg_slot, table_width, heads, kv_heads, page_size, window, scale, chunk, (float*)scratch, counters,
        max_splits);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate (declared in attention_decode_static.h).
// Same kernel as above; the partial states and the per-(request, kv head) counters live in a
// fixed array inside this library instead of a buffer the caller allocates.
// ---------------------------------------------------------------------------------------------
namespace mlr {

constexpr size_t STATIC_STATE_BYTES = 4u << 20;       // partial softmax states
constexpr size_t STATIC_COUNTER_BYTES = 64u << 10;    // 16384 counters
static __device__ __align__(256) unsigned char static_scratch[STATIC_STATE_BYTES + STATIC_COUNTER_BYTES];

constexpr int STATIC_MAX_DEVICES = 64;
static void* static_scratch_address[STATIC_MAX_DEVICES];   // device address of the array, per device

}  // namespace mlr

MLR_EXPORT long long mlr_attention_decode_static_capacity(void) { return (long long)STATIC_STATE_BYTES; }

MLR_EXPORT int mlr_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out,
                                           const int* decode_seg, const int* seg_q_start, const int* seg_pos0,
                                           const int* block_table, int table_width, int rows, int heads,
                                           int kv_heads, int head_dim, int page_size, int window, float scale,
                                           int chunk, int max_splits, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  // every check of the ordinary entry comes first, so that a refused call enqueues nothing at all
  const int refused = decode_arguments_status(rows, heads, kv_heads, head_dim, page_size, chunk, max_splits, table_width);
  if (refused != MLR_OK) return refused;
  // Refuse what does not fit the fixed array: the caller cannot be given more, and must not be
  // given less than the kernel will write.
  if (mlr_attention_decode_scratch(rows, heads, head_dim, max_splits) > (long long)STATIC_STATE_BYTES ||
      (size_t)rows * kv_heads * sizeof(int) > STATIC_COUNTER_BYTES)
    return MLR_TOO_LARGE;
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= STATIC_MAX_DEVICES) return MLR_TOO_LARGE;
  if (static_scratch_address[device] == nullptr) {
    // In host code `static_scratch` is only a handle; the kernel needs the array's address on the
    // current device, which the runtime reports here.  Done once per device.
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, static_scratch);
    if (err != cudaSuccess) return (int)err;
    static_scratch_address[device] = address;
  }
  unsigned char* base = (unsigned char*)static_scratch_address[device];
  int* counters = (int*)(base + STATIC_STATE_BYTES);
  // The array keeps whatever the previous call left; the counters must start at zero.
  err = cudaMemsetAsync(counters, 0, (size_t)rows * kv_heads * sizeof(int), stream);
  if (err != cudaSuccess) return (int)err;
  return mlr_attention_decode(q, k_pool, v_pool, out, decode_seg, seg_q_start, seg_pos0, block_table, nullptr,
                              table_width, rows, heads, kv_heads, head_dim, page_size, window, scale, chunk,
                              max_splits, base, counters, stream);
}
