// Memory-bound kernels of the decoder: embedding gather, RMSNorm (alone and fused with the
// residual add), rotate-half position encoding fused with the write of K and V into cache pages,
// SwiGLU, and a row gather.  Each is templated on the storage type (float or bfloat16); all
// arithmetic is float32.  Any width is accepted (no power-of-two or vector-width assumption).
//
// Formulas follow the reference's torch code (src/mini_llm_runtime/qwen_model_runner.py):
// RMSNorm :22-26, RoPE :34-61, SwiGLU :215-217, K/V written after RoPE :105-109.
#include "common.cuh"

namespace mlr {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 T* __restrict__ out, int width, int vocab) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  int id = ids[row];
  // Host code validates ids; clamp so a bad id can never read outside the table.
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const T* src = table + (size_t)id * width;
  T* dst = out + (size_t)row * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------- gather rows
template <typename T>
__global__ void gather_rows_kernel(const T* x, const int* __restrict__ rows,
                                   T* __restrict__ out, int width) {
  pdl_trigger();
  pdl_wait();
  const T* src = x + (size_t)rows[blockIdx.x] * width;
  T* dst = out + (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------- RMSNorm (+ residual add)
// One block per row.  If `delta` is given the row becomes residual + delta (added in float32,
// rounded once to T and stored back to `residual`); the norm is then taken of the stored value,
// so the fused kernel equals "add, then norm" exactly.  The row is staged in shared memory as
// float32 so that global memory is read once.
template <typename T, typename W>
__global__ void rms_norm_kernel(T* residual, const T* delta,
                                const W* __restrict__ weight, T* __restrict__ out, int width,
                                float eps) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float row_cache[];
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * width;
  float partial = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = to_float(residual[base + i]);
    if (delta != nullptr) {
      T stored = from_float<T>(v + to_float(delta[base + i]));
      residual[base + i] = stored;
      v = to_float(stored);
    }
    row_cache[i] = v;
    partial += v * v;
  }
  const float total = block_sum(partial, scratch);
  const float scale = rsqrtf(total / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float w = weight != nullptr ? to_float(weight[i]) : 1.f;   // no weight: normalise only
    out[base + i] = from_float<T>(w * (row_cache[i] * scale));
  }
}

// bfloat16 rows whose width is a multiple of 8 (at most 256 * VECS * WARPS_PER_ROW): one, two or
// four warps per row, each lane keeps its 16-byte pieces of the row in registers (at most 8 of
// the row and 8 of the delta: a lane with more spills, and a 64 x 5120 norm then takes 31 us
// instead of 4), so global memory is read once with wide loads.  Same arithmetic as above: float32
// add rounded once and stored back, float32 sum of squares, weight * (value * scale).
template <typename W, int VECS, int WARPS_PER_ROW>
__global__ void __launch_bounds__(128)
rms_norm_rows_kernel(bf16* residual, const bf16* delta, const W* __restrict__ weight, bf16* __restrict__ out,
                     int rows, int width, float eps) {
  __shared__ float warp_squares[4];
  pdl_trigger();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * (4 / WARPS_PER_ROW) + warp / WARPS_PER_ROW;
  const int share = warp % WARPS_PER_ROW;              // this warp's pieces: lane + 32 * (share + WARPS_PER_ROW * j)
  const bool live = row < rows;
  const int pieces = live ? width >> 3 : 0;
  const size_t base = (size_t)(live ? row : 0) * width;
  uint4* stream = reinterpret_cast<uint4*>(residual + base);
  const uint4* added = delta != nullptr ? reinterpret_cast<const uint4*>(delta + base) : nullptr;
  uint4* dst = reinterpret_cast<uint4*>(out + base);
  uint4 raw[VECS], extra[VECS];
#pragma unroll
  for (int j = 0; j < VECS; ++j) {
    const int piece = lane + 32 * (share + WARPS_PER_ROW * j);
    raw[j] = piece < pieces ? stream[piece] : make_uint4(0u, 0u, 0u, 0u);
    if (added != nullptr) extra[j] = piece < pieces ? added[piece] : make_uint4(0u, 0u, 0u, 0u);
  }
  float partial = 0.f;
#pragma unroll
  for (int j = 0; j < VECS; ++j) {
    const int piece = lane + 32 * (share + WARPS_PER_ROW * j);
    __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&raw[j]);
    if (added != nullptr) {
      const __nv_bfloat162* more = reinterpret_cast<const __nv_bfloat162*>(&extra[j]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = __bfloat1622float2(pairs[e]), b = __bfloat1622float2(more[e]);
        pairs[e] = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
      }
      if (piece < pieces) stream[piece] = raw[j];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(pairs[e]);
      partial += a.x * a.x + a.y * a.y;
    }
  }
  float squares = warp_sum(partial);
  if (WARPS_PER_ROW > 1) {             // the row's warps add their sums in warp order
    if (lane == 0) warp_squares[warp] = squares;
    __syncthreads();
    squares = 0.f;
#pragma unroll
    for (int v = 0; v < WARPS_PER_ROW; ++v) squares += warp_squares[warp / WARPS_PER_ROW * WARPS_PER_ROW + v];
  }
  const float scale = rsqrtf(squares / (float)width + eps);
#pragma unroll
  for (int j = 0; j < VECS; ++j) {
    const int piece = lane + 32 * (share + WARPS_PER_ROW * j);
    if (piece >= pieces) continue;
    const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
    float w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = weight != nullptr ? to_float(weight[piece * 8 + e]) : 1.f;
    uint4 packed;
    __nv_bfloat162* result = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 a = __bfloat1622float2(pairs[e]);
      result[e] = __floats2bfloat162_rn(w[2 * e] * (a.x * scale), w[2 * e + 1] * (a.y * scale));
    }
    dst[piece] = packed;
  }
}

// ---------------------------------------------------------------- in-place add
template <typename T>
__global__ void add_inplace_kernel(T* target, const T* delta, size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x)
    target[idx] = from_float<T>(to_float(target[idx]) + to_float(delta[idx]));
}

// ---------------------------------------------------------------- SwiGLU
// in: [rows, 2*inner].  Each row holds blocks of `block` gate values followed by the `block` up
// values of the same outputs; block == inner is the plain "all gates, then all ups" layout.
template <typename T>
__global__ void swiglu_kernel(const T* gate_up, T* __restrict__ out, int inner, int block,
                              size_t total) {
  pdl_trigger();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / inner;
    const int col = (int)(idx - row * inner);
    const size_t at = row * 2 * inner + (size_t)(col / block) * 2 * block + col % block;
    const float g = to_float(gate_up[at]);
    const float u = to_float(gate_up[at + block]);
    out[idx] = from_float<T>((g / (1.f + expf(-g))) * u);
  }
}

// ---------------------------------------------------------------- RoPE + paged K/V write
// qkv: [tokens, (heads + 2*kv_heads) * head_dim] = q heads, then k heads, then v heads.
// Writes rotated q to q_out [tokens, heads*head_dim]; rotated k and raw v to the page pools
// [pages, kv_heads, page_size, head_dim] at slot = page * page_size + offset (slot < 0: the
// token is padding, nothing is stored).  angle = position * inv_freq[i] in float32; element i
// pairs with element i + head_dim/2.
template <typename T>
__global__ void rope_kv_write_kernel(const T* qkv, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq,
                                     const long long* __restrict__ slots, T* __restrict__ q_out,
                                     T* __restrict__ k_pool, T* __restrict__ v_pool, int heads,
                                     int kv_heads, int head_dim, int page_size, int write_kv) {
  // The token's sines and cosines (one per pair index) are taken once, into shared memory: every
  // head uses the same head_dim/2 angles.
  __shared__ float sines[128], cosines[128];
  pdl_trigger();
  pdl_wait();
  const int token = blockIdx.x;
  const int half = head_dim >> 1;
  const int row_width = (heads + 2 * kv_heads) * head_dim;
  const T* row = qkv + (size_t)token * row_width;
  const float position = (float)positions[token];
  const long long slot = slots[token];
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int offset = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const bool store = write_kv != 0 && slot >= 0;
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(position * inv_freq[i], &sines[i], &cosines[i]);
  __syncthreads();

  const int rotated_heads = heads + kv_heads;
  constexpr int VEC = 16 / sizeof(T);            // elements per 16-byte access
  const bool wide = half % VEC == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)q_out & 15) == 0 &&
                    ((uintptr_t)k_pool & 15) == 0 && ((uintptr_t)v_pool & 15) == 0;
  if (wide) {
    // an item: VEC adjacent pair indices of one head, i.e. 16 bytes of the first half of the head
    // and the matching 16 bytes of the second
    const int chunks = half / VEC;
    for (int item = threadIdx.x; item < rotated_heads * chunks; item += blockDim.x) {
      const int head = item / chunks, i0 = (item - head * chunks) * VEC;
      T* dst = nullptr;
      if (head < heads) dst = q_out + ((size_t)token * heads + head) * head_dim;
      else if (store) dst = k_pool + (((size_t)page * kv_heads + (head - heads)) * page_size + offset) * head_dim;
      if (dst == nullptr) continue;
      const T* src = row + head * head_dim + i0;
      const uint4 lo = *reinterpret_cast<const uint4*>(src);
      const uint4 hi = *reinterpret_cast<const uint4*>(src + half);
      const T* x1 = reinterpret_cast<const T*>(&lo);
      const T* x2 = reinterpret_cast<const T*>(&hi);
      uint4 out_lo, out_hi;
      T* y1 = reinterpret_cast<T*>(&out_lo);
      T* y2 = reinterpret_cast<T*>(&out_hi);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float r1, r2;
        rotate_pair(to_float(x1[e]), to_float(x2[e]), sines[i0 + e], cosines[i0 + e], &r1, &r2);
        y1[e] = from_float<T>(r1);
        y2[e] = from_float<T>(r2);
      }
      *reinterpret_cast<uint4*>(dst + i0) = out_lo;
      *reinterpret_cast<uint4*>(dst + i0 + half) = out_hi;
    }
    if (store) {
      const T* v_row = row + (size_t)(heads + kv_heads) * head_dim;
      const int per_head = head_dim / VEC;
      for (int item = threadIdx.x; item < kv_heads * per_head; item += blockDim.x) {
        const int kv_head = item / per_head, i0 = (item - kv_head * per_head) * VEC;
        *reinterpret_cast<uint4*>(v_pool + (((size_t)page * kv_heads + kv_head) * page_size + offset) * head_dim + i0) =
            *reinterpret_cast<const uint4*>(v_row + kv_head * head_dim + i0);
      }
    }
    return;
  }
  for (int item = threadIdx.x; item < rotated_heads * half; item += blockDim.x) {
    const int head = item / half, i = item - head * half;
    const float x1 = to_float(row[head * head_dim + i]);
    const float x2 = to_float(row[head * head_dim + i + half]);
    float y1, y2;
    rotate_pair(x1, x2, sines[i], cosines[i], &y1, &y2);
    if (head < heads) {
      T* dst = q_out + ((size_t)token * heads + head) * head_dim;
      dst[i] = from_float<T>(y1);
      dst[i + half] = from_float<T>(y2);
    } else if (store) {
      const int kv_head = head - heads;
      T* dst = k_pool + (((size_t)page * kv_heads + kv_head) * page_size + offset) * head_dim;
      dst[i] = from_float<T>(y1);
      dst[i + half] = from_float<T>(y2);
    }
  }
  if (store) {
    const T* v_row = row + (size_t)(heads + kv_heads) * head_dim;
    for (int item = threadIdx.x; item < kv_heads * head_dim; item += blockDim.x) {
      const int kv_head = item / head_dim, i = item - kv_head * head_dim;
      v_pool[(((size_t)page * kv_heads + kv_head) * page_size + offset) * head_dim + i] = v_row[item];
    }
  }
}


// ---------------------------------------------------------------- resident tables and slot state
// The three kernels below write the step's metadata on the device.  Later kernels of the same
// step read that metadata before their own griddepcontrol.wait, so these kernels never let their
// successor start early: they do not call pdl_trigger(), and the next kernel is launched only
// once they have completed and their writes are visible.

// dst[row_index[i]] = src[i] for rows of `width` 32-bit words: changed block-table rows and new
// slot records, sent by the host in one buffer, land in the tables that stay on the device.
__global__ void scatter_rows_kernel(int* __restrict__ dst, const int* __restrict__ row_index,
                                    const int* __restrict__ src, int width) {
  pdl_wait();
  const int* from = src + (size_t)blockIdx.x * width;
  int* to = dst + (size_t)row_index[blockIdx.x] * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) to[i] = from[i];
}

// A step of decoded tokens, described by the slots of its requests alone: position (and segment
// start) = the slot's length, input token = the slot's last sampled token (if token_ids is given),
// and the place where the new key and value go = page of that position in the slot's table row.
__global__ void decode_prepare_kernel(const int* __restrict__ seg_slot, const SlotState* state, int count,
                                      int* token_ids, int* positions, int* seg_pos0,
                                      const int* table, int table_width, int page_size, long long* kv_slots) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int slot = seg_slot[i];
  const int position = state[slot].length;
  if (token_ids != nullptr) token_ids[i] = state[slot].last_token;
  if (positions != nullptr) positions[i] = position;
  if (seg_pos0 != nullptr) seg_pos0[i] = position;
  if (kv_slots != nullptr) {
    const int logical = position / page_size;
    const int page = logical < table_width ? table[(size_t)slot * table_width + logical] : -1;
    kv_slots[i] = page >= 0 ? (long long)page * page_size + (position - logical * page_size) : -1;
  }
}

// After a step: every request of it holds seg_q_len more tokens.  With seg_pos0 the new length is
// set from the host's figures (pos0 + len); without, the slot's own length grows by len (or by one
// when seg_q_len is null).
__global__ void advance_slots_kernel(const int* __restrict__ seg_slot, const int* __restrict__ seg_q_len,
                                     const int* __restrict__ seg_pos0, int count, SlotState* state) {
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int grow = seg_q_len != nullptr ? seg_q_len[i] : 1;
  SlotState* mine = state + seg_slot[i];
  mine->length = (seg_pos0 != nullptr ? seg_pos0[i] : mine->length) + grow;
}

template <typename T>
int rope_kv_write_launch(const void* qkv, const int* positions, const float* inv_freq,
                         const long long* slots, void* q_out, void* k_pool, void* v_pool,
                         int tokens, int heads, int kv_heads, int head_dim, int page_size,
                         int write_kv, cudaStream_t stream) {
  // items of 16 bytes of a head's first half and the 16 bytes they pair with (scalar pairs where
  // the head size does not allow that)
  int work = (heads + kv_heads) * (head_dim / 2) / (int)(16 / sizeof(T));
  int threads = work >= 192 ? 256 : (work >= 96 ? 128 : 64);
  launch_kernel(rope_kv_write_kernel<T>, dim3(tokens), dim3(threads), 0, stream, 
      (const T*)qkv, positions, inv_freq, slots, (T*)q_out, (T*)k_pool, (T*)v_pool, heads,
      kv_heads, head_dim, page_size, write_kv);
  return launch_status();
}

static int row_threads(int width) {
  if (width >= 2048) return 512;
  if (width >= 512) return 256;
  if (width >= 128) return 128;
  return 64;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

MLR_EXPORT int mlr_embedding(const int* ids, const void* table, void* out, int rows, int width,
                             int vocab, int dtype, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0 || vocab <= 0) return MLR_BAD_SIZE;
  const int threads = row_threads(width);
  if (dtype == MLR_F32)
    launch_kernel(embedding_kernel<float>, dim3(rows), dim3(threads), 0, stream, ids, (const float*)table, (float*)out, width, vocab);
  else if (dtype == MLR_BF16)
    launch_kernel(embedding_kernel<bf16>, dim3(rows), dim3(threads), 0, stream, ids, (const bf16*)table, (bf16*)out, width, vocab);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_gather_rows(const void* x, const int* rows, void* out, int count, int width,
                               int dtype, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0 || width <= 0) return MLR_BAD_SIZE;
  const int threads = row_threads(width);
  if (dtype == MLR_F32)
    launch_kernel(gather_rows_kernel<float>, dim3(count), dim3(threads), 0, stream, (const float*)x, rows, (float*)out, width);
  else if (dtype == MLR_BF16)
    launch_kernel(gather_rows_kernel<bf16>, dim3(count), dim3(threads), 0, stream, (const bf16*)x, rows, (bf16*)out, width);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

template <typename T, typename W>
static int rms_norm_launch(void* residual, const void* delta, const void* weight, void* out, int rows,
                           int width, float eps, cudaStream_t stream) {
  const size_t shared = (size_t)width * sizeof(float);
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(rms_norm_kernel<T, W>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  launch_kernel(rms_norm_kernel<T, W>, dim3(rows), dim3(row_threads(width)), shared, stream, 
      (T*)residual, (const T*)delta, (const W*)weight, (T*)out, width, eps);
  return launch_status();
}

// residual is updated in place when delta != nullptr; out may alias neither.  The weight may be
// stored in float32 while the rows are bfloat16 (a checkpoint's 32-bit tensor stays 32-bit).
MLR_EXPORT int mlr_rms_norm(void* residual, const void* delta, const void* weight, void* out,
                            int rows, int width, float eps, int dtype, int weight_dtype,
                            cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || width <= 0) return MLR_BAD_SIZE;
  if ((size_t)width * sizeof(float) > 200 * 1024) return MLR_TOO_LARGE;
  if (dtype == MLR_F32 && weight_dtype == MLR_F32)
    return rms_norm_launch<float, float>(residual, delta, weight, out, rows, width, eps, stream);
  if (dtype == MLR_BF16 && width % 8 == 0 && width <= 8192 && (((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)out) & 15) == 0) {
    // the row in the registers of one, two or four warps (at most 8 pieces of 16 bytes per lane)
#define MLR_ROWS(W_, V_, P_)                                                                                 \
  launch_kernel(rms_norm_rows_kernel<W_, V_, P_>, dim3((rows * P_ + 3) / 4), dim3(128), 0, stream,           \
                (bf16*)residual, (const bf16*)delta, (const W_*)weight, (bf16*)out, rows, width, eps)
#define MLR_ROWS_BY_WIDTH(W_)                                                                                \
  do {                                                                                                       \
    if (width <= 256) MLR_ROWS(W_, 1, 1); else if (width <= 512) MLR_ROWS(W_, 2, 1);                         \
    else if (width <= 1024) MLR_ROWS(W_, 4, 1); else if (width <= 2048) MLR_ROWS(W_, 8, 1);                  \
    else if (width <= 4096) MLR_ROWS(W_, 8, 2); else MLR_ROWS(W_, 8, 4);                                     \
  } while (0)
    if (weight_dtype == MLR_F32) MLR_ROWS_BY_WIDTH(float);
    else if (weight_dtype == MLR_BF16) MLR_ROWS_BY_WIDTH(bf16);
    else return MLR_BAD_DTYPE;
#undef MLR_ROWS_BY_WIDTH
#undef MLR_ROWS
    return launch_status();
  }
  if (dtype == MLR_BF16 && weight_dtype == MLR_BF16)
    return rms_norm_launch<bf16, bf16>(residual, delta, weight, out, rows, width, eps, stream);
  if (dtype == MLR_BF16 && weight_dtype == MLR_F32)
    return rms_norm_launch<bf16, float>(residual, delta, weight, out, rows, width, eps, stream);
  return MLR_BAD_DTYPE;
}

MLR_EXPORT int mlr_add_inplace(void* target, const void* delta, long long total, int dtype, cudaStream_t stream) {
  if (total == 0) return MLR_OK;
  if (total < 0) return MLR_BAD_SIZE;
  size_t blocks = ((size_t)total + 255) / 256;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  if (dtype == MLR_F32)
    launch_kernel(add_inplace_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)target, (const float*)delta, (size_t)total);
  else if (dtype == MLR_BF16)
    launch_kernel(add_inplace_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, (bf16*)target, (const bf16*)delta, (size_t)total);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_swiglu(const void* gate_up, void* out, long long rows, int inner, int block, int dtype,
                          cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || inner <= 0 || block <= 0 || inner % block != 0) return MLR_BAD_SIZE;
  const size_t total = (size_t)rows * inner;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > (size_t)sm_count() * 32) blocks = (size_t)sm_count() * 32;
  if (dtype == MLR_F32)
    launch_kernel(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inner, block, total);
  else if (dtype == MLR_BF16)
    launch_kernel(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inner, block, total);
  else
    return MLR_BAD_DTYPE;
  return launch_status();
}

MLR_EXPORT int mlr_rope_kv_write(const void* qkv, const int* positions, const float* inv_freq,
                                 const long long* slots, void* q_out, void* k_pool, void* v_pool,
                                 int tokens, int heads, int kv_heads, int head_dim, int page_size,
                                 int write_kv, int dtype, cudaStream_t stream) {
  if (tokens == 0) return MLR_OK;
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || page_size <= 0)
    return MLR_BAD_SIZE;
  if (head_dim > 256) return MLR_TOO_LARGE;       // the kernel keeps head_dim/2 sines and cosines in shared memory
  if (dtype == MLR_F32)
    return rope_kv_write_launch<float>(qkv, positions, inv_freq, slots, q_out, k_pool, v_pool, tokens,
                                       heads, kv_heads, head_dim, page_size, write_kv, stream);
  if (dtype == MLR_BF16)
    return rope_kv_write_launch<bf16>(qkv, positions, inv_freq, slots, q_out, k_pool, v_pool, tokens,
                                      heads, kv_heads, head_dim, page_size, write_kv, stream);
  return MLR_BAD_DTYPE;
}

// dst: int32 [table rows, width]; row_index int32 [count]; src int32 [count, width].
MLR_EXPORT int mlr_scatter_rows(int* dst, const int* row_index, const int* src, int count, int width,
                                cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0 || width <= 0) return MLR_BAD_SIZE;
  launch_kernel(scatter_rows_kernel, dim3(count), dim3(width >= 256 ? 256 : 64), 0, stream, dst, row_index, src, width);
  return launch_status();
}

// state: SlotState records (eight 32-bit words each).  token_ids, positions, seg_pos0 and kv_slots
// may each be null; a model with several cache groups calls once per group with its table.
MLR_EXPORT int mlr_decode_prepare(const int* seg_slot, const void* state, int count, int* token_ids,
                                  int* positions, int* seg_pos0, const int* table, int table_width,
                                  int page_size, long long* kv_slots, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0 || (kv_slots != nullptr && (table == nullptr || table_width <= 0 || page_size <= 0)))
    return MLR_BAD_SIZE;
  launch_kernel(decode_prepare_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, seg_slot,
                (const SlotState*)state, count, token_ids, positions, seg_pos0, table, table_width, page_size,
                kv_slots);
  return launch_status();
}

MLR_EXPORT int mlr_advance_slots(const int* seg_slot, const int* seg_q_len, const int* seg_pos0, int count,
                                 void* state, cudaStream_t stream) {
  if (count == 0) return MLR_OK;
  if (count < 0) return MLR_BAD_SIZE;
  launch_kernel(advance_slots_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, seg_slot, seg_q_len,
                seg_pos0, count, (SlotState*)state);
  return launch_status();
}
