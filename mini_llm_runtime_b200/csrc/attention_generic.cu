// Causal attention of a ragged batch over the paged K/V cache, on the CUDA cores in float32.
//
// One kernel serves prompt portions and single decoded tokens alike: the batch is a list of
// segments (one per request); a segment's rows are the request's next tokens at positions
// pos0, pos0+1, ..; row r sees the cached keys at positions max(0, p-window+1) .. p of its own
// request, its own key included (it was written to the cache just before).  Keys are fetched
// page by page through the request's block table.
//
// Semantics follow the reference: scores = (q.k) * head_dim^-0.5, softmax and accumulation in
// float32 with the online (running max / running sum) recurrence of
// csrc/paged_attention_cuda.cu:50-105, query head h reading kv head h / (heads / kv_heads)
// (:44-46).  The sliding window has no counterpart there.
//
// Keys are walked in tiles of 32 aligned to absolute positions (tile t = keys 32t .. 32t+31), and
// every reduction has a fixed lane order, so a row's result depends only on its own request's
// cache: not on how the prompt was cut into steps, nor on the other rows of the batch.
// This is the attention of the 32-bit path and the fallback of the bfloat16 path.
// Accepts any head_dim <= 256, any head counts, any page size.
#include "common.cuh"

namespace mlr {

constexpr int ROWS_PER_TILE = 16;  // query rows per CTA (4 per warp)
constexpr int KEYS_PER_TILE = 32;  // one key per lane
constexpr int MAX_HEAD_DIM = 256;

template <typename T>
__global__ void __launch_bounds__(128)
attention_generic_kernel(const T* q, const T* k_pool,
                         const T* v_pool, T* __restrict__ out,
                         const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                         const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                         const int* __restrict__ seg_pos0, const int* __restrict__ block_table, const int* __restrict__ seg_slot,
                         int table_width, int heads, int kv_heads, int head_dim, int page_size,
                         int window, float scale) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ float shared[];
  const int D = head_dim;
  float* q_rows = shared;                                   // [16][D]
  float* k_tile = q_rows + ROWS_PER_TILE * D;               // [32][D+1]
  float* v_tile = k_tile + KEYS_PER_TILE * (D + 1);         // [32][D]
  float* p_tile = v_tile + KEYS_PER_TILE * D;               // [4 warps][4 rows][32]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int kv_head = head / (heads / kv_heads);
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int q_start = seg_q_start[seg], q_len = seg_q_len[seg], pos0 = seg_pos0[seg];
  const int rows = min(ROWS_PER_TILE, q_len - row0);
  const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  for (int idx = threadIdx.x; idx < ROWS_PER_TILE * D; idx += blockDim.x) {
    const int r = idx / D, d = idx - r * D;
    q_rows[idx] = r < rows ? to_float(q[((size_t)(q_start + row0 + r) * heads + head) * D + d]) : 0.f;
  }

  float m[4], l[4], acc[4][MAX_HEAD_DIM / 32];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < MAX_HEAD_DIM / 32; ++c) acc[i][c] = 0.f;
  }

  const int first_pos = pos0 + row0, last_pos = pos0 + row0 + rows - 1;
  const int lowest_key = window > 0 ? max(0, first_pos - window + 1) : 0;
  for (int k0 = (lowest_key / KEYS_PER_TILE) * KEYS_PER_TILE; k0 <= last_pos; k0 += KEYS_PER_TILE) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < KEYS_PER_TILE * D; idx += blockDim.x) {
      const int j = idx / D, d = idx - j * D;
      const int key = k0 + j;
      float kv = 0.f, vv = 0.f;
      if (key <= last_pos) {
        const int page = table[key / page_size];
        if (page >= 0) {
          const size_t at = (((size_t)page * kv_heads + kv_head) * page_size + key % page_size) * D + d;
          kv = to_float(k_pool[at]);
          vv = to_float(v_pool[at]);
        }
      }
      k_tile[j * (D + 1) + d] = kv;
      v_tile[j * D + d] = vv;
    }
    __syncthreads();

    const int key = k0 + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = warp * 4 + i;
      if (r >= rows) continue;  // uniform per warp
      const int p = first_pos + r;
      const bool visible = key <= p && (window <= 0 || key > p - window);
      float s = 0.f;
      const float* qr = q_rows + r * D;
      const float* kr = k_tile + lane * (D + 1);
      for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
      s = visible ? s * scale : -INFINITY;
      const float m_new = fmaxf(m[i], warp_max(s));
      if (m_new == -INFINITY) continue;  // no visible key yet (uniform per warp)
      const float alpha = expf(m[i] - m_new);  // m = -inf gives 0
      const float prob = visible ? expf(s - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(prob);
      m[i] = m_new;
      float* pw = p_tile + (warp * 4 + i) * KEYS_PER_TILE;
      pw[lane] = prob;
      __syncwarp();
#pragma unroll
      for (int c = 0; c < MAX_HEAD_DIM / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < D) {
          float a = acc[i][c] * alpha;
          for (int j = 0; j < KEYS_PER_TILE; ++j) a = fmaf(pw[j], v_tile[j * D + d], a);
          acc[i][c] = a;
        }
      }
      __syncwarp();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp * 4 + i;
    if (r >= rows) continue;
    const float inv = 1.f / l[i];
    T* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * D;
#pragma unroll
    for (int c = 0; c < MAX_HEAD_DIM / 32; ++c) {
      const int d = lane + 32 * c;
      if (d < D) dst[d] = from_float<T>(acc[i][c] * inv);
    }
  }
}

template <typename T>
int attention_generic_launch(const void* q, const void* k_pool, const void* v_pool, void* out,
                             const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                             const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                             int table_width, int tiles, int heads, int kv_heads, int head_dim,
                             int page_size, int window, float scale, cudaStream_t stream) {
  const size_t shared = sizeof(float) * ((size_t)ROWS_PER_TILE * head_dim + (size_t)KEYS_PER_TILE * (head_dim + 1) +
                                         (size_t)KEYS_PER_TILE * head_dim + 16 * KEYS_PER_TILE);
  if (shared > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(attention_generic_kernel<T>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
  }
  dim3 grid(tiles, heads);
  launch_kernel(attention_generic_kernel<T>, dim3(grid), dim3(128), shared, stream, 
      (const T*)q, (const T*)k_pool, (const T*)v_pool, (T*)out, tile_seg, tile_row0, seg_q_start,
      seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads, head_dim, page_size, window, scale);
  return launch_status();
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// q, out: [rows, heads, head_dim]; pools: [pages, kv_heads, page_size, head_dim].
// tile_seg/tile_row0: one entry per CTA tile of up to 16 rows of one segment.
// window <= 0 means every earlier key is visible.
MLR_EXPORT int mlr_attention_generic(const void* q, const void* k_pool, const void* v_pool, void* out,
                                     const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                     const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                                     int table_width, int tiles, int heads, int kv_heads, int head_dim,
                                     int page_size, int window, float scale, int dtype,
                                     cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || head_dim <= 0 ||
      page_size <= 0 || table_width <= 0)
    return MLR_BAD_SIZE;
  if (head_dim > MAX_HEAD_DIM || heads > 65535) return MLR_TOO_LARGE;
  if (dtype == MLR_F32)
    return attention_generic_launch<float>(q, k_pool, v_pool, out, tile_seg, tile_row0, seg_q_start,
                                           seg_q_len, seg_pos0, block_table, seg_slot, table_width, tiles, heads,
                                           kv_heads, head_dim, page_size, window, scale, stream);
  if (dtype == MLR_BF16)
    return attention_generic_launch<bf16>(q, k_pool, v_pool, out, tile_seg, tile_row0, seg_q_start,
                                          seg_q_len, seg_pos0, block_table, seg_slot, table_width, tiles, heads,
                                          kv_heads, head_dim, page_size, window, scale, stream);
  return MLR_BAD_DTYPE;
}
