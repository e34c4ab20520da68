// Tensor-core attention over the paged bfloat16 K/V cache (head_dim 64 or 128), two kernels that
// share their tile loader and fragment code:
//
//   prefill_attention_kernel  rows = the query positions of a prompt portion.  One CTA owns 64
//       rows of one query head; its 4 warps own 16 rows each and walk the request's keys in tiles
//       of 64, K and V fetched page by page with cp.async into swizzled shared memory (double
//       buffered), S = Q K^T and O += P V on mma.sync m16n8k16 (bfloat16 in, float32 out), the
//       online softmax kept in registers.  Causal limit, window and the portion's start position
//       are applied per element, so a portion in the middle of a request reads earlier keys from
//       the cache exactly like a whole prompt.
//   decode_attention_mma_kernel  rows = the query heads that share one kv head (one decoded token).
//       One CTA owns (request, kv head, chunk of keys); its 4 warps take 16 keys each of every
//       64-key tile, all tiles of the chunk are requested up front (4 cp.async stages in flight),
//       the warps' states are merged in shared memory, and the chunks' states are merged by the CTA
//       that finishes last for that (request, kv head), in chunk order.
//
// Semantics as in the reference (scores = q.k * head_dim^-0.5, float32 softmax with running max and
// sum, csrc/paged_attention_cuda.cu:50-105; GQA head mapping :44-46; causal mask
// src/mini_llm_runtime/qwen_model_runner.py:157-177).  Keys beyond a row's limit, and slots of pages
// the request does not hold, are loaded as zeros and their scores set to -inf before the softmax.
//
// mma.sync is the legacy tensor path on sm_100a; attention here is far from the bound of either
// path for the model sizes served (the projections dominate), and tcgen05 serves those.
#include "tma.cuh"

namespace mlr {

constexpr int ATTN_WARPS = 4;
constexpr int ATTN_THREADS = ATTN_WARPS * 32;
constexpr int TILE_Q = 64;
constexpr int TILE_KV = 64;

__device__ __forceinline__ uint32_t shared_address(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;   // 0: the 16 destination bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(shared_address(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(shared_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(shared_address(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&pair);
}

// A tile in shared memory: rows of D bfloat16, the 16-byte chunks of a row XOR-swizzled by the row
// index so that ldmatrix (8 rows x 16 bytes) is free of bank conflicts.
// HALVES (head_dim 128 as the tensor memory accelerator delivers it): two sub-tiles of 64 columns,
// each with rows of 128 bytes and the same swizzle; for head_dim 64 both layouts coincide.
template <int D, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ bf16* tile_at(bf16* tile, int row, int chunk) {
  if (HALVES && D > 64) return tile + (chunk >> 3) * (TKV * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
  return tile + row * D + ((chunk ^ (row & 7)) << 3);
}

// Fetch `rows` rows starting at key `key0` of one kv head into a swizzled tile.  Keys outside
// [key_lo, key_hi] and keys on pages the request does not hold become zeros.
// `page_shift` is log2(page_size) when the page size is a power of two (the usual case: address
// arithmetic by shifts), else -1 (division).
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* tile, const bf16* pool, const int* __restrict__ table,
                                             int key0, int rows, int key_lo, int key_hi, int kv_heads, int kv_head,
                                             int page_size, int page_shift) {
  constexpr int CHUNKS = D / 8;
  for (int item = threadIdx.x; item < rows * CHUNKS; item += ATTN_THREADS) {
    const int r = item / CHUNKS, c = item - r * CHUNKS;
    const int key = key0 + r;
    bool valid = key >= key_lo && key <= key_hi;
    const bf16* src = pool;
    if (valid) {
      const int logical = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int offset = page_shift >= 0 ? key & (page_size - 1) : key - logical * page_size;
      const int page = table[logical];
      valid = page >= 0;
      if (valid) src = pool + (((size_t)page * kv_heads + kv_head) * page_size + offset) * D + c * 8;
    }
    cp_async_16(tile_at<D>(tile, r, c), src, valid);
  }
}

// One warp: S[16 x (8*NT)] = Q[16 x D] K^T for keys key_row0.. of a K tile.
template <int D, int NT, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ void warp_qk(float (*s)[4], const uint32_t (*q_frag)[4], bf16* k_tile, int key_row0, int lane) {
#pragma unroll
  for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int jp = 0; jp < NT / 2; ++jp) {
      uint32_t b[4];
      const int key = key_row0 + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int chunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b, tile_at<D, HALVES, TKV>(k_tile, key, chunk));
      mma_bf16(s[2 * jp], q_frag[ks], b[0], b[1]);
      mma_bf16(s[2 * jp + 1], q_frag[ks], b[2], b[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x (8*NT)] V for keys key_row0.. of a V tile; P comes from the score
// registers, rounded to bfloat16.
template <int D, int NT, bool HALVES = false, int TKV = TILE_KV>
__device__ __forceinline__ void warp_pv(float (*o)[4], const float (*p)[4], bf16* v_tile, int key_row0, int lane) {
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      const int key = key_row0 + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int chunk = dp * 2 + (lane >> 4);
      ldmatrix_x4_trans(b, tile_at<D, HALVES, TKV>(v_tile, key, chunk));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online softmax step on one warp's score fragment.  Thread owns rows r0 = lane/4 and r0 + 8;
// limit_lo[i] <= key <= limit_hi[i] are visible for row i.  Scores arrive unscaled; `scale_log2`
// = head_dim^-0.5 * log2(e).  Leaves probabilities in s and rescales o.
// MASKED = false: the caller knows that every key of the tile is visible to every row.
template <int NT, int OT, bool MASKED = true>
__device__ __forceinline__ void softmax_step(float (*s)[4], float (*o)[4], float* m, float* l, int key_base,
                                             const int* limit_lo, const int* limit_hi, float scale_log2, int lane) {
  float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int key = key_base + j * 8 + (lane & 3) * 2 + (e & 1);
      const int i = e >> 1;
      const bool visible = !MASKED || (key >= limit_lo[i] && key <= limit_hi[i]);
      s[j][e] = visible ? s[j][e] * scale_log2 : -INFINITY;
      tile_max[i] = fmaxf(tile_max[i], s[j][e]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
  }
  float alpha[2], row_sum[2] = {0.f, 0.f}, base[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float m_new = fmaxf(m[i], tile_max[i]);
    base[i] = m_new == -INFINITY ? 0.f : m_new;       // nothing visible yet: keep everything at zero
    alpha[i] = exp2f(m[i] - base[i]);                  // m = -inf gives 0
    m[i] = m_new;
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float prob = exp2f(s[j][e] - base[e >> 1]);   // -inf gives 0
      s[j][e] = prob;
      row_sum[e >> 1] += prob;
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 1);
    row_sum[i] += __shfl_xor_sync(0xffffffffu, row_sum[i], 2);
    l[i] = l[i] * alpha[i] + row_sum[i];
  }
#pragma unroll
  for (int t = 0; t < OT; ++t) {
    o[t][0] *= alpha[0]; o[t][1] *= alpha[0];
    o[t][2] *= alpha[1]; o[t][3] *= alpha[1];
  }
}

// ------------------------------------------------------------------------------------------ prefill
template <int D>
__global__ void __launch_bounds__(ATTN_THREADS)
prefill_attention_kernel(const bf16* q, const bf16* k_pool, const bf16* v_pool,
                         bf16* __restrict__ out, const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                         const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                         const int* __restrict__ seg_pos0, const int* __restrict__ block_table, const int* __restrict__ seg_slot, int table_width,
                         int heads, int kv_heads, int page_size, int page_shift, int window, float scale_log2) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t attn_shared[];
  bf16* q_tile = reinterpret_cast<bf16*>(attn_shared);         // [64][D]
  bf16* k_tiles = q_tile + TILE_Q * D;                          // 2 x [64][D]
  bf16* v_tiles = k_tiles + 2 * TILE_KV * D;                    // 2 x [64][D]

  // Tiles are listed in order of position; the last ones see the most keys, so they go first.
  const int tile = gridDim.x - 1 - blockIdx.x, head = blockIdx.y;
  const int kv_head = head / (heads / kv_heads);
  const int seg = tile_seg[tile], row0 = tile_row0[tile];
  const int q_start = seg_q_start[seg], q_len = seg_q_len[seg], pos0 = seg_pos0[seg];
  const int rows = min(TILE_Q, q_len - row0);
  const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
  const int lowest = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int tile_begin = lowest / TILE_KV, tile_end = last_pos / TILE_KV;   // inclusive

  // Q tile (rows beyond the segment are zeros) and the first K/V tile
  constexpr int CHUNKS = D / 8;
  for (int item = threadIdx.x; item < TILE_Q * CHUNKS; item += ATTN_THREADS) {
    const int r = item / CHUNKS, c = item - r * CHUNKS;
    const bool valid = r < rows;
    const bf16* src = valid ? q + ((size_t)(q_start + row0 + r) * heads + head) * D + c * 8 : q;
    cp_async_16(tile_at<D>(q_tile, r, c), src, valid);
  }
  load_kv_tile<D>(k_tiles, k_pool, table, tile_begin * TILE_KV, TILE_KV, lowest, last_pos, kv_heads, kv_head, page_size, page_shift);
  load_kv_tile<D>(v_tiles, v_pool, table, tile_begin * TILE_KV, TILE_KV, lowest, last_pos, kv_heads, kv_head, page_size, page_shift);
  cp_async_commit();

  // per-thread rows and their visibility limits
  int limit_lo[2], limit_hi[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + (lane >> 2) + 8 * i;
    const int position = first_pos + r;
    limit_hi[i] = r < rows ? position : -1;                       // rows past the segment see nothing
    limit_lo[i] = window > 0 ? max(0, position - window + 1) : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  uint32_t q_frag[D / 16][4];

  for (int t = tile_begin; t <= tile_end; ++t) {
    const int buffer = (t - tile_begin) & 1;
    if (t < tile_end) {
      const int next = buffer ^ 1;
      load_kv_tile<D>(k_tiles + next * TILE_KV * D, k_pool, table, (t + 1) * TILE_KV, TILE_KV, lowest, last_pos,
                      kv_heads, kv_head, page_size, page_shift);
      load_kv_tile<D>(v_tiles + next * TILE_KV * D, v_pool, table, (t + 1) * TILE_KV, TILE_KV, lowest, last_pos,
                      kv_heads, kv_head, page_size, page_shift);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == tile_begin) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(q_frag[ks], tile_at<D>(q_tile, r, ks * 2 + (lane >> 4)));
      }
    }
    // a warp whose rows all end before this tile has nothing left to do in it
    const int warp_last = first_pos + min(rows - 1, warp * 16 + 15);
    if (warp * 16 < rows && t * TILE_KV <= warp_last) {
      float s[TILE_KV / 8][4];
      warp_qk<D, TILE_KV / 8>(s, q_frag, k_tiles + buffer * TILE_KV * D, 0, lane);
      softmax_step<TILE_KV / 8, D / 8>(s, o, m, l, t * TILE_KV, limit_lo, limit_hi, scale_log2, lane);
      warp_pv<D, TILE_KV / 8>(o, s, v_tiles + buffer * TILE_KV * D, 0, lane);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = warp * 16 + (lane >> 2) + 8 * i;
    if (r >= rows) continue;
    const float inv = 1.f / l[i];
    bf16* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * D + (lane & 3) * 2;
#pragma unroll
    for (int t = 0; t < D / 8; ++t)
      *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16(o[t][2 * i] * inv, o[t][2 * i + 1] * inv);
  }
}

// ------------------------------------------------------------------------------------ prefill, TMA
// The prefill kernel of choice: the arithmetic of prefill_attention_kernel with three changes that
// remove most of its instructions and its idle time.
//   * K and V tiles arrive by bulk tensor copies (one per page and 64-column half, as in the decode
//     kernel) into a ring of STAGES stages; a full/empty pair of mbarriers per stage replaces the
//     two CTA-wide barriers per key tile.  The warps take turns issuing: at the start of iteration j
//     warp (j + STAGES - 1) % 4 waits until all four have released the stage of tile j - 1 and
//     refills it with tile j + STAGES - 1.
//   * Work items (64 query rows of one head) are drawn from a counter in global memory, heaviest
//     first (the host lists the tiles by falling number of keys), by as many CTAs as fit on the
//     GPU at once: the causal triangle no longer leaves SMs idle while the last tiles finish.
//   * Key tiles that every row of a warp sees completely skip the per-element mask.
// Keys outside [lowest, last position of the tile] are masked to -inf; the V rows of such keys are
// overwritten with zeros before use (first and last key tile of an item only), so that whatever
// lies in slots the request does not own cannot reach the result.
template <int D, int STAGES>
__global__ void __launch_bounds__(ATTN_THREADS)
prefill_attention_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                             const bf16* q, bf16* __restrict__ out, const int* __restrict__ tile_seg,
                             const int* __restrict__ tile_row0, const int* __restrict__ seg_q_start,
                             const int* __restrict__ seg_q_len, const int* __restrict__ seg_pos0,
                             const int* __restrict__ block_table, const int* __restrict__ seg_slot, int table_width, int num_tiles, int heads,
                             int kv_heads, int page_size, int page_shift, int window, float scale_log2,
                             int* queue, int* error_word) {
  constexpr int HALVES = D / 64;
  constexpr int TILE_ELEMS = TILE_KV * D;
  constexpr int NT = TILE_KV / 8;
  constexpr int CHUNKS = D / 8;
  extern __shared__ uint8_t attn_shared_raw[];
  uint8_t* aligned = (uint8_t*)(((uintptr_t)attn_shared_raw + 1023) & ~(uintptr_t)1023);
  bf16* kv_tiles = reinterpret_cast<bf16*>(aligned);                 // STAGES x (K [64][D], V [64][D])
  bf16* q_tile = kv_tiles + (size_t)STAGES * 2 * TILE_ELEMS;         // [64][D]
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ int item_shared;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], ATTN_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
  }
  pdl_trigger();
  __syncthreads();
  pdl_wait();                       // before the first draw from the queue and the first read of q

  const int total_items = num_tiles * heads;
  const int boxes = page_size >= TILE_KV ? 1 : TILE_KV >> page_shift;
  const int box_rows = page_size >= TILE_KV ? TILE_KV : page_size;
  unsigned loads_before = 0;        // tiles this CTA has loaded in earlier items (the ring runs on across items)
  bool gave_up = false;             // a wait ran out: skip all later waits, finish, let the host raise

  for (;;) {
    if (threadIdx.x == 0) item_shared = atomicAdd(&queue[0], 1);
    __syncthreads();
    const int item = item_shared;
    if (item >= total_items) break;
    const int tile = item / heads, head = item - tile * heads;
    const int kv_head = head / (heads / kv_heads);
    const int seg = tile_seg[tile], row0 = tile_row0[tile];
    const int q_start = seg_q_start[seg], q_len = seg_q_len[seg], pos0 = seg_pos0[seg];
    const int rows = min(TILE_Q, q_len - row0);
    const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
    const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
    const int lowest = window > 0 ? max(0, first_pos - window + 1) : 0;
    const int tile_begin = lowest / TILE_KV, tile_end = last_pos / TILE_KV;   // inclusive
    const int tiles = tile_end - tile_begin + 1;

    for (int idx = threadIdx.x; idx < TILE_Q * CHUNKS; idx += ATTN_THREADS) {
      const int r = idx / CHUNKS, c = idx - r * CHUNKS;
      const bool valid = r < rows;
      const bf16* src = valid ? q + ((size_t)(q_start + row0 + r) * heads + head) * D + c * 8 : q;
      cp_async_16(tile_at<D>(q_tile, r, c), src, valid);
    }
    cp_async_commit();

    // the whole warp calls this; lane b fetches the b-th page (or the one 64-key box) of key tile j
    auto issue = [&](int j) {
      const unsigned load = loads_before + (unsigned)j;
      const int stage = load % STAGES;
      const unsigned use = load / STAGES;
      if (use > 0 && !gave_up) gave_up = !mbar_wait(&empty_bar[stage], (use - 1) & 1u, error_word, 0x51);
      gave_up = __any_sync(0xffffffffu, gave_up);
      if (gave_up) return;
      uint64_t* bar = &full_bar[stage];
      if (lane == 0) mbar_expect_tx(bar, 2u * TILE_ELEMS * 2u);
      __syncwarp();
      if (lane < boxes) {
        const int key0 = (tile_begin + j) * TILE_KV + lane * box_rows;
        const int logical = key0 >> page_shift;
        int page = logical < table_width ? table[logical] : -1;
        int offset = key0 & (page_size - 1);
        if (page < 0) { page = 0; offset = 0; }
        const int y = (page * kv_heads + kv_head) * page_size + offset;
        bf16* k_dst = kv_tiles + (size_t)stage * 2 * TILE_ELEMS + lane * box_rows * 64;
        bf16* v_dst = k_dst + TILE_ELEMS;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          tma_load_2d(&k_map, bar, k_dst + h * (TILE_KV * 64), h * 64, y);
          tma_load_2d(&v_map, bar, v_dst + h * (TILE_KV * 64), h * 64, y);
        }
      }
    };
    for (int j = 0; j < STAGES - 1 && j < tiles; ++j)
      if (warp == j % ATTN_WARPS) issue(j);

    int limit_lo[2], limit_hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = warp * 16 + (lane >> 2) + 8 * i;
      const int position = first_pos + r;
      limit_hi[i] = r < rows ? position : -1;                       // rows past the segment see nothing
      limit_lo[i] = window > 0 ? max(0, position - window + 1) : 0;
    }
    // every row of the warp sees all of a key tile [key0, key0 + 63] if it ends at or before the
    // warp's first position and begins at or after the window start of the warp's last row
    const bool warp_full = warp * 16 + 15 < rows;
    const int warp_first = first_pos + warp * 16;
    const int warp_last = first_pos + min(rows - 1, warp * 16 + 15);
    const int warp_lo = window > 0 ? max(0, warp_last - window + 1) : 0;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
    uint32_t q_frag[D / 16][4];
    cp_async_wait<0>();
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int r = warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      ldmatrix_x4(q_frag[ks], tile_at<D>(q_tile, r, ks * 2 + (lane >> 4)));
    }

    for (int j = 0; j < tiles; ++j) {
      if (j + STAGES - 1 < tiles && warp == (j + STAGES - 1) % ATTN_WARPS) issue(j + STAGES - 1);
      const unsigned load = loads_before + (unsigned)j;
      const int stage = load % STAGES;
      if (!gave_up) gave_up = !mbar_wait(&full_bar[stage], (load / STAGES) & 1u, error_word, 0x52);
      gave_up = __any_sync(0xffffffffu, gave_up);
      bf16* k_tile = kv_tiles + (size_t)stage * 2 * TILE_ELEMS;
      bf16* v_tile = k_tile + TILE_ELEMS;
      const int key0 = (tile_begin + j) * TILE_KV;
      if (key0 < lowest || key0 + TILE_KV - 1 > last_pos) {          // the same answer in every warp
        for (int idx = lane; idx < 16 * CHUNKS; idx += 32) {
          const int r = warp * 16 + idx / CHUNKS, c = idx % CHUNKS;
          if (key0 + r < lowest || key0 + r > last_pos)
            *reinterpret_cast<uint4*>(tile_at<D, true>(v_tile, r, c)) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // a later bulk copy reuses the stage
        __syncthreads();
      }
      // a warp whose rows all end before this tile has nothing to do in it
      if (warp * 16 < rows && key0 <= warp_last) {
        float s[NT][4];
        warp_qk<D, NT, true>(s, q_frag, k_tile, 0, lane);
        if (warp_full && key0 + TILE_KV - 1 <= warp_first && key0 >= warp_lo)
          softmax_step<NT, D / 8, false>(s, o, m, l, key0, limit_lo, limit_hi, scale_log2, lane);
        else
          softmax_step<NT, D / 8, true>(s, o, m, l, key0, limit_lo, limit_hi, scale_log2, lane);
        warp_pv<D, NT, true>(o, s, v_tile, 0, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
    loads_before += (unsigned)tiles;

#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = warp * 16 + (lane >> 2) + 8 * i;
      if (r >= rows) continue;
      const float inv = 1.f / l[i];
      bf16* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * D + (lane & 3) * 2;
#pragma unroll
      for (int t = 0; t < D / 8; ++t)
        *reinterpret_cast<uint32_t*>(dst + t * 8) = pack_bf16(o[t][2 * i] * inv, o[t][2 * i + 1] * inv);
    }
    __syncthreads();                // q_tile and item_shared are rewritten by the next item
  }
  // the CTA that leaves last puts the queue back for the next launch
  if (threadIdx.x == 0) {
    const int left = atomicAdd(&queue[1], 1);
    if (left == (int)gridDim.x - 1) { queue[0] = 0; queue[1] = 0; }
  }
}

// Thread-block clusters: barrier over all CTAs of the cluster (release / acquire), the address of a
// peer CTA's copy of a shared-memory location, and a load from it.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_address(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ float load_cluster_shared(uint32_t address) {
  float value;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(value) : "r"(address) : "memory");
  return value;
}

// The end of both decode kernels: merge the four warps' states (each saw a quarter of the keys) in
// shared memory, write the output if the request has one chunk, else store the chunk's state and
// let the CTA that arrives last for this (request, kv head) merge all chunks in chunk order.
template <int D>
__device__ __forceinline__ void decode_finish(float* merge, int* last_flag_ptr, const float* m, const float* l,
                                              const float (*o)[4], bf16* out, float* scratch, int* counters,
                                              int index, int row, int heads, int kv_heads, int kv_head, int group,
                                              int split, int splits, int max_splits, int cluster_size = 0) {
  constexpr int STATE = D + 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // ---- merge the four warps (each saw a quarter of the keys)
  float* mine = merge + (size_t)warp * 16 * STATE;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int g = (lane >> 2) + 8 * i;
    if ((lane & 3) == 0) { mine[g * STATE] = m[i]; mine[g * STATE + 1] = l[i]; }
#pragma unroll
    for (int t = 0; t < D / 8; ++t) {
      mine[g * STATE + 2 + t * 8 + (lane & 3) * 2] = o[t][2 * i];
      mine[g * STATE + 2 + t * 8 + (lane & 3) * 2 + 1] = o[t][2 * i + 1];
    }
  }
  __syncthreads();
  if (cluster_size > 1) {
    // The chunks of one (request, kv head) are the CTAs of one cluster: each leaves its state in its
    // own shared memory, and after one cluster barrier every CTA merges a slice of the outputs from
    // all of them through distributed shared memory, in chunk order.  No scratch memory, fence or
    // counter in global memory lies on the way.  A CTA without keys (a context shorter than the
    // grid's chunks) contributes max -inf and takes part in the barriers like the others.
    float* cta_state = merge + (size_t)ATTN_WARPS * 16 * STATE;          // [16][STATE]
    for (int item = threadIdx.x; item < group * D; item += ATTN_THREADS) {
      const int g = item / D, d = item - g * D;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + g) * STATE]);
      float l_all = 0.f, a_all = 0.f;
#pragma unroll
      for (int w = 0; w < ATTN_WARPS; ++w) {
        const float* state = merge + ((size_t)w * 16 + g) * STATE;
        const float factor = m_all == -INFINITY ? 0.f : exp2f(state[0] - m_all);
        l_all += state[1] * factor;
        a_all += state[2 + d] * factor;
      }
      cta_state[g * STATE + 2 + d] = a_all;
      if (d == 0) { cta_state[g * STATE] = m_all; cta_state[g * STATE + 1] = l_all; }
    }
    cluster_sync();
    const int total = group * D, per = (total + cluster_size - 1) / cluster_size;
    const int end = min(total, (split + 1) * per);
    for (int item = split * per + threadIdx.x; item < end; item += ATTN_THREADS) {
      const int g = item / D, d = item - g * D;
      const uint32_t local = smem_u32(cta_state + g * STATE);
      float ms[16], ls[16], as[16];
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        ms[s] = -INFINITY; ls[s] = 0.f; as[s] = 0.f;
        if (s < cluster_size) {
          const uint32_t remote = cluster_address(local, (uint32_t)s);
          ms[s] = load_cluster_shared(remote);
          ls[s] = load_cluster_shared(remote + 4);
          as[s] = load_cluster_shared(remote + 8 + (uint32_t)d * 4);
        }
      }
      float m_all = -INFINITY;
#pragma unroll
      for (int s = 0; s < 16; ++s) m_all = fmaxf(m_all, ms[s]);
      float l_all = 0.f, a_all = 0.f;
#pragma unroll
      for (int s = 0; s < 16; ++s) {                       // in chunk order
        const float factor = exp2f(ms[s] - m_all);         // a chunk without keys: 0
        l_all += ls[s] * factor;
        a_all += as[s] * factor;
      }
      out[((size_t)row * heads + kv_head * group + g) * D + d] = __float2bfloat16_rn(a_all / l_all);
    }
    cluster_sync();            // no CTA leaves while another may still read its state
    return;
  }
  const size_t state_base = ((size_t)index * heads + kv_head * group) * max_splits;
  for (int item = threadIdx.x; item < group * D; item += ATTN_THREADS) {
    const int g = item / D, d = item - g * D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + g) * STATE]);
    float l_all = 0.f, a_all = 0.f;
#pragma unroll
    for (int w = 0; w < ATTN_WARPS; ++w) {
      const float* state = merge + ((size_t)w * 16 + g) * STATE;
      const float factor = exp2f(state[0] - m_all);      // a warp without keys has m = -inf: factor 0
      l_all += state[1] * factor;
      a_all += state[2 + d] * factor;
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
  if (threadIdx.x == 0) (*last_flag_ptr) = (atomicAdd(&counters[index * kv_heads + kv_head], 1) == splits - 1);
  __syncthreads();
  if (!(*last_flag_ptr)) return;
  __threadfence();
  // (1) every chunk's (max, sum) into shared memory with one round of loads
  float* max_s = merge;                         // [group][splits], later the chunks' weights
  float* sum_s = merge + 16 * max_splits;       // [group][splits]
  float* inv_s = sum_s + 16 * max_splits;       // [group]
  for (int item = threadIdx.x; item < group * splits; item += ATTN_THREADS) {
    const int g = item / splits, s = item - g * splits;
    const float2 pair = __ldcg(reinterpret_cast<const float2*>(
        scratch + (state_base + (size_t)g * max_splits + s) * STATE));
    max_s[g * max_splits + s] = pair.x;
    sum_s[g * max_splits + s] = pair.y;
  }
  __syncthreads();
  // (2) per head: overall max, each chunk's weight exp2(m_s - max), overall sum (chunk order)
  if (threadIdx.x < group) {
    const int g = threadIdx.x;
    float m_all = -INFINITY;
    for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, max_s[g * max_splits + s]);
    float l_all = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float factor = exp2f(max_s[g * max_splits + s] - m_all);
      max_s[g * max_splits + s] = factor;
      l_all += sum_s[g * max_splits + s] * factor;
    }
    inv_s[g] = 1.f / l_all;
  }
  __syncthreads();
  // (3) weighted sum of the chunks' accumulators; the loads of four outputs and eight chunks are
  // issued together so that their latencies overlap, the additions run in chunk order
  constexpr int PER_PASS = 4;
  for (int item0 = threadIdx.x; item0 < group * D; item0 += ATTN_THREADS * PER_PASS) {
    float total[PER_PASS];
#pragma unroll
    for (int i = 0; i < PER_PASS; ++i) total[i] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 8) {
      float part[PER_PASS][8];
#pragma unroll
      for (int i = 0; i < PER_PASS; ++i) {
        const int item = item0 + i * ATTN_THREADS;
        const int g = min(item / D, group - 1), d = item % D;
        const float* states = scratch + (state_base + (size_t)g * max_splits) * STATE + 2 + d;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          part[i][j] = (item < group * D && s0 + j < splits) ? __ldcg(&states[(size_t)(s0 + j) * STATE]) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < PER_PASS; ++i) {
        const int g = min((item0 + i * ATTN_THREADS) / D, group - 1);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (s0 + j < splits) total[i] += part[i][j] * max_s[g * max_splits + s0 + j];
      }
    }
#pragma unroll
    for (int i = 0; i < PER_PASS; ++i) {
      const int item = item0 + i * ATTN_THREADS;
      if (item < group * D) {
        const int g = item / D, d = item % D;
        out[((size_t)row * heads + kv_head * group + g) * D + d] = __float2bfloat16_rn(total[i] * inv_s[g]);
      }
    }
  }
  if (threadIdx.x == 0) counters[index * kv_heads + kv_head] = 0;
}

// ------------------------------------------------------------------------------------------ decode
// STAGES: 64-key tiles in flight per CTA.  Four when a chunk is short and CTAs are few (every load
// of the chunk is requested at once); two when chunks are long and CTAs many (four CTAs then
// fit on an SM and hide one another's waits).
template <int D, int DECODE_STAGES>
__global__ void __launch_bounds__(ATTN_THREADS)
decode_attention_mma_kernel(const bf16* q, const bf16* k_pool, const bf16* v_pool,
                            bf16* __restrict__ out, const int* __restrict__ decode_seg,
                            const int* __restrict__ seg_q_start, const int* __restrict__ seg_pos0,
                            const int* __restrict__ block_table, const int* __restrict__ seg_slot, int table_width, int heads, int kv_heads,
                            int page_size, int page_shift, int window, float scale_log2, int chunk,
                            float* __restrict__ scratch,
                            int* __restrict__ counters, int max_splits) {
  pdl_trigger();
  pdl_wait();
  extern __shared__ __align__(128) uint8_t attn_shared[];
  bf16* q_tile = reinterpret_cast<bf16*>(attn_shared);            // [16][D], rows >= group are zeros
  bf16* k_tiles = q_tile + 16 * D;                                 // STAGES x [64][D]
  bf16* v_tiles = k_tiles + DECODE_STAGES * TILE_KV * D;           // STAGES x [64][D]
  float* merge = reinterpret_cast<float*>(v_tiles + DECODE_STAGES * TILE_KV * D);   // [4 warps][16][D + 2]
  __shared__ int last_flag;

  const int group = heads / kv_heads;
  const int split = blockIdx.x, kv_head = blockIdx.y, index = blockIdx.z;
  const int seg = decode_seg[index];
  const int row = seg_q_start[seg];
  const int position = seg_pos0[seg];
  const int lowest = window > 0 ? max(0, position - window + 1) : 0;
  const int first_chunk = lowest / chunk;
  const int splits = position / chunk - first_chunk + 1;
  if (split >= splits) return;
  const int k_begin = max(lowest, (first_chunk + split) * chunk);
  const int k_end = min(position + 1, (first_chunk + split + 1) * chunk);   // exclusive
  const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_begin = k_begin / TILE_KV, tile_end = (k_end - 1) / TILE_KV;   // inclusive
  const int tiles = tile_end - tile_begin + 1;

  constexpr int CHUNKS = D / 8;
  for (int item = threadIdx.x; item < 16 * CHUNKS; item += ATTN_THREADS) {
    const int g = item / CHUNKS, c = item - g * CHUNKS;
    const bool valid = g < group;
    const bf16* src = valid ? q + ((size_t)row * heads + kv_head * group + g) * D + c * 8 : q;
    cp_async_16(tile_at<D>(q_tile, g, c), src, valid);
  }
  // request the first tiles of the chunk at once: their latencies overlap
#pragma unroll
  for (int s = 0; s < DECODE_STAGES; ++s) {
    if (s < tiles) {
      load_kv_tile<D>(k_tiles + s * TILE_KV * D, k_pool, table, (tile_begin + s) * TILE_KV, TILE_KV, k_begin, k_end - 1,
                      kv_heads, kv_head, page_size, page_shift);
      load_kv_tile<D>(v_tiles + s * TILE_KV * D, v_pool, table, (tile_begin + s) * TILE_KV, TILE_KV, k_begin, k_end - 1,
                      kv_heads, kv_head, page_size, page_shift);
    }
    cp_async_commit();     // one group per stage, empty or not, so that the wait counts line up
  }

  int limit_lo[2] = {k_begin, k_begin}, limit_hi[2];
  limit_hi[0] = (lane >> 2) < group ? k_end - 1 : -1;          // rows that are no real head see nothing
  limit_hi[1] = (lane >> 2) + 8 < group ? k_end - 1 : -1;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  uint32_t q_frag[D / 16][4];

  for (int t = 0; t < tiles; ++t) {
    const int stage = t % DECODE_STAGES;
    cp_async_wait<DECODE_STAGES - 1>();
    __syncthreads();
    if (t == 0) {
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(q_frag[ks], tile_at<D>(q_tile, r, ks * 2 + (lane >> 4)));
      }
    }
    const int key0 = (tile_begin + t) * TILE_KV + warp * 16;     // this warp's 16 keys of the tile
    if (key0 < k_end && key0 + 16 > k_begin) {
      float s[2][4];
      warp_qk<D, 2>(s, q_frag, k_tiles + stage * TILE_KV * D, warp * 16, lane);
      softmax_step<2, D / 8>(s, o, m, l, key0, limit_lo, limit_hi, scale_log2, lane);
      warp_pv<D, 2>(o, s, v_tiles + stage * TILE_KV * D, warp * 16, lane);
    }
    __syncthreads();
    if (t + DECODE_STAGES < tiles) {
      load_kv_tile<D>(k_tiles + stage * TILE_KV * D, k_pool, table, (tile_begin + t + DECODE_STAGES) * TILE_KV, TILE_KV,
                      k_begin, k_end - 1, kv_heads, kv_head, page_size, page_shift);
      load_kv_tile<D>(v_tiles + stage * TILE_KV * D, v_pool, table, (tile_begin + t + DECODE_STAGES) * TILE_KV, TILE_KV,
                      k_begin, k_end - 1, kv_heads, kv_head, page_size, page_shift);
    }
    cp_async_commit();
  }

  decode_finish<D>(merge, &last_flag, m, l, o, out, scratch, counters, index, row, heads, kv_heads, kv_head, group,
                   split, splits, max_splits);
}

// ------------------------------------------------------------------------------------- decode, TMA
// The decode kernel of choice: the same work as decode_attention_mma_kernel, with K and V brought in
// by the tensor memory accelerator and no CTA-wide barrier in the loop.
//
// The pools are described as [pages * kv_heads * page_size, D] matrices; one cp.async.bulk.tensor
// per page (and per 64-column half) lands a page's keys of one kv head in the 128-byte-swizzled
// tile that ldmatrix reads, and an mbarrier per stage counts the bytes.  No thread computes an
// address per 16 bytes.  Each warp owns whole tiles of TKV keys (tile t of the chunk belongs to
// warp t % 4) and its own ring of STAGES stages: it waits for its tile, computes, and - being the
// only reader - refills the stage itself.  The warps meet once, for the merge of their states.
// For page sizes that are a power of two >= 8 (larger pages are read in boxes of TKV keys).
//
// Slots of pages the request does not hold (beyond its last page, or released by the window) are
// filled from page 0 of the pool.  Keys outside the chunk's range - those slots, the rest of the
// last page, keys the window has passed - get the score -inf whatever was loaded, and their V rows
// are overwritten with zeros in shared memory before use (only a chunk's first and last tile can
// hold such keys), so that nothing a request does not own reaches its result.
//
// Fused position encoding (qkv != null): the kernel takes the projection's raw output
// [tokens, (heads + 2 kv_heads) * D] instead of rotated queries.  Every CTA rotates its group's
// queries while it fills the Q tile (rotate-half pairs, angle = position * inv_freq[i], float32,
// exactly as the stand-alone kernel does); the CTA that holds the request's newest position rotates
// the new key, and puts it and the new value both into the cache pages (if write_kv) and into its
// own tile in shared memory, over the stale row the bulk copy delivered.  No kernel in between.
//
// With even_split every request divides its own context evenly over the grid's max_splits chunks
// (the host fixes only their number), so a launch captured in a CUDA graph adapts to the contexts
// of each replay.
//
// Chunks other than a request's last hold no key of this step, so their first loads are issued
// before the wait on the previous kernel (which writes this step's keys); the rotation's angles and
// the new token's cache slot are taken before that wait too, and the step's key and value are
// fetched right after it, beside the queries.
// The stages are reused as the merge area once every warp has consumed its last tile.
//
// Merge of a request's chunks.  With cluster_merge the launch's chunks of one (request, kv head)
// are the CTAs of one thread-block cluster (2..16 of them): each leaves its state in its own
// shared memory, and after one cluster barrier every CTA merges a slice of the outputs from all of
// them through distributed shared memory, in chunk order; a second barrier keeps every CTA's
// memory alive until the others have read it.  Inside a captured decode step of the 0.5B sizes this
// costs 10.7 us per layer against 15.2 us for the other way: partial states to scratch memory, a
// fence, a counter, and the CTA that arrives last merging them.  That way remains for launches
// with more chunks or more clusters than run together.
template <int D, int TKV, int STAGES>
__global__ void __launch_bounds__(ATTN_THREADS, 3)     // three CTAs per SM with one stage: at most 168 registers
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            const bf16* q, bf16* __restrict__ out, const int* __restrict__ decode_seg,
                            const int* __restrict__ seg_q_start, const int* __restrict__ seg_pos0,
                            const int* __restrict__ block_table, const int* __restrict__ seg_slot, int table_width, int heads, int kv_heads,
                            int page_size, int page_shift, int window, float scale_log2, int chunk_arg,
                            int even_split, float* __restrict__ scratch, int* __restrict__ counters,
                            int max_splits, int* error_word, const bf16* qkv, const float* __restrict__ inv_freq,
                            const long long* __restrict__ slots, bf16* k_pool_w, bf16* v_pool_w, int write_kv,
                            int cluster_merge) {
  constexpr int HALVES = D / 64;
  constexpr int TILE_ELEMS = TKV * D;
  constexpr int NT = TKV / 8;
  extern __shared__ uint8_t attn_shared_raw[];
  uint8_t* aligned = (uint8_t*)(((uintptr_t)attn_shared_raw + 1023) & ~(uintptr_t)1023);
  bf16* kv_tiles = reinterpret_cast<bf16*>(aligned);      // [warp][stage] x (K [TKV][D], V [TKV][D])
  bf16* q_tile = kv_tiles + (size_t)ATTN_WARPS * STAGES * 2 * TILE_ELEMS;   // [16][D], rows >= group are zeros
  float* merge = reinterpret_cast<float*>(aligned);       // after the loop: [4 warps][16][D + 2]
  __shared__ uint64_t full_bar[ATTN_WARPS][STAGES];
  __shared__ int last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Step metadata was copied to the device before the first kernel of the step: safe to read at
  // once, and asked for before the barriers are set up, since every round trip to memory up to the
  // first bulk copy lies on the launch's critical path.
  const int group = heads / kv_heads;
  const int split = blockIdx.x, kv_head = blockIdx.y, index = blockIdx.z;
  // decode_seg null: every segment of the step is one decoded row, so segment and row are the index
  // itself (one round trip less)
  const int seg = decode_seg != nullptr ? decode_seg[index] : index;
  const int row = decode_seg != nullptr ? seg_q_start[seg] : index;
  const int position = seg_pos0[seg];
  const int table_row = seg_slot != nullptr ? seg_slot[seg] : seg;
  // the rotation's frequencies (of pair threadIdx.x % HALF for the queries; of pairs lane, lane + 32, ..
  // for the step's key, should this CTA turn out to hold it)
  constexpr int HALF = D / 2;
  const bool fused = qkv != nullptr;
  float query_frequency = 0.f, key_frequency[HALF / 32];
  if (fused) {
    query_frequency = inv_freq[threadIdx.x % HALF];
#pragma unroll
    for (int j = 0; j < HALF / 32; ++j) key_frequency[j] = inv_freq[lane + 32 * j];
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < ATTN_WARPS * STAGES; ++i) mbar_init(&full_bar[0][0] + i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
  }
  pdl_trigger();
  __syncthreads();
  const int lowest = window > 0 ? max(0, position - window + 1) : 0;
  // even_split: the request's own context divided over the grid's chunks (at least chunk_arg keys
  // each), so that one captured launch fits every context length; else chunks of chunk_arg keys
  int chunk = chunk_arg;
  if (even_split) chunk = max(chunk_arg, ((position + max_splits) / max_splits + TKV - 1) / TKV * TKV);
  const int first_chunk = lowest / chunk;
  const int splits = position / chunk - first_chunk + 1;
  // A CTA beyond the request's chunks has nothing to do; as a member of a cluster that merges
  // through shared memory it stays, without keys, for the cluster's barriers.
  const bool idle = split >= splits;
  if (splits == 1) cluster_merge = 0;       // one chunk (the same answer in every CTA of the cluster): nothing to merge
  if (idle && !cluster_merge) return;
  const int k_begin = max(lowest, (first_chunk + split) * chunk);
  const int k_end = min(position + 1, (first_chunk + split + 1) * chunk);   // exclusive
  const int* table = block_table + (size_t)table_row * table_width;
  const int tile_begin = k_begin / TKV, tile_end = (k_end - 1) / TKV;       // inclusive
  const int tiles = idle ? 0 : tile_end - tile_begin + 1;
  const int my_tiles = tiles > warp ? (tiles - warp + ATTN_WARPS - 1) / ATTN_WARPS : 0;   // tiles warp, warp + 4, ..

  // lane j fetches the j-th page (or the one TKV-key box) of the warp's n-th tile, K and V
  const int boxes = page_size >= TKV ? 1 : TKV >> page_shift;
  const int box_rows = page_size >= TKV ? TKV : page_size;
  bf16* my_stages = kv_tiles + (size_t)warp * STAGES * 2 * TILE_ELEMS;
  // The pool row (the bulk copy's y) of this lane's box of the warp's n-th tile: one read of the
  // block table, asked for ahead of the copy so that its round trip does not delay the copy.
  auto lookup = [&](int n) -> int {
    if (lane >= boxes) return 0;
    const int key0 = (tile_begin + warp + n * ATTN_WARPS) * TKV + lane * box_rows;
    const int logical = key0 >> page_shift;
    int page = logical < table_width ? table[logical] : -1;
    int offset = key0 & (page_size - 1);
    if (page < 0) { page = 0; offset = 0; }
    return (page * kv_heads + kv_head) * page_size + offset;
  };
  auto issue = [&](int n, int y) {
    const int stage = n % STAGES;
    uint64_t* bar = &full_bar[warp][stage];
    if (lane == 0) mbar_expect_tx(bar, 2u * TILE_ELEMS * 2u);
    __syncwarp();
    if (lane < boxes) {
      bf16* k_dst = my_stages + (size_t)stage * 2 * TILE_ELEMS + lane * box_rows * 64;
      bf16* v_dst = k_dst + TILE_ELEMS;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tma_load_2d(&k_map, bar, k_dst + h * (TKV * 64), h * 64, y);
        tma_load_2d(&v_map, bar, v_dst + h * (TKV * 64), h * 64, y);
      }
    }
  };
  const bool holds_new_key = split == splits - 1;
  const bool inject = fused && write_kv != 0 && holds_new_key;   // this CTA stores the step's key and value
  // The newest key's row is stale in the pool until this step stores it: a CTA that reads it from
  // the pool waits for the previous kernel first; one that overwrites it in shared memory need not.
  const bool early = !holds_new_key || inject;
  // The first ring-full of tiles: all table reads, then all copies.
  int first_rows[STAGES];
#pragma unroll
  for (int n = 0; n < STAGES; ++n) first_rows[n] = n < my_tiles ? lookup(n) : 0;
  if (early) {
#pragma unroll
    for (int n = 0; n < STAGES; ++n)
      if (n < my_tiles) issue(n, first_rows[n]);
  }
  // The rotation's angles depend on the position only: taken before the wait, like the new token's
  // cache slot, so that after it only the values themselves are fetched.
  constexpr int CHUNKS = D / 8;
  float sine = 0.f, cosine = 1.f;            // of pair threadIdx.x % HALF (the same for all of a thread's query items)
  float key_sine[HALF / 32], key_cosine[HALF / 32];     // of pairs lane, lane + 32, ..: the new key's
  long long new_slot = -1;
  if (fused) {
    if (inject) new_slot = slots[row];
    sincosf((float)position * query_frequency, &sine, &cosine);
    if (inject) {
#pragma unroll
      for (int j = 0; j < HALF / 32; ++j) sincosf((float)position * key_frequency[j], &key_sine[j], &key_cosine[j]);
    }
  }
  pdl_wait();
  if (!early) {
#pragma unroll
    for (int n = 0; n < STAGES; ++n)
      if (n < my_tiles) issue(n, first_rows[n]);
  }

  const size_t qkv_width = (size_t)(heads + 2 * kv_heads) * D;
  // The warp whose tile holds the newest position fetches the step's key and value now, beside the
  // queries, instead of when it reaches that tile.
  const int newest_tile = position / TKV - tile_begin;          // among this chunk's tiles, if it holds it
  const bool owns_newest = inject && newest_tile % ATTN_WARPS == warp;
  bf16 new_key[HALF / 32][2], new_value[D / 32];
  if (owns_newest) {
    const bf16* k_src = qkv + (size_t)row * qkv_width + (size_t)(heads + kv_head) * D;
    const bf16* v_src = k_src + (size_t)kv_heads * D;
#pragma unroll
    for (int j = 0; j < HALF / 32; ++j) {
      new_key[j][0] = k_src[lane + 32 * j];
      new_key[j][1] = k_src[lane + 32 * j + HALF];
    }
#pragma unroll
    for (int j = 0; j < D / 32; ++j) new_value[j] = v_src[lane + 32 * j];
  }
  if (fused) {
    // thread -> pair index i (the same for all its items, as 128 % HALF == 0) and rows g0, g0 + 128/HALF, ..
    const int i = threadIdx.x % HALF;
    const bf16* q_row = qkv + (size_t)row * qkv_width + (size_t)kv_head * group * D;
    constexpr int STEP = ATTN_THREADS / HALF, MINE = 16 / STEP;     // this thread's rows: g0, g0 + STEP, ..
    const int g0 = threadIdx.x / HALF;
    bf16 low[MINE], high[MINE];                                     // every load before the first store
#pragma unroll
    for (int j = 0; j < MINE; ++j) {
      const int g = g0 + j * STEP;
      low[j] = g < group ? q_row[g * D + i] : __float2bfloat16_rn(0.f);
      high[j] = g < group ? q_row[g * D + i + HALF] : __float2bfloat16_rn(0.f);
    }
#pragma unroll
    for (int j = 0; j < MINE; ++j) {
      const int g = g0 + j * STEP;
      float y1, y2;
      rotate_pair(__bfloat162float(low[j]), __bfloat162float(high[j]), sine, cosine, &y1, &y2);
      tile_at<D>(q_tile, g, i >> 3)[i & 7] = __float2bfloat16_rn(y1);
      tile_at<D>(q_tile, g, (i + HALF) >> 3)[(i + HALF) & 7] = __float2bfloat16_rn(y2);
    }
  } else {
    for (int item = threadIdx.x; item < 16 * CHUNKS; item += ATTN_THREADS) {
      const int g = item / CHUNKS, c = item - g * CHUNKS;
      const bool valid = g < group;
      const bf16* src = valid ? q + ((size_t)row * heads + kv_head * group + g) * D + c * 8 : q;
      cp_async_16(tile_at<D>(q_tile, g, c), src, valid);
    }
  }
  cp_async_commit();

  // Rows that are no real head (the group padded to the MMA's 16 rows) have zero queries; their
  // states are computed like the others and never stored.
  int limit_lo[2] = {k_begin, k_begin}, limit_hi[2] = {k_end - 1, k_end - 1};
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[D / 8][4];
#pragma unroll
  for (int t = 0; t < D / 8; ++t) o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.f;
  uint32_t q_frag[D / 16][4];
  cp_async_wait<0>();
  __syncthreads();
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int r = (lane & 7) + (((lane >> 3) & 1) << 3);
    ldmatrix_x4(q_frag[ks], tile_at<D>(q_tile, r, ks * 2 + (lane >> 4)));
  }

  bool gave_up = false;       // after one wait ran out, later waits are skipped: the kernel ends, the host raises
  for (int n = 0; n < my_tiles; ++n) {
    const int stage = n % STAGES;
    const int refill_row = n + STAGES < my_tiles ? lookup(n + STAGES) : 0;     // in flight during this tile
    if (!gave_up) gave_up = !mbar_wait(&full_bar[warp][stage], (uint32_t)(n / STAGES) & 1u, error_word, 0x41);
    gave_up = __any_sync(0xffffffffu, gave_up);                  // warp-uniform: the warp issues as one
    bf16* k_tile = my_stages + (size_t)stage * 2 * TILE_ELEMS;
    bf16* v_tile = k_tile + TILE_ELEMS;
    const int key0 = (tile_begin + warp + n * ATTN_WARPS) * TKV;
    if (inject && warp + n * ATTN_WARPS == newest_tile) {
      // the step's own key and value: into the pages and over the stale row of this tile
      const int r = position - key0;
      const long long slot = new_slot;
      const long long page = slot / page_size;
      const size_t at = (((size_t)page * kv_heads + kv_head) * page_size + (size_t)(slot - page * page_size)) * D;
#pragma unroll
      for (int j = 0; j < HALF / 32; ++j) {
        const int i = lane + 32 * j;
        float r1, r2;
        rotate_pair(__bfloat162float(new_key[j][0]), __bfloat162float(new_key[j][1]), key_sine[j], key_cosine[j], &r1, &r2);
        const bf16 y1 = __float2bfloat16_rn(r1), y2 = __float2bfloat16_rn(r2);
        tile_at<D, true, TKV>(k_tile, r, i >> 3)[i & 7] = y1;
        tile_at<D, true, TKV>(k_tile, r, (i + HALF) >> 3)[(i + HALF) & 7] = y2;
        if (slot >= 0) { k_pool_w[at + i] = y1; k_pool_w[at + i + HALF] = y2; }
      }
#pragma unroll
      for (int j = 0; j < D / 32; ++j) {
        const int i = lane + 32 * j;
        const bf16 v = new_value[j];
        tile_at<D, true, TKV>(v_tile, r, i >> 3)[i & 7] = v;
        if (slot >= 0) v_pool_w[at + i] = v;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
    }
    float s[NT][4];
    if (key0 < k_begin || key0 + TKV > k_end) {
      // a ragged tile: zero the V rows outside the range, mask the scores
      for (int item = lane; item < TKV * CHUNKS; item += 32) {
        const int r = item / CHUNKS, c = item - r * CHUNKS;
        if (key0 + r < k_begin || key0 + r >= k_end)
          *reinterpret_cast<uint4*>(tile_at<D, true, TKV>(v_tile, r, c)) = make_uint4(0u, 0u, 0u, 0u);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // a later bulk copy reuses the stage
      __syncwarp();
      warp_qk<D, NT, true, TKV>(s, q_frag, k_tile, 0, lane);
      softmax_step<NT, D / 8, true>(s, o, m, l, key0, limit_lo, limit_hi, scale_log2, lane);
    } else {
      warp_qk<D, NT, true, TKV>(s, q_frag, k_tile, 0, lane);
      softmax_step<NT, D / 8, false>(s, o, m, l, key0, limit_lo, limit_hi, scale_log2, lane);
    }
    warp_pv<D, NT, true, TKV>(o, s, v_tile, 0, lane);
    __syncwarp();                                                // every lane is done with this stage
    if (n + STAGES < my_tiles && !gave_up) issue(n + STAGES, refill_row);
  }
  // No load is in flight here: every issued tile was waited for (or its wait ran out after a second).
  __syncthreads();                                               // the merge area overlays the stages
  decode_finish<D>(merge, &last_flag, m, l, o, out, scratch, counters, index, row, heads, kv_heads, kv_head, group,
                   split, splits, max_splits, cluster_merge ? max_splits : 0);
}

// Opt in to more than 48 KB of dynamic shared memory, once per kernel and size (the attribute call
// costs the host a microsecond or two, and eager steps launch these kernels once per layer).
template <typename Kernel>
static int set_shared(Kernel kernel, size_t bytes) {
  if (bytes <= 48 * 1024) return MLR_OK;
  static Kernel known[16];
  static size_t granted[16];
  static int count = 0;
  for (int i = 0; i < count; ++i)
    if (known[i] == kernel && granted[i] >= bytes) return MLR_OK;
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (err != cudaSuccess) return (int)err;
  if (count < 16) { known[count] = kernel; granted[count] = bytes; ++count; }
  return MLR_OK;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

constexpr float LOG2_E = 1.4426950408889634f;

static int shift_of(int page_size) {
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) return shift;
  return -1;
}

// Prompt portions: tiles of up to 64 rows of one segment (tile_seg, tile_row0).
MLR_EXPORT int mlr_attention_prefill_mma(const void* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                         const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                                         int table_width, int tiles, int heads, int kv_heads, int head_dim,
                                         int page_size, int window, float scale, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || table_width <= 0)
    return MLR_BAD_SIZE;
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  if (heads > 65535) return MLR_TOO_LARGE;
  const size_t shared = (size_t)(TILE_Q + 4 * TILE_KV) * head_dim * 2;
  const int page_shift = shift_of(page_size);
  dim3 grid(tiles, heads);
  int status;
  if (head_dim == 64) {
    if ((status = set_shared(prefill_attention_kernel<64>, shared)) != MLR_OK) return status;
    launch_kernel(prefill_attention_kernel<64>, dim3(grid), dim3(ATTN_THREADS), shared, stream, 
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, tile_seg, tile_row0, seg_q_start,
        seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads, page_size, page_shift, window, scale * LOG2_E);
  } else {
    if ((status = set_shared(prefill_attention_kernel<128>, shared)) != MLR_OK) return status;
    launch_kernel(prefill_attention_kernel<128>, dim3(grid), dim3(ATTN_THREADS), shared, stream, 
        (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, tile_seg, tile_row0, seg_q_start,
        seg_q_len, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads, page_size, page_shift, window, scale * LOG2_E);
  }
  return launch_status();
}

// Decoded tokens: same contract as mlr_attention_decode (same scratch layout and counters).
MLR_EXPORT int mlr_attention_decode_mma(const void* q, const void* k_pool, const void* v_pool, void* out,
                                        const int* decode_seg, const int* seg_q_start, const int* seg_pos0,
                                        const int* block_table, const int* seg_slot, int table_width, int rows, int heads, int kv_heads,
                                        int head_dim, int page_size, int window, float scale, int chunk,
                                        int max_splits, void* scratch, int* counters, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || chunk <= 0 ||
      chunk % TILE_KV != 0 || max_splits <= 0 || table_width <= 0)
    return MLR_BAD_SIZE;
  if (heads / kv_heads > 16 || rows > 65535 || kv_heads > 65535) return MLR_TOO_LARGE;
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  // the final merge keeps 2 * 16 * max_splits + 16 floats in the warps' merge area
  if ((size_t)(2 * 16 * max_splits + 16) > (size_t)ATTN_WARPS * 16 * (head_dim + 2)) return MLR_TOO_LARGE;
  // long chunks on a grid of several waves: fewer stages, more CTAs per SM
  const bool deep = chunk <= 4 * TILE_KV || (long long)max_splits * kv_heads * rows <= 2 * sm_count();
  const int stages = deep ? 4 : 2;
  const size_t shared = (size_t)(16 + 2 * stages * TILE_KV) * head_dim * 2 +
                        (size_t)ATTN_WARPS * 16 * (head_dim + 2) * sizeof(float);
  dim3 grid(max_splits, kv_heads, rows);
  const int page_shift = shift_of(page_size);
  int status;
#define MLR_LAUNCH_DECODE(D_, S_)                                                                          \
  do {                                                                                                     \
    if ((status = set_shared(decode_attention_mma_kernel<D_, S_>, shared)) != MLR_OK) return status;       \
    launch_kernel(decode_attention_mma_kernel<D_, S_>, dim3(grid), dim3(ATTN_THREADS), shared, stream,     \
                  (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, (bf16*)out, decode_seg,        \
                  seg_q_start, seg_pos0, block_table, seg_slot, table_width, heads, kv_heads, page_size, page_shift, \
                  window, scale * LOG2_E, chunk, (float*)scratch, counters, max_splits);                   \
  } while (0)
  if (head_dim == 64) {
    if (deep) MLR_LAUNCH_DECODE(64, 4); else MLR_LAUNCH_DECODE(64, 2);
  } else {
    if (deep) MLR_LAUNCH_DECODE(128, 4); else MLR_LAUNCH_DECODE(128, 2);
  }
#undef MLR_LAUNCH_DECODE
  return launch_status();
}

// Decoded tokens with K/V fetched by the tensor memory accelerator.  Same contract as
// mlr_attention_decode_mma plus: pool_pages = pages in each pool (for the tensor maps), page_size a
// power of two >= 8, even_split (chunk is then the smallest chunk; each request divides its context
// over max_splits chunks), stages = tiles per warp in flight or in use (0 = default), error_word =
// host-visible int that receives a code if a wait runs out.  qkv != null: the fused position
// encoding described at the kernel (q is then unused; inv_freq [head_dim/2] float32; slots [tokens]
// int64, page * page_size + offset of each token's cache slot; write_kv = 0 leaves the pages alone).
// cluster_merge != 0 (2 <= max_splits <= 16): the chunks merge through their cluster's shared
// memory, and scratch and counters are not touched.
MLR_EXPORT int mlr_attention_decode_tma(const void* q, const void* k_pool, const void* v_pool, void* out,
                                        const int* decode_seg, const int* seg_q_start, const int* seg_pos0,
                                        const int* block_table, const int* seg_slot, int table_width, int rows, int heads, int kv_heads,
                                        int head_dim, int page_size, int pool_pages, int window, float scale,
                                        int chunk, int even_split, int max_splits, int stages, void* scratch,
                                        int* counters, int* error_word, const void* qkv, const float* inv_freq,
                                        const long long* slots, int write_kv, int cluster_merge, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || chunk <= 0 ||
      chunk % TILE_KV != 0 || max_splits <= 0 || table_width <= 0 || pool_pages <= 0 || error_word == nullptr)
    return MLR_BAD_SIZE;
  if (heads / kv_heads > 16 || rows > 65535 || kv_heads > 65535) return MLR_TOO_LARGE;
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  if (qkv != nullptr && (inv_freq == nullptr || slots == nullptr)) return MLR_BAD_SIZE;
  const int page_shift = shift_of(page_size);
  if (page_shift < 3) return MLR_BAD_SIZE;
  if (((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15)) return MLR_BAD_ALIGNMENT;
  const long long pool_rows = (long long)pool_pages * kv_heads * page_size;
  if (pool_rows >= (1ll << 31)) return MLR_TOO_LARGE;           // tile coordinates are 32-bit
  if ((size_t)(2 * 16 * max_splits + 16) > (size_t)ATTN_WARPS * 16 * (head_dim + 2)) return MLR_TOO_LARGE;
  const int tile_keys = (head_dim == 64 && stages < 10) || stages == 21 ? 64 : 32;
  const int box_rows = page_size >= tile_keys ? tile_keys : page_size;
  CUtensorMap k_map, v_map;
  if (!cached_tile_map(&k_map, k_pool, pool_rows, head_dim, box_rows) ||
      !cached_tile_map(&v_map, v_pool, pool_rows, head_dim, box_rows))
    return MLR_BAD_SIZE;
  dim3 grid(max_splits, kv_heads, rows);
  // cluster_merge: the chunks of a (request, kv head) form one thread-block cluster (the grid's x
  // extent, at most 16 CTAs; more than 8 is the hardware's non-portable size) and merge through
  // shared memory; otherwise through scratch memory and counters.
  if (cluster_merge && (max_splits < 2 || max_splits > 16)) return MLR_BAD_SIZE;
  int status;
#define MLR_LAUNCH_DECODE_TMA(D_, T_, S_)                                                                  \
  do {                                                                                                     \
    const size_t shared = 1024 + (size_t)(16 + 2 * ATTN_WARPS * S_ * T_) * D_ * 2;                         \
    static_assert((size_t)(ATTN_WARPS + 1) * 16 * (D_ + 2) * 4 <= (size_t)2 * ATTN_WARPS * S_ * T_ * D_ * 2, "merge area"); \
    if ((status = set_shared(decode_attention_tma_kernel<D_, T_, S_>, shared)) != MLR_OK) return status;   \
    if (cluster_merge) {                                                                                   \
      static bool wide_clusters = false;                                                                   \
      if (max_splits > 8 && !wide_clusters) {                                                              \
        cudaError_t err = cudaFuncSetAttribute(decode_attention_tma_kernel<D_, T_, S_>,                     \
                                               cudaFuncAttributeNonPortableClusterSizeAllowed, 1);        \
        if (err != cudaSuccess) return (int)err;                                                           \
        wide_clusters = true;                                                                              \
      }                                                                                                    \
      launch_kernel_clustered_balanced(decode_attention_tma_kernel<D_, T_, S_>, dim3(grid), dim3(ATTN_THREADS), shared, stream, \
                  max_splits, k_map, v_map, (const bf16*)q, (bf16*)out, decode_seg, seg_q_start, seg_pos0, block_table, seg_slot, \
                  table_width, heads, kv_heads, page_size, page_shift, window, scale * LOG2_E, chunk,      \
                  even_split, (float*)scratch, counters, max_splits, error_word, (const bf16*)qkv, inv_freq, \
                  slots, (bf16*)const_cast<void*>(k_pool), (bf16*)const_cast<void*>(v_pool), write_kv, 1);  \
    } else {                                                                                               \
      launch_kernel(decode_attention_tma_kernel<D_, T_, S_>, dim3(grid), dim3(ATTN_THREADS), shared, stream, \
                  k_map, v_map, (const bf16*)q, (bf16*)out, decode_seg, seg_q_start, seg_pos0, block_table, seg_slot, \
                  table_width, heads, kv_heads, page_size, page_shift, window, scale * LOG2_E, chunk,      \
                  even_split, (float*)scratch, counters, max_splits, error_word, (const bf16*)qkv, inv_freq, \
                  slots, (bf16*)const_cast<void*>(k_pool), (bf16*)const_cast<void*>(v_pool), write_kv, 0);  \
    }                                                                                                      \
  } while (0)
  // stages: tiles each warp keeps in flight or in use; 0 = the default.  Tiles hold 64 keys
  // (head_dim 64) or 32 keys (head_dim 128): 16 KB of K and V per stage either way.
  if (stages == 0) stages = 1;       // three CTAs per SM, twelve tiles in flight: measured best at every batch size
  if (head_dim == 64) {
    switch (stages) {
      case 1: MLR_LAUNCH_DECODE_TMA(64, 64, 1); break;
      case 2: MLR_LAUNCH_DECODE_TMA(64, 64, 2); break;
      case 3: MLR_LAUNCH_DECODE_TMA(64, 64, 3); break;
      case 12: MLR_LAUNCH_DECODE_TMA(64, 32, 2); break;    // 32-key tiles, two in flight: for chunks of many tiles
      case 13: MLR_LAUNCH_DECODE_TMA(64, 32, 3); break;
      case 14: MLR_LAUNCH_DECODE_TMA(64, 32, 4); break;
      default: return MLR_BAD_SIZE;
    }
  } else {
    switch (stages) {
      case 1: MLR_LAUNCH_DECODE_TMA(128, 32, 1); break;
      case 2: MLR_LAUNCH_DECODE_TMA(128, 32, 2); break;
      case 3: MLR_LAUNCH_DECODE_TMA(128, 32, 3); break;
      case 21: MLR_LAUNCH_DECODE_TMA(128, 64, 1); break;   // 64-key tiles, for measurements
      default: return MLR_BAD_SIZE;
    }
  }
#undef MLR_LAUNCH_DECODE_TMA
  return launch_status();
}

// Prompt portions with K/V fetched by the tensor memory accelerator and work drawn from a queue.
// Same contract as mlr_attention_prefill_mma plus: pool_pages = pages in each pool, page_size a power
// of two >= 8, queue = two zeroed ints in device memory (left zeroed), error_word = host-visible
// int that receives a code if a wait runs out.  The tile list is best ordered by falling key count.
MLR_EXPORT int mlr_attention_prefill_tma(const void* q, const void* k_pool, const void* v_pool, void* out,
                                         const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                         const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                                         int table_width, int tiles, int heads, int kv_heads, int head_dim,
                                         int page_size, int pool_pages, int window, float scale, int* queue,
                                         int* error_word, cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 || table_width <= 0 ||
      pool_pages <= 0 || queue == nullptr || error_word == nullptr)
    return MLR_BAD_SIZE;
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  if ((long long)tiles * heads >= (1ll << 30)) return MLR_TOO_LARGE;
  const int page_shift = shift_of(page_size);
  if (page_shift < 3) return MLR_BAD_SIZE;
  if (((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)q & 15)) return MLR_BAD_ALIGNMENT;
  const long long pool_rows = (long long)pool_pages * kv_heads * page_size;
  if (pool_rows >= (1ll << 31)) return MLR_TOO_LARGE;
  const int box_rows = page_size >= TILE_KV ? TILE_KV : page_size;
  CUtensorMap k_map, v_map;
  if (!cached_tile_map(&k_map, k_pool, pool_rows, head_dim, box_rows) ||
      !cached_tile_map(&v_map, v_pool, pool_rows, head_dim, box_rows))
    return MLR_BAD_SIZE;
  int status;
#define MLR_LAUNCH_PREFILL_TMA(D_, S_, PER_SM_)                                                             \
  do {                                                                                                      \
    const size_t shared = 1024 + (size_t)(TILE_Q + 2 * S_ * TILE_KV) * D_ * 2;                              \
    if ((status = set_shared(prefill_attention_tma_kernel<D_, S_>, shared)) != MLR_OK) return status;       \
    const long long items = (long long)tiles * heads;                                                       \
    const int ctas = (int)(items < sm_count() * PER_SM_ ? items : sm_count() * PER_SM_);                                  \
    launch_kernel(prefill_attention_tma_kernel<D_, S_>, dim3(ctas), dim3(ATTN_THREADS), shared, stream,     \
                  k_map, v_map, (const bf16*)q, (bf16*)out, tile_seg, tile_row0, seg_q_start, seg_q_len,    \
                  seg_pos0, block_table, seg_slot, table_width, tiles, heads, kv_heads, page_size, page_shift, window, \
                  scale * LOG2_E, queue, error_word);                                                       \
  } while (0)
  if (head_dim == 64) MLR_LAUNCH_PREFILL_TMA(64, 3, 3); else MLR_LAUNCH_PREFILL_TMA(128, 2, 2);
#undef MLR_LAUNCH_PREFILL_TMA
  return launch_status();
}


