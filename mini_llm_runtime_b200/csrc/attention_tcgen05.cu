// Causal attention of prompt portions over the paged bfloat16 K/V cache on the 5th-generation
// tensor cores (head_dim 64): S = Q K^T and P V run as tcgen05.mma with their results in tensor
// memory; the online softmax runs on the CUDA cores, one thread per query row.
//
// One work item is 128 query rows of one head.  A CTA has five warps:
//   warps 0..3  softmax: thread r owns query row r (tensor-memory lane r).  Per 64-key tile it reads
//               its row of S from tensor memory (64 values), masks (causal limit, window, rows past
//               the portion), keeps the running max and sum, writes the probabilities as bfloat16
//               into a 128-byte-swizzled tile in shared memory (the A operand of P V; two buffers),
//               and only then reads the previous tile's P V from tensor memory (two buffers) and adds
//               it to its output row in registers, times the factor by which the max moved: the MMA
//               runs under the next tile's exponentials.  No shuffles: a row lives in one thread.
//   warp 4      loads and issues: Q by one bulk tensor copy per item, K and V page by page (one
//               copy per page and kv head, as in the other attention kernels) into a ring of
//               stages; one lane issues the MMAs: S_{j+1} = Q K_{j+1}^T goes out before the warp
//               waits for tile j's probabilities (two S buffers), then P_j V_j.  K is the K-major B
//               operand; V ([keys][head_dim], head_dim contiguous) is the MN-major B operand.
// Items are drawn heaviest-first from a counter in global memory by the resident CTAs (two per SM,
// so one CTA's MMAs run under the other's softmax).
//
// Semantics as in the other kernels (scores = q.k * head_dim^-0.5, float32 softmax with running
// max and sum; reference: csrc/paged_attention_cuda.cu:50-105 and the causal mask of
// src/mini_llm_runtime/qwen_model_runner.py:157-177).  Keys outside [lowest, last position of the
// item] score -inf whatever was loaded, and their V rows are overwritten with zeros before use.
// Every mbarrier wait is bounded; a wait that runs out reports through the error word and the CTA
// goes on without waiting (its result is invalid, the host raises).
#include "tma.cuh"

namespace mlr {

constexpr int FA_ROWS = 128;        // query rows per item = MMA M
constexpr int FA_KEYS = 64;         // keys per tile = MMA N of S, K of P V
constexpr int FA_D = 64;            // head_dim
constexpr int FA_STAGES = 3;
constexpr int FA_SOFTMAX_THREADS = 128;
constexpr int FA_THREADS = FA_SOFTMAX_THREADS + 32;
constexpr uint32_t FA_TMEM_COLS = 256;   // S0 | S1 | PV0 | PV1
constexpr int FA_KV_TILE_BYTES = FA_KEYS * FA_D * 2;       // one K or V tile
constexpr int FA_Q_BYTES = FA_ROWS * FA_D * 2;

// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t fa_desc_k_major(uint32_t address) {
  uint64_t desc = 0;
  desc |= (uint64_t)((address & 0x3FFFFu) >> 4);
  desc |= (uint64_t)1 << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// MN-major operand, 128-byte swizzle: each row of 128 bytes holds 64 MN-contiguous elements of one
// k; 8 consecutive k (1024 bytes) form a swizzle atom; atoms along k follow one another (stride
// 1024 bytes); along MN there is one atom only (leading offset unused, 1024 given).
__device__ __forceinline__ uint64_t fa_desc_mn_major(uint32_t address) {
  uint64_t desc = 0;
  desc |= (uint64_t)((address & 0x3FFFFu) >> 4);
  desc |= (uint64_t)(1024 >> 4) << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}
// kind::f16 instruction descriptor: float32 accumulator, bfloat16 A and B, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t fa_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void fa_mma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void fa_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fa_tmem_load16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 2^x with the hardware approximation (subnormal results flush to zero; -inf gives 0).
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Bounded wait that remembers a failure: after the first wait that ran out, later waits return at once.
__device__ __forceinline__ void fa_wait(uint64_t* bar, uint32_t parity, int* error_word, int code, bool& gave_up) {
  if (!gave_up) gave_up = !mbar_wait(bar, parity, error_word, code);
}

__global__ void __launch_bounds__(FA_THREADS, 2)      // two CTAs per SM: at most 204 registers
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map, bf16* __restrict__ out,
                                 const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                                 const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                                 const int* __restrict__ seg_pos0, const int* __restrict__ block_table, const int* __restrict__ seg_slot,
                                 int table_width, int num_tiles, int heads, int kv_heads, int page_size,
                                 int page_shift, int window, float scale_log2, int* queue, int* error_word,
                                 int max_parts, int tiles_per_unit, float* __restrict__ scratch,
                                 int* __restrict__ counters) {
  extern __shared__ uint8_t fa_shared_raw[];
  uint8_t* aligned = (uint8_t*)(((uintptr_t)fa_shared_raw + 1023) & ~(uintptr_t)1023);
  bf16* q_tile = reinterpret_cast<bf16*>(aligned);                                   // [128][64]
  uint8_t* p_tiles = aligned + FA_Q_BYTES;                                           // 2 x [128][64]
  uint8_t* kv_ring = aligned + 3 * FA_Q_BYTES;                                       // STAGES x (K, V)
  __shared__ uint64_t q_full, kv_full[FA_STAGES], kv_empty[FA_STAGES], s_ready[2], s_free[2], p_ready, pv_ready;
  __shared__ uint32_t tmem_holder;
  __shared__ int item_shared, last_shared;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&s_ready[b], 1); mbar_init(&s_free[b], 4); }
    mbar_init(&p_ready, 4);
    mbar_init(&pv_ready, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)), "r"(FA_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fa_fence_before();
  pdl_trigger();
  __syncthreads();
  fa_fence_after();
  const uint32_t tmem_base = tmem_holder;
  pdl_wait();                       // before the first draw from the queue, the first read of q and the first write

  const int total_items = num_tiles * heads;
  const int total_units = total_items * max_parts;     // part p of every item, for p = 0, 1, ..: many are empty
  const int boxes = page_size >= FA_KEYS ? 1 : FA_KEYS >> page_shift;
  const int box_rows = page_size >= FA_KEYS ? FA_KEYS : page_size;
  unsigned tiles_before = 0;        // key tiles of this CTA's earlier items: rings and phases run on across items
  unsigned items_before = 0;
  bool gave_up = false;

  for (;;) {
    if (threadIdx.x == 0) item_shared = atomicAdd(&queue[0], 1);
    __syncthreads();
    const int unit = item_shared;
    if (unit >= total_units) break;
    const int part = unit / total_items, item = unit - part * total_items;
    const int tile = item / heads, head = item - tile * heads;
    const int kv_head = head / (heads / kv_heads);
    const int seg = tile_seg[tile], row0 = tile_row0[tile];
    const int q_start = seg_q_start[seg], q_len = seg_q_len[seg], pos0 = seg_pos0[seg];
    const int rows = min(FA_ROWS, q_len - row0);
    const int* table = block_table + (size_t)(seg_slot != nullptr ? seg_slot[seg] : seg) * table_width;
    const int first_pos = pos0 + row0, last_pos = first_pos + rows - 1;
    const int lowest = window > 0 ? max(0, first_pos - window + 1) : 0;
    // An item with many key tiles is cut into parts of equal length; each part is a unit of its
    // own (its state goes to scratch memory, the part that finishes last merges them in part order).
    const int item_begin = lowest / FA_KEYS, item_tiles = last_pos / FA_KEYS - item_begin + 1;
    const int parts = min(max_parts, (item_tiles + tiles_per_unit - 1) / tiles_per_unit);
    if (part >= parts) {
      __syncthreads();              // item_shared is rewritten by the next draw
      continue;
    }
    const int per_part = (item_tiles + parts - 1) / parts;
    const int tile_begin = item_begin + part * per_part;
    const int tiles = min(per_part, item_tiles - part * per_part);

    if (warp == 4) {
      // ------------------------------------------------------------ loads and MMAs
      auto issue_load = [&](int j) {
        const unsigned load = tiles_before + (unsigned)j;
        const int stage = load % FA_STAGES;
        const unsigned use = load / FA_STAGES;
        if (use > 0) fa_wait(&kv_empty[stage], (use - 1) & 1u, error_word, 0x61, gave_up);
        gave_up = __any_sync(0xffffffffu, gave_up);
        if (gave_up) return;
        if (lane == 0) mbar_expect_tx(&kv_full[stage], 2u * FA_KV_TILE_BYTES);
        __syncwarp();
        if (lane < boxes) {
          const int key0 = (tile_begin + j) * FA_KEYS + lane * box_rows;
          const int logical = key0 >> page_shift;
          int page = logical < table_width ? table[logical] : -1;
          int offset = key0 & (page_size - 1);
          if (page < 0) { page = 0; offset = 0; }
          const int y = (page * kv_heads + kv_head) * page_size + offset;
          uint8_t* k_dst = kv_ring + (size_t)stage * 2 * FA_KV_TILE_BYTES + lane * box_rows * 128;
          tma_load_2d(&k_map, &kv_full[stage], k_dst, 0, y);
          tma_load_2d(&v_map, &kv_full[stage], k_dst + FA_KV_TILE_BYTES, 0, y);
        }
      };
      if (lane == 0) {
        mbar_expect_tx(&q_full, FA_Q_BYTES);
        tma_load_2d(&q_map, &q_full, q_tile, head * FA_D, q_start + row0);
      }
      for (int j = 0; j < FA_STAGES - 1 && j < tiles; ++j) issue_load(j);

      constexpr uint32_t idesc_qk = fa_idesc(FA_ROWS, FA_KEYS, false);
      constexpr uint32_t idesc_pv = fa_idesc(FA_ROWS, FA_D, true);
      const uint32_t q_addr = smem_u32(q_tile), p_addr0 = smem_u32(p_tiles);
      auto issue_qk = [&](int j) {
        const unsigned t = tiles_before + (unsigned)j;
        const int stage = t % FA_STAGES, buffer = t & 1;
        fa_wait(&kv_full[stage], (t / FA_STAGES) & 1u, error_word, 0x62, gave_up);
        if (t >= 2) fa_wait(&s_free[buffer], ((t >> 1) - 1) & 1u, error_word, 0x63, gave_up);
        gave_up = __any_sync(0xffffffffu, gave_up);
        fa_fence_after();
        if (lane == 0 && !gave_up) {
          const uint32_t k_addr = smem_u32(kv_ring + (size_t)stage * 2 * FA_KV_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < FA_D / 16; ++k)
            fa_mma(tmem_base + buffer * FA_KEYS, fa_desc_k_major(q_addr + k * 32), fa_desc_k_major(k_addr + k * 32),
                   idesc_qk, k > 0 ? 1u : 0u);
          fa_commit(&s_ready[buffer]);
        }
        __syncwarp();
      };
      fa_wait(&q_full, items_before & 1u, error_word, 0x64, gave_up);
      issue_qk(0);
      for (int j = 0; j < tiles; ++j) {
        if (j + FA_STAGES - 1 < tiles) issue_load(j + FA_STAGES - 1);
        if (j + 1 < tiles) issue_qk(j + 1);
        const unsigned t = tiles_before + (unsigned)j;
        const int stage = t % FA_STAGES;
        fa_wait(&p_ready, t & 1u, error_word, 0x65, gave_up);
        gave_up = __any_sync(0xffffffffu, gave_up);
        fa_fence_after();
        if (lane == 0 && !gave_up) {
          const uint32_t v_addr = smem_u32(kv_ring + (size_t)stage * 2 * FA_KV_TILE_BYTES + FA_KV_TILE_BYTES);
#pragma unroll
          const uint32_t p_addr = p_addr0 + (t & 1u) * FA_Q_BYTES;
          for (int k = 0; k < FA_KEYS / 16; ++k)
            fa_mma(tmem_base + (2 + (t & 1u)) * FA_KEYS, fa_desc_k_major(p_addr + k * 32),
                   fa_desc_mn_major(v_addr + k * 2048), idesc_pv, k > 0 ? 1u : 0u);
          fa_commit(&pv_ready);
          fa_commit(&kv_empty[stage]);
        }
        __syncwarp();
      }
    } else {
      // ------------------------------------------------------------ softmax, one thread per query row
      const int r = threadIdx.x;                                    // row of the item = tensor-memory lane
      const int position = first_pos + r;
      const int limit_hi = r < rows ? position : -1;                // rows past the portion see nothing
      const int limit_lo = window > 0 ? max(0, position - window + 1) : 0;
      const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
      // every row of this warp sees all of a key tile that ends at or before the warp's first
      // position and begins at or after the window start of the warp's last row
      const bool warp_full = warp * 32 + 31 < rows;
      const int warp_first = first_pos + warp * 32;
      const int warp_lo = window > 0 ? max(0, first_pos + min(rows - 1, warp * 32 + 31) - window + 1) : 0;
      float m = -INFINITY, l = 0.f;
      float o[FA_D];
#pragma unroll
      for (int d = 0; d < FA_D; ++d) o[d] = 0.f;

      for (int j = 0; j < tiles; ++j) {
        const unsigned t = tiles_before + (unsigned)j;
        const int buffer = t & 1, stage = t % FA_STAGES;
        const int key0 = (tile_begin + j) * FA_KEYS;
        fa_wait(&s_ready[buffer], (t >> 1) & 1u, error_word, 0x66, gave_up);
        fa_fence_after();
        float s[FA_KEYS];
#pragma unroll
        for (int c = 0; c < FA_KEYS; c += 16) fa_tmem_load16(lane_base + buffer * FA_KEYS + c, reinterpret_cast<uint32_t*>(s) + c);
        fa_tmem_wait_ld();
        fa_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[buffer]);

        // scores stay unscaled until the exponent: p = 2^(s * scale - max), one multiply-add each
        // (four interleaved chains for the max and the sum: a single chain of 64 dependent
        // operations would cost more than all the exponentials)
        if (!(warp_full && key0 + FA_KEYS - 1 <= warp_first && key0 >= warp_lo)) {
#pragma unroll
          for (int c = 0; c < FA_KEYS; ++c) {
            const int key = key0 + c;
            if (!(key >= limit_lo && key <= limit_hi)) s[c] = -INFINITY;
          }
        }
        float part_max[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < FA_KEYS; c += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) part_max[e] = fmaxf(part_max[e], s[c + e]);
        }
        const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
        const float m_new = fmaxf(m, tile_max * scale_log2);       // the scale is positive
        const float base = m_new == -INFINITY ? 0.f : m_new;       // nothing visible yet: keep everything at zero
        const float alpha = fa_exp2(m - base);                     // m = -inf gives 0
        m = m_new;
        float part_sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < FA_KEYS; c += 4) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float x = fmaf(s[c + e], scale_log2, -base);
            s[c + e] = fa_exp2(x);
            part_sum[e] += s[c + e];
          }
        }
        l = l * alpha + ((part_sum[0] + part_sum[1]) + (part_sum[2] + part_sum[3]));
        if (alpha != 1.f) {
#pragma unroll
          for (int d = 0; d < FA_D; ++d) o[d] *= alpha;
        }
        if (j > 0) {
          // the previous tile's P V, which ran while this tile's exponentials were taken; it is
          // relative to the previous max, so it takes this tile's factor too
          fa_wait(&pv_ready, (t - 1) & 1u, error_word, 0x67, gave_up);
          fa_fence_after();
#pragma unroll
          for (int c = 0; c < FA_D; c += 32) {         // two loads in flight per wait
            float pv[32];
            fa_tmem_load16(lane_base + (2 + ((t - 1) & 1u)) * FA_KEYS + c, reinterpret_cast<uint32_t*>(pv));
            fa_tmem_load16(lane_base + (2 + ((t - 1) & 1u)) * FA_KEYS + c + 16, reinterpret_cast<uint32_t*>(pv) + 16);
            fa_tmem_wait_ld();
#pragma unroll
            for (int d = 0; d < 32; ++d) o[c + d] = fmaf(pv[d], alpha, o[c + d]);
          }
        }

        if (key0 < lowest || key0 + FA_KEYS - 1 > last_pos) {
          // ragged tile: V rows of keys outside the range become zeros (this thread takes its share of rows)
          fa_wait(&kv_full[stage], (t / FA_STAGES) & 1u, error_word, 0x68, gave_up);
          uint8_t* v_tile = kv_ring + (size_t)stage * 2 * FA_KV_TILE_BYTES + FA_KV_TILE_BYTES;
          for (int idx = threadIdx.x; idx < FA_KEYS * 8; idx += FA_SOFTMAX_THREADS) {
            const int row = idx >> 3;
            if (key0 + row < lowest || key0 + row > last_pos)
              *reinterpret_cast<uint4*>(v_tile + row * 128 + (idx & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        // probabilities of this tile, bfloat16, row r of the swizzled A operand
        {
          uint8_t* p_row = p_tiles + (t & 1u) * FA_Q_BYTES + r * 128;
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk) {
            uint32_t packed[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(s[chunk * 8 + 2 * e], s[chunk * 8 + 2 * e + 1]);
              packed[e] = *reinterpret_cast<uint32_t*>(&pair);
            }
            *reinterpret_cast<uint4*>(p_row + ((chunk ^ (r & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P and the zeroed V rows, for the MMA
        fa_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready);
      }
      // the last tile's P V
      {
        const unsigned t = tiles_before + (unsigned)tiles - 1;
        fa_wait(&pv_ready, t & 1u, error_word, 0x69, gave_up);
        fa_fence_after();
        float pv[FA_D];
#pragma unroll
        for (int c = 0; c < FA_D; c += 16) fa_tmem_load16(lane_base + (2 + (t & 1u)) * FA_KEYS + c, reinterpret_cast<uint32_t*>(pv) + c);
        fa_tmem_wait_ld();
        fa_fence_before();
        if (parts == 1) {
          if (r < rows) {
            const float inv = 1.f / l;
            bf16* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * FA_D;
#pragma unroll
            for (int chunk = 0; chunk < 8; ++chunk) {
              uint32_t packed[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 pair = __floats2bfloat162_rn((o[chunk * 8 + 2 * e] + pv[chunk * 8 + 2 * e]) * inv,
                                                            (o[chunk * 8 + 2 * e + 1] + pv[chunk * 8 + 2 * e + 1]) * inv);
                packed[e] = *reinterpret_cast<uint32_t*>(&pair);
              }
              *reinterpret_cast<uint4*>(dst + chunk * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            }
          }
        } else {
          // this part's state of row r: running max, sum, unnormalised output; laid out
          // [value][row] so that the 128 threads write and read neighbouring addresses
          constexpr int STATE = FA_D + 2;
          float* states = scratch + (size_t)item * max_parts * STATE * FA_ROWS + r;
          float* mine = states + (size_t)part * STATE * FA_ROWS;
          mine[0] = m;
          mine[FA_ROWS] = l;
#pragma unroll
          for (int d = 0; d < FA_D; ++d) mine[(2 + d) * FA_ROWS] = o[d] + pv[d];
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 0) last_shared = (atomicAdd(&counters[item], 1) == parts - 1);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (last_shared) {
            __threadfence();
            float m_all = -INFINITY;
            for (int q = 0; q < parts; ++q) m_all = fmaxf(m_all, __ldcg(states + (size_t)q * STATE * FA_ROWS));
            if (r < rows && m_all != -INFINITY) {
              float l_all = 0.f;
#pragma unroll
              for (int d = 0; d < FA_D; ++d) o[d] = 0.f;
              for (int q = 0; q < parts; ++q) {              // in part order
                const float* theirs = states + (size_t)q * STATE * FA_ROWS;
                const float factor = fa_exp2(__ldcg(theirs) - m_all);      // a part that saw nothing: 0
                l_all = fmaf(__ldcg(theirs + FA_ROWS), factor, l_all);
#pragma unroll
                for (int d = 0; d < FA_D; ++d) o[d] = fmaf(__ldcg(theirs + (2 + d) * FA_ROWS), factor, o[d]);
              }
              const float inv = 1.f / l_all;
              bf16* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * FA_D;
#pragma unroll
              for (int chunk = 0; chunk < 8; ++chunk) {
                uint32_t packed[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  __nv_bfloat162 pair = __floats2bfloat162_rn(o[chunk * 8 + 2 * e] * inv, o[chunk * 8 + 2 * e + 1] * inv);
                  packed[e] = *reinterpret_cast<uint32_t*>(&pair);
                }
                *reinterpret_cast<uint4*>(dst + chunk * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              }
            }
            if (threadIdx.x == 0) counters[item] = 0;       // ready for the next launch
          }
        }
      }
    }
    tiles_before += (unsigned)tiles;
    items_before += 1;
    __syncthreads();                // Q, P and item_shared are rewritten by the next item
  }

  fa_fence_before();
  __syncthreads();
  if (warp == 4) {
    fa_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FA_TMEM_COLS) : "memory");
  }
  // the CTA that leaves last puts the queue back for the next launch
  if (threadIdx.x == 0) {
    const int left = atomicAdd(&queue[1], 1);
    if (left == (int)gridDim.x - 1) { queue[0] = 0; queue[1] = 0; }
  }
}

static int fa_shift_of(int page_size) {
  for (int shift = 0; shift < 31; ++shift)
    if ((1 << shift) == page_size) return shift;
  return -1;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// Units of work aimed at per resident CTA when items are cut into parts.
static const int units_per_cta = 2;

// Prompt portions, head_dim 64, page_size a power of two >= 8.  q, out: [q_rows, heads * 64]
// bfloat16; pools [pool_pages, kv_heads, page_size, 64]; tile_seg / tile_row0: tiles of up to 128 rows
// of one segment, best ordered by falling key count; queue: two zeroed ints in device memory
// (left zeroed); error_word: host-visible int that receives a code if a wait runs out; max_kv_len:
// the longest key range of the step; scratch (scratch_bytes) and counters (counters_len zeroed ints,
// left zeroed): room for the states of items that are cut into parts, may be null.
MLR_EXPORT int mlr_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, void* out,
                                             const int* tile_seg, const int* tile_row0, const int* seg_q_start,
                                             const int* seg_q_len, const int* seg_pos0, const int* block_table, const int* seg_slot,
                                             int table_width, int tiles, int q_rows, int heads, int kv_heads,
                                             int head_dim, int page_size, int pool_pages, int window, float scale,
                                             int max_kv_len, int* queue, int* error_word, void* scratch,
                                             long long scratch_bytes, int* counters, int counters_len,
                                             cudaStream_t stream) {
  if (tiles == 0) return MLR_OK;
  if (tiles < 0 || q_rows <= 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || page_size <= 0 ||
      table_width <= 0 || pool_pages <= 0 || queue == nullptr || error_word == nullptr)
    return MLR_BAD_SIZE;
  if (head_dim != FA_D) return MLR_BAD_SIZE;
  if ((long long)tiles * heads >= (1ll << 30)) return MLR_TOO_LARGE;
  const int page_shift = fa_shift_of(page_size);
  if (page_shift < 3) return MLR_BAD_SIZE;
  if (((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)q & 15)) return MLR_BAD_ALIGNMENT;
  const long long pool_rows = (long long)pool_pages * kv_heads * page_size;
  if (pool_rows >= (1ll << 31)) return MLR_TOO_LARGE;
  const int box_rows = page_size >= FA_KEYS ? FA_KEYS : page_size;
  CUtensorMap q_map, k_map, v_map;
  if (!cached_tile_map(&q_map, q, q_rows, (long long)heads * FA_D, FA_ROWS) ||
      !cached_tile_map(&k_map, k_pool, pool_rows, FA_D, box_rows) ||
      !cached_tile_map(&v_map, v_pool, pool_rows, FA_D, box_rows))
    return MLR_BAD_SIZE;
  const size_t shared = 1024 + 3 * (size_t)FA_Q_BYTES + (size_t)FA_STAGES * 2 * FA_KV_TILE_BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(prefill_attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const long long items = (long long)tiles * heads;
  // Few items with long key ranges (one prompt of a few thousand tokens) would leave the launch as
  // long as its heaviest item: cut items into up to 8 parts so that about two units per resident CTA
  // exist.  Needs scratch for the parts' states and one counter per item; without them, no cutting.
  const int resident = sm_count() * 2;
  const int max_key_tiles = max_kv_len > 0 ? max_kv_len / FA_KEYS + 1 : 1;
  int parts_target = (int)((units_per_cta * resident + items - 1) / items);
  parts_target = parts_target < 1 ? 1 : (parts_target > 8 ? 8 : parts_target);
  int tiles_per_unit = (max_key_tiles + parts_target - 1) / parts_target;
  if (tiles_per_unit < 4) tiles_per_unit = 4;
  int max_parts = (max_key_tiles + tiles_per_unit - 1) / tiles_per_unit;
  if (max_parts > 8) max_parts = 8;
  const long long need = items * max_parts * FA_ROWS * (FA_D + 2) * (long long)sizeof(float);
  if (max_parts > 1 && (scratch == nullptr || counters == nullptr || need > scratch_bytes || items > counters_len)) {
    max_parts = 1;
    tiles_per_unit = 1 << 30;
  }
  const long long units = items * max_parts;
  const int ctas = (int)(units < resident ? units : resident);
  launch_kernel(prefill_attention_tcgen05_kernel, dim3(ctas), dim3(FA_THREADS), shared, stream, q_map, k_map, v_map,
                (bf16*)out, tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, table_width, tiles, heads,
                kv_heads, page_size, page_shift, window, scale * 1.4426950408889634f, queue, error_word, max_parts,
                tiles_per_unit, (float*)scratch, counters);
  return launch_status();
}
