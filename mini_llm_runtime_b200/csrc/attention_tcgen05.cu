// Causal attention of prompt portions over the paged bfloat16 K/V cache on the 5th-generation
// tensor cores (head_dim 64 or 128): S = Q K^T and O += P V run as tcgen05.mma with their results
// in tensor memory; the online softmax runs on the CUDA cores, one thread per query row.
//
// One work item is 128 query rows of one head.  A CTA has six warps:
//   warps 0..3  softmax: thread r owns query row r (tensor-memory lane r).  Per 64-key tile it reads
//               its row of S from tensor memory (64 values), masks (causal limit, window, rows past
//               the portion), keeps the running max and sum, and writes the probabilities as
//               bfloat16 into a 128-byte-swizzled tile in shared memory (the A operand of P V).
//               The output row stays in tensor memory, where the MMAs of all key tiles accumulate
//               into it.  It is relative to a base exponent that follows the running max lazily:
//               only when the max has moved by more than 2^8 since the base was set does the warp
//               read its output rows, scale them and write them back (sum, probabilities and
//               output always use the same base, so the result is exact either way).  On most
//               tiles the softmax threads therefore never touch the output.  The arithmetic uses
//               the paired float32 instructions (two multiply-adds or adds per issue slot) and the
//               three-input max, because the instruction stream, not a pipe, bounds this loop.
//               No shuffles: a row lives in one thread.
//   warp 4      issues the MMAs (one lane).  The scores run two key tiles ahead of the softmax (two
//               S buffers): per tile the warp waits for the tile's probabilities, issues O += P_j V_j
//               at once (the next tile's softmax needs it done midway), then S_{j+2} = Q K_{j+2}^T.
//               K is the K-major B operand; V ([keys][head_dim], head_dim contiguous) is the
//               MN-major B operand.  One commit per product: the same barrier tells the softmax
//               that the product exists and the load warp that the product's stage is free.
//   warp 5      loads: Q by bulk tensor copies per item, K and V page by page (one copy per page, kv
//               head and 64-wide half of the head, as in the other attention kernels) into a K ring
//               and a V ring of their own: a K stage is free once the scores that read it exist, a V
//               stage once its P V product is done, so K runs further ahead than V could.  The
//               block-table read that a copy needs is made a key tile before the copy.  (Table reads,
//               waits and the issue of up to 16 copies per key tile took the MMA warp longer than
//               the softmax takes, when one warp did both: 2,600 to 3,600 cycles per key tile, of
//               which the softmax waited 1,000 to 1,900 for its scores; now 2,200 to 2,300.)
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
constexpr int FA_SOFTMAX_THREADS = 128;
constexpr int FA_THREADS = FA_SOFTMAX_THREADS + 64;      // + the warp that issues MMAs and the warp that loads
constexpr uint32_t FA_TMEM_COLS = 256;   // S0 | S1 | O (head_dim columns)
constexpr uint32_t FA_TMEM_O = 2 * FA_KEYS;
constexpr int FA_P_BYTES = FA_ROWS * FA_KEYS * 2;          // one tile of probabilities
constexpr float FA_LAZY = 8.f;      // the base exponent follows the running max in steps of more than this

// Sizes that depend on the head size.  With 128 the shared memory of two resident CTAs only fits
// with a two-stage ring and one buffer of probabilities.
template <int D>
struct FaShape {
  static constexpr int HALVES = D / 64;                      // 64-wide (128-byte) column blocks of a row
  static constexpr int STAGES = D == 64 ? 4 : 2;
  static constexpr int P_BUFFERS = 1;
  static constexpr int Q_BYTES = FA_ROWS * D * 2;
  static constexpr int Q_HALF_BYTES = FA_ROWS * 128;
  static constexpr int KV_TILE_BYTES = FA_KEYS * D * 2;      // one K or V tile
  static constexpr int KV_HALF_BYTES = FA_KEYS * 128;
  static constexpr int DATA_BYTES = Q_BYTES + P_BUFFERS * FA_P_BYTES + STAGES * 2 * KV_TILE_BYTES;
};

// Barriers and the few words the warps share; behind the tiles in dynamic shared memory.
struct FaControl {
  // qk_done[stage]: the scores that read this K stage exist (the softmax waits for it, and the load
  // warp before it refills the stage); pv_done[stage]: likewise the P V product and the V stage
  uint64_t q_full, k_full[4], v_full[4], qk_done[4], pv_done[4], p_ready;
  uint32_t tmem_holder;
  int item, last;
};
constexpr int FA_CONTROL_BYTES = 256;
static_assert(sizeof(FaControl) <= FA_CONTROL_BYTES, "control block");

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
// offset 1024 bytes); the next 64 elements along MN lie `mn_stride` bytes on (leading offset).
__device__ __forceinline__ uint64_t fa_desc_mn_major(uint32_t address, uint32_t mn_stride) {
  uint64_t desc = 0;
  desc |= (uint64_t)((address & 0x3FFFFu) >> 4);
  desc |= (uint64_t)(mn_stride >> 4) << 16;
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
__device__ __forceinline__ void fa_tmem_store16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void fa_tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fa_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 2^x with the hardware approximation (subnormal results flush to zero; -inf gives 0).
__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fa_max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

// Bounded wait that remembers a failure: after the first wait that ran out, later waits return at once.
__device__ __forceinline__ void fa_wait(uint64_t* bar, uint32_t parity, int* error_word, int code, bool& gave_up) {
  if (!gave_up) gave_up = !mbar_wait(bar, parity, error_word, code);
}

// 32 values of one output row, scaled, as bfloat16 to global memory.
__device__ __forceinline__ void fa_store32(bf16* dst, const float* v, float factor) {
#pragma unroll
  for (int chunk = 0; chunk < 4; ++chunk) {
    uint32_t packed[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat162 pair = __floats2bfloat162_rn(v[chunk * 8 + 2 * e] * factor, v[chunk * 8 + 2 * e + 1] * factor);
      packed[e] = *reinterpret_cast<uint32_t*>(&pair);
    }
    *reinterpret_cast<uint4*>(dst + chunk * 8) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 2)      // two CTAs per SM: at most 204 registers
prefill_attention_tcgen05_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                                 const __grid_constant__ CUtensorMap v_map, bf16* __restrict__ out,
                                 const int* __restrict__ tile_seg, const int* __restrict__ tile_row0,
                                 const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                                 const int* __restrict__ seg_pos0, const int* __restrict__ block_table, const int* __restrict__ seg_slot,
                                 int table_width, int num_tiles, int heads, int kv_heads, int page_size,
                                 int page_shift, int window, float scale_log2, int* queue, int* error_word,
                                 int max_parts, int tiles_per_unit, float* __restrict__ scratch,
                                 int* __restrict__ counters, int shared_bytes) {
  using Shape = FaShape<D>;
  constexpr int STAGES = Shape::STAGES;
  extern __shared__ uint8_t fa_shared_raw[];
  uint8_t* aligned = (uint8_t*)(((uintptr_t)fa_shared_raw + 1023) & ~(uintptr_t)1023);
  if (aligned + Shape::DATA_BYTES + FA_CONTROL_BYTES > fa_shared_raw + shared_bytes) {
    // the launch gave no room for the 1024-byte alignment the swizzled tiles need
    if (threadIdx.x == 0) atomicCAS(error_word, 0, 0x6f);
    return;
  }
  uint8_t* q_tile = aligned;                                                         // [halves][128][64]
  uint8_t* p_tiles = aligned + Shape::Q_BYTES;                                       // P_BUFFERS x [128][64]
  uint8_t* kv_ring = p_tiles + Shape::P_BUFFERS * FA_P_BYTES;                        // STAGES x (K, V), each [halves][64][64]
  FaControl& ctl = *reinterpret_cast<FaControl*>(kv_ring + STAGES * 2 * Shape::KV_TILE_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&ctl.q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl.k_full[s], 1); mbar_init(&ctl.qk_done[s], 1);
      mbar_init(&ctl.v_full[s], 1); mbar_init(&ctl.pv_done[s], 1);
    }
    mbar_init(&ctl.p_ready, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&k_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&v_map) : "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl.tmem_holder)), "r"(FA_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fa_fence_before();
  pdl_trigger();
  __syncthreads();
  fa_fence_after();
  const uint32_t tmem_base = ctl.tmem_holder;
  pdl_wait();                       // before the first draw from the queue, the first read of q and the first write

  const int total_items = num_tiles * heads;
  const int total_units = total_items * max_parts;     // part p of every item, for p = 0, 1, ..: many are empty
  const int boxes = page_size >= FA_KEYS ? 1 : FA_KEYS >> page_shift;
  const int box_rows = page_size >= FA_KEYS ? FA_KEYS : page_size;
  unsigned tiles_before = 0;        // key tiles of this CTA's earlier items: rings and phases run on across items
  unsigned items_before = 0;
  bool gave_up = false;

  for (;;) {
    if (threadIdx.x == 0) ctl.item = atomicAdd(&queue[0], 1);
    __syncthreads();
    const int unit = ctl.item;
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
      __syncthreads();              // ctl.item is rewritten by the next draw
      continue;
    }
    const int per_part = (item_tiles + parts - 1) / parts;
    const int tile_begin = item_begin + part * per_part;
    const int tiles = min(per_part, item_tiles - part * per_part);

    if (warp == 5) {
      // ------------------------------------------------------------ loads
      // K and V tiles have rings of their own.  A K stage is free again once the scores that read it
      // exist, a V stage once the P V product that read it is done; so with S stages the K tile
      // j + S + 1 is on its way while tile j is in the softmax.  The block-table read that a copy
      // needs is made at least a key tile before the copy.  (This warp does nothing else: table
      // reads, waits and the issue of up to 16 bulk copies per key tile took the MMA warp longer
      // than the softmax takes, when it did both.)
      auto lookup = [&](int j) -> int {                     // the page, or -1
        if (j >= tiles || lane >= boxes * Shape::HALVES) return -1;
        const int logical = ((tile_begin + j) * FA_KEYS + (lane % boxes) * box_rows) >> page_shift;
        return logical < table_width ? table[logical] : -1;
      };
      auto load_tile = [&](int j, int page, bool values) {
        const unsigned load = tiles_before + (unsigned)j;
        const int stage = load % STAGES;
        const unsigned use = load / STAGES;
        uint64_t* full = values ? &ctl.v_full[stage] : &ctl.k_full[stage];
        if (use > 0) fa_wait(values ? &ctl.pv_done[stage] : &ctl.qk_done[stage], (use - 1) & 1u, error_word, 0x61, gave_up);
        gave_up = __any_sync(0xffffffffu, gave_up);
        if (gave_up) return;
        if (lane == 0) mbar_expect_tx(full, (uint32_t)Shape::KV_TILE_BYTES);
        __syncwarp();
        if (lane < boxes * Shape::HALVES) {
          const int box = lane % boxes, half = lane / boxes;
          int offset = ((tile_begin + j) * FA_KEYS + box * box_rows) & (page_size - 1);
          if (page < 0) { page = 0; offset = 0; }
          const int y = (page * kv_heads + kv_head) * page_size + offset;
          uint8_t* dst = kv_ring + (size_t)stage * 2 * Shape::KV_TILE_BYTES + (values ? Shape::KV_TILE_BYTES : 0)
                         + half * Shape::KV_HALF_BYTES + box * box_rows * 128;
          tma_load_2d(values ? &v_map : &k_map, full, dst, half * 64, y);
        }
      };
      if (lane == 0) {
        mbar_expect_tx(&ctl.q_full, Shape::Q_BYTES);
#pragma unroll
        for (int half = 0; half < Shape::HALVES; ++half)
          tma_load_2d(&q_map, &ctl.q_full, q_tile + half * Shape::Q_HALF_BYTES, head * D + half * 64, q_start + row0);
      }
      // pages[i]: of tile j + STAGES - 1 + i in iteration j (i = 0: its V is asked for then, i = 2: its K)
      int pages[3];
      {
        int first_pages[STAGES];            // the first ring-full: all table reads, then all copies
#pragma unroll
        for (int j = 0; j < STAGES; ++j) first_pages[j] = lookup(j);
        pages[0] = first_pages[STAGES - 1];
        pages[1] = lookup(STAGES);
        pages[2] = lookup(STAGES + 1);
#pragma unroll
        for (int j = 0; j < STAGES; ++j)
          if (j < tiles) { load_tile(j, first_pages[j], false); load_tile(j, first_pages[j], true); }
      }
      if (STAGES < tiles) load_tile(STAGES, pages[1], false);       // where tile 0's K was
      for (int j = 0; j < tiles; ++j) {
        const int page_after = lookup(j + STAGES + 2);         // in flight during this iteration
        // in the order in which the MMA warp frees the stages: V of tile j + STAGES - 1 goes where tile
        // j - 1's was, K of tile j + STAGES + 1 where tile j + 1's was
        if (j >= 1 && j + STAGES - 1 < tiles) load_tile(j + STAGES - 1, pages[0], true);
        if (j + STAGES + 1 < tiles) load_tile(j + STAGES + 1, pages[2], false);
        pages[0] = pages[1];
        pages[1] = pages[2];
        pages[2] = page_after;
      }
    } else if (warp == 4) {
      // ------------------------------------------------------------ MMAs
      constexpr uint32_t idesc_qk = fa_idesc(FA_ROWS, FA_KEYS, false);
      constexpr uint32_t idesc_pv = fa_idesc(FA_ROWS, D, true);
      const uint32_t q_addr = smem_u32(q_tile), p_addr0 = smem_u32(p_tiles);
      // descriptors differ from tile to tile in their address field only (bytes / 16 in the low bits)
      const uint64_t q_desc = fa_desc_k_major(q_addr), kv_desc = fa_desc_k_major(smem_u32(kv_ring));
      const uint64_t v_desc = fa_desc_mn_major(smem_u32(kv_ring) + Shape::KV_TILE_BYTES, Shape::KV_HALF_BYTES);
      const uint64_t p_desc = fa_desc_k_major(p_addr0);
      auto issue_qk = [&](int j) {
        const unsigned t = tiles_before + (unsigned)j;
        const int stage = t % STAGES, buffer = t & 1;
        fa_wait(&ctl.k_full[stage], (t / STAGES) & 1u, error_word, 0x62, gave_up);
        // The score buffer is free: scores go out two tiles ahead, after the probabilities of tile
        // j - 2 arrived, and a softmax warp arrives there only after it has read that tile's scores
        // (the same buffer); a unit's first two tiles follow the previous unit's end.
        gave_up = __any_sync(0xffffffffu, gave_up);
        fa_fence_after();
        if (lane == 0 && !gave_up) {
          const uint64_t k_desc = kv_desc + (uint64_t)((stage * 2 * Shape::KV_TILE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            fa_mma(tmem_base + buffer * FA_KEYS, q_desc + (uint64_t)(((k >> 2) * Shape::Q_HALF_BYTES + (k & 3) * 32) >> 4),
                   k_desc + (uint64_t)(((k >> 2) * Shape::KV_HALF_BYTES + (k & 3) * 32) >> 4), idesc_qk, k > 0 ? 1u : 0u);
          fa_commit(&ctl.qk_done[stage]);
        }
        __syncwarp();
      };
      // The scores run two key tiles ahead of the softmax (both score buffers in use), so that the
      // softmax of a tile does not wait for this warp: per tile it waits for the probabilities,
      // issues P V at once (the softmax of the next tile needs it done midway), then the scores of
      // the tile after next.
      fa_wait(&ctl.q_full, items_before & 1u, error_word, 0x64, gave_up);
      issue_qk(0);
      if (tiles > 1) issue_qk(1);
      for (int j = 0; j < tiles; ++j) {
        const unsigned t = tiles_before + (unsigned)j;
        const int stage = t % STAGES;
        fa_wait(&ctl.p_ready, t & 1u, error_word, 0x65, gave_up);
        fa_wait(&ctl.v_full[stage], (t / STAGES) & 1u, error_word, 0x6a, gave_up);
        gave_up = __any_sync(0xffffffffu, gave_up);
        fa_fence_after();
        if (lane == 0 && !gave_up) {
          const uint64_t v_tile = v_desc + (uint64_t)((stage * 2 * Shape::KV_TILE_BYTES) >> 4);
          const uint64_t p_tile = p_desc + (uint64_t)(((Shape::P_BUFFERS == 2 ? (t & 1u) : 0u) * FA_P_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < FA_KEYS / 16; ++k)       // the output row accumulates over all key tiles of the unit
            fa_mma(tmem_base + FA_TMEM_O, p_tile + (uint64_t)((k * 32) >> 4), v_tile + (uint64_t)((k * 2048) >> 4), idesc_pv,
                   (j > 0 || k > 0) ? 1u : 0u);
          fa_commit(&ctl.pv_done[stage]);
        }
        __syncwarp();
        if (j + 2 < tiles) issue_qk(j + 2);
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
      float m_run = -INFINITY;      // the running max of the scaled scores (base-2 exponent)
      float m_base = -INFINITY;     // the exponent that sum, probabilities and output are relative to
      float l = 0.f;
      const float2 scale2 = make_float2(scale_log2, scale_log2);

      for (int j = 0; j < tiles; ++j) {
        const unsigned t = tiles_before + (unsigned)j;
        const int buffer = t & 1, stage = t % STAGES;
        const int key0 = (tile_begin + j) * FA_KEYS;
        fa_wait(&ctl.qk_done[stage], (t / STAGES) & 1u, error_word, 0x66, gave_up);
        fa_fence_after();
        float s[FA_KEYS];
#pragma unroll
        for (int c = 0; c < FA_KEYS; c += 16) fa_tmem_load16(lane_base + buffer * FA_KEYS + c, reinterpret_cast<uint32_t*>(s) + c);
        fa_tmem_wait_ld();
        fa_fence_before();

        if (!(warp_full && key0 + FA_KEYS - 1 <= warp_first && key0 >= warp_lo)) {
#pragma unroll
          for (int c = 0; c < FA_KEYS; ++c) {
            const int key = key0 + c;
            if (!(key >= limit_lo && key <= limit_hi)) s[c] = -INFINITY;
          }
        }
        // four interleaved chains of three-input max (one chain of dependent operations would cost
        // more than all the exponentials)
        float part_max[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
        for (int c = 4; c < FA_KEYS - 4; c += 8) {
#pragma unroll
          for (int e = 0; e < 4; ++e) part_max[e] = fa_max3(part_max[e], s[c + 2 * e], s[c + 2 * e + 1]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) part_max[e] = fmaxf(part_max[e], s[FA_KEYS - 4 + e]);
        const float tile_max = fmaxf(fmaxf(part_max[0], part_max[1]), fmaxf(part_max[2], part_max[3]));
        m_run = fmaxf(m_run, tile_max * scale_log2);               // the scale is positive
        // The base follows the max only in steps: (-inf) - (-inf) is NaN and compares false (nothing
        // visible yet: no step); the first visible key gives +inf and sets the base.
        const bool step = m_run - m_base > FA_LAZY;
        const float alpha = step ? fa_exp2(m_base - m_run) : 1.f;   // a base of -inf gives 0
        if (step) m_base = m_run;
        const float base = m_base == -INFINITY ? 0.f : m_base;     // nothing visible yet: everything stays zero
        const float2 minus_base = make_float2(-base, -base);
        // scores stay unscaled until the exponent: p = 2^(s * scale - base), two per multiply-add
        float2 part_sum[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
        for (int c = 0; c < FA_KEYS; c += 8) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = __ffma2_rn(make_float2(s[c + 2 * e], s[c + 2 * e + 1]), scale2, minus_base);
            s[c + 2 * e] = fa_exp2(x.x);
            s[c + 2 * e + 1] = fa_exp2(x.y);
            part_sum[e] = __fadd2_rn(part_sum[e], make_float2(s[c + 2 * e], s[c + 2 * e + 1]));
          }
        }
        const float2 sum2 = __fadd2_rn(__fadd2_rn(part_sum[0], part_sum[1]), __fadd2_rn(part_sum[2], part_sum[3]));
        l = fmaf(l, alpha, sum2.x + sum2.y);

        // The output rows in tensor memory hold the sum of the earlier tiles' P V.  They are touched
        // only when a row of this warp moved its base.  The previous tile's P V is waited for on
        // every tile all the same (it was issued a whole tile ago): a warp must not arrive for this
        // tile's probabilities while the barrier still counts the previous tile's arrivals, and
        // with one buffer of probabilities the MMA must have read it.
        const bool rescale = j > 0 && __any_sync(0xffffffffu, step);
        if (j > 0) {
          fa_wait(&ctl.pv_done[(t - 1) % STAGES], ((t - 1) / STAGES) & 1u, error_word, 0x67, gave_up);
          fa_fence_after();
        }
        if (rescale) {
          const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            float o[32];
            fa_tmem_load16(lane_base + FA_TMEM_O + c, reinterpret_cast<uint32_t*>(o));
            fa_tmem_load16(lane_base + FA_TMEM_O + c + 16, reinterpret_cast<uint32_t*>(o) + 16);
            fa_tmem_wait_ld();
#pragma unroll
            for (int d = 0; d < 32; d += 2) {
              const float2 scaled = __fmul2_rn(make_float2(o[d], o[d + 1]), alpha2);
              o[d] = scaled.x;
              o[d + 1] = scaled.y;
            }
            fa_tmem_store16(lane_base + FA_TMEM_O + c, reinterpret_cast<const uint32_t*>(o));
            fa_tmem_store16(lane_base + FA_TMEM_O + c + 16, reinterpret_cast<const uint32_t*>(o) + 16);
          }
          fa_tmem_wait_st();
        }

        if (key0 < lowest || key0 + FA_KEYS - 1 > last_pos) {
          // ragged tile: V rows of keys outside the range become zeros (this thread takes its share of rows)
          fa_wait(&ctl.v_full[stage], (t / STAGES) & 1u, error_word, 0x68, gave_up);
          uint8_t* v_tile = kv_ring + (size_t)stage * 2 * Shape::KV_TILE_BYTES + Shape::KV_TILE_BYTES;
          for (int idx = threadIdx.x; idx < FA_KEYS * 8 * Shape::HALVES; idx += FA_SOFTMAX_THREADS) {
            const int half = idx / (FA_KEYS * 8), within = idx - half * (FA_KEYS * 8);
            const int row = within >> 3;
            if (key0 + row < lowest || key0 + row > last_pos)
              *reinterpret_cast<uint4*>(v_tile + half * Shape::KV_HALF_BYTES + row * 128 + (within & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        // probabilities of this tile, bfloat16, row r of the swizzled A operand
        {
          uint8_t* p_row = p_tiles + (Shape::P_BUFFERS == 2 ? (t & 1u) : 0u) * FA_P_BYTES + r * 128;
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
        if (lane == 0) mbar_arrive(&ctl.p_ready);
      }
      // the finished output rows, after the last tile's P V
      {
        const unsigned t = tiles_before + (unsigned)tiles - 1;
        fa_wait(&ctl.pv_done[t % STAGES], (t / STAGES) & 1u, error_word, 0x69, gave_up);
        fa_fence_after();
        constexpr int STATE = D + 2;
        // a part's state of row r: base exponent, sum, unnormalised output; laid out [value][row]
        // so that the 128 threads write and read neighbouring addresses
        float* states = scratch + (size_t)item * max_parts * STATE * FA_ROWS + r;
        float* mine = states + (size_t)part * STATE * FA_ROWS;
        const float inv = 1.f / l;
        bf16* dst = out + ((size_t)(q_start + row0 + r) * heads + head) * D;
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          float o[32];
          fa_tmem_load16(lane_base + FA_TMEM_O + c, reinterpret_cast<uint32_t*>(o));
          fa_tmem_load16(lane_base + FA_TMEM_O + c + 16, reinterpret_cast<uint32_t*>(o) + 16);
          fa_tmem_wait_ld();
          if (parts == 1) {
            if (r < rows) fa_store32(dst + c, o, inv);
          } else {
#pragma unroll
            for (int d = 0; d < 32; ++d) mine[(2 + c + d) * FA_ROWS] = o[d];
          }
        }
        fa_fence_before();
        if (parts > 1) {
          mine[0] = m_base;
          mine[FA_ROWS] = l;
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 0) ctl.last = (atomicAdd(&counters[item], 1) == parts - 1);
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (ctl.last) {
            __threadfence();
            float m_all = -INFINITY;
            for (int q = 0; q < parts; ++q) m_all = fmaxf(m_all, __ldcg(states + (size_t)q * STATE * FA_ROWS));
            if (r < rows && m_all != -INFINITY) {
              float factor[8];
              float l_all = 0.f;
#pragma unroll
              for (int q = 0; q < 8; ++q) {                 // in part order
                factor[q] = 0.f;
                if (q < parts) {
                  const float* theirs = states + (size_t)q * STATE * FA_ROWS;
                  factor[q] = fa_exp2(__ldcg(theirs) - m_all);           // a part that saw nothing: 0
                  l_all = fmaf(__ldcg(theirs + FA_ROWS), factor[q], l_all);
                }
              }
              const float inv_all = 1.f / l_all;
#pragma unroll
              for (int c = 0; c < D; c += 32) {
                float o[32];
#pragma unroll
                for (int d = 0; d < 32; ++d) o[d] = 0.f;
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  if (q < parts) {
                    const float* theirs = states + (size_t)q * STATE * FA_ROWS + (size_t)(2 + c) * FA_ROWS;
#pragma unroll
                    for (int d = 0; d < 32; ++d) o[d] = fmaf(__ldcg(theirs + d * FA_ROWS), factor[q], o[d]);
                  }
                }
                fa_store32(dst + c, o, inv_all);
              }
            }
            if (threadIdx.x == 0) counters[item] = 0;       // ready for the next launch
          }
        }
      }
    }
    tiles_before += (unsigned)tiles;
    items_before += 1;
    __syncthreads();                // Q, P and ctl.item are rewritten by the next item
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

// Units of work aimed at per resident CTA when items are cut into parts.  One: a 2,048-row prompt
// takes 38 us at 14 heads of 64 and 52 us at 28 heads of 128 against 43 and 67 us with two (more,
// shorter units mean more starts, ends and merges).
static const int units_per_cta = 1;

namespace mlr {

template <int D>
static int fa_launch(const void* q, const void* k_pool, const void* v_pool, void* out, const int* tile_seg,
                     const int* tile_row0, const int* seg_q_start, const int* seg_q_len, const int* seg_pos0,
                     const int* block_table, const int* seg_slot, int table_width, int tiles, int q_rows, int heads,
                     int kv_heads, int page_size, int page_shift, long long pool_rows, int window, float scale,
                     int max_kv_len, int* queue, int* error_word, void* scratch, long long scratch_bytes,
                     int* counters, int counters_len, cudaStream_t stream) {
  using Shape = FaShape<D>;
  const int box_rows = page_size >= FA_KEYS ? FA_KEYS : page_size;
  CUtensorMap q_map, k_map, v_map;
  if (!cached_tile_map(&q_map, q, q_rows, (long long)heads * D, FA_ROWS) ||
      !cached_tile_map(&k_map, k_pool, pool_rows, D, box_rows) ||
      !cached_tile_map(&v_map, v_pool, pool_rows, D, box_rows))
    return MLR_BAD_SIZE;
  // With head_dim 128 two CTAs fit an SM only without the spare kilobyte for aligning the tiles:
  // dynamic shared memory then has to start on a 1024-byte boundary, which it does when the kernel
  // has no static shared memory; the kernel checks and reports through the error word if not.
  const size_t shared = (D == 64 ? 1024 : 0) + (size_t)Shape::DATA_BYTES + FA_CONTROL_BYTES;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(prefill_attention_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
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
  const long long need = items * max_parts * FA_ROWS * (D + 2) * (long long)sizeof(float);
  if (max_parts > 1 && (scratch == nullptr || counters == nullptr || need > scratch_bytes || items > counters_len)) {
    max_parts = 1;
    tiles_per_unit = 1 << 30;
  }
  const long long units = items * max_parts;
  const int ctas = (int)(units < resident ? units : resident);
  launch_kernel(prefill_attention_tcgen05_kernel<D>, dim3(ctas), dim3(FA_THREADS), shared, stream, q_map, k_map, v_map,
                (bf16*)out, tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table, seg_slot, table_width, tiles, heads,
                kv_heads, page_size, page_shift, window, scale * 1.4426950408889634f, queue, error_word, max_parts,
                tiles_per_unit, (float*)scratch, counters, (int)shared);
  return launch_status();
}

}  // namespace mlr

// Prompt portions, head_dim 64 or 128, page_size a power of two >= 8.  q, out: [q_rows, heads *
// head_dim] bfloat16; pools [pool_pages, kv_heads, page_size, head_dim]; tile_seg / tile_row0: tiles
// of up to 128 rows of one segment, best ordered by falling key count; queue: two zeroed ints in
// device memory (left zeroed); error_word: host-visible int that receives a code if a wait runs out;
// max_kv_len: the longest key range of the step; scratch (scratch_bytes) and counters (counters_len
// zeroed ints, left zeroed): room for the states of items that are cut into parts, may be null.
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
  if (head_dim != 64 && head_dim != 128) return MLR_BAD_SIZE;
  if ((long long)tiles * heads >= (1ll << 30)) return MLR_TOO_LARGE;
  const int page_shift = fa_shift_of(page_size);
  if (page_shift < 3) return MLR_BAD_SIZE;
  if (((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15) || ((uintptr_t)q & 15)) return MLR_BAD_ALIGNMENT;
  const long long pool_rows = (long long)pool_pages * kv_heads * page_size;
  if (pool_rows >= (1ll << 31)) return MLR_TOO_LARGE;
  if (head_dim == 64)
    return fa_launch<64>(q, k_pool, v_pool, out, tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table,
                         seg_slot, table_width, tiles, q_rows, heads, kv_heads, page_size, page_shift, pool_rows, window,
                         scale, max_kv_len, queue, error_word, scratch, scratch_bytes, counters, counters_len, stream);
  return fa_launch<128>(q, k_pool, v_pool, out, tile_seg, tile_row0, seg_q_start, seg_q_len, seg_pos0, block_table,
                        seg_slot, table_width, tiles, q_rows, heads, kv_heads, page_size, page_shift, pool_rows, window,
                        scale, max_kv_len, queue, error_word, scratch, scratch_bytes, counters, counters_len, stream);
}
