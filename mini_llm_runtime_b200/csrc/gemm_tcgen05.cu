// bfloat16 matrix product on the 5th-generation tensor cores: y[M,N] = x[M,K] * W[N,K]^T (+ bias),
// float32 accumulation in tensor memory, output bfloat16 or float32.
//
// One CTA computes one 128 x BN accumulator tile:
//   warp 0 (one lane)  TMA producer: cp.async.bulk.tensor loads of 128B-swizzled [rows x 64] tiles
//                      of both operands into a ring of shared-memory stages, signalled by mbarriers
//   warp 1             allocates tensor memory; one lane issues tcgen05.mma (M=128, N=BN, K=16) on
//                      shared-memory descriptors and commits each stage back to the producer
//   warps 2..5         epilogue: tcgen05.ld the accumulator (one TMEM lane = one tile row per
//                      thread), add bias, convert, store
// Both operands are K-major, as activations [M,K] and checkpoint weights [N,K] are stored.
// For products of many rows a CTA may also compute two such tiles (256 x 256) side by side in tensor
// memory from one load of the BN-row operand: half the traffic of that operand per MMA.  Or the
// 256 x 256 tile lies over an SM pair (a cluster of two CTAs, tcgen05 cta_group::2): each CTA loads
// its 128 rows and half of the BN-row operand, one thread of the even CTA issues MMAs of 256 rows
// for both, each CTA holds and writes out the accumulator of its rows; with half the shared and
// tensor memory per CTA, two CTAs fit an SM and one's epilogue overlaps the other's MMAs.
//
// Orientation.  With many rows (prefill) x is the 128-row operand and 128 weight rows form the
// N side.  With few rows (decode) the roles swap: 128 weight rows fill the MMA's M side and the
// BN = 16..128 token rows its N side, so that a step streams every weight byte exactly once through
// full-width tiles.  K may be split over gridDim.z CTAs; partial tiles go to a float32 scratch
// buffer and the CTA that arrives last for a tile adds them in split order (deterministic) and
// writes the output.
// No CTA waits for another CTA, the two of a pair excepted: they meet at the hardware cluster barrier
// after their barriers are set up and before tensor memory is freed, and the odd CTA's loads and
// the even CTA's MMAs signal each other's mbarriers.
// Every wait on an mbarrier is bounded; a wait that runs out stores a code into the error word
// (host-visible memory), the CTA stops issuing work, frees its tensor memory and returns.
// TMA loads use no cluster multicast.  Requirements: K % 8 == 0 (16-byte row pitch for TMA) and
// 16-byte aligned base pointers; the caller falls back to the SIMT kernel otherwise.
#include "tma.cuh"

namespace mlr {

constexpr int TILE_ROWS = 128;      // MMA M
constexpr int TILE_K = 64;          // one 128-byte swizzle atom of bfloat16
constexpr int MMA_K = 16;
constexpr int GEMM_THREADS = 192;
// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 128 bytes, groups of
// 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
  uint64_t desc = 0;
  desc |= (uint64_t)((address & 0x3FFFFu) >> 4);
  desc |= (uint64_t)1 << 16;            // leading byte offset (unused with swizzled K-major)
  desc |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  desc |= (uint64_t)1 << 46;            // version
  desc |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return desc;
}

// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 A and B, both K-major.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The same load without the wait, so that several can be in flight; tmem_wait_loads() before the
// registers are read.
__device__ __forceinline__ void tmem_issue_load16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_loads() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- two CTAs on one tile (a cluster of two: an SM pair).  Each CTA holds its own 128 rows of the
// 128-row operand and half of the BN-row operand; one thread of the even CTA issues MMAs of 256
// rows that read both CTAs' shared memory and write both CTAs' tensor memory.  Loads of both CTAs
// count on the even CTA's barrier; a commit arrives on the barriers of both.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t address_in_cta(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
// `barrier`: shared::cluster address of the barrier that counts the bytes (the even CTA's)
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t barrier, void* dst, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(barrier), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the MMAs issued so far have finished, on the barrier at this address in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

struct GemmParams {
  int M, N, K;
  int k_blocks_per_split;   // 64-wide k blocks each split handles
  int splits;
  int stages;               // shared-memory stages in the ring (2..8)
  const bf16* bias;
  void* out;
  int out_f32;
  float* scratch;           // [tiles][splits][BN][128] partial tiles (splits > 1)
  int* counters;            // one per output tile, zero between launches
  int* error_word;
};

constexpr int MAX_STAGES = 8;


// Sum of the splits' partial values of 16 columns of one tile row, in split order.  Loads of four
// splits are issued together so that their latencies overlap; a missing split adds zeros.
template <int BN>
__device__ __forceinline__ void reduce_partials(const float* partials, int splits, int c0, int row, float* v) {
#pragma unroll
  for (int c = 0; c < 16; ++c) v[c] = 0.f;
  for (int s0 = 0; s0 < splits; s0 += 4) {
    float t[4][16];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 16; ++c)
        t[j][c] = s0 + j < splits ? __ldcg(&partials[((size_t)(s0 + j) * BN + c0 + c) * TILE_ROWS + row]) : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 16; ++c) v[c] += t[j][c];
  }
}

// The last CTA's reduction in the swapped orientation (tile row = output column n, tile column =
// token m), for all 128 epilogue threads together: a thread owns four adjacent tile rows (one
// 16-byte load per split and tile column) and every fourth (eighth with SwiGLU) tile column, so the
// whole tile is fetched with a quarter of the loads and written in 8-byte pieces.  Splits are added
// in split order.  `t` = 0..127.
// SHARED: `partials` is one tile in shared memory (the CTA's own accumulator, staged there so that
// the same wide, row-major stores serve the product without split-K).
template <int BN, bool SHARED>
__device__ __forceinline__ void reduce_swapped(const float* partials, int splits, const GemmParams& p, int t,
                                               int a_row0, int b_row0) {
  const int rg = t & 31, cg = t >> 5;
  const int n0 = a_row0 + 4 * rg;
  if (n0 >= p.N) return;
  float bias[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) bias[j] = (p.bias != nullptr && n0 + j < p.N) ? to_float(p.bias[n0 + j]) : 0.f;
  const bool wide = (p.N & 3) == 0;                   // then n0 + 3 < N and the stores are aligned
  constexpr int CB = 4;                                // tile columns in flight per thread
  for (int c = cg; c < BN; c += 4 * CB) {
    float4 acc[CB];
#pragma unroll
    for (int j = 0; j < CB; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float4 part[4][CB];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          const int col = c + 4 * j;
          const float4* at = reinterpret_cast<const float4*>(partials + ((size_t)(s0 + i) * BN + col) * TILE_ROWS + 4 * rg);
          part[i][j] = (s0 + i < splits && col < BN && b_row0 + col < p.M) ? (SHARED ? *at : __ldcg(at))
                                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          acc[j].x += part[i][j].x; acc[j].y += part[i][j].y; acc[j].z += part[i][j].z; acc[j].w += part[i][j].w;
        }
    }
#pragma unroll
    for (int j = 0; j < CB; ++j) {
      const int col = c + 4 * j, m = b_row0 + col;
      if (col >= BN || m >= p.M) continue;
      const float v[4] = {acc[j].x + bias[0], acc[j].y + bias[1], acc[j].z + bias[2], acc[j].w + bias[3]};
      if (p.out_f32) {
        float* dst = (float*)p.out + (size_t)m * p.N + n0;
        if (wide) *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        else for (int e = 0; e < 4; ++e) if (n0 + e < p.N) dst[e] = v[e];
      } else {
        bf16* dst = (bf16*)p.out + (size_t)m * p.N + n0;
        if (wide) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
          *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        } else {
          for (int e = 0; e < 4; ++e) if (n0 + e < p.N) dst[e] = __float2bfloat16_rn(v[e]);
        }
      }
    }
  }
}

// The same with the fused SwiGLU: tile rows 0..63 are gate rows, 64..127 the up rows of the same
// 64 outputs; a thread owns four gate rows, their up rows, and every eighth tile column.
template <int BN, bool SHARED>
__device__ __forceinline__ void reduce_swapped_swiglu(const float* partials, int splits, const GemmParams& p, int t,
                                                      int tile_x, int b_row0) {
  const int rg = t & 15, cg = t >> 4;
  const int half = p.N >> 1;
  const int n0 = tile_x * 64 + 4 * rg;
  if (n0 >= half) return;
  const bool wide = (half & 3) == 0;
  constexpr int CB = 2;
  for (int c = cg; c < BN; c += 8 * CB) {
    float4 gate[CB], up[CB];
#pragma unroll
    for (int j = 0; j < CB; ++j) gate[j] = up[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < splits; s0 += 4) {
      float4 pg[4][CB], pu[4][CB];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          const int col = c + 8 * j;
          const bool live = s0 + i < splits && col < BN && b_row0 + col < p.M;
          const float4* base = reinterpret_cast<const float4*>(partials + ((size_t)(s0 + i) * BN + col) * TILE_ROWS + 4 * rg);
          pg[i][j] = live ? (SHARED ? base[0] : __ldcg(base)) : make_float4(0.f, 0.f, 0.f, 0.f);
          pu[i][j] = live ? (SHARED ? base[16] : __ldcg(base + 16)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < CB; ++j) {
          gate[j].x += pg[i][j].x; gate[j].y += pg[i][j].y; gate[j].z += pg[i][j].z; gate[j].w += pg[i][j].w;
          up[j].x += pu[i][j].x; up[j].y += pu[i][j].y; up[j].z += pu[i][j].z; up[j].w += pu[i][j].w;
        }
    }
#pragma unroll
    for (int j = 0; j < CB; ++j) {
      const int col = c + 8 * j, m = b_row0 + col;
      if (col >= BN || m >= p.M) continue;
      const float v[4] = {silu_times(gate[j].x, up[j].x), silu_times(gate[j].y, up[j].y),
                          silu_times(gate[j].z, up[j].z), silu_times(gate[j].w, up[j].w)};
      bf16* dst = (bf16*)p.out + (size_t)m * half + n0;
      if (wide) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        for (int e = 0; e < 4; ++e) if (n0 + e < half) dst[e] = __float2bfloat16_rn(v[e]);
      }
    }
  }
}

// SWAP = true:  A (128 rows) = weights, B (BN rows) = activations; tile row = output column n.
// SWAP = false: A (128 rows) = activations, B (BN rows) = weights; tile row = output row m.
// SWIGLU: the weight rows come in blocks of 128 = 64 gate rows followed by the 64 up rows of the
// same outputs; the epilogue writes silu(gate) * up, [M, N/2].
// BM = 256 (many rows only): the CTA computes two 128-row accumulators side by side in tensor memory
// from one load of the BN-row operand, which halves that operand's traffic from L2 per MMA (the
// bound of the large products); no split-K in that form.
// PAIR (many rows only): the tile is 256 x BN over two CTAs as described above; the grid's x
// extent counts 128-row halves, consecutive CTAs forming a cluster.
template <int BN, bool SWAP, bool SWIGLU, int BM = TILE_ROWS, bool PAIR = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const GemmParams p) {
  constexpr int HALVES = BM / TILE_ROWS;
  constexpr uint32_t HALF_BYTES = TILE_ROWS * TILE_K * 2;
  constexpr uint32_t A_BYTES = BM * TILE_K * 2;
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;               // rows of the BN-row operand this CTA loads
  constexpr uint32_t B_BYTES = B_ROWS * TILE_K * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BN * HALVES < 32 ? 32 : BN * HALVES;
  static_assert(!SWIGLU || SWAP || BN % 128 == 0, "fused SwiGLU needs gate and up columns in one tile");
  static_assert(BM == TILE_ROWS || (BM == 2 * TILE_ROWS && !SWAP && BN * HALVES <= 512), "two accumulators: many rows, 512 columns");
  static_assert(!PAIR || (BM == TILE_ROWS && !SWAP && BN % 32 == 0), "an SM pair: many rows, one accumulator per CTA");

  extern __shared__ uint8_t raw_shared[];
  uint8_t* tiles = (uint8_t*)(((uintptr_t)raw_shared + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], accumulator_bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int is_last_cta, epilogue_failed;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int a_row0 = blockIdx.x * BM;          // first row of the 128-row (or 256-row) operand
  const int b_row0 = blockIdx.y * BN;          // first row of the BN-row operand
  const uint32_t pair_rank = PAIR ? cluster_cta_rank() : 0u;
  const int split = blockIdx.z;
  const int total_kb = (p.K + TILE_K - 1) / TILE_K;
  const int kb_begin = split * p.k_blocks_per_split;
  const int kb_end = min(total_kb, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;        // >= 1 by construction of the grid

  if (threadIdx.x == 0) {
    epilogue_failed = 0;
    for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&accumulator_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  if (warp == 1) {
    if (PAIR) {      // the same warp of both CTAs: the same columns in both SMs' tensor memory
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_holder)), "r"(TMEM_COLS) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();        // the other CTA's barriers exist before anything is sent to them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_holder;

  pdl_trigger();
  if (warp == 0 && lane == 0) {
    // ---------------- producer
    // The weight tiles of the first ring-full of k blocks do not depend on the kernel before this
    // one: request them at once, then wait for that kernel and request the activation tiles.
    // In a pair both CTAs load (their rows of the one operand, their half of the other) and all bytes
    // count on the even CTA's barrier, which alone expects them.
    auto load_a = [&](int s, int k) {
      uint8_t* stage = tiles + (size_t)s * STAGE_BYTES;
      if (PAIR) {
        tma_load_2d_pair(&map_a, address_in_cta(smem_u32(&full_bar[s]), 0), stage, k, a_row0);
      } else {
#pragma unroll
        for (int half = 0; half < HALVES; ++half)
          tma_load_2d(&map_a, &full_bar[s], stage + half * HALF_BYTES, k, a_row0 + half * TILE_ROWS);
      }
    };
    auto load_b = [&](int s, int k) {
      uint8_t* stage = tiles + (size_t)s * STAGE_BYTES;
      if (PAIR) tma_load_2d_pair(&map_b, address_in_cta(smem_u32(&full_bar[s]), 0), stage + A_BYTES, k, b_row0 + (int)pair_rank * B_ROWS);
      else tma_load_2d(&map_b, &full_bar[s], stage + A_BYTES, k, b_row0);
    };
    auto expect = [&](int s) {
      if (!PAIR) mbar_expect_tx(&full_bar[s], STAGE_BYTES);
      else if (pair_rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
    };
    const int ahead = min(stages, num_kb);
    for (int i = 0; i < ahead; ++i) {
      expect(i);
      const int k = (kb_begin + i) * TILE_K;
      if (SWAP) load_a(i, k); else load_b(i, k);
    }
    pdl_wait();
    for (int i = 0; i < ahead; ++i) {
      const int k = (kb_begin + i) * TILE_K;
      if (SWAP) load_b(i, k); else load_a(i, k);
    }
    int s = ahead == stages ? 0 : ahead, round = ahead == stages ? 1 : 0;
    for (int i = ahead; i < num_kb; ++i) {
      if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, p.error_word, 1)) break;
      expect(s);
      const int k = (kb_begin + i) * TILE_K;
      load_a(s, k);
      load_b(s, k);
      if (++s == stages) { s = 0; ++round; }
    }
  } else if (warp == 1 && lane == 0 && pair_rank == 0) {
    // ---------------- MMA issuer (of a pair: the even CTA's, for both)
    constexpr uint32_t idesc = instruction_descriptor(PAIR ? 2 * TILE_ROWS : TILE_ROWS, BN);
    int s = 0, round = 0;
    for (int i = 0; i < num_kb; ++i) {
      if (!mbar_wait(&full_bar[s], round & 1, p.error_word, 2)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
      const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
      for (int k = 0; k < TILE_K / MMA_K; ++k) {
        if (PAIR) {
          umma_pair(tmem_base, smem_descriptor(a_addr + k * MMA_K * 2), smem_descriptor(b_addr + k * MMA_K * 2), idesc,
                    (i > 0 || k > 0) ? 1u : 0u);
        } else {
#pragma unroll
          for (int half = 0; half < HALVES; ++half)
            umma(tmem_base + half * BN, smem_descriptor(a_addr + half * HALF_BYTES + k * MMA_K * 2),
                 smem_descriptor(b_addr + k * MMA_K * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
      }
      if (PAIR) umma_commit_pair(&empty_bar[s]); else umma_commit(&empty_bar[s]);
      if (++s == stages) { s = 0; ++round; }
    }
    // arrives once every MMA issued above has finished (in a pair: on both CTAs' barriers)
    if (PAIR) umma_commit_pair(&accumulator_bar); else umma_commit(&accumulator_bar);
  } else if (warp >= 2) {
    // ---------------- epilogue: thread <-> TMEM lane <-> tile row
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    pdl_wait();                                         // before any write of this kernel
    if (!mbar_wait(&accumulator_bar, 0, p.error_word, 3)) atomicOr(&epilogue_failed, 1);
    asm volatile("bar.sync 1, 128;" ::: "memory");     // all four epilogue warps always get here
    const bool ok = epilogue_failed == 0;               // the same answer in all of them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (ok && p.splits > 1) {
      float* mine = p.scratch + ((size_t)tile_id * p.splits + split) * BN * TILE_ROWS;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_load16(lane_base + c0, r);
#pragma unroll
        for (int c = 0; c < 16; ++c) mine[(size_t)(c0 + c) * TILE_ROWS + row] = __uint_as_float(r[c]);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (warp == 2 && lane == 0) is_last_cta = (atomicAdd(&p.counters[tile_id], 1) == p.splits - 1);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    const bool reduce = ok && p.splits > 1 && is_last_cta;
    const bool finish = ok && (p.splits == 1 || reduce);
    if (reduce) __threadfence();
    const float* partials = p.scratch + (size_t)tile_id * p.splits * BN * TILE_ROWS;
    bf16* out_bf16 = (bf16*)p.out;
    float* out_f32 = (float*)p.out;

    if (SWAP) {
      // Tile row = output column n, tile column = token m: the tile is written row-major in m by
      // threads that own four adjacent n each, from the splits' partial tiles (split-K) or from the
      // CTA's own accumulator staged in shared memory (the stage ring is idle by now).
      if (reduce) {
        if (SWIGLU) reduce_swapped_swiglu<BN, false>(partials, p.splits, p, row, blockIdx.x, b_row0);
        else reduce_swapped<BN, false>(partials, p.splits, p, row, a_row0, b_row0);
      } else if (finish) {                               // the same answer in all four epilogue warps
        float* exchange = reinterpret_cast<float*>(tiles);            // [BN][128]
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_load16(lane_base + c0, r);
#pragma unroll
          for (int c = 0; c < 16; ++c) exchange[(c0 + c) * TILE_ROWS + row] = __uint_as_float(r[c]);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (SWIGLU) reduce_swapped_swiglu<BN, true>(exchange, 1, p, row, blockIdx.x, b_row0);
        else reduce_swapped<BN, true>(exchange, 1, p, row, a_row0, b_row0);
      }
    } else if (SWIGLU) {
      // not swapped: each group of 128 columns holds 64 gate columns, then the 64 up columns of
      // the same outputs, all in this thread's TMEM lane.
      // tcgen05.ld is warp-collective: every lane runs the loads, only the stores depend on m.
      const int half = p.N >> 1;
      if (finish) {
#pragma unroll 1
        for (int cc = 0; cc < HALVES * (BN / 2); cc += 32) {
          const int accumulator = cc / (BN / 2), within = cc - accumulator * (BN / 2);
          const int block = within >> 6, c0 = within & 63;   // which 128-column group, offset in it
          const int m = a_row0 + accumulator * TILE_ROWS + row;
          const uint32_t from = lane_base + accumulator * BN + block * 128;
          uint32_t g[32], u[32];
          tmem_issue_load16(from + c0, g);
          tmem_issue_load16(from + c0 + 16, g + 16);
          tmem_issue_load16(from + 64 + c0, u);
          tmem_issue_load16(from + 64 + c0 + 16, u + 16);
          tmem_wait_loads();
          if (m >= p.M) continue;
#pragma unroll
          for (int q = 0; q < 32; q += 16) {
            const int n0 = (blockIdx.y * (BN / 128) + block) * 64 + c0 + q;
            uint32_t packed[8];
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
              __nv_bfloat162 pair = __floats2bfloat162_rn(
                  silu_times(__uint_as_float(g[q + c]), __uint_as_float(u[q + c])),
                  silu_times(__uint_as_float(g[q + c + 1]), __uint_as_float(u[q + c + 1])));
              packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
            }
            if ((half & 7) == 0 && n0 + 16 <= half) {
              uint4* dst = reinterpret_cast<uint4*>(out_bf16 + (size_t)m * half + n0);
              dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            } else {
              const bf16* values = reinterpret_cast<const bf16*>(packed);
              for (int c = 0; c < 16; ++c)
                if (n0 + c < half) out_bf16[(size_t)m * half + n0 + c] = values[c];
            }
          }
        }
      }
    } else if (finish) {
      // 64 columns per round: four tensor-memory loads in flight, one wait, then convert and store
      // (a load and its wait per 16 columns made the epilogue as long as a short main loop)
      constexpr int ROUND = BN >= 64 ? 64 : BN;
#pragma unroll 1
      for (int cc = 0; cc < HALVES * BN; cc += ROUND) {
        const int accumulator = cc / BN, c00 = cc - accumulator * BN;
        float v[ROUND];
        if (reduce) {
#pragma unroll
          for (int q = 0; q < ROUND; q += 16) reduce_partials<BN>(partials, p.splits, c00 + q, row, v + q);
        } else {
#pragma unroll
          for (int q = 0; q < ROUND; q += 16)
            tmem_issue_load16(lane_base + accumulator * BN + c00 + q, reinterpret_cast<uint32_t*>(v) + q);
          tmem_wait_loads();
        }
        const int m = a_row0 + accumulator * TILE_ROWS + row;
        if (m >= p.M) continue;
#pragma unroll
        for (int q = 0; q < ROUND; q += 16) {
          const int n0 = b_row0 + c00 + q;
          if (n0 >= p.N) break;
          if (!p.out_f32 && (p.N & 7) == 0 && n0 + 16 <= p.N) {
            uint32_t packed[8];
#pragma unroll
            for (int c = 0; c < 16; c += 2) {
              const float b0 = p.bias != nullptr ? to_float(p.bias[n0 + c]) : 0.f;
              const float b1 = p.bias != nullptr ? to_float(p.bias[n0 + c + 1]) : 0.f;
              __nv_bfloat162 pair = __floats2bfloat162_rn(v[q + c] + b0, v[q + c + 1] + b1);
              packed[c >> 1] = *reinterpret_cast<uint32_t*>(&pair);
            }
            uint4* dst = reinterpret_cast<uint4*>(out_bf16 + (size_t)m * p.N + n0);
            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          } else {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
              const int n = n0 + c;
              if (n < p.N) {
                const float b = p.bias != nullptr ? to_float(p.bias[n]) : 0.f;
                if (p.out_f32) out_f32[(size_t)m * p.N + n] = v[q + c] + b;
                else out_bf16[(size_t)m * p.N + n] = __float2bfloat16_rn(v[q + c] + b);
              }
            }
          }
        }
      }
    }
    if (reduce && warp == 2 && lane == 0) p.counters[tile_id] = 0;   // ready for the next launch
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync_all();        // both CTAs are done with tensor memory and with each other's shared memory
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// ---------------------------------------------------------------- host side
template <int BN, bool SWAP, bool SWIGLU, int BM = TILE_ROWS>
static int launch(const void* x, const void* w, const GemmParams& p, int splits, cudaStream_t stream) {
  const size_t shared = (size_t)p.stages * (BM * TILE_K * 2 + BN * TILE_K * 2) + 1024;
  if (BM != TILE_ROWS && splits != 1) return MLR_BAD_SIZE;
  static size_t configured = 0;
  if (shared > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, SWAP, SWIGLU, BM>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = shared;
  }
  const void* a_base = SWAP ? w : x;
  const void* b_base = SWAP ? x : w;
  const int a_rows = SWAP ? p.N : p.M, b_rows = SWAP ? p.M : p.N;
  CUtensorMap map_a, map_b;
  if (!cached_tile_map(&map_a, a_base, a_rows, p.K, TILE_ROWS) || !cached_tile_map(&map_b, b_base, b_rows, p.K, BN))
    return MLR_BAD_ALIGNMENT;
  dim3 grid((a_rows + BM - 1) / BM, (b_rows + BN - 1) / BN, splits);
  launch_kernel(gemm_tcgen05_kernel<BN, SWAP, SWIGLU, BM>, dim3(grid), dim3(GEMM_THREADS), shared, stream, map_a, map_b, p);
  return launch_status();
}

// A 256 x BN tile over an SM pair: a cluster of two CTAs, 128 rows and BN/2 weight rows each.
template <int BN, bool SWIGLU>
static int launch_pair(const void* x, const void* w, const GemmParams& p, cudaStream_t stream) {
  const size_t shared = (size_t)p.stages * (TILE_ROWS * TILE_K * 2 + BN / 2 * TILE_K * 2) + 1024;
  static size_t configured = 0;
  if (shared > configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, false, SWIGLU, TILE_ROWS, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return (int)err;
    configured = shared;
  }
  CUtensorMap map_a, map_b;
  if (!cached_tile_map(&map_a, x, p.M, p.K, TILE_ROWS) || !cached_tile_map(&map_b, w, p.N, p.K, BN / 2))
    return MLR_BAD_ALIGNMENT;
  dim3 grid(2 * ((p.M + 2 * TILE_ROWS - 1) / (2 * TILE_ROWS)), (p.N + BN - 1) / BN, 1);
  launch_kernel_clustered(gemm_tcgen05_kernel<BN, false, SWIGLU, TILE_ROWS, true>, grid, dim3(GEMM_THREADS), shared, stream, 2,
                          map_a, map_b, p);
  return launch_status();
}

// Tile shape, split count and ring depth for a product of this shape.  pair: the 256 x 256 tile lies
// over two CTAs (one accumulator of 256 columns each) instead of in one CTA with two accumulators.
struct GemmPlan { int bn, tiles, splits, stages, kb_per_split, bm; bool pair; };

// Overrides for measurements (0 = the planner decides): tile width and ring depth of many-row products.
static int forced_bn = 0, forced_stages = 0, forced_splits = 0, forced_bm = 0, forced_pair = 0;

// Many rows (M > 128): tile width, ring depth and split count by a small model of the kernel,
// in microseconds.  A CTA costs a fixed 1.5 us (barriers, tensor-memory allocation, first loads)
// plus its k blocks plus its epilogue (1.5 us per 128 columns).  A k block costs the largest of
//   the MMAs' time: 0.14 us per 128 columns, times the CTAs sharing the SM's tensor pipe;
//   the load latency spread over the ring: (0.5 + 0.03 per KB of a stage) / stages
//     (56 k blocks, one CTA per SM: 4 stages of 32 KB 23.5 us, 4 stages of 48 KB 31.6 us);
//   the SM's operand bandwidth from L2, about 112 GB/s, shared by its CTAs
//     (8,192^3 with two CTAs per SM and 48 KB stages: 0.43 us per k block and SM); 90 GB/s when three
//     CTAs with 32 KB stages share it (9728 x 896 with SwiGLU at 2,048 rows: 53.7 us as 128 x 128
//     tiles in two stages, 43.8 as 128 x 256 in two stages, 46.0 as 128 x 128 in three).
// CTAs per SM follow from shared and tensor memory; a launch takes ceil(CTAs / resident) rounds; with
// a single CTA per SM nothing hides a CTA's start and end, which costs about 4 us more per round.
// Checked against: 9728 x 896 at 2,048 rows 45 (measured 44.6); 4608 x 3584 at 520 rows, 128 wide,
// 4 stages 53 (47), 256 wide 31.7 (31.6); 37888 x 3584 with SwiGLU at 520 rows, two CTAs per SM 176
// (168), one CTA per SM 178 (180).  It is there to tell a plan with two half-empty rounds from one
// with a single round, no more.
static GemmPlan plan_many_rows(int M, int N, int K, bool swiglu, int sms) {
  const int total_kb = (K + TILE_K - 1) / TILE_K;
  const int tiles_m = (M + TILE_ROWS - 1) / TILE_ROWS;
  GemmPlan best = {128, tiles_m * ((N + 127) / 128), 1, 2, total_kb, TILE_ROWS, false};
  double best_cost = 1e30;
  for (int shape = 0; shape < 3; ++shape) {
    // 128 x 128, 128 x 256, and 256 x 256 (two accumulators per CTA; no split-K)
    const int bn = shape == 0 ? 128 : 256, bm = shape == 2 ? 2 * TILE_ROWS : TILE_ROWS;
    if (bn == 256 && N < 256) continue;
    if (bm > TILE_ROWS && M < 2 * bm) continue;
    if (forced_bn != 0 && forced_bn != bn) continue;
    if (forced_bm != 0 && forced_bm != bm) continue;
    const size_t stage_bytes = (size_t)bm * TILE_K * 2 + (size_t)bn * TILE_K * 2;
    const int tiles = ((M + bm - 1) / bm) * ((N + bn - 1) / bn);
    for (int stages = 2; stages <= MAX_STAGES; ++stages) {
      const size_t shared = stages * stage_bytes + 2048;
      if (shared > 225 * 1024) break;
      if (forced_stages >= 2 && forced_stages != stages) continue;
      int per_sm = (int)((227 * 1024) / shared);
      const int by_tensor_memory = 512 / (bn * (bm / TILE_ROWS));
      if (per_sm > by_tensor_memory) per_sm = by_tensor_memory;
      if (per_sm > 3) per_sm = 3;
      for (int splits = 1; splits <= 4; ++splits) {
        if (splits > 1 && (swiglu || M > 1024 || total_kb < 8 * splits || bm > TILE_ROWS)) break;   // that epilogue reads tensor memory only
        if (forced_splits >= 1 && forced_splits != splits) continue;
        if (splits > 1 && (long long)tiles * splits * bn * TILE_ROWS * 4 > (24ll << 20)) break;
        const long long ctas = (long long)tiles * splits;
        const long long resident = (long long)per_sm * sms;
        const long long rounds = (ctas + resident - 1) / resident;
        const int sharing = (int)(ctas < resident ? (ctas + sms - 1) / sms : per_sm);   // CTAs that really share an SM
        const double kb = (double)((total_kb + splits - 1) / splits);
        const double stage_kb = (double)stage_bytes / 1024.0;
        double per_kb = 0.14 * (bn / 128) * (bm / TILE_ROWS) * sharing;                // tensor pipe
        if ((0.5 + 0.03 * stage_kb) / stages > per_kb) per_kb = (0.5 + 0.03 * stage_kb) / stages;   // load latency
        const double sm_gbs = sharing >= 3 ? 90.0 : 112.0;     // three small rings take in less than two larger ones
        if (sharing * stage_kb / sm_gbs > per_kb) per_kb = sharing * stage_kb / sm_gbs;  // operand bandwidth of the SM
        // per 128 columns; SwiGLU writes half as many, but two accumulators per CTA leave nobody to run under
        const double epilogue = (swiglu && bm == TILE_ROWS) ? 1.0 : 1.5;
        double cost = rounds * (1.5 + kb * per_kb + epilogue * (bn / 128) * (bm / TILE_ROWS) + ((per_sm == 1 && rounds > 1) ? 4.0 : 0.0));
        if (splits > 1) cost += 4.0 + (double)splits * bn * 512.0 / 50e3;
        if (cost < best_cost) {
          best_cost = cost;
          best.bn = bn; best.tiles = tiles; best.splits = splits; best.stages = stages; best.bm = bm;
        }
      }
    }
  }
  best.kb_per_split = (total_kb + best.splits - 1) / best.splits;
  best.splits = (total_kb + best.kb_per_split - 1) / best.kb_per_split;      // no empty split
  // The 256 x 256 tile over an SM pair, with rings of three stages so that two CTAs share an SM and
  // one's epilogue runs under the other's MMAs: that pays where the epilogue is long, which is the
  // SwiGLU one (the gate/up product of 37888 x 3584 at 2,048 rows: 400 us against 424 us in one CTA
  // and 433 us as 128 x 256 tiles; at 520 rows 151 against 162 and 155; 27648 x 5120 at 4,096 rows
  // 825 against 838 and 845; at 384 rows the padding to 512 eats the gain).  The other products are
  // as fast or faster in one CTA with its ring of 64 KB stages.
  const bool pair_fits = N >= 256 && M > 2 * TILE_ROWS;
  // (With 14 k blocks, 9728 x 896, the pair's longer start and end cost more than its epilogue's
  // overlap brings: 46.4 us against 43.8 us as 128 x 256 tiles in two stages; with 24, 17920 x 1536,
  // 90.9 against 92.4.)
  const bool pair_pays = swiglu && best.bn == 256 && M > 3 * TILE_ROWS && total_kb >= 24;
  if (pair_fits && (forced_pair > 0 || (forced_pair == 0 && pair_pays))) {
    best.bn = 256; best.bm = 2 * TILE_ROWS; best.pair = true;
    best.tiles = ((M + 255) / 256) * ((N + 255) / 256);
    best.splits = 1; best.kb_per_split = total_kb;
    best.stages = forced_stages >= 2 ? (forced_stages > 6 ? 6 : forced_stages) : (forced_pair == 1 ? 6 : 3);
  }
  return best;
}

static GemmPlan plan_gemm(int M, int N, int K, bool swiglu) {
  const int sms = sm_count();
  if (M > 128) return plan_many_rows(M, N, K, swiglu, sms);
  GemmPlan plan;
  plan.bm = TILE_ROWS;
  plan.pair = false;
  const int total_kb = (K + TILE_K - 1) / TILE_K;
  plan.bn = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
  plan.tiles = (N + TILE_ROWS - 1) / TILE_ROWS;
  int splits = 1;
  {
    // Few tiles cannot keep every SM streaming weights, so K is cut; but the CTA that arrives last
    // for a tile re-reads every split's partial tile (splits x bn x 512 bytes), which soon costs
    // more than the streaming saves when there are many token rows.  Estimate both and take the
    // cheapest count (microseconds; one CTA of this kernel streams about 50 GB/s - measured: 56 CTAs
    // read a 136 MB matrix at 2.8 TB/s - all of them at most 6 TB/s; two CTAs share an SM; a
    // reduction costs 3.5 us of fences and round trips before its first byte: fitted to 1152 x 896
    // at 64 rows, 7.3 us unsplit against 8.6 / 8.2 / 8.2 / 9.4 us with 2 / 3 / 4 / 6 splits).
    const double sm_bytes_per_us = 50e3, all_bytes_per_us = 6.0e6;
    const double tile_bytes = (double)(TILE_ROWS + plan.bn) * K * 2;
    const int most = total_kb / 2 < 16 ? (total_kb / 2 < 1 ? 1 : total_kb / 2) : 16;
    double best = 1e30;
    for (int candidate = 1; candidate <= most; ++candidate) {
      const double ctas = (double)plan.tiles * candidate;
      const double resident = ctas < 2 * sms ? ctas : 2 * sms;
      const double waves = ctas <= 2 * sms ? 1.0 : ctas / (2.0 * sms);
      double rate = all_bytes_per_us / resident;
      if (rate > sm_bytes_per_us) rate = sm_bytes_per_us;
      double cost = waves * tile_bytes / candidate / rate;
      if (candidate > 1) cost += 3.5 + (double)candidate * plan.bn * 512.0 / sm_bytes_per_us;
      if (cost < best) { best = cost; splits = candidate; }
    }
  }
  if (forced_splits >= 1 && forced_splits <= 16 && forced_splits <= total_kb) splits = forced_splits;
  plan.kb_per_split = (total_kb + splits - 1) / splits;
  plan.splits = (total_kb + plan.kb_per_split - 1) / plan.kb_per_split;   // no empty split
  // A ring as deep as the split is long (at most 6 stages) leaves room for several CTAs per SM,
  // so that one CTA's prologue and epilogue overlap another's streaming.
  int stages = plan.kb_per_split < 2 ? 2 : (plan.kb_per_split > 6 ? 6 : plan.kb_per_split);
  // Few rows but more CTAs than SMs (the head's matrix): keep the ring within 110 KB so that two
  // CTAs share an SM and one's epilogue runs while the other streams (measured on 151936 x 896 at
  // 64 rows: 86 us with one CTA per SM, 64 us with two).
  const size_t few_rows_stage = TILE_ROWS * TILE_K * 2 + (size_t)plan.bn * TILE_K * 2;
  if (forced_stages >= 2) stages = forced_stages <= MAX_STAGES ? forced_stages : MAX_STAGES;
  else if (plan.tiles * plan.splits > sms)
    while (stages > 2 && stages * few_rows_stage > 110 * 1024) --stages;
  const size_t stage_bytes = TILE_ROWS * TILE_K * 2 + (size_t)plan.bn * TILE_K * 2;
  while (stages > 2 && stages * stage_bytes + 1024 > 200 * 1024) --stages;
  plan.stages = stages;
  return plan;
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// For measurements only (the engine never calls it): overrides of the planner; 0 leaves a choice to it.
MLR_EXPORT void mlr_gemm_tcgen05_debug(int bn, int stages, int splits, int bm) {
  forced_bn = bn;
  forced_stages = stages;
  forced_splits = splits;
  forced_bm = bm;
}
// 0: the planner decides whether 256 x 256 tiles lie over SM pairs; -1: never; 1: wherever the shape
// allows, with rings of six stages (one CTA per SM); 2: the same with three stages (two CTAs per SM).
MLR_EXPORT void mlr_gemm_tcgen05_debug_pair(int pair) { forced_pair = pair; }

// Scratch needed for a product of this shape (bytes of float32 partial tiles); 0 without split-K.
// `splits_out` receives the split count the launcher will use, `tiles_out` the number of tiles.
MLR_EXPORT long long mlr_gemm_tcgen05_plan(int M, int N, int K, int swiglu, int* splits_out, int* tiles_out) {
  const GemmPlan plan = plan_gemm(M, N, K, swiglu != 0);
  if (splits_out) *splits_out = plan.splits;
  if (tiles_out) *tiles_out = plan.tiles;
  return plan.splits > 1 ? (long long)plan.tiles * plan.splits * plan.bn * TILE_ROWS * 4 : 0;
}

// x [M,K], w [N,K], bias [N] or null, all bfloat16; out [M,N] bfloat16 (out_f32 = 0) or float32.
// swiglu != 0: w holds blocks of 64 gate rows followed by the 64 up rows of the same outputs
// (N % 128 == 0, no bias) and out is silu(gate) * up, [M, N/2] bfloat16.
// scratch: at least mlr_gemm_tcgen05_plan(...) bytes; counters: one zeroed int per tile;
// error_word: host-visible int that receives a non-zero code if a wait inside the kernel runs out.
MLR_EXPORT int mlr_gemm_tcgen05(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                                int out_f32, int swiglu, void* scratch, int* counters, int* error_word,
                                cudaStream_t stream) {
  if (M == 0) return MLR_OK;
  if (M < 0 || N <= 0 || K <= 0) return MLR_BAD_SIZE;
  if (K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return MLR_BAD_ALIGNMENT;
  if (swiglu && (N % 128 != 0 || bias != nullptr || out_f32)) return MLR_BAD_SIZE;
  const GemmPlan plan = plan_gemm(M, N, K, swiglu != 0);
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.k_blocks_per_split = plan.kb_per_split;
  p.splits = plan.splits;
  p.stages = plan.stages;
  p.bias = (const bf16*)bias;
  p.out = out;
  p.out_f32 = out_f32;
  p.scratch = (float*)scratch;
  p.counters = counters;
  p.error_word = error_word;
  if (plan.splits > 1 && (scratch == nullptr || counters == nullptr)) return MLR_BAD_SIZE;
  if (swiglu) {
    if (M <= 16) return launch<16, true, true>(x, w, p, plan.splits, stream);
    if (M <= 32) return launch<32, true, true>(x, w, p, plan.splits, stream);
    if (M <= 64) return launch<64, true, true>(x, w, p, plan.splits, stream);
    if (M <= 128) return launch<128, true, true>(x, w, p, plan.splits, stream);
    if (plan.pair) return launch_pair<256, true>(x, w, p, stream);
    if (plan.bm == 2 * TILE_ROWS) return launch<256, false, true, 2 * TILE_ROWS>(x, w, p, plan.splits, stream);
    if (plan.bn == 256) return launch<256, false, true>(x, w, p, plan.splits, stream);
    return launch<128, false, true>(x, w, p, plan.splits, stream);
  }
  if (M <= 16) return launch<16, true, false>(x, w, p, plan.splits, stream);
  if (M <= 32) return launch<32, true, false>(x, w, p, plan.splits, stream);
  if (M <= 64) return launch<64, true, false>(x, w, p, plan.splits, stream);
  if (M <= 128) return launch<128, true, false>(x, w, p, plan.splits, stream);
  if (plan.pair) return launch_pair<256, false>(x, w, p, stream);
  if (plan.bm == 2 * TILE_ROWS) return launch<256, false, false, 2 * TILE_ROWS>(x, w, p, plan.splits, stream);
  if (plan.bn == 256) return launch<256, false, false>(x, w, p, plan.splits, stream);
  return launch<128, false, false>(x, w, p, plan.splits, stream);
}
