// y[M,N] = x[M,K] * W[N,K]^T (+ bias) for few rows (M <= 64, a decode step of a small batch),
// bfloat16 in, float32 accumulate, for the layer products whose weight matrix is too small to
// give every SM a 128-row tcgen05 tile: there the cost is a chain of latencies, not bandwidth, and
// this kernel keeps the chain short.
//
// One CTA owns 16 weight rows (output columns; 8 in one variant).  Its warps split K between them in blocks of 32;
// every lane fetches its pieces of W and x with plain 16-byte loads - all loads of a batch of
// k blocks are issued before any is used - and feeds them to mma.sync.m16n8k16 with the 16 weight
// rows on the M side and up to 8 tokens on the N side.  The 16 bytes a lane loads from a row are 8
// consecutive k values; A and B fragments take them in the same (permuted) k order, which leaves
// the dot products unchanged and needs no shared-memory staging.  The warps' partial tiles are
// added in warp order through shared memory (deterministic), bias is added, and for the fused
// gate/up product (weight rows in blocks of 64 gate rows followed by the 64 up rows of the same
// outputs, as the tensor-core kernel takes them) silu(gate) * up is applied before the store.
//
// Two fusions ride along for free.  (1) RMS norm: with rms_eps >= 0 the product is taken of the
// normalised rows x * rsqrt(mean(x^2) + eps); the sums of squares come from the x pieces the lanes
// hold anyway, and the row scale is applied to the finished tile (the norm's weight is expected
// folded into w).  (2) Residual: with a residual pointer the result is added to it (it may be the
// output itself: every element is read and written by the same thread).
//
// Weight loads of the first batch and the bias are issued before the programmatic dependency wait:
// they do not depend on the previous kernel; the residual is asked for right after it, beside x,
// not after the reduction.  The kernel's time inside a decode step is a few round trips to memory,
// so two things are arranged by shape: long rows of few outputs get CTAs of 8 weight rows (ROWS8),
// which hold a whole row in one batch of loads, and register budgets are set so that a product's
// CTAs are all resident at once; mlr_gemm_skinny_rounds tells a caller whether they are.
// Requires K % 8 == 0 and 16-byte aligned rows.
#include "common.cuh"

namespace mlr {

// k blocks (of 32) whose loads are in flight together: fewer when more tokens need registers
__host__ __device__ constexpr int skinny_batch(int tokens8) { return tokens8 <= 2 ? 8 : (tokens8 == 4 ? 4 : 2); }
// CTAs per SM the compiler is asked to leave registers for.  The fused gate/up product of up to 8
// tokens with a batch of 7 fits 168 registers, so that three of its CTAs share an SM: with two, the
// 304 CTAs of a 4864-wide product were 8 more than 148 SMs hold, and those 8 ran as a second round
// that doubled the kernel's time (7.1 instead of 3.6 us inside a decode step).
__host__ __device__ constexpr int skinny_ctas_per_sm(int warps, int groups, int tokens8, int batch) {
  return (warps == 4 && groups == 2 && tokens8 == 1 && batch <= 7) ? 3 : 0;     // 0: no request
}

__device__ __forceinline__ void mma_16x8x16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// GROUPS: 16-row groups per CTA (2 for the fused gate/up product: the gate rows and their up rows).
// TOKENS8: token blocks of 8 (1 for M <= 8, 2 for M <= 16, 4 for M <= 32, 8 for M <= 64).
// SKINNY_BATCH: k blocks per warp whose loads are in flight together.
// ROWS8: the CTA owns 8 weight rows instead of 16 (the MMA's other 8 rows are zeros): twice the CTAs
// and, in the registers of the missing rows, more k blocks in flight per warp, for long rows of few outputs
// (a down projection of 896 outputs: 112 CTAs with their whole rows in flight instead of 56 CTAs
// that fetch theirs in two batches, one after the other).
template <int WARPS, int GROUPS, int TOKENS8, bool SWIGLU, int SKINNY_BATCH = skinny_batch(TOKENS8), bool ROWS8 = false>
__global__ void __launch_bounds__(WARPS * 32, skinny_ctas_per_sm(WARPS, GROUPS, TOKENS8, SKINNY_BATCH))
skinny_gemm_kernel(const bf16* x, const bf16* __restrict__ w, const bf16* __restrict__ bias, void* out,
                   const bf16* residual, int M, int N, int K, int out_f32, float rms_eps) {
  constexpr int ROWS = ROWS8 ? 8 : 16;               // weight rows (output columns) per group
  constexpr int HALVES = ROWS8 ? 1 : 2;              // of the MMA's two row halves, those that hold rows
  static_assert(!ROWS8 || (GROUPS == 1 && !SWIGLU), "8-row CTAs: plain products only");
  extern __shared__ float partial_raw[];
  float (*partial)[GROUPS * TOKENS8 * 4][32] = reinterpret_cast<float (*)[GROUPS * TOKENS8 * 4][32]>(partial_raw);
  __shared__ float squares[WARPS][TOKENS8 * 8];     // per warp: sum of x^2 over its share of K, per token
  __shared__ float row_scale[TOKENS8 * 8];
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int k_blocks = (K + 31) / 32;

  // first weight row of each group of 16
  int row0[GROUPS];
  if (SWIGLU) {
    const int o0 = blockIdx.x * 16;                       // first output column of this CTA
    row0[0] = (o0 / 64) * 128 + (o0 % 64);                // its gate rows
    row0[GROUPS - 1] = row0[0] + 64;                      // and the up rows of the same outputs
  } else {
    row0[0] = blockIdx.x * ROWS;
  }
  const uint4* w_row[GROUPS][HALVES];
  bool w_valid[GROUPS][HALVES];
#pragma unroll
  for (int r = 0; r < GROUPS; ++r)
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
      const int row = row0[r] + g + 8 * h;
      w_valid[r][h] = row < N;
      w_row[r][h] = reinterpret_cast<const uint4*>(w + (size_t)(w_valid[r][h] ? row : 0) * K);
    }
  const uint4* x_row[TOKENS8];
  bool x_valid[TOKENS8];
#pragma unroll
  for (int n = 0; n < TOKENS8; ++n) {
    const int token = n * 8 + g;
    x_valid[n] = token < M;
    x_row[n] = reinterpret_cast<const uint4*>(x + (size_t)(x_valid[n] ? token : 0) * K);
  }

  // the epilogue's bias (rows g and g + 8 of warp 0's lanes): asked for now, not after the reduction
  float bias_value[2] = {0.f, 0.f};
  if (!SWIGLU && bias != nullptr && warp == 0) {
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
      if (row0[0] + g + 8 * h < N) bias_value[h] = to_float(bias[row0[0] + g + 8 * h]);
  }
  bf16 residual_value[TOKENS8][4];          // likewise the residual, as soon as the previous kernel is done

  float acc[GROUPS][TOKENS8][4];
#pragma unroll
  for (int r = 0; r < GROUPS; ++r)
#pragma unroll
    for (int n = 0; n < TOKENS8; ++n) acc[r][n][0] = acc[r][n][1] = acc[r][n][2] = acc[r][n][3] = 0.f;

  float square_sum[TOKENS8];
#pragma unroll
  for (int n = 0; n < TOKENS8; ++n) square_sum[n] = 0.f;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  bool waited = false;
  auto fetch_residual = [&]() {
    if (SWIGLU || residual == nullptr || warp != 0) return;
#pragma unroll
    for (int n = 0; n < TOKENS8; ++n)
#pragma unroll
      for (int e = 0; e < 2 * HALVES; ++e) {
        const int token = n * 8 + 2 * t + (e & 1), row = row0[0] + g + 8 * (e >> 1);
        if (token < M && row < N) residual_value[n][e] = residual[(size_t)token * N + row];
      }
  };
  for (int first = warp; first < k_blocks; first += WARPS * SKINNY_BATCH) {
    uint4 wv[SKINNY_BATCH][GROUPS][HALVES], xv[SKINNY_BATCH][TOKENS8];
#pragma unroll
    for (int i = 0; i < SKINNY_BATCH; ++i) {
      const int piece = (first + i * WARPS) * 4 + t;          // index of this lane's 16 bytes in the row
      const bool in_range = first + i * WARPS < k_blocks && piece * 8 < K;
#pragma unroll
      for (int r = 0; r < GROUPS; ++r)
#pragma unroll
        for (int h = 0; h < HALVES; ++h) wv[i][r][h] = (in_range && w_valid[r][h]) ? __ldg(w_row[r][h] + piece) : zero;
    }
    if (!waited) {
      pdl_wait();                                             // x comes from the kernel before this one
      waited = true;
      fetch_residual();
    }
#pragma unroll
    for (int i = 0; i < SKINNY_BATCH; ++i) {
      const int piece = (first + i * WARPS) * 4 + t;
      const bool in_range = first + i * WARPS < k_blocks && piece * 8 < K;
#pragma unroll
      for (int n = 0; n < TOKENS8; ++n) xv[i][n] = (in_range && x_valid[n]) ? __ldcg(x_row[n] + piece) : zero;
    }
    if (rms_eps >= 0.f) {
#pragma unroll
      for (int i = 0; i < SKINNY_BATCH; ++i)
#pragma unroll
        for (int n = 0; n < TOKENS8; ++n) {
          const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&xv[i][n]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 two = __bfloat1622float2(pairs[j]);
            square_sum[n] += two.x * two.x + two.y * two.y;
          }
        }
    }
#pragma unroll
    for (int i = 0; i < SKINNY_BATCH; ++i)
#pragma unroll
      for (int r = 0; r < GROUPS; ++r)
#pragma unroll
        for (int n = 0; n < TOKENS8; ++n) {
          // the lane's 8 k values: (x, y) feed one MMA, (z, w) the next, same order in A and B
          const uint4 lower = wv[i][r][0], upper = ROWS8 ? zero : wv[i][r][HALVES - 1];
          mma_16x8x16(acc[r][n], lower.x, upper.x, lower.y, upper.y, xv[i][n].x, xv[i][n].y);
          mma_16x8x16(acc[r][n], lower.z, upper.z, lower.w, upper.w, xv[i][n].z, xv[i][n].w);
        }
  }
  if (!waited) {
    pdl_wait();
    fetch_residual();
  }

  // ---- add the warps' partial tiles in warp order
#pragma unroll
  for (int r = 0; r < GROUPS; ++r)
#pragma unroll
    for (int n = 0; n < TOKENS8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) partial[warp][(r * TOKENS8 + n) * 4 + e][lane] = acc[r][n][e];
  // the four lanes of a token (t = 0..3) hold disjoint pieces of its row
#pragma unroll
  for (int n = 0; n < TOKENS8; ++n) {
    float sum = square_sum[n];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (t == 0) squares[warp][n * 8 + g] = sum;
  }
  __syncthreads();
  if (warp != 0) return;
  if (lane < TOKENS8 * 8) {
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < WARPS; ++v) sum += squares[v][lane];
    row_scale[lane] = rms_eps >= 0.f ? rsqrtf(sum / (float)K + rms_eps) : 1.f;
  }
  if (TOKENS8 * 8 > 32 && lane + 32 < TOKENS8 * 8) {
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < WARPS; ++v) sum += squares[v][lane + 32];
    row_scale[lane + 32] = rms_eps >= 0.f ? rsqrtf(sum / (float)K + rms_eps) : 1.f;
  }
  __syncwarp();
#pragma unroll
  for (int r = 0; r < GROUPS; ++r)
#pragma unroll
    for (int n = 0; n < TOKENS8; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < WARPS; ++v) sum += partial[v][(r * TOKENS8 + n) * 4 + e][lane];
        acc[r][n][e] = sum;
      }

  // ---- epilogue: element e of a tile is (row g + 8*(e/2), token n*8 + 2t + e%2)
  bf16* out_bf16 = (bf16*)out;
  float* out_f32p = (float*)out;
#pragma unroll
  for (int n = 0; n < TOKENS8; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int token = n * 8 + 2 * t + (e & 1);
      if (token >= M) continue;
      const float scale = row_scale[token];
      if (SWIGLU) {
        const int column = blockIdx.x * 16 + g + 8 * (e >> 1);
        const int half = N >> 1;
        if (column < half) {
          const float gate = acc[0][n][e] * scale, up = acc[GROUPS - 1][n][e] * scale;
          out_bf16[(size_t)token * half + column] = __float2bfloat16_rn(silu_times(gate, up));
        }
      } else {
        if (ROWS8 && e >= 2) continue;                     // the MMA's upper rows hold nothing
        const int row = row0[0] + g + 8 * (e >> 1);
        if (row < N) {
          float value = acc[0][n][e] * scale + bias_value[e >> 1];
          if (residual != nullptr) value += to_float(residual_value[n][e]);
          if (out_f32) out_f32p[(size_t)token * N + row] = value;
          else out_bf16[(size_t)token * N + row] = __float2bfloat16_rn(value);
        }
      }
    }
}

template <int WARPS, int GROUPS, int TOKENS8, bool SWIGLU, int BATCH = skinny_batch(TOKENS8), bool ROWS8 = false>
static int skinny_launch_one(const void* x, const void* w, const void* bias, void* out, const void* residual, int M,
                             int N, int K, int out_f32, float rms_eps, int groups_of_rows, cudaStream_t stream,
                             int* rounds_out) {
  const size_t shared = (size_t)WARPS * GROUPS * TOKENS8 * 4 * 32 * sizeof(float);
  if (shared > 48 * 1024) {
    static bool configured = false;
    if (!configured) {
      cudaError_t err = cudaFuncSetAttribute(skinny_gemm_kernel<WARPS, GROUPS, TOKENS8, SWIGLU, BATCH, ROWS8>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      if (err != cudaSuccess) return (int)err;
      configured = true;
    }
  }
  if (rounds_out != nullptr) {
    // a question, not a launch: in how many rounds would this grid's CTAs run (by what the device
    // says it holds of this instantiation)
    static int per_sm = 0;
    if (per_sm == 0) {
      int blocks = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, skinny_gemm_kernel<WARPS, GROUPS, TOKENS8, SWIGLU, BATCH, ROWS8>,
                                                        WARPS * 32, shared) != cudaSuccess || blocks < 1)
        blocks = 1;
      per_sm = blocks;
    }
    const int together = per_sm * sm_count();
    *rounds_out = (groups_of_rows + together - 1) / together;
    return MLR_OK;
  }
  launch_kernel(skinny_gemm_kernel<WARPS, GROUPS, TOKENS8, SWIGLU, BATCH, ROWS8>, dim3(groups_of_rows), dim3(WARPS * 32), shared,
                stream, (const bf16*)x, (const bf16*)w, (const bf16*)bias, out, (const bf16*)residual, M, N, K, out_f32,
                rms_eps);
  return launch_status();
}

template <int WARPS, int TOKENS8>
static int skinny_launch(const void* x, const void* w, const void* bias, void* out, const void* residual, int M, int N,
                         int K, int out_f32, int swiglu, float rms_eps, cudaStream_t stream, int* rounds_out) {
  if constexpr (WARPS <= 8) {
    if (swiglu) {
      if constexpr (WARPS == 4 && TOKENS8 == 1) {
        // rows of at most 7 k blocks per warp (896 wide): a batch of 7 leaves registers for a third CTA per SM
        if ((K + 31) / 32 <= 7 * WARPS)
          return skinny_launch_one<WARPS, 2, TOKENS8, true, 7>(x, w, bias, out, residual, M, N, K, out_f32, rms_eps,
                                                               (N / 2 + 15) / 16, stream, rounds_out);
      }
      return skinny_launch_one<WARPS, 2, TOKENS8, true>(x, w, bias, out, residual, M, N, K, out_f32, rms_eps,
                                                        (N / 2 + 15) / 16, stream, rounds_out);
    }
  }
  return skinny_launch_one<WARPS, 1, TOKENS8, false>(x, w, bias, out, residual, M, N, K, out_f32, rms_eps,
                                                     (N + 15) / 16, stream, rounds_out);
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

static int skinny_dispatch(const void* x, const void* w, const void* bias, void* out, const void* residual,
                           int M, int N, int K, int out_f32, int swiglu, float rms_eps, cudaStream_t stream,
                           int* rounds_out) {
  if (M == 0) return MLR_OK;
  if (M < 0 || N <= 0 || K <= 0) return MLR_BAD_SIZE;
  if (M > 64) return MLR_TOO_LARGE;
  if (K % 8 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return MLR_BAD_ALIGNMENT;
  if (swiglu && (N % 128 != 0 || bias != nullptr || out_f32 || residual != nullptr)) return MLR_BAD_SIZE;
  if (swiglu && K > 2048) return MLR_TOO_LARGE;      // two row groups and a long K do not fit the registers
  // The CTA's warps share K.  Short rows: 4 warps (8 once many tokens shrink the load batches);
  // long rows (the down projection): 16 warps, or 8 where 16 would run out of registers.
  const bool long_rows = K > 2048;
  if (M <= 8) {
    // 16 warps fill an SM's register file with one CTA; rows of up to 4,096 go to 8 warps, two CTAs
    // per SM, so that the 224 to 288 CTAs of a 7B attention projection run in one round
    // (longer rows too when there are more CTAs than SMs: one 16-warp CTA per SM would come in three rounds)
    // and where 8-row CTAs still fit one round and hold a whole row in one batch, those (see ROWS8)
    if (!swiglu && K > 4096 && (N + 7) / 8 <= sm_count() && (K + 31) / 32 <= 16 * 10)
      return skinny_launch_one<16, 1, 1, false, 10, true>(x, w, bias, out, residual, M, N, K, out_f32, rms_eps,
                                                          (N + 7) / 8, stream, rounds_out);
    if (K > 4096 && (N + 15) / 16 <= sm_count())
      return skinny_launch<16, 1>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
    if (long_rows) return skinny_launch<8, 1>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
    return skinny_launch<4, 1>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
  }
  if (M <= 16) {
    if (long_rows) return skinny_launch<8, 2>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
    return skinny_launch<4, 2>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
  }
  if (M <= 32) return skinny_launch<8, 4>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
  return skinny_launch<8, 8>(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, rounds_out);
}


// x [M,K], w [N,K], bias [N] or null (bfloat16); out [M,N] bfloat16 or float32 (out_f32).
// swiglu != 0: w interleaves blocks of 64 gate rows with the 64 up rows of the same outputs
// (N % 128 == 0, no bias); out is silu(gate) * up, [M, N/2] bfloat16.  M <= 64, K % 8 == 0.
// rms_eps >= 0: the product acts on the RMS-normalised rows of x.  residual: [M,N] bfloat16 added
// to the result (it may be `out`), or null; not with swiglu.
MLR_EXPORT int mlr_gemm_skinny(const void* x, const void* w, const void* bias, void* out, const void* residual,
                               int M, int N, int K, int out_f32, int swiglu, float rms_eps, cudaStream_t stream) {
  return skinny_dispatch(x, w, bias, out, residual, M, N, K, out_f32, swiglu, rms_eps, stream, nullptr);
}

// Rounds in which the CTAs of that product would run on this device (1: all of them at once), or a
// negative number if the kernel does not take the shape.  Launches nothing.
MLR_EXPORT int mlr_gemm_skinny_rounds(int M, int N, int K, int swiglu) {
  int rounds = 0;
  alignas(16) static const char aligned[16] = {0};
  const int status = skinny_dispatch(aligned, aligned, nullptr, nullptr, nullptr, M, N, K, 0, swiglu, -1.f, nullptr, &rounds);
  return status == MLR_OK ? rounds : -1;
}
