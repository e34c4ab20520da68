// y[M,N] = x[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores, float32 multiply-add throughout.
//
// This is the matrix product of the true 32-bit path (no tensor cores, no TF32) and the fallback
// of the bfloat16 path for shapes the tensor-core kernel refuses.  Weights keep the checkpoint's
// [out, in] layout, as the reference's F.linear calls do (qwen_model_runner.py:88-102,183,215-217).
//
// Every output element is one chain of fmaf over k = 0..K-1 in ascending order, whatever M, the
// tile shape or the position of the row in the batch: results do not depend on how tokens are
// batched.  Any M, N, K is accepted.
#include "common.cuh"

namespace mlr {

constexpr int BN = 64;
constexpr int BK = 16;

template <typename TIn, typename TOut, int BM>
__global__ void __launch_bounds__(256)
linear_simt_kernel(const TIn* x, const TIn* __restrict__ w, const TIn* __restrict__ bias,
                   TOut* __restrict__ y, int M, int N, int K) {
  pdl_trigger();
  pdl_wait();
  constexpr int TM = BM / 16;  // rows per thread
  constexpr int TN = BN / 16;  // columns per thread
  __shared__ float a_tile[BK][BM + 1];
  __shared__ float b_tile[BK][BN + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
      const int r = idx / BK, c = idx - r * BK;
      const int gm = m0 + r, gk = k0 + c;
      a_tile[c][r] = (gm < M && gk < K) ? to_float(x[(size_t)gm * K + gk]) : 0.f;
    }
    for (int idx = threadIdx.x; idx < BN * BK; idx += 256) {
      const int r = idx / BK, c = idx - r * BK;
      const int gn = n0 + r, gk = k0 + c;
      b_tile[c][r] = (gn < N && gk < K) ? to_float(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = a_tile[k][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = b_tile[k][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty + 16 * i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx + 16 * j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += to_float(bias[gn]);
      y[(size_t)gm * N + gn] = from_float<TOut>(v);
    }
  }
}

template <typename TIn, typename TOut>
int linear_simt_launch(const void* x, const void* w, const void* bias, void* y, int M, int N, int K,
                       cudaStream_t stream) {
  if (M <= 16) {
    dim3 grid((N + BN - 1) / BN, (M + 15) / 16);
    launch_kernel(linear_simt_kernel<TIn, TOut, 16>, dim3(grid), dim3(256), 0, stream, (const TIn*)x, (const TIn*)w,
                                                                 (const TIn*)bias, (TOut*)y, M, N, K);
  } else {
    dim3 grid((N + BN - 1) / BN, (M + 63) / 64);
    launch_kernel(linear_simt_kernel<TIn, TOut, 64>, dim3(grid), dim3(256), 0, stream, (const TIn*)x, (const TIn*)w,
                                                                 (const TIn*)bias, (TOut*)y, M, N, K);
  }
  return launch_status();
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// in_dtype: storage of x, w and bias.  out_dtype: storage of y (float32 output from bfloat16
// inputs is used for logits).
MLR_EXPORT int mlr_linear_simt(const void* x, const void* w, const void* bias, void* y, int M, int N,
                               int K, int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0) return MLR_OK;
  if (M < 0 || N <= 0 || K <= 0) return MLR_BAD_SIZE;
  if ((M + 15) / 16 > 65535) return MLR_TOO_LARGE;
  if (in_dtype == MLR_F32 && out_dtype == MLR_F32)
    return linear_simt_launch<float, float>(x, w, bias, y, M, N, K, stream);
  if (in_dtype == MLR_BF16 && out_dtype == MLR_BF16)
    return linear_simt_launch<bf16, bf16>(x, w, bias, y, M, N, K, stream);
  if (in_dtype == MLR_BF16 && out_dtype == MLR_F32)
    return linear_simt_launch<bf16, float>(x, w, bias, y, M, N, K, stream);
  return MLR_BAD_DTYPE;
}
