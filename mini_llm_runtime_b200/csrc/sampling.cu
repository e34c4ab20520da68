// Next-token choice from float32 logits, one CTA per row: greedy argmax (lowest index wins a tie,
// like the torch.argmax the reference calls at src/mini_llm_runtime/engine.py:222,246) and
// temperature sampling, which the reference does not have.
//
// Temperature sampling: p = softmax(logits / T) in float32; u in [0,1) comes from a counter-based
// generator keyed by the request's seed and the index of the token being produced, so a request's
// tokens do not depend on which other requests share the batch; the token is the first index
// whose cumulative probability exceeds u.  The cumulative sum is taken in a fixed order (warp w
// owns one contiguous stretch of the vocabulary, walked 32 entries at a time).  Any vocabulary
// size is accepted.
#include "common.cuh"

namespace mlr {

constexpr int SAMPLE_THREADS = 1024;
constexpr int SAMPLE_WARPS = SAMPLE_THREADS / 32;

__device__ __forceinline__ float uniform_from_seed(unsigned long long seed, long long index) {
  unsigned long long z = seed + (unsigned long long)(index + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* logits, const float* __restrict__ temperatures,
              const long long* __restrict__ seeds, const long long* __restrict__ counters,
              int* __restrict__ tokens, int vocab, const int* __restrict__ row_slot, SlotState* state,
              int advance) {
  // With `state`, a row's temperature, seed and counter come from the slot record of its request
  // (row_slot[row]); the chosen token is also written there as the request's last token, the
  // counter grows by one and, with `advance`, so does the slot's length (a step in which every
  // request brought exactly one token).  The record was written by the previous step's launch of
  // this kernel, hence plain loads after the wait.
  pdl_trigger();
  pdl_wait();
  __shared__ float scratch[32];
  __shared__ int scratch_index[32];
  __shared__ float warp_totals[SAMPLE_WARPS];
  __shared__ int chosen;
  const float* row = logits + (size_t)blockIdx.x * vocab;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  SlotState* record = state != nullptr ? state + row_slot[blockIdx.x] : nullptr;
  const float temperature = record != nullptr ? record->temperature : temperatures[blockIdx.x];

  // ---- argmax with the lowest index on ties (also gives the softmax's max)
  float best = -INFINITY;
  int best_index = vocab;
  if ((vocab & 3) == 0) {
    // 16-byte loads, four rounds in flight: the row is walked by one CTA, so the loop is a chain of
    // load latencies and fewer, wider rounds are what shortens it
    const float4* row4 = reinterpret_cast<const float4*>(row);
    const int pieces = vocab >> 2;
    for (int p0 = threadIdx.x; p0 < pieces; p0 += 4 * SAMPLE_THREADS) {
      float4 v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = p0 + j * SAMPLE_THREADS;
        v[j] = p < pieces ? row4[p] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {              // ascending index within the thread: the first maximum is kept
        const int i = (p0 + j * SAMPLE_THREADS) * 4;
        if (v[j].x > best) { best = v[j].x; best_index = i; }
        if (v[j].y > best) { best = v[j].y; best_index = i + 1; }
        if (v[j].z > best) { best = v[j].z; best_index = i + 2; }
        if (v[j].w > best) { best = v[j].w; best_index = i + 3; }
      }
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += SAMPLE_THREADS) {
      const float v = row[i];
      if (v > best) { best = v; best_index = i; }  // ascending i: the first maximum is kept
    }
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, best, offset);
    const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
    if (other > best || (other == best && other_index < best_index)) { best = other; best_index = other_index; }
  }
  if (lane == 0) { scratch[warp] = best; scratch_index[warp] = best_index; }
  __syncthreads();
  if (warp == 0) {
    best = scratch[lane];
    best_index = scratch_index[lane];
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
      if (other > best || (other == best && other_index < best_index)) { best = other; best_index = other_index; }
    }
    if (lane == 0) { scratch[0] = best; scratch_index[0] = best_index < vocab ? best_index : 0; }
  }
  __syncthreads();
  const float row_max = scratch[0];
  if (!(temperature > 0.f)) {
    if (threadIdx.x == 0) {
      tokens[blockIdx.x] = scratch_index[0];
      if (record != nullptr) {
        record->last_token = scratch_index[0];
        record->counter += 1;
        if (advance) record->length += 1;
      }
    }
    return;
  }

  // ---- sum of exp((x - max) / T); warp w owns [w*stretch, (w+1)*stretch)
  const float inv_t = 1.f / temperature;
  const int stretch = ((vocab + SAMPLE_WARPS - 1) / SAMPLE_WARPS + 31) / 32 * 32;
  const int begin = warp * stretch, end = min(vocab, begin + stretch);
  float total = 0.f;  // identical in every lane of the warp
  for (int base = begin; base < end; base += 32) {
    const int i = base + lane;
    const float e = i < end ? expf((row[i] - row_max) * inv_t) : 0.f;
    total += warp_sum(e);
  }
  if (lane == 0) warp_totals[warp] = total;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();

  float before = 0.f, everything = 0.f;  // sum of the warps before mine; sum of all
  for (int w = 0; w < SAMPLE_WARPS; ++w) {
    if (w == warp) before = everything;
    everything += warp_totals[w];
  }
  const unsigned long long seed = record != nullptr
      ? ((unsigned long long)record->seed_high << 32) | record->seed_low : (unsigned long long)seeds[blockIdx.x];
  const long long counter = record != nullptr ? (long long)record->counter : counters[blockIdx.x];
  const float u = uniform_from_seed(seed, counter);
  const float target = u * everything;
  const bool mine = target >= before && (target < before + total);
  if (mine) {
    float running = before;
    int found = -1;
    for (int base = begin; base < end && found < 0; base += 32) {
      const int i = base + lane;
      const float e = i < end ? expf((row[i] - row_max) * inv_t) : 0.f;
      float inclusive = e;
#pragma unroll
      for (int offset = 1; offset < 32; offset <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += up;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, i < end && running + inclusive > target);
      if (hit != 0u) found = base + (__ffs(hit) - 1);
      running += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (lane == 0) chosen = found >= 0 ? found : end - 1;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // Rounding can leave the target just past the last stretch; take the last token then.
    const int token = chosen >= 0 ? chosen : vocab - 1;
    tokens[blockIdx.x] = token;
    if (record != nullptr) {
      record->last_token = token;
      record->counter += 1;
      if (advance) record->length += 1;
    }
  }
}

}  // namespace mlr

using namespace mlr;

MLR_DEFINE_PDL_SWITCH

// temperatures[r] <= 0 selects greedy for row r.  tokens: int32 [rows].
MLR_EXPORT int mlr_sample(const float* logits, const float* temperatures, const long long* seeds,
                          const long long* counters, int* tokens, int rows, int vocab,
                          cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || vocab <= 0) return MLR_BAD_SIZE;
  launch_kernel(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, temperatures, seeds, counters,
                tokens, vocab, (const int*)nullptr, (SlotState*)nullptr, 0);
  return launch_status();
}

// The same choice with the sampling parameters taken from, and the result recorded in, the slot
// records of the rows' requests: row_slot int32 [rows], state: SlotState records.  A request must
// not own two rows of one call.
MLR_EXPORT int mlr_sample_slots(const float* logits, const int* row_slot, void* state, int* tokens, int rows,
                                int vocab, int advance, cudaStream_t stream) {
  if (rows == 0) return MLR_OK;
  if (rows < 0 || vocab <= 0 || row_slot == nullptr || state == nullptr) return MLR_BAD_SIZE;
  launch_kernel(sample_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, stream, logits, (const float*)nullptr,
                (const long long*)nullptr, (const long long*)nullptr, tokens, vocab, row_slot, (SlotState*)state,
                advance);
  return launch_status();
}
