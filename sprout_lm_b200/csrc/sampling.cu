// Sampling from float32 logits on the device, one block per row.
//   greedy: the lowest index among the maxima; a row with a non-finite logit gives -1
//           and sets a status bit (the reference's argmax rule and failure).
//   temperature: p = softmax(logits / T) in float32, then the inverse of the cumulative
//           distribution at a uniform number u in [0, 1) that the host derives from
//           (seed, request, index of the output token), so the draw does not depend on
//           the batch.  Rows with T == 0 are greedy.
#include "common.cuh"

namespace {

constexpr int THREADS = 1024;

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ temperature,
              const float* __restrict__ uniform, int* __restrict__ out, int vocab, int* status) {
  __shared__ float scratch[33];
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_prefix[THREADS];
  __shared__ int s_result;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;

  // every thread owns a contiguous segment, so that cumulative sums follow index order
  const int seg = (vocab + THREADS - 1) / THREADS;
  const int begin = min(tid * seg, vocab), end = min(begin + seg, vocab);

  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = begin; i < end; i++) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    if (v > best) { best = v; best_i = i; }
  }
  // argmax with the lowest index winning ties
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  const int any_bad = __syncthreads_or(bad ? 1 : 0);
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = s_val[lane];
    best_i = s_idx[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
  }
  __syncthreads();
  if (any_bad) {
    if (tid == 0) { out[r] = -1; atomicOr(status, SPROUT_STATUS_NONFINITE); }
    return;
  }
  const float top = s_val[0];
  const float temp = temperature ? temperature[r] : 0.f;
  if (!(temp > 0.f)) {
    if (tid == 0) out[r] = s_idx[0];
    return;
  }
  // softmax(logits / T): weights exp((v - top) / T), summed per segment then across segments
  float local = 0.f;
  for (int i = begin; i < end; i++) local += expf((row[i] - top) / temp);
  s_prefix[tid] = local;
  __syncthreads();
  const float total = block_sum(local, scratch);
  // exclusive prefix over segments, done by one warp over 32 values per lane (fixed order)
  if (warp == 0) {
    float run = 0.f;
    float mine[THREADS / 32];
#pragma unroll
    for (int j = 0; j < THREADS / 32; j++) { mine[j] = s_prefix[lane * (THREADS / 32) + j]; run += mine[j]; }
    float incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    float excl = incl - run;
#pragma unroll
    for (int j = 0; j < THREADS / 32; j++) { s_prefix[lane * (THREADS / 32) + j] = excl; excl += mine[j]; }
  }
  if (tid == 0) s_result = -1;
  __syncthreads();
  const float target = uniform[r] * total;
  // segment intervals [prefix[tid], prefix[tid + 1]) cover [0, inf) without gap or overlap
  const float before = s_prefix[tid];
  const bool last_segment = (tid == THREADS - 1) || ((tid + 1) * seg >= vocab);
  const float after = last_segment ? INFINITY : s_prefix[tid + 1];
  if (begin < end && target >= before && target < after) {
    float run = before;
    int pick = end - 1;
    for (int i = begin; i < end; i++) {
      run += expf((row[i] - top) / temp);
      if (target < run) { pick = i; break; }
    }
    atomicMax(&s_result, pick);
  }
  __syncthreads();
  if (tid == 0) {
    int pick = s_result;
    if (pick < 0) {
      // rounding left the target beyond the last segment's end: take the last index with weight
      pick = vocab - 1;
    }
    out[r] = pick;
  }
}

}  // namespace

// logits [rows, vocab] with row stride ld; temperature and uniform may be null (all greedy).
SPROUT_API int sprout_sample(const float* logits, int ld, const float* temperature, const float* uniform,
                             int* out, int rows, int vocab, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
  SPROUT_REQUIRE(logits && out && status, "sample: null pointer");
  SPROUT_REQUIRE((temperature == nullptr) == (uniform == nullptr), "sample: temperature and uniform go together");
  sample_kernel<<<rows, THREADS, 0, stream>>>(logits, ld, temperature, uniform, out, vocab, status);
  return sprout_check_launch("sample");
}

// ------------------------------------------------------------------ feeding a decode step's output back
// After a decode step on the device: every request's sampled token becomes its next input
// token, its position and cache length grow by one, and the tokens are recorded in row
// `*step_counter` of `history` ([max_steps, requests]); the counter then advances.  This lets
// several decode steps run back to back (or as one replayed CUDA graph) without the host.
__global__ void advance_decode_kernel(int* token_ids, int* positions, int* context_lens, const int* sampled,
                                      int* history, int* step_counter, int requests, int max_steps) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int step = *step_counter;
  if (r < requests) {
    const int token = sampled[r];
    token_ids[r] = token < 0 ? 0 : token;
    positions[r] += 1;
    context_lens[r] += 1;
    if (step < max_steps) history[(size_t)step * requests + r] = token;
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0 && gridDim.x == 1) *step_counter = step + 1;
}

SPROUT_API int sprout_advance_decode(int* token_ids, int* positions, int* context_lens, const int* sampled,
                                     int* history, int* step_counter, int requests, int max_steps,
                                     cudaStream_t stream) {
  SPROUT_REQUIRE(requests > 0 && requests <= 1024 && max_steps > 0, "advance_decode: 1..1024 requests, max_steps > 0");
  SPROUT_REQUIRE(token_ids && positions && context_lens && sampled && history && step_counter, "advance_decode: null pointer");
  advance_decode_kernel<<<1, 1024, 0, stream>>>(token_ids, positions, context_lens, sampled, history, step_counter,
                                                requests, max_steps);
  return sprout_check_launch("advance_decode");
}
