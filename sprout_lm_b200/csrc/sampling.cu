// Sampling from float32 logits on the device.
//   greedy: the lowest index among the maxima; a row with a non-finite logit gives -1
//           and sets a status bit (the reference's argmax rule and failure).
//   temperature: p = softmax(logits / T) in float32, then the inverse of the cumulative
//           distribution at a uniform number u in [0, 1) that the host derives from
//           (seed, request, index of the output token), so the draw does not depend on
//           the batch.  Rows with T == 0 are greedy.
// Two launches: the vocabulary of every row is cut into CHUNKS runs, one block per (run, row)
// finds the run's maximum, its first index and (for T > 0) the sum of exp((v - max) / T) with
// coalesced reads; one block per row then merges the runs in index order and, for T > 0, scans
// the one run in which the draw falls.  The partial results live in a buffer the caller gives.
#include "common.cuh"

namespace {

constexpr int CHUNKS = 64, PART_THREADS = 256, FINAL_THREADS = 1024;

struct Partial { float max; int index; float sum; int bad; };

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

__global__ void __launch_bounds__(PART_THREADS)
sample_partial_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ temperature,
                      Partial* __restrict__ partials, int vocab) {
  __shared__ float s_val[PART_THREADS / 32];
  __shared__ int s_idx[PART_THREADS / 32];
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, r = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int len = (vocab + CHUNKS - 1) / CHUNKS;
  const int begin = min(chunk * len, vocab), end = min(begin + len, vocab);
  const float* row = logits + (size_t)r * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  int bad = 0;
  for (int i = begin + tid; i < end; i += PART_THREADS) {
    const float v = row[i];
    if (!isfinite(v)) bad = 1;
    if (v > best) { best = v; best_i = i; }        // ascending i: the first maximum stays
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    better(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
  bad = __syncthreads_or(bad);
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  best = s_val[0]; best_i = s_idx[0];
#pragma unroll
  for (int w = 1; w < PART_THREADS / 32; w++) better(best, best_i, s_val[w], s_idx[w]);
  float sum = 0.f;
  const float temp = temperature ? temperature[r] : 0.f;
  if (temp > 0.f && !bad && begin < end) {
    for (int i = begin + tid; i < end; i += PART_THREADS) sum += __expf((row[i] - best) / temp);
    sum = block_sum(sum, scratch);
  }
  if (tid == 0) partials[(size_t)r * CHUNKS + chunk] = Partial{best, best_i, sum, bad};
}

__global__ void __launch_bounds__(FINAL_THREADS)
sample_final_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ temperature,
                    const float* __restrict__ uniform, const Partial* __restrict__ partials,
                    int* __restrict__ out, int vocab, int* status) {
  __shared__ Partial s_part[CHUNKS];
  __shared__ float s_prefix[FINAL_THREADS];
  __shared__ int s_chunk, s_result, s_last_weighted, s_best;
  __shared__ float s_before, s_top;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)r * ld;
  if (tid < CHUNKS) s_part[tid] = partials[(size_t)r * CHUNKS + tid];
  __syncthreads();
  const float temp = temperature ? temperature[r] : 0.f;
  if (tid == 0) {
    float best = -INFINITY, total = 0.f;
    int best_i = 0x7fffffff, bad = 0;
    for (int c = 0; c < CHUNKS; c++) { better(best, best_i, s_part[c].max, s_part[c].index); bad |= s_part[c].bad; }
    s_top = best;
    s_best = best_i;
    s_last_weighted = -1;
    s_chunk = -1;
    if (bad) {
      out[r] = -1;
      atomicOr(status, SPROUT_STATUS_NONFINITE);
    } else if (!(temp > 0.f)) {
      out[r] = best_i;
    } else {
      // weights of the runs against the row's maximum, in index order; the run the draw falls in
      for (int c = 0; c < CHUNKS; c++) total += s_part[c].sum * __expf((s_part[c].max - best) / temp);
      const float target = uniform[r] * total;
      float before = 0.f;
      int pick = -1, last = 0;
      for (int c = 0; c < CHUNKS; c++) {
        const float w = s_part[c].sum * __expf((s_part[c].max - best) / temp);
        if (w > 0.f) last = c;
        if (pick < 0 && target < before + w) { pick = c; break; }
        before += w;
      }
      if (pick < 0) {                  // rounding pushed the target past the end: the last run with weight
        pick = last;
        before = 0.f;
        for (int c = 0; c < last; c++) before += s_part[c].sum * __expf((s_part[c].max - best) / temp);
      }
      s_chunk = pick;
      s_before = target - before;      // the draw, counted from the run's start
      s_result = -1;
    }
  }
  __syncthreads();
  const int chunk = s_chunk;
  if (chunk < 0) return;
  // scan the run: each thread owns a contiguous piece, pieces are summed in index order
  const int len = (vocab + CHUNKS - 1) / CHUNKS;
  const int c_begin = min(chunk * len, vocab), c_end = min(c_begin + len, vocab);
  const int seg = (c_end - c_begin + FINAL_THREADS - 1) / FINAL_THREADS;
  const int begin = min(c_begin + tid * seg, c_end), end = min(begin + seg, c_end);
  const float top = s_top, target = s_before;
  float local = 0.f;
  for (int i = begin; i < end; i++) local += __expf((row[i] - top) / temp);
  s_prefix[tid] = local;
  if (local > 0.f) atomicMax(&s_last_weighted, tid);
  __syncthreads();
  if (warp == 0) {
    float run = 0.f;
    float mine[FINAL_THREADS / 32];
#pragma unroll
    for (int j = 0; j < FINAL_THREADS / 32; j++) { mine[j] = s_prefix[lane * (FINAL_THREADS / 32) + j]; run += mine[j]; }
    float incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    float excl = incl - run;
#pragma unroll
    for (int j = 0; j < FINAL_THREADS / 32; j++) { s_prefix[lane * (FINAL_THREADS / 32) + j] = excl; excl += mine[j]; }
  }
  __syncthreads();
  // Piece intervals [prefix[tid], prefix[tid + 1]) cover [0, inf) without gap or overlap; the last
  // piece that has any weight reaches to infinity, so a target that rounding pushed past the total
  // (the run's weight was summed in another order by the first kernel) lands on a token with
  // probability above zero, never on a tail of zeros.
  const float before = s_prefix[tid];
  const float after = tid == s_last_weighted ? INFINITY : (tid + 1 < FINAL_THREADS ? s_prefix[tid + 1] : before);
  if (begin < end && local > 0.f && target >= before && target < after) {
    float run = before;
    int pick = -1, last_weighted = begin;
    for (int i = begin; i < end; i++) {
      const float e = __expf((row[i] - top) / temp);
      run += e;
      if (e > 0.f) last_weighted = i;
      if (target < run) { pick = i; break; }
    }
    atomicMax(&s_result, pick >= 0 ? pick : last_weighted);
  }
  __syncthreads();
  if (tid == 0) out[r] = s_result >= 0 ? s_result : s_best;      // a run without any weight cannot be picked; the maximum then
}

}  // namespace

// Bytes of scratch that sampling `rows` rows needs.
SPROUT_API long long sprout_sample_scratch_bytes(int rows) { return (long long)rows * CHUNKS * sizeof(Partial); }

// logits [rows, vocab] with row stride ld; temperature and uniform may be null (all greedy);
// scratch: sprout_sample_scratch_bytes(rows) bytes, 16-byte aligned.
SPROUT_API int sprout_sample(const float* logits, int ld, const float* temperature, const float* uniform,
                             int* out, void* scratch, int rows, int vocab, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows > 0 && rows <= 65535 && vocab > 0 && ld >= vocab, "sample: bad sizes rows=%d vocab=%d ld=%d", rows, vocab, ld);
  SPROUT_REQUIRE(logits && out && status && scratch, "sample: null pointer");
  SPROUT_REQUIRE((temperature == nullptr) == (uniform == nullptr), "sample: temperature and uniform go together");
  sprout_launch(sample_partial_kernel, dim3(CHUNKS, rows), dim3(PART_THREADS), 0, stream, logits, ld, temperature, (Partial*)scratch, vocab);
  if (sprout_check_launch("sample_partial")) return 1;
  sprout_launch(sample_final_kernel, dim3(rows), dim3(FINAL_THREADS), 0, stream, logits, ld, temperature, uniform, (const Partial*)scratch, out, vocab, status);
  return sprout_check_launch("sample_final");
}

// ------------------------------------------------------------------ feeding a decode step's output back
// After a decode step on the device: every request's sampled token becomes its next input
// token, its position and cache length grow by one, and the tokens are recorded in row
// `*step_counter` of `history` ([max_steps, requests]); the counter then advances.  This lets
// several decode steps run back to back (or as one replayed CUDA graph) without the host.
__global__ void advance_decode_kernel(int* token_ids, int* positions, int* context_lens, const int* sampled,
                                      int* history, int* step_counter, int requests, int max_steps) {
  pdl_launch_dependents();
  pdl_wait();
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
  sprout_launch(advance_decode_kernel, dim3(1), dim3(1024), 0, stream, token_ids, positions, context_lens, sampled, history,
                step_counter, requests, max_steps);
  return sprout_check_launch("advance_decode");
}

// A decode step that is launched before the step before it has been read back takes its input
// tokens on the device: token_ids[r] = fed[rows[r]] where rows[r] >= 0 (the row of the step before
// that sampled this request's token; `fed` holds that step's tokens), else it keeps the token the
// host staged.  A token that is no valid id (a step that flagged a non-finite logit) becomes 0;
// the status word already tells.
__global__ void feed_tokens_kernel(int* token_ids, const int* rows, const int* fed, int requests, int fed_rows, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < requests) {
    const int row = rows[r];
    if (row >= 0 && row < fed_rows) {
      const int token = fed[row];
      token_ids[r] = token < 0 || token >= vocab ? 0 : token;
    }
  }
}

SPROUT_API int sprout_feed_tokens(int* token_ids, const int* rows, const int* fed, int requests, int fed_rows, int vocab,
                                  cudaStream_t stream) {
  SPROUT_REQUIRE(requests > 0 && fed_rows > 0 && vocab > 0, "feed_tokens: sizes must be positive");
  SPROUT_REQUIRE(token_ids && rows && fed, "feed_tokens: null pointer");
  sprout_launch(feed_tokens_kernel, dim3((requests + 255) / 256), dim3(256), 0, stream, token_ids, rows, fed, requests, fed_rows, vocab);
  return sprout_check_launch("feed_tokens");
}
