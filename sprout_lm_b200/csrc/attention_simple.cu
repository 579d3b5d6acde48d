// Paged causal attention, one block per (token, query head), float32 arithmetic throughout.
// It is the attention of the true 32-bit path and the plain device reference for the
// tensor-core attention kernels.  Query token t of sequence r, at position pos, attends the
// keys at positions 0..pos of r, found through r's block table; query head h reads key/value
// head h / (heads / kv_heads).  Keys are walked in chunks of 128 aligned to absolute position
// with a running maximum and sum, so the operations done for a query do not depend on how
// the tokens were cut into steps or on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int CHUNK = 128;   // keys per pass == threads per block

template <typename T>
__global__ void __launch_bounds__(CHUNK)
attention_simple_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                        const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        T* __restrict__ out, int out_stride, int heads, int kv_heads, int head_dim,
                        int page_tokens, int num_pages, int* status) {
  extern __shared__ float smem[];
  float* qs = smem;                       // head_dim
  float* probs = qs + head_dim;           // CHUNK
  float* scratch = probs + CHUNK;         // 33
  long long* row_offset = (long long*)(scratch + 34);   // CHUNK (8-byte aligned: sizes below are even)

  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (heads / kv_heads);
  const int seq = seq_of_token[t];
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq * table_stride;

  for (int d = tid; d < head_dim; d += CHUNK) qs[d] = to_float(q[(size_t)t * q_stride + h * head_dim + d]);
  __syncthreads();

  const float root = sqrtf((float)head_dim);
  float m_run = -INFINITY, l_run = 0.f;
  float acc0 = 0.f, acc1 = 0.f;           // output dims tid and tid + CHUNK

  for (int base = 0; base <= pos; base += CHUNK) {
    const int p = base + tid;
    bool valid = p <= pos;
    long long offset = 0;
    if (valid) {
      const int page = table[p / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, SPROUT_STATUS_BAD_PAGE);
        valid = false;
      } else {
        offset = (((long long)page * kv_heads + g) * page_tokens + (p % page_tokens)) * head_dim;
      }
    }
    float s = -INFINITY;
    if (valid) {
      const T* key = k_cache + offset;
      float dot = 0.f;
      for (int d = 0; d < head_dim; d++) dot = fmaf(qs[d], to_float(key[d]), dot);
      s = dot / root;
    }
    row_offset[tid] = valid ? offset : -1;
    const float c_max = block_max(s, scratch);
    const float m_new = fmaxf(m_run, c_max);
    const float e = valid ? expf(s - m_new) : 0.f;
    probs[tid] = e;
    const float c_sum = block_sum(e, scratch);   // has barriers: probs and row_offset are visible after it
    const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    l_run = l_run * alpha + c_sum;
    acc0 *= alpha;
    acc1 *= alpha;
    const int count = min(CHUNK, pos - base + 1);
    if (tid < head_dim) {
      for (int j = 0; j < count; j++) {
        const long long off = row_offset[j];
        if (off >= 0) acc0 = fmaf(probs[j], to_float(v_cache[off + tid]), acc0);
      }
    }
    if (tid + CHUNK < head_dim) {
      for (int j = 0; j < count; j++) {
        const long long off = row_offset[j];
        if (off >= 0) acc1 = fmaf(probs[j], to_float(v_cache[off + tid + CHUNK]), acc1);
      }
    }
    m_run = m_new;
    __syncthreads();
  }
  T* dst = out + (size_t)t * out_stride + h * head_dim;
  if (tid < head_dim) dst[tid] = from_float<T>(acc0 / l_run);
  if (tid + CHUNK < head_dim) dst[tid + CHUNK] = from_float<T>(acc1 / l_run);
}

}  // namespace

SPROUT_API int sprout_attention_simple(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                       const int* block_table, int table_stride, const int* seq_of_token,
                                       const int* positions, void* out, int out_stride, int dtype,
                                       int num_tokens, int heads, int kv_heads, int head_dim, int page_tokens,
                                       int num_pages, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(num_tokens > 0 && heads > 0 && kv_heads > 0 && page_tokens > 0 && num_pages > 0,
                 "attention_simple: sizes must be positive");
  SPROUT_REQUIRE(heads % kv_heads == 0, "attention_simple: heads (%d) must be a multiple of kv_heads (%d)", heads, kv_heads);
  SPROUT_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && head_dim <= 2 * CHUNK,
                 "attention_simple: head_dim must be even and at most %d (got %d)", 2 * CHUNK, head_dim);
  SPROUT_REQUIRE(heads <= 65535, "attention_simple: too many heads (%d)", heads);
  SPROUT_REQUIRE(q && k_cache && v_cache && block_table && seq_of_token && positions && out && status,
                 "attention_simple: null pointer");
  const size_t smem = (size_t)(head_dim + CHUNK + 34) * sizeof(float) + CHUNK * sizeof(long long);
  dim3 grid(num_tokens, heads);
  if (dtype == SPROUT_F32)
    sprout_launch(attention_simple_kernel<float>, grid, dim3(CHUNK), smem, stream, 
        (const float*)q, q_stride, (const float*)k_cache, (const float*)v_cache, block_table, table_stride,
        seq_of_token, positions, (float*)out, out_stride, heads, kv_heads, head_dim, page_tokens, num_pages, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(attention_simple_kernel<__nv_bfloat16>, grid, dim3(CHUNK), smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache,
        block_table, table_stride, seq_of_token, positions, (__nv_bfloat16*)out, out_stride, heads, kv_heads,
        head_dim, page_tokens, num_pages, status);
  else
    return sprout_fail("attention_simple: unknown dtype %d", dtype);
  return sprout_check_launch("attention_simple");
}
