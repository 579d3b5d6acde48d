// Memory-bound kernels of the decoder step: embedding gather, RMSNorm,
// SwiGLU on an interleaved gate/up row, rotary position encoding fused with
// the append of keys and values into the paged cache.  All arithmetic is
// float32; the element type of activations (float or bfloat16) is a template
// parameter.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// x[t, :] = table[token[t], :] widened to float32 (the residual stream is float32).
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int hidden, int vocab, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int token = tokens[t];
  if (token < 0 || token >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_TOKEN);
    token = 0;
  }
  const TW* row = table + (size_t)token * hidden;
  float* dst = out + (size_t)t * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(row[i]);
}

SPROUT_API int sprout_embed(const void* table, int table_dtype, const int* tokens, float* out,
                            int num_tokens, int hidden, int vocab, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(num_tokens > 0 && hidden > 0 && vocab > 0, "embed: sizes must be positive");
  SPROUT_REQUIRE(table && tokens && out && status, "embed: null pointer");
  if (table_dtype == SPROUT_F32)
    sprout_launch(embed_kernel<float>, dim3(num_tokens), dim3(256), 0, stream, (const float*)table, tokens, out, hidden, vocab, status);
  else if (table_dtype == SPROUT_BF16)
    sprout_launch(embed_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(256), 0, stream, (const __nv_bfloat16*)table, tokens, out, hidden, vocab, status);
  else
    return sprout_fail("embed: unknown dtype %d", table_dtype);
  return sprout_check_launch("embed");
}

// ---------------------------------------------------------------- RMSNorm
// out[r, i] = (x[src(r), i] * rsqrt(mean(x^2) + eps)) * gain[i]; the normalised value is
// rounded to float32 before the gain multiplies it.  `rows`, when given, selects source rows
// (used to norm only the rows whose logits are wanted).
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               TO* __restrict__ out, const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const float* src = x + (size_t)(rows ? rows[r] : r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) { float v = src[i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float n = src[i] * scale;
    dst[i] = from_float<TO>(n * gain[i]);
  }
}

// Fast path for hidden sizes that are multiples of 4: 256 threads, each holding up to VEC float4
// of the row in registers between the sum of squares and the scaling (one read of x).
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ gain, TO* __restrict__ out,
                   const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, quads = hidden >> 2;
  const float4* src = (const float4*)(x + (size_t)(rows ? rows[r] : r) * hidden);
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    v[k] = i < quads ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < VEC; k++) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    if (i < quads) {
      const float4 g = ((const float4*)gain)[i];
      const float a = (v[k].x * scale) * g.x, b = (v[k].y * scale) * g.y, c = (v[k].z * scale) * g.z, d = (v[k].w * scale) * g.w;
      if (sizeof(TO) == 4) {
        ((float4*)dst)[i] = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        ((uint2*)dst)[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  }
}

// Many rows (a prefill): a warp per row, the row in registers, no block-wide barrier.
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ gain, TO* __restrict__ out,
                    const int* __restrict__ rows, int num_rows, int hidden, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), quads = hidden >> 2;
  if (r >= num_rows) return;
  const float4* src = (const float4*)(x + (size_t)(rows ? rows[r] : r) * hidden);
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = lane + k * 32;
    v[k] = i < quads ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < VEC; k++) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  TO* dst = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = lane + k * 32;
    if (i < quads) {
      const float4 g = ((const float4*)gain)[i];
      const float a = (v[k].x * scale) * g.x, b = (v[k].y * scale) * g.y, c = (v[k].z * scale) * g.z, d = (v[k].w * scale) * g.w;
      if (sizeof(TO) == 4) {
        ((float4*)dst)[i] = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        ((uint2*)dst)[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  }
}

// Which kernel runs.  A float32 output is the true 32-bit path, whose results must not depend on how
// many rows a call brings: there the choice follows the row length alone (a warp per row with the
// row in registers, or the block kernel with a block size fixed by the length), so a row's sum of
// squares is added up in the same order whether it comes alone or among two thousand.  For
// bfloat16 the choice also follows the number of rows (speed; the orders differ by rounding).
template <typename TO>
static void launch_rmsnorm(const float* x, const float* gain, TO* out, const int* rows, int num_rows, int hidden,
                           float eps, cudaStream_t stream) {
  const int quads = hidden / 4;
  const bool aligned = hidden % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const bool fixed_order = sizeof(TO) == 4;
  if (aligned && (num_rows >= 64 || fixed_order) && quads <= 512) {
    const dim3 grid((num_rows + 7) / 8);
    if (quads <= 128) sprout_launch(rmsnorm_warp_kernel<TO, 4>, grid, dim3(256), 0, stream, x, gain, out, rows, num_rows, hidden, eps);
    else if (quads <= 256) sprout_launch(rmsnorm_warp_kernel<TO, 8>, grid, dim3(256), 0, stream, x, gain, out, rows, num_rows, hidden, eps);
    else sprout_launch(rmsnorm_warp_kernel<TO, 16>, grid, dim3(256), 0, stream, x, gain, out, rows, num_rows, hidden, eps);
  }
  else if (aligned && !fixed_order && quads <= 256) sprout_launch(rmsnorm_vec_kernel<TO, 1>, dim3(num_rows), dim3(256), 0, stream, x, gain, out, rows, hidden, eps);
  else if (aligned && !fixed_order && quads <= 512) sprout_launch(rmsnorm_vec_kernel<TO, 2>, dim3(num_rows), dim3(256), 0, stream, x, gain, out, rows, hidden, eps);
  else if (aligned && quads <= 1024) sprout_launch(rmsnorm_vec_kernel<TO, 4>, dim3(num_rows), dim3(256), 0, stream, x, gain, out, rows, hidden, eps);
  else if (aligned && quads <= 2048) sprout_launch(rmsnorm_vec_kernel<TO, 8>, dim3(num_rows), dim3(256), 0, stream, x, gain, out, rows, hidden, eps);
  else sprout_launch(rmsnorm_kernel<TO>, dim3(num_rows), dim3(hidden >= 1024 ? 256 : 128), 0, stream, x, gain, out, rows, hidden, eps);
}

SPROUT_API int sprout_rmsnorm(const float* x, const float* gain, void* out, int out_dtype, const int* rows,
                              int num_rows, int hidden, float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(num_rows > 0 && hidden > 0, "rmsnorm: sizes must be positive");
  SPROUT_REQUIRE(x && gain && out, "rmsnorm: null pointer");
  SPROUT_REQUIRE(eps > 0.f, "rmsnorm: eps must be positive");
  if (out_dtype == SPROUT_F32) launch_rmsnorm<float>(x, gain, (float*)out, rows, num_rows, hidden, eps, stream);
  else if (out_dtype == SPROUT_BF16) launch_rmsnorm<__nv_bfloat16>(x, gain, (__nv_bfloat16*)out, rows, num_rows, hidden, eps, stream);
  else return sprout_fail("rmsnorm: unknown dtype %d", out_dtype);
  return sprout_check_launch("rmsnorm");
}

// ---------------------------------------------------------------- SwiGLU
// Input rows hold gate and up interleaved in blocks of `block`: columns [2 block b, 2 block b + block)
// are gate values block b .. block b + block - 1 and the next `block` columns the matching up values
// (block 8 for the tensor-core products' fused gate/up matrix; block == inter for a plain
// concatenation, gate first).  out = silu(gate) * up with the SiLU rounded to float32 first.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int tokens, int inter, int block) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)tokens * inter;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / inter), i = (int)(idx % inter);
    const T* row = gu + (size_t)t * 2 * inter;
    const int col = (i / block) * 2 * block + (i % block);
    const float g = to_float(row[col]), u = to_float(row[col + block]);
    const float s = g / (1.0f + expf(-g));
    out[idx] = from_float<T>(s * u);
  }
}

SPROUT_API int sprout_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter, int block, cudaStream_t stream) {
  SPROUT_REQUIRE(tokens > 0 && inter > 0, "swiglu: sizes must be positive");
  SPROUT_REQUIRE(block > 0 && inter % block == 0, "swiglu: the intermediate size must be a multiple of %d, the gate/up block (got %d)", block, inter);
  const size_t total = (size_t)tokens * inter;
  const size_t cap = (size_t)sprout_sm_count() * 16;
  const int blocks = (int)((total + 255) / 256 < cap ? (total + 255) / 256 : cap);
  if (dtype == SPROUT_F32)
    sprout_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, tokens, inter, block);
  else if (dtype == SPROUT_BF16)
    sprout_launch(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, tokens, inter, block);
  else
    return sprout_fail("swiglu: unknown dtype %d", dtype);
  return sprout_check_launch("swiglu");
}

// ---------------------------------------------------------------- rotary positions + cache append
// One block per token.  qkv rows hold [q heads | k heads | v heads].  q and k are rotated by
// the token's position; q is rotated in place, the rotated k and the unrotated v go to the
// token's slot of the paged cache:
//   page = block_table[seq, pos / page_tokens], slot = pos % page_tokens,
//   element ((page * kv_heads + head) * page_tokens + slot) * head_dim + d.
// The rotation takes the first `rotary_dim` elements of a head (head_dim: all of it) in pairs:
// half-split pairs (d, d + rotary_dim/2), or with `interleaved` pairs (2d, 2d + 1); pair d turns by
// the angle whose cosine and sine are cos/sin[pos, d].  The tables are float32
// [max_positions, rotary_dim/2]; the host fills them from float64 angles.  Elements beyond
// rotary_dim pass through.  A page id outside the pool sets a status bit and skips the write.
// With `acc` given, the projections come from there instead: float32 sums [tokens, width] that a
// split-K product accumulated, to which `bias` is added here; q is then written (rotated) to
// qkv, and every element of acc of the token is set back to zero for the next product (also when
// the token's position is refused).
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, float* acc, const float* __restrict__ bias,
                                   const int* __restrict__ positions,
                                   const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                                   int table_stride, const float* __restrict__ cos_table,
                                   const float* __restrict__ sin_table, int max_positions,
                                   T* __restrict__ k_cache, T* __restrict__ v_cache, int heads, int kv_heads,
                                   int head_dim, int rotary_dim, int interleaved, int page_tokens, int num_pages,
                                   int write_cache, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = head_dim >> 1, rot_half = rotary_dim >> 1;
  const int pos = positions[t];
  const bool rotate = cos_table != nullptr;   // no tables: no position encoding, q and k stay as projected
  const int width = (heads + 2 * kv_heads) * head_dim;
  float* acc_row = acc ? acc + (size_t)t * width : nullptr;
  if (pos < 0 || (rotate && pos >= max_positions)) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
    if (acc_row) for (int i = threadIdx.x; i < width; i += blockDim.x) acc_row[i] = 0.f;   // nothing stale for the next product
    return;
  }
  T* row = qkv + (size_t)t * width;
  const float* cs = rotate ? cos_table + (size_t)pos * rot_half : nullptr;
  const float* sn = rotate ? sin_table + (size_t)pos * rot_half : nullptr;
  int page = 0, slot = 0;
  bool page_ok = false;
  if (write_cache) {
    const int seq = seq_of_token[t];
    page = block_table[(size_t)seq * table_stride + pos / page_tokens];
    slot = pos % page_tokens;
    page_ok = page >= 0 && page < num_pages;
    if (!page_ok && threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
  }
  auto value = [&](int i) -> float {
    if (!acc_row) return to_float(row[i]);
    const float v = acc_row[i] + (bias ? bias[i] : 0.f);
    acc_row[i] = 0.f;
    return v;
  };
  // one thread per pair of a head's elements: the first rotary_dim/2 pairs are rotated, the others
  // (elements rotary_dim .. head_dim - 1, two by two) pass through; q heads in place, k heads into the cache
  for (int i = threadIdx.x; i < (heads + kv_heads) * half; i += blockDim.x) {
    const int h = i / half, d = i % half;
    const bool turned = rotate && d < rot_half;
    int e0, e1;
    if (d < rot_half) { e0 = interleaved ? 2 * d : d; e1 = interleaved ? 2 * d + 1 : d + rot_half; }
    else { e0 = rotary_dim + 2 * (d - rot_half); e1 = e0 + 1; }
    const float c = turned ? cs[d] : 1.f, s = turned ? sn[d] : 0.f;
    if (h < heads) {
      if (!turned && !acc_row) continue;
      const float a = value(h * head_dim + e0), b = value(h * head_dim + e1);
      T* x = row + h * head_dim;
      x[e0] = from_float<T>(a * c - b * s);
      x[e1] = from_float<T>(b * c + a * s);
    } else {
      const int kh = h - heads;
      const float a = value(h * head_dim + e0), b = value(h * head_dim + e1);
      if (page_ok) {
        T* dst = k_cache + (((size_t)page * kv_heads + kh) * page_tokens + slot) * head_dim;
        dst[e0] = from_float<T>(a * c - b * s);
        dst[e1] = from_float<T>(b * c + a * s);
      }
    }
  }
  if (page_ok || acc_row) {
    const int v0 = (heads + kv_heads) * head_dim;
    for (int i = threadIdx.x; i < kv_heads * head_dim; i += blockDim.x) {
      const int h = i / head_dim, d = i % head_dim;
      const T v = acc_row ? from_float<T>(value(v0 + i)) : row[v0 + i];
      if (page_ok) v_cache[(((size_t)page * kv_heads + h) * page_tokens + slot) * head_dim + d] = v;
    }
  }
}

// bfloat16 without float32 sums, head_dim a multiple of 16: a thread takes 8 consecutive elements
// of a head's first half with the matching 8 of its second half (16-byte loads and stores), or 8
// elements of a v head; the items of all tokens are spread over the grid.
__global__ void __launch_bounds__(256)
rope_append_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                       const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_stride,
                       const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_positions,
                       __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int num_tokens,
                       int heads, int kv_heads, int head_dim, int page_tokens, int num_pages, int write_cache,
                       int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = head_dim >> 1, half_chunks = half >> 3;
  const int rot_items = (heads + kv_heads) * half_chunks;        // rotated pairs of 8
  const int v_items = write_cache ? kv_heads * (head_dim >> 3) : 0;
  const int per_token = rot_items + v_items;
  const int width = (heads + 2 * kv_heads) * head_dim;
  const bool rotate = cos_table != nullptr;
  const long long total = (long long)num_tokens * per_token;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_token), item = (int)(idx % per_token);
    const int pos = positions[t];
    if (pos < 0 || (rotate && pos >= max_positions)) {
      if (item == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
      continue;
    }
    __nv_bfloat16* row = qkv + (size_t)t * width;
    int page = 0;
    bool page_ok = false;
    const bool to_cache = item >= heads * half_chunks;
    if (to_cache && write_cache) {
      page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_tokens];
      page_ok = page >= 0 && page < num_pages;
      if (!page_ok && item == heads * half_chunks) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    }
    const int slot = pos % page_tokens;
    if (item < rot_items) {
      const int h = item / half_chunks, d = (item % half_chunks) * 8;
      if (h < heads && !rotate) continue;                       // q stays as projected
      if (h >= heads && !page_ok) continue;
      const uint4 ra = *(const uint4*)(row + h * head_dim + d), rb = *(const uint4*)(row + h * head_dim + half + d);
      float c[8], sn[8];
      if (rotate) {
        const float4* cp = (const float4*)(cos_table + (size_t)pos * half + d);
        const float4* sp = (const float4*)(sin_table + (size_t)pos * half + d);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) { c[i] = 1.f; sn[i] = 0.f; }
      }
      const __nv_bfloat16* pa = (const __nv_bfloat16*)&ra;
      const __nv_bfloat16* pb = (const __nv_bfloat16*)&rb;
      uint4 oa, ob;
      __nv_bfloat16* qa = (__nv_bfloat16*)&oa;
      __nv_bfloat16* qb = (__nv_bfloat16*)&ob;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float a = __bfloat162float(pa[i]), b = __bfloat162float(pb[i]);
        qa[i] = __float2bfloat16_rn(a * c[i] - b * sn[i]);
        qb[i] = __float2bfloat16_rn(b * c[i] + a * sn[i]);
      }
      __nv_bfloat16* dst = h < heads ? row + h * head_dim
                                     : k_cache + (((size_t)page * kv_heads + (h - heads)) * page_tokens + slot) * head_dim;
      *(uint4*)(dst + d) = oa;
      *(uint4*)(dst + half + d) = ob;
    } else if (page_ok) {
      const int vi = item - rot_items, h = vi / (head_dim >> 3), d = (vi % (head_dim >> 3)) * 8;
      *(uint4*)(v_cache + (((size_t)page * kv_heads + h) * page_tokens + slot) * head_dim + d) =
          *(const uint4*)(row + (heads + kv_heads + h) * head_dim + d);
    }
  }
}

// The same from float32 sums (what a split-K product leaves) plus a bias: the sums are read as
// float4, cleared, rotated; q goes to qkv as bfloat16, k and v to the cache.
__global__ void __launch_bounds__(256)
rope_append_acc_vec_kernel(__nv_bfloat16* __restrict__ qkv, float* __restrict__ acc, const float* __restrict__ bias,
                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                           const int* __restrict__ block_table, int table_stride, const float* __restrict__ cos_table,
                           const float* __restrict__ sin_table, int max_positions, __nv_bfloat16* __restrict__ k_cache,
                           __nv_bfloat16* __restrict__ v_cache, int num_tokens, int heads, int kv_heads, int head_dim,
                           int page_tokens, int num_pages, int write_cache, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = head_dim >> 1, half_chunks = half >> 3;
  const int rot_items = (heads + kv_heads) * half_chunks;
  const int v_items = kv_heads * (head_dim >> 3);                // the v sums are cleared even when nothing is stored
  const int per_token = rot_items + v_items;
  const int width = (heads + 2 * kv_heads) * head_dim;
  const bool rotate = cos_table != nullptr;
  const long long total = (long long)num_tokens * per_token;
  auto take8 = [&](float* src, const float* b, float (&v)[8]) {   // sums + bias, and the sums cleared
    const float4 lo = ((const float4*)src)[0], hi = ((const float4*)src)[1];
    ((float4*)src)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    ((float4*)src)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    if (b) {
      const float4 blo = ((const float4*)b)[0], bhi = ((const float4*)b)[1];
      v[0] += blo.x; v[1] += blo.y; v[2] += blo.z; v[3] += blo.w; v[4] += bhi.x; v[5] += bhi.y; v[6] += bhi.z; v[7] += bhi.w;
    }
  };
  auto pack8 = [](const float (&v)[8]) {
    uint4 o;
    __nv_bfloat16* q = (__nv_bfloat16*)&o;
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __float2bfloat16_rn(v[i]);
    return o;
  };
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / per_token), item = (int)(idx % per_token);
    const int pos = positions[t];
    float* acc_row = acc + (size_t)t * width;
    if (pos < 0 || (rotate && pos >= max_positions)) {
      if (item == 0) {
        atomicOr(status, SPROUT_STATUS_BAD_POSITION);
        for (int i = 0; i < width; i += 4) *(float4*)(acc_row + i) = make_float4(0.f, 0.f, 0.f, 0.f);   // nothing stale for the next product
      }
      continue;
    }
    int page = 0;
    bool page_ok = false;
    const bool to_cache = item >= heads * half_chunks;
    if (to_cache && write_cache) {
      page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_tokens];
      page_ok = page >= 0 && page < num_pages;
      if (!page_ok && item == heads * half_chunks) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    }
    const int slot = pos % page_tokens;
    if (item < rot_items) {
      const int h = item / half_chunks, d = (item % half_chunks) * 8;
      float a[8], b[8];
      take8(acc_row + h * head_dim + d, bias ? bias + h * head_dim + d : nullptr, a);
      take8(acc_row + h * head_dim + half + d, bias ? bias + h * head_dim + half + d : nullptr, b);
      if (h >= heads && !page_ok) continue;
      float ra[8], rb[8];
      if (rotate) {
        const float4* cp = (const float4*)(cos_table + (size_t)pos * half + d);
        const float4* sp = (const float4*)(sin_table + (size_t)pos * half + d);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int i = 0; i < 8; i++) { ra[i] = a[i] * c[i] - b[i] * sn[i]; rb[i] = b[i] * c[i] + a[i] * sn[i]; }
      } else {
#pragma unroll
        for (int i = 0; i < 8; i++) { ra[i] = a[i]; rb[i] = b[i]; }
      }
      __nv_bfloat16* dst = h < heads ? qkv + (size_t)t * width + h * head_dim
                                     : k_cache + (((size_t)page * kv_heads + (h - heads)) * page_tokens + slot) * head_dim;
      *(uint4*)(dst + d) = pack8(ra);
      *(uint4*)(dst + half + d) = pack8(rb);
    } else {
      const int vi = item - rot_items, h = vi / (head_dim >> 3), d = (vi % (head_dim >> 3)) * 8;
      float v[8];
      const int col = (heads + kv_heads + h) * head_dim + d;
      take8(acc_row + col, bias ? bias + col : nullptr, v);
      if (page_ok) *(uint4*)(v_cache + (((size_t)page * kv_heads + h) * page_tokens + slot) * head_dim + d) = pack8(v);
    }
  }
}

// rotary_dim: how many leading elements of a head are rotated (even, at most head_dim; the tables are
// [max_positions, rotary_dim / 2]); interleaved: pairs (2d, 2d + 1) instead of (d, d + rotary_dim / 2).
SPROUT_API int sprout_rope_append(void* qkv, float* acc, const float* bias, int dtype, const int* positions, const int* seq_of_token,
                                  const int* block_table, int table_stride, const float* cos_table,
                                  const float* sin_table, int max_positions, void* k_cache, void* v_cache,
                                  int num_tokens, int heads, int kv_heads, int head_dim, int rotary_dim, int interleaved,
                                  int page_tokens, int num_pages, int write_cache, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(num_tokens > 0 && heads > 0 && kv_heads > 0 && page_tokens > 0 && num_pages > 0,
                 "rope_append: sizes must be positive");
  SPROUT_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "rope_append: head_dim must be even (got %d)", head_dim);
  SPROUT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim,
                 "rope_append: rotary_dim must be even and at most head_dim (got %d of %d)", rotary_dim, head_dim);
  SPROUT_REQUIRE(qkv && positions && seq_of_token && block_table && status, "rope_append: null pointer");
  SPROUT_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "rope_append: cos and sin tables go together");
  SPROUT_REQUIRE(!write_cache || (k_cache && v_cache), "rope_append: cache pointers missing");
  const int pairs = (heads + kv_heads) * (head_dim / 2);
  const int threads = pairs >= 1024 ? 1024 : (pairs + 31) / 32 * 32;
  const bool aligned = ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
                       ((uintptr_t)cos_table & 15) == 0 && ((uintptr_t)sin_table & 15) == 0;
  // the 16-byte kernels are written for the whole head in half-split pairs (or no rotation at all)
  const bool plain_pairs = !cos_table || (rotary_dim == head_dim && !interleaved);
  if (dtype == SPROUT_BF16 && acc && plain_pairs && head_dim % 16 == 0 && aligned && ((uintptr_t)acc & 15) == 0 && ((uintptr_t)bias & 15) == 0 &&
      num_tokens >= 16) {
    const long long items = (long long)num_tokens * ((heads + kv_heads) * (head_dim / 16) + kv_heads * (head_dim / 8));
    const long long cap = (long long)sprout_sm_count() * 8;
    const int blocks = (int)((items + 255) / 256 < cap ? (items + 255) / 256 : cap);
    sprout_launch(rope_append_acc_vec_kernel, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)qkv, acc, bias, positions,
        seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions, (__nv_bfloat16*)k_cache,
        (__nv_bfloat16*)v_cache, num_tokens, heads, kv_heads, head_dim, page_tokens, num_pages, write_cache, status);
    return sprout_check_launch("rope_append");
  }
  if (dtype == SPROUT_BF16 && !acc && plain_pairs && head_dim % 16 == 0 && aligned && num_tokens >= 64) {
    const long long items = (long long)num_tokens * ((heads + kv_heads) * (head_dim / 16) + kv_heads * (head_dim / 8));
    const long long cap = (long long)sprout_sm_count() * 8;
    const int blocks = (int)((items + 255) / 256 < cap ? (items + 255) / 256 : cap);
    sprout_launch(rope_append_vec_kernel, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)qkv, positions, seq_of_token,
        block_table, table_stride, cos_table, sin_table, max_positions, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
        num_tokens, heads, kv_heads, head_dim, page_tokens, num_pages, write_cache, status);
    return sprout_check_launch("rope_append");
  }
  if (dtype == SPROUT_F32)
    sprout_launch(rope_append_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream,
        (float*)qkv, acc, bias, positions, seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions,
        (float*)k_cache, (float*)v_cache, heads, kv_heads, head_dim, rotary_dim, interleaved, page_tokens, num_pages,
        write_cache, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(rope_append_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
        (__nv_bfloat16*)qkv, acc, bias, positions, seq_of_token, block_table, table_stride, cos_table, sin_table,
        max_positions, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, heads, kv_heads, head_dim, rotary_dim, interleaved,
        page_tokens, num_pages, write_cache, status);
  else
    return sprout_fail("rope_append: unknown dtype %d", dtype);
  return sprout_check_launch("rope_append");
}
