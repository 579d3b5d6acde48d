// Decode attention with the whole context of a (request, key/value head) resident in shared memory.
//
// One CTA serves one request and one key/value head with all the query heads of its group.  All
// the request's cached keys and values of that head (up to `cap_keys`, a few hundred) are
// fetched by TMA, one box per cache page, into shared memory in one go: every copy is in flight
// at once, and they are requested before the wait for the step's earlier kernels, because the
// keys and values of earlier positions were written by earlier steps.  So the bytes stream while
// the projection before this kernel still runs, and after the wait only the new token's own
// work is left: its query (and, in the fused form, its key and value) from the float32 sums of
// the q/k/v product, then S = Q K^T, the softmax and O = P V on `mma.sync.m16n8k16` with the
// group's query heads as the 16 rows of the tile.  Eight warps take the keys in blocks of 32,
// each with a running maximum and sum; their partial results meet in shared memory.  No split
// across CTAs, no cluster, no second kernel: the chain after the wait is one CTA's.
//
// A page of one head is `page_tokens` contiguous rows of the cache, so a box is [page_tokens
// rows, 64 columns] with the 128-byte swizzle (two boxes per page for head size 128); the pages
// lie one after the other in shared memory, and a key's row is found there by its position
// alone.  Copies complete on one mbarrier per 128 keys, so the first warps start while later
// keys still arrive.
//
// Takes head sizes 64 and 128, pages of 8 to 128 tokens (a power of two), up to 16 query heads
// per key/value head and contexts up to `cap_keys` (what fits in shared memory: 768 keys of
// head size 64, 384 of 128); the split-key kernels (attention_decode_mma.cuh, attention_bf16.cu) take everything else.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA leaves
// once its copies have landed or their wait has run out too.
#include <cuda_bf16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int RES_THREADS = 256;          // 8 warps
constexpr int RES_WARPS = 8;
constexpr int RES_MAX_CHUNKS = 8;         // mbarriers: one per 128 keys
constexpr int RES_SMEM_LIMIT = 227 * 1024 - 1024;

struct ResidentParams {
  const __nv_bfloat16* q; int q_stride;     // not fused: the queries [requests, heads * head_dim]
  __nv_bfloat16* k_cache; __nv_bfloat16* v_cache;
  const int* block_table; int table_stride;
  const int* context_lens;
  __nv_bfloat16* out; int out_stride;
  int heads, kv_heads, page_shift, num_pages, cap_keys;
  int* status;
  // fused projection tail: float32 sums [requests, (heads + 2 kv_heads) * head_dim] of the q/k/v
  // product for each request's new token (position context_lens - 1), their bias, the rotation
  float* acc; const float* bias; const float* cos_table; const float* sin_table; int max_positions, rotary_dim, interleaved;
  // sums of a product whose normalised input went without its scale: rows before the norm [requests, norm_width];
  // request r's sums are multiplied by 1 / sqrt(mean(norm_x[r]^2) + norm_eps).  Null: no scale.
  const float* norm_x; int norm_width; float norm_eps;
};

__device__ __forceinline__ void res_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void res_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void res_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t res_pack(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}

// Byte offset, inside the K (or V) region, of 16-byte chunk `chunk` (0 .. HD/8 - 1) of the key at
// position `key`: pages one after the other, a page as HD/64 swizzled tiles of [page_tokens rows,
// 128 bytes].
template <int HD>
__device__ __forceinline__ uint32_t res_offset(int key, int chunk, int page_shift) {
  const int page = key >> page_shift, row = key & ((1 << page_shift) - 1);
  const uint32_t page_bytes = (uint32_t)HD * 2u << page_shift;
  return (uint32_t)page * page_bytes + (uint32_t)(chunk >> 3) * (128u << page_shift) + (uint32_t)row * 128u +
         (uint32_t)(((chunk & 7) ^ (row & 7)) << 4);
}

template <int HD, bool FUSED>
__global__ void __launch_bounds__(RES_THREADS, 1)
attention_decode_resident_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                 const ResidentParams p) {
  constexpr int STRIDE = HD + 8, CHUNKS = HD / 8;
  extern __shared__ uint8_t res_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)res_raw + 1023) & ~(uintptr_t)1023);
  const uint32_t kv_bytes = (uint32_t)p.cap_keys * HD * 2;
  uint8_t* sK = smem;
  uint8_t* sV = smem + kv_bytes;
  __nv_bfloat16* sQ = (__nv_bfloat16*)(sV + kv_bytes);       // [16][STRIDE]
  float* wm = (float*)(sQ + 16 * STRIDE);                    // [8 warps][16 rows] running maxima
  float* wl = wm + RES_WARPS * 16;                           // [8][16] sums
  uint64_t* bars = (uint64_t*)(wl + RES_WARPS * 16);         // [RES_MAX_CHUNKS]
  __shared__ int s_failed;
  __shared__ float s_norm[RES_WARPS];

  pdl_launch_dependents();
  SPROUT_TL_ENTRY(0);
  const int g = blockIdx.x, r = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = p.heads / p.kv_heads;
  const int page_tokens = 1 << p.page_shift;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  const int len = p.context_lens[r];
  const int width = (p.heads + 2 * p.kv_heads) * HD;
  const int pos = len - 1;
  const float scale = 1.0f / sqrtf((float)HD);
  const bool usable = len > 0 && len <= p.cap_keys;
  const int chunks = usable ? (len + 127) >> 7 : 0;
  const int pages = usable ? (len + page_tokens - 1) >> p.page_shift : 0;

  if (tid == 0) {
    s_failed = 0;
    for (int c = 0; c < RES_MAX_CHUNKS; c++) mbar_init(&bars[c], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (!usable) atomicOr(p.status, SPROUT_STATUS_BAD_LAYOUT);     // a context beyond what this launch has room for
  }
  __syncthreads();

  // ---- all the pages' copies, before the wait for the step's earlier kernels
  if (warp == 0 && usable) {
    const uint32_t page_bytes = (uint32_t)HD * 2u << p.page_shift;
    const int pages_per_chunk = 128 >> p.page_shift;
    if (lane < chunks) {
      const int first = lane * pages_per_chunk;
      const int count = min(pages, first + pages_per_chunk) - first;
      mbar_expect_tx(&bars[lane], (uint32_t)count * page_bytes * 2u);
    }
    __syncwarp();
    for (int i = lane; i < pages; i += 32) {
      int page = table[i];
      if (page < 0 || page >= p.num_pages) { atomicOr(p.status, SPROUT_STATUS_BAD_PAGE); page = 0; }   // flagged; the copy still completes
      const int row0 = (page * p.kv_heads + g) << p.page_shift;
      uint64_t* bar = &bars[(i << p.page_shift) >> 7];
#pragma unroll
      for (int a = 0; a < HD / 64; a++) {
        tma_load_2d(sK + (size_t)i * page_bytes + a * (128u << p.page_shift), &map_k, bar, a * 64, row0);
        tma_load_2d(sV + (size_t)i * page_bytes + a * (128u << p.page_shift), &map_v, bar, a * 64, row0);
      }
    }
  }

  pdl_wait();
  SPROUT_TL_WAITED(0);
  if (!usable) return;                                         // nothing was issued

  // ---- the new token: its query rows, and (fused) its key and value
  const bool rotate = FUSED && p.cos_table != nullptr;
  float inv_rms = 1.0f;
  if (FUSED && p.norm_x) {
    const float* xr = p.norm_x + (size_t)r * p.norm_width;
    float ss = 0.f;
    for (int i = tid; i < p.norm_width; i += RES_THREADS) { const float v = __ldcg(xr + i); ss += v * v; }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
    if (lane == 0) s_norm[warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < RES_WARPS; w2++) total += s_norm[w2];
    inv_rms = 1.0f / sqrtf(total / (float)p.norm_width + p.norm_eps);
  }
  // (fused) the new token's key pair and value element of this thread: read now, with the q sums, not
  // after the copies have landed (one trip to L2 less on the way to the first product)
  float new_k0 = 0.f, new_k1 = 0.f, new_kb0 = 0.f, new_kb1 = 0.f, new_cos = 1.f, new_sin = 0.f, new_v = 0.f, new_vb = 0.f;
  int new_page = -1;
  if (FUSED) {
    constexpr int HALF = HD / 2;
    const int rot_half = p.rotary_dim >> 1;
    const int safe = min(pos, max(p.max_positions - 1, 0));
    const float* k_acc = p.acc + (size_t)r * width + (p.heads + g) * HD;
    const float* v_acc = p.acc + (size_t)r * width + (p.heads + p.kv_heads + g) * HD;
    new_page = table[pos >> p.page_shift];
    if (tid < HALF) {
      const int d = tid;
      const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
      const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
      new_k0 = k_acc[e0]; new_k1 = k_acc[e1];
      if (p.bias) { new_kb0 = p.bias[(p.heads + g) * HD + e0]; new_kb1 = p.bias[(p.heads + g) * HD + e1]; }
      if (rotate && d < rot_half) { new_cos = p.cos_table[(size_t)safe * rot_half + d]; new_sin = p.sin_table[(size_t)safe * rot_half + d]; }
    }
    if (tid < HD) {
      new_v = v_acc[tid];
      if (p.bias) new_vb = p.bias[(p.heads + p.kv_heads + g) * HD + tid];
    }
  }
  if (FUSED) {
    if (rotate && pos >= p.max_positions) { if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_POSITION); }
    const int safe = min(pos, max(p.max_positions - 1, 0));
    constexpr int HALF = HD / 2;
    const int rot_half = p.rotary_dim >> 1;
    const float* sums = p.acc + (size_t)r * width + (size_t)g * group * HD;
    const float* bias = p.bias ? p.bias + (size_t)g * group * HD : nullptr;
    for (int idx = tid; idx < group * HALF; idx += RES_THREADS) {
      const int row = idx / HALF, d = idx % HALF;
      const bool turned = rotate && d < rot_half;
      const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
      const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
      const float a = sums[row * HD + e0] * inv_rms + (bias ? bias[row * HD + e0] : 0.f);
      const float b = sums[row * HD + e1] * inv_rms + (bias ? bias[row * HD + e1] : 0.f);
      const float c = turned ? p.cos_table[(size_t)safe * rot_half + d] : 1.f, sn = turned ? p.sin_table[(size_t)safe * rot_half + d] : 0.f;
      sQ[row * STRIDE + e0] = __float2bfloat16_rn(a * c - b * sn);
      sQ[row * STRIDE + e1] = __float2bfloat16_rn(b * c + a * sn);
    }
    for (int idx = group * CHUNKS + tid; idx < 16 * CHUNKS; idx += RES_THREADS)      // the tile's unused rows
      *(uint4*)(sQ + (idx / CHUNKS) * STRIDE + (idx % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
  } else {
    for (int idx = tid; idx < 16 * CHUNKS; idx += RES_THREADS) {
      const int row = idx / CHUNKS, c = idx % CHUNKS;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (row < group) v = *(const uint4*)(p.q + (size_t)r * p.q_stride + (size_t)(g * group + row) * HD + c * 8);
      *(uint4*)(sQ + row * STRIDE + c * 8) = v;
    }
  }
  // The last 128 keys' copies must have landed before anything is written over them: the new
  // token's row (which the early copy brought as it lay in the cache before this step) and the
  // rows beyond the context.
  if (!mbar_wait(&bars[chunks - 1], 0)) s_failed = 1;
  __syncthreads();
  if (s_failed) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT);
    if (warp == 0) for (int c = lane; c < chunks - 1; c += 32) mbar_wait(&bars[c], 0);   // copies in flight still write this CTA's memory
    return;
  }
  {
    const int page = FUSED ? new_page : table[pos >> p.page_shift];
    const bool page_ok = page >= 0 && page < p.num_pages;
    const long long dst = page_ok ? (((long long)page * p.kv_heads + g) * page_tokens + (pos & (page_tokens - 1))) * HD : 0;
    if (FUSED) {
      constexpr int HALF = HD / 2;
      const int rot_half = p.rotary_dim >> 1;
      float* k_acc = p.acc + (size_t)r * width + (p.heads + g) * HD;
      float* v_acc = p.acc + (size_t)r * width + (p.heads + p.kv_heads + g) * HD;
      if (tid < HALF) {
        const int d = tid;
        const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
        const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
        const float a = new_k0 * inv_rms + new_kb0, b = new_k1 * inv_rms + new_kb1;
        k_acc[e0] = 0.f; k_acc[e1] = 0.f;
        const __nv_bfloat16 lo = __float2bfloat16_rn(a * new_cos - b * new_sin), hi = __float2bfloat16_rn(b * new_cos + a * new_sin);
        *(__nv_bfloat16*)(sK + res_offset<HD>(pos, e0 >> 3, p.page_shift) + (e0 & 7) * 2) = lo;
        *(__nv_bfloat16*)(sK + res_offset<HD>(pos, e1 >> 3, p.page_shift) + (e1 & 7) * 2) = hi;
        if (page_ok) { p.k_cache[dst + e0] = lo; p.k_cache[dst + e1] = hi; }
      }
      if (tid < HD) {
        const __nv_bfloat16 v = __float2bfloat16_rn(new_v * inv_rms + new_vb);
        v_acc[tid] = 0.f;
        *(__nv_bfloat16*)(sV + res_offset<HD>(pos, tid >> 3, p.page_shift) + (tid & 7) * 2) = v;
        if (page_ok) p.v_cache[dst + tid] = v;
      }
    } else if (page_ok) {
      // the newest position's key and value were appended by a kernel of this step, after the early copies
      for (int c = tid; c < 2 * CHUNKS; c += RES_THREADS) {
        const int cc = c % CHUNKS;
        if (c < CHUNKS) *(uint4*)(sK + res_offset<HD>(pos, cc, p.page_shift)) = *(const uint4*)(p.k_cache + dst + cc * 8);
        else *(uint4*)(sV + res_offset<HD>(pos, cc, p.page_shift)) = *(const uint4*)(p.v_cache + dst + cc * 8);
      }
    }
    // value rows beyond the context, up to the end of the last block of 32 keys: whatever lies there
    // (the rest of a page that another request used before, or nothing this CTA has written) would
    // meet probability zero, and zero times a non-finite value is not zero
    const int beyond = ((len + 31) & ~31) - len;
    for (int idx = tid; idx < beyond * CHUNKS; idx += RES_THREADS)
      *(uint4*)(sV + res_offset<HD>(len + idx / CHUNKS, idx % CHUNKS, p.page_shift)) = make_uint4(0, 0, 0, 0);
  }
  __syncthreads();

  // ---- each warp takes every eighth block of 32 keys
  const int gr = lane >> 2, qc = lane & 3;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kk = 0; kk < HD / 16; kk++)
    res_ldmatrix_x4(qf[kk], smem_u32(sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + kk * 16 + (lane >> 4) * 8));
  const uint32_t k_base = smem_u32(sK), v_base = smem_u32(sV);
  bool ok = true;
  for (int key0 = warp * 32; key0 < len; key0 += RES_WARPS * 32) {
    if (!mbar_wait(&bars[key0 >> 7], 0)) { ok = false; break; }
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
      for (int n2 = 0; n2 < 2; n2++) {
        uint32_t b[4];
        res_ldmatrix_x4(b, k_base + res_offset<HD>(key0 + n2 * 16 + (lane & 7) + (lane >> 4) * 8, kk * 2 + ((lane >> 3) & 1), p.page_shift));
        res_mma(s[2 * n2], qf[kk], b[0], b[1]);
        res_mma(s[2 * n2 + 1], qf[kk], b[2], b[3]);
      }
    }
    float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int k = key0 + i * 8 + qc * 2;
      s[i][0] = k < len ? s[i][0] * scale : -INFINITY;
      s[i][1] = k + 1 < len ? s[i][1] * scale : -INFINITY;
      s[i][2] = k < len ? s[i][2] * scale : -INFINITY;
      s[i][3] = k + 1 < len ? s[i][3] * scale : -INFINITY;
      t0 = fmaxf(t0, fmaxf(s[i][0], s[i][1]));
      t1 = fmaxf(t1, fmaxf(s[i][2], s[i][3]));
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);       // finite: key0 < len, so every row has a key
    const float alpha0 = m0 == -INFINITY ? 0.f : __expf(m0 - n0), alpha1 = m1 == -INFINITY ? 0.f : __expf(m1 - n1);
    m0 = n0; m1 = n1;
    l0 *= alpha0; l1 *= alpha1;
#pragma unroll
    for (int i = 0; i < HD / 8; i++) { o[i][0] *= alpha0; o[i][1] *= alpha0; o[i][2] *= alpha1; o[i][3] *= alpha1; }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      s[i][0] = __expf(s[i][0] - n0); s[i][1] = __expf(s[i][1] - n0);
      s[i][2] = __expf(s[i][2] - n1); s[i][3] = __expf(s[i][3] - n1);
      l0 += s[i][0] + s[i][1];
      l1 += s[i][2] + s[i][3];
    }
#pragma unroll
    for (int kk = 0; kk < 2; kk++) {
      uint32_t a[4];
      a[0] = res_pack(s[2 * kk][0], s[2 * kk][1]);
      a[1] = res_pack(s[2 * kk][2], s[2 * kk][3]);
      a[2] = res_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = res_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < HD / 16; d2++) {
        uint32_t b[4];
        res_ldmatrix_x4_trans(b, v_base + res_offset<HD>(key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, d2 * 2 + (lane >> 4), p.page_shift));
        res_mma(o[2 * d2], a, b[0], b[1]);
        res_mma(o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
  }
  if (!ok) s_failed = 1;

  // ---- the warps' partial results meet in shared memory (over the keys, which are done with), in
  //      the layout the MMA left them in: a lane holds the same (row, column) places in every warp
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  if (s_failed) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT);
    if (warp == 0) for (int c = lane; c < chunks; c += 32) mbar_wait(&bars[c], 0);
    return;
  }
  float4* frag = (float4*)sK;                          // [8 warps][HD / 8 column blocks][32 lanes]
  {
    float4* mine = frag + warp * (HD / 8) * 32 + lane;
#pragma unroll
    for (int i = 0; i < HD / 8; i++) mine[i * 32] = make_float4(o[i][0], o[i][1], o[i][2], o[i][3]);
    if (qc == 0) {
      wm[warp * 16 + gr] = m0; wm[warp * 16 + gr + 8] = m1;
      wl[warp * 16 + gr] = l0; wl[warp * 16 + gr + 8] = l1;
    }
  }
  __syncthreads();
  {
    float wa[RES_WARPS], wb[RES_WARPS];                // the warps' weights for rows gr and gr + 8
    float ma = -INFINITY, mb = -INFINITY, la = 0.f, lb = 0.f;
#pragma unroll
    for (int w = 0; w < RES_WARPS; w++) { wa[w] = wm[w * 16 + gr]; wb[w] = wm[w * 16 + gr + 8]; ma = fmaxf(ma, wa[w]); mb = fmaxf(mb, wb[w]); }
#pragma unroll
    for (int w = 0; w < RES_WARPS; w++) {
      wa[w] = wa[w] == -INFINITY ? 0.f : __expf(wa[w] - ma);
      wb[w] = wb[w] == -INFINITY ? 0.f : __expf(wb[w] - mb);
      la += wl[w * 16 + gr] * wa[w];
      lb += wl[w * 16 + gr + 8] * wb[w];
    }
    const bool row_a = gr < group, row_b = gr + 8 < group;
    const float inv_a = 1.0f / la, inv_b = 1.0f / lb;
    for (int i = warp; i < HD / 8; i += RES_WARPS) {
      float xa = 0.f, ya = 0.f, xb = 0.f, yb = 0.f;
#pragma unroll
      for (int w = 0; w < RES_WARPS; w++) {
        const float4 f = frag[(w * (HD / 8) + i) * 32 + lane];
        xa += f.x * wa[w]; ya += f.y * wa[w]; xb += f.z * wb[w]; yb += f.w * wb[w];
      }
      const int d = i * 8 + qc * 2;
      if (row_a) {
        const int head = g * group + gr;
        *(__nv_bfloat162*)(p.out + (size_t)r * p.out_stride + (size_t)head * HD + d) = __floats2bfloat162_rn(xa * inv_a, ya * inv_a);
        if (FUSED) *(float2*)(p.acc + (size_t)r * width + (size_t)head * HD + d) = make_float2(0.f, 0.f);   // this CTA alone read these q sums
      }
      if (row_b) {
        const int head = g * group + gr + 8;
        *(__nv_bfloat162*)(p.out + (size_t)r * p.out_stride + (size_t)head * HD + d) = __floats2bfloat162_rn(xb * inv_b, yb * inv_b);
        if (FUSED) *(float2*)(p.acc + (size_t)r * width + (size_t)head * HD + d) = make_float2(0.f, 0.f);
      }
    }
  }
  SPROUT_TL_EXIT(0);
}

size_t resident_smem_bytes(int head_dim, int cap_keys) {
  return (size_t)2 * cap_keys * head_dim * 2 + (size_t)16 * (head_dim + 8) * 2 + (size_t)2 * RES_WARPS * 16 * 4 +
         RES_MAX_CHUNKS * 8 + 1024 /* room to start the pages on a 1024-byte boundary */;
}

template <int HD, bool FUSED>
int launch_resident(const CUtensorMap& map_k, const CUtensorMap& map_v, const ResidentParams& p, int requests, cudaStream_t stream) {
  const size_t smem = resident_smem_bytes(HD, p.cap_keys);
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_decode_resident_kernel<HD, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, RES_SMEM_LIMIT);
    if (err != cudaSuccess) return sprout_fail("attention_decode_resident: cannot reserve shared memory: %s", cudaGetErrorString(err));
    cudaFuncSetAttribute(attention_decode_resident_kernel<HD, FUSED>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = RES_SMEM_LIMIT;
  }
  sprout_launch(attention_decode_resident_kernel<HD, FUSED>, dim3(p.kv_heads, requests), dim3(RES_THREADS), smem, stream, map_k, map_v, p);
  return sprout_check_launch("attention_decode_resident");
}

int log2_exact(int v) {
  for (int s = 0; s < 31; s++) if ((1 << s) == v) return s;
  return -1;
}

}  // namespace

// The largest context (a multiple of 128 keys) that the resident kernel takes for these sizes, or
// 0 where it does not apply: head sizes 64 and 128, pages of 8 to 128 tokens (a power of two), up
// to 16 query heads per key/value head.
SPROUT_API int sprout_attention_decode_resident_cap(int heads, int kv_heads, int head_dim, int page_tokens) {
  if ((head_dim != 64 && head_dim != 128) || kv_heads <= 0 || heads % kv_heads || heads / kv_heads > 16) return 0;
  const int shift = log2_exact(page_tokens);
  if (shift < 3 || shift > 7) return 0;
  int cap = 0;
  for (int keys = 128; keys <= RES_MAX_CHUNKS * 128; keys += 128)
    if (resident_smem_bytes(head_dim, keys) <= (size_t)RES_SMEM_LIMIT) cap = keys;
  return cap;
}

// One query token per request with the whole context in shared memory (see the top of this file).
// acc != null: the fused form (as sprout_attention_decode_fused: sums, bias, rotation tables;
// appends the new token's key and value and clears the sums), q is ignored; acc == null: q holds
// the queries and the cache already holds the new token.  cap_keys: room for this many keys per
// request (a multiple of 128, at most sprout_attention_decode_resident_cap(...)); a request with a
// longer context sets the status word's layout bit and gets no output.
SPROUT_API int sprout_attention_decode_resident(float* acc, const float* bias, const float* cos_table, const float* sin_table,
                                                int max_positions, int rotary_dim, int interleaved, const void* q, int q_stride,
                                                void* k_cache, void* v_cache, const int* block_table, int table_stride,
                                                const int* context_lens, void* out, int out_stride, int requests, int heads,
                                                int kv_heads, int head_dim, int page_tokens, int num_pages, int cap_keys,
                                                const float* norm_x, int norm_width, float norm_eps, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(requests > 0 && requests <= 65535 && heads > 0 && kv_heads > 0 && num_pages > 0, "attention_decode_resident: sizes must be positive");
  const int cap_max = sprout_attention_decode_resident_cap(heads, kv_heads, head_dim, page_tokens);
  SPROUT_REQUIRE(cap_max > 0, "attention_decode_resident: takes head_dim 64 or 128, pages of 8, 16, 32, 64 or 128 tokens and up to 16 "
                 "query heads per key/value head (got head_dim %d, page %d, heads %d / %d)", head_dim, page_tokens, heads, kv_heads);
  SPROUT_REQUIRE(cap_keys >= 128 && cap_keys % 128 == 0 && cap_keys <= cap_max,
                 "attention_decode_resident: cap_keys must be a multiple of 128 up to %d for these sizes (got %d)", cap_max, cap_keys);
  SPROUT_REQUIRE((acc || q) && k_cache && v_cache && block_table && context_lens && out && status, "attention_decode_resident: null pointer");
  SPROUT_REQUIRE(((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && out_stride % 2 == 0 && ((uintptr_t)out & 3) == 0 &&
                 (acc || (q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0)), "attention_decode_resident: misaligned operands");
  SPROUT_REQUIRE((cos_table == nullptr) == (sin_table == nullptr), "attention_decode_resident: cos and sin tables go together");
  SPROUT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim, "attention_decode_resident: rotary_dim must be even and at most head_dim");
  const long long cache_rows = (long long)num_pages * kv_heads * page_tokens;
  SPROUT_REQUIRE(cache_rows <= 0x7fffffffLL, "attention_decode_resident: the cache has too many rows for a tensor map");
  ResidentParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
  p.block_table = block_table; p.table_stride = table_stride; p.context_lens = context_lens;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.heads = heads; p.kv_heads = kv_heads; p.page_shift = log2_exact(page_tokens); p.num_pages = num_pages; p.cap_keys = cap_keys;
  p.status = status;
  p.acc = acc; p.bias = bias; p.cos_table = cos_table; p.sin_table = sin_table; p.max_positions = max_positions;
  p.rotary_dim = cos_table ? rotary_dim : 0; p.interleaved = interleaved ? 1 : 0;
  SPROUT_REQUIRE(!norm_x || (acc && norm_width > 0 && norm_eps > 0.f), "attention_decode_resident: a scale needs the sums, a width and a positive eps");
  p.norm_x = norm_x; p.norm_width = norm_width; p.norm_eps = norm_eps;
  CUtensorMap map_k, map_v;
  if (tensor_map(k_cache, (int)cache_rows, head_dim, head_dim, page_tokens, &map_k)) return 1;
  if (tensor_map(v_cache, (int)cache_rows, head_dim, head_dim, page_tokens, &map_v)) return 1;
  if (head_dim == 64) return acc ? launch_resident<64, true>(map_k, map_v, p, requests, stream) : launch_resident<64, false>(map_k, map_v, p, requests, stream);
  return acc ? launch_resident<128, true>(map_k, map_v, p, requests, stream) : launch_resident<128, false>(map_k, map_v, p, requests, stream);
}

SPROUT_TL_READER(attention_decode_resident)
