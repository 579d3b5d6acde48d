// out += a W^T for up to 16 tokens of a small layer, in a kernel that is light enough to share
// an SM with its neighbours in the stream: the q/k/v product (with the RMSNorm before it folded
// in) and the output projection of a decode step.
//
// Why: for a handful of tokens these products are a few hundred kilobytes to a few megabytes of
// weights; what they cost is the fixed time of a kernel in a chain of dependent kernels.  A CTA
// here needs some 20 KB of shared memory and no tensor memory, so it becomes resident while the
// kernel before it still runs, has its weights in shared memory by the time that kernel ends,
// and leaves room for the CTAs of the kernel after it to do the same.
//
// How: the matrix [N, K] is cut into row_groups x k_splits pieces, one per CTA (plan_pieces); a
// CTA asks for its piece by TMA (boxes of 64 columns, 128-byte swizzle) before it waits for the
// earlier kernels, then brings its K range of the tokens' rows into shared memory as bfloat16,
// either copied from a bfloat16 input or normalised from the float32 residual stream (every CTA
// computes the rows' scale from the whole row, float32 arithmetic, and converts only its K
// range), multiplies with `mma.sync.m16n8k16` (weights the 16-row operand, tokens the 8 columns, in one or two tiles of tokens)
// and adds its partial sums to the float32 output with atomic adds.  The output is the residual
// stream (output projection) or a zeroed workspace whose reader clears it again (q/k/v).
//
// Sizes: tokens 1..16, N and K multiples of 16, pieces of at most 64 KB
// (sprout_linear_decode_supported says); everything else takes the tcgen05 product.
#include "small_batch.cuh"

namespace {

constexpr int LIN_THREADS = 256;
constexpr int LIN_MAX_SMEM = 96 * 1024;

struct LinPlan {
  int tokens, n, k;
  int tiles, ksteps;            // 16-row tiles, 16-wide K steps of the matrix
  int row_groups, k_splits;
  int max_tiles, max_ksteps, boxes, box_bytes;
  int off_act, off_gain, off_stage, off_bar, smem_bytes;
  int lda, ldo;                 // row strides of the bfloat16 input and of the output, in elements
  int normed;                   // 1: the input is the float32 residual stream, normalised here
  float eps;
};

// The products of a CTA's piece: a warp per 16-row tile, NT tiles of 8 tokens, even and odd K steps as
// two chains of products per token tile; the sums are added into the float32 output.
template <int NT>
__device__ __forceinline__ void lin_products(const LinPlan& p, const uint8_t* w, const uint8_t* actbuf, float* __restrict__ out,
                                             int stride_b, int t_begin, int nt, int nk, int lane, int warp) {
  const uint8_t* b_base = actbuf + (size_t)(lane >> 2) * stride_b + (lane & 3) * 4;
  const uint32_t w_addr = smem_u32(w);
  for (int tile = warp; tile < nt; tile += LIN_THREADS / 32) {
    float d[NT][4], e[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
      for (int j = 0; j < 4; j++) d[n][j] = e[n][j] = 0.f;
    const int a_row = tile * 16 + (lane & 15);
    for (int k = 0; k < nk; k += 2) {
      const bool two = k + 1 < nk;
      uint32_t f[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int kk = (u == 0 || two) ? k + u : k;
        ldmatrix_x4(swizzled(w_addr + (uint32_t)(kk >> 2) * p.box_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                    f[u][0], f[u][1], f[u][2], f[u][3]);
      }
#pragma unroll
      for (int n = 0; n < NT; n++) {
        const uint8_t* b = b_base + (size_t)n * 8 * stride_b;
        mma_bf16(d[n], f[0][0], f[0][1], f[0][2], f[0][3], *(const uint32_t*)(b + k * 32), *(const uint32_t*)(b + k * 32 + 16));
        if (two) mma_bf16(e[n], f[1][0], f[1][1], f[1][2], f[1][3], *(const uint32_t*)(b + (k + 1) * 32), *(const uint32_t*)(b + (k + 1) * 32 + 16));
      }
    }
    const int row = (t_begin + tile) * 16 + (lane >> 2);
#pragma unroll
    for (int n = 0; n < NT; n++) {
      const int t0 = n * 8 + (lane & 3) * 2;
      if (t0 < p.tokens) {
        atomicAdd(out + (size_t)t0 * p.ldo + row, d[n][0] + e[n][0]);
        atomicAdd(out + (size_t)t0 * p.ldo + row + 8, d[n][2] + e[n][2]);
      }
      if (t0 + 1 < p.tokens) {
        atomicAdd(out + (size_t)(t0 + 1) * p.ldo + row, d[n][1] + e[n][1]);
        atomicAdd(out + (size_t)(t0 + 1) * p.ldo + row + 8, d[n][3] + e[n][3]);
      }
    }
  }
}

__global__ void __launch_bounds__(LIN_THREADS)
linear_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __nv_bfloat16* __restrict__ a,
                     const float* __restrict__ x, const float* __restrict__ gain, float* __restrict__ out,
                     int* status, const LinPlan p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ int failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* w = smem;
  uint8_t* actbuf = smem + p.off_act;
  float* gain_s = (float*)(smem + p.off_gain);
  uint8_t* stage = smem + p.off_stage;
  uint64_t* bar = (uint64_t*)(smem + p.off_bar);

  pdl_launch_dependents();
  SPROUT_TL_ENTRY(p.normed ? 0 : 1);

  const int group = blockIdx.x / p.k_splits, split = blockIdx.x % p.k_splits;
  const int t_begin = share_begin(p.tiles, group, p.row_groups);
  const int nt = share_begin(p.tiles, group + 1, p.row_groups) - t_begin;
  const int k_begin = share_begin(p.ksteps, split, p.k_splits);
  const int nk = share_begin(p.ksteps, split + 1, p.k_splits) - k_begin;

  if (tid == 0) {
    failed = 0;
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar, (uint32_t)p.boxes * (uint32_t)p.box_bytes);
    for (int b = 0; b < p.boxes; b++)
      tma_load_2d_addr(smem_u32(w) + (uint32_t)b * p.box_bytes, &map_w, smem_u32(bar), k_begin * 16 + b * 64, t_begin * 16);
  }
  // the norm's gains of this CTA's K range are weights too: in shared memory before the wait
  if (p.normed)
    for (int i = tid; i < nk * 16; i += LIN_THREADS) gain_s[i] = gain[k_begin * 16 + i];

  pdl_wait();
  SPROUT_TL_WAITED(p.normed ? 0 : 1);

  // ---- this CTA's K range of the tokens' rows, bfloat16, rows of nk * 32 + 16 bytes
  const int stride_b = nk * 32 + 16;
  const int rows_held = token_rows(p.tokens);
  if (p.normed) {
    __syncthreads();                                 // the gains are in shared memory
    for (int t = warp; t < rows_held; t += LIN_THREADS / 32) {
    if (t < p.tokens) {
      // one pass over the row: the sum of squares of all of it; this CTA's K range is scaled
      // and converted once the sum is known
      const float4* src = (const float4*)(x + (size_t)t * p.k);
      uint8_t* dst = actbuf + (size_t)t * stride_b;
      const int quads = p.k >> 2, first = k_begin * 4, last = first + nk * 4;
      float ss = 0.f;
      if (quads <= 256) {                            // the row stays in registers; all its loads are in flight at once
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int i = lane + j * 32;
          v[j] = i < quads ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) ss += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)p.k + p.eps);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int i = lane + j * 32;
          if (i >= first && i < last) {
            const float4 g = ((const float4*)gain_s)[i - first];
            __nv_bfloat162 lo = __floats2bfloat162_rn((v[j].x * scale) * g.x, (v[j].y * scale) * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((v[j].z * scale) * g.z, (v[j].w * scale) * g.w);
            *(uint2*)(dst + (size_t)(i - first) * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
          }
        }
      } else {                                       // longer rows: the K range waits in shared memory as float32
        float4* aside = (float4*)(stage + (size_t)t * nk * 64);
#pragma unroll 4
        for (int i = lane; i < quads; i += 32) {
          const float4 v = __ldcg(src + i);
          ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
          if (i >= first && i < last) aside[i - first] = v;
        }
        ss = warp_sum(ss);
        __syncwarp();                                // the lanes read what other lanes set aside
        const float scale = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        for (int i = lane; i < nk * 4; i += 32) {
          const float4 v = aside[i], g = ((const float4*)gain_s)[i];
          __nv_bfloat162 lo = __floats2bfloat162_rn((v.x * scale) * g.x, (v.y * scale) * g.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v.z * scale) * g.z, (v.w * scale) * g.w);
          *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        }
      }
    } else {
      for (int i = lane; i < nk * 2; i += 32) *(uint4*)(actbuf + (size_t)t * stride_b + (size_t)i * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    }
  } else {
    const int chunks = nk * 2;                       // 16-byte pieces per token
    for (int i = tid; i < rows_held * chunks; i += LIN_THREADS) {
      const int t = i / chunks, c = i - t * chunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t < p.tokens) v = __ldcg((const uint4*)(a + (size_t)t * p.lda + (size_t)k_begin * 16) + c);
      *(uint4*)(actbuf + (size_t)t * stride_b + c * 16) = v;
    }
  }
  __syncthreads();
  if (!mbar_wait(bar, 0)) failed = 1;
  __syncthreads();

  if (failed == 0) {
    if (rows_held == 8) lin_products<1>(p, w, actbuf, out, stride_b, t_begin, nt, nk, lane, warp);
    else lin_products<2>(p, w, actbuf, out, stride_b, t_begin, nt, nk, lane, warp);
  } else if (tid == 0) {
    atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
  }
  SPROUT_TL_EXIT(p.normed ? 0 : 1);
}

// Up to 8 tokens (one tile of the MMA's columns): the kernel as it was tuned for the step of a small
// batch, kept apart from the form for one or two tiles above (which costs it a little per launch).
__global__ void __launch_bounds__(LIN_THREADS)
linear_decode_kernel8(const __grid_constant__ CUtensorMap map_w, const __nv_bfloat16* __restrict__ a,
                     const float* __restrict__ x, const float* __restrict__ gain, float* __restrict__ out,
                     int* status, const LinPlan p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ int failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* w = smem;
  uint8_t* actbuf = smem + p.off_act;
  float* gain_s = (float*)(smem + p.off_gain);
  uint8_t* stage = smem + p.off_stage;
  uint64_t* bar = (uint64_t*)(smem + p.off_bar);

  pdl_launch_dependents();
  SPROUT_TL_ENTRY(p.normed ? 0 : 1);

  const int group = blockIdx.x / p.k_splits, split = blockIdx.x % p.k_splits;
  const int t_begin = share_begin(p.tiles, group, p.row_groups);
  const int nt = share_begin(p.tiles, group + 1, p.row_groups) - t_begin;
  const int k_begin = share_begin(p.ksteps, split, p.k_splits);
  const int nk = share_begin(p.ksteps, split + 1, p.k_splits) - k_begin;

  if (tid == 0) {
    failed = 0;
    mbar_init(bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    mbar_expect_tx(bar, (uint32_t)p.boxes * (uint32_t)p.box_bytes);
    for (int b = 0; b < p.boxes; b++)
      tma_load_2d_addr(smem_u32(w) + (uint32_t)b * p.box_bytes, &map_w, smem_u32(bar), k_begin * 16 + b * 64, t_begin * 16);
  }
  // the norm's gains of this CTA's K range are weights too: in shared memory before the wait
  if (p.normed)
    for (int i = tid; i < nk * 16; i += LIN_THREADS) gain_s[i] = gain[k_begin * 16 + i];

  pdl_wait();
  SPROUT_TL_WAITED(p.normed ? 0 : 1);

  // ---- this CTA's K range of the tokens' rows, bfloat16, rows of nk * 32 + 16 bytes
  const int stride_b = nk * 32 + 16;
  if (p.normed) {
    __syncthreads();                                 // the gains are in shared memory
    if (warp < p.tokens) {
      // one pass over the row: the sum of squares of all of it; this CTA's K range is scaled
      // and converted once the sum is known
      const float4* src = (const float4*)(x + (size_t)warp * p.k);
      uint8_t* dst = actbuf + (size_t)warp * stride_b;
      const int quads = p.k >> 2, first = k_begin * 4, last = first + nk * 4;
      float ss = 0.f;
      if (quads <= 256) {                            // the row stays in registers; all its loads are in flight at once
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int i = lane + j * 32;
          v[j] = i < quads ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) ss += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)p.k + p.eps);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          const int i = lane + j * 32;
          if (i >= first && i < last) {
            const float4 g = ((const float4*)gain_s)[i - first];
            __nv_bfloat162 lo = __floats2bfloat162_rn((v[j].x * scale) * g.x, (v[j].y * scale) * g.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn((v[j].z * scale) * g.z, (v[j].w * scale) * g.w);
            *(uint2*)(dst + (size_t)(i - first) * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
          }
        }
      } else {                                       // longer rows: the K range waits in shared memory as float32
        float4* aside = (float4*)(stage + (size_t)warp * nk * 64);
#pragma unroll 4
        for (int i = lane; i < quads; i += 32) {
          const float4 v = __ldcg(src + i);
          ss += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
          if (i >= first && i < last) aside[i - first] = v;
        }
        ss = warp_sum(ss);
        __syncwarp();                                // the lanes read what other lanes set aside
        const float scale = 1.0f / sqrtf(ss / (float)p.k + p.eps);
        for (int i = lane; i < nk * 4; i += 32) {
          const float4 v = aside[i], g = ((const float4*)gain_s)[i];
          __nv_bfloat162 lo = __floats2bfloat162_rn((v.x * scale) * g.x, (v.y * scale) * g.y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v.z * scale) * g.z, (v.w * scale) * g.w);
          *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        }
      }
    } else {
      for (int i = lane; i < nk * 2; i += 32) *(uint4*)(actbuf + (size_t)warp * stride_b + (size_t)i * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
  } else {
    const int chunks = nk * 2;                       // 16-byte pieces per token
    for (int i = tid; i < 8 * chunks; i += LIN_THREADS) {
      const int t = i / chunks, c = i - t * chunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t < p.tokens) v = __ldcg((const uint4*)(a + (size_t)t * p.lda + (size_t)k_begin * 16) + c);
      *(uint4*)(actbuf + (size_t)t * stride_b + c * 16) = v;
    }
  }
  __syncthreads();
  if (!mbar_wait(bar, 0)) failed = 1;
  __syncthreads();

  if (failed == 0) {
    const uint8_t* b_base = actbuf + (size_t)(lane >> 2) * stride_b + (lane & 3) * 4;
    const uint32_t w_addr = smem_u32(w);
    for (int tile = warp; tile < nt; tile += LIN_THREADS / 32) {
      float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};   // even and odd K steps: two chains of products
      const int a_row = tile * 16 + (lane & 15);
      for (int k = 0; k < nk; k += 2) {
        const bool two = k + 1 < nk;
        uint32_t b[2][2], f[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int kk = (u == 0 || two) ? k + u : k;
          b[u][0] = *(const uint32_t*)(b_base + kk * 32);
          b[u][1] = *(const uint32_t*)(b_base + kk * 32 + 16);
          ldmatrix_x4(swizzled(w_addr + (uint32_t)(kk >> 2) * p.box_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                      f[u][0], f[u][1], f[u][2], f[u][3]);
        }
        mma_bf16(d, f[0][0], f[0][1], f[0][2], f[0][3], b[0][0], b[0][1]);
        if (two) mma_bf16(e, f[1][0], f[1][1], f[1][2], f[1][3], b[1][0], b[1][1]);
      }
      const int row = (t_begin + tile) * 16 + (lane >> 2), t0 = (lane & 3) * 2;
      if (t0 < p.tokens) {
        atomicAdd(out + (size_t)t0 * p.ldo + row, d[0] + e[0]);
        atomicAdd(out + (size_t)t0 * p.ldo + row + 8, d[2] + e[2]);
      }
      if (t0 + 1 < p.tokens) {
        atomicAdd(out + (size_t)(t0 + 1) * p.ldo + row, d[1] + e[1]);
        atomicAdd(out + (size_t)(t0 + 1) * p.ldo + row + 8, d[3] + e[3]);
      }
    }
  } else if (tid == 0) {
    atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
  }
  SPROUT_TL_EXIT(p.normed ? 0 : 1);
}

bool lin_make_plan(int tokens, int n, int k, int ctas, LinPlan* out) {
  if (tokens < 1 || tokens > SMALL_MAX_TOKENS || n < 16 || k < 16 || n % 16 || k % 16 || ctas < 1) return false;
  LinPlan p = {};
  p.tokens = tokens; p.n = n; p.k = k;
  p.tiles = n / 16;
  p.ksteps = k / 16;
  if (!plan_pieces(p.tiles, p.ksteps, ctas, &p.row_groups, &p.k_splits)) return false;
  p.max_tiles = (p.tiles + p.row_groups - 1) / p.row_groups;
  p.max_ksteps = (p.ksteps + p.k_splits - 1) / p.k_splits;
  p.boxes = (p.max_ksteps + 3) / 4;
  p.box_bytes = p.max_tiles * 2048;
  long long at = (long long)p.boxes * p.box_bytes;
  p.off_act = (int)at;
  at += (long long)token_rows(tokens) * (p.max_ksteps * 32 + 16);
  p.off_gain = (int)at;
  at += (long long)p.max_ksteps * 64;
  p.off_stage = (int)at;                 // the tokens' float32 values of the K range, before they are scaled
  at += (long long)token_rows(tokens) * p.max_ksteps * 64;
  p.off_bar = (int)at;
  at += 16 + 1024;                       // the barrier; room to start the tiles on a 1024-byte boundary
  if (at > LIN_MAX_SMEM) return false;
  p.smem_bytes = (int)at;
  *out = p;
  return true;
}

}  // namespace

// 1 when sprout_linear_decode takes these sizes on this device, else 0.
SPROUT_API int sprout_linear_decode_supported(int tokens, int n, int k) {
  LinPlan plan;
  return lin_make_plan(tokens, n, k, sm_count(), &plan) ? 1 : 0;
}

// The launch layout for these sizes on `ctas` CTAs, for inspection by host-side tests: 1 and the
// plan's 13 numbers in `out` (in the order of the list below), or 0 when the sizes are refused.
SPROUT_API int sprout_linear_decode_plan(int tokens, int n, int k, int ctas, int* out) {
  LinPlan p;
  if (!out || !lin_make_plan(tokens, n, k, ctas, &p)) return 0;
  const int fields[13] = {p.tiles, p.ksteps, p.row_groups, p.k_splits, p.max_tiles, p.max_ksteps, p.boxes, p.box_bytes,
                          p.off_act, p.off_gain, p.off_stage, p.off_bar, p.smem_bytes};
  for (int i = 0; i < 13; i++) out[i] = fields[i];
  return 1;
}

// out [tokens, n] float32 (row stride ldo) += input W^T, W bfloat16 [n, k] contiguous.  The input
// is `a`, bfloat16 [tokens, k] with row stride lda, or, when `a` is null, rmsnorm(x, gain, eps)
// of the float32 rows x [tokens, k].
SPROUT_API int sprout_linear_decode(const void* a, int lda, const float* x, const float* gain, float eps, const void* weight,
                                    float* out, int ldo, int tokens, int n, int k, int* status, cudaStream_t stream) {
  LinPlan plan;
  SPROUT_REQUIRE(weight && out && status && (a || (x && gain)), "linear_decode: a pointer is missing");
  SPROUT_REQUIRE(lin_make_plan(tokens, n, k, sm_count(), &plan),
                 "linear_decode: tokens 1..%d, N and K multiples of 16 and pieces that fit (got tokens %d, N %d, K %d)",
                 SMALL_MAX_TOKENS, tokens, n, k);
  plan.normed = a ? 0 : 1;
  plan.eps = eps;
  plan.lda = lda;
  plan.ldo = ldo;
  SPROUT_REQUIRE(plan.normed ? eps > 0.f && ((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0
                             : lda >= k && lda % 8 == 0 && ((uintptr_t)a & 15) == 0,
                 "linear_decode: the input must be 16-byte aligned with rows of at least K elements (eps positive)");
  SPROUT_REQUIRE(ldo >= n && ((uintptr_t)weight & 15) == 0, "linear_decode: output rows shorter than N, or unaligned weights");
  CUtensorMap map_w;
  if (tensor_map(weight, n, k, k, plan.max_tiles * 16, &map_w)) return 1;
  static bool configured = false;
  if (!configured) {
    for (auto kernel : {linear_decode_kernel, linear_decode_kernel8}) {
      cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LIN_MAX_SMEM);
      SPROUT_REQUIRE(err == cudaSuccess, "linear_decode: cudaFuncSetAttribute failed: %s", cudaGetErrorString(err));
      // the same split between L1 and shared memory as its neighbours in the stream, so that their CTAs share SMs
      cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    }
    configured = true;
  }
  cudaError_t err = sprout_launch(tokens <= 8 ? linear_decode_kernel8 : linear_decode_kernel, dim3(plan.row_groups * plan.k_splits),
                                  dim3(LIN_THREADS), (size_t)plan.smem_bytes, stream, map_w, (const __nv_bfloat16*)a, x, gain, out, status, plan);
  SPROUT_REQUIRE(err == cudaSuccess, "linear_decode: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

SPROUT_TL_READER(linear_decode)
