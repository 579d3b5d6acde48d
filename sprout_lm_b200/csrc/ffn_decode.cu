// Decode feed-forward of a small model in ONE kernel: RMSNorm, gate/up product, SwiGLU, down
// product and the residual sum, for up to 16 tokens (one per request).
//
// Why: a decode step of a small model is a chain of short kernels, each of which costs a few
// microseconds whatever it computes (launch, first load, drain).  The norm, the gate/up product
// and the down product are three links of that chain per layer; here they are one launch, and
// the activation between the two products never leaves the SMs: it is exchanged among the CTAs
// of a thread-block cluster through distributed shared memory, behind the cluster's hardware
// barrier, where a trip through memory (store, flag, poll, fetch) costs three times as long.
//
// How: one CTA per SM, in clusters of 2, 4 or 8.  Every CTA owns a contiguous share of the 16-row
// tiles of the interleaved gate/up matrix (rows 16b..16b+7 gate, 16b+8..16b+15 up) and asks for
// them by TMA tile copies (boxes of 64 columns, 128-byte swizzle) into its shared memory before it
// waits for the kernels before it.  With 160 KB of shared memory at the 0.5B sizes the CTA fits
// beside a CTA of the attention kernel, so the weights stream from memory while the attention
// half of the layer still runs.  After the wait each warp normalises one token's row of the
// residual stream (float32 arithmetic) into a bfloat16 operand in shared memory; the products run
// on `mma.sync.m16n8k16` with the weights as the 16-row operand and the tokens as the 8 columns
// (for eight tokens the tensor cores' rate does not matter, latency does); a warp takes a 16-row
// tile over the whole K, so the gate value and its up value end up in one thread's registers,
// where SwiGLU is applied.  The warp writes its 8 activation columns into the shared memory of
// every CTA of its cluster.  The activation columns that a cluster produces are the K range of
// the down product that the cluster works on: each of its CTAs takes a share of the down matrix's
// rows over that K range (TMA, requested as soon as the gate/up products are done with the room),
// multiplies it with the exchanged activation and adds the result into the float32 residual
// stream with atomic adds (the order of those float32 additions is not fixed).
//
// Sizes: tokens 1..16 (one or two tiles of 8 for the MMA), hidden and intermediate sizes multiples of 16, and a layer whose per-CTA
// share of the weights fits in shared memory (sprout_ffn_decode_supported says); larger models
// keep the separate kernels, whose products are bound by bandwidth, not by latency.
//
// Every wait on an mbarrier is bounded: one that runs out sets the status word's WAIT_TIMEOUT bit
// and the CTA skips its arithmetic, but it still meets its cluster at the (hardware) barriers.
#include <cooperative_groups.h>
#include <stdlib.h>

#include "small_batch.cuh"

// With -DFFN_STAMPS the first thread of the first and of the last CTA records the time (%globaltimer)
// at the end of each phase; sprout_ffn_stamps copies the last launch's records out.  Measurements
// of where the kernel's time goes inside a real decode step come from such a build.
#ifdef FFN_STAMPS
__device__ unsigned long long g_ffn_stamps[2][16];
#define FFN_STAMP(i) do { if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) g_ffn_stamps[blockIdx.x ? 1 : 0][i] = global_ns(); } while (0)
extern "C" __attribute__((visibility("default"))) void sprout_ffn_stamps(unsigned long long* out) { cudaMemcpyFromSymbol(out, g_ffn_stamps, sizeof(g_ffn_stamps)); }
#else
#define FFN_STAMP(i) do { } while (0)
#endif

namespace {

namespace cg = cooperative_groups;

constexpr int FFN_THREADS = 256;            // 8 warps
constexpr int FFN_MAX_TOKENS = SMALL_MAX_TOKENS;
constexpr int FFN_MAX_TILES = FFN_THREADS / 32;   // gate/up tiles of a CTA: a warp each
constexpr int FFN_SMEM_LIMIT = 227 * 1024 - 1024;   // dynamic shared memory; the rest is for the kernel's static variables

struct FfnPlan {
  int tokens, hidden, inter;
  int rows_held;         // rows of the tokens' operands: 8 or 16 (whole tiles of the MMA's 8 columns)
  int ctas, cluster;     // CTAs of the launch, CTAs of a cluster
  int tiles1;            // 16-row tiles of the gate/up matrix: inter / 8 (each gives 8 activation columns)
  int base_tiles1, max_tiles1;   // what every CTA has at least (some have one more), at most
  int boxes1, box1_bytes;        // 64-column boxes along K of a CTA's gate/up rows
  int tiles2;            // 16-row tiles of the down matrix: hidden / 16; a cluster's CTAs share them
  int max_tiles2;        // the most of them a CTA has
  int box_rows2, row_boxes2;     // its rows come in boxes of box_rows2 rows (at most 256)
  int max_ktiles, max_ksteps;    // the most activation tiles (8 columns) a cluster produces; 16-wide K steps over them
  int col_boxes2, box2_bytes;    // 64-column boxes over a cluster's K range; bytes of a box
  int stride1;           // bytes between the tokens' rows of the normalised operand in shared memory
  int stride_x;          // bytes between the tokens' rows of the exchanged activation
  int off_w2, off_act, off_xchg, off_bar, smem_bytes;
  float eps;
};

__device__ __forceinline__ float ffn_silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// The cluster's hardware barrier in two halves: arrive (with release: what this thread wrote, also
// into other CTAs' shared memory, is visible to those who have waited) and wait (with acquire).
__device__ __forceinline__ void ffn_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void ffn_cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// A warp's gate/up tile over the whole K for NT tiles of 8 tokens.  The tile's fragment holds gate
// rows 0-7 and their up rows 8-15 in the same thread, so SwiGLU is applied on the registers; the
// tile's 8 activation columns go into the shared memory of every CTA of the cluster.  Eight chains of
// products (K steps 0, 8, 16.. / 1, 9, .. for one token tile; 0, 4, .. for two) keep the dependent
// `mma.sync` apart.
template <int NT>
__device__ __forceinline__ void ffn_gate_up(const FfnPlan& p, cg::cluster_group& cluster, const uint8_t* w1, const uint8_t* actbuf,
                                            uint8_t* xchg, bool ok1, int t1_begin, int kt_begin, int nkt, int lane, int warp) {
  constexpr int CHAINS = 8 / NT;
  float s[NT][4];
#pragma unroll
  for (int n = 0; n < NT; n++) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
  if (ok1) {
    const int ksteps1 = p.hidden >> 4;
    const uint32_t w1_addr = smem_u32(w1);
    const int a_row = warp * 16 + (lane & 15);
    const uint8_t* b_base = actbuf + (size_t)(lane >> 2) * p.stride1 + (lane & 3) * 4;
    float acc[CHAINS][NT][4];
#pragma unroll
    for (int c = 0; c < CHAINS; c++)
#pragma unroll
      for (int n = 0; n < NT; n++) acc[c][n][0] = acc[c][n][1] = acc[c][n][2] = acc[c][n][3] = 0.f;
    int k = 0;
    for (; k + CHAINS <= ksteps1; k += CHAINS) {
      uint32_t b[CHAINS][NT][2], a[CHAINS][4];
#pragma unroll
      for (int u = 0; u < CHAINS; u++) {                  // all the loads of the steps, then their products
        const int kk = k + u;
#pragma unroll
        for (int n = 0; n < NT; n++) {
          b[u][n][0] = *(const uint32_t*)(b_base + (size_t)n * 8 * p.stride1 + kk * 32);
          b[u][n][1] = *(const uint32_t*)(b_base + (size_t)n * 8 * p.stride1 + kk * 32 + 16);
        }
        ldmatrix_x4(swizzled(w1_addr + (uint32_t)(kk >> 2) * p.box1_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                    a[u][0], a[u][1], a[u][2], a[u][3]);
      }
#pragma unroll
      for (int u = 0; u < CHAINS; u++)
#pragma unroll
        for (int n = 0; n < NT; n++) mma_bf16(acc[u][n], a[u][0], a[u][1], a[u][2], a[u][3], b[u][n][0], b[u][n][1]);
    }
    for (; k < ksteps1; k++) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(swizzled(w1_addr + (uint32_t)(k >> 2) * p.box1_bytes, a_row, (k & 3) * 2 + (lane >> 4)), a0, a1, a2, a3);
#pragma unroll
      for (int n = 0; n < NT; n++) {
        const uint8_t* b = b_base + (size_t)n * 8 * p.stride1 + k * 32;
        mma_bf16(acc[0][n], a0, a1, a2, a3, *(const uint32_t*)b, *(const uint32_t*)(b + 16));
      }
    }
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float sum = 0.f;
        if constexpr (CHAINS == 8)
          sum = ((acc[0][n][j] + acc[1][n][j]) + (acc[2][n][j] + acc[3][n][j])) + ((acc[4][n][j] + acc[5][n][j]) + (acc[6][n][j] + acc[7][n][j]));
        else
          sum = (acc[0][n][j] + acc[1][n][j]) + (acc[2][n][j] + acc[3][n][j]);
        s[n][j] = sum;
      }
  }
  // fragment rows 0-7 are gate rows, rows 8-15 the matching up rows: (0, 2) and (1, 3) pair up
  const int col = (t1_begin - kt_begin + warp) * 8 + (lane >> 2);
  const bool closes = (nkt & 1) && t1_begin + warp == kt_begin + nkt - 1;   // the cluster's last tile ends half a K step: the other half is zero
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
#pragma unroll
  for (int n = 0; n < NT; n++) {
    const int t0 = n * 8 + (lane & 3) * 2;
    const __nv_bfloat16 a0 = __float2bfloat16_rn(t0 < p.tokens ? ffn_silu_mul(s[n][0], s[n][2]) : 0.f);
    const __nv_bfloat16 a1 = __float2bfloat16_rn(t0 + 1 < p.tokens ? ffn_silu_mul(s[n][1], s[n][3]) : 0.f);
    for (int q = 0; q < p.cluster; q++) {
      __nv_bfloat16* theirs = (__nv_bfloat16*)cluster.map_shared_rank(xchg, q);
      __nv_bfloat16* r0 = (__nv_bfloat16*)((uint8_t*)theirs + (size_t)t0 * p.stride_x);
      __nv_bfloat16* r1 = (__nv_bfloat16*)((uint8_t*)theirs + (size_t)(t0 + 1) * p.stride_x);
      r0[col] = a0;
      r1[col] = a1;
      if (closes) { r0[col + 8] = zero; r1[col + 8] = zero; }
    }
  }
}

// The CTA's row tiles of the down matrix over the cluster's K range, for NT tiles of 8 tokens, added
// into the residual stream.
template <int NT>
__device__ __forceinline__ void ffn_down(const FfnPlan& p, const uint8_t* w2, const uint8_t* xchg, float* __restrict__ x,
                                         int t2_begin, int nt2, int ksteps2, int lane, int warp) {
  const uint8_t* b_base = xchg + (size_t)(lane >> 2) * p.stride_x + (lane & 3) * 4;
  const uint32_t w2_addr = smem_u32(w2);
  for (int tile = warp; tile < nt2; tile += FFN_THREADS / 32) {
    float d[NT][4], e[NT][4];                        // even and odd K steps: two chains of products per token tile
#pragma unroll
    for (int n = 0; n < NT; n++)
#pragma unroll
      for (int j = 0; j < 4; j++) d[n][j] = e[n][j] = 0.f;
    const int row_in_part = tile * 16 + (lane & 15);
    const uint32_t box_row = w2_addr + (uint32_t)(row_in_part / p.box_rows2) * p.box2_bytes;
    const int a_row = row_in_part % p.box_rows2;
    for (int k = 0; k < ksteps2; k += 2) {
      const bool two = k + 1 < ksteps2;
      uint32_t a[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const int kk = (u == 0 || two) ? k + u : k;
        ldmatrix_x4(swizzled(box_row + (uint32_t)((kk >> 2) * p.row_boxes2) * p.box2_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                    a[u][0], a[u][1], a[u][2], a[u][3]);
      }
#pragma unroll
      for (int n = 0; n < NT; n++) {
        const uint8_t* b = b_base + (size_t)n * 8 * p.stride_x;
        mma_bf16(d[n], a[0][0], a[0][1], a[0][2], a[0][3], *(const uint32_t*)(b + k * 32), *(const uint32_t*)(b + k * 32 + 16));
        if (two) mma_bf16(e[n], a[1][0], a[1][1], a[1][2], a[1][3], *(const uint32_t*)(b + (k + 1) * 32), *(const uint32_t*)(b + (k + 1) * 32 + 16));
      }
    }
    const int row = (t2_begin + tile) * 16 + (lane >> 2);
#pragma unroll
    for (int n = 0; n < NT; n++) {
      const int t0 = n * 8 + (lane & 3) * 2;
      if (t0 < p.tokens) {
        atomicAdd(x + (size_t)t0 * p.hidden + row, d[n][0] + e[n][0]);
        atomicAdd(x + (size_t)t0 * p.hidden + row + 8, d[n][2] + e[n][2]);
      }
      if (t0 + 1 < p.tokens) {
        atomicAdd(x + (size_t)(t0 + 1) * p.hidden + row, d[n][1] + e[n][1]);
        atomicAdd(x + (size_t)(t0 + 1) * p.hidden + row + 8, d[n][3] + e[n][3]);
      }
    }
  }
}

// NT: tiles of 8 tokens (1 or 2).
template <int NT>
__device__ __forceinline__ void ffn_decode_body(const CUtensorMap& map_gu_base, const CUtensorMap& map_gu_tile, const CUtensorMap& map_down,
                                                float* __restrict__ x, const float* __restrict__ gain, int* status, const FfnPlan& p) {
  extern __shared__ uint8_t smem_raw[];
  // every CTA of the cluster lays its shared memory out alike (the same offset from the same alignment)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles start on 1024 bytes
  __shared__ int failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, ctas = gridDim.x;
  uint8_t* w1 = smem;
  uint8_t* w2 = smem + p.off_w2;
  uint8_t* actbuf = smem + p.off_act;
  uint8_t* xchg = smem + p.off_xchg;
  uint64_t* bars = (uint64_t*)(smem + p.off_bar);
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), first_cta = cta - rank;

  pdl_launch_dependents();
  ffn_cluster_arrive();                              // "this CTA runs": awaited before anyone writes into its shared memory
  SPROUT_TL_ENTRY(0);
  FFN_STAMP(0);

  // this CTA's share of the gate/up tiles; its cluster's activation tiles; its rows of the down matrix
  const int t1_begin = share_begin(p.tiles1, cta, ctas);
  const int nt1 = share_begin(p.tiles1, cta + 1, ctas) - t1_begin;
  const int kt_begin = share_begin(p.tiles1, first_cta, ctas);
  const int nkt = share_begin(p.tiles1, first_cta + p.cluster, ctas) - kt_begin;
  const int ksteps2 = (nkt + 1) >> 1;                // 16-wide K steps over the cluster's nkt * 8 activation columns
  const int t2_begin = share_begin(p.tiles2, rank, p.cluster);
  const int nt2 = share_begin(p.tiles2, rank + 1, p.cluster) - t2_begin;
  const bool has2 = nt2 > 0 && nkt > 0;

  if (tid == 0) {
    failed = 0;
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // ---- this CTA's gate/up tiles, requested before the wait for the earlier kernels: every CTA
  //      has base_tiles1 tiles (one box per 64 columns), some have one more (a 16-row box each)
  if (warp == 0) {
    const uint32_t bar = smem_u32(&bars[0]);
    const uint32_t base_bytes = (uint32_t)p.base_tiles1 * 2048;
    if (lane == 0) mbar_expect_tx(&bars[0], (uint32_t)p.boxes1 * (uint32_t)nt1 * 2048);
    __syncwarp();
    for (int b = lane; b < p.boxes1; b += 32) {
      const uint32_t dst = smem_u32(w1) + (uint32_t)b * p.box1_bytes;
      if (p.base_tiles1 > 0) tma_load_2d_addr(dst, &map_gu_base, bar, b * 64, t1_begin * 16);
      if (nt1 > p.base_tiles1) tma_load_2d_addr(dst + base_bytes, &map_gu_tile, bar, b * 64, (t1_begin + p.base_tiles1) * 16);
    }
  }
  // operand rows of the tokens that are not there: zero
  {
    uint4* pad = (uint4*)(actbuf + (size_t)p.tokens * p.stride1);
    const int count = (p.rows_held - p.tokens) * (p.stride1 >> 4);
    for (int i = tid; i < count; i += FFN_THREADS) pad[i] = make_uint4(0u, 0u, 0u, 0u);
  }

  // the norm's gains are weights too: in registers before the wait (rows of up to 1,024 values)
  const float4* g4 = (const float4*)gain;
  float4 g[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int i = lane + k * 32;
    g[k] = (warp < p.tokens && i < (p.hidden >> 2) && (p.hidden >> 2) <= 256) ? g4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  FFN_STAMP(1);
  pdl_wait();
  SPROUT_TL_WAITED(0);
  FFN_STAMP(2);

  // ---- RMSNorm: warp w normalises tokens w and w + 8 into the bfloat16 operand (float32 arithmetic)
  for (int t = warp; t < p.tokens; t += FFN_THREADS / 32) {
    const float4* src = (const float4*)(x + (size_t)t * p.hidden);
    uint8_t* dst = actbuf + (size_t)t * p.stride1;
    const int quads = p.hidden >> 2;
    float ss = 0.f;
    if (quads <= 256) {                              // the row stays in registers between the two passes
      float4 v[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int i = lane + k * 32;
        v[k] = i < quads ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int k = 0; k < 8; k++) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int i = lane + k * 32;
        if (i < quads) {
          __nv_bfloat162 lo = __floats2bfloat162_rn((v[k].x * scale) * g[k].x, (v[k].y * scale) * g[k].y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v[k].z * scale) * g[k].z, (v[k].w * scale) * g[k].w);
          *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        }
      }
    } else {
      for (int i = lane; i < quads; i += 32) {
        const float4 a = __ldcg(src + i);
        ss += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
      }
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
      for (int i = lane; i < quads; i += 32) {
        const float4 a = __ldcg(src + i), gi = g4[i];
        __nv_bfloat162 lo = __floats2bfloat162_rn((a.x * scale) * gi.x, (a.y * scale) * gi.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn((a.z * scale) * gi.z, (a.w * scale) * gi.w);
        *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  }
  __syncthreads();
  FFN_STAMP(3);
  if (!mbar_wait(&bars[0], 0)) failed = 1;
  __syncthreads();
  FFN_STAMP(4);
  const bool ok1 = failed == 0;
  ffn_cluster_wait();                                // every CTA of the cluster runs: their shared memory may be written

  // ---- gate/up: a warp per 16-row tile of the CTA's share (a CTA has at most 8), over the whole K
  if (warp < nt1) {
    ffn_gate_up<NT>(p, cluster, w1, actbuf, xchg, ok1, t1_begin, kt_begin, nkt, lane, warp);
  }
  ffn_cluster_arrive();                              // this CTA's columns are written, here and in the other CTAs
  __syncthreads();                                   // the operand rows and the gate/up tiles have been read
  FFN_STAMP(5);
  // The gate/up weights have been used: this CTA's rows of the down matrix, over the cluster's K
  // range, take their place.  They arrive while the cluster meets.
  if (tid == 0 && has2) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t bar = smem_u32(&bars[1]);
    mbar_expect_tx(&bars[1], (uint32_t)(p.row_boxes2 * p.col_boxes2) * (uint32_t)p.box2_bytes);
    for (int cb = 0; cb < p.col_boxes2; cb++)
      for (int rb = 0; rb < p.row_boxes2; rb++)
        tma_load_2d_addr(smem_u32(w2) + (uint32_t)(cb * p.row_boxes2 + rb) * p.box2_bytes, &map_down, bar,
                         kt_begin * 8 + cb * 64, t2_begin * 16 + rb * p.box_rows2);
  }
  ffn_cluster_wait();                                // the cluster's activation columns are all here
  FFN_STAMP(6);
  if (has2 && !mbar_wait(&bars[1], 0)) failed = 1;
  __syncthreads();
  FFN_STAMP(7);

  // ---- down: this CTA's row tiles over the cluster's K range, added into the residual stream
  if (has2 && failed == 0) {
    ffn_down<NT>(p, w2, xchg, x, t2_begin, nt2, ksteps2, lane, warp);
  }
  __syncthreads();
  FFN_STAMP(8);
  if (tid == 0 && failed) atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
  SPROUT_TL_EXIT(0);
}

// Up to 8 tokens (one tile of the MMA's columns): the kernel as it was tuned for the step of a
// small batch, where a microsecond per layer shows; it is kept apart from the two-tile form below
// (the shared form of both cost it 0.5 to 1 us per launch).
__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_decode_kernel8(const __grid_constant__ CUtensorMap map_gu_base, const __grid_constant__ CUtensorMap map_gu_tile,
                  const __grid_constant__ CUtensorMap map_down, float* __restrict__ x, const float* __restrict__ gain,
                  int* status, const FfnPlan p) {
  extern __shared__ uint8_t smem_raw[];
  // every CTA of the cluster lays its shared memory out alike (the same offset from the same alignment)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);   // swizzled tiles start on 1024 bytes
  __shared__ int failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, ctas = gridDim.x;
  uint8_t* w1 = smem;
  uint8_t* w2 = smem + p.off_w2;
  uint8_t* actbuf = smem + p.off_act;
  uint8_t* xchg = smem + p.off_xchg;
  uint64_t* bars = (uint64_t*)(smem + p.off_bar);
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank(), first_cta = cta - rank;

  pdl_launch_dependents();
  ffn_cluster_arrive();                              // "this CTA runs": awaited before anyone writes into its shared memory
  SPROUT_TL_ENTRY(0);
  FFN_STAMP(0);

  // this CTA's share of the gate/up tiles; its cluster's activation tiles; its rows of the down matrix
  const int t1_begin = share_begin(p.tiles1, cta, ctas);
  const int nt1 = share_begin(p.tiles1, cta + 1, ctas) - t1_begin;
  const int kt_begin = share_begin(p.tiles1, first_cta, ctas);
  const int nkt = share_begin(p.tiles1, first_cta + p.cluster, ctas) - kt_begin;
  const int ksteps2 = (nkt + 1) >> 1;                // 16-wide K steps over the cluster's nkt * 8 activation columns
  const int t2_begin = share_begin(p.tiles2, rank, p.cluster);
  const int nt2 = share_begin(p.tiles2, rank + 1, p.cluster) - t2_begin;
  const bool has2 = nt2 > 0 && nkt > 0;

  if (tid == 0) {
    failed = 0;
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // ---- this CTA's gate/up tiles, requested before the wait for the earlier kernels: every CTA
  //      has base_tiles1 tiles (one box per 64 columns), some have one more (a 16-row box each)
  if (warp == 0) {
    const uint32_t bar = smem_u32(&bars[0]);
    const uint32_t base_bytes = (uint32_t)p.base_tiles1 * 2048;
    if (lane == 0) mbar_expect_tx(&bars[0], (uint32_t)p.boxes1 * (uint32_t)nt1 * 2048);
    __syncwarp();
    for (int b = lane; b < p.boxes1; b += 32) {
      const uint32_t dst = smem_u32(w1) + (uint32_t)b * p.box1_bytes;
      if (p.base_tiles1 > 0) tma_load_2d_addr(dst, &map_gu_base, bar, b * 64, t1_begin * 16);
      if (nt1 > p.base_tiles1) tma_load_2d_addr(dst + base_bytes, &map_gu_tile, bar, b * 64, (t1_begin + p.base_tiles1) * 16);
    }
  }
  // operand rows of the tokens that are not there: zero
  {
    uint4* pad = (uint4*)(actbuf + (size_t)p.tokens * p.stride1);
    const int count = (8 - p.tokens) * (p.stride1 >> 4);
    for (int i = tid; i < count; i += FFN_THREADS) pad[i] = make_uint4(0u, 0u, 0u, 0u);
  }

  // the norm's gains are weights too: in registers before the wait (rows of up to 1,024 values)
  const float4* g4 = (const float4*)gain;
  float4 g[8];
#pragma unroll
  for (int k = 0; k < 8; k++) {
    const int i = lane + k * 32;
    g[k] = (warp < p.tokens && i < (p.hidden >> 2) && (p.hidden >> 2) <= 256) ? g4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  FFN_STAMP(1);
  pdl_wait();
  SPROUT_TL_WAITED(0);
  FFN_STAMP(2);

  // ---- RMSNorm: warp w normalises token w into the bfloat16 operand (float32 arithmetic)
  if (warp < p.tokens) {
    const float4* src = (const float4*)(x + (size_t)warp * p.hidden);
    uint8_t* dst = actbuf + (size_t)warp * p.stride1;
    const int quads = p.hidden >> 2;
    float ss = 0.f;
    if (quads <= 256) {                              // the row stays in registers between the two passes
      float4 v[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int i = lane + k * 32;
        v[k] = i < quads ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int k = 0; k < 8; k++) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int i = lane + k * 32;
        if (i < quads) {
          __nv_bfloat162 lo = __floats2bfloat162_rn((v[k].x * scale) * g[k].x, (v[k].y * scale) * g[k].y);
          __nv_bfloat162 hi = __floats2bfloat162_rn((v[k].z * scale) * g[k].z, (v[k].w * scale) * g[k].w);
          *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
        }
      }
    } else {
      for (int i = lane; i < quads; i += 32) {
        const float4 a = __ldcg(src + i);
        ss += (a.x * a.x + a.y * a.y) + (a.z * a.z + a.w * a.w);
      }
      ss = warp_sum(ss);
      const float scale = 1.0f / sqrtf(ss / (float)p.hidden + p.eps);
      for (int i = lane; i < quads; i += 32) {
        const float4 a = __ldcg(src + i), gi = g4[i];
        __nv_bfloat162 lo = __floats2bfloat162_rn((a.x * scale) * gi.x, (a.y * scale) * gi.y);
        __nv_bfloat162 hi = __floats2bfloat162_rn((a.z * scale) * gi.z, (a.w * scale) * gi.w);
        *(uint2*)(dst + (size_t)i * 8) = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  }
  __syncthreads();
  FFN_STAMP(3);
  if (!mbar_wait(&bars[0], 0)) failed = 1;
  __syncthreads();
  FFN_STAMP(4);
  const bool ok1 = failed == 0;
  ffn_cluster_wait();                                // every CTA of the cluster runs: their shared memory may be written

  // ---- gate/up: a warp per 16-row tile of the CTA's share (a CTA has at most 8), over the whole K.
  //      The tile's fragment holds gate rows 0-7 and their up rows 8-15 in the same thread, so SwiGLU
  //      is applied on the registers; the tile's 8 activation columns go into the shared memory of
  //      every CTA of the cluster.  Eight chains of products per tile (K steps 0, 8, 16.. / 1, 9, ..)
  //      keep the dependent `mma.sync` apart.
  if (warp < nt1) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (ok1) {
    const int ksteps1 = p.hidden >> 4;
    const uint32_t w1_addr = smem_u32(w1);
    const int a_row = warp * 16 + (lane & 15);
    const uint8_t* b_base = actbuf + (size_t)(lane >> 2) * p.stride1 + (lane & 3) * 4;
    constexpr int CHAINS = 8;
    float acc[CHAINS][4];
#pragma unroll
    for (int c = 0; c < CHAINS; c++) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;
    int k = 0;
    for (; k + CHAINS <= ksteps1; k += CHAINS) {
      uint32_t b[CHAINS][2], a[CHAINS][4];
#pragma unroll
      for (int u = 0; u < CHAINS; u++) {                  // all the loads of the steps, then their products
        const int kk = k + u;
        b[u][0] = *(const uint32_t*)(b_base + kk * 32);
        b[u][1] = *(const uint32_t*)(b_base + kk * 32 + 16);
        ldmatrix_x4(swizzled(w1_addr + (uint32_t)(kk >> 2) * p.box1_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                    a[u][0], a[u][1], a[u][2], a[u][3]);
      }
#pragma unroll
      for (int u = 0; u < CHAINS; u++) mma_bf16(acc[u], a[u][0], a[u][1], a[u][2], a[u][3], b[u][0], b[u][1]);
    }
    for (; k < ksteps1; k++) {
      uint32_t a0, a1, a2, a3;
      const uint32_t b0 = *(const uint32_t*)(b_base + k * 32), b1 = *(const uint32_t*)(b_base + k * 32 + 16);
      ldmatrix_x4(swizzled(w1_addr + (uint32_t)(k >> 2) * p.box1_bytes, a_row, (k & 3) * 2 + (lane >> 4)), a0, a1, a2, a3);
      mma_bf16(acc[0], a0, a1, a2, a3, b0, b1);
    }
#pragma unroll
    for (int j = 0; j < 4; j++)
      s[j] = ((acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j])) + ((acc[4][j] + acc[5][j]) + (acc[6][j] + acc[7][j]));
    }
    // fragment rows 0-7 are gate rows, rows 8-15 the matching up rows: (0, 2) and (1, 3) pair up
    const int col = (t1_begin - kt_begin + warp) * 8 + (lane >> 2), t0 = (lane & 3) * 2;
    const __nv_bfloat16 a0 = __float2bfloat16_rn(t0 < p.tokens ? ffn_silu_mul(s[0], s[2]) : 0.f);
    const __nv_bfloat16 a1 = __float2bfloat16_rn(t0 + 1 < p.tokens ? ffn_silu_mul(s[1], s[3]) : 0.f);
    const bool closes = (nkt & 1) && t1_begin + warp == kt_begin + nkt - 1;   // the cluster's last tile ends half a K step: the other half is zero
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (int q = 0; q < p.cluster; q++) {
      __nv_bfloat16* theirs = (__nv_bfloat16*)cluster.map_shared_rank(xchg, q);
      __nv_bfloat16* r0 = (__nv_bfloat16*)((uint8_t*)theirs + (size_t)t0 * p.stride_x);
      __nv_bfloat16* r1 = (__nv_bfloat16*)((uint8_t*)theirs + (size_t)(t0 + 1) * p.stride_x);
      r0[col] = a0;
      r1[col] = a1;
      if (closes) { r0[col + 8] = zero; r1[col + 8] = zero; }
    }
  }
  ffn_cluster_arrive();                              // this CTA's columns are written, here and in the other CTAs
  __syncthreads();                                   // the operand rows and the gate/up tiles have been read
  FFN_STAMP(5);
  // The gate/up weights have been used: this CTA's rows of the down matrix, over the cluster's K
  // range, take their place.  They arrive while the cluster meets.
  if (tid == 0 && has2) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t bar = smem_u32(&bars[1]);
    mbar_expect_tx(&bars[1], (uint32_t)(p.row_boxes2 * p.col_boxes2) * (uint32_t)p.box2_bytes);
    for (int cb = 0; cb < p.col_boxes2; cb++)
      for (int rb = 0; rb < p.row_boxes2; rb++)
        tma_load_2d_addr(smem_u32(w2) + (uint32_t)(cb * p.row_boxes2 + rb) * p.box2_bytes, &map_down, bar,
                         kt_begin * 8 + cb * 64, t2_begin * 16 + rb * p.box_rows2);
  }
  ffn_cluster_wait();                                // the cluster's activation columns are all here
  FFN_STAMP(6);
  if (has2 && !mbar_wait(&bars[1], 0)) failed = 1;
  __syncthreads();
  FFN_STAMP(7);

  // ---- down: this CTA's row tiles over the cluster's K range, added into the residual stream
  if (has2 && failed == 0) {
    const uint8_t* b_base = xchg + (size_t)(lane >> 2) * p.stride_x + (lane & 3) * 4;
    const uint32_t w2_addr = smem_u32(w2);
    for (int tile = warp; tile < nt2; tile += FFN_THREADS / 32) {
      float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};   // even and odd K steps: two chains of products
      const int row_in_part = tile * 16 + (lane & 15);
      const uint32_t box_row = w2_addr + (uint32_t)(row_in_part / p.box_rows2) * p.box2_bytes;
      const int a_row = row_in_part % p.box_rows2;
      for (int k = 0; k < ksteps2; k += 2) {
        const bool two = k + 1 < ksteps2;
        uint32_t b[2][2], a[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int kk = (u == 0 || two) ? k + u : k;
          b[u][0] = *(const uint32_t*)(b_base + kk * 32);
          b[u][1] = *(const uint32_t*)(b_base + kk * 32 + 16);
          ldmatrix_x4(swizzled(box_row + (uint32_t)((kk >> 2) * p.row_boxes2) * p.box2_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
                      a[u][0], a[u][1], a[u][2], a[u][3]);
        }
        mma_bf16(d, a[0][0], a[0][1], a[0][2], a[0][3], b[0][0], b[0][1]);
        if (two) mma_bf16(e, a[1][0], a[1][1], a[1][2], a[1][3], b[1][0], b[1][1]);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) d[j] += e[j];
      const int row = (t2_begin + tile) * 16 + (lane >> 2), t0 = (lane & 3) * 2;
      if (t0 < p.tokens) {
        atomicAdd(x + (size_t)t0 * p.hidden + row, d[0]);
        atomicAdd(x + (size_t)t0 * p.hidden + row + 8, d[2]);
      }
      if (t0 + 1 < p.tokens) {
        atomicAdd(x + (size_t)(t0 + 1) * p.hidden + row, d[1]);
        atomicAdd(x + (size_t)(t0 + 1) * p.hidden + row + 8, d[3]);
      }
    }
  }
  __syncthreads();
  FFN_STAMP(8);
  if (tid == 0 && failed) atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
  SPROUT_TL_EXIT(0);
}

// 9 to 16 tokens: two tiles of tokens.
__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_decode_kernel16(const __grid_constant__ CUtensorMap map_gu_base, const __grid_constant__ CUtensorMap map_gu_tile,
                    const __grid_constant__ CUtensorMap map_down, float* __restrict__ x, const float* __restrict__ gain,
                    int* status, const FfnPlan p) {
  ffn_decode_body<2>(map_gu_base, map_gu_tile, map_down, x, gain, status, p);
}

}  // namespace

namespace {

// The layout of a launch for these sizes on `ctas` CTAs in clusters of `cluster`; false when the
// sizes are outside the kernel's rules or a CTA's share of the weights does not fit in shared memory.
bool ffn_make_plan(int tokens, int hidden, int inter, int ctas, int cluster, float eps, FfnPlan* out) {
  if (tokens < 1 || tokens > FFN_MAX_TOKENS || hidden < 16 || inter < 16 || hidden % 16 || inter % 16) return false;
  if (cluster < 1 || cluster > 8 || (cluster & (cluster - 1)) || ctas < cluster || ctas % cluster) return false;
  FfnPlan p = {};
  p.tokens = tokens; p.hidden = hidden; p.inter = inter; p.eps = eps;
  p.rows_held = token_rows(tokens);
  p.ctas = ctas; p.cluster = cluster;
  p.tiles1 = inter / 8;
  p.tiles2 = hidden / 16;
  p.base_tiles1 = p.tiles1 / ctas;
  p.max_tiles1 = (p.tiles1 + ctas - 1) / ctas;
  if (p.max_tiles1 > FFN_MAX_TILES) return false;
  p.boxes1 = (hidden + 63) / 64;
  p.box1_bytes = p.max_tiles1 * 2048;
  p.stride1 = hidden * 2 + 16;
  // the down matrix: a cluster works on the K range its own CTAs produce; its CTAs share the rows
  p.max_tiles2 = (p.tiles2 + cluster - 1) / cluster;
  const int max_rows2 = p.max_tiles2 * 16;
  p.row_boxes2 = (max_rows2 + 255) / 256;
  p.box_rows2 = ((p.max_tiles2 + p.row_boxes2 - 1) / p.row_boxes2) * 16;
  p.max_ktiles = 0;
  for (int c = 0; c < ctas; c += cluster) {
    const int n = share_begin(p.tiles1, c + cluster, ctas) - share_begin(p.tiles1, c, ctas);
    if (n > p.max_ktiles) p.max_ktiles = n;
  }
  p.max_ksteps = (p.max_ktiles + 1) / 2;
  p.col_boxes2 = (p.max_ksteps + 3) / 4;
  p.box2_bytes = p.box_rows2 * 128;
  p.stride_x = p.max_ksteps * 32 + 16;
  long long at = (long long)p.boxes1 * p.box1_bytes;          // the down rows come where the gate/up tiles were
  const long long down = (long long)p.row_boxes2 * p.col_boxes2 * p.box2_bytes;
  if (down > at) at = down;
  p.off_w2 = 0;
  p.off_act = (int)at;
  at += (long long)p.rows_held * p.stride1;                   // the normalised rows
  p.off_xchg = (int)at;
  at += (((long long)p.rows_held * p.stride_x) + 15) / 16 * 16;   // the cluster's activation columns, written by all its CTAs
  p.off_bar = (int)at;
  at += 64 + 1024;                       // the barriers; room to start the tiles on a 1024-byte boundary
  if (at > FFN_SMEM_LIMIT) return false;
  p.smem_bytes = (int)at;
  *out = p;
  return true;
}

// How many CTAs, in clusters of how many, a launch gets on the current device: as many clusters as
// the device holds at once (all CTAs of the launch run together: a cluster that had to wait for a
// free place would double the kernel's time), the largest cluster size for which those cover
// nearly all SMs.  Asked once per device and size.
bool ffn_launch_shape(int hidden, int inter, int tokens, int* ctas_out, int* cluster_out) {
  tokens = token_rows(tokens);                       // the layout depends on the tiles of tokens, not on their number
  struct Known { int device, hidden, inter, tokens, ctas, cluster; };
  static Known known[16];
  static int known_count = 0;
  static std::mutex lock;
  int device = -1;
  const bool have_device = cudaGetDevice(&device) == cudaSuccess;
  if (!have_device) { cudaGetLastError(); device = -1; }
  std::lock_guard<std::mutex> guard(lock);
  for (int i = 0; i < known_count; i++)
    if (known[i].device == device && known[i].hidden == hidden && known[i].inter == inter && known[i].tokens == tokens) {
      *ctas_out = known[i].ctas; *cluster_out = known[i].cluster;
      return known[i].ctas > 0;
    }
  const int sms = sm_count();
  int best_ctas = 0, best_cluster = 0;
  const char* forced_text = getenv("SPROUT_FFN_CLUSTER");          // for measurements: this cluster size or none
  const int forced = forced_text ? atoi(forced_text) : 0;
  for (int cluster = 8; cluster >= 1; cluster >>= 1) {
    if (forced && cluster != forced) continue;
    int clusters = sms / cluster;
    FfnPlan plan;
    if (clusters < 1 || !ffn_make_plan(tokens, hidden, inter, clusters * cluster, cluster, 1e-6f, &plan)) continue;
    if (have_device && cluster > 1) {
      cudaLaunchConfig_t config = {};
      config.gridDim = dim3(clusters * cluster);
      config.blockDim = dim3(FFN_THREADS);
      config.dynamicSmemBytes = plan.smem_bytes;
      cudaLaunchAttribute attribute[1];
      attribute[0].id = cudaLaunchAttributeClusterDimension;
      attribute[0].val.clusterDim.x = cluster; attribute[0].val.clusterDim.y = 1; attribute[0].val.clusterDim.z = 1;
      config.attrs = attribute; config.numAttrs = 1;
      const void* kernel = tokens == 8 ? (const void*)ffn_decode_kernel8 : (const void*)ffn_decode_kernel16;
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FFN_SMEM_LIMIT);
      int active = 0;
      if (cudaOccupancyMaxActiveClusters(&active, kernel, &config) != cudaSuccess) { cudaGetLastError(); continue; }
      if (active < clusters) clusters = active;
      if (clusters < 1 || !ffn_make_plan(tokens, hidden, inter, clusters * cluster, cluster, 1e-6f, &plan)) continue;
    }
    // larger clusters mean fewer additions into the residual stream and more of the activation
    // exchanged on the SMs; they are taken as long as they leave no more than one SM in sixteen idle
    if (clusters * cluster * 16 >= sms * 15 || cluster == 1 || forced) { best_ctas = clusters * cluster; best_cluster = cluster; break; }
    if (clusters * cluster > best_ctas) { best_ctas = clusters * cluster; best_cluster = cluster; }
  }
  if (known_count < 16) known[known_count++] = Known{device, hidden, inter, tokens, best_ctas, best_cluster};
  *ctas_out = best_ctas; *cluster_out = best_cluster;
  return best_ctas > 0;
}

}  // namespace

// 1 when sprout_ffn_decode takes these sizes on this device, else 0.
SPROUT_API int sprout_ffn_decode_supported(int tokens, int hidden, int inter) {
  int ctas = 0, cluster = 0;
  FfnPlan plan;
  return ffn_launch_shape(hidden, inter, tokens, &ctas, &cluster) && ffn_make_plan(tokens, hidden, inter, ctas, cluster, 1e-6f, &plan) ? 1 : 0;
}

// The launch layout for these sizes on `ctas` CTAs in clusters of `cluster`, for inspection by
// host-side tests: 1 and the plan's numbers in `out` (in the order of the list below), or 0 when
// the sizes are refused.  ctas == 0: the shape the current device would get.
SPROUT_API int sprout_ffn_decode_plan(int tokens, int hidden, int inter, int ctas, int cluster, int* out) {
  FfnPlan p;
  if (!out) return 0;
  if (ctas == 0 && !ffn_launch_shape(hidden, inter, tokens, &ctas, &cluster)) return 0;
  if (!ffn_make_plan(tokens, hidden, inter, ctas, cluster, 1e-6f, &p)) return 0;
  const int fields[22] = {p.ctas, p.cluster, p.tiles1, p.base_tiles1, p.max_tiles1, p.boxes1, p.box1_bytes, p.tiles2, p.max_tiles2,
                          p.box_rows2, p.row_boxes2, p.max_ktiles, p.max_ksteps, p.col_boxes2, p.box2_bytes, p.stride1, p.stride_x,
                          p.off_w2, p.off_act, p.off_xchg, p.off_bar, p.smem_bytes};
  for (int i = 0; i < 22; i++) out[i] = fields[i];
  return 1;
}

// x [tokens, hidden] float32 += W_down (silu(W_gate h) * W_up h) with h = rmsnorm(x, gain, eps).
// w_gate_up: bfloat16 [2 * inter, hidden], gate and up rows interleaved in blocks of 8;
// w_down: bfloat16 [hidden, inter]; status: the device status word.
SPROUT_API int sprout_ffn_decode(float* x, const float* gain, const void* w_gate_up, const void* w_down, int* status,
                                 int tokens, int hidden, int inter, float eps, cudaStream_t stream) {
  FfnPlan plan;
  int ctas = 0, cluster = 0;
  SPROUT_REQUIRE(x && gain && w_gate_up && w_down && status, "ffn_decode: a pointer is missing");
  SPROUT_REQUIRE(eps > 0.f, "ffn_decode: eps must be positive");
  SPROUT_REQUIRE(ffn_launch_shape(hidden, inter, tokens, &ctas, &cluster) && ffn_make_plan(tokens, hidden, inter, ctas, cluster, eps, &plan),
                 "ffn_decode: tokens 1..%d, hidden and intermediate sizes multiples of 16 and a layer whose share per "
                 "CTA fits in shared memory (got tokens %d, hidden %d, intermediate %d)", FFN_MAX_TOKENS, tokens, hidden, inter);
  SPROUT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)w_gate_up & 15) == 0 &&
                 ((uintptr_t)w_down & 15) == 0, "ffn_decode: pointers must be 16-byte aligned");
  const int which = plan.rows_held == 8 ? 0 : 1;
  const void* kernel = which == 0 ? (const void*)ffn_decode_kernel8 : (const void*)ffn_decode_kernel16;
  static bool configured[2] = {false, false};
  if (!configured[which]) {
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FFN_SMEM_LIMIT);
    SPROUT_REQUIRE(err == cudaSuccess, "ffn_decode: cudaFuncSetAttribute failed: %s", cudaGetErrorString(err));
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured[which] = true;
  }
  CUtensorMap map_base, map_tile, map_down;
  if (tensor_map(w_gate_up, 2 * inter, hidden, hidden, 16, &map_tile)) return 1;
  map_base = map_tile;
  if (plan.base_tiles1 > 0 && tensor_map(w_gate_up, 2 * inter, hidden, hidden, plan.base_tiles1 * 16, &map_base)) return 1;
  if (tensor_map(w_down, hidden, inter, inter, plan.box_rows2, &map_down)) return 1;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(FFN_THREADS);
  config.dynamicSmemBytes = (size_t)plan.smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = cluster;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = sprout_pdl_enabled() ? 2 : 1;
  cudaError_t err = which == 0 ? cudaLaunchKernelEx(&config, ffn_decode_kernel8, map_base, map_tile, map_down, x, gain, status, plan)
                               : cudaLaunchKernelEx(&config, ffn_decode_kernel16, map_base, map_tile, map_down, x, gain, status, plan);
  SPROUT_REQUIRE(err == cudaSuccess, "ffn_decode: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

SPROUT_TL_READER(ffn_decode)
