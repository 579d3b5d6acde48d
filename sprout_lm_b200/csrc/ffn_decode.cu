// Decode feed-forward of a small model in ONE kernel: RMSNorm, gate/up product, SwiGLU, down
// product and the residual sum, for up to 8 tokens (one per request).
//
// Why: a decode step of a small model is a chain of short kernels, each of which costs a few
// microseconds whatever it computes (launch, first load, drain).  The norm, the gate/up product
// and the down product are three links of that chain per layer; here they are one launch whose
// two halves are separated by a barrier among its own CTAs (about 1.2 us) instead.
//
// How: one CTA per SM.  Every CTA owns a contiguous share of the 16-row tiles of the interleaved
// gate/up matrix (rows 16b..16b+7 gate, 16b+8..16b+15 up) and one (row group, K range) piece of
// the down matrix, and asks for its gate/up weights by TMA tile copies (boxes of 64 columns,
// 128-byte swizzle: a dozen large copies, not a copy per row) into its shared memory before it
// waits for the kernels before it; its piece of the down matrix takes the same room as soon as
// the gate/up products are done and arrives while the CTAs meet at the barrier.  With under
// 160 KB of shared memory at the 0.5B sizes the CTA fits beside a CTA of the attention kernel,
// so the weights stream from memory while the attention half of the layer still runs.  After
// the wait each warp normalises one token's row of the residual stream (float32 arithmetic) into
// a bfloat16 operand in shared memory; the products run on `mma.sync.m16n8k16` with the weights as the 16-row operand and the
// tokens as the 8 columns (for eight tokens the tensor cores' rate does not matter, latency
// does); a warp takes a 16-row tile over the whole K, so the gate value and its up value end up
// in one thread's registers, SwiGLU is applied there and the activation goes to memory as
// bfloat16 [tokens, intermediate].  After the barrier each CTA multiplies its piece
// of the down matrix with its K range of the activation and adds the result into the float32
// residual stream with atomic adds (the order of those float32 additions is not fixed).
//
// Sizes: tokens 1..8, hidden and intermediate sizes multiples of 16, and a layer whose per-CTA
// share of the weights fits in shared memory (sprout_ffn_decode_supported says); larger models
// keep the separate kernels, whose products are bound by bandwidth, not by latency.
//
// Every wait is bounded: an mbarrier or barrier wait that runs out sets the status word's
// WAIT_TIMEOUT bit, the CTA skips its arithmetic but still arrives at the barrier and leaves.
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

constexpr int FFN_THREADS = 256;            // 8 warps
constexpr int FFN_MAX_TOKENS = SMALL_MAX_TOKENS;
constexpr int FFN_MAX_TILES = FFN_THREADS / 32;   // gate/up tiles of a CTA: a warp each
constexpr int FFN_SMEM_LIMIT = 227 * 1024 - 1024;   // dynamic shared memory; the rest is for the kernel's static variables
constexpr uint32_t FFN_SPIN_LIMIT = 1u << 21;     // polls of the barrier counter (an L2 round trip each): a second or so

struct FfnPlan {
  int tokens, hidden, inter;
  int tiles1;            // 16-row tiles of the gate/up matrix: inter / 8
  int tiles2, ksteps2;   // 16-row tiles of the down matrix (hidden / 16), its 16-wide K steps (inter / 16)
  int row_groups, k_splits;   // pieces of the down product: row_groups * k_splits <= CTAs
  int base_tiles1, max_tiles1, max_tiles2, max_ksteps2;   // base_tiles1: what every CTA has at least (some have one more)
  int boxes1, boxes2;    // 64-column boxes along K of a CTA's gate/up rows, of its piece of the down matrix
  int box1_bytes, box2_bytes;
  int stride1;           // bytes between the tokens' rows of the normalised operand in shared memory
  int off_w2, off_act, off_bar, smem_bytes;
  float eps;
  unsigned spin_limit;   // polls of the barrier among the CTAs before a CTA gives up
};

__device__ __forceinline__ float ffn_silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// Barrier among all CTAs of the grid (all are resident: one per SM or fewer).  False when the
// bounded wait ran out.
__device__ __forceinline__ bool ffn_grid_barrier(unsigned* arrived, unsigned ctas, unsigned spin_limit) {
  __shared__ int passed;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrived, 1u);
    int ok = 0;
    for (uint32_t spins = 0; spins < spin_limit; spins++) {
      unsigned seen;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrived) : "memory");
      if (seen >= ctas) { ok = 1; break; }
    }
    passed = ok;
  }
  __syncthreads();
  return passed != 0;
}

}  // namespace

namespace {

__global__ void __launch_bounds__(FFN_THREADS, 1)
ffn_decode_kernel(const __grid_constant__ CUtensorMap map_gu_base, const __grid_constant__ CUtensorMap map_gu_tile,
                  const __grid_constant__ CUtensorMap map_down, float* __restrict__ x, const float* __restrict__ gain,
                  __nv_bfloat16* __restrict__ act, unsigned* sync, int* status, const FfnPlan p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);   // swizzled tiles start on 1024 bytes
  __shared__ int failed;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cta = blockIdx.x, ctas = gridDim.x;
  uint8_t* w1 = smem;
  uint8_t* w2 = smem + p.off_w2;
  uint8_t* actbuf = smem + p.off_act;
  uint64_t* bars = (uint64_t*)(smem + p.off_bar);

  pdl_launch_dependents();
  SPROUT_TL_ENTRY(0);
  FFN_STAMP(0);

  // this CTA's share of the gate/up tiles and its piece of the down matrix
  const int t1_begin = share_begin(p.tiles1, cta, ctas);
  const int nt1 = share_begin(p.tiles1, cta + 1, ctas) - t1_begin;
  const bool has2 = cta < p.row_groups * p.k_splits;
  const int group = has2 ? cta / p.k_splits : 0, split = has2 ? cta % p.k_splits : 0;
  const int t2_begin = share_begin(p.tiles2, group, p.row_groups);
  const int nt2 = has2 ? share_begin(p.tiles2, group + 1, p.row_groups) - t2_begin : 0;
  const int k2_begin = share_begin(p.ksteps2, split, p.k_splits);
  const int nk2 = has2 ? share_begin(p.ksteps2, split + 1, p.k_splits) - k2_begin : 0;

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
    const int count = (FFN_MAX_TOKENS - p.tokens) * (p.stride1 >> 4);
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

  // ---- gate/up: a warp per 16-row tile of the CTA's share (a CTA has at most 8), over the whole K.
  //      The tile's fragment holds gate rows 0-7 and their up rows 8-15 in the same thread, so SwiGLU
  //      is applied on the registers and the activation goes straight to memory: nothing is
  //      gathered among the warps.  Eight chains of products per tile (K steps 0, 8, 16.. / 1, 9, ..)
  //      keep the dependent `mma.sync` apart.
  if (ok1 && warp < nt1) {
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
    float s[4];
#pragma unroll
    for (int j = 0; j < 4; j++)
      s[j] = ((acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j])) + ((acc[4][j] + acc[5][j]) + (acc[6][j] + acc[7][j]));
    // fragment rows 0-7 are gate rows, rows 8-15 the matching up rows: (0, 2) and (1, 3) pair up
    const int col = (t1_begin + warp) * 8 + (lane >> 2), t0 = (lane & 3) * 2;
    if (t0 < p.tokens) act[(size_t)t0 * p.inter + col] = __float2bfloat16_rn(ffn_silu_mul(s[0], s[2]));
    if (t0 + 1 < p.tokens) act[(size_t)(t0 + 1) * p.inter + col] = __float2bfloat16_rn(ffn_silu_mul(s[1], s[3]));
  }
  __syncthreads();                                   // the operand rows and the gate/up tiles have been read
  FFN_STAMP(5);
  // The gate/up weights have been used: this CTA's piece of the down matrix takes their place.
  // It arrives while the CTAs meet at the barrier.
  if (tid == 0 && has2) {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const uint32_t bar = smem_u32(&bars[1]);
    mbar_expect_tx(&bars[1], (uint32_t)p.boxes2 * (uint32_t)p.box2_bytes);
    for (int b = 0; b < p.boxes2; b++)
      tma_load_2d_addr(smem_u32(w2) + (uint32_t)b * p.box2_bytes, &map_down, bar, k2_begin * 16 + b * 64, t2_begin * 16);
  }

  // ---- every CTA's share of the activation is in memory after this
  const bool through = ffn_grid_barrier(sync, (unsigned)ctas, p.spin_limit);
  FFN_STAMP(6);
  if (!through && tid == 0) failed = 1;

  // ---- down: this CTA's K range of the activation into shared memory, then its row tiles
  const int stride_b = nk2 * 32 + 16;
  if (has2) {
    const int chunks = nk2 * 2;                      // 16-byte pieces per token
    for (int i = tid; i < FFN_MAX_TOKENS * chunks; i += FFN_THREADS) {
      const int t = i / chunks, c = i - t * chunks;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t < p.tokens) v = __ldcg((const uint4*)(act + (size_t)t * p.inter + (size_t)k2_begin * 16) + c);
      *(uint4*)(actbuf + (size_t)t * stride_b + c * 16) = v;
    }
  }
  __syncthreads();
  FFN_STAMP(7);
  if (has2 && !mbar_wait(&bars[1], 0)) failed = 1;
  __syncthreads();
  FFN_STAMP(8);
  if (has2 && failed == 0) {
    const uint8_t* b_base = actbuf + (size_t)(lane >> 2) * stride_b + (lane & 3) * 4;
    for (int tile = warp; tile < nt2; tile += FFN_THREADS / 32) {
      float d[4] = {0.f, 0.f, 0.f, 0.f}, e[4] = {0.f, 0.f, 0.f, 0.f};   // even and odd K steps: two chains of products
      const uint32_t w2_addr = smem_u32(w2);
      const int a_row = tile * 16 + (lane & 15);
      for (int k = 0; k < nk2; k += 2) {
        const bool two = k + 1 < nk2;
        uint32_t b[2][2], a[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int kk = (u == 0 || two) ? k + u : k;
          b[u][0] = *(const uint32_t*)(b_base + kk * 32);
          b[u][1] = *(const uint32_t*)(b_base + kk * 32 + 16);
          ldmatrix_x4(swizzled(w2_addr + (uint32_t)(kk >> 2) * p.box2_bytes, a_row, (kk & 3) * 2 + (lane >> 4)),
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
  FFN_STAMP(9);
  if (tid == 0) {
    if (failed) atomicOr(status, (int)SPROUT_STATUS_WAIT_TIMEOUT);
    // the last CTA to leave puts the barrier's counters back to zero for the next launch
    __threadfence();
    if (atomicAdd(sync + 1, 1u) == (unsigned)ctas - 1) {
      sync[0] = 0u;
      sync[1] = 0u;
    }
  }
  SPROUT_TL_EXIT(0);
}

}  // namespace

namespace {

unsigned g_spin_limit = FFN_SPIN_LIMIT;

// The layout of a launch for these sizes on `ctas` CTAs; false when the sizes are outside the
// kernel's rules or a CTA's share of the weights does not fit in shared memory.
bool ffn_make_plan(int tokens, int hidden, int inter, int ctas, float eps, FfnPlan* out) {
  if (tokens < 1 || tokens > FFN_MAX_TOKENS || hidden < 16 || inter < 16 || hidden % 16 || inter % 16 || ctas < 1) return false;
  FfnPlan p = {};
  p.tokens = tokens; p.hidden = hidden; p.inter = inter; p.eps = eps;
  p.spin_limit = g_spin_limit;
  p.tiles1 = inter / 8;
  p.tiles2 = hidden / 16;
  p.ksteps2 = inter / 16;
  p.base_tiles1 = p.tiles1 / ctas;
  p.max_tiles1 = (p.tiles1 + ctas - 1) / ctas;
  if (p.max_tiles1 > FFN_MAX_TILES) return false;
  if (!plan_pieces(p.tiles2, p.ksteps2, ctas, &p.row_groups, &p.k_splits)) return false;
  p.max_tiles2 = (p.tiles2 + p.row_groups - 1) / p.row_groups;
  p.max_ksteps2 = (p.ksteps2 + p.k_splits - 1) / p.k_splits;
  p.boxes1 = (hidden + 63) / 64;
  p.boxes2 = (p.max_ksteps2 + 3) / 4;
  p.box1_bytes = p.max_tiles1 * 2048;
  p.box2_bytes = p.max_tiles2 * 2048;
  p.stride1 = hidden * 2 + 16;
  const int stride_b = p.max_ksteps2 * 32 + 16;
  long long at = (long long)p.boxes1 * p.box1_bytes;          // the down piece comes where the gate/up tiles were
  if ((long long)p.boxes2 * p.box2_bytes > at) at = (long long)p.boxes2 * p.box2_bytes;
  p.off_w2 = 0;
  p.off_act = (int)at;
  long long act_room = (long long)FFN_MAX_TOKENS * p.stride1;                       // the normalised rows,
  if ((long long)FFN_MAX_TOKENS * stride_b > act_room) act_room = (long long)FFN_MAX_TOKENS * stride_b;   // then the activation's K range
  at += act_room;
  p.off_bar = (int)at;
  at += 64 + 1024;                       // the barriers; room to start the tiles on a 1024-byte boundary
  if (at > FFN_SMEM_LIMIT) return false;
  p.smem_bytes = (int)at;
  *out = p;
  return true;
}

}  // namespace

// How often a CTA of sprout_ffn_decode polls the barrier among the CTAs before it gives up, sets the
// status word's WAIT_TIMEOUT bit and leaves (0: the default, about a second).  For tests of that path.
SPROUT_API void sprout_set_spin_limit(unsigned polls) { g_spin_limit = polls ? polls : FFN_SPIN_LIMIT; }

// 1 when sprout_ffn_decode takes these sizes on this device, else 0.
SPROUT_API int sprout_ffn_decode_supported(int tokens, int hidden, int inter) {
  FfnPlan plan;
  return ffn_make_plan(tokens, hidden, inter, sm_count(), 1e-6f, &plan) ? 1 : 0;
}

// The launch layout for these sizes on `ctas` CTAs, for inspection by host-side tests: 1 and the
// plan's 18 numbers in `out` (in the order of the list below), or 0 when the sizes are refused.
SPROUT_API int sprout_ffn_decode_plan(int tokens, int hidden, int inter, int ctas, int* out) {
  FfnPlan p;
  if (!out || !ffn_make_plan(tokens, hidden, inter, ctas, 1e-6f, &p)) return 0;
  const int fields[18] = {p.tiles1, p.tiles2, p.ksteps2, p.row_groups, p.k_splits, p.base_tiles1, p.max_tiles1, p.max_tiles2,
                          p.max_ksteps2, p.boxes1, p.boxes2, p.box1_bytes, p.box2_bytes, p.stride1, p.off_w2, p.off_act,
                          p.off_bar, p.smem_bytes};
  for (int i = 0; i < 18; i++) out[i] = fields[i];
  return 1;
}

// x [tokens, hidden] float32 += W_down (silu(W_gate h) * W_up h) with h = rmsnorm(x, gain, eps).
// w_gate_up: bfloat16 [2 * inter, hidden], gate and up rows interleaved in blocks of 8;
// w_down: bfloat16 [hidden, inter]; act: bfloat16 scratch [tokens, inter]; sync: two 32-bit
// words that are zero before the first launch (the kernel leaves them zero); status: the
// device status word.
SPROUT_API int sprout_ffn_decode(float* x, const float* gain, const void* w_gate_up, const void* w_down, void* act,
                                 void* sync, int* status, int tokens, int hidden, int inter, float eps,
                                 cudaStream_t stream) {
  FfnPlan plan;
  SPROUT_REQUIRE(x && gain && w_gate_up && w_down && act && sync && status, "ffn_decode: a pointer is missing");
  SPROUT_REQUIRE(eps > 0.f, "ffn_decode: eps must be positive");
  SPROUT_REQUIRE(ffn_make_plan(tokens, hidden, inter, sm_count(), eps, &plan),
                 "ffn_decode: tokens 1..%d, hidden and intermediate sizes multiples of 16 and a layer whose share per "
                 "CTA fits in shared memory (got tokens %d, hidden %d, intermediate %d)", FFN_MAX_TOKENS, tokens, hidden, inter);
  SPROUT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)w_gate_up & 15) == 0 &&
                 ((uintptr_t)w_down & 15) == 0 && ((uintptr_t)act & 15) == 0 && ((uintptr_t)sync & 3) == 0,
                 "ffn_decode: pointers must be 16-byte aligned");
  static int smem_set = 0;
  if (plan.smem_bytes > smem_set) {
    cudaError_t err = cudaFuncSetAttribute(ffn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FFN_SMEM_LIMIT);
    SPROUT_REQUIRE(err == cudaSuccess, "ffn_decode: cudaFuncSetAttribute failed: %s", cudaGetErrorString(err));
    cudaFuncSetAttribute(ffn_decode_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    smem_set = FFN_SMEM_LIMIT;
  }
  CUtensorMap map_base, map_tile, map_down;
  if (tensor_map(w_gate_up, 2 * inter, hidden, hidden, 16, &map_tile)) return 1;
  map_base = map_tile;
  if (plan.base_tiles1 > 0 && tensor_map(w_gate_up, 2 * inter, hidden, hidden, plan.base_tiles1 * 16, &map_base)) return 1;
  if (tensor_map(w_down, hidden, inter, inter, plan.max_tiles2 * 16, &map_down)) return 1;
  cudaError_t err = sprout_launch(ffn_decode_kernel, dim3(sm_count()), dim3(FFN_THREADS), (size_t)plan.smem_bytes, stream,
                                  map_base, map_tile, map_down, x, gain, (__nv_bfloat16*)act, (unsigned*)sync, status, plan);
  SPROUT_REQUIRE(err == cudaSuccess, "ffn_decode: launch failed: %s", cudaGetErrorString(err));
  return 0;
}

SPROUT_TL_READER(ffn_decode)
