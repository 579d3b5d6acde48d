// Prefill attention over the paged cache on the fifth-generation tensor cores (sm_100a).
//
// One CTA owns 128 rows, a row being a (token, query head) pair of one request and one key/value
// head, and walks the request's keys in tiles of 128:
//
//   S = Q K^T      tcgen05.mma, Q and K K-major in shared memory, S in tensor memory (2 buffers)
//   softmax        four warps, one thread per row: tcgen05.ld of its row of S, running maximum and
//                  sum in float32, P = exp2(..) written as bfloat16 into shared memory in the
//                  K-major swizzled layout the next product reads
//   O_tile = P V   tcgen05.mma, V as it lies in the cache ([key, head_dim]: MN-major B operand),
//                  the tile's product in tensor memory; the row's thread adds it to its float32
//                  accumulator in registers, rescaled when the maximum moved
//
// K and V tiles come by TMA, one box per page (a page of one head is `page_tokens` contiguous
// rows of the cache), through a two-stage ring.  One warp looks the pages up and issues the
// copies (a lane per box), one thread issues the MMAs.  With head_dim 64 two CTAs share an SM, and
// the softmax of one runs under the MMAs of the other; with head_dim 128 there is one CTA per SM,
// S has two buffers and S(j+1) is issued before P(j) V(j), so that it runs under the softmax of
// tile j.
// Every mbarrier wait is bounded: on a timeout the CTA sets the status word, waits (bounded) for
// its copies in flight, frees its tensor memory and returns.
//
// Takes head_dim 64 or 128 and page sizes that divide 128 (from 8) or are multiples of 128; the
// mma.sync kernel in attention_bf16.cu takes everything else.
#include <cuda_bf16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int TC_ROWS = 128, TC_KEYS = 128, KV_STAGES = 2;
constexpr int TC_THREADS = 256;           // warpgroup 0: copy warp, MMA warp (two warps idle); warpgroup 1: softmax
constexpr int ATOM_BYTES = 128 * 128;     // a [128 rows, 64 bf16] swizzled tile

struct TcParams {
  const __nv_bfloat16* q; int q_stride;
  const int* block_table; int table_stride;
  const int* q_start;                 // [requests + 1]
  const int* positions;               // [tokens]
  __nv_bfloat16* out; int out_stride;
  int requests, heads, kv_heads, page_tokens, num_pages, box_rows;
  float scale;
  int* status;
};

// head_dim 64: one S buffer, 112 KB of shared memory, 256 columns of tensor memory and 128
// registers a thread at launch, so that two CTAs share an SM and one's softmax runs under the
// other's MMAs; the softmax warpgroup takes the registers that the other warpgroup gives up.
// head_dim 128: the row's 128 accumulators leave room for one CTA per SM; S has two buffers,
// and S(j+1) runs under the softmax of tile j.
template <int HD>
struct TcLayout {
  static constexpr int KB = HD / 64;                       // 64-element blocks along head_dim
  static constexpr int CTAS_PER_SM = HD == 64 ? 2 : 1;
  static constexpr int S_BUFFERS = HD == 64 ? 1 : 2;
  static constexpr int TMEM_COLS = HD == 64 ? 256 : 512;   // S buffers, then the O tile
  static constexpr int O_COLUMN = S_BUFFERS * TC_KEYS;
  static constexpr int Q_BYTES = KB * ATOM_BYTES;
  static constexpr int KV_BYTES = KB * ATOM_BYTES;         // one stage of K (or of V)
  static constexpr int P_BYTES = 2 * ATOM_BYTES;           // [128 rows, 128 keys]
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 128;
};

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int HD>
__global__ void __launch_bounds__(TC_THREADS, TcLayout<HD>::CTAS_PER_SM)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const TcParams p) {
  using L = TcLayout<HD>;
  // no static shared memory and no slack: the swizzled tiles need the dynamic region to start on
  // a 1024-byte boundary, which is checked below
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sQ = smem;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;
  uint8_t* sP = smem + L::OFF_P;
  uint64_t* bars = (uint64_t*)(smem + L::OFF_BAR);
  uint64_t* k_full = bars;            // [2] copies of a K stage have landed
  uint64_t* k_empty = bars + 2;       // [2] the MMAs that read a K stage have completed
  uint64_t* v_full = bars + 4;
  uint64_t* v_empty = bars + 6;
  uint64_t* s_full = bars + 8;        // [2] S of a tile is complete in tensor memory
  uint64_t* p_full = bars + 10;       // [1] P of a tile is written to shared memory (4 warps arrive)
  uint64_t* o_full = bars + 11;       // [1] P V of a tile is complete in tensor memory
  uint32_t* tmem_slot = (uint32_t*)(bars + 12);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = blockIdx.x % p.kv_heads;
  const int group = p.heads / p.kv_heads;

  // which request and which 128-row tile of it: the tiles of a request are handed out from the
  // last (the longest under the causal mask) to the first, the heads of a tile side by side
  int r = 0, tile = blockIdx.x / p.kv_heads;
  for (; r < p.requests; r++) {
    const int tiles = ((p.q_start[r + 1] - p.q_start[r]) * group + TC_ROWS - 1) / TC_ROWS;
    if (tile < tiles) { tile = tiles - 1 - tile; break; }
    tile -= tiles;
  }
  if (r >= p.requests) return;
  if ((smem_u32(smem) & 1023) != 0) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_LAYOUT);
    return;
  }
  const int q0 = p.q_start[r], q_count = p.q_start[r + 1] - q0;
  const int rows_total = q_count * group;
  const int row_base = tile * TC_ROWS;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  // positions grow with the row index: the last row of the tile sees the most keys
  const int max_limit = p.positions[q0 + (min(rows_total, row_base + TC_ROWS) - 1) / group];
  const int n_tiles = max_limit / TC_KEYS + 1;

  // rows of a stage that no copy fills (keys beyond the request) must hold finite numbers: their
  // probabilities are zero, and zero times a stale NaN is not
  for (int i = tid; i < 2 * KV_STAGES * L::KV_BYTES / 16; i += TC_THREADS) ((uint4*)sK)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < 10; i++) mbar_init(&bars[i], 1);
    mbar_init(&p_full[0], 4);
    mbar_init(&o_full[0], 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, L::TMEM_COLS);

  // Q rows -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r at chunk
  // position c ^ (r & 7)), one 16 KB atom per 64 elements of head_dim; a row is a (token, head) pair
  constexpr int CHUNKS = HD / 8;
  for (int idx = tid; idx < TC_ROWS * CHUNKS; idx += TC_THREADS) {
    const int row = idx / CHUNKS, c = idx % CHUNKS;
    const int gi = row_base + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gi < rows_total)
      v = *(const uint4*)(p.q + (size_t)(q0 + gi / group) * p.q_stride + (size_t)(g * group + gi % group) * HD + c * 8);
    *(uint4*)(sQ + (c >> 3) * ATOM_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int k_issued = 0, v_issued = 0;                     // tiles whose copies were issued (lane 0 of the producer warp)
  if (warp < 4) {
#ifndef PROBE_NO_SETMAXNREG
  if (L::CTAS_PER_SM == 2) warpgroup_regs_give<56>();
#endif
  if (warp == 0) {
    // ---------------- producer: one TMA box per page (or per 128 keys of a larger page); lane b
    // looks box b's page up and issues its copies, lane 0 waits for the stage and posts the bytes
    const int boxes = TC_KEYS / p.box_rows;
    auto box_row = [&](int j) {
      const int key = j * TC_KEYS + lane * p.box_rows;
      if (lane >= boxes || j >= n_tiles || key > max_limit) return -1;
      const int page = table[key / p.page_tokens];
      if (page < 0 || page >= p.num_pages) { atomicOr(p.status, SPROUT_STATUS_BAD_PAGE); return -1; }
      return (page * p.kv_heads + g) * p.page_tokens + key % p.page_tokens;
    };
    int next_row = box_row(0);
    for (int j = 0; j < n_tiles; j++) {
      const int s = j % KV_STAGES;
      const uint32_t parity = ((j / KV_STAGES) & 1) ^ 1;
      const int row_at = next_row;
      const uint32_t bytes = (uint32_t)__popc(__ballot_sync(0xffffffffu, row_at >= 0)) * p.box_rows * 128 * L::KB;
      bool ok = true;
      if (lane == 0) {
        ok = !*abort_flag && mbar_wait(&k_empty[s], parity);
        if (ok) mbar_expect_tx(&k_full[s], bytes);
        else { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (row_at >= 0)
        for (int kb = 0; kb < L::KB; kb++)
          tma_load_2d(sK + s * L::KV_BYTES + kb * ATOM_BYTES + lane * p.box_rows * 128, &map_k, &k_full[s], kb * 64, row_at);
      k_issued = j + 1;
      next_row = box_row(j + 1);                      // the lookup runs under the wait below
      if (lane == 0) {
        ok = !*abort_flag && mbar_wait(&v_empty[s], parity);
        if (ok) mbar_expect_tx(&v_full[s], bytes);
        else { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      }
      if (!__shfl_sync(0xffffffffu, ok, 0)) break;
      if (row_at >= 0)
        for (int kb = 0; kb < L::KB; kb++)
          tma_load_2d(sV + s * L::KV_BYTES + kb * ATOM_BYTES + lane * p.box_rows * 128, &map_v, &v_full[s], kb * 64, row_at);
      v_issued = j + 1;
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    const uint32_t idesc_s = umma_idesc(TC_ROWS, TC_KEYS);
    const uint32_t idesc_o = umma_idesc_b_mn(TC_ROWS, HD);
    bool ok = true;
    auto issue_s = [&](int j) {
      const int s = j % KV_STAGES;
      if (*abort_flag || !mbar_wait(&k_full[s], (j / KV_STAGES) & 1)) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); ok = false; return; }
      tc_fence_after();
      const uint32_t d = tmem_base + (j % L::S_BUFFERS) * TC_KEYS;
#pragma unroll
      for (int kb = 0; kb < L::KB; kb++) {
        const uint64_t a = umma_smem_desc(sQ + kb * ATOM_BYTES), b = umma_smem_desc(sK + s * L::KV_BYTES + kb * ATOM_BYTES);
#pragma unroll
        for (int kk = 0; kk < 4; kk++) umma_bf16(d, a + 2 * kk, b + 2 * kk, idesc_s, (kb | kk) != 0);
      }
      umma_commit(&k_empty[s]);
      umma_commit(&s_full[j % L::S_BUFFERS]);
    };
    issue_s(0);
    for (int j = 0; j < n_tiles && ok; j++) {
      // with two S buffers, S of the next tile runs under the softmax of this one (its buffer held
      // S(j-1), which the softmax warps had read before they signalled P(j-1)); with one, it
      // follows P(j) V(j), after the softmax warps have read S(j)
      if (L::S_BUFFERS == 2 && j + 1 < n_tiles) { issue_s(j + 1); if (!ok) break; }
      const int s = j % KV_STAGES;
      if (*abort_flag || !mbar_wait(&p_full[0], j & 1) || !mbar_wait(&v_full[s], (j / KV_STAGES) & 1)) {
        *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); break;
      }
      tc_fence_after();
#pragma unroll
      for (int ks = 0; ks < TC_KEYS / 16; ks++) {
        const uint64_t a = umma_smem_desc(sP + (ks >> 2) * ATOM_BYTES) + 2 * (ks & 3);
        const uint64_t b = umma_smem_desc_mn(sV + s * L::KV_BYTES + ks * 2048, ATOM_BYTES);
        umma_bf16(tmem_base + L::O_COLUMN, a, b, idesc_o, ks != 0);
      }
      umma_commit(&v_empty[s]);
      umma_commit(&o_full[0]);
      if (L::S_BUFFERS == 1 && j + 1 < n_tiles) issue_s(j + 1);
    }
  }
  } else {
    // ---------------- softmax and accumulation: one thread per row
#ifndef PROBE_NO_SETMAXNREG
    if (L::CTAS_PER_SM == 2) warpgroup_regs_take<200>();
#endif
    const int quarter = warp & 3;                      // a warp reads TMEM lanes 32 * (warp % 4) ..
    const int row = quarter * 32 + lane;
    const int gi = row_base + row;
    const bool row_valid = gi < rows_total;
    const int token = q0 + (row_valid ? gi / group : 0), head = g * group + gi % group;
    const int limit = row_valid ? p.positions[token] : -1;   // last visible key of the row
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; i++) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;                      // running maximum of the unscaled scores, running sum
    bool ok = true;
    for (int j = 0; j < n_tiles; j++) {
      ok = !*abort_flag && mbar_wait(&s_full[j % L::S_BUFFERS], (j / L::S_BUFFERS) & 1);
      if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      ok = __all_sync(0xffffffffu, ok);                // tcgen05.ld is warp-wide: all lanes or none
      if (!ok) break;
      tc_fence_after();
      const int kv0 = j * TC_KEYS;
      const uint32_t s_addr = lane_addr + (j % L::S_BUFFERS) * TC_KEYS;
      const bool masked = kv0 + TC_KEYS - 1 > limit;   // some key of the tile lies beyond this row's limit
      // first pass over the row: its maximum
      float t_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < TC_KEYS / 64; c++) {
        uint32_t ra[32], rb[32];
        tmem_load32_issue(s_addr + c * 64, ra);
        tmem_load32_issue(s_addr + c * 64 + 32, rb);
        tmem_load_wait(ra);
        tmem_load_wait(rb);
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; i++) {
            if (kv0 + c * 64 + i <= limit) t_max = fmaxf(t_max, __uint_as_float(ra[i]));
            if (kv0 + c * 64 + 32 + i <= limit) t_max = fmaxf(t_max, __uint_as_float(rb[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i++) t_max = fmaxf(t_max, fmaxf(__uint_as_float(ra[i]), __uint_as_float(rb[i])));
        }
      }
      const float n = fmaxf(m, t_max);
      const float base = n == -INFINITY ? 0.f : n * scale_log2;
      const float alpha = m == -INFINITY ? 0.f : exp2f(m * scale_log2 - base);
      m = n;
      // the previous tile's P V: add it, then bring everything to the new maximum
      if (j > 0) {
        ok = !*abort_flag && mbar_wait(&o_full[0], (j - 1) & 1);
        if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; c++) {
          uint32_t raw[32];
          tmem_load32(lane_addr + L::O_COLUMN + c * 32, raw);
#pragma unroll
          for (int i = 0; i < 32; i++) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(raw[i])) * alpha;
        }
      }
      l *= alpha;
      // second pass: probabilities, their sum, and P as bfloat16 into shared memory (the P V
      // product of the previous tile, which read the buffer, is complete: o_full above)
      uint8_t* p_row = sP + row * 128;
#pragma unroll 1
      for (int c = 0; c < TC_KEYS / 32; c++) {
        uint32_t raw[32];
        tmem_load32(s_addr + c * 32, raw);
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = exp2f(fmaf(__uint_as_float(raw[i]), scale_log2, -base));
          float p1 = exp2f(fmaf(__uint_as_float(raw[i + 1]), scale_log2, -base));
          if (masked) {
            if (kv0 + c * 32 + i > limit) p0 = 0.f;
            if (kv0 + c * 32 + i + 1 > limit) p1 = 0.f;
          }
          l += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *(uint32_t*)&h;
        }
        uint8_t* atom = p_row + (c >> 1) * ATOM_BYTES;
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
          const int chunk = (c & 1) * 4 + q4;
          *(uint4*)(atom + ((chunk ^ (row & 7)) << 4)) = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      if (j == n_tiles - 1 && kv0 + row > max_limit) {
        // the last tile's pages may reach beyond the request's keys, into slots that hold whatever
        // was there before: their probabilities are zero, but zero times a NaN is not, so the V
        // row of such a key is cleared once its copy has landed
        const int s = j % KV_STAGES;
        if (*abort_flag || !mbar_wait(&v_full[s], (j / KV_STAGES) & 1)) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
#pragma unroll
        for (int kb = 0; kb < L::KB; kb++)
#pragma unroll
          for (int c = 0; c < 8; c++) *(uint4*)(sV + s * L::KV_BYTES + kb * ATOM_BYTES + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[0]);
    }
    if (ok) {
      ok = !*abort_flag && mbar_wait(&o_full[0], (n_tiles - 1) & 1);
      if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < HD / 32; c++) {
        uint32_t raw[32];
        tmem_load32(lane_addr + L::O_COLUMN + c * 32, raw);
#pragma unroll
        for (int i = 0; i < 32; i++) o[c * 32 + i] += __uint_as_float(raw[i]);
      }
      if (row_valid) {
        const float inv = 1.0f / l;
        __nv_bfloat16* dst = p.out + (size_t)token * p.out_stride + (size_t)head * HD;
#pragma unroll
        for (int i = 0; i < HD; i += 8) {
          uint32_t packed[4];
#pragma unroll
          for (int k2 = 0; k2 < 4; k2++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(o[i + 2 * k2] * inv, o[i + 2 * k2 + 1] * inv);
            packed[k2] = *(uint32_t*)&h;
          }
          *(uint4*)(dst + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 0 && lane == 0) {
    // copies already issued still write shared memory: wait for them (bounded) before leaving
    for (int j = max(0, k_issued - KV_STAGES); j < k_issued; j++) mbar_wait(&k_full[j % KV_STAGES], (j / KV_STAGES) & 1);
    for (int j = max(0, v_issued - KV_STAGES); j < v_issued; j++) mbar_wait(&v_full[j % KV_STAGES], (j / KV_STAGES) & 1);
  }
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

template <int HD>
int launch_tc(const CUtensorMap& map_k, const CUtensorMap& map_v, const TcParams& p, int grid, cudaStream_t stream) {
  using L = TcLayout<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (err != cudaSuccess) return sprout_fail("attention_prefill: cannot reserve %d bytes of shared memory: %s", L::SMEM_BYTES, cudaGetErrorString(err));
    // all of the SM's memory as shared memory: two CTAs of the head_dim 64 kernel fit only then
    cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  sprout_launch(attention_prefill_tc_kernel<HD>, dim3(grid), dim3(TC_THREADS), L::SMEM_BYTES, stream, map_k, map_v, p);
  return sprout_check_launch("attention_prefill (tcgen05)");
}

}  // namespace

// Whether the tcgen05 kernel takes these sizes.
SPROUT_API int sprout_attention_prefill_tc_supported(int head_dim, int page_tokens, int out_stride) {
  const bool pages_ok = page_tokens >= 8 && (TC_KEYS % page_tokens == 0 || page_tokens % TC_KEYS == 0);
  return (head_dim == 64 || head_dim == 128) && pages_ok && out_stride % 8 == 0;
}

// CTAs of the kernel that one SM holds at a time (2 for head_dim 64 when all of the SM's memory
// is shared memory), 0 for a head_dim the kernel does not take; -1 with the error text set.
SPROUT_API int sprout_attention_prefill_tc_occupancy(int head_dim) {
  int blocks = 0;
  cudaError_t err = cudaSuccess;
  if (head_dim == 64) {
    cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcLayout<64>::SMEM_BYTES);
    cudaFuncSetAttribute(attention_prefill_tc_kernel<64>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_prefill_tc_kernel<64>, TC_THREADS, TcLayout<64>::SMEM_BYTES);
  } else if (head_dim == 128) {
    cudaFuncSetAttribute(attention_prefill_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcLayout<128>::SMEM_BYTES);
    err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, attention_prefill_tc_kernel<128>, TC_THREADS, TcLayout<128>::SMEM_BYTES);
  }
  if (err != cudaSuccess) { sprout_fail("attention_prefill: occupancy query failed: %s", cudaGetErrorString(err)); return -1; }
  return blocks;
}

// The arguments of sprout_attention_prefill, checked there.
int sprout_attention_prefill_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* q_start, const int* positions,
                                void* out, int out_stride, int num_tokens, int requests, int heads, int kv_heads,
                                int head_dim, int page_tokens, int num_pages, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(sprout_attention_prefill_tc_supported(head_dim, page_tokens, out_stride) && ((uintptr_t)out & 15) == 0,
                 "attention_prefill (tcgen05): head_dim %d, page size %d or the output's alignment is not taken", head_dim, page_tokens);
  const long long cache_rows = (long long)num_pages * kv_heads * page_tokens;
  SPROUT_REQUIRE(cache_rows <= 0x7fffffffLL, "attention_prefill (tcgen05): the cache has too many rows for a tensor map coordinate");
  TcParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.positions = positions;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.requests = requests; p.heads = heads; p.kv_heads = kv_heads; p.page_tokens = page_tokens; p.num_pages = num_pages;
  p.box_rows = page_tokens < TC_KEYS ? page_tokens : TC_KEYS;
  p.scale = 1.0f / sqrtf((float)head_dim); p.status = status;
  CUtensorMap map_k, map_v;
  if (tensor_map(k_cache, (int)cache_rows, head_dim, head_dim, p.box_rows, &map_k)) return 1;
  if (tensor_map(v_cache, (int)cache_rows, head_dim, head_dim, p.box_rows, &map_v)) return 1;
  const int group = heads / kv_heads;
  const long long bound = (((long long)num_tokens * group + TC_ROWS - 1) / TC_ROWS + requests) * kv_heads;
  SPROUT_REQUIRE(bound <= 0x7fffffffLL, "attention_prefill: too many tokens");
  if (head_dim == 64) return launch_tc<64>(map_k, map_v, p, (int)bound, stream);
  return launch_tc<128>(map_k, map_v, p, (int)bound, stream);
}
