// Prefill attention over the paged cache on the fifth-generation tensor cores (sm_100a).
//
// One CTA owns 256 rows, a row being a (token, query head) pair of one request and one key/value
// head, as two Q tiles of 128 rows, and walks the request's keys in tiles (128 keys for head_dim
// 64, 64 keys for head_dim 128).  For each Q tile and key tile:
//
//   S = Q K^T      tcgen05.mma, Q and K K-major in shared memory, S in tensor memory
//   softmax        a warpgroup per Q tile, one thread per row: tcgen05.ld of its row of S, running
//                  maximum and sum in float32, P = exp2(..) written as bfloat16 into shared memory
//                  in the K-major swizzled layout the next product reads
//   O_tile = P V   tcgen05.mma, V as it lies in the cache ([key, head_dim]: MN-major B operand),
//                  the tile's product in tensor memory; the row's thread adds it to its float32
//                  accumulator in registers, rescaled when the maximum moved
//
// The two Q tiles alternate: while the softmax warpgroup of one works on its S, the tensor cores
// run P V and the next S of the other.  (A kernel that allocates tensor memory gets one CTA per
// SM, so the overlap has to happen inside the CTA.)  The softmax warpgroups take the registers
// that the copy/MMA warpgroup gives up: a row's thread holds head_dim accumulators and a whole
// row of S.
//
// K and V tiles come by TMA, one box per page (a page of one head is `page_tokens` contiguous
// rows of the cache), through a two-stage ring.  One warp looks the pages up and issues the
// copies (a lane per box), one thread issues the MMAs.  Every mbarrier wait is bounded: on a
// timeout the CTA sets the status word, waits (bounded) for its copies in flight, frees its
// tensor memory and returns.
//
// Takes head_dim 64 or 128 and page sizes of 8, 16, 32, 64 or a multiple of 128 tokens; the
// mma.sync kernel in attention_bf16.cu takes everything else.
#include <cuda_bf16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int TC_ROWS = 128;              // rows of a Q tile == TMEM lanes
constexpr int TC_QTILES = 2;              // Q tiles of a CTA
constexpr int KV_STAGES = 2;
constexpr int TC_THREADS = 384;           // warpgroup 0: copy warp, MMA warp (two warps idle); 1, 2: softmax of Q tile 0, 1
constexpr int TC_TMEM_COLS = 512;
constexpr int SPROUT_PREFILL_SPLIT_MAX = 160;   // pieces that can get a second CTA (fewer than the SMs of any GPU this runs on)
constexpr int Q_ATOM_BYTES = 128 * 128;   // a [128 rows, 64 bf16] swizzled tile

struct TcParams {
  const __nv_bfloat16* q; int q_stride;
  const int* block_table; int table_stride;
  const int* q_start;                 // [requests + 1]
  const int* positions;               // [tokens]
  __nv_bfloat16* out; int out_stride;
  int requests, heads, kv_heads, page_tokens, num_pages, box_rows;
  int split_pieces;                   // SPLIT kernel: pieces (in launch order) that two CTAs share
  float* scratch;                     // [split_pieces][2][256 rows][head_dim + 4] partial results
  int* counters;                      // [split_pieces][2 Q tiles], zero between launches
  float scale;
  int* status;
};

template <int HD>
struct TcLayout {
  static constexpr int KB = HD / 64;                       // 64-element blocks along head_dim
  static constexpr int KEYS = HD == 64 ? 128 : 64;         // keys of a tile: a softmax thread holds HD + KEYS floats
  static constexpr int KV_ATOM_BYTES = KEYS * 128;         // [KEYS rows, 64 bf16]
  static constexpr int Q_BYTES = KB * Q_ATOM_BYTES;        // one Q tile
  static constexpr int KV_BYTES = KB * KV_ATOM_BYTES;      // one stage of K (or of V)
  static constexpr int P_BYTES = (KEYS / 64) * Q_ATOM_BYTES;   // [128 rows, KEYS keys] of one Q tile
  static constexpr int OFF_K = TC_QTILES * Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + TC_QTILES * P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256;
  static constexpr int O_COLUMN = TC_QTILES * KEYS;        // tensor memory: S of the Q tiles, then their O tiles
  static_assert(O_COLUMN + TC_QTILES * HD <= TC_TMEM_COLS, "tensor memory columns");
};

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Two float32 in one 64-bit register pair: sm_100a adds, multiplies and fuses them pairwise in
// one instruction, which halves the FMA-pipe work of the softmax.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^x for x <= 0 (a probability): the hardware approximation, results below the normal range are zero
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// SPLIT: the launch has fewer 256-row pieces than the GPU has SMs.  The first `split_pieces`
// pieces of the launch (the longest) then get two CTAs each, which take alternate key tiles.
// Each leaves its partial result (maximum, sum and accumulators of every row) in global scratch
// memory and counts itself in; the one that finds the other already counted merges the two and
// writes the rows.  Nobody waits for anybody.
template <int HD, bool SPLIT>
__global__ void __launch_bounds__(TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                            const TcParams p) {
  using L = TcLayout<HD>;
  constexpr int KEYS = L::KEYS;
  // no static shared memory: the swizzled tiles need the dynamic region to start on a 1024-byte
  // boundary, which is checked below
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
  uint64_t* s_full = bars + 8;        // [2] S of a Q tile's key tile is complete in tensor memory
  uint64_t* o_full = bars + 10;       // [2] P V of a Q tile's key tile is complete in tensor memory
  uint64_t* p_full = bars + 12;       // [2] P of a Q tile's key tile is written to shared memory (4 warps arrive)
  uint32_t* tmem_slot = (uint32_t*)(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  // What this kernel reads before it waits for the step's earlier kernels (the request's bounds
  // and positions, the block table) was written before the step's first kernel; the queries and
  // the newest keys and values are read after the wait, below.
  pdl_launch_dependents();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bool paired = SPLIT && (int)blockIdx.x < 2 * p.split_pieces;      // one of the two CTAs of a piece
  const int piece_index = !SPLIT ? (int)blockIdx.x : paired ? (int)blockIdx.x >> 1 : (int)blockIdx.x - p.split_pieces;
  const int rank = paired ? blockIdx.x & 1 : 0;
  const int g = piece_index % p.kv_heads;
  const int group = p.heads / p.kv_heads;
  constexpr int CTA_ROWS = TC_QTILES * TC_ROWS;

  // which request and which 256-row piece of it: the pieces of a request are handed out from the
  // last (the longest under the causal mask) to the first, the heads of a piece side by side
  int r = 0, piece = piece_index / p.kv_heads;
  for (; r < p.requests; r++) {
    const int pieces = ((p.q_start[r + 1] - p.q_start[r]) * group + CTA_ROWS - 1) / CTA_ROWS;
    if (piece < pieces) { piece = pieces - 1 - piece; break; }
    piece -= pieces;
  }
  if (r >= p.requests) return;
  if ((smem_u32(smem) & 1023) != 0) {
    if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_LAYOUT);
    return;
  }
  const int q0 = p.q_start[r], q_count = p.q_start[r + 1] - q0;
  const int rows_total = q_count * group;
  const int row_base = piece * CTA_ROWS;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  // positions grow with the row index: the last row of a Q tile sees the most keys
  const bool two = row_base + TC_ROWS < rows_total;       // the second Q tile has rows
  const int limit_a = p.positions[q0 + (min(rows_total, row_base + TC_ROWS) - 1) / group];
  const int max_limit = two ? p.positions[q0 + (min(rows_total, row_base + CTA_ROWS) - 1) / group] : limit_a;
  const int all_tiles = max_limit / KEYS + 1;              // key tiles of the piece
  // this CTA's share: all of them, or every second one from its rank; below, j counts the CTA's
  // own tiles and first + step * j is the tile among the piece's
  const bool split = paired && all_tiles >= 4;
  if (paired && !split && rank == 1) return;
  const int first = split ? rank : 0, step = split ? 2 : 1;
  const int tiles_a = (limit_a / KEYS + 1 - first + step - 1) / step;     // own key tiles that Q tile 0 needs
  const int n_tiles = (all_tiles - first + step - 1) / step;              // and Q tile 1 (or the CTA)

  // rows of a stage that no copy fills (keys beyond the request) must hold finite numbers: their
  // probabilities are zero, and zero times a stale NaN is not
  for (int i = tid; i < 2 * KV_STAGES * L::KV_BYTES / 16; i += TC_THREADS) ((uint4*)sK)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < 12; i++) mbar_init(&bars[i], 1);
    mbar_init(&p_full[0], 4); mbar_init(&p_full[1], 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TC_TMEM_COLS);
  pdl_wait();

  // Q rows -> shared memory, K-major with the 128-byte swizzle (16-byte chunk c of row r at chunk
  // position c ^ (r & 7)), one 16 KB atom per Q tile and 64 elements of head_dim
  constexpr int CHUNKS = HD / 8;
  for (int idx = tid; idx < CTA_ROWS * CHUNKS; idx += TC_THREADS) {
    const int crow = idx / CHUNKS, c = idx % CHUNKS;
    const int gi = row_base + crow;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (gi < rows_total)
      v = *(const uint4*)(p.q + (size_t)(q0 + gi / group) * p.q_stride + (size_t)(g * group + gi % group) * HD + c * 8);
    const int row = crow & (TC_ROWS - 1);
    *(uint4*)(sQ + (crow >> 7) * L::Q_BYTES + (c >> 3) * Q_ATOM_BYTES + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v;
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  int k_issued = 0, v_issued = 0;                     // tiles whose copies were issued (lane 0 of the copy warp)
  if (warp < 4) {
    warpgroup_regs_give<56>();
    if (warp == 0) {
      // ---------------- copies: one TMA box per page (or per KEYS keys of a larger page); lane b
      // looks box b's page up and issues its copies, lane 0 waits for the stage and posts the bytes
      const int boxes = KEYS / p.box_rows;
      auto box_row = [&](int j) {
        const int key = (first + step * j) * KEYS + lane * p.box_rows;
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
            tma_load_2d(sK + s * L::KV_BYTES + kb * L::KV_ATOM_BYTES + lane * p.box_rows * 128, &map_k, &k_full[s], kb * 64, row_at);
        k_issued = j + 1;
        next_row = box_row(j + 1);                    // the lookup runs under the wait below
        if (lane == 0) {
          ok = !*abort_flag && mbar_wait(&v_empty[s], parity);
          if (ok) mbar_expect_tx(&v_full[s], bytes);
          else { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) break;
        if (row_at >= 0)
          for (int kb = 0; kb < L::KB; kb++)
            tma_load_2d(sV + s * L::KV_BYTES + kb * L::KV_ATOM_BYTES + lane * p.box_rows * 128, &map_v, &v_full[s], kb * 64, row_at);
        v_issued = j + 1;
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer.  Order: S0(0) S1(0), then for every key tile
      //   [P0(j)] P0 V(j), S0(j+1), [P1(j)] P1 V(j), S1(j+1)
      // so that the products of one Q tile run under the softmax of the other.  S of a Q tile has
      // one buffer: S(j+1) follows the wait for P(j), by which the softmax warps have read S(j).
      const uint32_t idesc_s = umma_idesc(TC_ROWS, KEYS);
      const uint32_t idesc_o = umma_idesc_b_mn(TC_ROWS, HD);
      bool ok = true;
      auto fail = [&]() { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); ok = false; };
      auto issue_s = [&](int q, int j) {             // the K stage of tile j has been waited for
        const int s = j % KV_STAGES;
#pragma unroll
        for (int kb = 0; kb < L::KB; kb++) {
          const uint64_t a = umma_smem_desc(sQ + q * L::Q_BYTES + kb * Q_ATOM_BYTES);
          const uint64_t b = umma_smem_desc(sK + s * L::KV_BYTES + kb * L::KV_ATOM_BYTES);
#pragma unroll
          for (int kk = 0; kk < 4; kk++) umma_bf16(tmem_base + q * KEYS, a + 2 * kk, b + 2 * kk, idesc_s, (kb | kk) != 0);
        }
        umma_commit(&s_full[q]);
      };
      auto issue_pv = [&](int q, int j) {
        const int s = j % KV_STAGES;
#pragma unroll
        for (int ks = 0; ks < KEYS / 16; ks++) {
          const uint64_t a = umma_smem_desc(sP + q * L::P_BYTES + (ks >> 2) * Q_ATOM_BYTES) + 2 * (ks & 3);
          const uint64_t b = umma_smem_desc_mn(sV + s * L::KV_BYTES + ks * 2048, L::KV_ATOM_BYTES);
          umma_bf16(tmem_base + L::O_COLUMN + q * HD, a, b, idesc_o, ks != 0);
        }
        umma_commit(&o_full[q]);
      };
      // the last product that reads a stage releases it: S1 (or S0 where Q tile 1 has no rows)
      // for K, P1 V (or P0 V) for V; Q tile 0 stops after tiles_a tiles
      if (*abort_flag || !mbar_wait(&k_full[0], 0)) fail();
      if (ok) {
        tc_fence_after();
        if (tiles_a > 0) issue_s(0, 0);
        if (two) issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; j++) {
        const int s = j % KV_STAGES, s_next = (j + 1) % KV_STAGES;
        const bool more = j + 1 < n_tiles;
        if (*abort_flag || !mbar_wait(&v_full[s], (j / KV_STAGES) & 1)) { fail(); break; }
        if (j < tiles_a) {
          if (*abort_flag || !mbar_wait(&p_full[0], j & 1)) { fail(); break; }
          tc_fence_after();
          issue_pv(0, j);
          if (!two) umma_commit(&v_empty[s]);
        }
        if (more && (*abort_flag || !mbar_wait(&k_full[s_next], ((j + 1) / KV_STAGES) & 1))) { fail(); break; }
        if (more && j + 1 < tiles_a) {
          tc_fence_after();
          issue_s(0, j + 1);
          if (!two) umma_commit(&k_empty[s_next]);
        }
        if (two) {
          if (*abort_flag || !mbar_wait(&p_full[1], j & 1)) { fail(); break; }
          tc_fence_after();
          issue_pv(1, j);
          umma_commit(&v_empty[s]);
          if (more) {
            issue_s(1, j + 1);
            umma_commit(&k_empty[s_next]);
          }
        }
      }
    }
  } else {
    // ---------------- softmax and accumulation: a warpgroup per Q tile, one thread per row
    warpgroup_regs_take<224>();
    const int q = (warp >> 2) - 1;
    const int my_tiles = q == 0 ? tiles_a : (two ? n_tiles : 0);
    const int quarter = warp & 3;                      // a warp reads TMEM lanes 32 * (warp % 4) ..
    const int row = quarter * 32 + lane;
    const int gi = row_base + q * TC_ROWS + row;
    const bool row_valid = gi < rows_total;
    const int token = q0 + (row_valid ? gi / group : 0), head = g * group + gi % group;
    const int limit = row_valid ? p.positions[token] : -1;   // last visible key of the row
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + q * KEYS, o_addr = lane_addr + L::O_COLUMN + q * HD;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    uint8_t* p_row = sP + q * L::P_BYTES + row * 128;
    uint64_t o2[HD / 2];                               // the row's accumulators, in pairs
#pragma unroll
    for (int i = 0; i < HD / 2; i++) o2[i] = 0ull;
    float m = -INFINITY;                               // running maximum of the unscaled scores
    uint64_t l2 = 0ull;                                // running sum, as two partial sums
    bool ok = true;
    auto add_o_tile = [&]() {                          // o += the product in tensor memory
#pragma unroll
      for (int c = 0; c < HD / 64; c++) {
        uint32_t ra[32], rb[32];
        tmem_load32_issue(o_addr + c * 64, ra);
        tmem_load32_issue(o_addr + c * 64 + 32, rb);
        tmem_load_wait(ra);
        tmem_load_wait(rb);
#pragma unroll
        for (int i = 0; i < 16; i++) {
          o2[c * 32 + i] = f2_add(o2[c * 32 + i], f2_pack(ra[2 * i], ra[2 * i + 1]));
          o2[c * 32 + 16 + i] = f2_add(o2[c * 32 + 16 + i], f2_pack(rb[2 * i], rb[2 * i + 1]));
        }
      }
    };
    for (int j = 0; j < my_tiles; j++) {
      if (j > 0) {
        // the previous tile's P V (it also frees the P buffer)
        ok = !*abort_flag && mbar_wait(&o_full[q], (j - 1) & 1);
        if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
        ok = __all_sync(0xffffffffu, ok);              // tcgen05.ld is warp-wide: all lanes or none
        if (!ok) break;
        tc_fence_after();
        add_o_tile();
      }
      ok = !*abort_flag && mbar_wait(&s_full[q], j & 1);
      if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int kv0 = (first + step * j) * KEYS;
      // the whole row of S
      uint32_t sc[KEYS / 32][32];
#pragma unroll
      for (int c = 0; c < KEYS / 32; c++) tmem_load32_issue(s_addr + c * 32, sc[c]);
#pragma unroll
      for (int c = 0; c < KEYS / 32; c++) tmem_load_wait(sc[c]);
      if (kv0 + KEYS - 1 > limit) {                    // some key of the tile lies beyond this row's limit
#pragma unroll
        for (int c = 0; c < KEYS / 32; c++)
#pragma unroll
          for (int i = 0; i < 32; i++) if (kv0 + c * 32 + i > limit) sc[c][i] = 0xff800000u;   // -inf
      }
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < KEYS / 32; c++)
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          mx[0] = max3(mx[0], __uint_as_float(sc[c][i]), __uint_as_float(sc[c][i + 1]));
          mx[1] = max3(mx[1], __uint_as_float(sc[c][i + 2]), __uint_as_float(sc[c][i + 3]));
          mx[2] = max3(mx[2], __uint_as_float(sc[c][i + 4]), __uint_as_float(sc[c][i + 5]));
          mx[3] = max3(mx[3], __uint_as_float(sc[c][i + 6]), __uint_as_float(sc[c][i + 7]));
        }
      const float n = max3(m, fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      const float base = n == -INFINITY ? 0.f : n * scale_log2;
      const float alpha = m == -INFINITY ? 0.f : exp2_fast(m * scale_log2 - base);
      m = n;
      if (!__all_sync(0xffffffffu, alpha == 1.0f)) {   // the maximum moved for some row: bring the sums to it
        const uint64_t alpha2 = f2_pack(alpha, alpha);
        l2 = f2_mul(l2, alpha2);
#pragma unroll
        for (int i = 0; i < HD / 2; i++) o2[i] = f2_mul(o2[i], alpha2);
      }
      // probabilities, their sum, and P as bfloat16 into shared memory
      const uint64_t scale2 = f2_pack(scale_log2, scale_log2), nbase2 = f2_pack(-base, -base);
#pragma unroll
      for (int c = 0; c < KEYS / 32; c++) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          f2_unpack(f2_fma(f2_pack(sc[c][i], sc[c][i + 1]), scale2, nbase2), x0, x1);
          const float p0 = exp2_fast(x0), p1 = exp2_fast(x1);
          l2 = f2_add(l2, f2_pack(p0, p1));
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *(uint32_t*)&h;
        }
        uint8_t* atom = p_row + (c >> 1) * Q_ATOM_BYTES;
#pragma unroll
        for (int q4 = 0; q4 < 4; q4++) {
          const int chunk = (c & 1) * 4 + q4;
          *(uint4*)(atom + ((chunk ^ (row & 7)) << 4)) = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      if (first + step * j == all_tiles - 1 && row < KEYS && kv0 + row > max_limit) {
        // the last tile's pages may reach beyond the request's keys, into slots that hold whatever
        // was there before: their probabilities are zero, but zero times a NaN is not, so the V
        // row of such a key is cleared once its copy has landed (by each Q tile that reads the
        // tile, before it signals its P: whichever P V comes first finds the rows cleared)
        const int s = j % KV_STAGES;
        if (*abort_flag || !mbar_wait(&v_full[s], (j / KV_STAGES) & 1)) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
#pragma unroll
        for (int kb = 0; kb < L::KB; kb++)
#pragma unroll
          for (int c = 0; c < 8; c++) *(uint4*)(sV + s * L::KV_BYTES + kb * L::KV_ATOM_BYTES + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[q]);
    }
    if (ok && my_tiles > 0) {
      ok = !*abort_flag && mbar_wait(&o_full[q], (my_tiles - 1) & 1);
      if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        add_o_tile();
      }
    }
    float l_lo, l_hi;
    f2_unpack(l2, l_lo, l_hi);
    float l = l_lo + l_hi;
    bool writes = !split;                              // this thread writes its row out
    if (SPLIT && split) {
      // this CTA's rows go to scratch memory; the warpgroup then counts itself in for its Q tile,
      // and if the other CTA was there before, it merges that CTA's rows into its own
      constexpr int ROW_FLOATS = HD + 4;
      float* mine = p.scratch + ((size_t)(piece_index * 2 + rank) * CTA_ROWS + q * TC_ROWS + row) * ROW_FLOATS;
      const float* theirs = p.scratch + ((size_t)(piece_index * 2 + (rank ^ 1)) * CTA_ROWS + q * TC_ROWS + row) * ROW_FLOATS;
#pragma unroll
      for (int i = 0; i < HD / 4; i++) {
        float a, b, c, d;
        f2_unpack(o2[2 * i], a, b);
        f2_unpack(o2[2 * i + 1], c, d);
        ((float4*)mine)[i] = make_float4(a, b, c, d);
      }
      *(float2*)(mine + HD) = make_float2(ok ? m : -INFINITY, l);
      __threadfence();
      asm volatile("bar.sync %0, 128;" ::"r"(1 + q) : "memory");          // the warpgroup's rows are written
      int* counter = p.counters + piece_index * TC_QTILES + q;
      int* seen = (int*)(smem + L::OFF_BAR + 192) + q;                     // behind the barriers and the TMEM slot
      if ((tid & 127) == 0) *seen = atomicAdd(counter, 1);
      asm volatile("bar.sync %0, 128;" ::"r"(1 + q) : "memory");
      if (*seen == 1) {
        __threadfence();
        if ((tid & 127) == 0) *counter = 0;                                // ready for the next launch
        const float2 ml = __ldcg((const float2*)(theirs + HD));
        const float m1 = ml.x, l1 = ml.y;
        const float top = fmaxf(m, m1);
        const float a0 = m == -INFINITY ? 0.f : exp2_fast((m - top) * scale_log2);
        const float a1 = m1 == -INFINITY ? 0.f : exp2_fast((m1 - top) * scale_log2);
        l = l * a0 + l1 * a1;
        const uint64_t a0_2 = f2_pack(a0, a0), a1_2 = f2_pack(a1, a1);
#pragma unroll
        for (int i = 0; i < HD / 4; i++) {
          const float4 t = __ldcg((const float4*)theirs + i);
          o2[2 * i] = f2_fma(o2[2 * i], a0_2, f2_mul(f2_pack(t.x, t.y), a1_2));
          o2[2 * i + 1] = f2_fma(o2[2 * i + 1], a0_2, f2_mul(f2_pack(t.z, t.w), a1_2));
        }
        writes = true;
      }
    }
    if (ok && row_valid && writes) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = p.out + (size_t)token * p.out_stride + (size_t)head * HD;
#pragma unroll
      for (int i = 0; i < HD; i += 8) {
        uint32_t packed[4];
#pragma unroll
        for (int k2 = 0; k2 < 4; k2++) {
          float lo, hi;
          f2_unpack(o2[i / 2 + k2], lo, hi);
          __nv_bfloat162 h = __floats2bfloat162_rn(lo * inv, hi * inv);
          packed[k2] = *(uint32_t*)&h;
        }
        *(uint4*)(dst + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
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
  if (warp == 1) tmem_dealloc(tmem_base, TC_TMEM_COLS);
}

// `pieces` bounds the 256-row pieces of the launch (times key/value heads).
template <int HD>
int launch_tc(const CUtensorMap& map_k, const CUtensorMap& map_v, TcParams p, int pieces, cudaStream_t stream) {
  using L = TcLayout<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (err == cudaSuccess)
      err = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (err != cudaSuccess) return sprout_fail("attention_prefill: cannot reserve %d bytes of shared memory: %s", L::SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  if (p.split_pieces > 0) {
    sprout_launch(attention_prefill_tc_kernel<HD, true>, dim3(pieces + p.split_pieces), dim3(TC_THREADS), L::SMEM_BYTES, stream, map_k, map_v, p);
    return sprout_check_launch("attention_prefill (tcgen05, split)");
  }
  sprout_launch(attention_prefill_tc_kernel<HD, false>, dim3(pieces), dim3(TC_THREADS), L::SMEM_BYTES, stream, map_k, map_v, p);
  return sprout_check_launch("attention_prefill (tcgen05)");
}

}  // namespace

// Whether the tcgen05 kernel takes these sizes.
SPROUT_API int sprout_attention_prefill_tc_supported(int head_dim, int page_tokens, int out_stride) {
  const bool pages_ok = page_tokens == 8 || page_tokens == 16 || page_tokens == 32 || page_tokens == 64 ||
                        (page_tokens > 0 && page_tokens % 128 == 0);
  return (head_dim == 64 || head_dim == 128) && pages_ok && out_stride % 8 == 0;
}

// Scratch floats and counters that let the kernel give the longest pieces of a small launch two
// CTAs each (at most SPROUT_PREFILL_SPLIT_MAX pieces).
SPROUT_API long long sprout_attention_prefill_scratch_floats(int head_dim) {
  return (long long)SPROUT_PREFILL_SPLIT_MAX * 2 * TC_QTILES * TC_ROWS * (head_dim + 4);
}
SPROUT_API int sprout_attention_prefill_counters() { return SPROUT_PREFILL_SPLIT_MAX * TC_QTILES; }

// The arguments of sprout_attention_prefill, checked there; scratch and counters may be null.
int sprout_attention_prefill_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* q_start, const int* positions,
                                void* out, int out_stride, int num_tokens, int requests, int heads, int kv_heads,
                                int head_dim, int page_tokens, int num_pages, float* scratch, long long scratch_floats,
                                int* counters, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(sprout_attention_prefill_tc_supported(head_dim, page_tokens, out_stride) && ((uintptr_t)out & 15) == 0,
                 "attention_prefill (tcgen05): head_dim %d, page size %d or the output's alignment is not taken", head_dim, page_tokens);
  const long long cache_rows = (long long)num_pages * kv_heads * page_tokens;
  SPROUT_REQUIRE(cache_rows <= 0x7fffffffLL, "attention_prefill (tcgen05): the cache has too many rows for a tensor map coordinate");
  TcParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.positions = positions;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.requests = requests; p.heads = heads; p.kv_heads = kv_heads; p.page_tokens = page_tokens; p.num_pages = num_pages;
  const int keys = head_dim == 64 ? TcLayout<64>::KEYS : TcLayout<128>::KEYS;
  p.box_rows = page_tokens < keys ? page_tokens : keys;
  p.scale = 1.0f / sqrtf((float)head_dim); p.status = status;
  CUtensorMap map_k, map_v;
  if (tensor_map(k_cache, (int)cache_rows, head_dim, head_dim, p.box_rows, &map_k)) return 1;
  if (tensor_map(v_cache, (int)cache_rows, head_dim, head_dim, p.box_rows, &map_v)) return 1;
  const int group = heads / kv_heads;
  const int cta_rows = TC_QTILES * TC_ROWS;
  const long long bound = (((long long)num_tokens * group + cta_rows - 1) / cta_rows + requests) * kv_heads;
  SPROUT_REQUIRE(bound <= 0x7fffffffLL, "attention_prefill: too many tokens");
  // fewer pieces than SMs: the longest pieces get a second CTA each, as far as SMs and scratch memory go
  p.split_pieces = 0; p.scratch = scratch; p.counters = counters;
  if (scratch && counters && bound < sm_count()) {
    const long long per_piece = 2LL * cta_rows * (head_dim + 4);
    long long n = sm_count() - bound;
    if (n > bound) n = bound;
    if (n > scratch_floats / per_piece) n = scratch_floats / per_piece;
    if (n > SPROUT_PREFILL_SPLIT_MAX) n = SPROUT_PREFILL_SPLIT_MAX;
    p.split_pieces = (int)n;
  }
  if (head_dim == 64) return launch_tc<64>(map_k, map_v, p, (int)bound, stream);
  return launch_tc<128>(map_k, map_v, p, (int)bound, stream);
}
