// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   out[m, n] = sum_k A[m, k] * W[n, k] (+ bias[n]) (+ residual[m, n])
// A (activations, [M, K]) and W (weights, [N, K]) are both K-major, which is the layout
// tcgen05.mma takes for both operands: no repacking.
//
// One CTA computes a 128 x BN tile of D: operand tiles of 64 K-elements (128 bytes, one
// swizzle row) are staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle)
// through a ring of stages guarded by mbarriers; one elected thread issues tcgen05.mma with
// the float32 accumulator in tensor memory; eight warps read the accumulator back with
// tcgen05.ld and apply the epilogue.  Warp 0 produces (TMA), warp 1 issues MMAs and owns the
// TMEM allocation, warps 2-9 run the epilogue (two per 32-lane quarter of tensor memory).
//
// Two orientations share the pipeline:
//   tokens on M (prefill): D rows are tokens, D columns output features; BN = 256 where that
//       tiles N exactly (less operand traffic from L2), else 128.
//   weights on M (decode, "swap"): D rows are output features, D columns tokens in tiles of
//       BN = 16..256.  A decode step streams every weight once and the 128-row tensor-core tile
//       is filled by weight rows instead of by a handful of tokens.
//       With split_k > 1 the K range is divided among CTAs (grid.z) and the partial sums are
//       added into the float32 output with atomics (residual epilogue only).
//
// Every wait on an mbarrier is bounded; a wait that runs out sets SPROUT_STATUS_WAIT_TIMEOUT,
// the CTA stops issuing, waits (bounded) for its copies in flight, frees its TMEM and returns.
#include <cuda.h>


#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BLOCK_M = 128;        // rows of D per CTA == TMEM lanes
constexpr int BLOCK_K = 64;         // bf16 elements per stage row: 128 bytes, one swizzle row
constexpr int NUM_THREADS = 320;      // TMA warp, MMA warp, 8 epilogue warps
constexpr int SMEM_BUDGET = 196 * 1024;    // for the operand stages; the staging tiles and barriers come on top

enum Epilogue : int { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_RESIDUAL_ATOMIC = 2, EPI_SWIGLU = 3, EPI_RESIDUAL_TMA = 4 };
constexpr int STAGING_BYTES = 2 * 128 * 128;    // two [128 rows, 32 float32] tiles for the TMA reduction of the residual epilogue

// SwiGLU epilogue: the weight rows interleave gate and up in blocks of 8 (rows 16b..16b+7 gate,
// 16b+8..16b+15 up), so output feature 8b+j is silu(D[.., 16b+j]) * D[.., 16b+8+j]; the output
// has N/2 features and is bfloat16.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

struct Params {
  const float* bias;     // [N] or null
  void* out;             // [M, N] row stride ldo, bf16 or f32
  int out_is_f32;
  int epilogue;
  int M, N, K;           // M tokens, N output features
  int ldo;
  int k_blocks_per_split;
  int* status;
  // weights on M only: the tokens' operand made in the kernel instead of copied: bfloat16(x * gain) of the
  // float32 rows x [M, K] (row stride ldx), written by the epilogue warps into the stages' token tiles
  const float* x32; const float* gain; int ldx;
};

// PAIR: two CTAs share a 256 x BN tile; each holds its own 128 rows of A and half of B's rows.
template <int BN, bool PAIR = false>
struct Layout {
  static constexpr int A_BYTES = BLOCK_M * BLOCK_K * 2;
  static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BLOCK_K * 2;
  static constexpr int B_PADDED = (B_BYTES + 1023) / 1024 * 1024;
  static constexpr int STAGE_BYTES = A_BYTES + B_PADDED;
  static constexpr int STAGES = (SMEM_BUDGET / STAGE_BYTES) > 12 ? 12 : (SMEM_BUDGET / STAGE_BYTES);
  // two accumulators; allocations are powers of two from 32 columns
  static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

// One unit of work: a 128 x BN tile of D over a range of K blocks.
struct Work { int row0, col0, kb_begin, num_kb, split; };

// SWAP == false: map_rows is the activation map (rows = tokens), map_cols the weight map.
// SWAP == true:  map_rows is the weight map (rows = output features), map_cols the activation map.
// The kernel is persistent: a CTA walks the work list with stride gridDim.x.  The TMA ring runs
// on across tiles, and two accumulators in tensor memory alternate, so that the epilogue of one
// tile overlaps the MMAs of the next.
//
// PAIR (tokens on M only): the CTAs come in clusters of two that work on 256 x BN tiles with
// tcgen05.mma.cta_group::2.  Each CTA copies its own 128 rows of A and half of the tile's rows of
// B (so a pair moves 2 x (16 + BN / 8) KB per k-block from L2 where two single CTAs move
// 2 x (16 + BN / 4) KB: the operand traffic from L2 is what bounds these products); the first
// CTA's thread issues the MMAs for both, each CTA's epilogue warps drain its own 128 rows from
// its own tensor memory.  The copies of both CTAs count on the first CTA's "full" barriers; the
// commits arrive on the "empty" and "accumulator full" barriers of both CTAs; the second CTA's
// epilogue warps arrive on the first CTA's "accumulator empty" barriers.
template <int BN, bool SWAP, bool PAIR = false>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_rows, const __grid_constant__ CUtensorMap map_cols,
                    const __grid_constant__ CUtensorMap map_out, const Params p) {
  static_assert(!(PAIR && SWAP), "pairs work on token tiles");
  using L = Layout<BN, PAIR>;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0;                       // 0 issues the MMAs
  const int first_work = PAIR ? (int)blockIdx.x >> 1 : (int)blockIdx.x;     // this CTA's (pair's) first item and stride
  const int work_stride = PAIR ? (int)gridDim.x >> 1 : (int)gridDim.x;
  constexpr int TILE_M = PAIR ? 2 * BLOCK_M : BLOCK_M;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* staging = smem + L::STAGES * L::STAGE_BYTES;
  uint64_t* full_bar = (uint64_t*)(staging + STAGING_BYTES);
  uint64_t* empty_bar = full_bar + L::STAGES;
  uint64_t* acc_full = empty_bar + L::STAGES;     // [2] accumulator complete (MMA -> epilogue)
  uint64_t* acc_empty = acc_full + 2;             // [2] accumulator read out (epilogue -> MMA)
  uint64_t* epi_bar = acc_empty + 2;              // the 8 epilogue warps meet here (bounded, unlike bar.sync)
  uint32_t* tmem_slot = (uint32_t*)(epi_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
  const int row_tiles = ((SWAP ? p.N : p.M) + TILE_M - 1) / TILE_M;
  const int col_tiles = ((SWAP ? p.M : p.N) + BN - 1) / BN;
  const int splits = (total_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
  const int total_work = row_tiles * col_tiles * splits;
  // consecutive work items share the weight tile where they can (tokens on M: same columns,
  // next rows), so that it is served from L2
  auto work_at = [&](int w) {
    Work k;
    k.split = w % splits;
    const int tile = w / splits;
    if (SWAP) { k.row0 = (tile / col_tiles) * BLOCK_M; k.col0 = (tile % col_tiles) * BN; }   // token tiles of one weight tile side by side
    else { k.row0 = (tile % row_tiles) * TILE_M + (int)rank * BLOCK_M; k.col0 = (tile / row_tiles) * BN; }   // this CTA's rows
    k.kb_begin = k.split * p.k_blocks_per_split;
    k.num_kb = min(total_kb, k.kb_begin + p.k_blocks_per_split) - k.kb_begin;
    return k;
  };

  pdl_launch_dependents();
  // instrumented builds: a decode layer's four products and the head keep a record each (q/k/v, output, gate/up, down, head)
#ifdef SPROUT_TIMELINE
  const int tl_slot = p.epilogue == EPI_SWIGLU ? 2 : p.epilogue == EPI_STORE ? 4 : p.N > p.K ? 0 : p.N == p.K ? 1 : 3;
  if (tl_slot >= 0) SPROUT_TL_ENTRY(tl_slot);
#endif
  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; s++) { mbar_init(&full_bar[s], (SWAP && p.x32) ? 2 : 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; a++) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], PAIR ? 16 : 8); }
    mbar_init(epi_bar, 8);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, L::TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (PAIR) {
    // The pair's MMAs write both CTAs' tensor memory at one address.  Each CTA has its SM to
    // itself (its shared memory leaves no room for another) and has allocated from an empty tensor
    // memory, so both got column 0; anything else is refused.  Nobody counts on the other CTA's
    // barriers before they are initialised: the cluster meets first.
    if (tmem_base != 0 && threadIdx.x == 0) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_BAD_LAYOUT); }
    cluster_barrier();
  }

  // The copy thread and the MMA thread each run one thread's worth of dependent instructions per
  // k-block, and the tensor cores finish a k-block in under 300 cycles: their loops keep the
  // stage, its phase, the barrier addresses and the descriptors in running variables, and read
  // the abort flag only while a wait is not satisfied at once.
  const uint32_t smem_base = smem_u32(smem), full_base = smem_u32(full_bar), empty_base = smem_u32(empty_bar);
  int issued = 0;
  if (warp == 0 && lane == 0) {
    // ---------------- producer: TMA loads of the two operand tiles, stage by stage.
    // The weights were written before any kernel of the step ran: their tiles for the first
    // round of stages are requested before waiting for the kernel that produces the activations.
    const CUtensorMap* weight_map = SWAP ? &map_rows : &map_cols;
    const CUtensorMap* act_map = SWAP ? &map_cols : &map_rows;
    constexpr uint32_t W_OFF = SWAP ? 0 : L::A_BYTES, X_OFF = SWAP ? L::A_BYTES : 0;
    uint32_t s = 0, parity = 1;                   // stage and the parity of its "empty" phase to wait for
    uint32_t stage_addr = smem_base;
    int it = 0;
    bool ok = true;
    // pairs: both CTAs' copies count on the first CTA's barrier, which expects both CTAs' bytes
    const uint32_t count_base = PAIR ? cluster_map_shared(full_base, 0) : full_base;
    const bool made_here = SWAP && p.x32 != nullptr;          // the token tiles are written by the epilogue warps
    const uint32_t STAGE_TX = made_here ? (uint32_t)L::A_BYTES : (uint32_t)((PAIR ? 2 : 1) * (L::A_BYTES + L::B_BYTES));
    auto copy = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
      if (PAIR) tma_load_2d_pair(dst, map, bar, x, y); else tma_load_2d_addr(dst, map, bar, x, y);
    };
    for (int w = first_work; w < total_work && ok; w += work_stride) {
      const Work k = work_at(w);
      const int weight_row = SWAP ? k.row0 : k.col0 + (PAIR ? (int)rank * (BN / 2) : 0), act_row = SWAP ? k.col0 : k.row0;
      int early = 0;
      if (w == first_work) {
        early = min(k.num_kb, L::STAGES);
        for (int i = 0; i < early; i++) {
          if (rank == 0) mbar_expect_tx_addr(full_base + 8 * i, STAGE_TX);
          copy(smem_base + i * L::STAGE_BYTES + W_OFF, weight_map, count_base + 8 * i, (k.kb_begin + i) * BLOCK_K, weight_row);
        }
        pdl_wait();
#ifdef SPROUT_TIMELINE
        if (tl_slot >= 0) SPROUT_TL_WAITED(tl_slot);
#endif
      }
      int x = k.kb_begin * BLOCK_K;
      for (int i = 0; i < k.num_kb; i++, it++, x += BLOCK_K) {
        const uint32_t count_addr = count_base + 8 * s;
        if (i >= early) {
          if (!mbar_wait_addr(empty_base + 8 * s, parity, abort_flag)) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); ok = false; break; }
          if (rank == 0) mbar_expect_tx_addr(full_base + 8 * s, STAGE_TX);
          copy(stage_addr + W_OFF, weight_map, count_addr, x, weight_row);
        }
        if (!made_here) copy(stage_addr + X_OFF, act_map, count_addr, x, act_row);
        issued = it + 1;
        if (++s == L::STAGES) { s = 0; parity ^= 1; stage_addr = smem_base; } else stage_addr += L::STAGE_BYTES;
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------- MMA issuer (of a pair: the first CTA's)
    const uint32_t idesc = umma_idesc(TILE_M, BN);
    const uint64_t a_desc0 = umma_smem_desc(smem), b_desc0 = umma_smem_desc(smem + L::A_BYTES);
    constexpr uint64_t STAGE_STEP = L::STAGE_BYTES >> 4;      // a stage further in the descriptor's address field
    uint64_t a_desc = a_desc0, b_desc = b_desc0;
    uint32_t s = 0, parity = 0;
    bool ok = true;
    int tiles_done = 0;
    for (int w = first_work; w < total_work && ok; w += work_stride, tiles_done++) {
      const Work k = work_at(w);
      const int acc = tiles_done & 1;
      // the epilogue (of both CTAs) must have read this accumulator's previous tile out
      const bool drained = PAIR ? mbar_wait_cluster(smem_u32(&acc_empty[acc]), ((tiles_done >> 1) & 1) ^ 1, abort_flag)
                                : mbar_wait(&acc_empty[acc], ((tiles_done >> 1) & 1) ^ 1, abort_flag);
      if (!drained) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      uint32_t accumulate = 0;
      for (int i = 0; i < k.num_kb; i++) {
        if (!mbar_wait_addr(full_base + 8 * s, parity, abort_flag)) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); ok = false; break; }
        tc_fence_after();
        // advancing 16 elements (32 bytes) along K inside the swizzled row: +2 in the address field
        if (PAIR) {
          umma_bf16_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
          umma_bf16_pair(d_tmem, a_desc + 2, b_desc + 2, idesc, 1);
          umma_bf16_pair(d_tmem, a_desc + 4, b_desc + 4, idesc, 1);
          umma_bf16_pair(d_tmem, a_desc + 6, b_desc + 6, idesc, 1);
          umma_commit_pair(empty_base + 8 * s, 3);   // the stage is free in both CTAs once these MMAs have read it
        } else {
          umma_bf16(d_tmem, a_desc, b_desc, idesc, accumulate);
          umma_bf16(d_tmem, a_desc + 2, b_desc + 2, idesc, 1);
          umma_bf16(d_tmem, a_desc + 4, b_desc + 4, idesc, 1);
          umma_bf16(d_tmem, a_desc + 6, b_desc + 6, idesc, 1);
          umma_commit_addr(empty_base + 8 * s);   // the stage is free once these MMAs have read it
        }
        accumulate = 1;
        if (++s == L::STAGES) { s = 0; parity ^= 1; a_desc = a_desc0; b_desc = b_desc0; } else { a_desc += STAGE_STEP; b_desc += STAGE_STEP; }
      }
      if (ok) {                              // the accumulator is complete once all MMAs are
        if (PAIR) umma_commit_pair(smem_u32(&acc_full[acc]), 3); else umma_commit(&acc_full[acc]);
      }
    }
  } else if (warp >= 2) {
    // ---------------- epilogue: TMEM -> registers -> global
    pdl_wait();                         // the epilogue reads and writes `out`
    const int quarter = warp & 3;       // a warp reads TMEM lanes 32 * (warp % 4) ..
    const int half = (warp - 2) >> 2;   // two warps per lane quarter take alternate 16-column chunks
    int tiles_done = 0;
    uint32_t groups_done = 0, epi_phase = 0;
    const bool issuer = warp == 2 && lane == 0;   // issues the reductions of the residual epilogue
    // all 8 warps meet; false when the wait ran out
    auto epi_sync = [&]() {
      bool met = true;
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(epi_bar);
        met = mbar_wait(epi_bar, epi_phase, abort_flag);
        if (!met) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      }
      epi_phase ^= 1;
      return (bool)__shfl_sync(0xffffffffu, met, 0);
    };
    if (SWAP && p.x32) {
      // The tokens' operand, made here: for every k-block of this CTA's (one) work item the tile
      // [BN tokens, 64 elements] = bfloat16(x * gain), in the layout the 128-byte swizzle gives a
      // copied tile (16-byte chunk c of row t at chunk c ^ (t & 7)); rows and columns beyond the
      // matrix are zero.  K ranges longer than the ring take a stage again once the products that
      // read it are done (its "empty" barrier, as the copy thread does for the weights).
      const Work k = work_at(first_work);
      const int et = (int)threadIdx.x - 64;                    // 0..255 among the epilogue warps
      if (first_work < total_work) {
        for (int i = 0; i < k.num_kb; i++) {
          const int stage = i % L::STAGES;
          if (i >= L::STAGES) {
            bool freed = true;
            if (lane == 0) {
              freed = mbar_wait(&empty_bar[stage], ((i / L::STAGES) - 1) & 1, abort_flag);
              if (!freed) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
            }
            if (!__shfl_sync(0xffffffffu, freed, 0)) break;
          }
          uint8_t* tile = smem + stage * L::STAGE_BYTES + L::A_BYTES;
          const int k0 = (k.kb_begin + i) * BLOCK_K;
          for (int idx = et; idx < BN * 8; idx += 256) {
            const int t = idx >> 3, c = idx & 7, m = k.col0 + t, kk = k0 + c * 8;
            uint4 packed = make_uint4(0u, 0u, 0u, 0u);
            if (m < p.M && kk < p.K) {                          // K is a multiple of 8: a chunk lies inside or outside
              const float4 a = __ldcg((const float4*)(p.x32 + (size_t)m * p.ldx + kk)), b = __ldcg((const float4*)(p.x32 + (size_t)m * p.ldx + kk) + 1);
              const float4 ga = *(const float4*)(p.gain + kk), gb = *((const float4*)(p.gain + kk) + 1);
              __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x * ga.x, a.y * ga.y), h1 = __floats2bfloat162_rn(a.z * ga.z, a.w * ga.w);
              __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x * gb.x, b.y * gb.y), h3 = __floats2bfloat162_rn(b.z * gb.z, b.w * gb.w);
              packed = make_uint4(*(uint32_t*)&h0, *(uint32_t*)&h1, *(uint32_t*)&h2, *(uint32_t*)&h3);
            }
            *(uint4*)(tile + t * 128 + ((c ^ (t & 7)) << 4)) = packed;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (!epi_sync()) break;                              // all eight warps have written their chunks
          if (issuer) mbar_arrive(&full_bar[stage]);
        }
      }
    }
    // the accumulator goes back to the MMA issuer: of a pair's second CTA, to the first CTA's barrier
    auto release_accumulator = [&](int acc) {
      if (PAIR && rank == 1) mbar_arrive_cluster(cluster_map_shared(smem_u32(&acc_empty[acc]), 0));
      else mbar_arrive(&acc_empty[acc]);
    };
    for (int w = first_work; w < total_work; w += work_stride, tiles_done++) {
      const Work k = work_at(w);
      const int acc = tiles_done & 1;
      const int row = k.row0 + quarter * 32 + lane;
      const int col0 = k.col0;
      // one lane waits for the barrier; tcgen05.ld is warp-wide: all lanes go on or none
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&acc_full[acc], (tiles_done >> 1) & 1, abort_flag);
        if (!ok) { *abort_flag = 1; atomicOr(p.status, SPROUT_STATUS_WAIT_TIMEOUT); }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
      const bool first_split = k.split == 0;
      if (!SWAP && p.epilogue == EPI_RESIDUAL_TMA) {
        // out += D through shared memory: the 8 warps fill a [128 rows, 32 columns] float32 tile
        // in the swizzled layout of the output's tensor map, one thread hands it to the TMA unit,
        // which adds it to the output in L2 (rows and columns beyond the matrix are clipped).
        // Two tiles alternate; a tile is written again once the reduction before last has read it.
        const int tile_row = quarter * 32 + lane;
        bool met = true;
#pragma unroll 1
        for (int c = half * 16; c < BN && met; c += 32, groups_done++) {
          uint32_t raw[16];
          tmem_load16(taddr + c, raw);
          const int n_base = col0 + c;
          uint8_t* tile = staging + (groups_done & 1) * (STAGING_BYTES / 2);
          if (groups_done >= 2) {
            if (issuer) bulk_wait_group_read<1>();
            met = epi_sync();
            if (!met) break;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) {
            float4 v;
            const bool biased = p.bias && first_split;     // the K splits of a tile all add into the output: one brings the bias
            v.x = __uint_as_float(raw[4 * q4]) + ((biased && n_base + 4 * q4 < p.N) ? p.bias[n_base + 4 * q4] : 0.f);
            v.y = __uint_as_float(raw[4 * q4 + 1]) + ((biased && n_base + 4 * q4 + 1 < p.N) ? p.bias[n_base + 4 * q4 + 1] : 0.f);
            v.z = __uint_as_float(raw[4 * q4 + 2]) + ((biased && n_base + 4 * q4 + 2 < p.N) ? p.bias[n_base + 4 * q4 + 2] : 0.f);
            v.w = __uint_as_float(raw[4 * q4 + 3]) + ((biased && n_base + 4 * q4 + 3 < p.N) ? p.bias[n_base + 4 * q4 + 3] : 0.f);
            const int chunk = half * 4 + q4;
            *(float4*)(tile + tile_row * 128 + ((chunk ^ (tile_row & 7)) << 4)) = v;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          met = epi_sync();
          if (!met) break;
          if (issuer) {
            tma_reduce_add_2d(&map_out, smem_u32(tile), col0 + (c & ~31), k.row0);
            bulk_commit_group();
          }
        }
        if (!met) break;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) release_accumulator(acc);
        continue;
      }
#pragma unroll 1
      for (int c = half * 16; c < BN; c += 32) {
        uint32_t raw[16];
        tmem_load16(taddr + c, raw);
        if (SWAP) {
          // row = output feature, columns = tokens: lanes hold consecutive features
          if (p.epilogue == EPI_SWIGLU) {
            // lanes l and l ^ 8 hold a gate row and its up row (128-row tiles start on multiples of 16)
            const int out_n = (row >> 4) * 8 + (row & 7);
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const float mine = __uint_as_float(raw[j]);
              const float other = __shfl_xor_sync(0xffffffffu, mine, 8);
              const int m = col0 + c + j;
              if ((lane & 8) == 0 && row < p.N && m < p.M)
                ((__nv_bfloat16*)p.out)[(size_t)m * p.ldo + out_n] = __float2bfloat16_rn(silu_mul(mine, other));
            }
          } else if (row < p.N) {
            const float b = (p.bias && first_split) ? p.bias[row] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; j++) {
              const int m = col0 + c + j;
              if (m >= p.M) break;
              const float v = __uint_as_float(raw[j]) + b;
              const size_t at = (size_t)m * p.ldo + row;
              if (p.epilogue == EPI_RESIDUAL_ATOMIC) atomicAdd((float*)p.out + at, v);
              else if (p.epilogue == EPI_RESIDUAL) ((float*)p.out)[at] += v;
              else if (p.out_is_f32) ((float*)p.out)[at] = v;
              else ((__nv_bfloat16*)p.out)[at] = __float2bfloat16_rn(v);
            }
          }
        } else {
          // row = token, columns = output features: each lane writes a contiguous run of its row
          if (row < p.M) {
            const int n_base = col0 + c;
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = __uint_as_float(raw[j]) + ((p.bias && n_base + j < p.N) ? p.bias[n_base + j] : 0.f);
            const size_t at = (size_t)row * p.ldo + n_base;
            const bool whole = n_base + 16 <= p.N;
            if (p.epilogue == EPI_SWIGLU) {
              if (n_base < p.N) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(silu_mul(v[2 * j], v[2 * j + 8]), silu_mul(v[2 * j + 1], v[2 * j + 9]));
                  packed[j] = *(uint32_t*)&h;
                }
                __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)row * p.ldo + (n_base >> 1);
                if ((((size_t)row * p.ldo + (n_base >> 1)) & 7) == 0) *(uint4*)o = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                else { for (int j = 0; j < 4; j++) ((uint32_t*)o)[j] = packed[j]; }
              }
            } else if (p.epilogue == EPI_RESIDUAL) {
              float* o = (float*)p.out + at;
              if (whole && (at & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                  float4 r = *(float4*)(o + j);
                  r.x += v[j]; r.y += v[j + 1]; r.z += v[j + 2]; r.w += v[j + 3];
                  *(float4*)(o + j) = r;
                }
              } else {
                for (int j = 0; j < 16 && n_base + j < p.N; j++) o[j] += v[j];
              }
            } else if (p.out_is_f32) {
              float* o = (float*)p.out + at;
              if (whole && (at & 3) == 0) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) *(float4*)(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
                for (int j = 0; j < 16 && n_base + j < p.N; j++) o[j] = v[j];
              }
            } else {
              __nv_bfloat16* o = (__nv_bfloat16*)p.out + at;
              if (whole && (at & 7) == 0) {
                uint32_t packed[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                  packed[j] = *(uint32_t*)&h;
                }
                *(uint4*)(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                *(uint4*)(o + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
              } else {
                for (int j = 0; j < 16 && n_base + j < p.N; j++) o[j] = __float2bfloat16_rn(v[j]);
              }
            }
          }
        }
      }
      // this warp has read the accumulator out: hand it back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) release_accumulator(acc);
    }
  }
  if (warp == 2 && lane == 0) bulk_wait_group<0>();     // the reductions have been performed
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 0 && lane == 0) {
    // copies already issued still write shared memory: wait for them (bounded) before leaving
    for (int i = max(0, issued - L::STAGES); i < issued; i++)
      mbar_wait(&full_bar[i % L::STAGES], (i / L::STAGES) & 1);
  }
  __syncthreads();
  if (PAIR) cluster_barrier();      // neither CTA leaves while the other may still count on its barriers or read its memory
  if (warp == 1) tmem_dealloc(tmem_base, L::TMEM_COLS);
#ifdef SPROUT_TIMELINE
  if (tl_slot >= 0) SPROUT_TL_EXIT(tl_slot);
#endif
}

// ------------------------------------------------------------------ host side
// `work` = tiles x K splits; the grid is one CTA per SM at most, each walking the work list.
// Pairs: `work` counts 256 x BN tiles; the grid is one cluster of two CTAs per two SMs at most.
template <int BN>
int launch_pair(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const CUtensorMap& out_map, const Params& p, int work,
                cudaStream_t stream) {
  using L = Layout<BN, true>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (err != cudaSuccess) return sprout_fail("gemm_bf16: cannot reserve %d bytes of shared memory: %s", L::SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  const int pairs = work < sm_count() / 2 ? work : sm_count() / 2;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(NUM_THREADS);
  config.dynamicSmemBytes = L::SMEM_BYTES;
  config.stream = stream;
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = sprout_pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&config, gemm_tcgen05_kernel<BN, false, true>, rows_map, cols_map, out_map, p);
  return sprout_check_launch("gemm_bf16 (pairs)");
}

template <int BN, bool SWAP>
int launch(const CUtensorMap& rows_map, const CUtensorMap& cols_map, const CUtensorMap& out_map, const Params& p, int work,
           cudaStream_t stream) {
  using L = Layout<BN>;
  const dim3 grid(work < sm_count() ? work : sm_count());
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, SWAP>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::SMEM_BYTES);
    if (err != cudaSuccess) return sprout_fail("gemm_bf16: cannot reserve %d bytes of shared memory: %s", L::SMEM_BYTES, cudaGetErrorString(err));
    configured = true;
  }
  sprout_launch(gemm_tcgen05_kernel<BN, SWAP>, grid, dim3(NUM_THREADS), L::SMEM_BYTES, stream, rows_map, cols_map, out_map, p);
  return sprout_check_launch("gemm_bf16");
}

}  // namespace

// A [M, K] bf16 row stride lda; W [N, K] bf16 contiguous; out [M, N] row stride ldo, bf16 or
// float32.  residual != 0: out is float32 and the product is added to it.  orientation: 0 picks
// by M (weight rows on the MMA's M axis up to 256 tokens, up to 64 with the SwiGLU epilogue, tokens on M beyond), 1 forces tokens
// on M (128 x 128 tiles, or 256 x 256 tiles of CTA pairs where N is a multiple of 256), 2 weights
// on M (tokens in tiles of 16..256), 3 tokens on M with single CTAs only, 4 with CTA pairs only.
// split_k > 1 (weights on M, residual, at most 256 tokens) divides K among CTAs and adds with
// atomics.
// residual == 2: the SwiGLU epilogue (no bias; out is bfloat16 [M, N/2]; N a multiple of 16).
SPROUT_API int sprout_gemm_bf16(const void* A, const void* W, const float* bias, void* out, int out_dtype,
                                int residual, int M, int N, int K, int lda, int ldo, int orientation,
                                int split_k, int* status, cudaStream_t stream) {
  const bool swiglu = residual == 2;
  if (swiglu) {
    residual = 0;
    SPROUT_REQUIRE(N % 16 == 0 && !bias && out_dtype == SPROUT_BF16 && ldo >= N / 2 && ldo % 2 == 0,
                   "gemm_bf16: the SwiGLU epilogue needs N %% 16 == 0, no bias and a bfloat16 output [M, N/2]");
  }
  SPROUT_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_bf16: sizes must be positive (M=%d N=%d K=%d)", M, N, K);
  SPROUT_REQUIRE(A && W && out && status, "gemm_bf16: null pointer");
  SPROUT_REQUIRE(K % 8 == 0 && lda % 8 == 0, "gemm_bf16: K (%d) and the row stride of A (%d) must be multiples of 8 "
                 "(TMA rows start on 16-byte boundaries)", K, lda);
  SPROUT_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_bf16: operands must be 16-byte aligned");
  SPROUT_REQUIRE(lda >= K && (swiglu || ldo >= N), "gemm_bf16: row strides smaller than the rows");
  SPROUT_REQUIRE(out_dtype == SPROUT_F32 || out_dtype == SPROUT_BF16, "gemm_bf16: unknown output dtype %d", out_dtype);
  SPROUT_REQUIRE(!residual || out_dtype == SPROUT_F32, "gemm_bf16: a residual needs a float32 output");
  // Which operand fills the MMA's 128 rows (orientation 0 picks): the weights for a stream of
  // weights past few tokens (up to 256 tokens; with split K where the epilogue adds).  The SwiGLU
  // epilogue cannot split K, so its 128-row weight tiles leave SMs idle while the token tiles grow:
  // measured at the 0.5B / 7B / 14B gate/up shapes, weights on M wins up to 64 tokens, tokens on M
  // with single CTAs from 65 to 128 (9.7 against 12.5 us at 128 tokens of the 0.5B shape), CTA
  // pairs beyond (12.7 against 18.1 us at 256).
  // Between 33 and 64 tokens the SwiGLU product goes tokens on M as well when its 128-row weight tiles
  // would leave more than two SMs in five idle (the 0.5B shape: 76 tiles, 9.2 against 9.8 us).
  const bool few_weight_tiles = swiglu && M > 32 && 5LL * ((N + BLOCK_M - 1) / BLOCK_M) < 3LL * sm_count();
  const bool swap = orientation == 2 || (orientation == 0 && M <= (swiglu ? 64 : 256) && !few_weight_tiles);    // 1: tokens on M in CTA pairs, 3: single CTAs
  if (split_k < 1) split_k = 1;
  SPROUT_REQUIRE(split_k == 1 || (swap && residual && M <= 256), "gemm_bf16: split_k needs weights-on-M with a residual output and at most 256 tokens "
                 "(with tokens on M the kernel splits K by itself where that pays)");

  Params p;
  p.bias = bias; p.out = out; p.out_is_f32 = out_dtype == SPROUT_F32;
  p.epilogue = swiglu ? EPI_SWIGLU : residual ? (split_k > 1 ? EPI_RESIDUAL_ATOMIC : EPI_RESIDUAL) : EPI_STORE;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.status = status;
  p.x32 = nullptr; p.gain = nullptr; p.ldx = 0;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (split_k > total_kb) split_k = total_kb;
  p.k_blocks_per_split = (total_kb + split_k - 1) / split_k;
  split_k = (total_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;

  CUtensorMap map_a, map_w;
  if (swap) {
    const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (tensor_map(W, N, K, K, BLOCK_M, &map_w)) return 1;
    if (tensor_map(A, M, K, lda, bn, &map_a)) return 1;
    const long long work = (long long)((N + BLOCK_M - 1) / BLOCK_M) * ((M + bn - 1) / bn) * split_k;
    SPROUT_REQUIRE(work <= 0x7fffffffLL, "gemm_bf16: too many tiles");
    switch (bn) {
      case 16: return launch<16, true>(map_w, map_a, map_a, p, (int)work, stream);
      case 32: return launch<32, true>(map_w, map_a, map_a, p, (int)work, stream);
      case 64: return launch<64, true>(map_w, map_a, map_a, p, (int)work, stream);
      case 128: return launch<128, true>(map_w, map_a, map_a, p, (int)work, stream);
      default: return launch<256, true>(map_w, map_a, map_a, p, (int)work, stream);
    }
  }
  // Tokens on M.  The residual epilogue goes through the TMA unit where the output's rows allow a
  // tensor map; its additions are atomic in L2, so a tile's K range may then be split among CTAs.
  const bool reduce = p.epilogue == EPI_RESIDUAL && ldo % 4 == 0 && ((uintptr_t)out & 15) == 0;
  // Tile width and K split: a k-block of a 128 x bn tile moves (128 + bn) x 128 bytes into shared
  // memory and out again, which is what its time follows; wider tiles move less per product but
  // make fewer CTAs.  The pick minimises rounds x k-blocks x (128 + bn) over the widths that
  // divide N (128 always) and, for the reducing epilogue, splits of at least 4 k-blocks.
  // N a multiple of 256: 256 x 256 tiles of CTA pairs (measured: gate/up 2048 x 9728 x 896
  // 41 -> 39 us, 8192 tokens 145 -> 134 us; on narrower tiles single CTAs are as fast).
  int bn = 128;
  split_k = 1;
  const bool pair = orientation == 4 || (orientation != 3 && N % 256 == 0 && !(orientation == 0 && swiglu && M <= 128));
  if (pair) {
    bn = N % 256 == 0 ? 256 : 128;
  } else if (orientation != 3) {
    const int widths[4] = {128, 192, 224, 256};
    const long long row_tiles = (M + BLOCK_M - 1) / BLOCK_M;
    long long best = -1;
    for (int width : widths) {
      if (width != 128 && N % width != 0) continue;
      for (int split = 1; split <= (reduce ? 4 : 1); split++) {
        const int kb = (total_kb + split - 1) / split;
        if (split > 1 && kb < 4) break;
        const long long items = row_tiles * ((N + width - 1) / width) * split;
        const long long rounds = (items + sm_count() - 1) / sm_count();
        const long long cost = rounds * (kb + 4 * (split > 1)) * (128 + width);   // a split costs another epilogue and its reduction
        if (best < 0 || cost < best) { best = cost; bn = width; split_k = split; }
      }
    }
  }
  p.k_blocks_per_split = (total_kb + split_k - 1) / split_k;
  split_k = (total_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
  if (tensor_map(A, M, K, lda, BLOCK_M, &map_a)) return 1;
  if (tensor_map(W, N, K, K, pair ? bn / 2 : bn, &map_w)) return 1;
  const long long work = (long long)((N + bn - 1) / bn) * ((M + (pair ? 2 : 1) * BLOCK_M - 1) / ((pair ? 2 : 1) * BLOCK_M)) * split_k;
  SPROUT_REQUIRE(work <= 0x7fffffffLL, "gemm_bf16: too many tiles");
  CUtensorMap map_out = map_a;
  if (reduce) {
    if (tensor_map(out, M, N, ldo, BLOCK_M, &map_out, 4)) return 1;
    p.epilogue = EPI_RESIDUAL_TMA;
  }
  if (pair) {
    if (bn == 256) return launch_pair<256>(map_a, map_w, map_out, p, (int)work, stream);
    return launch_pair<128>(map_a, map_w, map_out, p, (int)work, stream);
  }
  switch (bn) {
    case 256: return launch<256, false>(map_a, map_w, map_out, p, (int)work, stream);
    case 224: return launch<224, false>(map_a, map_w, map_out, p, (int)work, stream);
    case 192: return launch<192, false>(map_a, map_w, map_out, p, (int)work, stream);
    default: return launch<128, false>(map_a, map_w, map_out, p, (int)work, stream);
  }
}

// out [M, N] float32 (row stride ldo) += bfloat16(x * gain) W^T for up to 256 tokens: the product of a
// normalised input without its scale.  x: float32 [M, K] (row stride ldx), the rows before
// normalisation; gain: float32 [K].  The consumer multiplies token m's sums by 1 / rms(x[m]) (the
// decode attention kernels do, with the bias and the rotation), which is the RMSNorm's arithmetic
// with the division moved behind the product.  Weights on M, K split among CTAs (atomic adds); the
// tokens' tiles are converted inside the kernel, so no kernel stands between the residual stream
// and this product.  Every CTA has one work item (it makes that item's token tiles), or the call is refused.
SPROUT_API int sprout_gemm_bf16_unscaled(const float* x, int ldx, const float* gain, const void* W, float* out, int M, int N, int K,
                                         int ldo, int split_k, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(M > 0 && M <= 256 && N > 0 && K > 0, "gemm_bf16_unscaled: 1..256 tokens, positive sizes (M=%d N=%d K=%d)", M, N, K);
  SPROUT_REQUIRE(x && gain && W && out && status, "gemm_bf16_unscaled: null pointer");
  SPROUT_REQUIRE(K % 8 == 0 && ldx % 4 == 0 && ldx >= K && ldo >= N, "gemm_bf16_unscaled: K (%d) must be a multiple of 8, the rows of x (%d) of 4", K, ldx);
  SPROUT_REQUIRE(((uintptr_t)x & 15) == 0 && ((uintptr_t)gain & 15) == 0 && ((uintptr_t)W & 15) == 0, "gemm_bf16_unscaled: operands must be 16-byte aligned");
  Params p;
  p.bias = nullptr; p.out = out; p.out_is_f32 = 1; p.epilogue = EPI_RESIDUAL_ATOMIC;
  p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.status = status;
  p.x32 = x; p.gain = gain; p.ldx = ldx;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (split_k < 1) split_k = 1;
  if (split_k > total_kb) split_k = total_kb;
  p.k_blocks_per_split = (total_kb + split_k - 1) / split_k;
  split_k = (total_kb + p.k_blocks_per_split - 1) / p.k_blocks_per_split;
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const long long work = (long long)((N + BLOCK_M - 1) / BLOCK_M) * ((M + bn - 1) / bn) * split_k;
  CUtensorMap map_w;
  if (tensor_map(W, N, K, K, BLOCK_M, &map_w)) return 1;
  SPROUT_REQUIRE(work <= sm_count(), "gemm_bf16_unscaled: %lld work items for %d SMs (a CTA makes the tokens' tiles of one item): "
                 "split K less or use the separate norm", work, sm_count());
  switch (bn) {
    case 16: return launch<16, true>(map_w, map_w, map_w, p, (int)work, stream);
    case 32: return launch<32, true>(map_w, map_w, map_w, p, (int)work, stream);
    case 64: return launch<64, true>(map_w, map_w, map_w, p, (int)work, stream);
    case 128: return launch<128, true>(map_w, map_w, map_w, p, (int)work, stream);
    default: return launch<256, true>(map_w, map_w, map_w, p, (int)work, stream);
  }
}

// 1 when sprout_gemm_bf16_unscaled takes these sizes with this K split on this device.
SPROUT_API int sprout_gemm_bf16_unscaled_supported(int M, int N, int K, int split_k) {
  if (M <= 0 || M > 256 || N <= 0 || K <= 0 || K % 8) return 0;
  const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
  if (split_k < 1) split_k = 1;
  if (split_k > total_kb) split_k = total_kb;
  const int per = (total_kb + split_k - 1) / split_k;
  split_k = (total_kb + per - 1) / per;
  const int bn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const long long work = (long long)((N + BLOCK_M - 1) / BLOCK_M) * ((M + bn - 1) / bn) * split_k;
  return work <= sm_count() ? 1 : 0;
}

SPROUT_TL_READER(gemm_tcgen05)
