// Shared by the kernels for steps of a few tokens (ffn_decode.cu, linear_decode.cu): weights as
// the 16-row operand of `mma.sync.m16n8k16`, the tokens as its 8 columns (one or two such tiles
// of tokens), weight tiles
// brought in by TMA with the 128-byte swizzle, and the division of a matrix into pieces for
// the CTAs.
#pragma once

#include "tcgen05.cuh"

namespace {

constexpr int SMALL_MAX_TOKENS = 16;        // two tiles of the MMA's N = 8

// Rows of the tokens' operand that a launch for `tokens` tokens holds: whole tiles of 8.
__host__ __device__ __forceinline__ int token_rows(int tokens) { return tokens <= 8 ? 8 : 16; }

// The split of a range of n items over parts: part p gets [n*p/parts, n*(p+1)/parts)  (n * parts stays far below 2^32).
__host__ __device__ __forceinline__ int share_begin(int n, int part, int parts) { return (int)(((unsigned)n * (unsigned)part) / (unsigned)parts); }

// Address of 16-byte chunk `chunk` (0..7) of row `row` in a tile of 128-byte rows that TMA wrote
// with its 128-byte swizzle (the tile starts on a 1024-byte boundary).
__device__ __forceinline__ uint32_t swizzled(uint32_t tile, int row, int chunk) {
  return tile + (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A [tiles x 16 rows, ksteps x 16 columns] matrix in row_groups x k_splits pieces, at most one per
// CTA, each at most 16 tiles high (256 rows: one TMA box).  A CTA's eight warps take its tiles in
// turn and walk a tile's K steps one after the other, so the split with the fewest steps per warp
// wins (a piece of one tile and many K steps would leave seven warps idle); among equals the one
// with the least bytes per piece, K counted in whole boxes of 64 columns.  False when no split
// exists.
inline bool plan_pieces(int tiles, int ksteps, int ctas, int* row_groups, int* k_splits) {
  long long best_steps = -1, best_bytes = -1;
  for (int groups = 1; groups <= tiles && groups <= ctas; groups++) {
    const int rows = (tiles + groups - 1) / groups;
    if (rows > 16) continue;
    int splits = ctas / groups;
    if (splits > ksteps) splits = ksteps;
    const int steps = (ksteps + splits - 1) / splits;
    const long long per_warp = (long long)((rows + 7) / 8) * steps;
    const long long bytes = (long long)rows * ((steps + 3) / 4 * 4);
    if (best_steps < 0 || per_warp < best_steps || (per_warp == best_steps && bytes < best_bytes)) {
      best_steps = per_warp; best_bytes = bytes; *row_groups = groups; *k_splits = splits;
    }
  }
  return best_steps >= 0;
}

}  // namespace
