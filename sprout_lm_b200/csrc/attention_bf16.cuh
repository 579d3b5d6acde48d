// What the bfloat16 attention kernels of attention_bf16.cu and attention_decode_mma.cu share: the
// tensor-core and copy helpers, and the parameters of a decode launch.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace sprout_attn {

// =============================================================================== tensor-core helpers
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_addr(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_addr(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&h;
}

// =============================================================================== decode
constexpr int DEC_THREADS = 128;      // == keys per pass
constexpr int MAX_GROUP = 16;         // query heads per key/value head served by one CTA pass

struct DecodeParams {
  const __nv_bfloat16* q; int q_stride;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* block_table; int table_stride;
  const int* context_lens;            // keys visible to the request's query: positions 0..len-1
  __nv_bfloat16* out; int out_stride;
  float* part_out;                    // [requests, heads, splits, head_dim]
  float* part_ml;                     // [requests, heads, splits, 2]
  int heads, kv_heads, head_dim, page_tokens, num_pages, split_keys, splits;
  int* status;
  // fused projection tail (tensor-core kernel, FUSED): q, k, v of the new token come as float32
  // sums [requests, heads + 2 kv_heads, head_dim] from a split-K product, plus a bias; the
  // kernel rotates q and k by the token's position (tables [max_positions, rotary_dim / 2], may be
  // null; the first rotary_dim elements of a head turn, in half-split pairs (d, d + rotary_dim / 2) or,
  // with `interleaved`, in pairs (2d, 2d + 1)), appends k and v to the cache and leaves the sums zeroed
  float* acc; const float* bias; const float* cos_table; const float* sin_table; int max_positions;
  int rotary_dim, interleaved;
  __nv_bfloat16* k_append; __nv_bfloat16* v_append;
  // The sums may be those of a product whose input was normalised without its scale (RMSNorm with the
  // division moved behind the product): norm_x [requests, norm_width] float32 are the rows before the
  // norm; the kernel multiplies request r's sums by 1 / sqrt(mean(norm_x[r]^2) + norm_eps).  Null: no scale.
  const float* norm_x; int norm_width; float norm_eps;
};

// The tensor-core decode kernel (attention_decode_mma.cu): launch for these parameters (head sizes of
// 16 to 128 in steps of 16), and how many of its CTAs an SM holds at once (0: not a head size it takes).
int launch_decode_mma_any(const DecodeParams& p, bool fused, bool cluster, int requests, cudaStream_t stream);
int decode_mma_ctas_per_sm_any(int head_dim, bool fused, bool cluster);

}  // namespace sprout_attn
