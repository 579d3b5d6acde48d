// The tensor-core decode attention kernel for bfloat16 caches (mma.sync, keys in passes of 128 staged
// by cp.async, splits merged in a thread-block cluster or through memory), its launch and its
// occupancy, as templates over the head size: attention_decode_mma.cu instantiates the head sizes up
// to 64, attention_decode_mma_wide.cu those from 80 to 128 (two compilation units build side by side).
#pragma once
#include "attention_bf16.cuh"

namespace cg = cooperative_groups;

// With -DATTN_STAMPS the first thread of the decode kernel's first CTA records the time
// (%globaltimer) at the end of each phase; sprout_attention_stamps copies the last launch's records out.
#ifdef ATTN_STAMPS
static __device__ unsigned long long g_attn_stamps[16];
#define ATTN_STAMP(i) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); g_attn_stamps[i] = t; } } while (0)
#else
#define ATTN_STAMP(i) do { } while (0)
#endif

namespace sprout_attn {
namespace {

// Decode attention on tensor cores (head sizes up to 128, up to 16 query heads per key/value
// head).  The query heads of the group are the 16 rows of an m16n8k16 tile (rows beyond the
// group are zero); each of the 4 warps takes 32 keys of a 128-key pass: S = Q K^T, running
// softmax, O += P V, all as mma.sync on keys and values staged in shared memory by cp.async.
// The warps' partial results are merged through shared memory into the CTA's partial result
// (maximum, sum, unnormalised output), which then goes the same ways as in the CUDA-core kernel of
// attention_bf16.cu: into the owners' shared memory in a cluster, or to scratch memory for the merge kernel.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
template <typename T>
__device__ __forceinline__ T* cluster_peer(T* mine, int rank) { return cg::this_cluster().map_shared_rank(mine, rank); }

// Shared memory of the tensor-core decode kernel: the query tile (padded rows), 128 key and 128
// value rows, a row offset per key, four floats for a norm's sums, and, for a launch in clusters,
// what the splits send one another.  The key and value rows of head size 128, and of head size 64
// where the splits go through memory (the launches that fill every SM: less shared memory per CTA
// and 5 to 9 % more bytes per second at 8,192 and 32,768 keys), are swizzled; all others are padded
// by 16 bytes (the cluster launches of head size 64, few CTAs on short contexts, are 1.5 % of a
// decode step faster with plain addresses).
template <int HD, bool CLUSTER>
struct DecodeSmem {
  static constexpr bool SWZ = HD == 128 || (HD == 64 && !CLUSTER);
  static constexpr int STRIDE = SWZ ? HD : HD + 8;
  static constexpr size_t BYTES = (size_t)16 * (HD + 8) * 2 + (size_t)2 * DEC_THREADS * STRIDE * 2 + (size_t)DEC_THREADS * 8 + 16
                                + (CLUSTER ? (size_t)(8 * HD + 8) * 8 + 256 * 4 : 0);
};

// Head sizes up to 64 leave shared memory for five CTAs per SM, but the fused variant takes 128
// registers: four CTAs per SM.  TIGHT (fused, splits through memory) holds the registers to what five
// CTAs need; the launch takes it when it has more CTAs than four per SM (many requests, long
// contexts: a launch planned for five per SM ran in two waves), and the variant with all its
// registers otherwise (few CTAs: latency).
#ifndef DEC_TIGHT_CTAS
#define DEC_TIGHT_CTAS 5
#endif
template <int HD, bool CLUSTER, bool FUSED, bool TIGHT = false>
__global__ void __launch_bounds__(DEC_THREADS, TIGHT ? DEC_TIGHT_CTAS : (HD == 128 ? 3 : (HD == 64 && !CLUSTER ? (FUSED ? 4 : DEC_TIGHT_CTAS) : 0)))
attention_decode_mma_kernel(const DecodeParams p) {
  // Key and value rows in shared memory: rows of 128 or 256 bytes (head sizes 64 and 128) lie side
  // by side with their 16-byte pieces swizzled (piece c of row r at piece c ^ (r % 8): what ldmatrix
  // reads of eight rows then lies in different banks); other head sizes pad each row by 16 bytes.
  constexpr bool SWZ = DecodeSmem<HD, CLUSTER>::SWZ;
  constexpr int STRIDE = DecodeSmem<HD, CLUSTER>::STRIDE, QSTRIDE = HD + 8, CHUNKS = HD / 8;
  auto at = [](int row, int col) { return row * STRIDE + (SWZ ? ((((col >> 3) ^ (row & 7)) << 3) | (col & 7)) : col); };
  extern __shared__ __align__(1024) uint8_t dmm[];    // swizzled rows start on multiples of their length
  __nv_bfloat16* sQ = (__nv_bfloat16*)dmm;            // [16][QSTRIDE]
  __nv_bfloat16* sK = sQ + 16 * QSTRIDE;              // [128][STRIDE]
  __nv_bfloat16* sV = sK + DEC_THREADS * STRIDE;      // [128][STRIDE]
  // What the splits of a cluster send one another: a CTA owns every count-th pair of (head, dim)
  // places and receives that pair's partial sums from all splits, and every split's maxima and sums.
  long long* rows = (long long*)(sV + DEC_THREADS * STRIDE);   // [128]
  float* s_norm = (float*)(rows + DEC_THREADS);       // [4]: the warps' sums of squares (no static shared memory: it would pad the dynamic part's alignment)
  float2* recv = (float2*)(s_norm + 4);               // [pairs owned][splits], at most 8 * HD + 8 pairs (a cluster's launch only)
  float* recv_ml = (float*)(recv + 8 * HD + 8);       // [8 splits][16 rows][2]
  float* wO = (float*)sK;                             // [4][16][HD]  (the keys' space, once they are done with)
  float* wm = wO + 4 * 16 * HD;                       // [4][16]
  float* wl = wm + 64;                                // [4][16]
  float inv_rms = 1.0f;                                // FUSED with norm_x: what the sums are multiplied by

  pdl_launch_dependents();
  if constexpr (CLUSTER) cluster_arrive();             // "this CTA runs": awaited before anyone writes into its shared memory
  SPROUT_TL_ENTRY(0);
  ATTN_STAMP(0);
  // What this step's earlier kernels wrote is the query (or the float32 sums) and the newest
  // position's key and value.  The block table and the lengths were copied before the step's first
  // kernel, and the keys and values of earlier positions were written in earlier steps (a step
  // ends with a copy to the host or a graph's end, which nothing overtakes): the first pass's
  // loads go out before the wait for the earlier kernels, the rest is read after it.
  const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = p.heads / p.kv_heads;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  const int begin = split * p.split_keys;
  const int len = p.context_lens[r];
  const int first_page = table[min((begin + tid) / p.page_tokens, p.table_stride - 1)];
  const int width = (p.heads + 2 * p.kv_heads) * HD;
  const int pos = len - 1;                             // FUSED: the new token's position
  const float scale = 1.0f / sqrtf((float)HD);

  const int gr = lane >> 2, qc = lane & 3;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // The first pass's keys and values are requested before the request's length is known (its load
  // is still in flight); what it brought from beyond the length is cleared once the length is
  // there.  Later passes know the length.
  int end = begin + p.split_keys;
  int next_page = first_page;
  // FUSED, the split that holds the new token: that token's key pair and value element of this
  // thread, read with the q sums right after the wait (not when the pass's rows have landed: the
  // split with the new token is the one its cluster waits for)
  // (the variant held to five CTAs per SM reads them where it needs them: it has no registers to spare)
  constexpr bool EARLY_NEW = FUSED && !TIGHT;
  const bool holds_new = EARLY_NEW && pos >= begin && pos < begin + p.split_keys;
  float new_k0 = 0.f, new_k1 = 0.f, new_kb0 = 0.f, new_kb1 = 0.f, new_cos = 1.f, new_sin = 0.f, new_v = 0.f, new_vb = 0.f;
  for (int base = begin; base < end; base += DEC_THREADS) {
    const bool first = base == begin;
    const int key = base + tid;
    long long off = -1;
    if (first || key < end) {
      const int page = next_page;                      // read while the pass before was on its way
      if (page >= 0 && page < p.num_pages) off = (((long long)page * p.kv_heads + g) * p.page_tokens + key % p.page_tokens) * HD;
      else if (!first || key < len) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
    }
    if (FUSED && !first && key == pos) off = -2;       // the new token's row is written below, not loaded
    rows[tid] = off;
    __syncthreads();                                   // offsets and q visible; the staging buffers are free
    if constexpr (DEC_THREADS % CHUNKS == 0) {
      // a thread keeps its 16-byte column and walks down the rows: neighbours in a warp copy
      // neighbouring pieces of a row, and nothing but the row's offset changes between copies
      constexpr int ROWS_AT_ONCE = DEC_THREADS / CHUNKS;
      const int c8 = (tid % CHUNKS) * 8, r0 = tid / CHUNKS;      // the rows a thread walks share r0 % 8: one swizzled column
      const uint32_t dk0 = (uint32_t)__cvta_generic_to_shared(sK + at(r0, c8));
      const uint32_t dv0 = (uint32_t)__cvta_generic_to_shared(sV + at(r0, c8));
      const __nv_bfloat16* kg = p.k_cache + c8;
      const __nv_bfloat16* vg = p.v_cache + c8;
#pragma unroll
      for (int k = 0; k < CHUNKS; k++) {
        const long long ro = rows[r0 + k * ROWS_AT_ONCE];
        const uint32_t step = (uint32_t)(k * ROWS_AT_ONCE * STRIDE * 2);
        if (ro >= 0) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dk0 + step), "l"(kg + ro));
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dv0 + step), "l"(vg + ro));
        } else if (ro == -1) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dk0 + step), "r"(0) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dv0 + step), "r"(0) : "memory");
        }
      }
    } else {
      for (int idx = tid; idx < DEC_THREADS * CHUNKS; idx += DEC_THREADS) {
        const int row = idx / CHUNKS, c = idx % CHUNKS;
        const long long ro = rows[row];
        __nv_bfloat16* dk = sK + at(row, c * 8);
        __nv_bfloat16* dv = sV + at(row, c * 8);
        if (ro >= 0) { cp_async16(dk, p.k_cache + ro + c * 8); cp_async16(dv, p.v_cache + ro + c * 8); }
        else if (ro == -1) { *(uint4*)dk = make_uint4(0, 0, 0, 0); *(uint4*)dv = make_uint4(0, 0, 0, 0); }
      }
    }
    cp_async_commit();
    // the next pass's page while this pass's rows are on their way (the block table was there before the step)
    if (base + DEC_THREADS < begin + p.split_keys) next_page = table[min((key + DEC_THREADS) / p.page_tokens, p.table_stride - 1)];
    if (first) { ATTN_STAMP(1); pdl_wait(); SPROUT_TL_WAITED(0); ATTN_STAMP(2); }    // the first pass's keys and values are on their way
    if (FUSED && first && p.norm_x) {
      // the row's scale: every thread adds a share of the squares, the warps meet in shared memory
      const float* xr = p.norm_x + (size_t)r * p.norm_width;
      float ss = 0.f;
      for (int i = tid; i < p.norm_width; i += DEC_THREADS) { const float v = __ldcg(xr + i); ss += v * v; }
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
      if (lane == 0) s_norm[warp] = ss;
      __syncthreads();
      float total = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < DEC_THREADS / 32; w2++) total += s_norm[w2];
      inv_rms = 1.0f / sqrtf(total / (float)p.norm_width + p.norm_eps);
    }
    if (!FUSED && first) {
      for (int idx = tid; idx < 16 * CHUNKS; idx += DEC_THREADS) {
        const int row = idx / CHUNKS, c = idx % CHUNKS;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < group) v = *(const uint4*)(p.q + (size_t)r * p.q_stride + (size_t)(g * group + row) * HD + c * 8);
        *(uint4*)(sQ + row * QSTRIDE + c * 8) = v;
      }
    }
    if (FUSED && first && holds_new) {
      constexpr int HALF = HD / 2;
      const int rot_half = p.rotary_dim >> 1;
      const int safe = min(max(pos, 0), max(p.max_positions - 1, 0));
      const float* k_acc = p.acc + (size_t)r * width + (p.heads + g) * HD;
      const float* v_acc = p.acc + (size_t)r * width + (p.heads + p.kv_heads + g) * HD;
      if (tid < HALF) {
        const int d = tid;
        const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
        const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
        new_k0 = k_acc[e0]; new_k1 = k_acc[e1];
        if (p.bias) { new_kb0 = p.bias[(p.heads + g) * HD + e0]; new_kb1 = p.bias[(p.heads + g) * HD + e1]; }
        if (p.cos_table != nullptr && d < rot_half) { new_cos = p.cos_table[(size_t)safe * rot_half + d]; new_sin = p.sin_table[(size_t)safe * rot_half + d]; }
      }
      if (tid < HD) {
        new_v = v_acc[tid];
        if (p.bias) new_vb = p.bias[(p.heads + p.kv_heads + g) * HD + tid];
      }
    }
    if (FUSED && first) {
      // q of the group's heads: sums + bias, rotated by the position, to shared memory as bfloat16
      const bool rotate = p.cos_table != nullptr;
      if (pos < 0 || (rotate && pos >= p.max_positions)) { if (tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_POSITION); }
      const int safe = min(max(pos, 0), max(p.max_positions - 1, 0));
      constexpr int HALF = HD / 2;
      const int rot_half = p.rotary_dim >> 1;
      const float* sums = p.acc + (size_t)r * width + (size_t)g * group * HD;
      const float* bias = p.bias ? p.bias + (size_t)g * group * HD : nullptr;
      for (int idx = tid; idx < group * HALF; idx += DEC_THREADS) {
        const int row = idx / HALF, d = idx % HALF;
        // pair d of the head: a rotated pair below rotary_dim / 2, two elements that pass through beyond
        const bool turned = rotate && d < rot_half;
        const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
        const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
        const float a = sums[row * HD + e0] * inv_rms + (bias ? bias[row * HD + e0] : 0.f);
        const float b = sums[row * HD + e1] * inv_rms + (bias ? bias[row * HD + e1] : 0.f);
        const float c = turned ? p.cos_table[(size_t)safe * rot_half + d] : 1.f, sn = turned ? p.sin_table[(size_t)safe * rot_half + d] : 0.f;
        sQ[row * QSTRIDE + e0] = __float2bfloat16_rn(a * c - b * sn);
        sQ[row * QSTRIDE + e1] = __float2bfloat16_rn(b * c + a * sn);
      }
      for (int idx = group * CHUNKS + tid; idx < 16 * CHUNKS; idx += DEC_THREADS)      // the tile's unused rows
        *(uint4*)(sQ + (idx / CHUNKS) * QSTRIDE + (idx % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
    }
    if (first) {
      end = min(len, begin + p.split_keys);
      if (!CLUSTER && begin >= len) { cp_async_wait<0>(); return; }   // the merge kernel knows which splits exist
    }
    cp_async_wait<0>();
    if (first && end - base < DEC_THREADS) {
      // The early loads brought rows beyond the request's length from its pages as they lay there:
      // a page that another request used before may hold anything, and probability zero times a
      // stale non-finite value would still poison the sum.  Each thread clears the value pieces that
      // its own copies wrote (keys need nothing: their scores are replaced, not multiplied).
      const int live = max(end - base, 0);
      if constexpr (DEC_THREADS % CHUNKS == 0) {
        constexpr int ROWS_AT_ONCE = DEC_THREADS / CHUNKS;
        const int c8 = (tid % CHUNKS) * 8, r0 = tid / CHUNKS;
#pragma unroll
        for (int k = 0; k < CHUNKS; k++) {
          const int row = r0 + k * ROWS_AT_ONCE;
          if (row >= live) *(uint4*)(sV + at(row, c8)) = make_uint4(0, 0, 0, 0);
        }
      } else {
        for (int idx = tid; idx < DEC_THREADS * CHUNKS; idx += DEC_THREADS) {
          const int row = idx / CHUNKS, c = idx % CHUNKS;
          if (row >= live) *(uint4*)(sV + at(row, c * 8)) = make_uint4(0, 0, 0, 0);
        }
      }
    }
    if (!FUSED && first && pos >= base && pos < base + DEC_THREADS && pos < begin + p.split_keys) {
      // the newest position's key and value may have been written after the early loads read them
      __syncthreads();                                 // the early loads of that row have landed
      const long long ro = rows[pos - base];
      if (ro >= 0)
        for (int c = tid; c < CHUNKS; c += DEC_THREADS) {
          *(uint4*)(sK + at(pos - base, c * 8)) = *(const uint4*)(p.k_cache + ro + c * 8);
          *(uint4*)(sV + at(pos - base, c * 8)) = *(const uint4*)(p.v_cache + ro + c * 8);
        }
    }
    if (FUSED && pos >= base && pos < base + DEC_THREADS && pos < begin + p.split_keys) {
      // This split holds the new token: its key (rotated) and value come from the sums, go to the
      // cache and, over whatever the first pass's early load brought, into this pass's tile.
      __syncthreads();                                 // the early loads of that row have landed
      constexpr int HALF = HD / 2;
      const int page = table[pos / p.page_tokens];
      const bool page_ok = page >= 0 && page < p.num_pages;
      if (!page_ok && tid == 0) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
      const long long dst = page_ok ? (((long long)page * p.kv_heads + g) * p.page_tokens + pos % p.page_tokens) * HD : 0;
      float* k_acc = p.acc + (size_t)r * width + (p.heads + g) * HD;
      float* v_acc = p.acc + (size_t)r * width + (p.heads + p.kv_heads + g) * HD;
      const int row = pos - base;
      const int rot_half = p.rotary_dim >> 1;
      if (tid < HALF) {                                // the sums were read after the wait (above), or are now
        const int d = tid;
        const int e0 = d < rot_half ? (p.interleaved ? 2 * d : d) : p.rotary_dim + 2 * (d - rot_half);
        const int e1 = d < rot_half ? (p.interleaved ? 2 * d + 1 : d + rot_half) : e0 + 1;
        float k0 = new_k0, k1 = new_k1, kb0 = new_kb0, kb1 = new_kb1, cs = new_cos, sn = new_sin;
        if constexpr (!EARLY_NEW) {
          const int safe = min(max(pos, 0), max(p.max_positions - 1, 0));
          k0 = k_acc[e0]; k1 = k_acc[e1];
          kb0 = p.bias ? p.bias[(p.heads + g) * HD + e0] : 0.f; kb1 = p.bias ? p.bias[(p.heads + g) * HD + e1] : 0.f;
          const bool turned = p.cos_table != nullptr && d < rot_half;
          cs = turned ? p.cos_table[(size_t)safe * rot_half + d] : 1.f; sn = turned ? p.sin_table[(size_t)safe * rot_half + d] : 0.f;
        }
        const float a = k0 * inv_rms + kb0, b = k1 * inv_rms + kb1;
        k_acc[e0] = 0.f; k_acc[e1] = 0.f;
        const __nv_bfloat16 lo = __float2bfloat16_rn(a * cs - b * sn), hi = __float2bfloat16_rn(b * cs + a * sn);
        sK[at(row, e0)] = lo; sK[at(row, e1)] = hi;
        if (page_ok) { p.k_append[dst + e0] = lo; p.k_append[dst + e1] = hi; }
      }
      if (tid < HD) {
        float nv = new_v, nvb = new_vb;
        if constexpr (!EARLY_NEW) {
          nv = v_acc[tid];
          nvb = p.bias ? p.bias[(p.heads + p.kv_heads + g) * HD + tid] : 0.f;
        }
        const __nv_bfloat16 v = __float2bfloat16_rn(nv * inv_rms + nvb);
        v_acc[tid] = 0.f;
        sV[at(row, tid)] = v;
        if (page_ok) p.v_append[dst + tid] = v;
      }
    }
    __syncthreads();
    if (first) ATTN_STAMP(3);

    const int key0 = base + warp * 32;                 // this warp's 32 keys
    if (key0 < end) {
      // A lane's ldmatrix addresses: its row's start plus a 16-byte piece.  With swizzled rows (which
      // start on multiples of their length) the piece of step kk / d2 is an exclusive-or of the lane's
      // address with a constant, one instruction where it is used and no register held for it.
      const uint32_t wK_lane = (uint32_t)__cvta_generic_to_shared(sK + warp * 32 * STRIDE) +
                               (uint32_t)(((lane & 7) + (lane >> 4) * 8) * STRIDE * 2) +
                               (SWZ ? (uint32_t)(((((lane >> 3) & 1)) ^ (lane & 7)) << 4) : (uint32_t)(((lane >> 3) & 1) * 16));
      const uint32_t wV_lane = (uint32_t)__cvta_generic_to_shared(sV + warp * 32 * STRIDE) +
                               (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE * 2) +
                               (SWZ ? (uint32_t)(((lane >> 4) ^ (lane & 7)) << 4) : (uint32_t)((lane >> 4) * 16));
      float s[4][4];
#pragma unroll
      for (int i = 0; i < 4; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        uint32_t a[4];
        ldmatrix_x4(a, sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * QSTRIDE + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < 2; n2++) {
          uint32_t b[4];
          const uint32_t row_addr = wK_lane + (uint32_t)(n2 * 16 * STRIDE * 2);
          ldmatrix_x4_addr(b, SWZ ? row_addr ^ (uint32_t)(kk << 5) : row_addr + (uint32_t)(kk << 5));
          mma_bf16(s[2 * n2], a, b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
        }
      }
      float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int k = key0 + i * 8 + qc * 2;
        s[i][0] = k < end ? s[i][0] * scale : -INFINITY;
        s[i][1] = k + 1 < end ? s[i][1] * scale : -INFINITY;
        s[i][2] = k < end ? s[i][2] * scale : -INFINITY;
        s[i][3] = k + 1 < end ? s[i][3] * scale : -INFINITY;
        t0 = fmaxf(t0, fmaxf(s[i][0], s[i][1]));
        t1 = fmaxf(t1, fmaxf(s[i][2], s[i][3]));
      }
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1)); t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1)); t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);       // finite: key0 < end, so every row has a key
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
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < HD / 16; d2++) {
          uint32_t b[4];
          const uint32_t row_addr = wV_lane + (uint32_t)(kk * 16 * STRIDE * 2);
          ldmatrix_x4_trans_addr(b, SWZ ? row_addr ^ (uint32_t)(d2 << 5) : row_addr + (uint32_t)(d2 << 5));
          mma_bf16(o[2 * d2], a, b[0], b[1]);
          mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        }
      }
    }
  }

  // The warps' partial results -> shared memory (over the keys, which are no longer needed), in
  // the layout the MMA left them in: a lane holds the same (row, column) places in every warp.
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  ATTN_STAMP(4);
  __syncthreads();
  float4* frag = (float4*)wO;                          // [4 warps][HD / 8 column blocks][32 lanes]
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
  // merge the 4 warps: each warp takes every fourth block of 8 columns, a lane its two rows
  {
    float wa[4], wb[4];                                // the warps' weights for rows gr and gr + 8
    float ma = -INFINITY, mb = -INFINITY, la = 0.f, lb = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) { wa[w] = wm[w * 16 + gr]; wb[w] = wm[w * 16 + gr + 8]; ma = fmaxf(ma, wa[w]); mb = fmaxf(mb, wb[w]); }
#pragma unroll
    for (int w = 0; w < 4; w++) {
      wa[w] = wa[w] == -INFINITY ? 0.f : __expf(wa[w] - ma);
      wb[w] = wb[w] == -INFINITY ? 0.f : __expf(wb[w] - mb);
    }
    la = (wl[gr] * wa[0] + wl[16 + gr] * wa[1]) + (wl[32 + gr] * wa[2] + wl[48 + gr] * wa[3]);
    lb = (wl[gr + 8] * wb[0] + wl[24 + gr] * wb[1]) + (wl[40 + gr] * wb[2] + wl[56 + gr] * wb[3]);
    const bool row_a = gr < group, row_b = gr + 8 < group;
    if constexpr (CLUSTER) cluster_wait();             // every CTA of the cluster runs: their shared memory may be written
    auto emit = [&](int row, int d, float x, float y, float l) {
      const int head = g * group + row;
      if constexpr (CLUSTER) {
        const int pair = (row * HD + d) >> 1;          // to the pair's owner, into this split's place
        *(cluster_peer(recv, pair % p.splits) + (pair / p.splits) * p.splits + split) = make_float2(x, y);
      } else if (p.splits == 1) {
        *(__nv_bfloat162*)(p.out + (size_t)r * p.out_stride + (size_t)head * HD + d) = __floats2bfloat162_rn(x / l, y / l);
        if (FUSED) *(float2*)(p.acc + (size_t)r * width + (size_t)head * HD + d) = make_float2(0.f, 0.f);   // the only reader of these q sums
      } else {
        const size_t slot = ((size_t)r * p.heads + head) * p.splits + split;
        *(float2*)(p.part_out + slot * HD + d) = make_float2(x, y);
      }
    };
    for (int i = warp; i < HD / 8; i += 4) {
      const float4 f0 = frag[(0 * (HD / 8) + i) * 32 + lane], f1 = frag[(1 * (HD / 8) + i) * 32 + lane];
      const float4 f2 = frag[(2 * (HD / 8) + i) * 32 + lane], f3 = frag[(3 * (HD / 8) + i) * 32 + lane];
      const int d = i * 8 + qc * 2;
      if (row_a) emit(gr, d, (f0.x * wa[0] + f1.x * wa[1]) + (f2.x * wa[2] + f3.x * wa[3]),
                      (f0.y * wa[0] + f1.y * wa[1]) + (f2.y * wa[2] + f3.y * wa[3]), la);
      if (row_b) emit(gr + 8, d, (f0.z * wb[0] + f1.z * wb[1]) + (f2.z * wb[2] + f3.z * wb[3]),
                      (f0.w * wb[0] + f1.w * wb[1]) + (f2.w * wb[2] + f3.w * wb[3]), lb);
    }
    if constexpr (CLUSTER) {                           // each row's maximum and sum to every split: warp w tells splits w and w + 4
      if (qc == 0)
        for (int to = warp; to < p.splits; to += 4) {
          float* theirs = cluster_peer(recv_ml, to) + split * 32;
          if (row_a) *(float2*)(theirs + 2 * gr) = make_float2(ma, la);
          if (row_b) *(float2*)(theirs + 2 * (gr + 8)) = make_float2(mb, lb);
        }
    }
    if (warp == 0 && qc == 0) {                        // each row's maximum and sum, once
      if constexpr (CLUSTER) {
      } else if (p.splits > 1) {
        if (row_a) { const size_t slot = ((size_t)r * p.heads + g * group + gr) * p.splits + split; p.part_ml[slot * 2] = ma; p.part_ml[slot * 2 + 1] = la; }
        if (row_b) { const size_t slot = ((size_t)r * p.heads + g * group + gr + 8) * p.splits + split; p.part_ml[slot * 2] = mb; p.part_ml[slot * 2 + 1] = lb; }
      }
    }
  }
  ATTN_STAMP(5);
  if constexpr (CLUSTER) {
    // Everything this CTA owns has arrived once every split has passed this barrier; a CTA reads
    // only its own shared memory afterwards, so it may leave without waiting for the others.
    cluster_arrive();
    cluster_wait();
    ATTN_STAMP(6);
    if (FUSED && split == 0) {                         // every split has read the q sums: clear them
      for (int i = tid; i < group * HD; i += DEC_THREADS) p.acc[(size_t)r * width + g * group * HD + i] = 0.f;
    }
    const int count = p.splits, pairs = group * HD / 2;
    for (int local = tid; local * count + split < pairs; local += DEC_THREADS) {
      const int i = 2 * (local * count + split), h = i / HD;
      float ms[8], ls[8];
      float2 os[8];
#pragma unroll
      for (int sp = 0; sp < 8; sp++) {
        if (sp < count) { ms[sp] = recv_ml[sp * 32 + 2 * h]; ls[sp] = recv_ml[sp * 32 + 2 * h + 1]; os[sp] = recv[local * count + sp]; }
        else { ms[sp] = -INFINITY; ls[sp] = 0.f; os[sp] = make_float2(0.f, 0.f); }
      }
      float m = ms[0];
#pragma unroll
      for (int sp = 1; sp < 8; sp++) m = fmaxf(m, ms[sp]);
      float l = 0.f, ax = 0.f, ay = 0.f;
#pragma unroll
      for (int sp = 0; sp < 8; sp++) {
        const float w = ms[sp] == -INFINITY ? 0.f : __expf(ms[sp] - m);
        l += ls[sp] * w;
        ax += os[sp].x * w;
        ay += os[sp].y * w;
      }
      *(__nv_bfloat162*)(p.out + (size_t)r * p.out_stride + (size_t)(g * group + h) * HD + (i % HD)) = __floats2bfloat162_rn(ax / l, ay / l);
    }
    ATTN_STAMP(7);
  }
  ATTN_STAMP(8);
  SPROUT_TL_EXIT(0);
}

template <int HD, bool FUSED>
int launch_decode_mma(const DecodeParams& p, bool cluster, int requests, cudaStream_t stream) {
  const size_t smem = cluster ? DecodeSmem<HD, true>::BYTES : DecodeSmem<HD, false>::BYTES;
  static bool configured[2] = {false, false};
  if (!configured[cluster]) {
    cudaError_t err = cudaSuccess;
    if (smem > 48 * 1024)
      err = cluster
          ? cudaFuncSetAttribute(attention_decode_mma_kernel<HD, true, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
          : cudaFuncSetAttribute(attention_decode_mma_kernel<HD, false, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return sprout_fail("attention_decode: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(err));
    // The kernels of a decode layer share SMs (each starts while its predecessor runs and brings
    // its weights in meanwhile); an SM holds CTAs of kernels with different splits between L1 and
    // shared memory only one after the other, so all of them ask for the largest shared memory.
    if (cluster) cudaFuncSetAttribute(attention_decode_mma_kernel<HD, true, FUSED>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    else cudaFuncSetAttribute(attention_decode_mma_kernel<HD, false, FUSED>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    configured[cluster] = true;
  }
  const dim3 grid(p.splits, p.kv_heads, requests);
  if (cluster) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = dim3(DEC_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = p.splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = sprout_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&config, attention_decode_mma_kernel<HD, true, FUSED>, p);
    return sprout_check_launch("attention_decode (tensor cores, cluster)");
  }
  if constexpr (FUSED && HD <= 64) {
    if ((long long)p.splits * p.kv_heads * requests > 4LL * sprout_sm_count()) {
      static bool tight_configured = false;
      if (!tight_configured) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attention_decode_mma_kernel<HD, false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaFuncSetAttribute(attention_decode_mma_kernel<HD, false, true, true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        tight_configured = true;
      }
      sprout_launch(attention_decode_mma_kernel<HD, false, true, true>, grid, dim3(DEC_THREADS), smem, stream, p);
      return sprout_check_launch("attention_decode (tensor cores, five CTAs per SM)");
    }
  }
  sprout_launch(attention_decode_mma_kernel<HD, false, FUSED>, grid, dim3(DEC_THREADS), smem, stream, p);
  return sprout_check_launch("attention_decode (tensor cores)");
}

// How many CTAs of the split-key decode kernel an SM holds at once (registers and shared memory), for
// the plan of a launch: of the fused kernel as a launch with many CTAs runs it, through memory or
// (cluster) in clusters, whose CTAs also hold what the splits send one another.
template <int HD, bool CLUSTER, bool FUSED, bool TIGHT>
int decode_mma_occupancy() {
  const size_t smem = DecodeSmem<HD, CLUSTER>::BYTES;
  int count = 0;
  if (smem > 48 * 1024) cudaFuncSetAttribute(attention_decode_mma_kernel<HD, CLUSTER, FUSED, TIGHT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaFuncSetAttribute(attention_decode_mma_kernel<HD, CLUSTER, FUSED, TIGHT>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&count, attention_decode_mma_kernel<HD, CLUSTER, FUSED, TIGHT>, DEC_THREADS, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return count;
}
template <int HD>
int decode_mma_ctas_per_sm(bool fused, bool cluster) {
  if (cluster) return fused ? decode_mma_occupancy<HD, true, true, false>() : decode_mma_occupancy<HD, true, false, false>();
  if (fused) return decode_mma_occupancy<HD, false, true, (HD <= 64)>();
  return decode_mma_occupancy<HD, false, false, false>();
}

}  // namespace

}  // namespace sprout_attn
