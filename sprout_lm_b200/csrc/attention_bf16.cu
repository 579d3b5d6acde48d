// bfloat16 paged attention for serving: scores, softmax and sums in float32.
//
// decode  (every request brings one query token): grid (splits, kv_heads, requests).  A CTA
//   takes a run of `split_keys` keys of one key/value head of one request and serves all the
//   query heads of that group from one read of the keys and values.  Partial results
//   (running maximum, sum, unnormalised output) are merged in one of two ways: with up to 8
//   splits the CTAs of a (request, key/value head) form a thread-block cluster and each of
//   them merges a share of the output from all partial results through distributed shared memory; with more
//   splits they go to scratch memory and a second kernel merges them.  The work of a query
//   does not depend on the batch around it.  The tensor-core kernel for head sizes up to 128 is
//   in attention_decode_mma.cuh (two compilation units); here are the CUDA-core kernel for larger
//   heads, the merge kernel and the entry points.
//
// prefill (portions of prompts, possibly beside single tokens): tensor-core flash attention
//   (mma.sync m16n8k16, float32 accumulation) over the pages.  The rows of a tile are (token,
//   query head of one group) pairs, so a short portion still fills the 16-row MMA tiles and
//   keys/values are read once per group; keys are walked in tiles of 64 with the causal limit
//   of each row applied inside the tile.
#include "attention_bf16.cuh"

namespace cg = cooperative_groups;

using namespace sprout_attn;

namespace {

__device__ __forceinline__ void dec_cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}

// Shared memory: q of the group as float32, the pass's probabilities, reduction slots, the
// pass's key rows' offsets, and the pass's keys and values themselves (copied with cp.async so
// that all of a pass's loads are in flight at once; rows padded by 16 bytes against bank
// conflicts).
template <bool CLUSTER>
__global__ void __launch_bounds__(DEC_THREADS)
attention_decode_kernel(const DecodeParams p) {
  extern __shared__ __align__(16) float dsm[];
  const int group = p.heads / p.kv_heads;
  const int stride = p.head_dim + 8;                // bf16 elements per staged row
  const int chunks = p.head_dim / 8;                // 16-byte chunks per row
  float* qs = dsm;                                  // [group][head_dim]
  float* probs = qs + group * p.head_dim;           // [group][DEC_THREADS]
  float* red = probs + group * DEC_THREADS;         // [MAX_GROUP][8]: 4 warp maxima, 4 warp sums
  long long* rows = (long long*)(red + MAX_GROUP * 8);            // [DEC_THREADS]
  __nv_bfloat16* sK = (__nv_bfloat16*)(rows + DEC_THREADS);       // [DEC_THREADS][stride]
  __nv_bfloat16* sV = sK + DEC_THREADS * stride;
  float* part_acc = (float*)(sV + DEC_THREADS * stride);          // [group][head_dim] this CTA's partial output (cluster merge)
  float* part_ml = part_acc + group * p.head_dim;                  // [group][2] its running maximum and sum

  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, g = blockIdx.y, r = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // independent loads first: the length, this thread's first page, the queries
  const int* table = p.block_table + (size_t)r * p.table_stride;
  const int begin = split * p.split_keys;
  const int len = p.context_lens[r];
  const int first_page = table[min((begin + tid) / p.page_tokens, p.table_stride - 1)];
  for (int i = tid; i < group * p.head_dim / 2; i += DEC_THREADS) {
    const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)(p.q + (size_t)r * p.q_stride + (size_t)g * group * p.head_dim + 2 * i));
    qs[2 * i] = f.x; qs[2 * i + 1] = f.y;
  }
  if (!CLUSTER && begin >= len) return;              // the merge kernel knows which splits exist
  const int end = min(len, begin + p.split_keys);
  const float scale = 1.0f / sqrtf((float)p.head_dim);

  // warp w accumulates output dims {2*lane, 2*lane+1} (+64 per chunk of 64 dims) of the heads
  // h = w, w + 4, ...
  float m_run[MAX_GROUP / 4], l_run[MAX_GROUP / 4];
  float acc[MAX_GROUP / 4][4][2];
#pragma unroll
  for (int a = 0; a < MAX_GROUP / 4; a++) {
    m_run[a] = -INFINITY; l_run[a] = 0.f;
#pragma unroll
    for (int c = 0; c < 4; c++) acc[a][c][0] = acc[a][c][1] = 0.f;
  }

  for (int base = begin; base < end; base += DEC_THREADS) {
    const int key = base + tid;
    bool valid = key < end;
    long long off = -1;
    if (valid) {
      const int page = base == begin ? first_page : table[key / p.page_tokens];
      if (page < 0 || page >= p.num_pages) { atomicOr(p.status, SPROUT_STATUS_BAD_PAGE); valid = false; }
      else off = (((long long)page * p.kv_heads + g) * p.page_tokens + key % p.page_tokens) * p.head_dim;
    }
    rows[tid] = off;
    __syncthreads();                                  // offsets (and, first time, q) visible; staging buffers free
    for (int idx = tid; idx < DEC_THREADS * chunks; idx += DEC_THREADS) {
      const int row = idx / chunks, c = idx % chunks;
      const long long ro = rows[row];
      __nv_bfloat16* dk = sK + row * stride + c * 8;
      __nv_bfloat16* dv = sV + row * stride + c * 8;
      if (ro >= 0) { dec_cp_async16(dk, p.k_cache + ro + c * 8); dec_cp_async16(dv, p.v_cache + ro + c * 8); }
      else { *(uint4*)dk = make_uint4(0, 0, 0, 0); *(uint4*)dv = make_uint4(0, 0, 0, 0); }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // scores of this thread's key against every head of the group
    float s[MAX_GROUP];
#pragma unroll
    for (int h = 0; h < MAX_GROUP; h++) s[h] = 0.f;
    {
      const uint4* kp = (const uint4*)(sK + tid * stride);
      for (int c = 0; c < chunks; c++) {
        const uint4 raw = kp[c];
        const __nv_bfloat162* k2 = (const __nv_bfloat162*)&raw;
        float kf[8];
#pragma unroll
        for (int j = 0; j < 4; j++) { const float2 f = __bfloat1622float2(k2[j]); kf[2 * j] = f.x; kf[2 * j + 1] = f.y; }
#pragma unroll
        for (int h = 0; h < MAX_GROUP; h++) {
          if (h < group) {
            const float4* qh = (const float4*)(qs + h * p.head_dim + c * 8);
            const float4 qa = qh[0], qb = qh[1];
            s[h] = fmaf(qa.x, kf[0], s[h]); s[h] = fmaf(qa.y, kf[1], s[h]);
            s[h] = fmaf(qa.z, kf[2], s[h]); s[h] = fmaf(qa.w, kf[3], s[h]);
            s[h] = fmaf(qb.x, kf[4], s[h]); s[h] = fmaf(qb.y, kf[5], s[h]);
            s[h] = fmaf(qb.z, kf[6], s[h]); s[h] = fmaf(qb.w, kf[7], s[h]);
          }
        }
      }
    }
    // per head: block maximum of the scores, exponentials into shared memory, block sum
#pragma unroll
    for (int h = 0; h < MAX_GROUP; h++) {
      if (h < group) {
        s[h] = valid ? s[h] * scale : -INFINITY;
        const float wm = warp_max(s[h]);
        if (lane == 0) red[h * 8 + warp] = wm;
      }
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < MAX_GROUP; h++) {
      if (h < group) {
        const float cm = fmaxf(fmaxf(red[h * 8], red[h * 8 + 1]), fmaxf(red[h * 8 + 2], red[h * 8 + 3]));
        const float e = valid ? __expf(s[h] - cm) : 0.f;     // cm is finite: the pass has at least one valid key
        probs[h * DEC_THREADS + tid] = e;
        const float ws = warp_sum(e);
        if (lane == 0) red[h * 8 + 4 + warp] = ws;
      }
    }
    __syncthreads();
    // output accumulation from the staged values: warp w handles heads w, w+4, ...; lanes run over the dims
    const int count = min(DEC_THREADS, end - base);
#pragma unroll
    for (int a = 0; a < MAX_GROUP / 4; a++) {
      const int h = warp + 4 * a;
      if (h < group) {
        const float cm = fmaxf(fmaxf(red[h * 8], red[h * 8 + 1]), fmaxf(red[h * 8 + 2], red[h * 8 + 3]));
        const float cs = (red[h * 8 + 4] + red[h * 8 + 5]) + (red[h * 8 + 6] + red[h * 8 + 7]);
        const float m_new = fmaxf(m_run[a], cm);
        const float alpha = m_run[a] == -INFINITY ? 0.f : __expf(m_run[a] - m_new);
        const float beta = __expf(cm - m_new);
        l_run[a] = l_run[a] * alpha + cs * beta;
        const float* ph = probs + h * DEC_THREADS;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int d = c * 64 + 2 * lane;
          if (d < p.head_dim) {
            float a0 = 0.f, a1 = 0.f;
            const __nv_bfloat16* vd = sV + d;
#pragma unroll 4
            for (int j = 0; j < count; j++) {
              const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(vd + j * stride));
              a0 = fmaf(ph[j], v.x, a0);
              a1 = fmaf(ph[j], v.y, a1);
            }
            acc[a][c][0] = acc[a][c][0] * alpha + a0 * beta;
            acc[a][c][1] = acc[a][c][1] * alpha + a1 * beta;
          }
        }
        m_run[a] = m_new;
      }
    }
  }

  if constexpr (CLUSTER) {
    // every split leaves its partial results in its own shared memory; the cluster's first CTA
    // reads them all through distributed shared memory and writes the rows out
    cg::cluster_group cluster = cg::this_cluster();
#pragma unroll
    for (int a = 0; a < MAX_GROUP / 4; a++) {
      const int h = warp + 4 * a;
      if (h < group) {
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int d = c * 64 + 2 * lane;
          if (d < p.head_dim) { part_acc[h * p.head_dim + d] = acc[a][c][0]; part_acc[h * p.head_dim + d + 1] = acc[a][c][1]; }
        }
        if (lane == 0) { part_ml[2 * h] = m_run[a]; part_ml[2 * h + 1] = l_run[a]; }
      }
    }
    cluster.sync();
    if (cluster.block_rank() == 0) {
      const int count = (int)cluster.num_blocks();
      for (int i = tid; i < group * p.head_dim; i += DEC_THREADS) {
        const int h = i / p.head_dim;
        float ms[8], ls[8], os[8];
#pragma unroll
        for (int sp = 0; sp < 8; sp++) {
          if (sp < count) {
            const float* their_ml = cluster.map_shared_rank(part_ml, sp);
            const float* their_acc = cluster.map_shared_rank(part_acc, sp);
            ms[sp] = their_ml[2 * h]; ls[sp] = their_ml[2 * h + 1]; os[sp] = their_acc[i];
          } else { ms[sp] = -INFINITY; ls[sp] = 0.f; os[sp] = 0.f; }
        }
        float m = ms[0];
#pragma unroll
        for (int sp = 1; sp < 8; sp++) m = fmaxf(m, ms[sp]);
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int sp = 0; sp < 8; sp++) {
          const float w = ms[sp] == -INFINITY ? 0.f : __expf(ms[sp] - m);
          l += ls[sp] * w;
          o += os[sp] * w;
        }
        p.out[(size_t)r * p.out_stride + (size_t)(g * group + h) * p.head_dim + (i % p.head_dim)] = __float2bfloat16_rn(o / l);
      }
    }
    cluster.sync();                                  // nobody leaves while its shared memory is being read
  } else {
#pragma unroll
  for (int a = 0; a < MAX_GROUP / 4; a++) {
    const int h = warp + 4 * a;
    if (h < group) {
      const int head = g * group + h;
      if (p.splits == 1) {
        __nv_bfloat16* o = p.out + (size_t)r * p.out_stride + (size_t)head * p.head_dim;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int d = c * 64 + 2 * lane;
          if (d < p.head_dim)
            *(__nv_bfloat162*)(o + d) = __floats2bfloat162_rn(acc[a][c][0] / l_run[a], acc[a][c][1] / l_run[a]);
        }
      } else {
        const size_t slot = ((size_t)r * p.heads + head) * p.splits + split;
        float* o = p.part_out + slot * p.head_dim;
#pragma unroll
        for (int c = 0; c < 4; c++) {
          const int d = c * 64 + 2 * lane;
          if (d < p.head_dim) { o[d] = acc[a][c][0]; o[d + 1] = acc[a][c][1]; }
        }
        if (lane == 0) { p.part_ml[slot * 2] = m_run[a]; p.part_ml[slot * 2 + 1] = l_run[a]; }
      }
    }
  }
  }
}

// Merge the splits of one (request, head): grid (heads, requests), head_dim threads (rounded up to a warp).
__global__ void attention_decode_merge_kernel(const DecodeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
  const int len = p.context_lens[r];
  const int live = min(p.splits, (len + p.split_keys - 1) / p.split_keys);
  const size_t slot0 = ((size_t)r * p.heads + head) * p.splits;
  float m = -INFINITY, l = 0.f, o = 0.f;
  for (int s0 = 0; s0 < live; s0 += 8) {             // eight splits' values in flight at a time
    float ms[8], ls[8], os[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const bool on = s0 + j < live;
      ms[j] = on ? p.part_ml[(slot0 + s0 + j) * 2] : -INFINITY;
      ls[j] = on ? p.part_ml[(slot0 + s0 + j) * 2 + 1] : 0.f;
      os[j] = (on && d < p.head_dim) ? p.part_out[(slot0 + s0 + j) * p.head_dim + d] : 0.f;
    }
    float m_new = m;
#pragma unroll
    for (int j = 0; j < 8; j++) m_new = fmaxf(m_new, ms[j]);
    const float keep = m == -INFINITY ? 0.f : __expf(m - m_new);
    l *= keep; o *= keep;
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float w = ms[j] == -INFINITY ? 0.f : __expf(ms[j] - m_new);
      l += ls[j] * w;
      o += os[j] * w;
    }
    m = m_new;
  }
  if (d < p.head_dim) {
    p.out[(size_t)r * p.out_stride + (size_t)head * p.head_dim + d] = __float2bfloat16_rn(o / l);
    // the fused kernel's splits have all read the q sums by now: clear them for the next product
    if (p.acc) p.acc[(size_t)r * (p.heads + 2 * p.kv_heads) * p.head_dim + (size_t)head * p.head_dim + d] = 0.f;
  }
}

// =============================================================================== prefill
constexpr int PF_THREADS = 128, PF_ROWS = 64, PF_KEYS = 64;

struct PrefillParams {
  const __nv_bfloat16* q; int q_stride;
  const __nv_bfloat16* k_cache; const __nv_bfloat16* v_cache;
  const int* block_table; int table_stride;
  const int* q_start;                 // [requests + 1] first token of each request in the batch
  const int* positions;               // [tokens]
  __nv_bfloat16* out; int out_stride;
  int requests, heads, kv_heads, page_tokens, num_pages;
  float scale;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const PrefillParams p) {
  constexpr int STRIDE = HD + 8;                      // bf16 elements per shared-memory row (16 bytes of padding)
  constexpr int CHUNKS = HD / 8;                      // 16-byte chunks per row
  extern __shared__ __align__(16) uint8_t psm[];
  __nv_bfloat16* sQ = (__nv_bfloat16*)psm;            // [64][STRIDE]
  __nv_bfloat16* sK = sQ + PF_ROWS * STRIDE;          // [2][64][STRIDE]
  __nv_bfloat16* sV = sK + 2 * PF_KEYS * STRIDE;      // [2][64][STRIDE]
  __shared__ int s_limit[PF_ROWS];                    // last visible key of each row, -1 for no row
  __shared__ int s_token[PF_ROWS];                    // batch index of the row's token
  __shared__ int s_head[PF_ROWS];
  __shared__ long long s_off[2][PF_KEYS];             // cache offsets of a tile's keys, -1 beyond the range

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.y;
  const int group = p.heads / p.kv_heads;

  // which request and which 64-row tile of it this CTA owns
  int r = 0, tile = blockIdx.x;
  for (; r < p.requests; r++) {
    const int tiles = ((p.q_start[r + 1] - p.q_start[r]) * group + PF_ROWS - 1) / PF_ROWS;
    if (tile < tiles) {
      // causal work grows with the tile index; CTAs are handed to SMs in launch order, so deal the
      // tiles out alternately from both ends: every SM gets a mix of short and long ones
      tile = (tile & 1) ? tiles - 1 - (tile >> 1) : (tile >> 1);
      break;
    }
    tile -= tiles;
  }
  if (r >= p.requests) return;
  const int q0 = p.q_start[r], q_count = p.q_start[r + 1] - q0;
  const int rows_total = q_count * group;
  const int row_base = tile * PF_ROWS;
  const int* table = p.block_table + (size_t)r * p.table_stride;

  if (tid < PF_ROWS) {
    const int gi = row_base + tid;
    if (gi < rows_total) {
      const int tok = q0 + gi / group;
      s_token[tid] = tok;
      s_head[tid] = g * group + gi % group;
      s_limit[tid] = p.positions[tok];
    } else {
      s_token[tid] = -1; s_head[tid] = 0; s_limit[tid] = -1;
    }
  }
  __syncthreads();
  const int last_row = min(rows_total, row_base + PF_ROWS) - 1 - row_base;
  const int max_limit = s_limit[last_row];            // positions grow with the row index
  const int kv_tiles = max_limit / PF_KEYS + 1;

  // Q rows -> shared memory
  for (int idx = tid; idx < PF_ROWS * CHUNKS; idx += PF_THREADS) {
    const int row = idx / CHUNKS, c = idx % CHUNKS;
    __nv_bfloat16* dst = sQ + row * STRIDE + c * 8;
    if (s_token[row] >= 0) cp_async16(dst, p.q + (size_t)s_token[row] * p.q_stride + (size_t)s_head[row] * HD + c * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  }

  auto find_rows = [&](int t, int buf) {
    if (tid < PF_KEYS) {
      const int key = t * PF_KEYS + tid;
      long long off = -1;
      if (key <= max_limit) {
        const int page = table[key / p.page_tokens];
        if (page < 0 || page >= p.num_pages) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
        else off = (((long long)page * p.kv_heads + g) * p.page_tokens + key % p.page_tokens) * HD;
      }
      s_off[buf][tid] = off;
    }
  };
  auto load_tile = [&](int buf) {
    for (int idx = tid; idx < PF_KEYS * CHUNKS; idx += PF_THREADS) {
      const int row = idx / CHUNKS, c = idx % CHUNKS;
      const long long off = s_off[buf][row];
      __nv_bfloat16* dk = sK + (buf * PF_KEYS + row) * STRIDE + c * 8;
      __nv_bfloat16* dv = sV + (buf * PF_KEYS + row) * STRIDE + c * 8;
      if (off >= 0) { cp_async16(dk, p.k_cache + off + c * 8); cp_async16(dv, p.v_cache + off + c * 8); }
      else { *(uint4*)dk = make_uint4(0, 0, 0, 0); *(uint4*)dv = make_uint4(0, 0, 0, 0); }
    }
  };

  find_rows(0, 0);
  __syncthreads();
  load_tile(0);
  cp_async_commit();

  const int gr = lane >> 2, qc = lane & 3;            // row within 8, column pair within the quad
  const int my_row0 = warp * 16 + gr, my_row1 = my_row0 + 8;
  const int limit0 = s_limit[my_row0], limit1 = s_limit[my_row1];
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // exp(s * scale - m * scale) as exp2 with the scale folded in: one multiply-add per score
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const int warp_min_limit = s_limit[min(warp * 16, last_row)];   // the smallest limit among this warp's rows
  constexpr bool Q_IN_REGISTERS = HD <= 64;
  uint32_t qf[Q_IN_REGISTERS ? HD / 16 : 1][4];

  for (int t = 0; t < kv_tiles; t++) {
    const int buf = t & 1;
    if (t + 1 < kv_tiles) find_rows(t + 1, buf ^ 1);
    __syncthreads();                                   // offsets visible; everyone is done with buffer buf^1
    if (t + 1 < kv_tiles) load_tile(buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();                                // tile t (and Q) have landed
    __syncthreads();
    if (Q_IN_REGISTERS && t == 0) {
#pragma unroll
      for (int kk = 0; kk < (Q_IN_REGISTERS ? HD / 16 : 1); kk++)
        ldmatrix_x4(qf[kk], sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + kk * 16 + (lane >> 4) * 8);
    }

    const __nv_bfloat16* tK = sK + buf * PF_KEYS * STRIDE;
    const __nv_bfloat16* tV = sV + buf * PF_KEYS * STRIDE;
    const int kv0 = t * PF_KEYS;
    // skip a tile that no row of this warp can see
    const int warp_limit = s_limit[min(warp * 16 + 15, last_row)];
    if (warp * 16 <= last_row && kv0 <= warp_limit) {
      float s[PF_KEYS / 8][4];
#pragma unroll
      for (int i = 0; i < PF_KEYS / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        uint32_t a_local[4];
        if (!Q_IN_REGISTERS)
          ldmatrix_x4(a_local, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + kk * 16 + (lane >> 4) * 8);
        const uint32_t (&a)[4] = Q_IN_REGISTERS ? qf[Q_IN_REGISTERS ? kk : 0] : a_local;
#pragma unroll
        for (int n2 = 0; n2 < PF_KEYS / 16; n2++) {
          uint32_t b[4];
          ldmatrix_x4(b, tK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * STRIDE + kk * 16 + ((lane >> 3) & 1) * 8);
          mma_bf16(s[2 * n2], a, b[0], b[1]);
          mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
        }
      }
      // causal mask (only on tiles that reach past some row's limit), running maximum; scores stay
      // unscaled, the scale is applied inside the exponential
      float t_max0 = -INFINITY, t_max1 = -INFINITY;
      if (kv0 + PF_KEYS - 1 > warp_min_limit) {
#pragma unroll
        for (int i = 0; i < PF_KEYS / 8; i++) {
          const int key = kv0 + i * 8 + qc * 2;
          if (key > limit0) s[i][0] = -INFINITY;
          if (key + 1 > limit0) s[i][1] = -INFINITY;
          if (key > limit1) s[i][2] = -INFINITY;
          if (key + 1 > limit1) s[i][3] = -INFINITY;
        }
      }
#pragma unroll
      for (int i = 0; i < PF_KEYS / 8; i++) {
        t_max0 = fmaxf(t_max0, fmaxf(s[i][0], s[i][1]));
        t_max1 = fmaxf(t_max1, fmaxf(s[i][2], s[i][3]));
      }
      t_max0 = fmaxf(t_max0, __shfl_xor_sync(0xffffffffu, t_max0, 1));
      t_max0 = fmaxf(t_max0, __shfl_xor_sync(0xffffffffu, t_max0, 2));
      t_max1 = fmaxf(t_max1, __shfl_xor_sync(0xffffffffu, t_max1, 1));
      t_max1 = fmaxf(t_max1, __shfl_xor_sync(0xffffffffu, t_max1, 2));
      const float n0 = fmaxf(m0, t_max0), n1 = fmaxf(m1, t_max1);     // running maxima of the unscaled scores
      const float base0 = n0 == -INFINITY ? 0.f : n0 * scale_log2, base1 = n1 == -INFINITY ? 0.f : n1 * scale_log2;
      const float alpha0 = m0 == -INFINITY ? 0.f : exp2f(m0 * scale_log2 - base0);
      const float alpha1 = m1 == -INFINITY ? 0.f : exp2f(m1 * scale_log2 - base1);
      m0 = n0; m1 = n1;
      l0 *= alpha0; l1 *= alpha1;
#pragma unroll
      for (int i = 0; i < HD / 8; i++) { o[i][0] *= alpha0; o[i][1] *= alpha0; o[i][2] *= alpha1; o[i][3] *= alpha1; }
#pragma unroll
      for (int i = 0; i < PF_KEYS / 8; i++) {
        s[i][0] = exp2f(fmaf(s[i][0], scale_log2, -base0)); s[i][1] = exp2f(fmaf(s[i][1], scale_log2, -base0));
        s[i][2] = exp2f(fmaf(s[i][2], scale_log2, -base1)); s[i][3] = exp2f(fmaf(s[i][3], scale_log2, -base1));
        l0 += s[i][0] + s[i][1];
        l1 += s[i][2] + s[i][3];
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < PF_KEYS / 16; kk++) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d2 = 0; d2 < HD / 16; d2++) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, tV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * STRIDE + d2 * 16 + (lane >> 4) * 8);
          mma_bf16(o[2 * d2], a, b[0], b[1]);
          mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();

  // sums across the quad, then the rows go out
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (s_token[my_row0] >= 0) {
    __nv_bfloat16* dst = p.out + (size_t)s_token[my_row0] * p.out_stride + (size_t)s_head[my_row0] * HD + qc * 2;
    const float inv = 1.0f / l0;
#pragma unroll
    for (int i = 0; i < HD / 8; i++) *(__nv_bfloat162*)(dst + i * 8) = __floats2bfloat162_rn(o[i][0] * inv, o[i][1] * inv);
  }
  if (s_token[my_row1] >= 0) {
    __nv_bfloat16* dst = p.out + (size_t)s_token[my_row1] * p.out_stride + (size_t)s_head[my_row1] * HD + qc * 2;
    const float inv = 1.0f / l1;
#pragma unroll
    for (int i = 0; i < HD / 8; i++) *(__nv_bfloat162*)(dst + i * 8) = __floats2bfloat162_rn(o[i][2] * inv, o[i][3] * inv);
  }
}

template <int HD>
int launch_prefill(const PrefillParams& p, int grid_x, cudaStream_t stream) {
  const int smem = (PF_ROWS + 4 * PF_KEYS) * (HD + 8) * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return sprout_fail("attention_prefill: cannot reserve %d bytes of shared memory: %s", smem, cudaGetErrorString(err));
    configured = true;
  }
  sprout_launch(attention_prefill_kernel<HD>, dim3(grid_x, p.kv_heads), dim3(PF_THREADS), smem, stream, p);
  return sprout_check_launch("attention_prefill");
}

}  // namespace

// Scratch floats that a decode call with `splits` splits needs: outputs and (max, sum) pairs.
SPROUT_API long long sprout_attention_decode_scratch_floats(int requests, int heads, int head_dim, int splits) {
  return (long long)requests * heads * splits * (head_dim + 2);
}

// CTAs of the split-key decode kernel (the tensor-core one; fused: with the projection's tail;
// cluster: the variant launched in clusters) that an SM of the current device holds at once, or 0
// for a head size that kernel does not take.
SPROUT_API int sprout_attention_decode_ctas_per_sm(int head_dim, int fused, int cluster) {
  return decode_mma_ctas_per_sm_any(head_dim, fused != 0, cluster != 0);
}

struct FusedTail { float* acc; const float* bias; const float* cos_table; const float* sin_table; int max_positions; int rotary_dim, interleaved;
                   const float* norm_x; int norm_width; float norm_eps; };

static int decode_launch(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                         const int* block_table, int table_stride, const int* context_lens, void* out, int out_stride,
                         float* scratch, int requests, int heads, int kv_heads, int head_dim, int page_tokens,
                         int num_pages, int split_keys, int splits, int* status, cudaStream_t stream,
                         const FusedTail* extra) {
  const bool fused_early = extra != nullptr;
  (void)fused_early;

  SPROUT_REQUIRE(requests > 0 && requests <= 65535 && heads > 0 && kv_heads > 0 && page_tokens > 0 && num_pages > 0,
                 "attention_decode: sizes must be positive (at most 65535 requests)");
  SPROUT_REQUIRE(heads % kv_heads == 0 && heads / kv_heads <= MAX_GROUP,
                 "attention_decode: heads / kv_heads must be a whole number up to %d (got %d / %d)", MAX_GROUP, heads, kv_heads);
  SPROUT_REQUIRE(head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 256,
                 "attention_decode: head_dim must be a multiple of 16 between 16 and 256 (got %d)", head_dim);
  SPROUT_REQUIRE(split_keys > 0 && split_keys % DEC_THREADS == 0 && splits > 0 && splits <= 65535,
                 "attention_decode: split_keys must be a positive multiple of %d", DEC_THREADS);
  SPROUT_REQUIRE((q || fused_early) && k_cache && v_cache && block_table && context_lens && out && status, "attention_decode: null pointer");
  SPROUT_REQUIRE(q_stride % 2 == 0 && out_stride % 2 == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0,
                 "attention_decode: misaligned operands");
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table; p.table_stride = table_stride; p.context_lens = context_lens;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.part_out = scratch;
  p.part_ml = scratch ? scratch + (size_t)requests * heads * splits * head_dim : nullptr;
  p.heads = heads; p.kv_heads = kv_heads; p.head_dim = head_dim; p.page_tokens = page_tokens; p.num_pages = num_pages;
  p.split_keys = split_keys; p.splits = splits; p.status = status;
  p.acc = nullptr; p.bias = nullptr; p.cos_table = nullptr; p.sin_table = nullptr; p.max_positions = 0;
  p.rotary_dim = head_dim; p.interleaved = 0;
  p.k_append = nullptr; p.v_append = nullptr;
  p.norm_x = nullptr; p.norm_width = 0; p.norm_eps = 0.f;
  const bool fused = fused_early;
  if (fused) {
    SPROUT_REQUIRE(extra->acc && head_dim <= 128 && (splits <= 8 || scratch), "attention_decode_fused: needs the sums, head_dim <= 128 and, "
                   "without scratch memory, at most 8 splits");
    SPROUT_REQUIRE((extra->cos_table == nullptr) == (extra->sin_table == nullptr), "attention_decode_fused: cos and sin tables go together");
    p.acc = extra->acc; p.bias = extra->bias; p.cos_table = extra->cos_table; p.sin_table = extra->sin_table;
    p.max_positions = extra->max_positions;
    SPROUT_REQUIRE(extra->rotary_dim >= 0 && extra->rotary_dim % 2 == 0 && extra->rotary_dim <= head_dim,
                   "attention_decode_fused: rotary_dim must be even and at most head_dim (got %d of %d)", extra->rotary_dim, head_dim);
    p.rotary_dim = extra->rotary_dim; p.interleaved = extra->interleaved ? 1 : 0;
    SPROUT_REQUIRE(!extra->norm_x || (extra->norm_width > 0 && extra->norm_eps > 0.f), "attention_decode_fused: the norm's width and eps must be positive");
    p.norm_x = extra->norm_x; p.norm_width = extra->norm_width; p.norm_eps = extra->norm_eps;
    p.k_append = (__nv_bfloat16*)k_cache; p.v_append = (__nv_bfloat16*)v_cache;
  }
  const int group = heads / kv_heads;
  const size_t smem = (size_t)(group * head_dim + group * DEC_THREADS + MAX_GROUP * 8) * sizeof(float)
      + DEC_THREADS * sizeof(long long) + (size_t)2 * DEC_THREADS * (head_dim + 8) * sizeof(__nv_bfloat16)
      + (size_t)(group * head_dim + 2 * group) * sizeof(float);
  // no scratch given and at most 8 splits: the splits of a (request, key/value head) are a cluster
  const bool cluster = fused ? scratch == nullptr : (scratch == nullptr && splits > 1 && splits <= 8);
  SPROUT_REQUIRE(splits == 1 || cluster || scratch, "attention_decode: scratch memory is needed for more than 8 splits");
  if (head_dim <= 128) {
    const int rc = launch_decode_mma_any(p, fused, cluster, requests, stream);
    if (rc) return rc;
  } else {
  static size_t configured[2] = {48 * 1024, 48 * 1024};
  if (smem > configured[cluster]) {
    cudaError_t err = cluster
        ? cudaFuncSetAttribute(attention_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(attention_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return sprout_fail("attention_decode: group %d with head_dim %d needs %zu bytes of shared memory: %s",
                                               group, head_dim, smem, cudaGetErrorString(err));
    configured[cluster] = smem;
  }
  if (cluster) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(splits, kv_heads, requests);
    config.blockDim = dim3(DEC_THREADS);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = sprout_pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&config, attention_decode_kernel<true>, p);
    if (sprout_check_launch("attention_decode (cluster)")) return 1;
  } else {
    sprout_launch(attention_decode_kernel<false>, dim3(splits, kv_heads, requests), dim3(DEC_THREADS), smem, stream, p);
    if (sprout_check_launch("attention_decode")) return 1;
  }
  }
  if (cluster) return 0;
  if (splits > 1) {
    const int threads = (head_dim + 31) / 32 * 32;
    sprout_launch(attention_decode_merge_kernel, dim3(heads, requests), dim3(threads), 0, stream, p);
    return sprout_check_launch("attention_decode_merge");
  }
  return 0;
}


// One query token per request.  q, out: [requests, heads * head_dim] (row strides given);
// context_lens[r] keys are visible to request r.  scratch: float32, at least
// sprout_attention_decode_scratch_floats(...) long; it may be null for up to 8 splits, which are
// then merged inside a thread-block cluster instead of through memory.
SPROUT_API int sprout_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                       const int* block_table, int table_stride, const int* context_lens,
                                       void* out, int out_stride, float* scratch, int requests, int heads,
                                       int kv_heads, int head_dim, int page_tokens, int num_pages, int split_keys,
                                       int splits, int* status, cudaStream_t stream) {
  return decode_launch(q, q_stride, k_cache, v_cache, block_table, table_stride, context_lens, out, out_stride, scratch,
                       requests, heads, kv_heads, head_dim, page_tokens, num_pages, split_keys, splits, status, stream, nullptr);
}

// The decode step's attention with the projection's tail folded in: instead of q and an already
// appended cache it takes the float32 sums of the q/k/v product for each request's new token
// (acc [requests, (heads + 2 kv_heads) * head_dim], contiguous) and their bias; it rotates q and k
// by the token's position context_lens[r] - 1 (tables [max_positions, rotary_dim / 2]; null: no rotation;
// rotary_dim and interleaved as for sprout_rope_append), appends k and v to the cache, attends, and
// leaves acc zeroed.  head_dim <= 128; without scratch memory (as for
// sprout_attention_decode) at most 8 splits, merged inside a cluster.
SPROUT_API int sprout_attention_decode_fused(float* acc, const float* bias, const float* cos_table, const float* sin_table,
                                             int max_positions, int rotary_dim, int interleaved, void* k_cache, void* v_cache, const int* block_table,
                                             int table_stride, const int* context_lens, void* out, int out_stride,
                                             float* scratch, int requests, int heads, int kv_heads, int head_dim,
                                             int page_tokens, int num_pages, int split_keys, int splits,
                                             const float* norm_x, int norm_width, float norm_eps, int* status,
                                             cudaStream_t stream) {
  FusedTail extra{acc, bias, cos_table, sin_table, max_positions, rotary_dim, interleaved, norm_x, norm_width, norm_eps};
  return decode_launch(nullptr, 0, k_cache, v_cache, block_table, table_stride, context_lens, out, out_stride, scratch,
                       requests, heads, kv_heads, head_dim, page_tokens, num_pages, split_keys, splits, status, stream, &extra);
}

// The tcgen05 kernel of attention_tcgen05.cu.
SPROUT_API int sprout_attention_prefill_tc_supported(int head_dim, int page_tokens, int out_stride);
int sprout_attention_prefill_tc(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                const int* block_table, int table_stride, const int* q_start, const int* positions,
                                void* out, int out_stride, int num_tokens, int requests, int heads, int kv_heads,
                                int head_dim, int page_tokens, int num_pages, float* scratch, long long scratch_floats,
                                int* counters, int* status, cudaStream_t stream);

// Portions of prompts (and single tokens) of several requests in one launch.  q_start[r] is the
// first token of request r in the batch; a token at position pos sees keys 0..pos of its request.
// variant: 0 chooses (the tcgen05 kernel where it takes the sizes and the requests bring 128 rows
// each on average, else the mma.sync kernel), 1 forces mma.sync, 2 forces tcgen05.  scratch
// (float32) and counters (int32, zero, left zero) are optional: with them the tcgen05 kernel
// spreads a launch that is too small for the GPU over more SMs.
SPROUT_API int sprout_attention_prefill(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                        const int* block_table, int table_stride, const int* q_start,
                                        const int* positions, void* out, int out_stride, int num_tokens,
                                        int requests, int heads, int kv_heads, int head_dim, int page_tokens,
                                        int num_pages, int variant, float* scratch, long long scratch_floats,
                                        int* counters, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(num_tokens > 0 && requests > 0 && heads > 0 && kv_heads > 0 && page_tokens > 0 && num_pages > 0,
                 "attention_prefill: sizes must be positive");
  SPROUT_REQUIRE(heads % kv_heads == 0, "attention_prefill: heads (%d) must be a multiple of kv_heads (%d)", heads, kv_heads);
  SPROUT_REQUIRE(kv_heads <= 65535, "attention_prefill: too many kv heads");
  SPROUT_REQUIRE(q && k_cache && v_cache && block_table && q_start && positions && out && status, "attention_prefill: null pointer");
  SPROUT_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0
                 && out_stride % 2 == 0, "attention_prefill: q rows and the caches must be 16-byte aligned");
  PrefillParams p;
  p.q = (const __nv_bfloat16*)q; p.q_stride = q_stride;
  p.k_cache = (const __nv_bfloat16*)k_cache; p.v_cache = (const __nv_bfloat16*)v_cache;
  p.block_table = block_table; p.table_stride = table_stride; p.q_start = q_start; p.positions = positions;
  p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.requests = requests; p.heads = heads; p.kv_heads = kv_heads; p.page_tokens = page_tokens; p.num_pages = num_pages;
  p.scale = 1.0f / sqrtf((float)head_dim); p.status = status;
  const int group = heads / kv_heads;
  SPROUT_REQUIRE(variant >= 0 && variant <= 2, "attention_prefill: unknown variant %d", variant);
  const bool tc_takes = sprout_attention_prefill_tc_supported(head_dim, page_tokens, out_stride) && ((uintptr_t)out & 15) == 0;
  SPROUT_REQUIRE(variant != 2 || tc_takes, "attention_prefill: the tcgen05 kernel takes head_dim 64 or 128, pages of 8, 16, 32, 64 "
                 "or a multiple of 128 tokens and 16-byte aligned output rows (head_dim %d, page %d)", head_dim, page_tokens);
  if (variant == 2 || (variant == 0 && tc_takes && (long long)num_tokens * group >= 128LL * requests))
    return sprout_attention_prefill_tc(q, q_stride, k_cache, v_cache, block_table, table_stride, q_start, positions, out,
                                       out_stride, num_tokens, requests, heads, kv_heads, head_dim, page_tokens, num_pages,
                                       scratch, scratch_floats, counters, status, stream);
  // every request has at most ceil(tokens * group / 64) tiles: an upper bound without reading q_start
  const long long bound = ((long long)num_tokens * group + PF_ROWS - 1) / PF_ROWS + requests;
  SPROUT_REQUIRE(bound <= 0x7fffffffLL, "attention_prefill: too many tokens");
  switch (head_dim) {
    case 16: return launch_prefill<16>(p, (int)bound, stream);
    case 32: return launch_prefill<32>(p, (int)bound, stream);
    case 48: return launch_prefill<48>(p, (int)bound, stream);
    case 64: return launch_prefill<64>(p, (int)bound, stream);
    case 80: return launch_prefill<80>(p, (int)bound, stream);
    case 96: return launch_prefill<96>(p, (int)bound, stream);
    case 112: return launch_prefill<112>(p, (int)bound, stream);
    case 128: return launch_prefill<128>(p, (int)bound, stream);
    default: return sprout_fail("attention_prefill: head_dim must be a multiple of 16 up to 128 (got %d)", head_dim);
  }
}

// =============================================================================== allocation-free variant
#include "no_alloc.h"

namespace {

// Partial results of the key splits for callers that cannot hand over scratch memory.  In host
// code this name stands for the symbol only; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_static_decode_scratch[SPROUT_STATIC_SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_static_scratch_address[MAX_DEVICES] = {};

// Device address of the scratch array on the current device, looked up on first use.
int static_scratch(float** address) {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return sprout_fail("attention_decode_static: cudaGetDevice failed: %s", cudaGetErrorString(err));
  if (device < 0 || device >= MAX_DEVICES) return sprout_fail("attention_decode_static: device %d out of range", device);
  if (!g_static_scratch_address[device]) {
    float* found = nullptr;
    err = cudaGetSymbolAddress((void**)&found, g_static_decode_scratch);
    if (err != cudaSuccess || !found)
      return sprout_fail("attention_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
    g_static_scratch_address[device] = found;
  }
  *address = g_static_scratch_address[device];
  return 0;
}

}  // namespace

// See no_alloc.h.  Same computation as sprout_attention_decode with the library's own scratch.
SPROUT_API int sprout_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                              const int* block_table, int table_stride, const int* context_lens,
                                              void* out, int out_stride, int requests, int heads, int kv_heads,
                                              int head_dim, int page_tokens, int num_pages, int split_keys,
                                              int splits, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(requests > 0 && heads > 0 && head_dim > 0 && splits > 0, "attention_decode_static: sizes must be positive");
  const long long need = sprout_attention_decode_scratch_floats(requests, heads, head_dim, splits);
  SPROUT_REQUIRE(need <= (long long)SPROUT_STATIC_SCRATCH_FLOATS,
                 "attention_decode_static: %d requests x %d heads x %d splits of head_dim %d need %lld floats of scratch; "
                 "the built-in array holds %d (use fewer splits or sprout_attention_decode with your own scratch)",
                 requests, heads, splits, head_dim, need, SPROUT_STATIC_SCRATCH_FLOATS);
  float* scratch = nullptr;
  if (static_scratch(&scratch)) return 1;
  return sprout_attention_decode(q, q_stride, k_cache, v_cache, block_table, table_stride, context_lens, out, out_stride,
                                 scratch, requests, heads, kv_heads, head_dim, page_tokens, num_pages, split_keys, splits,
                                 status, stream);
}

