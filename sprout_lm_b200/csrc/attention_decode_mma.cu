// Decode attention on tensor cores, head sizes 16 to 64, and the dispatch over all head sizes (the
// kernel itself is in attention_decode_mma.cuh; head sizes 80 to 128 are built in attention_decode_mma_wide.cu).
#include "attention_decode_mma.cuh"

namespace sprout_attn {

int launch_decode_mma_narrow(const DecodeParams& p, bool fused, bool cluster, int requests, cudaStream_t stream) {
  switch (p.head_dim) {
    case 16: return fused ? launch_decode_mma<16, true>(p, cluster, requests, stream) : launch_decode_mma<16, false>(p, cluster, requests, stream);
    case 32: return fused ? launch_decode_mma<32, true>(p, cluster, requests, stream) : launch_decode_mma<32, false>(p, cluster, requests, stream);
    case 48: return fused ? launch_decode_mma<48, true>(p, cluster, requests, stream) : launch_decode_mma<48, false>(p, cluster, requests, stream);
    case 64: return fused ? launch_decode_mma<64, true>(p, cluster, requests, stream) : launch_decode_mma<64, false>(p, cluster, requests, stream);
    default: return sprout_fail("attention_decode: the tensor-core kernel takes head sizes of 16 to 128 in steps of 16, not %d", p.head_dim);
  }
}

int decode_mma_ctas_per_sm_narrow(int head_dim, bool fused, bool cluster) {
  switch (head_dim) {
    case 16: return decode_mma_ctas_per_sm<16>(fused, cluster);
    case 32: return decode_mma_ctas_per_sm<32>(fused, cluster);
    case 48: return decode_mma_ctas_per_sm<48>(fused, cluster);
    case 64: return decode_mma_ctas_per_sm<64>(fused, cluster);
    default: return 0;
  }
}

int launch_decode_mma_wide(const DecodeParams& p, bool fused, bool cluster, int requests, cudaStream_t stream);
int decode_mma_ctas_per_sm_wide(int head_dim, bool fused, bool cluster);

int launch_decode_mma_any(const DecodeParams& p, bool fused, bool cluster, int requests, cudaStream_t stream) {
  return p.head_dim <= 64 ? launch_decode_mma_narrow(p, fused, cluster, requests, stream) : launch_decode_mma_wide(p, fused, cluster, requests, stream);
}

int decode_mma_ctas_per_sm_any(int head_dim, bool fused, bool cluster) {
  return head_dim <= 64 ? decode_mma_ctas_per_sm_narrow(head_dim, fused, cluster) : decode_mma_ctas_per_sm_wide(head_dim, fused, cluster);
}

}  // namespace sprout_attn

#ifdef ATTN_STAMPS
extern "C" __attribute__((visibility("default"))) void sprout_attention_stamps(unsigned long long* out) { cudaMemcpyFromSymbol(out, g_attn_stamps, sizeof(g_attn_stamps)); }
#endif

SPROUT_TL_READER(attention_bf16)
