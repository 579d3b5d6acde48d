// Decode attention on tensor cores, head sizes 80 to 128 (the kernel is in attention_decode_mma.cuh).
#include "attention_decode_mma.cuh"

namespace sprout_attn {

int launch_decode_mma_wide(const DecodeParams& p, bool fused, bool cluster, int requests, cudaStream_t stream) {
  switch (p.head_dim) {
    case 80: return fused ? launch_decode_mma<80, true>(p, cluster, requests, stream) : launch_decode_mma<80, false>(p, cluster, requests, stream);
    case 96: return fused ? launch_decode_mma<96, true>(p, cluster, requests, stream) : launch_decode_mma<96, false>(p, cluster, requests, stream);
    case 112: return fused ? launch_decode_mma<112, true>(p, cluster, requests, stream) : launch_decode_mma<112, false>(p, cluster, requests, stream);
    case 128: return fused ? launch_decode_mma<128, true>(p, cluster, requests, stream) : launch_decode_mma<128, false>(p, cluster, requests, stream);
    default: return sprout_fail("attention_decode: the tensor-core kernel takes head sizes of 16 to 128 in steps of 16, not %d", p.head_dim);
  }
}

int decode_mma_ctas_per_sm_wide(int head_dim, bool fused, bool cluster) {
  switch (head_dim) {
    case 80: return decode_mma_ctas_per_sm<80>(fused, cluster);
    case 96: return decode_mma_ctas_per_sm<96>(fused, cluster);
    case 112: return decode_mma_ctas_per_sm<112>(fused, cluster);
    case 128: return decode_mma_ctas_per_sm<128>(fused, cluster);
    default: return 0;
  }
}

}  // namespace sprout_attn

SPROUT_TL_READER(attention_bf16_wide)
