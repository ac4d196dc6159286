// attn_mma.cu — tensor-core form of the paged decode attention (placeholder until built).
#include "common.cuh"

namespace novab {
bool attn_mma_built() { return false; }
int attn_default_ctas_mma() { return 148; }
int launch_attn_mma(const AttnLaunch&, int, int, cudaStream_t) { return NOVA_ERR_UNSUPPORTED; }
}  // namespace novab
