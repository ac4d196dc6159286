// shim_exec.cpp — TEST INFRASTRUCTURE.  The reference's own call sites for this path (RopeKvOp / AttnOp of
// code/graph/dense.h:75-95, spelled through nova::Kernel of include/nova/kernel.h) compiled against
// include/nova_b200_shim.h instead of the reference's src/kernel/*.cu, as a shared library that the GPU tests load
// and EXECUTE: the reference-side binding is not only shown to compile and link, it is run and its results are
// compared with the oracle.  Built by oracle/build.py into oracle/_ref/libnova_shim_<model>.so from the reference
// headers where they lie; the product never loads it.
#include <cstdint>
#include <cuda_runtime.h>

#include "nova/kernel.h"
#include "graph/kv_pool_cfg.h"
#include "nova_b200_shim.h"

extern "C" {

void shim_shape(int32_t* out6) {
    out6[0] = nova::Model::L;  out6[1] = nova::Model::NH; out6[2] = nova::Model::NKV;
    out6[3] = nova::Model::HD; out6[4] = nova::kKvBlock;  out6[5] = nova::Model::theta;
}

// launch_rope_table (src/model.cpp:119): kCtx rows
void shim_rope_table(float* cs, float* sn, void* stream) { nova::Kernel::rope_table(cs, sn, (cudaStream_t)stream); }

// One decode step of one session in one layer, in the reference's order: RopeKvOp then AttnOp.
void shim_decode_layer(float* q, float* k, float* v, float* pool_k, float* pool_v, const int32_t* table, int layer,
                       int nb, int64_t pos, const float* cs, const float* sn, float* out, float* scratch, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    nova::Kernel::rope_batch(q, k, 1, pos, cs, sn, s);
    nova::Kernel::kv_store_paged(pool_k, pool_v, table, layer, nb, 1, pos, k, v, s);
    nova::Kernel::attn_decode_paged(q, pool_k, pool_v, table, layer, nb, (int)pos + 1, out, scratch, s);
}

}  // extern "C"
