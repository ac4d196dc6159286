// ref_gpu_shim.cu — TEST INFRASTRUCTURE.  C entry points around the reference's own
// CUDA launchers for this path (src/kernel/rope.cu, elem.cu, attn.cu), which are
// compiled unmodified for sm_100a from the reference tree where it lies (see
// oracle/build.py) together with this file into
// oracle/_ref/libnova_ref_gpu_<model>.so.  The model shape is the reference's
// compile-time ActiveModel (-DNOVA_MODEL_QWEN25_7B / -DNOVA_MODEL_QWEN25_1P5B).
// Used by the GPU parity tests and by the bench's "reference kernels on this GPU"
// figure; the product never loads it.
#include <cstdint>
#include <cuda_runtime.h>
#include "nova/kernel.h"
#include "graph/kv_pool_cfg.h"

extern "C" {

void ref_gpu_shape(int32_t* out6) {
    out6[0] = nova::Model::L;  out6[1] = nova::Model::NH; out6[2] = nova::Model::NKV;
    out6[3] = nova::Model::HD; out6[4] = nova::kKvBlock;  out6[5] = nova::Model::theta;
}
int ref_gpu_kctx(void) { return nova::kCtx; }

void ref_gpu_rope_table(float* cs, float* sn, void* stream) {
    nova::launch_rope_table(cs, sn, (cudaStream_t)stream);
}
void ref_gpu_rope_batch(float* q, float* k, int n, int64_t pos0, const float* cs, const float* sn,
                        void* stream) {
    nova::launch_rope_batch(q, k, n, pos0, cs, sn, (cudaStream_t)stream);
}
void ref_gpu_rope(float* q, float* k, int64_t pos, const float* cs, const float* sn, void* stream) {
    nova::launch_rope(q, k, pos, cs, sn, (cudaStream_t)stream);
}
void ref_gpu_kv_store_paged(float* pool_k, float* pool_v, const int32_t* table, int layer, int nb,
                            int n, int64_t pos0, const float* k, const float* v, void* stream) {
    nova::launch_kv_store_paged(pool_k, pool_v, table, layer, nb, n, pos0, k, v, (cudaStream_t)stream);
}
void ref_gpu_attn_decode_paged(const float* q, const float* pool_k, const float* pool_v,
                               const int32_t* table, int layer, int nb, int n_keys, float* o,
                               float* scratch, void* stream) {
    nova::launch_attn_decode_paged(q, pool_k, pool_v, table, layer, nb, n_keys, o, scratch,
                                   (cudaStream_t)stream);
}
void ref_gpu_attn_prefill_paged(const float* q, const float* pool_k, const float* pool_v, const int32_t* table,
                                int layer, int nb, int n_q, int n_past, float* o, void* stream) {
    nova::launch_attn_prefill_paged(q, pool_k, pool_v, table, layer, nb, n_q, n_past, o, (cudaStream_t)stream);
}
void ref_gpu_attn_decode(const float* q, const float* kc, const float* vc, float* o, int n_past,
                         float* scratch, void* stream) {
    nova::launch_attn_decode(q, kc, vc, o, n_past, scratch, (cudaStream_t)stream);
}
// One decode step of n sessions in one layer in the reference's order (per session: rope_batch, kv_store_paged,
// attn_decode_paged = RopeKvOp then AttnOp, code/graph/dense.h:75-95), issued from one C call so that a timing of it
// is not bound by an interpreter's loop.  Rows of session i at i * q_stride / i * kv_stride floats.
void ref_gpu_decode_layer_sessions(int n, float* pool_k, float* pool_v, const int32_t* const* tables, int layer, int nb,
                                   const int64_t* pos, float* q, float* k, const float* v, size_t q_stride, size_t kv_stride,
                                   const float* cs, const float* sn, float* o, float* scratch, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    for (int i = 0; i < n; ++i) {
        float* qi = q + (size_t)i * q_stride;
        float* ki = k + (size_t)i * kv_stride;
        const float* vi = v + (size_t)i * kv_stride;
        nova::launch_rope_batch(qi, ki, 1, pos[i], cs, sn, s);
        nova::launch_kv_store_paged(pool_k, pool_v, tables[i], layer, nb, 1, pos[i], ki, vi, s);
        nova::launch_attn_decode_paged(qi, pool_k, pool_v, tables[i], layer, nb, (int)pos[i] + 1, o + (size_t)i * q_stride, scratch, s);
    }
}
int ref_gpu_last_error(void) { return (int)cudaGetLastError(); }

}  // extern "C"
