// nova_b200_shim.h — the reference-side binding: Conflux Nova's four hot-path launchers
// (include/nova/kernel.h:44-49,62-64) defined on top of the C ABI of nova_b200.h, so that the
// reference's call sites (RopeKvOp / AttnOp in code/graph/dense.h:75-95, Engine::decode_batch in
// src/model.cpp:281-290) compile and link unchanged against libnova_b200.so once the definitions in
// src/kernel/{rope,elem,attn}.cu are left out of the build.  fp32 pools (the reference's format).
//
// Include AFTER the reference's "nova/kernel.h" (it needs nova::Model, ArchTraits, kCtx) and
// "graph/kv_pool_cfg.h" (kKvBlock).  Errors abort, as everything does in the reference (NOVA_CU).
#pragma once
#include <cstdio>
#include <cstdlib>

#include "nova_b200.h"

namespace nova {

inline nova_kv_shape b200_shape() {
    return {Model::NH, Model::NKV, Model::HD, kKvBlock, NOVA_KV_F32,
            ArchTraits<typename Model::arch>::kRope == RopeLayout::Neox ? 1 : 0};
}
inline void b200_check(int rc, const char* what) {
    if (rc < 0) {
        std::fprintf(stderr, "[nova] FATAL %s: %s %s\n", what, nova_status_string(rc), nova_last_cuda_error());
        std::abort();
    }
}

inline void launch_rope_table(float* cs, float* sn, cudaStream_t s) {
    b200_check(nova_launch_rope_table(cs, sn, kCtx, Model::HD, Model::theta, s), "rope_table");
}

// RopeKvOp calls rope_batch and kv_store_paged back to back with the same (n, pos0, k).  The pair is one
// fused launch here: rope_batch only notes its arguments, kv_store_paged issues the launch.
struct B200PendingRope {
    float* q = nullptr;
    float* k = nullptr;
    const float* cs = nullptr;
    const float* sn = nullptr;
    int n = 0;
    int64_t pos0 = 0;
};
inline B200PendingRope& b200_pending() {
    static thread_local B200PendingRope p;
    return p;
}
inline void launch_rope_batch(float* q, float* k, int n, int64_t pos0, const float* cs, const float* sn, cudaStream_t) {
    B200PendingRope& p = b200_pending();
    p.q = q; p.k = k; p.cs = cs; p.sn = sn; p.n = n; p.pos0 = pos0;
}
inline void launch_kv_store_paged(float* pool_k, float* pool_v, const int32_t* table, int layer, int nb, int n,
                                  int64_t pos0, const float* k, const float* v, cudaStream_t s) {
    B200PendingRope& p = b200_pending();
    if (p.k != k || p.n != n || p.pos0 != pos0) {
        std::fprintf(stderr, "[nova] FATAL kv_store_paged without the matching rope_batch before it\n");
        std::abort();
    }
    const nova_kv_shape sh = b200_shape();
    b200_check(nova_launch_rope_append_paged(&sh, pool_k, pool_v, table, layer, nb, n, pos0, p.q, p.k, v, p.cs, p.sn, s),
               "rope_append_paged");
    p = B200PendingRope{};
}
inline void launch_attn_decode_paged(const float* q, const float* pool_k, const float* pool_v, const int32_t* table,
                                     int layer, int nb, int n_keys, float* o, float* scratch, cudaStream_t s) {
    const nova_kv_shape sh = b200_shape();
    b200_check(nova_launch_attn_decode_paged(&sh, q, pool_k, pool_v, table, layer, nb, n_keys, o, scratch, s),
               "attn_decode_paged");
}

}  // namespace nova
