// ref_host_shim.cpp — TEST INFRASTRUCTURE.  C entry points around the reference's
// own host headers (code/graph/kv_pool.h, kv_block.h, kv_registry.h), compiled from
// the reference tree where it lies (see oracle/build.py) into
// oracle/_ref/libnova_ref_host.so.  Only tests/, the smoke check and the bench's
// CPU baseline load it; the product never does.
//
// The reference keeps its free lists private; parity tests need their ORDER, so
// the headers are included with `private` opened up.  The standard headers they
// use are included first so that only the reference's classes are affected.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#define private public
#include "graph/kv_pool.h"
#include "graph/kv_registry.h"
#undef private

namespace {
nova::KvSlice* slice_by_id(nova::KvPool* p, int id) {
    for (auto& s : p->slices_) if (s.id == id) return &s;
    return nullptr;
}
template <class V>
int dump(const V& v, int32_t* out, int cap) {
    const int n = (int)v.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = (int32_t)v[(size_t)i];
    return n;
}
}  // namespace

extern "C" {

int ref_kv_block(void) { return nova::kKvBlock; }

void* ref_pool_create(void) { return new nova::KvPool(); }
void ref_pool_destroy(void* p) { delete (nova::KvPool*)p; }
void ref_pool_init(void* p, int n_slices, int64_t ctx) { ((nova::KvPool*)p)->init(n_slices, ctx); }
int ref_pool_acquire(void* p) {
    nova::KvSlice* s = ((nova::KvPool*)p)->acquire();
    return s ? s->id : -3;
}
int ref_pool_release(void* p, int id) {
    auto* kp = (nova::KvPool*)p;
    nova::KvSlice* s = slice_by_id(kp, id);
    if (!s) return -1;
    kp->release(s);
    return 0;
}
int ref_pool_alloc_block(void* p) { return ((nova::KvPool*)p)->alloc_block(); }
void ref_pool_free_block(void* p, int b) { ((nova::KvPool*)p)->free_block(b); }
void ref_pool_ref_block(void* p, int b) { ((nova::KvPool*)p)->ref_block(b); }
int ref_pool_refcnt(void* p, int b) { return ((nova::KvPool*)p)->refcnt(b); }
int ref_pool_attach(void* p, int dst, int src, int k) {
    auto* kp = (nova::KvPool*)p;
    nova::KvSlice *d = slice_by_id(kp, dst), *s = slice_by_id(kp, src);
    if (!d || !s) return -1;
    kp->attach(*d, *s, k);
    return 0;
}
int ref_pool_attach_prefix(void* p, int dst, int src, int64_t n) {
    auto* kp = (nova::KvPool*)p;
    nova::KvSlice *d = slice_by_id(kp, dst), *s = slice_by_id(kp, src);
    if (!d || !s) return -1;
    kp->attach_prefix(*d, *s, n);
    return 0;
}
int ref_pool_cow_slice(void* p, int id, int64_t pos) {
    auto* kp = (nova::KvPool*)p;
    nova::KvSlice* s = slice_by_id(kp, id);
    if (!s) return -1;
    return kp->cow_slice(*s, pos);
}
int ref_pool_need_copy(void* p, int id, int* from, int* blk) {
    nova::KvSlice* s = slice_by_id((nova::KvPool*)p, id);
    if (!s) return -1;
    *from = s->need_copy_from;
    *blk = s->need_copy_blk;
    return 0;
}
int ref_pool_clear_need_copy(void* p, int id) {   // what Engine::cow_guard does (src/model.cpp:176)
    nova::KvSlice* s = slice_by_id((nova::KvPool*)p, id);
    if (!s) return -1;
    s->need_copy_from = -1;
    return 0;
}
int64_t ref_pool_n_past(void* p, int id) {
    nova::KvSlice* s = slice_by_id((nova::KvPool*)p, id);
    return s ? s->n_past : -1;
}
int ref_pool_nb_total(void* p) { return ((nova::KvPool*)p)->nb_total(); }
int ref_pool_nblocks(void* p) { return ((nova::KvPool*)p)->nblocks(); }
int ref_pool_cow_count(void* p) { return ((nova::KvPool*)p)->cow_count(); }
int ref_pool_free_blocks(void* p) { return ((nova::KvPool*)p)->free_blocks(); }
int ref_pool_free_slices(void* p) { return ((nova::KvPool*)p)->free_slices(); }
int ref_pool_used(void* p) { return ((nova::KvPool*)p)->used(); }
int ref_pool_get_table(void* p, int id, int32_t* out, int cap) {
    nova::KvSlice* s = slice_by_id((nova::KvPool*)p, id);
    return s ? dump(s->table, out, cap) : -1;
}
int ref_pool_get_refcnts(void* p, int32_t* out, int cap) { return dump(((nova::KvPool*)p)->refcnt_, out, cap); }
int ref_pool_get_free_list(void* p, int32_t* out, int cap) { return dump(((nova::KvPool*)p)->free_blocks_, out, cap); }
int ref_pool_get_free_slices(void* p, int32_t* out, int cap) { return dump(((nova::KvPool*)p)->free_, out, cap); }
int ref_pool_get_live_slices(void* p, int32_t* out, int cap) {
    auto* kp = (nova::KvPool*)p;
    const int n = (int)kp->slices_.size();
    for (int i = 0; i < n && i < cap; ++i) out[i] = kp->slices_[(size_t)i].id;
    return n;
}

uint64_t ref_kv_hash_ids(const int32_t* ids, size_t n) {
    std::vector<int> v(ids, ids + n);
    return nova::kv_hash_ids(v);
}
uint64_t ref_kv_hash_text(const char* b, size_t n) { return nova::kv_hash_text(std::string(b, n)); }
void ref_kv_hash_hex(uint64_t v, char* out17) {
    const std::string s = nova::kv_hash_hex(v);
    std::memcpy(out17, s.c_str(), 17);
}
void ref_kv_block_id(uint64_t a, uint64_t b, char* out40) {
    const std::string s = nova::kv_block_id(a, b);
    std::memcpy(out40, s.c_str(), s.size() + 1);
}

struct RefBlock { uint64_t prefix, suffix; int32_t session, turn; int64_t pos0, pos1; };
void* ref_registry_create(void) { return new nova::BlockRegistry(); }
void ref_registry_destroy(void* r) { delete (nova::BlockRegistry*)r; }
void ref_registry_set_capacity(void* r, size_t n) { ((nova::BlockRegistry*)r)->set_capacity(n); }
size_t ref_registry_capacity(void* r) { return ((nova::BlockRegistry*)r)->capacity(); }
void ref_registry_put(void* r, const RefBlock* b) {
    nova::KvBlock k;
    k.prefix = b->prefix; k.suffix = b->suffix; k.session = b->session; k.turn = b->turn;
    k.pos0 = b->pos0; k.pos1 = b->pos1;
    ((nova::BlockRegistry*)r)->put(k);
}
int ref_registry_find(void* r, uint64_t p, uint64_t s, RefBlock* out) {
    const nova::KvBlock* k = ((nova::BlockRegistry*)r)->find(p, s);
    if (!k) return 0;
    out->prefix = k->prefix; out->suffix = k->suffix; out->session = k->session; out->turn = k->turn;
    out->pos0 = k->pos0; out->pos1 = k->pos1;
    return 1;
}
int ref_registry_live(void* r) { return ((nova::BlockRegistry*)r)->live(); }
int ref_registry_total(void* r) { return ((nova::BlockRegistry*)r)->total(); }

}  // extern "C"
