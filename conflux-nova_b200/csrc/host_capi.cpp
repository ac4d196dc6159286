// host_capi.cpp — C ABI of the host-only parts: block-ID hashing, BlockRegistry and the page
// pool.  No CUDA in this file.
#include <cstring>

#include "../../include/nova_b200.h"
#include "handles.hpp"

namespace {
template <class V>
int dump_ints(const V& v, int32_t* out, int cap) {
    const int n = (int)v.size();
    if (out)
        for (int i = 0; i < n && i < cap; ++i) out[i] = (int32_t)v[(size_t)i];
    return n;
}
}  // namespace

extern "C" {

uint64_t nova_kv_hash_ids(const int32_t* ids, size_t n) { return (ids && n) ? novab::hash_ids(ids, n) : 0; }
uint64_t nova_kv_hash_text(const char* bytes, size_t n) { return (bytes && n) ? novab::hash_text(bytes, n) : 0; }
void nova_kv_hash_hex(uint64_t v, char* out17) {
    if (out17) novab::hash_hex(v, out17);
}
void nova_kv_block_id(uint64_t prefix, uint64_t suffix, char* out40) {
    if (out40) novab::block_id(prefix, suffix, out40);
}

nova_registry* nova_registry_create(void) { return new nova_registry(); }
void nova_registry_destroy(nova_registry* r) { delete r; }
void nova_registry_set_capacity(nova_registry* r, size_t n) {
    if (r) r->r.set_capacity(n);
}
size_t nova_registry_capacity(const nova_registry* r) { return r ? r->r.capacity() : 0; }
void nova_registry_put(nova_registry* r, const nova_kv_block* b) {
    if (!r || !b) return;
    novab::BlockEntry e;
    e.prefix = b->prefix; e.suffix = b->suffix; e.session = b->session; e.turn = b->turn;
    e.pos0 = b->pos0; e.pos1 = b->pos1;
    r->r.put(e);
}
int nova_registry_find(const nova_registry* r, uint64_t prefix, uint64_t suffix, nova_kv_block* out) {
    if (!r) return 0;
    const novab::BlockEntry* e = r->r.find(prefix, suffix);
    if (!e) return 0;
    if (out) {
        out->prefix = e->prefix; out->suffix = e->suffix; out->session = e->session; out->turn = e->turn;
        out->pos0 = e->pos0; out->pos1 = e->pos1;
    }
    return 1;
}
int nova_registry_live(const nova_registry* r) { return r ? r->r.live() : 0; }
int nova_registry_total(const nova_registry* r) { return r ? r->r.total() : 0; }

nova_pool* nova_pool_create(int kv_block) {
    nova_pool* p = new nova_pool();
    if (!p->p.set_block(kv_block)) {
        delete p;
        return nullptr;
    }
    return p;
}
void nova_pool_destroy(nova_pool* p) { delete p; }
int nova_pool_init(nova_pool* p, int n_slices, int64_t ctx) {
    if (!p || n_slices <= 0 || ctx <= 0) return NOVA_ERR_INVALID;
    const int64_t nblocks = (ctx + p->p.kv_block() - 1) / p->p.kv_block();
    if (nblocks * n_slices > 0x7fffffffLL) return NOVA_ERR_TOO_LARGE;
    p->p.init(n_slices, ctx);
    return NOVA_OK;
}
int nova_pool_acquire(nova_pool* p) {
    if (!p) return NOVA_ERR_INVALID;
    const int id = p->p.acquire();
    return id < 0 ? NOVA_ERR_NO_SLICE : id;
}
int nova_pool_release(nova_pool* p, int slice) {
    if (!p) return NOVA_ERR_INVALID;
    return p->p.release(slice) ? NOVA_OK : NOVA_ERR_INVALID;
}
int nova_pool_alloc_block(nova_pool* p) { return p ? p->p.alloc_page() : NOVA_ERR_INVALID; }
int nova_pool_free_block(nova_pool* p, int b) {
    if (!p) return NOVA_ERR_INVALID;
    p->p.free_page(b);
    return NOVA_OK;
}
int nova_pool_ref_block(nova_pool* p, int b) {
    if (!p) return NOVA_ERR_INVALID;
    p->p.ref_page(b);
    return NOVA_OK;
}
int nova_pool_refcnt(const nova_pool* p, int b) { return p ? p->p.refcnt(b) : 0; }
int nova_pool_attach(nova_pool* p, int dst, int src, int k) {
    if (!p) return NOVA_ERR_INVALID;
    return p->p.attach(dst, src, k) ? NOVA_OK : NOVA_ERR_INVALID;
}
int nova_pool_attach_prefix(nova_pool* p, int dst, int src, int64_t n_tokens) {
    if (!p) return NOVA_ERR_INVALID;
    return p->p.attach_prefix(dst, src, n_tokens) ? NOVA_OK : NOVA_ERR_INVALID;
}
int nova_pool_cow_slice(nova_pool* p, int slice, int64_t pos) {
    if (!p || !p->p.find(slice)) return -1;
    return p->p.cow(slice, pos);   // new page, -1 (nothing to do) or -2 == NOVA_ERR_POOL_FULL
}
int nova_pool_need_copy(const nova_pool* p, int slice, int* from, int* blk) {
    const novab::SliceState* s = p ? p->p.find(slice) : nullptr;
    if (!s) return NOVA_ERR_INVALID;
    if (from) *from = s->copy_from;
    if (blk) *blk = s->copy_to;
    return NOVA_OK;
}
int nova_pool_clear_need_copy(nova_pool* p, int slice) {
    novab::SliceState* s = p ? p->p.find(slice) : nullptr;
    if (!s) return NOVA_ERR_INVALID;
    s->copy_from = -1;   // the reference's cow_guard clears only the source (src/model.cpp:175-176)
    return NOVA_OK;
}
int nova_pool_next_slice(const nova_pool* p) { return p ? p->p.next_slice() : NOVA_ERR_INVALID; }
int nova_pool_foreign_mappings(const nova_pool* p, int slice) {
    if (!p || slice < 0 || (int64_t)(slice + 1) * p->p.nblocks() > p->p.nb_total()) return NOVA_ERR_INVALID;
    return p->p.foreign_mappings(slice);
}
int nova_pool_nb_total(const nova_pool* p) { return p ? p->p.nb_total() : 0; }
int nova_pool_nblocks(const nova_pool* p) { return p ? p->p.nblocks() : 0; }
int nova_pool_cow_count(const nova_pool* p) { return p ? p->p.cow_count() : 0; }
int nova_pool_free_blocks(const nova_pool* p) { return p ? p->p.free_pages() : 0; }
int nova_pool_free_slices(const nova_pool* p) { return p ? p->p.free_slices() : 0; }
int nova_pool_used(const nova_pool* p) { return p ? p->p.used() : 0; }
int64_t nova_pool_n_past(const nova_pool* p, int slice) {
    const novab::SliceState* s = p ? p->p.find(slice) : nullptr;
    return s ? s->n_past : -1;
}
int nova_pool_set_n_past(nova_pool* p, int slice, int64_t n_past) {
    novab::SliceState* s = p ? p->p.find(slice) : nullptr;
    if (!s) return NOVA_ERR_INVALID;
    s->n_past = n_past;
    return NOVA_OK;
}
int nova_pool_get_table(const nova_pool* p, int slice, int32_t* out, int cap) {
    const novab::SliceState* s = p ? p->p.find(slice) : nullptr;
    return s ? dump_ints(s->table, out, cap) : NOVA_ERR_INVALID;
}
int nova_pool_get_refcnts(const nova_pool* p, int32_t* out, int cap) {
    return p ? dump_ints(p->p.refs(), out, cap) : NOVA_ERR_INVALID;
}
int nova_pool_get_free_list(const nova_pool* p, int32_t* out, int cap) {
    return p ? dump_ints(p->p.page_stack(), out, cap) : NOVA_ERR_INVALID;
}
int nova_pool_get_free_slices(const nova_pool* p, int32_t* out, int cap) {
    return p ? dump_ints(p->p.slice_stack(), out, cap) : NOVA_ERR_INVALID;
}
int nova_pool_get_live_slices(const nova_pool* p, int32_t* out, int cap) {
    if (!p) return NOVA_ERR_INVALID;
    const auto& lv = p->p.live();
    const int n = (int)lv.size();
    if (out)
        for (int i = 0; i < n && i < cap; ++i) out[i] = lv[(size_t)i].id;
    return n;
}

}  // extern "C"
