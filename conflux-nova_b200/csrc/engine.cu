// engine.cu — the engine-side glue of the paged-KV decode path behind the C ABI: page pools,
// block tables and RoPE tables in device memory (Engine, include/nova/model.h:117-179 and
// src/model.cpp:93-96,115-119 of the reference), sessions with their own streams
// (SessionManager, code/session.h:74-150), the copy-on-write guard (src/model.cpp:171-191),
// the raw launcher entry points (include/nova/kernel.h:44-49,62-64) and the batched
// per-layer / all-layer decode calls that replace the per-session loop of
// Engine::decode_batch (src/model.cpp:281-290).
#include <algorithm>
#include <atomic>
#include <cstring>
#include <limits>
#include <mutex>
#include <new>
#include <vector>

#include "common.cuh"
#include "handles.hpp"

using namespace novab;

namespace {
struct SessionRec {
    bool used = false;
    int slice = -1;
    cudaStream_t stream = nullptr;
};
constexpr int kMaxSplitCtas = kMaxSms * 8;   // upper bound of CTAs of any attention launch (partial slots)
}  // namespace

struct nova_engine {
    nova_engine_desc d{};
    nova_pool pool;
    void* pool_k = nullptr;
    void* pool_v = nullptr;
    int32_t* tables = nullptr;       // [n_slices][nblocks]
    float* cs = nullptr;
    float* sn = nullptr;
    int32_t* status = nullptr;       // device status word shared by all launches of this engine
    size_t page_bytes = 0;
    size_t elem_bytes = 0;
    int nb = 0, nblocks = 0;
    int kv_group = 0;
    int kv_shift = kKvShift;         // log2(tokens per page)
    alignas(128) unsigned char tmap_k[128];   // CUtensorMap of each fp16 pool (tensor-core attention)
    alignas(128) unsigned char tmap_v[128];
    alignas(128) unsigned char tmap_k1[128];  // one kv head per box (prefill)
    alignas(128) unsigned char tmap_v1[128];
    bool tmaps_ok = false;           // tmap_k / tmap_v (kv-group boxes) are valid: the tensor-core decode kernel can run
    bool tmaps1_ok = false;          // tmap_k1 / tmap_v1 (one kv head per box) too: prefill tiles, 8-token pages
    std::vector<SessionRec> sess;
    std::mutex mu;
};

struct nova_batch {
    nova_engine* e = nullptr;
    int n = 0;
    std::vector<int> sessions, slices;
    int32_t* d_slices = nullptr;
    int32_t* d_n_past = nullptr;
    int32_t* h_n_past = nullptr;     // pinned staging
    float* part = nullptr;
    int kernel = 0;                  // 0 SIMT, 1 tensor-core
    int fused = 0;                   // 1: RoPE+append done inside the tensor-core attention launch
    int pdl = 0;                     // 1: layers after the first of a step launch as programmatic dependents; 2: the same, but
                                     // they read their q / new k / new v only once the launches before them have finished
    int row_setup = 2;               // work-split weight of a row start, in pages (see AttnLaunch)
    int window = 0;                  // prefill: sliding window in tokens (0: plain causal)
    int prefill_tc5 = 1;             // 1: prefill attention on tcgen05 + tensor memory where it applies (attn_prefill_tc5.cu), 0: mma.sync tiles
    int split_ctas = 0;              // CTAs of a chained one-layer attention launch; 0: chosen from the work (pick_split_ctas)
    int cascade = 0;                 // 1: the shared leading pages of the batch's sessions are attended once for all
    int casc_pages = 0;              // shared leading pages found by the last nova_batch_cow (0: none worth it)
    float* xparts = nullptr;         // [S * NH][130] this rank's partial rows of one layer before they are exchanged
    float* casc_parts = nullptr;     // [chunks + 1][S * NH][130] partials of the cascade
    size_t casc_floats = 0;
    // staging for the host-buffer step and the graph replay
    float *dq = nullptr, *dk = nullptr, *dv = nullptr, *dout = nullptr;
    float *dq2 = nullptr, *dk2 = nullptr, *dv2 = nullptr, *dout2 = nullptr;   // second set: host-buffer steps alternate
    unsigned host_seq = 0;             // host-buffer steps issued so far (set = host_seq & 1)
    cudaGraphExec_t graph = nullptr;   // one per-layer decode step on the staging buffers
    int graph_kernel = -1;
    unsigned long long* timeline = nullptr;   // caller-owned profiling buffer, see nova_batch_set_timeline
    mutable unsigned tl_seq = 0;              // attention launches since the buffer was set (ring of 4 records)
    std::vector<cudaEvent_t> ev;       // event pool for per-launch timing
    cudaStream_t s_in = nullptr, s_out = nullptr;      // copy streams of the host-buffer step
    cudaEvent_t ev_in[4] = {}, ev_cmp[4] = {}, ev_out = nullptr;
    cudaEvent_t ev_free[2] = {}, ev_dl[2] = {};      // per staging set: its inputs consumed / its outputs downloaded
};

namespace {

int check_desc(const nova_engine_desc& d) {
    if (d.n_layers <= 0 || d.n_heads <= 0 || d.n_kv_heads <= 0 || d.n_slices <= 0 || d.ctx <= 0) return NOVA_ERR_INVALID;
    if (d.n_heads % d.n_kv_heads) return NOVA_ERR_INVALID;
    if (d.head_dim != kHeadDim || kv_shift_of_block(d.kv_block) < 0) return NOVA_ERR_UNSUPPORTED;
    if (d.kv_dtype != NOVA_KV_F32 && d.kv_dtype != NOVA_KV_F16) return NOVA_ERR_UNSUPPORTED;
    const int g = d.n_heads / d.n_kv_heads;
    if (!(g == 1 || g == 2 || (g >= 4 && g <= 8))) return NOVA_ERR_UNSUPPORTED;
    const int kvg = d.n_kv_heads < 4 ? d.n_kv_heads : 4;
    if (d.n_kv_heads % kvg) return NOVA_ERR_UNSUPPORTED;
    return NOVA_OK;
}

int kv_group_of(int n_kv_heads) { return n_kv_heads < 4 ? n_kv_heads : 4; }

SessionRec* session_of(nova_engine* e, int id) {
    if (!e || id < 0 || id >= (int)e->sess.size() || !e->sess[(size_t)id].used) return nullptr;
    return &e->sess[(size_t)id];
}
const SessionRec* session_of(const nova_engine* e, int id) {
    if (!e || id < 0 || id >= (int)e->sess.size() || !e->sess[(size_t)id].used) return nullptr;
    return &e->sess[(size_t)id];
}

int upload_table(nova_engine* e, int slice, cudaStream_t s) {
    const SliceState* st = e->pool.p.find(slice);
    if (!st) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaMemcpyAsync(e->tables + (size_t)slice * e->nblocks, st->table.data(),
                                  (size_t)e->nblocks * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    return NOVA_OK;
}

// KvPool::cow_slice for every logical block of [pos0, pos0+n), collecting the device copies.
int collect_cow(nova_engine* e, int slice, int64_t pos0, int n, std::vector<CowEvent>& ev) {
    if (n <= 0) return NOVA_OK;
    PagePool& pp = e->pool.p;
    const int b0 = pp.block_index(pos0), b1 = pp.block_index(pos0 + n - 1);
    for (int b = b0; b <= b1; ++b) {
        const int fresh = pp.cow(slice, (int64_t)b * pp.kv_block());
        if (fresh == -2) return NOVA_ERR_POOL_FULL;
        if (fresh < 0) continue;
        SliceState* st = pp.find(slice);
        CowEvent c;
        c.src = st->copy_from;
        c.dst = fresh;
        c.table_entry = e->tables + (size_t)slice * e->nblocks + b;
        st->copy_from = -1;                       // one-shot request consumed (src/model.cpp:175-176)
        ev.push_back(c);
    }
    return NOVA_OK;
}

void fill_attn(const nova_batch* b, AttnLaunch& a) {
    const nova_engine* e = b->e;
    std::memset(&a, 0, sizeof(a));
    a.pool_k = e->pool_k;
    a.pool_v = e->pool_v;
    a.table_base = e->tables;
    a.table_stride = e->nblocks;
    a.slice_ids = b->d_slices;
    a.n_past = b->d_n_past;
    a.keys_add = 1;
    a.part = b->part;
    a.status = e->status;
    a.n_sessions = b->n;
    a.nb = e->nb;
    a.n_heads = e->d.n_heads;
    a.n_kv_heads = e->d.n_kv_heads;
    a.kv_group = e->kv_group;
    a.kv_shift = e->kv_shift;
    a.page_lo = 0;
    a.page_hi = -1;
    a.row_setup_pages = b->row_setup;
    a.tmap_k = e->tmaps_ok ? e->tmap_k : nullptr;
    a.tmap_v = e->tmaps_ok ? e->tmap_v : nullptr;
    a.tmap_k1 = e->tmaps1_ok ? e->tmap_k1 : nullptr;
    a.tmap_v1 = e->tmaps1_ok ? e->tmap_v1 : nullptr;
    a.timeline = b->timeline ? b->timeline + (size_t)(b->tl_seq++ % 4u) * (kTimelineCtas * 12) : nullptr;
}

int pick_split_ctas(const nova_batch* b, const AttnLaunch& a);

// Split kernel, then the merge of the rows that more than one CTA worked on.
int run_attn(const nova_batch* b, const AttnLaunch& a, cudaStream_t s) {
    int rc, ctas;
    const bool f16 = b->e->d.kv_dtype == NOVA_KV_F16;
    if (b->kernel == 1 && f16 && a.n_q > 1 && a.n_layers == 1 && !a.write_partial_only) {
        // query-tiled prefill: every row complete in one CTA, no merge
        if (b->prefill_tc5 && attn_prefill_tc5_supports(a)) {
            // Longest context first: a CTA's work grows with its session's context, and the launch ends with the CTAs
            // that were handed out last (host positions, the same ones pick_split_ctas reads).
            AttnLaunch pa = a;
            const PagePool& pp = b->e->pool.p;
            if (b->n >= 2 && b->n <= 64 && a.n_sessions == b->n) {
                int64_t len[64];
                for (int i = 0; i < b->n; ++i) {
                    const SliceState* st = pp.find(b->slices[i]);
                    len[i] = st ? st->n_past : 0;
                    pa.sess_order[i] = (unsigned char)i;
                }
                std::stable_sort(pa.sess_order, pa.sess_order + b->n, [&](unsigned char x, unsigned char y) { return len[x] > len[y]; });
                pa.n_order = b->n;
            }
            return launch_attn_prefill_tc5(pa, s);
        }
        return launch_attn_prefill(a, s);
    }
    if (b->kernel == 1 && f16 && b->cascade && b->casc_pages > 0 && a.n_layers == 1 && a.n_q <= 1 && !a.write_partial_only &&
        a.page_lo == 0 && a.page_hi < 0) {
        // Cascade over a shared prefix: (1) all sessions' queries against the shared pages, read once, as
        // partials per page chunk; (2) the usual split over each session's own pages from the first private
        // page on, also as partials; (3) the merge kernel: split-K slots, then the chunks, then the output.
        const int P = b->casc_pages << (b->e->kv_shift > 4 ? b->e->kv_shift - 4 : 0);      // the shared pages as 16-key tiles
        const int rows = b->n * a.n_heads;
        // tcgen05 tiles (256 rows, a third of the SMs, the split runs beside them) where they apply, else mma.sync tiles
        AttnLaunch ta = a;
        ta.n_q = b->n;                // the sessions are the query rows of the prefix launch
        const bool tc5 = b->prefill_tc5 && attn_prefill_tc5_supports(ta);
        const int chunks = tc5 ? attn_prefix_tc5_chunks(b->n, a.n_heads, a.n_kv_heads, P, nullptr)
                               : attn_prefix_chunks(b->n, a.n_heads, a.n_kv_heads, P, nullptr);
        if ((size_t)(chunks + 1) * rows * kPartW > b->casc_floats) return NOVA_ERR_TOO_LARGE;
        AttnLaunch pa = a;
        pa.out_part = b->casc_parts;
        if (pa.timeline) pa.timeline += 4 * (size_t)(kTimelineCtas * 12);       // profiling build: records 4-7 are the prefix launches
        rc = tc5 ? launch_attn_prefix_tc5(pa, P, s) : launch_attn_prefix(pa, P, s);
        if (rc != NOVA_OK) return rc;
        AttnLaunch sa = a;
        sa.pdl_spare = 0;             // the chain here is prefix -> split -> merge -> final merge: early start only
        sa.page_lo = b->casc_pages;
        sa.write_partial_only = 1;
        sa.out_part = b->casc_parts + (size_t)chunks * rows * kPartW;
        sa.extra_parts = b->casc_parts;          // the merge kernel folds the chunks in and writes the output
        sa.n_extra = chunks;
        ctas = pick_split_ctas(b, sa);
        if (tc5) {
            // the prefix CTAs hold an SM each until they finish: the split takes the other SMs (an SM streams about as
            // fast with either kernel, so the two finish together when the SMs are shared out by bytes)
            const int tq5 = 256 / (a.n_heads / a.n_kv_heads);
            const int prefix_ctas = ((b->n + tq5 - 1) / tq5) * a.n_kv_heads * chunks;
            const int rest = sm_count() - prefix_ctas;
            if (rest >= sm_count() / 4 && rest < ctas) ctas = rest;
        }
        rc = launch_attn_mma(sa, b->e->d.kv_dtype, ctas, s);
        if (rc != NOVA_OK) return rc;
        return launch_attn_combine(sa, ctas, s);
    }
    if (b->kernel == 1 && (f16 || a.n_q <= 1)) {
        ctas = pick_split_ctas(b, a);
        rc = launch_attn_mma(a, b->e->d.kv_dtype, ctas, s);
    } else {
        ctas = attn_split_ctas_simt(a, 0);
        rc = launch_attn_simt(a, b->e->d.kv_dtype, ctas, s);
    }
    if (rc != NOVA_OK) return rc;
    return launch_attn_combine(a, ctas, s);
}

bool use_fused(const nova_batch* b) { return b->fused && b->kernel == 1 && b->e->d.rope_neox; }

// CTAs of one tensor-core attention launch.  A launch of a programmatic chain (one layer per launch) that has
// little to stream - fewer than 16 pages per CTA, so that a CTA's start-up outweighs its streaming - takes only
// half (or a third) of the SMs: consecutive layers then run side by side on different SMs, one starting up (positions, work
// split, first table entries, first pages) while the other streams or waits for the launch before it.
int pick_split_ctas(const nova_batch* b, const AttnLaunch& a) {
    const int all = attn_split_ctas_mma(a, 0);
    if (b->split_ctas > 0) return b->split_ctas < all ? b->split_ctas : all;
    if (!(a.pdl && a.pdl_spare && a.n_layers == 1 && a.n_q <= 1)) return all;
    const PagePool& pp = b->e->pool.p;
    int64_t pages = 0;
    for (int slice : b->slices) {
        const SliceState* st = pp.find(slice);
        if (!st) continue;
        // in tiles of min(16, page) keys, as the kernels count them
        const int ts = b->e->kv_shift < 4 ? b->e->kv_shift : 4, tpp = b->e->kv_shift - ts;
        int64_t total = (st->n_past + 1 + (1 << ts) - 1) >> ts;
        const int64_t lo = a.page_lo > 0 ? (a.page_lo << tpp) : 0;
        const int64_t hi = (a.page_hi >= 0 && (a.page_hi << tpp) < total) ? (a.page_hi << tpp) : total;
        if (hi > lo) pages += hi - lo;
    }
    pages *= a.n_kv_heads / a.kv_group;
    const int per_sm = a.kv_group >= 4 ? 1 : 4 / a.kv_group;
    const int half = (sm_count() / 2) * per_sm, third = (sm_count() / 3) * per_sm;
    // measured on one 7B-shaped session (per layer): 1024 pages 8.7-9.4 us with 37-56 CTAs, 9.5 with 74, 11.8 with 136;
    // 2048 pages 14.3 with 74 or 136; 4096 pages 24.5 with 74, 23.0 with 136
    // a handful of pages (one short session): a CTA per four pages, at least eight - the merge then has few partial slots
    // to fold (1.5B shape, 1 x 1024 tokens = 64 pages per layer: 0.180 ms per step with 64 CTAs, 0.167 with 16)
    if (pages <= 128) {
        int few = (int)(pages / 4);
        if (few < 8) few = 8;
        if (few > third) few = third;
        return few < all ? few : all;
    }
    if (pages < (int64_t)all * 8) return third < all ? third : all;
    return pages < (int64_t)all * 16 ? (half < all ? half : all) : all;
}

// RopeKvOp + AttnOp for layers [layer0, layer0 + n_layers) in one split launch (+ combine):
// k rotated in place and appended with v, q read un-rotated and left as it is.
int run_attn_fused(const nova_batch* b, int layer0, int n_layers, const float* q, float* k, const float* v,
                   float* out, cudaStream_t s, bool pdl = false, float* out_part = nullptr, int64_t page_lo = 0,
                   int64_t page_hi = -1) {
    const nova_engine* e = b->e;
    AttnLaunch a;
    fill_attn(b, a);
    a.q = q; a.out = out;
    if (out_part) {                       // un-normalised partials over the page window [page_lo, page_hi)
        a.out_part = out_part;
        a.write_partial_only = 1;
        a.page_lo = page_lo;
        a.page_hi = page_hi;
    }
    a.layer0 = layer0; a.n_layers = n_layers;
    a.fuse_append = 1;
    a.pool_k_w = e->pool_k; a.pool_v_w = e->pool_v;
    a.k_new = k; a.v_new = v;
    a.rope_cs = e->cs; a.rope_sn = e->sn; a.rope_rows = e->d.rope_positions;
    a.pdl = pdl ? (b->pdl == 2 ? 2 : 1) : 0;
    a.pdl_spare = a.pdl != 0;
    return run_attn(b, a, s);
}

void fill_append(const nova_batch* b, AppendLaunch& a) {
    const nova_engine* e = b->e;
    std::memset(&a, 0, sizeof(a));
    a.pool_k = e->pool_k;
    a.pool_v = e->pool_v;
    a.table_base = e->tables;
    a.table_stride = e->nblocks;
    a.kv_shift = e->kv_shift;
    a.slice_ids = b->d_slices;
    a.n_past = b->d_n_past;
    a.cs = e->cs;
    a.sn = e->sn;
    a.rope_rows = e->d.rope_positions;
    a.status = e->status;
    a.n_sessions = b->n;
    a.n_tok = 1;
    a.nb = e->nb;
    a.n_heads = e->d.n_heads;
    a.n_kv_heads = e->d.n_kv_heads;
    a.neox = e->d.rope_neox;
    a.kv_dtype = e->d.kv_dtype;
}

}  // namespace

extern "C" {

int nova_engine_create(const nova_engine_desc* desc, nova_engine** out) {
    if (!desc || !out) return NOVA_ERR_INVALID;
    *out = nullptr;
    nova_engine_desc d = *desc;
    if (d.max_sessions <= 0 || d.max_sessions > d.n_slices) d.max_sessions = d.n_slices;
    if (d.rope_positions <= 0) d.rope_positions = d.ctx;
    const int rc = check_desc(d);
    if (rc != NOVA_OK) return rc;
    NOVA_CUDA_TRY(cudaSetDevice(d.device));

    nova_engine* e = new (std::nothrow) nova_engine();
    if (!e) return NOVA_ERR_INVALID;
    e->d = d;
    e->pool.p.set_block(d.kv_block);
    const int64_t nblocks = (d.ctx + d.kv_block - 1) / d.kv_block;
    if (nblocks * d.n_slices > 0x7fffffffLL) { delete e; return NOVA_ERR_TOO_LARGE; }
    e->pool.p.init(d.n_slices, d.ctx);
    e->nblocks = e->pool.p.nblocks();
    e->nb = e->pool.p.nb_total();
    e->elem_bytes = d.kv_dtype == NOVA_KV_F16 ? 2 : 4;
    e->page_bytes = (size_t)d.kv_block * d.n_kv_heads * d.head_dim * e->elem_bytes;
    e->kv_group = kv_group_of(d.n_kv_heads);
    e->kv_shift = kv_shift_of_block(d.kv_block);
    e->sess.resize((size_t)d.max_sessions);

    const size_t pool_bytes = (size_t)d.n_layers * (size_t)e->nb * e->page_bytes;
    const size_t rope_bytes = (size_t)d.rope_positions * (kHeadDim / 2) * sizeof(float);
    cudaError_t ce = cudaSuccess;
    if (ce == cudaSuccess) ce = cudaMalloc(&e->pool_k, pool_bytes);
    if (ce == cudaSuccess) ce = cudaMalloc(&e->pool_v, pool_bytes);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&e->tables, (size_t)d.n_slices * e->nblocks * sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&e->cs, rope_bytes);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&e->sn, rope_bytes);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&e->status, sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMemset(e->status, 0, sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMemset(e->tables, 0xff, (size_t)d.n_slices * e->nblocks * sizeof(int32_t));
    if (ce != cudaSuccess) {
        set_cuda_error(ce, "engine allocation");
        nova_engine_destroy(e);
        return NOVA_ERR_CUDA;
    }
    if (d.kv_dtype == NOVA_KV_F16 && attn_mma_built()) {
        const int64_t slot_rows = (int64_t)d.n_layers * e->nb * d.kv_block;
        const int box_rows = d.kv_block < kTileKeysMax ? d.kv_block : kTileKeysMax;      // a tile of the page
        e->tmaps_ok = attn_make_tmap(e->tmap_k, e->pool_k, slot_rows, d.n_kv_heads, e->kv_group, box_rows, 2) == NOVA_OK &&
                      attn_make_tmap(e->tmap_v, e->pool_v, slot_rows, d.n_kv_heads, e->kv_group, box_rows, 2) == NOVA_OK &&
                      attn_make_tmap(e->tmap_k1, e->pool_k, slot_rows, d.n_kv_heads, 1, box_rows, 2) == NOVA_OK &&
                      attn_make_tmap(e->tmap_v1, e->pool_v, slot_rows, d.n_kv_heads, 1, box_rows, 2) == NOVA_OK;
        e->tmaps1_ok = e->tmaps_ok;
    } else if (d.kv_dtype == NOVA_KV_F32 && attn_mma_built() && d.kv_block == kTileKeysMax) {
        // fp32 pools through the tensor-core decode kernel (rows converted to fp16 on the way in): boxes of 32 dims
        const int64_t slot_rows = (int64_t)d.n_layers * e->nb * d.kv_block;
        e->tmaps_ok = attn_make_tmap(e->tmap_k, e->pool_k, slot_rows, d.n_kv_heads, e->kv_group, kTileKeysMax, 4) == NOVA_OK &&
                      attn_make_tmap(e->tmap_v, e->pool_v, slot_rows, d.n_kv_heads, e->kv_group, kTileKeysMax, 4) == NOVA_OK;
    }
    int r = launch_rope_table(e->cs, e->sn, d.rope_positions, d.rope_theta, 0);   // Kernel::rope_table, model.cpp:119
    if (r == NOVA_OK && cudaDeviceSynchronize() != cudaSuccess) r = NOVA_ERR_CUDA;
    if (r != NOVA_OK) {
        nova_engine_destroy(e);
        return r;
    }
    *out = e;
    return NOVA_OK;
}

void nova_engine_destroy(nova_engine* e) {
    if (!e) return;
    cudaSetDevice(e->d.device);
    for (auto& s : e->sess)
        if (s.used && s.stream) cudaStreamDestroy(s.stream);
    cudaFree(e->pool_k);
    cudaFree(e->pool_v);
    cudaFree(e->tables);
    cudaFree(e->cs);
    cudaFree(e->sn);
    cudaFree(e->status);
    delete e;
}

int nova_engine_desc_get(const nova_engine* e, nova_engine_desc* out) {
    if (!e || !out) return NOVA_ERR_INVALID;
    *out = e->d;
    return NOVA_OK;
}

void* nova_kv_k_base(const nova_engine* e) { return e ? e->pool_k : nullptr; }
void* nova_kv_v_base(const nova_engine* e) { return e ? e->pool_v : nullptr; }
int32_t* nova_kv_table_slot(const nova_engine* e, int slice) {
    if (!e || slice < 0 || slice >= e->d.n_slices) return nullptr;
    return e->tables + (size_t)slice * e->nblocks;
}
int nova_kv_nb(const nova_engine* e) { return e ? e->nb : 0; }
int nova_kv_nblocks(const nova_engine* e) { return e ? e->nblocks : 0; }
int nova_kv_width(const nova_engine* e) { return e ? e->d.n_kv_heads * e->d.head_dim : 0; }
size_t nova_kv_page_bytes(const nova_engine* e) { return e ? e->page_bytes : 0; }
const float* nova_rope_cos(const nova_engine* e) { return e ? e->cs : nullptr; }
const float* nova_rope_sin(const nova_engine* e) { return e ? e->sn : nullptr; }
nova_pool* nova_engine_pool(nova_engine* e) { return e ? &e->pool : nullptr; }

int nova_session_create(nova_engine* e) {
    if (!e) return NOVA_ERR_INVALID;
    std::lock_guard<std::mutex> lk(e->mu);
    int slot = -1;
    for (size_t i = 0; i < e->sess.size(); ++i)
        if (!e->sess[i].used) { slot = (int)i; break; }
    if (slot < 0) return NOVA_ERR_NO_SESSION;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    // KvPool::acquire resets the count of every identity page of the slice it hands out.  While another live
    // session still maps one of them (a fork whose parent was destroyed, a copy-on-write page taken from this
    // slice while it was free) the two would write the same pages unnoticed: refuse instead.
    const int next = e->pool.p.next_slice();
    if (next < 0) return NOVA_ERR_NO_SLICE;
    if (e->pool.p.foreign_mappings(next) > 0) return NOVA_ERR_BUSY;
    const int slice = e->pool.p.acquire();
    if (slice < 0) return NOVA_ERR_NO_SLICE;
    cudaStream_t st = nullptr;
    cudaError_t ce = cudaStreamCreate(&st);
    if (ce != cudaSuccess) {
        set_cuda_error(ce, "cudaStreamCreate");
        e->pool.p.release(slice);
        return NOVA_ERR_CUDA;
    }
    int rc = upload_table(e, slice, st);
    if (rc == NOVA_OK && e->d.zero_pages)
        rc = launch_zero_pages(e->pool_k, e->pool_v, e->d.n_layers, e->nb, e->page_bytes,
                               e->tables + (size_t)slice * e->nblocks, e->nblocks, st);
    if (rc == NOVA_OK) {
        ce = cudaStreamSynchronize(st);
        if (ce != cudaSuccess) {
            set_cuda_error(ce, "cudaStreamSynchronize");
            rc = NOVA_ERR_CUDA;
        }
    }
    if (rc != NOVA_OK) {               // leave nothing behind: the slice, the stream and the slot stay free
        cudaStreamDestroy(st);
        e->pool.p.release(slice);
        return rc;
    }
    SessionRec& r = e->sess[(size_t)slot];
    r.used = true;
    r.slice = slice;
    r.stream = st;
    return slot;
}

int nova_session_destroy(nova_engine* e, int session) {
    if (!e) return NOVA_ERR_INVALID;
    std::lock_guard<std::mutex> lk(e->mu);
    SessionRec* r = session_of(e, session);
    if (!r) return NOVA_ERR_INVALID;
    cudaStreamDestroy(r->stream);
    e->pool.p.release(r->slice);
    *r = SessionRec{};
    return NOVA_OK;
}

int nova_session_live_count(nova_engine* e) {
    if (!e) return 0;
    std::lock_guard<std::mutex> lk(e->mu);
    int n = 0;
    for (const auto& s : e->sess) n += s.used ? 1 : 0;
    return n;
}
int nova_session_slice(const nova_engine* e, int session) {
    const SessionRec* r = session_of(e, session);
    return r ? r->slice : NOVA_ERR_INVALID;
}
nova_stream_t nova_session_stream(const nova_engine* e, int session) {
    const SessionRec* r = session_of(e, session);
    return r ? (nova_stream_t)r->stream : nullptr;
}
int64_t nova_session_n_past(const nova_engine* e, int session) {
    const SessionRec* r = session_of(e, session);
    if (!r) return -1;
    const SliceState* st = e->pool.p.find(r->slice);
    return st ? st->n_past : -1;
}
int nova_session_set_n_past(nova_engine* e, int session, int64_t n_past) {
    SessionRec* r = session_of(e, session);
    if (!r || n_past < 0) return NOVA_ERR_INVALID;
    SliceState* st = e->pool.p.find(r->slice);
    if (!st) return NOVA_ERR_INVALID;
    st->n_past = n_past;
    return NOVA_OK;
}

int nova_session_attach(nova_engine* e, int dst, int src, int k) {
    SessionRec *d = session_of(e, dst), *s = session_of(e, src);
    if (!d || !s) return NOVA_ERR_INVALID;
    if (!e->pool.p.attach(d->slice, s->slice, k)) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    const int rc = upload_table(e, d->slice, d->stream);
    if (rc != NOVA_OK) return rc;
    NOVA_CUDA_TRY(cudaStreamSynchronize(d->stream));
    return NOVA_OK;
}

int nova_session_attach_prefix(nova_engine* e, int dst, int src, int64_t n_tokens) {
    SessionRec *d = session_of(e, dst), *s = session_of(e, src);
    if (!d || !s) return NOVA_ERR_INVALID;
    if (!e->pool.p.attach_prefix(d->slice, s->slice, n_tokens)) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    const int rc = upload_table(e, d->slice, d->stream);
    if (rc != NOVA_OK) return rc;
    NOVA_CUDA_TRY(cudaStreamSynchronize(d->stream));
    return NOVA_OK;
}

int nova_session_fork(nova_engine* e, int src) {
    const SessionRec* s = session_of(e, src);
    if (!s) return NOVA_ERR_INVALID;
    const SliceState* st = e->pool.p.find(s->slice);
    if (!st || st->n_past <= 0) return NOVA_ERR_INVALID;
    const int64_t tokens = st->n_past;
    const int dst = nova_session_create(e);
    if (dst < 0) return dst;
    const int rc = nova_session_attach_prefix(e, dst, src, tokens);
    if (rc != NOVA_OK) {
        nova_session_destroy(e, dst);
        return rc;
    }
    return dst;
}

int64_t nova_session_attach_block(nova_engine* e, const nova_registry* r, uint64_t prefix, uint64_t suffix, int dst) {
    if (!e || !r || !session_of(e, dst)) return NOVA_ERR_INVALID;
    nova_kv_block blk;
    if (!nova_registry_find(r, prefix, suffix, &blk)) return 0;
    if (blk.session == dst || blk.pos1 <= 0) return 0;
    const SessionRec* src = session_of(e, blk.session);
    if (!src) return 0;                                  // the producing session has been closed
    const SliceState* st = e->pool.p.find(src->slice);
    if (!st || st->n_past < blk.pos1) return 0;          // ... or re-used for something shorter
    const int rc = nova_session_attach_prefix(e, dst, blk.session, blk.pos1);
    return rc == NOVA_OK ? blk.pos1 : (int64_t)rc;
}

int nova_engine_telemetry(const nova_engine* e, nova_telemetry* out) {
    if (!e || !out) return NOVA_ERR_INVALID;
    const PagePool& pp = e->pool.p;
    std::memset(out, 0, sizeof(*out));
    out->blocks_total = pp.nb_total();
    out->blocks_free = pp.free_pages();
    int shared = 0;
    for (int r : pp.refs()) shared += r > 1;
    out->blocks_shared = shared;
    out->cow_count = pp.cow_count();
    out->slices_free = pp.free_slices();
    int live = 0;
    for (const SessionRec& s : e->sess) live += s.used ? 1 : 0;
    out->sessions_live = live;
    const uint64_t per_page = (uint64_t)e->page_bytes * 2ull * (uint64_t)e->d.n_layers;
    out->kv_bytes_cap = per_page * (uint64_t)pp.nb_total();
    out->kv_bytes_used = per_page * (uint64_t)(pp.nb_total() - pp.free_pages());
    return NOVA_OK;
}

int nova_session_cow_on(nova_engine* e, int session, int64_t pos0, int n, nova_stream_t stream) {
    SessionRec* r = session_of(e, session);
    if (!r || pos0 < 0) return NOVA_ERR_INVALID;
    std::vector<CowEvent> ev;
    const int rc = collect_cow(e, r->slice, pos0, n, ev);
    if (!ev.empty()) {
        NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
        const int lrc = launch_cow_copy(e->pool_k, e->pool_v, e->d.n_layers, e->nb, e->page_bytes, ev.data(),
                                        (int)ev.size(), (cudaStream_t)stream);
        if (lrc != NOVA_OK) return lrc;
    }
    return rc != NOVA_OK ? rc : (int)ev.size();
}

int nova_session_cow(nova_engine* e, int session, int64_t pos0, int n) {
    const SessionRec* r = session_of(e, session);
    if (!r) return NOVA_ERR_INVALID;
    return nova_session_cow_on(e, session, pos0, n, (nova_stream_t)r->stream);
}

int nova_session_permute_pages(nova_engine* e, int session, const int32_t* perm, int n) {
    SessionRec* r = session_of(e, session);
    if (!r || !perm || n != e->nblocks) return NOVA_ERR_INVALID;
    std::vector<char> seen((size_t)n, 0);
    for (int i = 0; i < n; ++i) {
        if (perm[i] < 0 || perm[i] >= n || seen[(size_t)perm[i]]) return NOVA_ERR_INVALID;
        seen[(size_t)perm[i]] = 1;
    }
    SliceState* st = e->pool.p.find(r->slice);
    const int first = r->slice * e->nblocks;
    for (int i = 0; i < n; ++i) {
        // only a table that still maps onto the slice's own pages may be permuted
        const int cur = st->table[(size_t)i];
        if (cur < first || cur >= first + n) return NOVA_ERR_INVALID;
    }
    for (int i = 0; i < n; ++i) st->table[(size_t)i] = first + perm[i];
    return nova_session_sync_table(e, session);
}

int nova_session_sync_table(nova_engine* e, int session) {
    SessionRec* r = session_of(e, session);
    if (!r) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    const int rc = upload_table(e, r->slice, r->stream);
    if (rc != NOVA_OK) return rc;
    NOVA_CUDA_TRY(cudaStreamSynchronize(r->stream));
    return NOVA_OK;
}

/* ------------------------------------------------------------- raw launchers */

int nova_launch_rope_table(float* cs, float* sn, int64_t n_pos, int32_t head_dim, int32_t theta, nova_stream_t s) {
    if (head_dim != kHeadDim) return NOVA_ERR_UNSUPPORTED;
    return launch_rope_table(cs, sn, n_pos, theta, (cudaStream_t)s);
}

int nova_launch_rope_append_paged(const nova_kv_shape* sh, void* pool_k, void* pool_v, const int32_t* table,
                                  int layer, int nb, int n, int64_t pos0, float* q, float* k, const float* v,
                                  const float* cs, const float* sn, nova_stream_t s) {
    if (!sh || !pool_k || !pool_v || !table || !k || !v || !cs || !sn || layer < 0 || nb <= 0 || pos0 < 0)
        return NOVA_ERR_INVALID;
    if (sh->head_dim != kHeadDim || kv_shift_of_block(sh->kv_block) < 0) return NOVA_ERR_UNSUPPORTED;
    AppendLaunch a;
    std::memset(&a, 0, sizeof(a));
    a.pool_k = pool_k; a.pool_v = pool_v;
    a.kv_shift = kv_shift_of_block(sh->kv_block);
    a.table_base = table;
    a.table_stride = std::numeric_limits<int32_t>::max();   // the caller vouches for the table length, as in the reference
    a.pos_imm = pos0;
    a.q = q; a.k = k; a.v = v; a.cs = cs; a.sn = sn;
    a.rope_rows = std::numeric_limits<int64_t>::max();
    a.n_sessions = 1; a.n_tok = n; a.layer0 = layer; a.n_layers = 1; a.nb = nb;
    a.n_heads = sh->n_heads; a.n_kv_heads = sh->n_kv_heads; a.neox = sh->rope_neox; a.kv_dtype = sh->kv_dtype;
    return launch_rope_append(a, (cudaStream_t)s);
}

size_t nova_attn_scratch_floats(const nova_kv_shape* sh) {
    return sh ? (size_t)sh->n_heads * 32 * (size_t)(sh->head_dim + 2) : 0;
}

// The literal launchers have no engine behind them, so the tensor maps of the pools they are given are kept here,
// one per (pool, element type, kv heads, rows covered): a map is encoded once and found again by a short scan.
namespace {
struct RawMap {
    const void* pool;
    int kv_dtype, n_kv_heads, kv_group;
    int64_t slot_rows;
    alignas(128) unsigned char map[128];
};
std::mutex g_raw_mu;
std::vector<RawMap*> g_raw_maps;
std::atomic<int> g_raw_kernel{0};

const void* raw_tmap(const void* pool, int kv_dtype, int n_kv_heads, int kv_group, int64_t slot_rows) {
    std::lock_guard<std::mutex> lk(g_raw_mu);
    for (RawMap* m : g_raw_maps)
        if (m->pool == pool && m->kv_dtype == kv_dtype && m->n_kv_heads == n_kv_heads && m->kv_group == kv_group && m->slot_rows >= slot_rows)
            return m->map;
    if (g_raw_maps.size() >= 4096) return nullptr;          // a caller that keeps changing pools: stay on the SIMT kernel
    RawMap* m = new (std::nothrow) RawMap;
    if (!m) return nullptr;
    m->pool = pool; m->kv_dtype = kv_dtype; m->n_kv_heads = n_kv_heads; m->kv_group = kv_group; m->slot_rows = slot_rows;
    if (attn_make_tmap(m->map, const_cast<void*>(pool), slot_rows, n_kv_heads, kv_group, kTileKeysMax, kv_dtype == NOVA_KV_F16 ? 2 : 4) != NOVA_OK) {
        delete m;
        return nullptr;
    }
    g_raw_maps.push_back(m);
    return m->map;
}
}  // namespace

int nova_launcher_set_kernel(int which) {
    if (which < 0 || which > 1) return NOVA_ERR_INVALID;
    if (which == 1 && !attn_mma_built()) return NOVA_ERR_UNSUPPORTED;
    g_raw_kernel.store(which);
    return NOVA_OK;
}

int nova_launch_attn_decode_paged(const nova_kv_shape* sh, const float* q, const void* pool_k, const void* pool_v,
                                  const int32_t* table, int layer, int nb, int n_keys, float* o, float* scratch,
                                  nova_stream_t s) {
    if (!sh || !q || !pool_k || !pool_v || !table || !o || !scratch || layer < 0 || nb <= 0) return NOVA_ERR_INVALID;
    if (sh->head_dim != kHeadDim || kv_shift_of_block(sh->kv_block) < 0) return NOVA_ERR_UNSUPPORTED;
    if (sh->n_kv_heads <= 0 || sh->n_heads % sh->n_kv_heads) return NOVA_ERR_INVALID;
    AttnLaunch a;
    std::memset(&a, 0, sizeof(a));
    a.pool_k = pool_k; a.pool_v = pool_v;
    a.kv_shift = kv_shift_of_block(sh->kv_block);
    a.table_base = table;
    a.table_stride = std::numeric_limits<int32_t>::max();
    a.keys_imm = n_keys;
    a.q = q; a.out = o; a.part = scratch;
    a.n_sessions = 1; a.layer0 = layer; a.n_layers = 1; a.nb = nb;
    a.n_heads = sh->n_heads; a.n_kv_heads = sh->n_kv_heads;
    a.kv_group = kv_group_of(sh->n_kv_heads);
    a.page_lo = 0; a.page_hi = -1;
    // The caller's scratch (NH*32*(HD+2) floats) holds so many partial slots; slot index = cta + row.
    const int heads_per_row = a.kv_group * (sh->n_heads / sh->n_kv_heads);
    const int rows = sh->n_kv_heads / a.kv_group;
    int ctas = (int)(nova_attn_scratch_floats(sh) / ((size_t)heads_per_row * kSlotW)) - rows;
    if (ctas < 1) return NOVA_ERR_UNSUPPORTED;
    if (g_raw_kernel.load() == 1 && a.kv_shift == 4 && sh->n_heads / sh->n_kv_heads <= 8) {
        // tensor-core kernel (nova_launcher_set_kernel): the pools' maps cover the rows up to this layer's last page
        const int64_t slot_rows = (int64_t)(layer + 1) * nb * sh->kv_block;
        a.tmap_k = raw_tmap(pool_k, sh->kv_dtype, sh->n_kv_heads, a.kv_group, slot_rows);
        a.tmap_v = raw_tmap(pool_v, sh->kv_dtype, sh->n_kv_heads, a.kv_group, slot_rows);
        if (a.tmap_k && a.tmap_v) {
            const int all = attn_split_ctas_mma(a, 0);
            const int c = ctas < all ? ctas : all;
            int rc = launch_attn_mma(a, sh->kv_dtype, c, (cudaStream_t)s);
            if (rc == NOVA_OK) return launch_attn_combine(a, c, (cudaStream_t)s);
            if (rc != NOVA_ERR_UNSUPPORTED) return rc;
        }
        a.tmap_k = a.tmap_v = nullptr;
    }
    const int want = attn_default_ctas_simt(sh->n_kv_heads);
    if (ctas > want) ctas = want;
    int rc = launch_attn_simt(a, sh->kv_dtype, ctas, (cudaStream_t)s);
    if (rc != NOVA_OK) return rc;
    return launch_attn_combine(a, ctas, (cudaStream_t)s);
}

// Declared in nova_b200_testing.h: the two literal launchers for n sessions of a layer, in the reference's call order.
int nova_launch_decode_layer_sessions(const nova_kv_shape* sh, int n, void* pool_k, void* pool_v, const int32_t* const* tables,
                                      int layer, int nb, const int64_t* pos, float* q, float* k, const float* v, size_t q_stride,
                                      size_t kv_stride, const float* cs, const float* sn, float* o, float* scratch,
                                      nova_stream_t s) {
    if (!sh || n < 0 || !tables || !pos || !q || !k || !v || !o) return NOVA_ERR_INVALID;
    for (int i = 0; i < n; ++i) {
        float* qi = q + (size_t)i * q_stride;
        float* ki = k + (size_t)i * kv_stride;
        int rc = nova_launch_rope_append_paged(sh, pool_k, pool_v, tables[i], layer, nb, 1, pos[i], qi, ki, v + (size_t)i * kv_stride,
                                               cs, sn, s);
        if (rc != NOVA_OK) return rc;
        rc = nova_launch_attn_decode_paged(sh, qi, pool_k, pool_v, tables[i], layer, nb, (int)pos[i] + 1, o + (size_t)i * q_stride,
                                           scratch, s);
        if (rc != NOVA_OK) return rc;
    }
    return NOVA_OK;
}

int nova_lse_combine(const float* parts, int n_parts, int n_rows, int head_dim, float* out, nova_stream_t s) {
    if (!parts || !out || head_dim != kHeadDim) return NOVA_ERR_INVALID;
    return launch_lse_combine(parts, n_parts, n_rows, out, (cudaStream_t)s);
}

size_t nova_peer_slot_bytes(int n_rows) {
    if (n_rows <= 0) return 0;
    return (size_t)kMaxPeerRanks * peer_region_bytes(n_rows);
}

int nova_lse_merge_peers(const float* part, void* const* peer_base, int n_ranks, int my_rank, size_t slot_bytes, int slot,
                         int n_rows, int64_t epoch, int timeout_ms, float* out, int32_t* status, nova_stream_t s) {
    if (!part || !peer_base || !out || n_ranks < 1 || n_ranks > kMaxPeerRanks || my_rank < 0 || my_rank >= n_ranks || slot < 0 ||
        n_rows < 0 || epoch < 1 || epoch > 0x7fffffffLL || timeout_ms < 1 || slot_bytes < nova_peer_slot_bytes(n_rows) ||
        slot_bytes % 128)
        return NOVA_ERR_INVALID;
    void* base[kMaxPeerRanks];
    for (int i = 0; i < n_ranks; ++i) {
        if (!peer_base[i]) return NOVA_ERR_INVALID;
        base[i] = static_cast<unsigned char*>(peer_base[i]) + (size_t)slot * slot_bytes;
    }
    return launch_lse_exchange(part, base, n_ranks, my_rank, n_rows, (long long)epoch,
                               (unsigned long long)timeout_ms * 1000000ull, out, status, (cudaStream_t)s);
}

/* ------------------------------------------------------------------- batches */

int nova_batch_create(nova_engine* e, const int32_t* sessions, int n, nova_batch** out) {
    if (!e || !sessions || n <= 0 || !out) return NOVA_ERR_INVALID;
    *out = nullptr;
    if ((int64_t)n * (e->d.n_kv_heads / e->kv_group) > kMaxRowsSmem) return NOVA_ERR_TOO_LARGE;
    nova_batch* b = new (std::nothrow) nova_batch();
    if (!b) return NOVA_ERR_INVALID;
    b->e = e;
    b->n = n;
    for (int i = 0; i < n; ++i) {
        const SessionRec* r = session_of(e, sessions[i]);
        if (!r) { delete b; return NOVA_ERR_INVALID; }
        b->sessions.push_back(sessions[i]);
        b->slices.push_back(r->slice);
    }
    {
        const cudaError_t de = cudaSetDevice(e->d.device);
        if (de != cudaSuccess) {
            set_cuda_error(de, "cudaSetDevice");
            delete b;
            return NOVA_ERR_CUDA;
        }
    }
    const int64_t rows = (int64_t)e->d.n_layers * n * (e->d.n_kv_heads / e->kv_group);
    const int heads_per_row = e->kv_group * (e->d.n_heads / e->d.n_kv_heads);
    const int64_t rows_alloc = rows > kMaxRowsSmem ? rows : kMaxRowsSmem;   // a prefill launch has up to kMaxRowsSmem rows
    const size_t part_floats = (size_t)(rows_alloc + kMaxSplitCtas) * heads_per_row * kSlotW;
    cudaError_t ce = cudaSuccess;
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->d_slices, (size_t)n * sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->d_n_past, (size_t)n * sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMallocHost((void**)&b->h_n_past, (size_t)n * sizeof(int32_t));
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->part, part_floats * sizeof(float));
    if (ce == cudaSuccess)
        ce = cudaMemcpy(b->d_slices, b->slices.data(), (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) {
        set_cuda_error(ce, "batch allocation");
        nova_batch_destroy(b);
        return NOVA_ERR_CUDA;
    }
    const int rc = nova_batch_sync_positions(b, nullptr);
    if (rc != NOVA_OK || cudaDeviceSynchronize() != cudaSuccess) {
        nova_batch_destroy(b);
        return rc != NOVA_OK ? rc : NOVA_ERR_CUDA;
    }
    *out = b;
    return NOVA_OK;
}

void nova_batch_destroy(nova_batch* b) {
    if (!b) return;
    cudaSetDevice(b->e->d.device);
    cudaFree(b->d_slices);
    cudaFree(b->d_n_past);
    cudaFreeHost(b->h_n_past);
    cudaFree(b->part);
    cudaFree(b->casc_parts);
    cudaFree(b->xparts);
    cudaFree(b->dq);
    cudaFree(b->dk);
    cudaFree(b->dv);
    cudaFree(b->dout);
    cudaFree(b->dq2);
    cudaFree(b->dk2);
    cudaFree(b->dv2);
    cudaFree(b->dout2);
    if (b->graph) cudaGraphExecDestroy(b->graph);
    for (cudaEvent_t e : b->ev) cudaEventDestroy(e);
    for (int i = 0; i < 4; ++i) {
        if (b->ev_in[i]) cudaEventDestroy(b->ev_in[i]);
        if (b->ev_cmp[i]) cudaEventDestroy(b->ev_cmp[i]);
    }
    if (b->ev_out) cudaEventDestroy(b->ev_out);
    for (int i = 0; i < 2; ++i) {
        if (b->ev_free[i]) cudaEventDestroy(b->ev_free[i]);
        if (b->ev_dl[i]) cudaEventDestroy(b->ev_dl[i]);
    }
    if (b->s_in) cudaStreamDestroy(b->s_in);
    if (b->s_out) cudaStreamDestroy(b->s_out);
    delete b;
}

int nova_batch_size(const nova_batch* b) { return b ? b->n : 0; }

int nova_batch_sync_positions(nova_batch* b, nova_stream_t s) {
    if (!b) return NOVA_ERR_INVALID;
    for (int i = 0; i < b->n; ++i) {
        const SliceState* st = b->e->pool.p.find(b->slices[(size_t)i]);
        if (!st || st->n_past > 0x7ffffff0LL) return NOVA_ERR_INVALID;
        b->h_n_past[i] = (int32_t)st->n_past;
    }
    NOVA_CUDA_TRY(cudaMemcpyAsync(b->d_n_past, b->h_n_past, (size_t)b->n * sizeof(int32_t), cudaMemcpyHostToDevice,
                                  (cudaStream_t)s));
    return NOVA_OK;
}

int nova_batch_set_kernel(nova_batch* b, int which) {
    if (!b || which < 0 || which > 1) return NOVA_ERR_INVALID;
    if (which == 1 && !b->e->tmaps_ok) return NOVA_ERR_UNSUPPORTED;      // (fp32 pools: 16-token pages only)
    b->kernel = which;
    if (which != 1) b->fused = 0;
    return NOVA_OK;
}
int nova_batch_set_timeline(nova_batch* b, void* dev_buf) {
    if (!b) return NOVA_ERR_INVALID;
#ifdef NOVA_TIMELINE
    b->timeline = static_cast<unsigned long long*>(dev_buf);
    b->tl_seq = 0;
    return NOVA_OK;
#else
    (void)dev_buf;
    return NOVA_ERR_UNSUPPORTED;      // the kernels carry the time stamps only in a -DNOVA_TIMELINE build
#endif
}
int nova_batch_set_fused_append(nova_batch* b, int on) {
    if (!b) return NOVA_ERR_INVALID;
    if (on && (b->kernel != 1 || !b->e->d.rope_neox)) return NOVA_ERR_UNSUPPORTED;
    b->fused = on ? 1 : 0;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    return NOVA_OK;
}
int nova_batch_set_row_setup_pages(nova_batch* b, int pages) {
    if (!b || pages < 0 || pages > 64) return NOVA_ERR_INVALID;
    b->row_setup = pages;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    return NOVA_OK;
}
int nova_batch_set_prefill_kernel(nova_batch* b, int which) {
    if (!b || which < 0 || which > 1) return NOVA_ERR_INVALID;
    if (which == 1 && (b->e->d.kv_dtype != NOVA_KV_F16 || !b->e->tmaps_ok || b->e->kv_shift < 4)) return NOVA_ERR_UNSUPPORTED;
    b->prefill_tc5 = which;
    return NOVA_OK;
}
int nova_batch_set_window(nova_batch* b, int window_tokens) {
    if (!b || window_tokens < 0) return NOVA_ERR_INVALID;
    b->window = window_tokens;
    return NOVA_OK;
}
int nova_batch_set_split_ctas(nova_batch* b, int n_ctas) {
    if (!b || n_ctas < 0 || n_ctas > kMaxSplitCtas) return NOVA_ERR_INVALID;
    b->split_ctas = n_ctas;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    return NOVA_OK;
}
int nova_batch_set_pdl(nova_batch* b, int on) {
    if (!b || on < 0 || on > 2) return NOVA_ERR_INVALID;
    b->pdl = on;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    return NOVA_OK;
}
int nova_batch_append_attn(nova_batch* b, int layer, float* q, float* k, const float* v, float* out, nova_stream_t s) {
    if (!b || !q || !k || !v || !out || layer < 0 || layer >= b->e->d.n_layers) return NOVA_ERR_INVALID;
    if (use_fused(b)) return run_attn_fused(b, layer, 1, q, k, v, out, (cudaStream_t)s);
    const int rc = nova_batch_append(b, layer, q, k, v, s);
    if (rc != NOVA_OK) return rc;
    return nova_batch_attn(b, layer, q, out, s);
}
int nova_batch_get_kernel(const nova_batch* b) { return b ? b->kernel : NOVA_ERR_INVALID; }

// Leading pages that every session of the batch maps to the same physical pages and that are full for all
// of them (whole pages below the smallest n_past): what the cascade attends once.  Host tables only.
static int shared_prefix_pages(const nova_batch* b) {
    const nova_engine* e = b->e;
    if (b->n < 4) return 0;
    const SliceState* first = e->pool.p.find(b->slices[0]);
    if (!first) return 0;
    int64_t limit = first->n_past >> e->kv_shift;
    for (int i = 1; i < b->n; ++i) {
        const SliceState* st = e->pool.p.find(b->slices[(size_t)i]);
        if (!st) return 0;
        if ((st->n_past >> e->kv_shift) < limit) limit = st->n_past >> e->kv_shift;
    }
    if (limit > (int64_t)first->table.size()) limit = (int64_t)first->table.size();
    for (int i = 1; i < b->n && limit > 0; ++i) {
        const SliceState* st = e->pool.p.find(b->slices[(size_t)i]);
        int64_t p = 0;
        while (p < limit && st->table[(size_t)p] == first->table[(size_t)p]) ++p;
        limit = p;
    }
    return (limit << e->kv_shift) >= 256 ? (int)limit : 0;        // below 256 shared tokens the extra launches cost more than they save
}

int nova_batch_set_cascade(nova_batch* b, int on) {
    if (!b) return NOVA_ERR_INVALID;
    if (on && b->kernel != 1) return NOVA_ERR_UNSUPPORTED;
    nova_engine* e = b->e;
    if (on && !b->casc_parts) {
        NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
        // the chunk count never exceeds what a huge prefix would get (the per-CTA minimum of four pages only lowers it)
        int max_chunks = attn_prefix_chunks(b->n, e->d.n_heads, e->d.n_kv_heads, 1 << 24, nullptr);
        const int tc5_chunks = attn_prefix_tc5_chunks(b->n, e->d.n_heads, e->d.n_kv_heads, 1 << 24, nullptr);
        if (tc5_chunks > max_chunks) max_chunks = tc5_chunks;
        b->casc_floats = (size_t)(max_chunks + 1) * b->n * e->d.n_heads * kPartW;
        NOVA_CUDA_TRY(cudaMalloc((void**)&b->casc_parts, b->casc_floats * sizeof(float)));
    }
    b->cascade = on ? 1 : 0;
    b->casc_pages = 0;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    return NOVA_OK;
}
int nova_batch_shared_prefix_pages(const nova_batch* b) { return b ? b->casc_pages : 0; }

int nova_batch_cow(nova_batch* b, nova_stream_t s) {
    if (!b) return NOVA_ERR_INVALID;
    nova_engine* e = b->e;
    std::vector<CowEvent> ev;
    int rc = NOVA_OK;
    for (int i = 0; i < b->n; ++i)        // a session of the batch was destroyed behind its back
        if (!e->pool.p.find(b->slices[(size_t)i])) return NOVA_ERR_INVALID;
    for (int i = 0; i < b->n && rc == NOVA_OK; ++i) {
        const SliceState* st = e->pool.p.find(b->slices[(size_t)i]);
        rc = collect_cow(e, b->slices[(size_t)i], st->n_past, 1, ev);
    }
    if (b->cascade) {                        // tables may just have changed: look for the shared prefix again
        const int pages = shared_prefix_pages(b);
        if (pages != b->casc_pages && b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
        b->casc_pages = pages;
    }
    if (!ev.empty()) {
        const int lrc = launch_cow_copy(e->pool_k, e->pool_v, e->d.n_layers, e->nb, e->page_bytes, ev.data(),
                                        (int)ev.size(), (cudaStream_t)s);
        if (lrc != NOVA_OK) return lrc;
    }
    return rc != NOVA_OK ? rc : (int)ev.size();
}

int nova_batch_append(nova_batch* b, int layer, float* q, float* k, const float* v, nova_stream_t s) {
    if (!b || !q || !k || !v || layer < 0 || layer >= b->e->d.n_layers) return NOVA_ERR_INVALID;
    AppendLaunch a;
    fill_append(b, a);
    a.q = q; a.k = k; a.v = v;
    a.layer0 = layer; a.n_layers = 1;
    return launch_rope_append(a, (cudaStream_t)s);
}

int nova_batch_append_layers(nova_batch* b, int layer0, int n_layers, float* q, float* k, const float* v,
                             nova_stream_t s) {
    if (!b || !k || !v || layer0 < 0 || n_layers < 1 || layer0 + n_layers > b->e->d.n_layers) return NOVA_ERR_INVALID;
    AppendLaunch a;
    fill_append(b, a);
    a.q = q; a.k = k; a.v = v;
    a.layer0 = layer0; a.n_layers = n_layers;
    return launch_rope_append(a, (cudaStream_t)s);
}

int nova_batch_attn(nova_batch* b, int layer, const float* q, float* out, nova_stream_t s) {
    if (!b || !q || !out || layer < 0 || layer >= b->e->d.n_layers) return NOVA_ERR_INVALID;
    AttnLaunch a;
    fill_attn(b, a);
    a.q = q; a.out = out;
    a.layer0 = layer; a.n_layers = 1;
    return run_attn(b, a, (cudaStream_t)s);
}

int nova_batch_advance_by(nova_batch* b, int n_tokens, nova_stream_t s) {
    if (!b || n_tokens < 0) return NOVA_ERR_INVALID;
    for (int i = 0; i < b->n; ++i) {
        SliceState* st = b->e->pool.p.find(b->slices[(size_t)i]);
        if (st) st->n_past += n_tokens;
    }
    return launch_advance(b->d_n_past, b->n, (cudaStream_t)s, n_tokens);
}

int nova_batch_advance(nova_batch* b, nova_stream_t s) { return nova_batch_advance_by(b, 1, s); }

int nova_batch_prefill_max_tokens(const nova_batch* b) {
    if (!b) return 0;
    if (b->kernel == 1) return 8192;             // the query-tiled kernel has no row table
    const int per = kMaxRowsSmem / (b->n * (b->e->d.n_kv_heads / b->e->kv_group));
    return per < 1 ? 0 : per;
}

// RopeKvOp + AttnOp with n > 1 (code/graph/dense.h:75-95): COW guard over [n_past, n_past + n), RoPE + append
// of n tokens per session, then causal attention of the n queries over the paged keys.
int nova_batch_prefill(nova_batch* b, int layer, int n_tokens, float* q, float* k, const float* v, float* out,
                       nova_stream_t s) {
    if (!b || !q || !k || !v || !out || layer < 0 || layer >= b->e->d.n_layers || n_tokens < 1) return NOVA_ERR_INVALID;
    if (n_tokens > nova_batch_prefill_max_tokens(b)) return NOVA_ERR_TOO_LARGE;
    if (b->window > 0 && b->kernel != 1) return NOVA_ERR_UNSUPPORTED;      // the window is a tensor-core prefill feature
    nova_engine* e = b->e;
    for (int i = 0; i < b->n; ++i)
        if (!e->pool.p.find(b->slices[(size_t)i])) return NOVA_ERR_INVALID;
    if (layer == 0) {        // un-share every page the new tokens will land in, once per prefill chunk
        std::vector<CowEvent> ev;
        int rc = NOVA_OK;
        for (int i = 0; i < b->n && rc == NOVA_OK; ++i) {
            const SliceState* st = e->pool.p.find(b->slices[(size_t)i]);
            rc = collect_cow(e, b->slices[(size_t)i], st->n_past, n_tokens, ev);
        }
        if (!ev.empty()) {
            const int lrc = launch_cow_copy(e->pool_k, e->pool_v, e->d.n_layers, e->nb, e->page_bytes, ev.data(),
                                            (int)ev.size(), (cudaStream_t)s);
            if (lrc != NOVA_OK) return lrc;
        }
        if (rc != NOVA_OK) return rc;
    }
    AppendLaunch ap;
    fill_append(b, ap);
    ap.q = q; ap.k = k; ap.v = v;
    ap.layer0 = layer; ap.n_layers = 1;
    ap.n_tok = n_tokens;
    int rc = launch_rope_append(ap, (cudaStream_t)s);
    if (rc != NOVA_OK) return rc;
    AttnLaunch at;
    fill_attn(b, at);
    at.q = q; at.out = out;
    at.layer0 = layer; at.n_layers = 1;
    at.n_q = n_tokens;
    at.window = b->window;
    return run_attn(b, at, (cudaStream_t)s);
}

int nova_batch_step_all_layers(nova_batch* b, float* q, float* k, const float* v, float* out, nova_stream_t s) {
    if (!b || !q || !k || !v || !out) return NOVA_ERR_INVALID;
    if (use_fused(b)) return run_attn_fused(b, 0, b->e->d.n_layers, q, k, v, out, (cudaStream_t)s);
    AppendLaunch ap;
    fill_append(b, ap);
    ap.q = q; ap.k = k; ap.v = v;
    ap.layer0 = 0; ap.n_layers = b->e->d.n_layers;
    int rc = launch_rope_append(ap, (cudaStream_t)s);
    if (rc != NOVA_OK) return rc;
    AttnLaunch at;
    fill_attn(b, at);
    at.q = q; at.out = out;
    at.layer0 = 0; at.n_layers = b->e->d.n_layers;
    return run_attn(b, at, (cudaStream_t)s);
}

static int ensure_staging(nova_batch* b);

int nova_batch_decode_step_host(nova_batch* b, const float* q, const float* k, const float* v, float* out,
                                int flags, nova_stream_t s) {
    if (!b || !q || !k || !v || !out || flags < 0 || flags > 3) return NOVA_ERR_INVALID;
    const bool per_layer_launch = (flags & 1) != 0, no_sync = (flags & 2) != 0;
    nova_engine* e = b->e;
    cudaStream_t st = (cudaStream_t)s;
    const int L = e->d.n_layers;
    const size_t S = (size_t)b->n;
    const size_t qs = S * e->d.n_heads * kHeadDim, ks = S * e->d.n_kv_heads * kHeadDim;   // floats per layer
    int rc = ensure_staging(b);
    if (rc != NOVA_OK) return rc;
    if (!b->s_in) {
        NOVA_CUDA_TRY(cudaStreamCreateWithFlags(&b->s_in, cudaStreamNonBlocking));
        NOVA_CUDA_TRY(cudaStreamCreateWithFlags(&b->s_out, cudaStreamNonBlocking));
        for (int i = 0; i < 4; ++i) {
            NOVA_CUDA_TRY(cudaEventCreateWithFlags(&b->ev_in[i], cudaEventDisableTiming));
            NOVA_CUDA_TRY(cudaEventCreateWithFlags(&b->ev_cmp[i], cudaEventDisableTiming));
        }
        for (int i = 0; i < 2; ++i) {
            NOVA_CUDA_TRY(cudaEventCreateWithFlags(&b->ev_free[i], cudaEventDisableTiming));
            NOVA_CUDA_TRY(cudaEventCreateWithFlags(&b->ev_dl[i], cudaEventDisableTiming));
        }
        NOVA_CUDA_TRY(cudaEventCreateWithFlags(&b->ev_out, cudaEventDisableTiming));
    }
    // Two sets of staging buffers, used in turn: while the kernels of one step run on its set, the inputs of the
    // next step are already arriving in the other one and the outputs of the step before are still leaving.
    const int set = (int)(b->host_seq++ & 1u);
    float* dq = set ? b->dq2 : b->dq;
    float* dk = set ? b->dk2 : b->dk;
    float* dv = set ? b->dv2 : b->dv;
    float* dout = set ? b->dout2 : b->dout;
    rc = nova_batch_cow(b, s);
    if (rc < 0) return rc;
    // the set's previous user (two steps ago) must have consumed its inputs before they are overwritten, and its
    // outputs must have left before this step's kernels write new ones (both events are complete when never recorded)
    NOVA_CUDA_TRY(cudaStreamWaitEvent(b->s_in, b->ev_free[set], 0));
    NOVA_CUDA_TRY(cudaStreamWaitEvent(st, b->ev_dl[set], 0));
    if (!per_layer_launch) {
        NOVA_CUDA_TRY(cudaMemcpyAsync(dq, q, L * qs * 4, cudaMemcpyHostToDevice, b->s_in));
        NOVA_CUDA_TRY(cudaMemcpyAsync(dk, k, L * ks * 4, cudaMemcpyHostToDevice, b->s_in));
        NOVA_CUDA_TRY(cudaMemcpyAsync(dv, v, L * ks * 4, cudaMemcpyHostToDevice, b->s_in));
        NOVA_CUDA_TRY(cudaEventRecord(b->ev_in[0], b->s_in));
        NOVA_CUDA_TRY(cudaStreamWaitEvent(st, b->ev_in[0], 0));
        rc = nova_batch_step_all_layers(b, dq, dk, dv, dout, s);
        if (rc != NOVA_OK) return rc;
        NOVA_CUDA_TRY(cudaEventRecord(b->ev_cmp[0], st));
        NOVA_CUDA_TRY(cudaStreamWaitEvent(b->s_out, b->ev_cmp[0], 0));
        NOVA_CUDA_TRY(cudaMemcpyAsync(out, dout, L * qs * 4, cudaMemcpyDeviceToHost, b->s_out));
    } else {
        // Layers are issued in order; their inputs arrive in up to four growing chunks on a copy stream
        // and finished outputs leave on another, so that only the first chunk's upload and the last
        // chunk's download are not hidden behind the attention launches.
        // Uploads go in growing chunks (layers [0,2), [2,6), [6,14), [14,L)), downloads in shrinking ones
        // ([0,L-14), [L-14,L-6), [L-6,L-2), [L-2,L)): what stays exposed is two layers' inputs before the
        // first launch and two layers' outputs after the last.
        int cin[5] = {0, L < 2 ? L : 2, L < 6 ? L : 6, L < 14 ? L : 14, L};
        int cout[5] = {0, L > 14 ? L - 14 : 0, L > 6 ? L - 6 : 0, L > 2 ? L - 2 : 0, L};
        if (no_sync) {       // queued steps hide each other's copies: one chunk each way, fewer calls on the host
            cin[1] = cin[2] = cin[3] = L;
            cout[1] = cout[2] = cout[3] = 0;
        }
        for (int c = 0; c < 4; ++c) {
            const int l0 = cin[c], n = cin[c + 1] - cin[c];
            if (n <= 0) continue;
            NOVA_CUDA_TRY(cudaMemcpyAsync(dq + l0 * qs, q + l0 * qs, n * qs * 4, cudaMemcpyHostToDevice, b->s_in));
            NOVA_CUDA_TRY(cudaMemcpyAsync(dk + l0 * ks, k + l0 * ks, n * ks * 4, cudaMemcpyHostToDevice, b->s_in));
            NOVA_CUDA_TRY(cudaMemcpyAsync(dv + l0 * ks, v + l0 * ks, n * ks * 4, cudaMemcpyHostToDevice, b->s_in));
            NOVA_CUDA_TRY(cudaEventRecord(b->ev_in[c], b->s_in));
        }
        int ci = 0, co = 0;
        for (int l = 0; l < L; ++l) {
            bool fresh = l == 0;                 // no dependent launch right after an event wait or record
            while (ci < 4 && cin[ci] <= l) {
                if (cin[ci + 1] > cin[ci] && cin[ci] == l) {
                    NOVA_CUDA_TRY(cudaStreamWaitEvent(st, b->ev_in[ci], 0));
                    fresh = true;
                }
                ++ci;
            }
            while (co < 4 && cout[co + 1] <= l) ++co;
            if (l > 0 && cout[co] == l) fresh = true;     // an output event was recorded just before this layer
            if (use_fused(b))
                rc = run_attn_fused(b, l, 1, dq + l * qs, dk + l * ks, dv + l * ks, dout + l * qs, st, b->pdl && !fresh);
            else
                rc = nova_batch_append_attn(b, l, dq + l * qs, dk + l * ks, dv + l * ks, dout + l * qs, s);
            if (rc != NOVA_OK) return rc;
            if (cout[co + 1] == l + 1) {                   // the chunk [cout[co], l + 1) is complete
                const int l0 = cout[co];
                NOVA_CUDA_TRY(cudaEventRecord(b->ev_cmp[co], st));
                NOVA_CUDA_TRY(cudaStreamWaitEvent(b->s_out, b->ev_cmp[co], 0));
                NOVA_CUDA_TRY(cudaMemcpyAsync(out + l0 * qs, dout + l0 * qs, (size_t)(l + 1 - l0) * qs * 4,
                                              cudaMemcpyDeviceToHost, b->s_out));
            }
        }
    }
    NOVA_CUDA_TRY(cudaEventRecord(b->ev_free[set], st));        // this set's inputs have been consumed
    NOVA_CUDA_TRY(cudaEventRecord(b->ev_dl[set], b->s_out));    // ... and its outputs are on their way out
    rc = nova_batch_advance(b, s);
    if (rc != NOVA_OK) return rc;
    if (no_sync) return NOVA_OK;
    NOVA_CUDA_TRY(cudaEventRecord(b->ev_out, b->s_out));
    NOVA_CUDA_TRY(cudaStreamWaitEvent(st, b->ev_out, 0));
    NOVA_CUDA_TRY(cudaStreamSynchronize(st));
    return NOVA_OK;
}

int nova_batch_host_wait(nova_batch* b, nova_stream_t s) {
    if (!b) return NOVA_ERR_INVALID;
    NOVA_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)s));
    if (b->s_out) NOVA_CUDA_TRY(cudaStreamSynchronize(b->s_out));
    return NOVA_OK;
}

static int ensure_staging(nova_batch* b) {
    if (b->dq) return NOVA_OK;
    const nova_engine* e = b->e;
    const size_t L = (size_t)e->d.n_layers, S = (size_t)b->n;
    const size_t q_elems = L * S * e->d.n_heads * kHeadDim, kv_elems = L * S * e->d.n_kv_heads * kHeadDim;
    cudaError_t ce = cudaMalloc((void**)&b->dq, q_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dk, kv_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dv, kv_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dout, q_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dq2, q_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dk2, kv_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dv2, kv_elems * 4);
    if (ce == cudaSuccess) ce = cudaMalloc((void**)&b->dout2, q_elems * 4);
    if (ce != cudaSuccess) { set_cuda_error(ce, "step staging"); return NOVA_ERR_CUDA; }
    return NOVA_OK;
}

// One decode step as per-layer launches on the staging buffers (everything but the COW guard).
static int issue_layers(nova_batch* b, float* q, float* k, const float* v, float* out, cudaStream_t st,
                        std::vector<cudaEvent_t>* ev, size_t* ev_used) {
    const nova_engine* e = b->e;
    const size_t S = (size_t)b->n;
    const size_t qs = S * e->d.n_heads * kHeadDim, ks = S * e->d.n_kv_heads * kHeadDim;
    for (int l = 0; l < e->d.n_layers; ++l) {
        int rc;
        if (use_fused(b)) {
            if (ev) NOVA_CUDA_TRY(cudaEventRecord((*ev)[(*ev_used)++], st));
            // Layers after the first follow a combine kernel of this same step: nothing they read before
            // their dependency wait (pages of earlier steps, tables, n_past) is written by it.
            rc = run_attn_fused(b, l, 1, q + l * qs, k + l * ks, v + l * ks, out + l * qs, st, b->pdl && l > 0);
        } else {
            rc = nova_batch_append(b, l, q + l * qs, k + l * ks, v + l * ks, (nova_stream_t)st);
            if (rc != NOVA_OK) return rc;
            if (ev) NOVA_CUDA_TRY(cudaEventRecord((*ev)[(*ev_used)++], st));
            rc = nova_batch_attn(b, l, q + l * qs, out + l * qs, (nova_stream_t)st);
        }
        if (rc != NOVA_OK) return rc;
        if (ev) NOVA_CUDA_TRY(cudaEventRecord((*ev)[(*ev_used)++], st));
    }
    return NOVA_OK;
}

// The per-layer step on the staging buffers as an executable graph; captured again whenever something baked into
// it has changed (kernel choice, fused append, number of shared pages of the cascade).
static int ensure_step_graph(nova_batch* b, cudaStream_t st) {
    if (b->graph && b->graph_kernel == b->kernel) return NOVA_OK;
    if (b->graph) { cudaGraphExecDestroy(b->graph); b->graph = nullptr; }
    cudaGraph_t g = nullptr;
    NOVA_CUDA_TRY(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    int rc = issue_layers(b, b->dq, b->dk, b->dv, b->dout, st, nullptr, nullptr);
    if (rc == NOVA_OK) rc = launch_advance(b->d_n_past, b->n, st);
    const cudaError_t ce = cudaStreamEndCapture(st, &g);
    if (rc != NOVA_OK) { if (g) cudaGraphDestroy(g); return rc; }
    if (ce != cudaSuccess) { set_cuda_error(ce, "cudaStreamEndCapture"); return NOVA_ERR_CUDA; }
    const cudaError_t ie = cudaGraphInstantiate(&b->graph, g, 0);
    cudaGraphDestroy(g);
    if (ie != cudaSuccess) { set_cuda_error(ie, "cudaGraphInstantiate"); return NOVA_ERR_CUDA; }
    b->graph_kernel = b->kernel;
    return NOVA_OK;
}

int nova_batch_run_steps(nova_batch* b, int n_steps, float* q, float* k, const float* v, float* out,
                         size_t q_stride, size_t kv_stride, int mode, float* attn_ms, nova_stream_t s) {
    if (!b || n_steps < 0 || !q || !k || !v || !out || mode < 0 || mode > 2) return NOVA_ERR_INVALID;
    if (attn_ms && mode == 2) return NOVA_ERR_INVALID;
    nova_engine* e = b->e;
    cudaStream_t st = (cudaStream_t)s;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    const size_t L = (size_t)e->d.n_layers, S = (size_t)b->n;
    const size_t q_elems = L * S * e->d.n_heads * kHeadDim, kv_elems = L * S * e->d.n_kv_heads * kHeadDim;
    size_t ev_used = 0;
    if (attn_ms) {
        const size_t need = (size_t)n_steps * (mode == 0 ? 2 : 2 * L);
        while (b->ev.size() < need) {
            cudaEvent_t ce = nullptr;
            NOVA_CUDA_TRY(cudaEventCreate(&ce));
            b->ev.push_back(ce);
        }
    }
    if (mode == 2) {
        const int rc = ensure_staging(b);
        if (rc != NOVA_OK) return rc;
        if (!st) return NOVA_ERR_INVALID;   // stream capture needs a real stream
    }
    for (int i = 0; i < n_steps; ++i) {
        float* qi = q + (size_t)i * q_stride;
        float* ki = k + (size_t)i * kv_stride;
        const float* vi = v + (size_t)i * kv_stride;
        float* oi = out + (size_t)i * q_stride;
        int rc = nova_batch_cow(b, s);
        if (rc < 0) return rc;
        if (mode == 0) {
            if (use_fused(b)) {
                if (attn_ms) NOVA_CUDA_TRY(cudaEventRecord(b->ev[ev_used++], st));
                rc = run_attn_fused(b, 0, e->d.n_layers, qi, ki, vi, oi, st);
            } else {
                AppendLaunch ap;
                fill_append(b, ap);
                ap.q = qi; ap.k = ki; ap.v = vi;
                ap.layer0 = 0; ap.n_layers = e->d.n_layers;
                rc = launch_rope_append(ap, st);
                if (rc != NOVA_OK) return rc;
                if (attn_ms) NOVA_CUDA_TRY(cudaEventRecord(b->ev[ev_used++], st));
                AttnLaunch at;
                fill_attn(b, at);
                at.q = qi; at.out = oi;
                at.layer0 = 0; at.n_layers = e->d.n_layers;
                rc = run_attn(b, at, st);
            }
            if (rc != NOVA_OK) return rc;
            if (attn_ms) NOVA_CUDA_TRY(cudaEventRecord(b->ev[ev_used++], st));
            rc = nova_batch_advance(b, s);
            if (rc != NOVA_OK) return rc;
        } else if (mode == 1) {
            rc = issue_layers(b, qi, ki, vi, oi, st, attn_ms ? &b->ev : nullptr, &ev_used);
            if (rc != NOVA_OK) return rc;
            rc = nova_batch_advance(b, s);
            if (rc != NOVA_OK) return rc;
        } else {
            rc = ensure_step_graph(b, st);          // after the COW guard: it may have changed what the graph bakes in
            if (rc != NOVA_OK) return rc;
            NOVA_CUDA_TRY(cudaMemcpyAsync(b->dq, qi, q_elems * 4, cudaMemcpyDeviceToDevice, st));
            NOVA_CUDA_TRY(cudaMemcpyAsync(b->dk, ki, kv_elems * 4, cudaMemcpyDeviceToDevice, st));
            NOVA_CUDA_TRY(cudaMemcpyAsync(b->dv, vi, kv_elems * 4, cudaMemcpyDeviceToDevice, st));
            NOVA_CUDA_TRY(cudaGraphLaunch(b->graph, st));
            count_launch((use_fused(b) ? 2 : 3) * e->d.n_layers + 1);
            NOVA_CUDA_TRY(cudaMemcpyAsync(qi, b->dq, q_elems * 4, cudaMemcpyDeviceToDevice, st));   // q, k rotated in place
            NOVA_CUDA_TRY(cudaMemcpyAsync(ki, b->dk, kv_elems * 4, cudaMemcpyDeviceToDevice, st));
            NOVA_CUDA_TRY(cudaMemcpyAsync(oi, b->dout, q_elems * 4, cudaMemcpyDeviceToDevice, st));
            for (int j = 0; j < b->n; ++j) {
                SliceState* sl = e->pool.p.find(b->slices[(size_t)j]);
                if (sl) sl->n_past += 1;
            }
        }
    }
    if (attn_ms) {
        NOVA_CUDA_TRY(cudaStreamSynchronize(st));
        float total = 0.f;
        for (size_t j = 0; j + 1 < ev_used; j += 2) {
            float ms = 0.f;
            NOVA_CUDA_TRY(cudaEventElapsedTime(&ms, b->ev[j], b->ev[j + 1]));
            total += ms;
        }
        *attn_ms = total;
    }
    return NOVA_OK;
}

int nova_batch_device_status(nova_batch* b) {
    if (!b) return NOVA_ERR_INVALID;
    int32_t v = 0;
    NOVA_CUDA_TRY(cudaMemcpy(&v, b->e->status, sizeof(v), cudaMemcpyDeviceToHost));
    if (v != 0) cudaMemset(b->e->status, 0, sizeof(v));
    return v;
}

int nova_batch_attn_partial_layers(nova_batch* b, int layer0, int n_layers, const float* q, int64_t page0,
                                   int64_t page1, float* part, nova_stream_t s) {
    if (!b || !q || !part || layer0 < 0 || n_layers < 1 || layer0 + n_layers > b->e->d.n_layers || page0 < 0 ||
        page1 < page0)
        return NOVA_ERR_INVALID;
    AttnLaunch a;
    fill_attn(b, a);
    a.q = q;
    a.out_part = part;
    a.write_partial_only = 1;
    a.page_lo = page0;
    a.page_hi = page1;
    a.layer0 = layer0; a.n_layers = n_layers;
    return run_attn(b, a, (cudaStream_t)s);
}

// One decode step of a session split over the GPUs of a node, in the engine's layer order and without any
// host-side collective: per layer the fused RoPE+append+attention over this rank's page range, then ONE launch
// that merges this rank's split-K partials, sends the finished rows to every peer, receives theirs and writes
// the merged output.
int nova_batch_step_partial_peers(nova_batch* b, float* q, float* k, const float* v, int64_t page0, int64_t page1,
                                  void* const* peer_base, int n_ranks, int my_rank, size_t slot_bytes, int n_slots,
                                  int64_t epoch0, int timeout_ms, float* out, int32_t* status, nova_stream_t s) {
    if (!b || !q || !k || !v || !out || !peer_base || n_ranks < 1 || n_ranks > kMaxPeerRanks || my_rank < 0 ||
        my_rank >= n_ranks || n_slots < 2 || epoch0 < 1 || page0 < 0 || page1 < page0 || timeout_ms < 1)
        return NOVA_ERR_INVALID;
    nova_engine* e = b->e;
    const int L = e->d.n_layers;
    const int rows = b->n * e->d.n_heads;
    if (epoch0 + L > 0x7fffffffLL) return NOVA_ERR_INVALID;
    if (slot_bytes < nova_peer_slot_bytes(rows) || slot_bytes % 128) return NOVA_ERR_INVALID;
    for (int i = 0; i < n_ranks; ++i)
        if (!peer_base[i]) return NOVA_ERR_INVALID;
    cudaStream_t st = (cudaStream_t)s;
    NOVA_CUDA_TRY(cudaSetDevice(e->d.device));
    if (!b->xparts) NOVA_CUDA_TRY(cudaMalloc((void**)&b->xparts, (size_t)rows * kPartW * sizeof(float)));
    const size_t qs = (size_t)b->n * e->d.n_heads * kHeadDim, ks = (size_t)b->n * e->d.n_kv_heads * kHeadDim;
    const unsigned long long timeout_ns = (unsigned long long)timeout_ms * 1000000ull;
    int rc = nova_batch_cow(b, s);
    if (rc < 0) return rc;
    for (int l = 0; l < L; ++l) {
        const int64_t epoch = epoch0 + l;
        void* base[kMaxPeerRanks];
        for (int i = 0; i < n_ranks; ++i)
            base[i] = static_cast<unsigned char*>(peer_base[i]) + (size_t)(epoch % n_slots) * slot_bytes;
        AttnLaunch a;
        fill_attn(b, a);
        a.q = q + l * qs;
        a.out = out + l * qs;
        a.out_part = b->xparts;
        a.write_partial_only = 1;
        a.page_lo = page0;
        a.page_hi = page1;
        a.layer0 = l;
        a.n_layers = 1;
        if (use_fused(b)) {
            a.fuse_append = 1;
            a.pool_k_w = e->pool_k; a.pool_v_w = e->pool_v;
            a.k_new = k + l * ks; a.v_new = v + l * ks;
            a.rope_cs = e->cs; a.rope_sn = e->sn; a.rope_rows = e->d.rope_positions;
            // layers after the first follow the previous layer's merge + exchange launch, which lets its dependents start early
            a.pdl = (b->pdl && l > 0) ? (b->pdl == 2 ? 2 : 1) : 0;
            a.pdl_spare = a.pdl != 0;
        } else {
            rc = nova_batch_append(b, l, q + l * qs, k + l * ks, v + l * ks, s);
            if (rc != NOVA_OK) return rc;
        }
        int ctas;
        if (b->kernel == 1) {
            ctas = pick_split_ctas(b, a);
            rc = launch_attn_mma(a, e->d.kv_dtype, ctas, st);
        } else {
            ctas = attn_split_ctas_simt(a, 0);
            rc = launch_attn_simt(a, e->d.kv_dtype, ctas, st);
        }
        if (rc != NOVA_OK) return rc;
        rc = launch_attn_combine_exchange(a, ctas, base, n_ranks, my_rank, (long long)epoch, timeout_ns, status, st);
        if (rc != NOVA_OK) return rc;
    }
    return nova_batch_advance(b, s);
}

int nova_batch_attn_partial(nova_batch* b, int layer, const float* q, int64_t page0, int64_t page1, float* part,
                            nova_stream_t s) {
    return nova_batch_attn_partial_layers(b, layer, 1, q, page0, page1, part, s);
}

}  // extern "C"
