// attn_plan.cuh — device-side stream-K partition of a decode-attention launch.
//
// Rows of one layer: r = s * n_groups + g (session s, kv-head group g); their page counts are
// prefix-summed into shared memory once per CTA.  The launch-wide page line has
// P = n_layers * P_layer entries and CTA c owns [c*P/C, (c+1)*P/C).  Everything below is
// computed redundantly (and identically) by every thread from that prefix array, so the
// host never has to build or upload a work list and the same launch can be replayed from a
// CUDA graph while n_past grows on the device.
#pragma once
#include "common.cuh"

namespace novab {

struct PlanView {
    const int* prefix;     // shared memory, rows_per_layer + 1 entries
    int rows_per_layer;    // S * n_groups
    int n_groups;
    int64_t pages_per_layer;
    int64_t pages_total;   // n_layers * pages_per_layer
    int n_ctas;
    bool small;            // (pages_total + 1) * (n_ctas + 1) fits 32 bits: the split arithmetic uses 32-bit divisions
};

__device__ __forceinline__ void plan_finish(PlanView& p) {
    p.small = (unsigned long long)(p.pages_total + 1) * (unsigned long long)(p.n_ctas + 1) < 0xffffffffULL;
}

struct Segment {
    int layer_local;   // 0 .. n_layers-1
    int row;           // row within the layer
    int session;       // the unit (session * n_q + query token)
    int group;
    int64_t row_id;    // layer_local * rows_per_layer + row
    int page_first;    // first REAL page of this segment, relative to the row's first page
    int page_count;    // real pages in the segment (0: only the row's set-up weight fell to this CTA)
    int span;          // how far the segment advances the launch-wide page line (set-up weight included)
    int c_first;       // first and last CTA that touch this row
    int c_last;
};

__device__ __forceinline__ int plan_nq(const AttnLaunch& a) { return a.n_q > 1 ? a.n_q : 1; }

// Page geometry of a launch.  Everything in this file that is called a "page" is a TILE: the unit the kernels
// stream, min(16, tokens per page) keys.  tpp_shift = log2(tiles per page): 0 for 8- and 16-token pages, 1 and 2
// for 32 and 64; tile i of a unit lives in block-table entry i >> tpp_shift at slot rows (i & (tpp - 1)) * 16.
struct PageGeom {
    int kv_shift, tile_shift, tpp_shift, tile_keys;
};
__device__ __forceinline__ PageGeom page_geom(int kv_shift_field) {
    PageGeom g;
    g.kv_shift = kv_shift_field ? kv_shift_field : kKvShift;
    g.tile_shift = g.kv_shift < 4 ? g.kv_shift : 4;
    g.tpp_shift = g.kv_shift - g.tile_shift;
    g.tile_keys = 1 << g.tile_shift;
    return g;
}

// Keys seen by unit u = s * n_q + t (query token t of session s).
__device__ __forceinline__ int plan_session_keys(const AttnLaunch& a, int u) {
    const int nq = plan_nq(a);
    const int s = u / nq, t = u - s * nq;
    return (a.n_past ? (a.n_past[s] + a.keys_add) : a.keys_imm) + t;
}

// First logical page and page count of a unit that sees n_keys keys, inside the launch's page window.
__device__ __forceinline__ void plan_pages_of_keys(const AttnLaunch& a, int n_keys, int& first, int& count) {
    const PageGeom pg = page_geom(a.kv_shift);
    int64_t total = n_keys > 0 ? (((int64_t)n_keys + pg.tile_keys - 1) >> pg.tile_shift) : 0;
    if (total > (a.table_stride << pg.tpp_shift)) total = a.table_stride << pg.tpp_shift;   // never walk past the table
    // the launch's window is given in pages of the pool
    int64_t lo = a.page_lo > 0 ? (a.page_lo << pg.tpp_shift) : 0;
    const int64_t hi_win = a.page_hi >= 0 ? (a.page_hi << pg.tpp_shift) : total;      // callers keep page_hi <= 2^40
    int64_t hi = hi_win < total ? hi_win : total;
    if (lo > hi) lo = hi;
    first = (int)lo;
    count = (int)(hi - lo);
}
__device__ __forceinline__ void plan_session_pages(const AttnLaunch& a, int s, int& first, int& count) {
    plan_pages_of_keys(a, plan_session_keys(a, s), first, count);
}

// Fills prefix[0..rows] (shared memory) with a warp scan; call from all threads of the CTA.
// slice_out (optional, shared memory, n_sessions entries) receives each session's slice id, fetched by
// the second warp at the same time, so that no later table lookup waits for it.
// keys_out (optional, shared memory, one entry per unit) receives plan_session_keys of every unit.
__device__ inline void plan_build_prefix(const AttnLaunch& a, int* prefix, int n_groups, int* slice_out = nullptr,
                                         int* keys_out = nullptr) {
    const int rows = a.n_sessions * plan_nq(a) * n_groups;
    if (slice_out && threadIdx.x >= 32 && threadIdx.x < 64)
        for (int s = (int)threadIdx.x - 32; s < a.n_sessions; s += 32) slice_out[s] = a.slice_ids ? a.slice_ids[s] : s;
    if (threadIdx.x < 32) {
        const int lane = (int)threadIdx.x;
        int carry = 0;
        if (lane == 0) prefix[0] = 0;
        for (int base = 0; base < rows; base += 32) {
            const int r = base + lane;
            int v = 0;
            if (r < rows) {
                int first, count;
                const int u = r / n_groups;
                const int n_keys = plan_session_keys(a, u);
                if (keys_out && r - u * n_groups == 0) keys_out[u] = n_keys;
                plan_pages_of_keys(a, n_keys, first, count);
                v = count > 0 ? count + a.row_setup_pages : 0;
            }
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += t;
            }
            if (r < rows) prefix[r + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int plan_owner(const PlanView& p, int64_t page) {
    if (p.small) return (int)((((unsigned)page + 1u) * (unsigned)p.n_ctas - 1u) / (unsigned)p.pages_total);
    return (int)((((page + 1) * (int64_t)p.n_ctas) - 1) / p.pages_total);
}

__device__ __forceinline__ int64_t plan_cta_begin(const PlanView& p, int c) {
    if (p.small) return (int64_t)(((unsigned)c * (unsigned)p.pages_total) / (unsigned)p.n_ctas);
    return ((int64_t)c * p.pages_total) / p.n_ctas;
}

// Segment that starts at launch-wide page `pos` and ends at the row's end or at `hi`.
__device__ inline Segment plan_segment(const PlanView& p, int64_t pos, int64_t hi, int setup) {
    Segment sg;
    sg.layer_local = p.small ? (int)((unsigned)pos / (unsigned)p.pages_per_layer) : (int)(pos / p.pages_per_layer);
    const int64_t layer_base = (int64_t)sg.layer_local * p.pages_per_layer;
    const int r = (int)(pos - layer_base);
    int lo = 0, up = p.rows_per_layer;           // find row with prefix[row] <= r < prefix[row+1]
    while (up - lo > 1) {
        const int mid = (lo + up) >> 1;
        if (p.prefix[mid] <= r) lo = mid; else up = mid;
    }
    // rows with zero pages share a prefix value with their successor: move to the last one
    while (lo + 1 < p.rows_per_layer && p.prefix[lo + 1] <= r) ++lo;
    sg.row = lo;
    sg.session = lo / p.n_groups;
    sg.group = lo - sg.session * p.n_groups;
    sg.row_id = (int64_t)sg.layer_local * p.rows_per_layer + lo;
    const int64_t row_begin = layer_base + p.prefix[lo];
    const int64_t row_end = layer_base + p.prefix[lo + 1];
    const int64_t end = row_end < hi ? row_end : hi;
    sg.span = (int)(end - pos);
    // the first `setup` entries of a row on the page line are weight only
    const int64_t r0 = pos - row_begin - setup, r1 = end - row_begin - setup;
    sg.page_first = (int)(r0 > 0 ? r0 : 0);
    sg.page_count = (int)((r1 > 0 ? r1 : 0) - sg.page_first);
    sg.c_first = plan_owner(p, row_begin);
    sg.c_last = plan_owner(p, row_end - 1);
    return sg;
}

}  // namespace novab
