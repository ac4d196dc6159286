// attn_simt.cu — paged split-K decode attention, SIMT form, for every session of a batch
// (and optionally every layer) in ONE launch.  Replaces fa_split_paged_kernel +
// fa_combine_kernel (src/kernel/attn.cu:197-289,163-191) and the per-session launch loop of
// Engine::decode_batch (src/model.cpp:286-290).
//
// One warp per kv head: the G = NH/NKV query heads that share it are packed, so every K and
// V row is read from HBM once (the reference reads it G times).  Each lane owns 4 of the 128
// dims; a key costs G 4-term dot partials, one transposing butterfly (9 shuffles + G
// broadcasts instead of 5G), an online softmax in the exp2 domain and 4G fp32 FMAs on V.
// Pages are walked straight from global memory with 8/16-byte loads, two batches of 8 (fp16) or
// 4 (fp32) keys in flight per warp.
// Work is cut stream-K style over pages (attn_plan.cuh); rows split over several CTAs leave
// partials for the combine kernel (attn_combine.cu) — no flags, no spinning anywhere.
//
// This is the fp32-accumulating reference form of the product: it serves fp32 pools (the
// reference's own format) and is the correctness anchor for the tensor-core kernel.
#include "attn_plan.cuh"

namespace novab {
namespace {

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void load4(const float* p, float (&x)[4]) {
    const float4 t = __ldcs(reinterpret_cast<const float4*>(p));
    x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
}
__device__ __forceinline__ void load4(const __half* p, float (&x)[4]) {
    const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}

// Raw (unconverted) 4-element pieces of a K or V row, kept in registers while later loads are in flight.
template <typename KvT> struct RawRow;
template <> struct RawRow<float> {
    using type = float4;
    static constexpr int kBatch = 4;       // keys per batch: 2 batches x (K + V) x 4 regs = 64 registers
    __device__ static __forceinline__ type load(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
    __device__ static __forceinline__ type zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ static __forceinline__ void unpack(const type& t, float (&x)[4]) { x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w; }
};
template <> struct RawRow<__half> {
    using type = uint2;
    static constexpr int kBatch = 8;
    __device__ static __forceinline__ type load(const __half* p) { return __ldcs(reinterpret_cast<const uint2*>(p)); }
    __device__ static __forceinline__ type zero() { return make_uint2(0u, 0u); }
    __device__ static __forceinline__ void unpack(const type& t, float (&x)[4]) {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
        x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    }
};

// Sum v[g] over the 32 lanes for up to 8 values at once: after three exchange-and-halve
// steps each lane holds one value's partial for head (lane>>2)&7, two more steps finish it.
template <int G>
__device__ __forceinline__ void reduce_heads(float (&v)[8], float (&out)[G], int lane) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float snd = b4 ? v[j] : v[j + 4];
        const float kp = b4 ? v[j + 4] : v[j];
        v[j] = kp + __shfl_xor_sync(0xffffffffu, snd, 16);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const float snd = b3 ? v[j] : v[j + 2];
        const float kp = b3 ? v[j + 2] : v[j];
        v[j] = kp + __shfl_xor_sync(0xffffffffu, snd, 8);
    }
    {
        const float snd = b2 ? v[0] : v[1];
        const float kp = b2 ? v[1] : v[0];
        v[0] = kp + __shfl_xor_sync(0xffffffffu, snd, 4);
    }
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
#pragma unroll
    for (int g = 0; g < G; ++g) out[g] = __shfl_sync(0xffffffffu, v[0], 4 * g);
}

template <int G>
struct HeadState {
    float m[G], l[G], acc[G][4];
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.f;
#pragma unroll
            for (int d = 0; d < 4; ++d) acc[g][d] = 0.f;
        }
    }
};

template <typename KvT, int G>
__global__ void __launch_bounds__(128) attn_simt_kernel(AttnLaunch a) {
    __shared__ int s_prefix[kMaxRowsSmem + 1];

    const int lane = (int)threadIdx.x & 31;
    const int warp = (int)threadIdx.x >> 5;
    const int KVG = a.kv_group;
    const int n_groups = a.n_kv_heads / KVG;
    const int NQ = plan_nq(a);
    const int NKV = a.n_kv_heads, NH = a.n_heads, S = a.n_sessions * NQ;    // S counts units
    const int heads_per_row = KVG * G;

    plan_build_prefix(a, s_prefix, n_groups);
    PlanView pv;
    pv.prefix = s_prefix;
    pv.rows_per_layer = S * n_groups;
    pv.n_groups = n_groups;
    pv.pages_per_layer = s_prefix[pv.rows_per_layer];
    pv.pages_total = pv.pages_per_layer * a.n_layers;
    // With fewer pages than CTAs only the first `pages_total` CTAs take part, so that every
    // participating CTA owns at least one page and a row's contributors are exactly
    // c_first .. c_last.
    pv.n_ctas = pv.pages_total < (int64_t)gridDim.x ? (int)pv.pages_total : (int)gridDim.x;
    plan_finish(pv);

    // Rows without any page in the window get their "nothing attended" result here.
    {
        const int64_t rows_total = (int64_t)pv.rows_per_layer * a.n_layers;
        for (int64_t v = blockIdx.x; v < rows_total; v += gridDim.x) {
            const int row = (int)(v % pv.rows_per_layer);
            if (s_prefix[row + 1] != s_prefix[row]) continue;
            const int ll = (int)(v / pv.rows_per_layer);
            const int s = row / n_groups, g = row - s * n_groups;
            const int kvh = g * KVG + warp;
            for (int h = 0; h < G; ++h) {
                const int64_t head = ((int64_t)ll * S + s) * NH + (int64_t)kvh * G + h;
                if (a.write_partial_only) {
                    float* op = a.out_part + head * kPartW;
                    if (lane == 0) { op[0] = -INFINITY; op[1] = 0.f; }
                    for (int d = 0; d < 4; ++d) op[2 + 4 * lane + d] = 0.f;
                } else {
                    *reinterpret_cast<float4*>(a.out + head * kHeadDim + 4 * lane) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        }
    }
    if (pv.pages_total == 0 || (int)blockIdx.x >= pv.n_ctas) return;

    const int64_t lo = plan_cta_begin(pv, (int)blockIdx.x);
    const int64_t hi = plan_cta_begin(pv, (int)blockIdx.x + 1);
    const KvT* pool_k = static_cast<const KvT*>(a.pool_k);
    const KvT* pool_v = static_cast<const KvT*>(a.pool_v);
    const int64_t row_elems = (int64_t)NKV * kHeadDim;
    constexpr float kQScale = kAttnScale * kLog2e;

    for (int64_t pos = lo; pos < hi;) {
        const Segment sg = plan_segment(pv, pos, hi, a.row_setup_pages);
        pos += sg.span;
        const int s = sg.session;
        const int kvh = sg.group * KVG + warp;
        const int layer = a.layer0 + sg.layer_local;
        const int n_keys = plan_session_keys(a, s);
        int first_page, n_pages_row;
        plan_session_pages(a, s, first_page, n_pages_row);
        const int rs = s / NQ;                            // the real session of this unit
        const int32_t* table = a.table_base + (int64_t)(a.slice_ids ? a.slice_ids[rs] : rs) * a.table_stride;
        const int64_t head0 = ((int64_t)sg.layer_local * S + s) * NH + (int64_t)kvh * G;

        float qr[G][4];
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float4 t = *reinterpret_cast<const float4*>(a.q + (head0 + g) * kHeadDim + 4 * lane);
            qr[g][0] = t.x * kQScale; qr[g][1] = t.y * kQScale; qr[g][2] = t.z * kQScale; qr[g][3] = t.w * kQScale;
        }
        HeadState<G> st;
        st.reset();

        // Keys are taken in batches of B (half or a quarter of a page).  The K and V pieces of batch j+1
        // are requested before batch j is used, so each warp keeps two batches of loads in flight; with
        // only the two keys of the inner step in flight the kernel was bound by memory latency.
        using RR = RawRow<KvT>;
        constexpr int B = RR::kBatch;
        const PageGeom geo = page_geom(a.kv_shift);
        const int BPP = geo.tile_keys / B;                 // batches per tile (a tile is 16 keys, 8 with 8-token pages)
        const int n_batches = sg.page_count * BPP;
        int chunk = -1, phys_lane = 0;
        typename RR::type rk[2][B], rv[2][B];
        int kc[2] = {0, 0};
        auto fetch = [&](int j, typename RR::type (&bk)[B], typename RR::type (&bv)[B], int& cnt) {
            cnt = 0;
#pragma unroll
            for (int i = 0; i < B; ++i) { bk[i] = RR::zero(); bv[i] = RR::zero(); }
            if (j >= n_batches) return;
            const int pg = j / BPP, slot0 = (j - pg * BPP) * B;
            if ((pg >> 5) != chunk) {                 // 32 block-table entries at a time, one per lane
                chunk = pg >> 5;
                const int idx = (chunk << 5) + lane;
                phys_lane = idx < sg.page_count ? __ldg(table + ((first_page + sg.page_first + idx) >> geo.tpp_shift)) : 0;
            }
            const int phys = __shfl_sync(0xffffffffu, phys_lane, pg & 31);
            if (phys < 0 || phys >= a.nb) {
                if (lane == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
                return;
            }
            const int page = first_page + sg.page_first + pg;        // tile index within the session
            int kcount = n_keys - (page << geo.tile_shift) - slot0;
            if (kcount > B) kcount = B;
            if (kcount <= 0) return;
            cnt = kcount;
            const int sub = (page & ((1 << geo.tpp_shift) - 1)) << 4;    // first slot row of the tile inside its page
            const int64_t base = ((((int64_t)layer * a.nb + phys) << geo.kv_shift) + sub + slot0) * row_elems + (int64_t)kvh * kHeadDim + 4 * lane;
#pragma unroll
            for (int i = 0; i < B; ++i)
                if (i < kcount) {
                    bk[i] = RR::load(pool_k + base + (int64_t)i * row_elems);
                    bv[i] = RR::load(pool_v + base + (int64_t)i * row_elems);
                }
        };
        auto consume = [&](const typename RR::type (&bk)[B], const typename RR::type (&bv)[B], int cnt) {
#pragma unroll
            for (int i = 0; i < B; i += 2) {
                if (i >= cnt) break;
                const bool two = i + 1 < cnt;
                float k0[4], k1[4], v0[4], v1[4];
                RR::unpack(bk[i], k0);
                RR::unpack(bk[i + 1], k1);
                RR::unpack(bv[i], v0);
                RR::unpack(bv[i + 1], v1);
                float d0[8], d1[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if (g < G) {
                        d0[g] = fmaf(qr[g][3], k0[3], fmaf(qr[g][2], k0[2], fmaf(qr[g][1], k0[1], qr[g][0] * k0[0])));
                        d1[g] = fmaf(qr[g][3], k1[3], fmaf(qr[g][2], k1[2], fmaf(qr[g][1], k1[1], qr[g][0] * k1[0])));
                    } else {
                        d0[g] = 0.f;
                        d1[g] = 0.f;
                    }
                }
                float s0[G], s1[G];
                reduce_heads<G>(d0, s0, lane);
                reduce_heads<G>(d1, s1, lane);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float sc1 = two ? s1[g] : -INFINITY;
                    const float mn = fmaxf(st.m[g], fmaxf(s0[g], sc1));
                    const float corr = ex2(st.m[g] - mn);
                    const float p0 = ex2(s0[g] - mn);
                    const float p1 = ex2(sc1 - mn);
                    st.l[g] = fmaf(st.l[g], corr, p0 + p1);
#pragma unroll
                    for (int d = 0; d < 4; ++d)
                        st.acc[g][d] = fmaf(p1, v1[d], fmaf(p0, v0[d], st.acc[g][d] * corr));
                    st.m[g] = mn;
                }
            }
        };
        fetch(0, rk[0], rv[0], kc[0]);
        for (int j = 0; j < n_batches; j += 2) {
            fetch(j + 1, rk[1], rv[1], kc[1]);
            consume(rk[0], rv[0], kc[0]);
            fetch(j + 2, rk[0], rv[0], kc[0]);
            consume(rk[1], rv[1], kc[1]);
        }

        const int n_contrib = sg.c_last - sg.c_first + 1;
        if (n_contrib == 1) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                if (a.write_partial_only) {
                    float* op = a.out_part + (head0 + g) * kPartW;
                    if (lane == 0) { op[0] = st.m[g] * (1.f / kLog2e); op[1] = st.l[g]; }
#pragma unroll
                    for (int d = 0; d < 4; ++d) op[2 + 4 * lane + d] = st.acc[g][d];
                } else {
                    const float inv = st.l[g] > 0.f ? 1.f / st.l[g] : 0.f;
                    *reinterpret_cast<float4*>(a.out + (head0 + g) * kHeadDim + 4 * lane) =
                        make_float4(st.acc[g][0] * inv, st.acc[g][1] * inv, st.acc[g][2] * inv, st.acc[g][3] * inv);
                }
            }
            continue;
        }
        // partial slot (cta + row): rows [heads_per_row][kSlotW], m in natural-log units
        {
            float* slot_base = a.part + (size_t)((int64_t)blockIdx.x + sg.row_id) * heads_per_row * kSlotW;
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float* pr = slot_base + (size_t)(warp * G + g) * kSlotW;
                if (lane == 0) *reinterpret_cast<float2*>(pr) = make_float2(st.m[g] * (1.f / kLog2e), st.l[g]);
                *reinterpret_cast<float4*>(pr + 4 + 4 * lane) = make_float4(st.acc[g][0], st.acc[g][1], st.acc[g][2], st.acc[g][3]);
            }
        }
    }
}

template <typename KvT>
int launch_simt_g(const AttnLaunch& a, int G, int n_ctas, cudaStream_t s) {
    const unsigned threads = 32u * (unsigned)a.kv_group;
    switch (G) {
#define NOVA_CASE(g) case g: attn_simt_kernel<KvT, g><<<(unsigned)n_ctas, threads, 0, s>>>(a); break;
        NOVA_CASE(1) NOVA_CASE(2) NOVA_CASE(4) NOVA_CASE(5) NOVA_CASE(6) NOVA_CASE(7) NOVA_CASE(8)
#undef NOVA_CASE
        default: return NOVA_ERR_UNSUPPORTED;
    }
    return NOVA_OK;
}

}  // namespace

int attn_default_ctas_simt(int n_kv_heads) {
    // 128-thread (or smaller) CTAs, 16 warps per SM resident: enough loads in flight without smem.
    const int kvg = n_kv_heads < 4 ? n_kv_heads : 4;
    return sm_count() * (16 / kvg);
}

int attn_split_ctas_simt(const AttnLaunch& a, int n_ctas) {
    return n_ctas > 0 ? n_ctas : attn_default_ctas_simt(a.n_kv_heads);
}

int launch_attn_simt(const AttnLaunch& a, int kv_dtype, int n_ctas, cudaStream_t s) {
    if (a.n_sessions <= 0 || a.n_layers <= 0) return NOVA_OK;
    if (a.n_heads % a.n_kv_heads || a.kv_group < 1 || a.kv_group > 4 || a.n_kv_heads % a.kv_group)
        return NOVA_ERR_INVALID;
    if ((int64_t)a.n_sessions * (a.n_q > 1 ? a.n_q : 1) * (a.n_kv_heads / a.kv_group) > kMaxRowsSmem) return NOVA_ERR_TOO_LARGE;
    n_ctas = attn_split_ctas_simt(a, n_ctas);
    const int G = a.n_heads / a.n_kv_heads;
    int rc;
    if (kv_dtype == NOVA_KV_F16) rc = launch_simt_g<__half>(a, G, n_ctas, s);
    else if (kv_dtype == NOVA_KV_F32) rc = launch_simt_g<float>(a, G, n_ctas, s);
    else return NOVA_ERR_UNSUPPORTED;
    if (rc != NOVA_OK) return rc;
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
