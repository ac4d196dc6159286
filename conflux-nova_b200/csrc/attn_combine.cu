// attn_combine.cu — log-sum-exp merge of split-K partials.  Replaces fa_combine_kernel
// (src/kernel/attn.cu:163-191 of the reference): m = max m_c, l = sum l_c e^{m_c - m},
// O = sum acc_c e^{m_c - m} / l, zero when l == 0, contributors taken in a fixed order.
//
// attn_combine_kernel follows either split kernel: one WARP per (row, query head) recomputes from
// the work split (attn_plan.cuh) which CTAs contributed and loads their (m, l) pairs (one lane per
// contributor) and all their accumulators (16-byte loads) in one batch of independent loads, so
// the merge costs one memory round trip per 32 contributors instead of two per contributor.  Rows covered by a single CTA were already written by the split kernel.
#include "attn_plan.cuh"

namespace novab {
namespace {

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float2 ld_cg_f2(const float* p) {
    float2 v;
    asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

// Folds up to 32 contributors' partial rows (slot layout: m, l, 2 pad, acc[128]; `stride` floats apart) into the
// running (M, L, acc) of a warp; lane i owns dims 4i..4i+3.  ONE memory round trip (about a microsecond here while
// a next layer streams): the (m, l) pair of contributor `lane` and the accumulators of all contributors are loaded
// before anything is used.  The loads are volatile asm so that they stay together in program order; kBlock of them
// are in flight per lane (16: 64 registers; a second block follows only when there are more contributors).
__device__ __forceinline__ void fold_contributors(const float* __restrict__ src, size_t stride, int cnt, int lane, float& M,
                                                  float& L, float4& acc) {
    constexpr int kBlock = 16;
    float2 ml = make_float2(-INFINITY, 0.f);
    if (lane < cnt) ml = ld_cg_f2(src + (size_t)lane * stride);
    float4 x[kBlock], y[kBlock];
#pragma unroll
    for (int i = 0; i < kBlock; ++i) {
        x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < cnt) x[i] = ld_cg_f4(src + (size_t)i * stride + 4 + 4 * lane);
    }
    const bool more = cnt > kBlock;           // warp-uniform
    if (more) {
#pragma unroll
        for (int i = 0; i < kBlock; ++i) {
            y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kBlock + i < cnt) y[i] = ld_cg_f4(src + (size_t)(kBlock + i) * stride + 4 + 4 * lane);
        }
    }
    const float mc = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
    const float Mn = fmaxf(M, mc);
    if (Mn == -INFINITY) return;                       // nothing attended in this chunk or before
    const float corr = __expf(M - Mn);                 // 0 on the first chunk (M = -inf)
    const float w = ml.y > 0.f ? __expf(ml.x - Mn) : 0.f;
    L = fmaf(L, corr, warp_sum(ml.y * w));
    acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
#pragma unroll
    for (int i = 0; i < kBlock; ++i) {
        const float wi = __shfl_sync(0xffffffffu, w, i);
        if (wi != 0.f) {                               // a slot with l == 0 carries no accumulator (and may hold anything)
            acc.x = fmaf(x[i].x, wi, acc.x);
            acc.y = fmaf(x[i].y, wi, acc.y);
            acc.z = fmaf(x[i].z, wi, acc.z);
            acc.w = fmaf(x[i].w, wi, acc.w);
        }
    }
    if (more) {
#pragma unroll
        for (int i = 0; i < kBlock; ++i) {
            const float wi = __shfl_sync(0xffffffffu, w, kBlock + i);
            if (wi != 0.f) {
                acc.x = fmaf(y[i].x, wi, acc.x);
                acc.y = fmaf(y[i].y, wi, acc.y);
                acc.z = fmaf(y[i].z, wi, acc.z);
                acc.w = fmaf(y[i].w, wi, acc.w);
            }
        }
    }
    M = Mn;
}

// Three warps per CTA, not four: the split kernel's CTAs have five warps of ~250 registers, so one of
// the SM's four register-file partitions holds two of them and has no room for a merge warp.  A
// three-warp CTA fits into the other three partitions and can sit on an SM next to a running split
// CTA; a four-warp one cannot, takes an SM of its own while it waits for the split kernel, and keeps
// the next layer's CTA off that SM until the merge is done.
#ifndef NOVA_COMBINE_WARPS
#define NOVA_COMBINE_WARPS 3
#endif
constexpr int kCombineWarps = NOVA_COMBINE_WARPS;

// kFold = true is the cascade's final merge (extra parts folded in, see AttnLaunch::extra_parts); it is a separate
// instantiation so that the plain merge keeps its register count (it has to share SMs with the split kernel).
// kCoop = true (launches with few (row, head) units, e.g. one long session): a unit belongs to a whole CTA and its
// contributors are dealt out to the warps 32 at a time, so a row that 136 CTAs worked on costs two memory round
// trips instead of five; the warps' results meet in shared memory.
// (Six warps of 128 registers for the cascade's merge were tried: such a CTA needs room in all four register-file
// partitions and no longer starts beside a split CTA; 0.65 -> 0.86 ms per config-3 step.)
constexpr int kFoldWarps = kCombineWarps;
template <bool kFold, bool kCoop = false>
__global__ void __launch_bounds__(32 * kCombineWarps) attn_combine_kernel(AttnLaunch a, int n_ctas_split) {
    constexpr int kWarps = kCombineWarps;
    __shared__ int s_prefix[kMaxRowsSmem + 1];
    __shared__ float s_ml[kCoop ? 2 * kCombineWarps : 1];
    __shared__ float4 s_acc[kCoop ? kCombineWarps * 32 : 1];
    const int lane = (int)threadIdx.x & 31;
    const int warp = (int)threadIdx.x >> 5;
#ifdef NOVA_TIMELINE      // profiling build only: stamps of the first CTAs go after the split kernel's block of stamps
    unsigned long long* tl = (a.timeline && blockIdx.x < kTimelineCtas) ? a.timeline + kTimelineCtas * 8 + (size_t)blockIdx.x * 4 : nullptr;
#else
    constexpr unsigned long long* tl = nullptr;
#endif
    if (tl && threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[0]));
        tl[2] = smid;
    }
    pdl_launch_dependents();
    const int KVG = a.kv_group;
    const int G = a.n_heads / a.n_kv_heads;
    const int n_groups = a.n_kv_heads / KVG;
    const int heads_per_row = KVG * G;
    plan_build_prefix(a, s_prefix, n_groups);     // n_past: not written by the split kernel before us
    PlanView pv;
    pv.prefix = s_prefix;
    const int S = a.n_sessions * plan_nq(a);        // units
    pv.rows_per_layer = S * n_groups;
    pv.n_groups = n_groups;
    pv.pages_per_layer = s_prefix[pv.rows_per_layer];
    pv.pages_total = pv.pages_per_layer * a.n_layers;
    pv.n_ctas = pv.pages_total < (int64_t)n_ctas_split ? (int)pv.pages_total : n_ctas_split;
    if (pv.pages_total > 0) plan_finish(pv);

    const int64_t units = pv.pages_total > 0 ? (int64_t)pv.rows_per_layer * a.n_layers * heads_per_row : 0;
    const size_t stride_c = (size_t)heads_per_row * kSlotW;
    // A (row, head) unit: where its split-K slots start, how many there are, which output row it is.  All of it
    // follows from the positions alone, so a warp works it out for its first units BEFORE the dependency wait;
    // what comes after the wait is on the layer's critical path.
    struct Unit {
        const float* base;
        int64_t head;
        int n;
        bool todo;
    };
    auto describe = [&](int64_t u, Unit& d) {
        const int64_t v = u / heads_per_row;
        const int hr = (int)(u - v * heads_per_row);            // kv head in group * G + query head
        const int row = (int)(v % pv.rows_per_layer);
        const bool no_pages = s_prefix[row + 1] == s_prefix[row];
        d.todo = false;
        d.base = nullptr;
        d.head = 0;
        d.n = 0;
        if (no_pages && !kFold) return;                          // no pages: written by the split kernel
        const int ll = (int)(v / pv.rows_per_layer);
        const int64_t row_begin = (int64_t)ll * pv.pages_per_layer + s_prefix[row];
        const int64_t row_end = (int64_t)ll * pv.pages_per_layer + s_prefix[row + 1];
        int c_first;
        if constexpr (kFold) {                                   // more parts to fold in: every row is ours to finish
            c_first = no_pages ? 0 : plan_owner(pv, row_begin);
            d.n = no_pages ? 0 : plan_owner(pv, row_end - 1) - c_first + 1;
        } else {
            c_first = plan_owner(pv, row_begin);
            d.n = plan_owner(pv, row_end - 1) - c_first + 1;
            if (d.n == 1) return;                                 // written by the split kernel
        }
        const int s = row / n_groups, grp = row - s * n_groups;
        d.head = ((int64_t)ll * S + s) * a.n_heads + (int64_t)(grp * KVG) * G + hr;
        d.base = a.part + ((size_t)(c_first + v) * heads_per_row + (size_t)hr) * kSlotW;
        d.todo = true;
    };
    auto process = [&](const Unit& d) {
        if constexpr (kFold) {
            // The usual cascade row - a few split-K slots (or the one partial the split kernel left) and up to 16 chunk
            // partials - in ONE memory round trip: every (m, l) pair and every accumulator is requested before
            // anything is used.  (Piece by piece - slots, chunk maxima, chunks eight at a time - a row cost four
            // dependent round trips, and a warp has several rows to finish.)
            const int na = d.n == 1 ? 0 : d.n, nb = a.n_extra;
            if (na <= 8 && nb <= 16) {
                const size_t estride = (size_t)S * a.n_heads * kPartW;
                const float* eb = a.extra_parts + d.head * kPartW;
                const float* pr = a.out_part + d.head * kPartW;
                float2 ml = make_float2(-INFINITY, 0.f);                 // lane = contributor: slots, chunks, lane 31 the lone partial
                if (lane < na) ml = ld_cg_f2(d.base + (size_t)lane * stride_c);
                else if (lane < na + nb) ml = ld_cg_f2(eb + (size_t)(lane - na) * estride);
                else if (lane == 31 && d.n == 1) ml = ld_cg_f2(pr);
                float4 xs[8];
                float2 e0[16], e1[16], s0 = make_float2(0.f, 0.f), s1 = s0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    xs[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (i < na) xs[i] = ld_cg_f4(d.base + (size_t)i * stride_c + 4 + 4 * lane);
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    e0[i] = e1[i] = make_float2(0.f, 0.f);
                    if (i < nb) {
                        const float* q = eb + (size_t)i * estride + 2 + 4 * lane;
                        e0[i] = ld_cg_f2(q);
                        e1[i] = ld_cg_f2(q + 2);
                    }
                }
                if (d.n == 1) {
                    s0 = ld_cg_f2(pr + 2 + 4 * lane);
                    s1 = ld_cg_f2(pr + 4 + 4 * lane);
                }
                const float Mx = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
                const float w = (ml.y > 0.f && Mx > -INFINITY) ? __expf(ml.x - Mx) : 0.f;
                const float Lx = warp_sum(ml.y * w);
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float wi = __shfl_sync(0xffffffffu, w, i);
                    if (i < na && wi != 0.f) {                 // a contributor with l == 0 carries no accumulator (and may hold anything)
                        acc.x = fmaf(xs[i].x, wi, acc.x);
                        acc.y = fmaf(xs[i].y, wi, acc.y);
                        acc.z = fmaf(xs[i].z, wi, acc.z);
                        acc.w = fmaf(xs[i].w, wi, acc.w);
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float wi = __shfl_sync(0xffffffffu, w, (na + i) & 31);
                    if (i < nb && wi != 0.f) {
                        acc.x = fmaf(e0[i].x, wi, acc.x);
                        acc.y = fmaf(e0[i].y, wi, acc.y);
                        acc.z = fmaf(e1[i].x, wi, acc.z);
                        acc.w = fmaf(e1[i].y, wi, acc.w);
                    }
                }
                const float ws = __shfl_sync(0xffffffffu, w, 31);
                if (d.n == 1 && ws != 0.f) {
                    acc.x = fmaf(s0.x, ws, acc.x);
                    acc.y = fmaf(s0.y, ws, acc.y);
                    acc.z = fmaf(s1.x, ws, acc.z);
                    acc.w = fmaf(s1.y, ws, acc.w);
                }
                const float inv = Lx > 0.f ? 1.f / Lx : 0.f;
                *reinterpret_cast<float4*>(a.out + d.head * kHeadDim + 4 * lane) =
                    make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
                return;
            }
        }
        // Contributors are taken 32 at a time: lane i holds (m, l) of contributor c0 + i while every
        // lane pulls its 4 dims of all 32 accumulators.  None of these loads depends on another, so a
        // chunk costs ONE memory round trip (a round trip is ~1 us here; a row usually fits one chunk).
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if constexpr (kFold) if (d.n == 1) {            // the split kernel left this row's partial (m, l, acc) in out_part
            const float* pr = a.out_part + d.head * kPartW;
            const float2 ml = __ldcg(reinterpret_cast<const float2*>(pr));
            const float2 y0 = __ldcg(reinterpret_cast<const float2*>(pr + 2 + 4 * lane));
            const float2 y1 = __ldcg(reinterpret_cast<const float2*>(pr + 4 + 4 * lane));
            if (ml.y > 0.f) {
                M = ml.x;
                L = ml.y;
                acc = make_float4(y0.x, y0.y, y1.x, y1.y);
            }
        }
        for (int c0 = kCoop ? 32 * warp : 0; c0 < ((kFold && d.n == 1) ? 0 : d.n); c0 += kCoop ? 32 * kCombineWarps : 32)
            fold_contributors(d.base + (size_t)c0 * stride_c, stride_c, d.n - c0 < 32 ? d.n - c0 : 32, lane, M, L, acc);
        if constexpr (kCoop) {       // the warps' shares of the row meet here; warp 0 finishes the row
            if (lane == 0) { s_ml[2 * warp] = M; s_ml[2 * warp + 1] = L; }
            s_acc[warp * 32 + lane] = acc;
            __syncthreads();
            if (warp == 0) {
                float Mx = -INFINITY;
#pragma unroll
                for (int w = 0; w < kCombineWarps; ++w)
                    if (s_ml[2 * w + 1] > 0.f) Mx = fmaxf(Mx, s_ml[2 * w]);
                L = 0.f;
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < kCombineWarps; ++w) {
                    const float lw = s_ml[2 * w + 1];
                    if (lw > 0.f) {
                        const float cw = __expf(s_ml[2 * w] - Mx);
                        const float4 x = s_acc[w * 32 + lane];
                        L = fmaf(lw, cw, L);
                        acc.x = fmaf(x.x, cw, acc.x);
                        acc.y = fmaf(x.y, cw, acc.y);
                        acc.z = fmaf(x.z, cw, acc.z);
                        acc.w = fmaf(x.w, cw, acc.w);
                    }
                }
                M = Mx;
            }
            __syncthreads();
            if (warp != 0) return;
        }
        if constexpr (kFold) {
            // the extra parts (a cascade's chunks over the shared pages), 32 (m, l) pairs and 8 accumulators at a time
            const size_t estride = (size_t)S * a.n_heads * kPartW;
            const float* eb = a.extra_parts + d.head * kPartW;
            for (int e0 = 0; e0 < a.n_extra; e0 += 32) {
                const int cnt = a.n_extra - e0 < 32 ? a.n_extra - e0 : 32;
                float2 ml = make_float2(-INFINITY, 0.f);
                if (lane < cnt) ml = __ldcg(reinterpret_cast<const float2*>(eb + (size_t)(e0 + lane) * estride));
                const float mc = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
                const float Mn = fmaxf(M, mc);
                if (Mn == -INFINITY) return;
                const float corr = __expf(M - Mn);
                const float w = ml.y > 0.f ? __expf(ml.x - Mn) : 0.f;
                L = fmaf(L, corr, warp_sum(ml.y * w));
                acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
                for (int i0 = 0; i0 < cnt; i0 += 8) {
                    float2 x0[8], x1[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        x0[i] = x1[i] = make_float2(0.f, 0.f);
                        if (i0 + i < cnt) {
                            const float* pr = eb + (size_t)(e0 + i0 + i) * estride + 2 + 4 * lane;
                            x0[i] = __ldcg(reinterpret_cast<const float2*>(pr));
                            x1[i] = __ldcg(reinterpret_cast<const float2*>(pr + 2));
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float wi = __shfl_sync(0xffffffffu, w, (i0 + i) & 31);
                        if (i0 + i < cnt && wi != 0.f) {
                            acc.x = fmaf(x0[i].x, wi, acc.x);
                            acc.y = fmaf(x0[i].y, wi, acc.y);
                            acc.z = fmaf(x1[i].x, wi, acc.z);
                            acc.w = fmaf(x1[i].y, wi, acc.w);
                        }
                    }
                }
                M = Mn;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4*>(a.out + d.head * kHeadDim + 4 * lane) =
                make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else if (a.write_partial_only) {
            float* op = a.out_part + d.head * kPartW;
            if (lane == 0) { op[0] = M; op[1] = L; }
            op[2 + 4 * lane + 0] = acc.x;
            op[2 + 4 * lane + 1] = acc.y;
            op[2 + 4 * lane + 2] = acc.z;
            op[2 + 4 * lane + 3] = acc.w;
        } else {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4*>(a.out + d.head * kHeadDim + 4 * lane) =
                make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        }
    };
    constexpr int kPre = (kFold && !kCoop) ? 6 : 1;
    const int64_t u_step = kCoop ? (int64_t)gridDim.x : (int64_t)gridDim.x * kWarps;
    int64_t u = kCoop ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * kWarps + warp;
    Unit pre[kPre];
    int n_pre = 0;
#pragma unroll
    for (int i = 0; i < kPre; ++i)
        if (u < units) {
            describe(u, pre[i]);
            ++n_pre;
            u += u_step;
        }
    pdl_wait();                                   // the split kernel's partials are complete from here on
    if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[1]));
#pragma unroll
    for (int i = 0; i < kPre; ++i)
        if (i < n_pre && pre[i].todo) process(pre[i]);
    for (; u < units; u += u_step) {
        Unit d;
        describe(u, d);
        if (d.todo) process(d);
    }
    if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[3]));
}

// LSE merge of n_parts stacked caller-visible partial buffers [n_parts][n_rows][130] -> out
// [n_rows][128], parts taken in index order (the multi-GPU merge after an all-gather, and the merge of a
// cascade's page chunks with the private part).  One warp per row, a lane owns four dims.  The loads
// are batched so that a row costs a few memory round trips whatever n_parts is: the (m, l) pairs come in
// 32 at a time (one per lane), the accumulators eight parts at a time; the arithmetic itself runs over
// the parts in order, one fused multiply-add per part and value, as a scalar loop would.
__global__ void __launch_bounds__(128) lse_combine_kernel(const float* __restrict__ parts, int n_parts, int n_rows,
                                                          float* __restrict__ out) {
    const int lane = (int)threadIdx.x & 31;
    const int row = (int)blockIdx.x * 4 + ((int)threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();                    // launched as a programmatic dependent of the kernels that write the parts
    if (row >= n_rows) return;
    const size_t part_stride = (size_t)n_rows * kPartW;
    const float* base = parts + (size_t)row * kPartW;
    float M = -INFINITY;
    for (int p0 = 0; p0 < n_parts; p0 += 32) {
        float2 ml = make_float2(-INFINITY, 0.f);
        if (p0 + lane < n_parts) ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)(p0 + lane) * part_stride));
        float mc = ml.y > 0.f ? ml.x : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, o));
        M = fmaxf(M, mc);
    }
    float L = 0.f;
    float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p0 = 0; p0 < n_parts; p0 += 32) {
        const int cnt = n_parts - p0 < 32 ? n_parts - p0 : 32;
        float2 ml = make_float2(-INFINITY, 0.f);
        if (lane < cnt) ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)(p0 + lane) * part_stride));
        const float w_mine = ml.y > 0.f ? __expf(ml.x - M) : 0.f;
        for (int i0 = 0; i0 < cnt; i0 += 8) {
            float2 x0[8], x1[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x0[i] = x1[i] = make_float2(0.f, 0.f);
                if (i0 + i < cnt) {
                    const float* pr = base + (size_t)(p0 + i0 + i) * part_stride + 2 + 4 * lane;
                    x0[i] = __ldcg(reinterpret_cast<const float2*>(pr));
                    x1[i] = __ldcg(reinterpret_cast<const float2*>(pr + 2));
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float w = __shfl_sync(0xffffffffu, w_mine, (i0 + i) & 31);
                const float lp = __shfl_sync(0xffffffffu, ml.y, (i0 + i) & 31);
                if (i0 + i < cnt && lp > 0.f) {
                    L = fmaf(lp, w, L);
                    A.x = fmaf(x0[i].x, w, A.x);
                    A.y = fmaf(x0[i].y, w, A.y);
                    A.z = fmaf(x1[i].x, w, A.z);
                    A.w = fmaf(x1[i].y, w, A.w);
                }
            }
        }
    }
    const bool some = L > 0.f;
    *reinterpret_cast<float4*>(out + (size_t)row * kHeadDim + 4 * lane) =
        make_float4(some ? A.x / L : 0.f, some ? A.y / L : 0.f, some ? A.z / L : 0.f, some ? A.w / L : 0.f);
}

// ---- exchange of partial rows between the GPUs of a node (one long session split over ranks) ---------------
//
// Every rank ends a layer with one un-normalised partial row (m, l, acc[128]) per (session, head) over its own
// pages.  The rows cross NVLink ONCE, one way: the warp that holds a finished row stores it straight into the
// exchange buffer of every peer (plain stores to the peer's memory, mapped through dev_ipc_open; no multicast,
// no tensor map over peer memory), then waits - bounded by wall clock - until the peers' rows have arrived in
// ITS OWN buffer, and merges all ranks' rows in rank order from local memory.
//
// There is no separate flag and no fence: a row travels as 16-byte words {value, epoch, value, epoch}; an
// aligned 8-byte half of such a word is written and read as one piece, so a reader that finds the expected
// epoch in both halves has the two values that were written with it (the protocol NCCL calls LL).  The epoch
// grows by one per exchange and a buffer has two slots (epoch parity), so what an earlier exchange left in a
// slot can never be mistaken for the current one.  A rank can be at most one epoch ahead of a peer that is
// still reading: its next exchange needs that peer's next row, which the peer sends only after the kernel of
// its previous exchange has finished (every kernel between two exchanges waits for its predecessor).
//
// Slot layout: [source rank 0..7][row][65 words of 16 B]; word 0 = (m, l), word 1 + 2i and 2 + 2i = the four
// accumulator values of lane i.
struct PeerSlots {
    unsigned char* base[kMaxPeerRanks];      // this epoch's slot in every rank's buffer
};

__device__ __forceinline__ void ll_store(void* p, float d0, float d1, uint32_t flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(d0)), "r"(flag),
                 "r"(__float_as_uint(d1)), "r"(flag)
                 : "memory");
}
__device__ __forceinline__ uint4 ll_load(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// One warp: sends its row (M, L, acc: lane i holds dims 4i..4i+3) to every peer, receives the peers' rows and
// merges all of them in rank order.  Returns false (and sets *status) when a peer's row did not arrive in time;
// then `acc` is left alone.  All 32 lanes must call it.
__device__ __forceinline__ bool exchange_and_merge(const PeerSlots& ps, const unsigned char* mine, size_t region_bytes, int n_ranks, int my_rank, int row,
                                          uint32_t epoch, unsigned long long timeout_ns, int32_t* status, float& M, float& L,
                                          float4& acc) {
    const int lane = (int)threadIdx.x & 31;
    const size_t row_off = (size_t)row * kLLRowBytes;
    // send: all stores of all peers are independent of one another
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {
        if (p < n_ranks && p != my_rank) {
            unsigned char* dst = ps.base[p] + (size_t)my_rank * region_bytes + row_off;
            if (lane == 0) ll_store(dst, M, L, epoch);
            ll_store(dst + 16 * (1 + 2 * lane), acc.x, acc.y, epoch);
            ll_store(dst + 16 * (2 + 2 * lane), acc.z, acc.w, epoch);
        }
    }
    // receive: poll this rank's own memory until every peer's words carry this epoch
    float pm[kMaxPeerRanks], pl[kMaxPeerRanks];
    float4 pa[kMaxPeerRanks];
    unsigned pending = 0;
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {
        pm[p] = -INFINITY;
        pl[p] = 0.f;
        pa[p] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p < n_ranks && p != my_rank) pending |= 1u << p;
    }
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool failed = false;
    // Two forms of the same poll, each measured where it is used.  Up to four ranks: every peer in one round, two loads
    // per peer and lane, the (m, l) word read by lane p alone and handed round by shuffle afterwards (config 5 on 4 GPUs:
    // 0.527 -> 0.507 ms per step).  More ranks: four peers at a time with every lane reading (m, l) itself - polling
    // all seven peers per round was 10 % slower on 8 GPUs (0.389 -> 0.427 ms).
    uint4 w0 = make_uint4(0u, 0u, 0u, 0u);
    const bool few = n_ranks <= 4;
    if (few) {
        while (__any_sync(0xffffffffu, pending != 0)) {
            uint4 w1[kMaxPeerRanks], w2[kMaxPeerRanks], w0n = w0;
#pragma unroll
            for (int p = 0; p < kMaxPeerRanks; ++p) {
                if (pending & (1u << p)) {
                    const unsigned char* src = mine + (size_t)p * region_bytes + row_off;
                    if (lane == p) w0n = ll_load(src);
                    w1[p] = ll_load(src + 16 * (1 + 2 * lane));
                    w2[p] = ll_load(src + 16 * (2 + 2 * lane));
                }
            }
#pragma unroll
            for (int p = 0; p < kMaxPeerRanks; ++p) {
                if (pending & (1u << p)) {
                    bool ok = w1[p].y == epoch && w1[p].w == epoch && w2[p].y == epoch && w2[p].w == epoch;
                    if (lane == p) ok = ok && w0n.y == epoch && w0n.w == epoch;
                    if (ok) {
                        if (lane == p) w0 = w0n;
                        pa[p] = make_float4(__uint_as_float(w1[p].x), __uint_as_float(w1[p].z), __uint_as_float(w2[p].x),
                                            __uint_as_float(w2[p].z));
                        pending &= ~(1u << p);
                    }
                }
            }
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (__any_sync(0xffffffffu, t1 - t0 > timeout_ns)) {     // a peer never got there: report, merge nothing
                failed = pending != 0;
                break;
            }
        }
    } else {
        while (__any_sync(0xffffffffu, pending != 0)) {
#pragma unroll
            for (int half = 0; half < kMaxPeerRanks; half += 4) {      // four peers at a time: all their loads first, then the checks
                uint4 v0[4], w1[4], w2[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int p = half + j;
                    if (pending & (1u << p)) {
                        const unsigned char* src = mine + (size_t)p * region_bytes + row_off;
                        v0[j] = ll_load(src);                       // every lane needs (m, l)
                        w1[j] = ll_load(src + 16 * (1 + 2 * lane));
                        w2[j] = ll_load(src + 16 * (2 + 2 * lane));
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int p = half + j;
                    if (pending & (1u << p)) {
                        const bool ok = v0[j].y == epoch && v0[j].w == epoch && w1[j].y == epoch && w1[j].w == epoch &&
                                        w2[j].y == epoch && w2[j].w == epoch;
                        if (ok) {
                            pm[p] = __uint_as_float(v0[j].x);
                            pl[p] = __uint_as_float(v0[j].z);
                            pa[p] = make_float4(__uint_as_float(w1[j].x), __uint_as_float(w1[j].z), __uint_as_float(w2[j].x),
                                                __uint_as_float(w2[j].z));
                            pending &= ~(1u << p);
                        }
                    }
                }
            }
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (__any_sync(0xffffffffu, t1 - t0 > timeout_ns)) {     // a peer never got there: report, merge nothing
                failed = pending != 0;
                break;
            }
        }
    }
    failed = __any_sync(0xffffffffu, failed);
    if (failed) {
        if (lane == 0 && status) atomicCAS(status, 0, NOVA_ERR_TIMEOUT);
        return false;
    }
    if (few) {
#pragma unroll
        for (int p = 0; p < kMaxPeerRanks; ++p) {             // (m, l) of peer p from the lane that read it
            const float m_p = __uint_as_float(__shfl_sync(0xffffffffu, w0.x, p));
            const float l_p = __uint_as_float(__shfl_sync(0xffffffffu, w0.z, p));
            if (p < n_ranks && p != my_rank) {
                pm[p] = m_p;
                pl[p] = l_p;
            }
        }
    }
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {             // this rank's own row sits at its place in the order
        if (p == my_rank) {
            pm[p] = M;
            pl[p] = L;
            pa[p] = acc;
        }
    }
    float Mx = -INFINITY;
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p)
        if (p < n_ranks && pl[p] > 0.f) Mx = fmaxf(Mx, pm[p]);
    float Ls = 0.f;
    float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {
        if (p < n_ranks && pl[p] > 0.f) {
            const float w = __expf(pm[p] - Mx);
            Ls = fmaf(pl[p], w, Ls);
            A.x = fmaf(pa[p].x, w, A.x);
            A.y = fmaf(pa[p].y, w, A.y);
            A.z = fmaf(pa[p].z, w, A.z);
            A.w = fmaf(pa[p].w, w, A.w);
        }
    }
    M = Mx;
    L = Ls;
    acc = A;
    return true;
}

// The exchange on its own, for partial rows that are already in memory (part [n_rows][130], written by the
// kernels before this one in the stream): one warp per row.  A one-warp CTA finds room on an SM next to a
// running attention CTA; a larger one would keep a next layer's CTAs off the SMs it takes.
__global__ void __launch_bounds__(32) lse_exchange_kernel(const float* __restrict__ part, PeerSlots ps, const unsigned char* mine, size_t region_bytes,
                                                          int n_ranks, int my_rank, int n_rows, uint32_t epoch,
                                                          unsigned long long timeout_ns, float* __restrict__ out,
                                                          int32_t* status) {
    const int row = (int)blockIdx.x;
    const int lane = (int)threadIdx.x;
    pdl_launch_dependents();
    pdl_wait();                                  // the rows come from the kernels before this one
    if (row >= n_rows) return;
    const float* pr = part + (size_t)row * kPartW;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(pr));
    const float2 a0 = __ldcg(reinterpret_cast<const float2*>(pr + 2 + 4 * lane));
    const float2 a1 = __ldcg(reinterpret_cast<const float2*>(pr + 4 + 4 * lane));
    float M = ml.x, L = ml.y;
    float4 acc = make_float4(a0.x, a0.y, a1.x, a1.y);
    if (!(L > 0.f)) {                            // nothing attended on this rank: send a clean empty row
        M = -INFINITY;
        L = 0.f;
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (!exchange_and_merge(ps, mine, region_bytes, n_ranks, my_rank, row, epoch, timeout_ns, status, M, L, acc)) return;
    const float inv = L > 0.f ? 1.f / L : 0.f;
    *reinterpret_cast<float4*>(out + (size_t)row * kHeadDim + 4 * lane) =
        make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// The merge that follows a split kernel with the exchange folded in: one CTA per (row, head) unit, the
// contributors of the split dealt out to its warps (as attn_combine_kernel<false, true>), then warp 0 sends the
// finished row to the peers, receives theirs and writes the output.  The split kernel ran with
// write_partial_only: rows that a single CTA covered (or that have no page on this rank) are in a.out_part.
__global__ void __launch_bounds__(32 * kCombineWarps) attn_combine_exchange_kernel(AttnLaunch a, int n_ctas_split, PeerSlots ps,
                                                                                   const unsigned char* mine, size_t region_bytes, int n_ranks, int my_rank,
                                                                                   uint32_t epoch, unsigned long long timeout_ns,
                                                                                   int32_t* xstatus) {
    __shared__ int s_prefix[kMaxRowsSmem + 1];
    __shared__ float s_ml[2 * kCombineWarps];
    __shared__ float4 s_acc[kCombineWarps * 32];
    const int lane = (int)threadIdx.x & 31;
    const int warp = (int)threadIdx.x >> 5;
#ifdef NOVA_TIMELINE
    unsigned long long* tl = (a.timeline && blockIdx.x < kTimelineCtas) ? a.timeline + kTimelineCtas * 8 + (size_t)blockIdx.x * 4 : nullptr;
#else
    constexpr unsigned long long* tl = nullptr;
#endif
    if (tl && threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[0]));
        tl[2] = smid;
    }
    pdl_launch_dependents();
    const int KVG = a.kv_group;
    const int G = a.n_heads / a.n_kv_heads;
    const int n_groups = a.n_kv_heads / KVG;
    const int heads_per_row = KVG * G;
    plan_build_prefix(a, s_prefix, n_groups);     // n_past: not written by the split kernel before us
    PlanView pv;
    pv.prefix = s_prefix;
    const int S = a.n_sessions * plan_nq(a);
    pv.rows_per_layer = S * n_groups;
    pv.n_groups = n_groups;
    pv.pages_per_layer = s_prefix[pv.rows_per_layer];
    pv.pages_total = pv.pages_per_layer * a.n_layers;
    pv.n_ctas = pv.pages_total < (int64_t)n_ctas_split ? (int)pv.pages_total : n_ctas_split;
    plan_finish(pv);
    pdl_wait();                                   // the split kernel's partials are complete from here on
    if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[1]));

    const int64_t units = (int64_t)pv.rows_per_layer * a.n_layers * heads_per_row;
    const size_t stride_c = (size_t)heads_per_row * kSlotW;
    for (int64_t u = blockIdx.x; u < units; u += gridDim.x) {
        const int64_t v = u / heads_per_row;
        const int hr = (int)(u - v * heads_per_row);
        const int row = (int)(v % pv.rows_per_layer);
        const int ll = (int)(v / pv.rows_per_layer);
        const bool no_pages = pv.pages_total == 0 || s_prefix[row + 1] == s_prefix[row];
        int c_first = 0, n = 0;
        if (!no_pages) {
            const int64_t row_begin = (int64_t)ll * pv.pages_per_layer + s_prefix[row];
            const int64_t row_end = (int64_t)ll * pv.pages_per_layer + s_prefix[row + 1];
            c_first = plan_owner(pv, row_begin);
            n = plan_owner(pv, row_end - 1) - c_first + 1;
        }
        const int s = row / n_groups, grp = row - s * n_groups;
        const int64_t head = ((int64_t)ll * S + s) * a.n_heads + (int64_t)(grp * KVG) * G + hr;
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n <= 1) {                 // the split kernel left this row's partial (or an empty row) in out_part
            if (warp == 0) {
                const float* pr = a.out_part + head * kPartW;
                const float2 ml = __ldcg(reinterpret_cast<const float2*>(pr));
                const float2 y0 = __ldcg(reinterpret_cast<const float2*>(pr + 2 + 4 * lane));
                const float2 y1 = __ldcg(reinterpret_cast<const float2*>(pr + 4 + 4 * lane));
                if (ml.y > 0.f) {
                    M = ml.x;
                    L = ml.y;
                    acc = make_float4(y0.x, y0.y, y1.x, y1.y);
                }
            }
        } else {
            const float* base = a.part + ((size_t)(c_first + v) * heads_per_row + (size_t)hr) * kSlotW;
            for (int c0 = 32 * warp; c0 < n; c0 += 32 * kCombineWarps)
                fold_contributors(base + (size_t)c0 * stride_c, stride_c, n - c0 < 32 ? n - c0 : 32, lane, M, L, acc);
            if (lane == 0) { s_ml[2 * warp] = M; s_ml[2 * warp + 1] = L; }
            s_acc[warp * 32 + lane] = acc;
            __syncthreads();
            if (warp == 0) {
                float Mx = -INFINITY;
#pragma unroll
                for (int w = 0; w < kCombineWarps; ++w)
                    if (s_ml[2 * w + 1] > 0.f) Mx = fmaxf(Mx, s_ml[2 * w]);
                L = 0.f;
                acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < kCombineWarps; ++w) {
                    const float lw = s_ml[2 * w + 1];
                    if (lw > 0.f) {
                        const float cw = __expf(s_ml[2 * w] - Mx);
                        const float4 x = s_acc[w * 32 + lane];
                        L = fmaf(lw, cw, L);
                        acc.x = fmaf(x.x, cw, acc.x);
                        acc.y = fmaf(x.y, cw, acc.y);
                        acc.z = fmaf(x.z, cw, acc.z);
                        acc.w = fmaf(x.w, cw, acc.w);
                    }
                }
                M = L > 0.f ? Mx : -INFINITY;
            }
            __syncthreads();
        }
        if (warp != 0) continue;
        if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[2]));     // (overwrites %smid) the rank's own row is ready
        if (!exchange_and_merge(ps, mine, region_bytes, n_ranks, my_rank, (int)head, epoch, timeout_ns, xstatus, M, L, acc)) continue;
        const float inv = L > 0.f ? 1.f / L : 0.f;
        *reinterpret_cast<float4*>(a.out + head * kHeadDim + 4 * lane) =
            make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[3]));
    }
}

}  // namespace

int launch_attn_combine(const AttnLaunch& a, int n_ctas_split, cudaStream_t s) {
    if (a.n_sessions <= 0 || a.n_layers <= 0) return NOVA_OK;
    const int G = a.n_heads / a.n_kv_heads;
    const int64_t units = (int64_t)a.n_sessions * (a.n_q > 1 ? a.n_q : 1) * (a.n_kv_heads / a.kv_group) * a.n_layers *
                          (int64_t)(a.kv_group * G);
    // Few CTAs, each looping over its share: every merge CTA must be able to start while the split
    // kernel still runs (next to a split CTA), because the next layer's programmatic launch waits for
    // all of them to have started, and they must not pile up on the SMs the split kernel left free for
    // that next layer.  Measured (64 sessions x 8192 tokens, 14B shape): up to 74 CTAs 6.13 TB/s,
    // 120: 5.94, 148: 5.89.
    const int warps = a.n_extra > 0 ? kFoldWarps : kCombineWarps;
    int64_t ctas = (units + warps - 1) / warps;
#ifndef NOVA_COMBINE_MAX_CTAS
#define NOVA_COMBINE_MAX_CTAS 76
#endif
    // (a launch that covers several layers is not part of such a chain and takes up to 8 CTAs per SM)
    // (the cascade's merge, n_extra > 0, is part of such a chain too: its CTAs share the SMs of the split over the private
    // pages - one beside each split CTA - because the shared-prefix tiles fill theirs)
    int64_t cap = (a.n_layers == 1 && a.pdl && (a.pdl_spare || a.n_extra > 0)) ? NOVA_COMBINE_MAX_CTAS : sm_count() * 8;
    if (a.n_layers == 1 && a.pdl && a.n_extra > 0 && n_ctas_split >= 8 && n_ctas_split < cap) cap = n_ctas_split;
    if (ctas > cap) ctas = cap;
    // Always a programmatic dependent of the split kernel launched just before it.
    const bool coop = a.n_extra == 0 && units <= NOVA_COMBINE_MAX_CTAS;      // few units: one CTA per unit
    if (coop) ctas = units;
    const cudaError_t le = a.n_extra > 0
        ? launch_kernel_pdl(attn_combine_kernel<true>, dim3((unsigned)ctas), dim3(32 * kFoldWarps), 0, s, true, a, n_ctas_split)
        : coop ? launch_kernel_pdl(attn_combine_kernel<false, true>, dim3((unsigned)ctas), dim3(32 * kCombineWarps), 0, s, true, a, n_ctas_split)
               : launch_kernel_pdl(attn_combine_kernel<false>, dim3((unsigned)ctas), dim3(32 * kCombineWarps), 0, s, true, a, n_ctas_split);
    if (le != cudaSuccess) {
        set_cuda_error(le, "combine launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

int launch_lse_combine(const float* parts, int n_parts, int n_rows, float* out, cudaStream_t s) {
    if (n_rows <= 0 || n_parts <= 0) return NOVA_OK;
    // always a programmatic dependent: the kernel waits for everything before it right at its start, so this is
    // the plain stream order with the launch latency hidden (and a next layer's kernels may be scheduled early)
    const cudaError_t le = launch_kernel_pdl(lse_combine_kernel, dim3((unsigned)((n_rows + 3) / 4)), dim3(128), 0, s, true, parts,
                                             n_parts, n_rows, out);
    if (le != cudaSuccess) {
        set_cuda_error(le, "merge launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab

namespace novab {

size_t peer_region_bytes(int n_rows) { return ((size_t)n_rows * kLLRowBytes + 127) / 128 * 128; }

static void fill_slots(PeerSlots& ps, void* const* slot_base, int n_ranks) {
    for (int i = 0; i < kMaxPeerRanks; ++i) ps.base[i] = i < n_ranks ? static_cast<unsigned char*>(slot_base[i]) : nullptr;
}

int launch_lse_exchange(const float* part, void* const* slot_base, int n_ranks, int my_rank, int n_rows, long long epoch,
                        unsigned long long timeout_ns, float* out, int32_t* status, cudaStream_t s) {
    if (n_rows <= 0) return NOVA_OK;
    PeerSlots ps;
    fill_slots(ps, slot_base, n_ranks);
    const cudaError_t le = launch_kernel_pdl(lse_exchange_kernel, dim3((unsigned)n_rows), dim3(32), 0, s, true, part, ps,
                                             static_cast<const unsigned char*>(slot_base[my_rank]), peer_region_bytes(n_rows), n_ranks, my_rank, n_rows, (uint32_t)epoch, timeout_ns, out,
                                             status);
    if (le != cudaSuccess) {
        set_cuda_error(le, "exchange launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

// After a split kernel that ran with write_partial_only (one layer): merge + exchange + output in one launch.
int launch_attn_combine_exchange(const AttnLaunch& a, int n_ctas_split, void* const* slot_base, int n_ranks, int my_rank,
                                 long long epoch, unsigned long long timeout_ns, int32_t* status, cudaStream_t s) {
    if (a.n_sessions <= 0 || a.n_layers != 1 || !a.out_part || !a.out) return NOVA_ERR_INVALID;
    const int n_rows = a.n_sessions * a.n_heads;
    PeerSlots ps;
    fill_slots(ps, slot_base, n_ranks);
    // one CTA per (row, head); more units than that loop (the CTAs wait for the peers, so they are kept few enough
    // to be resident together next to the attention CTAs)
    int ctas = n_rows;
    const int cap = 2 * sm_count();
    if (ctas > cap) ctas = cap;
    const cudaError_t le = launch_kernel_pdl(attn_combine_exchange_kernel, dim3((unsigned)ctas), dim3(32 * kCombineWarps), 0, s, true,
                                             a, n_ctas_split, ps, static_cast<const unsigned char*>(slot_base[my_rank]),
                                             peer_region_bytes(n_rows), n_ranks, my_rank, (uint32_t)epoch,
                                             timeout_ns, status);
    if (le != cudaSuccess) {
        set_cuda_error(le, "merge + exchange launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
