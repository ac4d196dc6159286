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
template <bool kFold, bool kCoop = false>
__global__ void __launch_bounds__(32 * kCombineWarps) attn_combine_kernel(AttnLaunch a, int n_ctas_split) {
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
    pdl_wait();                                   // the split kernel's partials are complete from here on
    if (tl && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tl[1]));
    PlanView pv;
    pv.prefix = s_prefix;
    const int S = a.n_sessions * plan_nq(a);        // units
    pv.rows_per_layer = S * n_groups;
    pv.n_groups = n_groups;
    pv.pages_per_layer = s_prefix[pv.rows_per_layer];
    pv.pages_total = pv.pages_per_layer * a.n_layers;
    pv.n_ctas = pv.pages_total < (int64_t)n_ctas_split ? (int)pv.pages_total : n_ctas_split;
    plan_finish(pv);
    if (pv.pages_total == 0) return;

    const int64_t units = (int64_t)pv.rows_per_layer * a.n_layers * heads_per_row;
    const size_t stride_c = (size_t)heads_per_row * kSlotW;
    for (int64_t u = kCoop ? (int64_t)blockIdx.x : (int64_t)blockIdx.x * kCombineWarps + warp; u < units;
         u += kCoop ? (int64_t)gridDim.x : (int64_t)gridDim.x * kCombineWarps) {
        const int64_t v = u / heads_per_row;
        const int hr = (int)(u - v * heads_per_row);            // kv head in group * G + query head
        const int row = (int)(v % pv.rows_per_layer);
        constexpr bool fold = kFold;                             // more parts to fold in: every row is ours to finish
        const bool no_pages = s_prefix[row + 1] == s_prefix[row];
        if (no_pages && !fold) continue;                         // no pages: written by the split kernel
        const int ll = (int)(v / pv.rows_per_layer);
        const int64_t row_begin = (int64_t)ll * pv.pages_per_layer + s_prefix[row];
        const int64_t row_end = (int64_t)ll * pv.pages_per_layer + s_prefix[row + 1];
        int c_first, n;
        if constexpr (kFold) {
            c_first = no_pages ? 0 : plan_owner(pv, row_begin);
            n = no_pages ? 0 : plan_owner(pv, row_end - 1) - c_first + 1;
        } else {
            c_first = plan_owner(pv, row_begin);
            n = plan_owner(pv, row_end - 1) - c_first + 1;
            if (n == 1) continue;                                 // written by the split kernel
        }
        const int s = row / n_groups, grp = row - s * n_groups;
        const int64_t head = ((int64_t)ll * S + s) * a.n_heads + (int64_t)(grp * KVG) * G + hr;
        const float* base = a.part + ((size_t)(c_first + v) * heads_per_row + (size_t)hr) * kSlotW;

        // Contributors are taken 32 at a time: lane i holds (m, l) of contributor c0 + i while every
        // lane pulls its 4 dims of all 32 accumulators.  None of these loads depends on another, so a
        // chunk costs ONE memory round trip (a round trip is ~1 us here; a row usually fits one chunk).
        float M = -INFINITY, L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        if constexpr (kFold) if (n == 1) {            // the split kernel left this row's partial (m, l, acc) in out_part
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
        for (int c0 = kCoop ? 32 * warp : 0; c0 < ((kFold && n == 1) ? 0 : n); c0 += kCoop ? 32 * kCombineWarps : 32) {
            const int cnt = n - c0 < 32 ? n - c0 : 32;
            const float* src = base + (size_t)c0 * stride_c;
            float2 ml = make_float2(-INFINITY, 0.f);
            if (lane < cnt) ml = __ldcg(reinterpret_cast<const float2*>(src + (size_t)lane * stride_c));
            float4 x[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < cnt) x[i] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)i * stride_c + 4 + 4 * lane));
            }
            const float mc = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
            const float Mn = fmaxf(M, mc);
            if (Mn == -INFINITY) continue;                       // nothing attended in this chunk or before
            const float corr = __expf(M - Mn);                   // 0 on the first chunk (M = -inf)
            const float w = ml.y > 0.f ? __expf(ml.x - Mn) : 0.f;
            L = fmaf(L, corr, warp_sum(ml.y * w));
            acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const float wi = __shfl_sync(0xffffffffu, w, i);
                if (wi != 0.f) {     // a slot with l == 0 carries no accumulator (and may hold anything)
                    acc.x = fmaf(x[i].x, wi, acc.x);
                    acc.y = fmaf(x[i].y, wi, acc.y);
                    acc.z = fmaf(x[i].z, wi, acc.z);
                    acc.w = fmaf(x[i].w, wi, acc.w);
                }
            }
            M = Mn;
        }
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
            if (warp != 0) continue;
        }
        if constexpr (kFold) {
            // the extra parts (a cascade's chunks over the shared pages), 32 (m, l) pairs and 8 accumulators at a time
            const size_t estride = (size_t)S * a.n_heads * kPartW;
            const float* eb = a.extra_parts + head * kPartW;
            for (int e0 = 0; e0 < a.n_extra; e0 += 32) {
                const int cnt = a.n_extra - e0 < 32 ? a.n_extra - e0 : 32;
                float2 ml = make_float2(-INFINITY, 0.f);
                if (lane < cnt) ml = __ldcg(reinterpret_cast<const float2*>(eb + (size_t)(e0 + lane) * estride));
                const float mc = warp_max(ml.y > 0.f ? ml.x : -INFINITY);
                const float Mn = fmaxf(M, mc);
                if (Mn == -INFINITY) continue;
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
            *reinterpret_cast<float4*>(a.out + head * kHeadDim + 4 * lane) =
                make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else if (a.write_partial_only) {
            float* op = a.out_part + head * kPartW;
            if (lane == 0) { op[0] = M; op[1] = L; }
            op[2 + 4 * lane + 0] = acc.x;
            op[2 + 4 * lane + 1] = acc.y;
            op[2 + 4 * lane + 2] = acc.z;
            op[2 + 4 * lane + 3] = acc.w;
        } else {
            const float inv = L > 0.f ? 1.f / L : 0.f;
            *reinterpret_cast<float4*>(a.out + head * kHeadDim + 4 * lane) =
                make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        }
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

// The same merge with the all-gather folded in: rank r's partial rows live in rank r's own memory
// (an exchange slot: a 128-byte header whose first 8 bytes are the epoch flag, then n_rows x 130
// floats) and every rank reads all of them over NVLink.  Each CTA first publishes this rank's flag
// (its rows were written by kernels that precede this one in the stream), then waits - bounded by
// wall clock - until every peer's flag has reached the epoch, then merges in rank order.  The kernels
// that wait on one another run on different GPUs, never on one.
struct PeerSlots {
    unsigned char* base[kMaxPeerRanks];
};

__device__ __forceinline__ void st_relaxed_sys(long long* p, long long v) {
    asm volatile("st.relaxed.sys.global.s64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ long long ld_relaxed_sys(const long long* p) {
    long long v;
    asm volatile("ld.relaxed.sys.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

// One warp per row (a one-warp CTA finds room on an SM next to a running attention CTA, a four-warp one
// does not and would keep the next layer's CTAs off the SMs it takes).
__global__ void __launch_bounds__(32) lse_merge_peers_kernel(PeerSlots ps, int n_ranks, int my_rank, int n_rows,
                                                             long long epoch, unsigned long long timeout_ns,
                                                             float* __restrict__ out, int32_t* status) {
    const int row = (int)blockIdx.x;
    const int lane = (int)threadIdx.x;
    // Launched as a programmatic dependent of whatever precedes it in the stream (the local merge of
    // this layer): the CTAs may become resident early and let a next layer's attention launch start, and
    // wait here until the kernels that wrote this rank's rows have finished.
    pdl_launch_dependents();
    pdl_wait();
    // Publish with a plain system-scope store: the rows were written by kernels that had completed before
    // this one started, so they are in this GPU's L2 (where a peer's loads are served) already; a release
    // fence here cost ~3 us and ordered nothing more.
    if (lane == 0) st_relaxed_sys(reinterpret_cast<long long*>(ps.base[my_rank]), epoch);   // the same value from every CTA
    int ok = 1;
    if (lane < n_ranks && lane != my_rank) {
        // poll with plain system-scope loads (an acquire on every poll would pay a fence per round trip)
        const long long* flag = reinterpret_cast<const long long*>(ps.base[lane]);
        unsigned long long t0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
        while (ld_relaxed_sys(flag) < epoch) {
            unsigned long long t1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
            if (t1 - t0 > timeout_ns) {            // the peer never got there: report, do not read its rows
                ok = 0;
                if (status) atomicCAS(status, 0, NOVA_ERR_TIMEOUT);
                break;
            }
        }
    }
    // The row loads below bypass the caches (ld.cv) and are issued only after the flag loads have returned
    // (the loop exit depends on them), so they see what the peer's earlier kernels wrote; no fence (~3 us).
    ok = __all_sync(0xffffffffu, ok);
    if (!ok || row >= n_rows) return;
    // All ranks' values first, as independent loads: a load from a peer is a ~2.5 us NVLink round trip,
    // and one after the other (as a merge over local memory would do it) they would add up.
    float2 ml[kMaxPeerRanks], a0[kMaxPeerRanks], a1[kMaxPeerRanks];
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {
        ml[p] = make_float2(-INFINITY, 0.f);
        a0[p] = a1[p] = make_float2(0.f, 0.f);
        if (p < n_ranks) {
            const float* pr = reinterpret_cast<const float*>(ps.base[p] + kPeerSlotHeader) + (size_t)row * kPartW;
            ml[p] = __ldcv(reinterpret_cast<const float2*>(pr));
            a0[p] = __ldcv(reinterpret_cast<const float2*>(pr + 2 + 4 * lane));
            a1[p] = __ldcv(reinterpret_cast<const float2*>(pr + 4 + 4 * lane));
        }
    }
    float M = -INFINITY;
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p)
        if (p < n_ranks && ml[p].y > 0.f) M = fmaxf(M, ml[p].x);
    float L = 0.f;
    float4 A = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kMaxPeerRanks; ++p) {
        if (p < n_ranks && ml[p].y > 0.f) {
            const float w = __expf(ml[p].x - M);
            L = fmaf(ml[p].y, w, L);
            A.x = fmaf(a0[p].x, w, A.x);
            A.y = fmaf(a0[p].y, w, A.y);
            A.z = fmaf(a1[p].x, w, A.z);
            A.w = fmaf(a1[p].y, w, A.w);
        }
    }
    const bool some = L > 0.f;
    *reinterpret_cast<float4*>(out + (size_t)row * kHeadDim + 4 * lane) =
        make_float4(some ? A.x / L : 0.f, some ? A.y / L : 0.f, some ? A.z / L : 0.f, some ? A.w / L : 0.f);
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
    int64_t ctas = (units + kCombineWarps - 1) / kCombineWarps;
#ifndef NOVA_COMBINE_MAX_CTAS
#define NOVA_COMBINE_MAX_CTAS 76
#endif
    // (a launch that covers several layers is not part of such a chain and takes up to 8 CTAs per SM)
    const int64_t cap = (a.n_layers == 1 && a.pdl && a.pdl_spare) ? NOVA_COMBINE_MAX_CTAS : sm_count() * 8;
    if (ctas > cap) ctas = cap;
    // Always a programmatic dependent of the split kernel launched just before it.
    const bool coop = a.n_extra == 0 && units <= NOVA_COMBINE_MAX_CTAS;      // few units: one CTA per unit
    if (coop) ctas = units;
    const cudaError_t le = a.n_extra > 0
        ? launch_kernel_pdl(attn_combine_kernel<true>, dim3((unsigned)ctas), dim3(32 * kCombineWarps), 0, s, true, a, n_ctas_split)
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

int launch_lse_merge_peers(void* const* slot_base, int n_ranks, int my_rank, int n_rows, long long epoch,
                           unsigned long long timeout_ns, float* out, int32_t* status, cudaStream_t s) {
    if (n_rows <= 0) return NOVA_OK;
    PeerSlots ps;
    for (int i = 0; i < kMaxPeerRanks; ++i) ps.base[i] = i < n_ranks ? static_cast<unsigned char*>(slot_base[i]) : nullptr;
    const cudaError_t le = launch_kernel_pdl(lse_merge_peers_kernel, dim3((unsigned)n_rows), dim3(32), 0, s, true, ps, n_ranks,
                                             my_rank, n_rows, epoch, timeout_ns, out, status);
    if (le != cudaSuccess) {
        set_cuda_error(le, "peer merge launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
