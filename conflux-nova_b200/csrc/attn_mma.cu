// attn_mma.cu — paged split-K decode attention for fp16 pools, tensor-core form.
// Same contract as attn_simt.cu (replaces fa_split_paged_kernel + fa_combine_kernel,
// src/kernel/attn.cu:197-289,163-191 of the reference, for all sessions / layers of a launch),
// built for the B200 memory system:
//
//   * One persistent CTA per SM (two for 2-kv-head models).  A producer warp walks the CTA's
//     stream-K page range and brings WHOLE pages into shared memory with TMA tensor copies
//     (cp.async.bulk.tensor, no multicast): a page of one pool is [16 slots][NKV][128] fp16 and
//     is fetched as two boxes [64 dims][16 slots][kv group] with the 128-byte swizzle, so that
//     each kv head's 16 key rows sit in 16 consecutive 128-byte lines.  A ring of
//     kStages page sets (K+V, 32 KiB each at 4 kv heads) keeps ~128 KiB per SM in flight.
//   * One consumer warp per kv head.  The G = NH/NKV query heads of that kv head are the rows
//     of an m16n8k16 tile: S = Q.K^T and O += P.V run on mma.sync (fp16 inputs, fp32
//     accumulate) with bank-conflict-free ldmatrix reads; q is split into fp16 hi + lo parts so
//     the scores keep fp32-level accuracy; the online softmax (exp2 domain) and all sums are
//     fp32.  A scalar fp32 version cannot keep up with HBM here: at G = 7 it needs ~3600 FMAs per
//     512 bytes of KV, more than the SM's FP32 pipes deliver at 20+ B/clk.
//   * Full/empty mbarriers hand the stages over; every wait is bounded by a wall-clock limit and
//     reports NOVA_ERR_TIMEOUT through the status word instead of spinning forever.
//   * Work split and partial slots are those of attn_plan.cuh; rows shared by several CTAs are
//     merged by the combine kernel that follows (attn_combine.cu) - no flags between CTAs.
//   * K/V copies carry an L2 evict-first hint: pages are read once per step, everything else
//     (tables, n_past, q, partial slots) is re-read and should stay in L2.
//   * Under a programmatic launch chain (one layer per launch, each launch a dependent of the one
//     before) the kernel computes without waiting, parks finished segments in shared memory and
//     waits for the previous kernels once, right before its first output write; such a launch
//     leaves NOVA_ATTN_SPARE_SMS SMs without a CTA so that consecutive layers overlap.
#include <type_traits>

#include "attn_plan.cuh"
#include "mma_common.cuh"

namespace novab {
namespace {

#ifndef NOVA_ATTN_STAGES
#define NOVA_ATTN_STAGES 4
#endif
constexpr int kStages = NOVA_ATTN_STAGES;   // page sets in flight per CTA; more only adds queueing delay in HBM
// A launch that is a programmatic dependent of the previous layer's kernels leaves this many SMs
// without a CTA of its own.  With one CTA for every SM each layer's CTAs all start at the same moment
// (when the previous layer's exit) and all sit in their ~3 us start-up (work split, first table
// entries, first pages) together, HBM idle; with a few SMs to spare the next layer's first CTAs start
// early, the layers drift apart and some CTAs are always streaming while others start.  Measured on
// 8 sessions x 2-8k tokens (7B shape): 0 spare 0.588 ms per 28-layer step, 4: 0.523, 8: 0.510,
// 12: 0.507, 16: 0.511, 32: 0.529.
#ifndef NOVA_ATTN_EVICT_FIRST
#define NOVA_ATTN_EVICT_FIRST 1
#endif
#ifndef NOVA_ATTN_SPARE_SMS
#define NOVA_ATTN_SPARE_SMS 12
#endif

// A CTA whose page range crosses a row boundary finishes a segment early.  Under a programmatic
// dependent launch its result cannot be written yet (the previous layer's merge may still read the
// partial slots), and waiting there would stall the rest of the CTA's range, so up to kStashSlots
// finished segments are parked in shared memory: per thread its 32 accumulator values, m, l and the
// segment's address words.
#ifndef NOVA_ATTN_STASH
#define NOVA_ATTN_STASH 2
#endif
constexpr int kStashSlots = NOVA_ATTN_STASH;
constexpr int kStashWords = 38;

// kF32: fp32 pools (the reference's own format).  The page copies then bring fp32 rows - boxes of [32 dims][16 slots]
// [KVG], eight per page set, two page sets of 64 KiB in flight - and each consumer warp first converts its kv head's
// 16 x 128 K and V values to fp16 into ONE shared page set laid out exactly like an fp16 stage (the raw stage is handed
// back to the producer as soon as that is done); from there on the tile arithmetic is the fp16 kernel's.  K and V are
// therefore rounded to fp16 on their way into the tensor cores (values beyond the fp16 range would saturate: the SIMT
// kernel stays the default for fp32 pools); 16-token pages only in this form.  The fused append
// stores the new token's fp32 rows into the pool and their fp16 roundings into the converted page set.
template <int KVG, bool kF32 = false>
struct MmaCfg {
    static constexpr int kBoxBytes = KVG * 16 * 128;          // one [64 dims fp16 | 32 dims fp32][16 slots][KVG] box
    static constexpr int kConvBytes = 4 * kBoxBytes;           // an fp16 page set: K lo/hi dims + V lo/hi dims
    static constexpr int kStageBytes = kF32 ? 8 * kBoxBytes : kConvBytes;
    static constexpr int kNStages = kF32 ? 2 : kStages;
    static constexpr int kStashBytes = kStashSlots * KVG * kStashWords * 128;   // finished segments parked until the first write
    static constexpr int kSmemBytes = kNStages * kStageBytes + (kF32 ? kConvBytes : 0) + kStashBytes + 1024;
    static constexpr int kThreads = 32 * (KVG + 1);
    static constexpr int kCtasPerSm = 4 / KVG >= 1 ? 4 / KVG : 1;
};

template <int KVG, bool kF32 = false>
__global__ void __launch_bounds__(MmaCfg<KVG, kF32>::kThreads, MmaCfg<KVG, kF32>::kCtasPerSm)
attn_mma_kernel(AttnLaunch a, const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv) {
    using Cfg = MmaCfg<KVG, kF32>;
    constexpr int kNStages = Cfg::kNStages;
    extern __shared__ unsigned char smem_raw[];
    __shared__ int s_prefix[kMaxRowsSmem + 1];
    __shared__ int s_slice[kMaxRowsSmem];
    __shared__ int s_keys[kMaxRowsSmem];          // keys seen by each unit (n_past + this step's token), fetched once
    __shared__ __align__(8) unsigned long long s_full[kStages];
    __shared__ __align__(8) unsigned long long s_empty[kStages];
    __shared__ int s_kcount[kStages];
    __shared__ int s_phys[kStages];
    __shared__ int s_abort;

    const int lane = (int)threadIdx.x & 31;
    const int warp = (int)threadIdx.x >> 5;
    const int G = a.n_heads / a.n_kv_heads;
    const int n_groups = a.n_kv_heads / KVG;
    const int NQ = plan_nq(a);
    const int NH = a.n_heads, S = a.n_sessions * NQ;     // S counts units (session x query token)
    const int heads_per_row = KVG * G;
    const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const PageGeom geo = page_geom(a.kv_shift);
    const int tpp_mask = (1 << geo.tpp_shift) - 1;

    pdl_launch_dependents();      // the combine kernel may be scheduled; it waits for this grid to finish
#ifdef NOVA_TIMELINE      // profiling build only: per-CTA %globaltimer stamps
    unsigned long long* tl = (a.timeline && blockIdx.x < kTimelineCtas) ? a.timeline + (size_t)blockIdx.x * 8 : nullptr;
#else
    constexpr unsigned long long* tl = nullptr;
#endif
    if (tl && threadIdx.x == 0) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        tl[0] = now_ns();
        tl[7] = smid;
    }
    if (threadIdx.x == 32 * (Cfg::kThreads / 32 - 1)) {      // the producer's lane 0; warp 0 is busy with the prefix scan
        for (int i = 0; i < kNStages; ++i) {
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&s_empty[i]), KVG);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == KVG && lane == 0) {     // the tensor maps are needed right after the first table entry
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmk) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmv) : "memory");
    }
    if (geo.tile_keys < kTileKeysMax) {
        // 8-token pages fill only the first 8 of a stage's 16 key rows per kv head.  The other rows take part in the
        // tile arithmetic with weight zero, so they must hold finite values: clear the ring once; the page copies
        // never touch those rows afterwards.
        for (uint32_t off = threadIdx.x * 16u; off < (uint32_t)(kNStages * Cfg::kStageBytes); off += blockDim.x * 16u)
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(stage0 + off), "r"(0u) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    plan_build_prefix(a, s_prefix, n_groups, s_slice, s_keys);   // ends with __syncthreads()

    PlanView pv;
    pv.prefix = s_prefix;
    pv.rows_per_layer = S * n_groups;
    pv.n_groups = n_groups;
    pv.pages_per_layer = s_prefix[pv.rows_per_layer];
    pv.pages_total = pv.pages_per_layer * a.n_layers;
    pv.n_ctas = pv.pages_total < (int64_t)gridDim.x ? (int)pv.pages_total : (int)gridDim.x;
    plan_finish(pv);

    const int g = lane >> 2, t = lane & 3;   // fragment row (query head within the kv head) / quad lane

    // Rows without any page in the window: "nothing attended".
    if (warp < KVG) {
        const int64_t rows_total = (int64_t)pv.rows_per_layer * a.n_layers;
        bool waited = a.pdl == 0;
        for (int64_t v = blockIdx.x; v < rows_total; v += gridDim.x) {
            const int row = (int)(v % pv.rows_per_layer);
            if (s_prefix[row + 1] != s_prefix[row]) continue;
            if (!waited) { pdl_wait(); waited = true; }      // an output write: the chain's one rule applies here too
            const int ll = (int)(v / pv.rows_per_layer);
            const int s = row / n_groups, grp = row - s * n_groups;
            const int kvh = grp * KVG + warp;
            if (g < G) {
                const int64_t head = ((int64_t)ll * S + s) * NH + (int64_t)kvh * G + g;
                if (a.write_partial_only) {
                    float* op = a.out_part + head * kPartW;
                    if (t == 0) { op[0] = -INFINITY; op[1] = 0.f; }
                    for (int j = 0; j < 16; ++j)
                        *reinterpret_cast<float2*>(op + 2 + 8 * j + 2 * t) = make_float2(0.f, 0.f);
                } else {
                    float* op = a.out + head * kHeadDim;
                    for (int j = 0; j < 16; ++j)
                        *reinterpret_cast<float2*>(op + 8 * j + 2 * t) = make_float2(0.f, 0.f);
                }
            }
        }
    }
    if (pv.pages_total == 0 || (int)blockIdx.x >= pv.n_ctas) return;

    const int64_t lo = plan_cta_begin(pv, (int)blockIdx.x);
    const int64_t hi = plan_cta_begin(pv, (int)blockIdx.x + 1);
    if (tl && threadIdx.x == 0) tl[1] = now_ns();

    // ------------------------------------------------------------------ producer warp
    if (warp == KVG) {
        // The whole warp walks the CTA's page range in batches of up to 32 pages: each lane fetches
        // one block-table entry of the NEXT batch while lane 0 issues the TMA copies of the current
        // one, so a table read (a ~1 us round trip when it misses) never stops the copy stream.
#if NOVA_ATTN_EVICT_FIRST
        const unsigned long long kv_policy = l2_policy_evict_first();
#endif
        struct Batch {
            int count;              // 0: no more work
            int layer, group, n_keys, page0;
            const int32_t* table;
        };
        int64_t pos = lo;
        Segment sg;
        sg.page_count = 0;
        int seg_done = 0, seg_first_page = 0, seg_keys = 0;
        const int32_t* seg_table = nullptr;
        bool first_segment = true;
        auto next_batch = [&]() -> Batch {
            Batch b;
            b.count = 0;
            while (seg_done >= sg.page_count) {          // open the next segment that has real pages
                if (pos >= hi) return b;
                sg = plan_segment(pv, pos, hi, a.row_setup_pages);
                pos += sg.span;
                seg_done = 0;
                const int s = sg.session;
                seg_keys = s_keys[s];
                int n_pages_row;
                plan_pages_of_keys(a, seg_keys, seg_first_page, n_pages_row);
                seg_table = a.table_base + (int64_t)s_slice[s / NQ] * a.table_stride;
                // Warm L2 with what the consumers will ask for when they reach this segment.  Not for the
                // CTA's first segment: the consumers fetch that themselves at this very moment, and the
                // hints would only delay the first page copies.
                if (first_segment) { first_segment = false; continue; }
                {
                const float* qrow = a.q + (((int64_t)sg.layer_local * S + s) * NH + (int64_t)sg.group * KVG * G) * kHeadDim;
                for (int i = lane; i < heads_per_row * 4; i += 32)
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(qrow + i * 32));
                if (a.fuse_append) {
                    const int64_t tok = (((int64_t)sg.layer_local * S + s) * a.n_kv_heads + (int64_t)sg.group * KVG) * kHeadDim;
                    for (int i = lane; i < KVG * 4; i += 32) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.k_new + tok + i * 32));
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(a.v_new + tok + i * 32));
                    }
                    const int pn = seg_keys - a.keys_add;      // n_past[s]
                    if (lane < 4 && pn >= 0 && pn < a.rope_rows)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"((lane < 2 ? a.rope_cs : a.rope_sn) +
                                                                       (int64_t)pn * (kHeadDim / 2) + (lane & 1) * 32));
                }
                }
            }
            b.count = sg.page_count - seg_done < 32 ? sg.page_count - seg_done : 32;
            b.layer = a.layer0 + sg.layer_local;
            b.group = sg.group;
            b.n_keys = seg_keys;
            b.page0 = seg_first_page + sg.page_first + seg_done;
            b.table = seg_table;
            seg_done += b.count;
            return b;
        };
        uint32_t it = 0;
        Batch cur = next_batch();
        int phys_cur = (cur.count > 0 && lane < cur.count) ? __ldg(cur.table + ((cur.page0 + lane) >> geo.tpp_shift)) : 0;
        while (cur.count > 0) {
            // Issue the first few pages of the batch before looking ahead, so that opening the next
            // segment (work split, prefetch hints) never delays copies that could already be in flight.
            const int head_n = cur.count < kNStages ? cur.count : kNStages;
            Batch nxt;
            int phys_nxt = 0;
            for (int j = 0; j < cur.count; ++j, ++it) {
                int phys = __shfl_sync(0xffffffffu, phys_cur, j);
                int ok = 1;
                if (lane == 0) {
                    const int stage = (int)(it % kNStages);
                    const uint32_t round = it / kNStages;
                    if (round > 0 && !mbar_wait(smem_u32(&s_empty[stage]), (round - 1) & 1, &s_abort)) {
                        if (a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
                        ok = 0;
                    } else {
                        const int page = cur.page0 + j;                  // tile index within the session
                        int kcount = cur.n_keys - (page << geo.tile_shift);
                        if (kcount > geo.tile_keys) kcount = geo.tile_keys;
                        if (phys < 0 || phys >= a.nb) {      // never follow a bad entry: load page 0, use none of it
                            if (a.status) atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
                            phys = 0;
                            kcount = 0;
                        }
                        s_kcount[stage] = kcount;
                        s_phys[stage] = phys;
                        const uint32_t bar = smem_u32(&s_full[stage]);
                        const uint32_t dst = stage0 + (uint32_t)stage * Cfg::kStageBytes;
                        const int c1 = (int)((((int64_t)cur.layer * a.nb + phys) << geo.kv_shift) + ((page & tpp_mask) << 4));
                        const int c2 = cur.group * KVG;
                        if constexpr (kF32) {
                            // fp32 rows: four boxes of 32 dims for K, four for V
                            mbar_expect_tx(bar, Cfg::kStageBytes);
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
#if NOVA_ATTN_EVICT_FIRST
                                tma_load_3d_hint(dst + (uint32_t)(c * Cfg::kBoxBytes), &tmk, 32 * c, c1, c2, bar, kv_policy);
                                tma_load_3d_hint(dst + (uint32_t)((4 + c) * Cfg::kBoxBytes), &tmv, 32 * c, c1, c2, bar, kv_policy);
#else
                                tma_load_3d(dst + (uint32_t)(c * Cfg::kBoxBytes), &tmk, 32 * c, c1, c2, bar);
                                tma_load_3d(dst + (uint32_t)((4 + c) * Cfg::kBoxBytes), &tmv, 32 * c, c1, c2, bar);
#endif
                            }
                            if (tl && it == 0) tl[2] = now_ns();
                        } else if (geo.tile_keys < kTileKeysMax) {
                            // 8-token pages: the maps' boxes are [64 dims][8 slots][1 kv head]; each kv head's box goes
                            // to the first half of that head's 16 rows
                            mbar_expect_tx(bar, Cfg::kStageBytes / 2);
                            for (int h = 0; h < KVG; ++h) {
                                const uint32_t d = dst + (uint32_t)h * 2048u;
                                tma_load_3d(d, &tmk, 0, c1, c2 + h, bar);
                                tma_load_3d(d + Cfg::kBoxBytes, &tmk, 64, c1, c2 + h, bar);
                                tma_load_3d(d + 2 * Cfg::kBoxBytes, &tmv, 0, c1, c2 + h, bar);
                                tma_load_3d(d + 3 * Cfg::kBoxBytes, &tmv, 64, c1, c2 + h, bar);
                            }
                            if (tl && it == 0) tl[2] = now_ns();
                        } else {
                        mbar_expect_tx(bar, Cfg::kStageBytes);
#if NOVA_ATTN_EVICT_FIRST
                        tma_load_3d_hint(dst, &tmk, 0, c1, c2, bar, kv_policy);
                        tma_load_3d_hint(dst + Cfg::kBoxBytes, &tmk, 64, c1, c2, bar, kv_policy);
                        tma_load_3d_hint(dst + 2 * Cfg::kBoxBytes, &tmv, 0, c1, c2, bar, kv_policy);
                        tma_load_3d_hint(dst + 3 * Cfg::kBoxBytes, &tmv, 64, c1, c2, bar, kv_policy);
#else
                        tma_load_3d(dst, &tmk, 0, c1, c2, bar);
                        tma_load_3d(dst + Cfg::kBoxBytes, &tmk, 64, c1, c2, bar);
                        tma_load_3d(dst + 2 * Cfg::kBoxBytes, &tmv, 0, c1, c2, bar);
                        tma_load_3d(dst + 3 * Cfg::kBoxBytes, &tmv, 64, c1, c2, bar);
#endif
                        if (tl && it == 0) tl[2] = now_ns();
                        }
                    }
                }
                if (!__shfl_sync(0xffffffffu, ok, 0)) return;
                if (j + 1 == head_n) {                      // look ahead: next batch's table entries in flight
                    nxt = next_batch();
                    phys_nxt = (nxt.count > 0 && lane < nxt.count) ? __ldg(nxt.table + ((nxt.page0 + lane) >> geo.tpp_shift)) : 0;
                }
            }
            cur = nxt;
            phys_cur = phys_nxt;
        }
        if (tl && lane == 0) tl[3] = now_ns();
        return;
    }

    // ------------------------------------------------------------------ consumer warps
    const int w = warp;                              // kv head within the group
    const int lm = lane >> 3, lr = lane & 7;         // ldmatrix: matrix index / row within it
    // K operand: matrices (keys 0-7 | 8-15) x (dims 16ks.. | 16ks+8..): key = (lm>>1)*8 + lr, chunk = 2ks + (lm&1)
    const uint32_t k_row = (uint32_t)(w * 2048 + (((lm >> 1) << 3) + lr) * 128);
    // V operand (transposed): matrices (keys 0-7 | 8-15) x (dims chunk c | c+1): key = (lm&1)*8 + lr, chunk = 2jp + (lm>>1)
    const uint32_t v_row = (uint32_t)(w * 2048 + (((lm & 1) << 3) + lr) * 128);
    constexpr float kQScale = kAttnScale * kLog2e;
    uint32_t it = 0;
    // Programmatic dependent launch: a launch that carries the attribute promises that the kernels
    // before it in the stream (the previous layer's split and merge) neither produce anything this
    // kernel READS (q, the new k/v, pages, tables, n_past) nor touch what it WRITES for its own layers
    // (their pages, k rows and outputs).  What they do share is the partial-slot scratch, which the
    // merge may still be reading, so each consumer warp waits for the previous kernel at the end of
    // its first segment, right before its first output or partial-slot write, and computes until then
    // (the new token goes into the pool without waiting).  That wait also keeps completion transitive:
    // this grid cannot finish before the one it depends on.
    bool dep_met = a.pdl == 0;      // plain launch: the stream already ordered us after everything before
    if (a.pdl == 2) {
        // The caller cannot make the promise above for q and the new k / v (in an engine they come out of
        // the kernels that consume the previous layer's output): wait here, before the first of those reads.
        // The producer warp does not wait - pages of earlier steps, tables and positions do not depend on
        // the previous layer - so the ring of page copies fills while the consumers sit here.
        pdl_wait();
        dep_met = true;
    }
    int n_stashed = 0;
    const uint32_t conv0 = stage0 + (uint32_t)(kNStages * Cfg::kStageBytes);      // kF32: the converted (fp16) page set
    float* stash = reinterpret_cast<float*>(smem_raw + (stage0 - smem_u32(smem_raw)) + kNStages * Cfg::kStageBytes +
                                            (kF32 ? Cfg::kConvBytes : 0));

    // One finished segment -> memory: the row's output when this CTA covered the whole row, else
    // (m, l, acc) into this CTA's partial slot for the merge kernel.
    auto emit = [&](bool whole_row, int64_t h0, int row_id, float m_, float l_, auto&& acc) {
        if (g >= G) return;
        if (whole_row) {
            if (a.write_partial_only) {
                float* op = a.out_part + (h0 + g) * kPartW;
                if (t == 0) { op[0] = m_ * (1.f / kLog2e); op[1] = l_; }
#pragma unroll
                for (int j = 0; j < 16; ++j) *reinterpret_cast<float2*>(op + 2 + 8 * j + 2 * t) = acc(j);
            } else {
                const float inv = l_ > 0.f ? 1.f / l_ : 0.f;
                float* op = a.out + (h0 + g) * kHeadDim;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float2 v = acc(j);
                    *reinterpret_cast<float2*>(op + 8 * j + 2 * t) = make_float2(v.x * inv, v.y * inv);
                }
            }
            return;
        }
        float* pr = a.part + ((size_t)((int64_t)blockIdx.x + row_id) * heads_per_row + (size_t)(w * G + g)) * kSlotW;
        if (t == 0) *reinterpret_cast<float2*>(pr) = make_float2(m_ * (1.f / kLog2e), l_);
#pragma unroll
        for (int j = 0; j < 16; ++j) *reinterpret_cast<float2*>(pr + 4 + 8 * j + 2 * t) = acc(j);
    };

    for (int64_t pos = lo; pos < hi;) {
        const Segment sg = plan_segment(pv, pos, hi, a.row_setup_pages);
        pos += sg.span;
        const int s = sg.session;
        const int kvh = sg.group * KVG + w;
        const int64_t head0 = ((int64_t)sg.layer_local * S + s) * NH + (int64_t)kvh * G;
        int first_page_c, n_pages_row_c;
        plan_pages_of_keys(a, s_keys[s], first_page_c, n_pages_row_c);

        // q fragments of row g (zero for padding rows): hi + lo fp16 parts of q * scale * log2(e).
        // With the fused append q arrives un-rotated: dims d and d+64 of a NeoX pair sit in the same
        // thread (k-steps ks and ks+4), so the rotation at n_past[s] is done here, in registers, with
        // the same fused form as the append kernel.
        uint32_t qh[8][2], ql[8][2];
        const int pos_new = a.fuse_append ? s_keys[s] - a.keys_add : -1;      // n_past[s] (the fused append has n_q == 1)
        {
            const float* qp = a.q + (head0 + (g < G ? g : 0)) * kHeadDim;
            float2 x[8][2];
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    x[ks][hlf] = make_float2(0.f, 0.f);
                    if (g < G) x[ks][hlf] = *reinterpret_cast<const float2*>(qp + 16 * ks + 8 * hlf + 2 * t);
                }
            if (a.fuse_append && pos_new >= 0 && pos_new < a.rope_rows) {
                const float* cr = a.rope_cs + (int64_t)pos_new * (kHeadDim / 2);
                const float* sr = a.rope_sn + (int64_t)pos_new * (kHeadDim / 2);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                    for (int hlf = 0; hlf < 2; ++hlf) {
                        const float2 c = *reinterpret_cast<const float2*>(cr + 16 * ks + 8 * hlf + 2 * t);
                        const float2 sn = *reinterpret_cast<const float2*>(sr + 16 * ks + 8 * hlf + 2 * t);
                        const float2 x0 = x[ks][hlf], x1 = x[ks + 4][hlf];
                        x[ks][hlf].x = __fmaf_rn(x0.x, c.x, -__fmul_rn(x1.x, sn.x));
                        x[ks][hlf].y = __fmaf_rn(x0.y, c.y, -__fmul_rn(x1.y, sn.y));
                        x[ks + 4][hlf].x = __fmaf_rn(x0.x, sn.x, __fmul_rn(x1.x, c.x));
                        x[ks + 4][hlf].y = __fmaf_rn(x0.y, sn.y, __fmul_rn(x1.y, c.y));
                    }
            } else if (a.fuse_append && lane == 0 && a.status) {
                atomicCAS(a.status, 0, NOVA_ERR_INVALID);      // position beyond the RoPE table
            }
            // the step's token has no block-table entry (the session is at its context limit): it cannot be stored
            if (a.fuse_append && lane == 0 && a.status && pos_new >= 0 && ((int64_t)pos_new >> geo.kv_shift) >= a.table_stride)
                atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    const float xs = x[ks][hlf].x * kQScale, ys = x[ks][hlf].y * kQScale;
                    const __half2 h = __floats2half2_rn(xs, ys);
                    const float2 hf = __half22float2(h);
                    qh[ks][hlf] = *reinterpret_cast<const uint32_t*>(&h);
                    ql[ks][hlf] = pack_h2(xs - hf.x, ys - hf.y);
                }
        }
        float m = -INFINITY, l = 0.f;
        float o[16][2];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = 0.f;

        for (int pg = 0; pg < sg.page_count; ++pg, ++it) {
            const int stage = (int)(it % kNStages);
            const uint32_t round = it / kNStages;
            if (!mbar_wait(smem_u32(&s_full[stage]), round & 1, &s_abort)) {
                if (lane == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
                return;
            }
            if (tl && threadIdx.x == 0 && it == 0) tl[4] = now_ns();
            const int kcount = s_kcount[stage];
            uint32_t sk = stage0 + (uint32_t)stage * Cfg::kStageBytes;
            if constexpr (kF32) {
                // This kv head's 16 x 128 K and V values, fp32 -> fp16, from the raw stage into the fp16 page set (a
                // lane takes 8 dims of a key at a time: two swizzled 16-byte pieces in, one out); then the raw stage
                // goes back to the producer.
                const uint32_t raw = sk;
#pragma unroll
                for (int which = 0; which < 2; ++which)
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int unit = lane + 32 * u, r = unit >> 4, ch = unit & 15;     // key row, 8-dim piece
                        const uint32_t src = raw + (uint32_t)((4 * which + (ch >> 2)) * Cfg::kBoxBytes + (w * 16 + r) * 128);
                        const uint32_t j0 = (uint32_t)((ch & 3) * 2);
                        float4 x0, x1;
                        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(x0.x), "=f"(x0.y), "=f"(x0.z), "=f"(x0.w)
                                     : "r"(src + ((j0 ^ (uint32_t)(r & 7)) << 4)));
                        asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(x1.x), "=f"(x1.y), "=f"(x1.z), "=f"(x1.w)
                                     : "r"(src + (((j0 + 1) ^ (uint32_t)(r & 7)) << 4)));
                        const uint32_t dst = conv0 + (uint32_t)((2 * which + (ch >> 3)) * Cfg::kBoxBytes + w * 2048 + r * 128 +
                                                                 (((ch & 7) ^ (r & 7)) << 4));
                        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(pack_h2(x0.x, x0.y)), "r"(pack_h2(x0.z, x0.w)),
                                     "r"(pack_h2(x1.x, x1.y)), "r"(pack_h2(x1.z, x1.w))
                                     : "memory");
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&s_empty[stage]));
                sk = conv0;
            }
            const uint32_t sv = sk + 2 * Cfg::kBoxBytes;

            if (kcount > 0) {
                bool patched = false;
                if (a.fuse_append && pos_new >= 0 && pos_new < a.rope_rows &&
                    (pos_new >> geo.tile_shift) == first_page_c + sg.page_first + pg) {
                    // This page receives the step's new token: rotate k, store k and v into the pool
                    // (for later steps) and straight into the staged copy (for this one).  The TMA
                    // copy of that slot may be old or new bytes; both are overwritten here.
                    patched = true;
                    const int slot = pos_new & (geo.tile_keys - 1);          // key row inside the staged tile
                    const int layer = a.layer0 + sg.layer_local;
                    const int64_t tok = ((int64_t)sg.layer_local * S + s) * a.n_kv_heads + kvh;
                    float* kn = a.k_new + tok * kHeadDim;
                    const float* vn = a.v_new + tok * kHeadDim;
                    const float* cr = a.rope_cs + (int64_t)pos_new * (kHeadDim / 2);
                    const float* sr = a.rope_sn + (int64_t)pos_new * (kHeadDim / 2);
                    const int64_t grow = ((((int64_t)layer * a.nb + s_phys[stage]) << geo.kv_shift) + (pos_new & ((1 << geo.kv_shift) - 1))) *
                                             (int64_t)a.n_kv_heads * kHeadDim + (int64_t)kvh * kHeadDim;
                    using PoolT = typename std::conditional<kF32, float, __half>::type;
                    PoolT* gk = static_cast<PoolT*>(a.pool_k_w) + grow;
                    PoolT* gv = static_cast<PoolT*>(a.pool_v_w) + grow;
                    const uint32_t srow = (uint32_t)(w * 2048 + slot * 128);
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const int i = lane + 32 * r;                 // pair (i, i + 64)
                        const float c = cr[i], sn = sr[i];
                        const float x0 = kn[i], x1 = kn[i + 64];
                        const float r0 = __fmaf_rn(x0, c, -__fmul_rn(x1, sn));
                        const float r1 = __fmaf_rn(x0, sn, __fmul_rn(x1, c));
                        kn[i] = r0;
                        kn[i + 64] = r1;
                        const float vf0 = vn[i], vf1 = vn[i + 64];
                        const __half k0 = __float2half_rn(r0), k1 = __float2half_rn(r1);
                        const __half v0 = __float2half_rn(vf0), v1 = __float2half_rn(vf1);
                        if constexpr (kF32) {          // the pool keeps the fp32 values, the staged fp16 copy their roundings
                            gk[i] = r0; gk[i + 64] = r1;
                            gv[i] = vf0; gv[i + 64] = vf1;
                        } else {
                            gk[i] = k0; gk[i + 64] = k1;
                            gv[i] = v0; gv[i + 64] = v1;
                        }
                        const uint32_t off = srow + ((((uint32_t)i >> 3) ^ (uint32_t)(slot & 7)) << 4) + (((uint32_t)i & 7) << 1);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(sk + off), "h"(__half_as_ushort(k0)) : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(sk + (uint32_t)Cfg::kBoxBytes + off), "h"(__half_as_ushort(k1)) : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(sv + off), "h"(__half_as_ushort(v0)) : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(sv + (uint32_t)Cfg::kBoxBytes + off), "h"(__half_as_ushort(v1)) : "memory");
                    }
                    __syncwarp();
                }
                if (kcount < geo.tile_keys) {
                    // Rows past the last key hold whatever the page held before: P is 0 there, but
                    // 0 * (Inf/NaN bit patterns) would poison O, so clear those V rows first.
                    for (int i = lane; i < (geo.tile_keys - kcount) * 16; i += 32) {
                        const int row = kcount + (i >> 4), c = i & 15;
                        const uint32_t addr = sv + (uint32_t)((c >> 3) * Cfg::kBoxBytes + w * 2048 + row * 128 + ((c & 7) << 4));
                        asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
                    }
                    __syncwarp();
                }
                // S = Q K^T for the 16 keys of the page: two n-tiles of 8 keys, hi and lo parts of q
                float sh[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, sl[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    uint32_t b[4];
                    const uint32_t chunk = (uint32_t)((2 * ks + (lm & 1)) & 7);
                    ldsm_x4(b, sk + (uint32_t)((ks >> 2) * Cfg::kBoxBytes) + k_row + ((chunk ^ (uint32_t)lr) << 4));
                    mma_top(sh[0][0], sh[0][1], qh[ks][0], qh[ks][1], b[0], b[1], sh[0][0], sh[0][1]);
                    mma_top(sh[1][0], sh[1][1], qh[ks][0], qh[ks][1], b[2], b[3], sh[1][0], sh[1][1]);
                    mma_top(sl[0][0], sl[0][1], ql[ks][0], ql[ks][1], b[0], b[1], sl[0][0], sl[0][1]);
                    mma_top(sl[1][0], sl[1][1], ql[ks][0], ql[ks][1], b[2], b[3], sl[1][0], sl[1][1]);
                }
                float sc[4] = {sh[0][0] + sl[0][0], sh[0][1] + sl[0][1], sh[1][0] + sl[1][0], sh[1][1] + sl[1][1]};
                if (kcount < kTileKeysMax) {   // keys 2t, 2t+1, 8+2t, 9+2t of the tile
                    if (2 * t >= kcount) sc[0] = -INFINITY;
                    if (2 * t + 1 >= kcount) sc[1] = -INFINITY;
                    if (8 + 2 * t >= kcount) sc[2] = -INFINITY;
                    if (9 + 2 * t >= kcount) sc[3] = -INFINITY;
                }
                float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float mn = fmaxf(m, mx);
                const float corr = ex2(m - mn);
                m = mn;
                const uint32_t p0 = pack_h2(ex2(sc[0] - mn), ex2(sc[1] - mn));
                const uint32_t p1 = pack_h2(ex2(sc[2] - mn), ex2(sc[3] - mn));
                {   // the row sum uses the fp16-rounded weights that multiply V
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&p0));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&p1));
                    l = fmaf(l, corr, (f0.x + f0.y) + (f1.x + f1.y));
                }
                if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        o[j][0] *= corr;
                        o[j][1] *= corr;
                    }
                }
                // O += P V : n-tiles of 8 dims, two per ldmatrix
#pragma unroll
                for (int jp = 0; jp < 8; ++jp) {
                    uint32_t b[4];
                    const uint32_t chunk = (uint32_t)((2 * jp + (lm >> 1)) & 7);
                    ldsm_x4_t(b, sv + (uint32_t)((jp >> 2) * Cfg::kBoxBytes) + v_row + ((chunk ^ (uint32_t)lr) << 4));
                    mma_top(o[2 * jp][0], o[2 * jp][1], p0, p1, b[0], b[1], o[2 * jp][0], o[2 * jp][1]);
                    mma_top(o[2 * jp + 1][0], o[2 * jp + 1][1], p0, p1, b[2], b[3], o[2 * jp + 1][0], o[2 * jp + 1][1]);
                }
                if (!kF32 && (kcount < geo.tile_keys || patched)) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            __syncwarp();
            if (!kF32 && lane == 0) mbar_arrive(smem_u32(&s_empty[stage]));
        }

        // ---- segment done: row sums, then direct output or a partial slot
        if (tl && threadIdx.x == 0) tl[5] = now_ns();
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int n_contrib = sg.c_last - sg.c_first + 1;
        if (!dep_met) {
            if (pos < hi && n_stashed < kStashSlots) {          // more work ahead: park this result, do not wait here
                float* st = stash + (size_t)((n_stashed * KVG + w) * kStashWords) * 32 + lane;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    st[(2 * j) * 32] = o[j][0];
                    st[(2 * j + 1) * 32] = o[j][1];
                }
                st[32 * 32] = m;
                st[33 * 32] = l;
                st[34 * 32] = __int_as_float(n_contrib == 1 ? -1 : sg.row_id);
                st[35 * 32] = __int_as_float((int)(head0 & 0xffffffffLL));
                st[36 * 32] = __int_as_float((int)(head0 >> 32));
                ++n_stashed;
                continue;
            }
            pdl_wait();
            dep_met = true;
            for (int si = 0; si < n_stashed; ++si) {
                const float* st = stash + (size_t)((si * KVG + w) * kStashWords) * 32 + lane;
                const int row_id = __float_as_int(st[34 * 32]);
                const int64_t h0 = (int64_t)(((unsigned long long)(unsigned)__float_as_int(st[36 * 32]) << 32) |
                                             (unsigned long long)(unsigned)__float_as_int(st[35 * 32]));
                emit(row_id < 0, h0, row_id, st[32 * 32], st[33 * 32],
                     [&](int j) { return make_float2(st[(2 * j) * 32], st[(2 * j + 1) * 32]); });
            }
        }
        emit(n_contrib == 1, head0, sg.row_id, m, l, [&](int j) { return make_float2(o[j][0], o[j][1]); });
        if (tl && threadIdx.x == 0) tl[6] = now_ns();
    }
}

template <int KVG, bool kF32 = false>
int launch_kvg(const AttnLaunch& a, int n_ctas, cudaStream_t s) {
    using Cfg = MmaCfg<KVG, kF32>;
    static bool attr_set[64] = {};          // the attribute is per device
    int dev = 0;
    NOVA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        NOVA_CUDA_TRY((cudaFuncSetAttribute(attn_mma_kernel<KVG, kF32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            Cfg::kSmemBytes)));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    // 8-token pages are fetched one kv head at a time (maps with [64][8][1] boxes)
    const bool per_head = (a.kv_shift ? a.kv_shift : kKvShift) < 4;
    const CUtensorMap* tk = static_cast<const CUtensorMap*>(per_head ? a.tmap_k1 : a.tmap_k);
    const CUtensorMap* tv = static_cast<const CUtensorMap*>(per_head ? a.tmap_v1 : a.tmap_v);
    const cudaError_t le = launch_kernel_pdl(attn_mma_kernel<KVG, kF32>, dim3((unsigned)n_ctas), dim3(Cfg::kThreads),
                                             (size_t)Cfg::kSmemBytes, s, a.pdl != 0, a, *tk, *tv);
    if (le != cudaSuccess) {
        set_cuda_error(le, "attention launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

bool attn_mma_built() { return true; }
int attn_default_ctas_mma() { return sm_count(); }
size_t attn_tmap_bytes() { return sizeof(CUtensorMap); }

// Tensor map over one fp16 pool [rows = L*NB*page tokens][NKV][128]: dim0 = 128 dims, dim1 = slot rows
// (stride NKV*256 B), dim2 = kv head (stride 256 B); box = [64][box_rows = 16 or 8][kv_group], 128-byte swizzle.
int attn_make_tmap(void* out_map, void* pool, int64_t slot_rows, int n_kv_heads, int kv_group, int box_rows, int elem_bytes) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        cudaDriverEntryPointQueryResult q;
        void* fn = nullptr;
        const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            set_cuda_error(e == cudaSuccess ? cudaErrorNotSupported : e, "cuTensorMapEncodeTiled entry point");
            return NOVA_ERR_CUDA;
        }
        encode = (EncodeTiledFn)fn;
    }
    if (slot_rows <= 0 || slot_rows > 0x7fffffffLL) return NOVA_ERR_TOO_LARGE;
    if ((box_rows != 8 && box_rows != 16) || (elem_bytes != 2 && elem_bytes != 4)) return NOVA_ERR_INVALID;
    const cuuint64_t dims[3] = {(cuuint64_t)kHeadDim, (cuuint64_t)slot_rows, (cuuint64_t)n_kv_heads};
    const cuuint64_t strides[2] = {(cuuint64_t)n_kv_heads * kHeadDim * (cuuint64_t)elem_bytes, (cuuint64_t)kHeadDim * (cuuint64_t)elem_bytes};
    const cuuint32_t box[3] = {(cuuint32_t)(128 / elem_bytes), (cuuint32_t)box_rows, (cuuint32_t)kv_group};      // 128-byte lines
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(static_cast<CUtensorMap*>(out_map), elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                              3, pool, dims, strides,
                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
        return NOVA_ERR_CUDA;
    }
    return NOVA_OK;
}

int attn_split_ctas_mma(const AttnLaunch& a, int n_ctas) {
    if (n_ctas > 0) return n_ctas;
    const int per_sm = a.kv_group >= 4 ? 1 : 4 / a.kv_group;
    return (sm_count() - ((a.pdl && a.pdl_spare) ? NOVA_ATTN_SPARE_SMS : 0)) * per_sm;
}

int launch_attn_mma(const AttnLaunch& a, int kv_dtype, int n_ctas, cudaStream_t s) {
    if ((kv_dtype != NOVA_KV_F16 && kv_dtype != NOVA_KV_F32) || !a.tmap_k || !a.tmap_v) return NOVA_ERR_UNSUPPORTED;
    // fp32 pools: converted to fp16 on the way in; 16-token pages only
    if (kv_dtype == NOVA_KV_F32 && (a.kv_shift ? a.kv_shift : kKvShift) != 4) return NOVA_ERR_UNSUPPORTED;
    if ((a.kv_shift ? a.kv_shift : kKvShift) < 4 && (!a.tmap_k1 || !a.tmap_v1)) return NOVA_ERR_UNSUPPORTED;
    if (a.fuse_append && a.n_q > 1) return NOVA_ERR_UNSUPPORTED;      // the fused append is a decode (one token) path
    if (a.fuse_append && (!a.n_past || !a.k_new || !a.v_new || !a.rope_cs || !a.rope_sn || !a.pool_k_w || !a.pool_v_w))
        return NOVA_ERR_INVALID;
    if (a.n_sessions <= 0 || a.n_layers <= 0) return NOVA_OK;
    if (a.n_heads % a.n_kv_heads || a.n_kv_heads % a.kv_group) return NOVA_ERR_INVALID;
    if (a.n_heads / a.n_kv_heads > 8) return NOVA_ERR_UNSUPPORTED;
    if ((int64_t)a.n_sessions * (a.n_q > 1 ? a.n_q : 1) * (a.n_kv_heads / a.kv_group) > kMaxRowsSmem) return NOVA_ERR_TOO_LARGE;
    if (kv_dtype == NOVA_KV_F32) {
        switch (a.kv_group) {
            case 4: return launch_kvg<4, true>(a, attn_split_ctas_mma(a, n_ctas), s);
            case 2: return launch_kvg<2, true>(a, attn_split_ctas_mma(a, n_ctas), s);
            case 1: return launch_kvg<1, true>(a, attn_split_ctas_mma(a, n_ctas), s);
            default: return NOVA_ERR_UNSUPPORTED;
        }
    }
    switch (a.kv_group) {
        case 4: return launch_kvg<4>(a, attn_split_ctas_mma(a, n_ctas), s);
        case 2: return launch_kvg<2>(a, attn_split_ctas_mma(a, n_ctas), s);
        case 1: return launch_kvg<1>(a, attn_split_ctas_mma(a, n_ctas), s);
        default: return NOVA_ERR_UNSUPPORTED;
    }
}

}  // namespace novab
