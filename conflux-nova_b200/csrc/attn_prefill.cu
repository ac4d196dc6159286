// attn_prefill.cu — paged prefill attention for fp16 pools, query-tiled, tensor cores.
// Replaces flash_paged_kernel (src/kernel/attn.cu:292-357 of the reference), which gives every
// (head, query) its own warp and streams all keys once per query.
//
// One CTA = (session, kv head, tile of TQ consecutive query tokens).  The TQ x G (query token,
// query head) pairs that share the kv head are the rows of a 64-row tile, 16 rows per warp; the
// kv head's pages come in once per TILE through the same TMA ring as the decode kernel (box
// [64 dims][16 slots][1 head], 128-byte swizzle) and all four warps read them from shared memory:
// K/V traffic drops by TQ (9 at G = 7) against a per-query stream and every row of the
// m16n8k16 tiles is a real query.  Causal: the row of query t sees keys 0 .. n_past + t; with a sliding
// window W (flash_paged_kernel<true>, attn.cu:317) only the last W of them, and the tile starts at the first
// page that any of its queries can see.
// fp16 operands, fp32 accumulation and softmax (exp2 domain), P rounded to fp16 for P.V.
// "Page" below is a tile of min(16, tokens per page) keys (attn_plan.cuh): pages of 32 / 64 tokens are 2 / 4
// tiles behind one block-table entry, pages of 8 tokens fill half a stage.
#include "attn_plan.cuh"
#include "mma_common.cuh"

namespace novab {
namespace {

constexpr int kPfStages = 6;
constexpr int kPfBox = 16 * 128;                  // one [64 dims][16 slots][1 head] box: 2 KiB
constexpr int kPfStage = 4 * kPfBox;              // K lo/hi dims + V lo/hi dims: 8 KiB
constexpr int kPfSmem = kPfStages * kPfStage + 1024;
constexpr int kPfWarps = 4;                       // consumer warps, 16 tile rows each

#ifndef NOVA_PREFILL_CTAS_PER_SM
#define NOVA_PREFILL_CTAS_PER_SM 2     // 204 registers, no spills; 3 CTAs (128 registers) measured slightly slower
#endif
// kPrefix = true is the shared-prefix form used by decode steps of sessions that share their first pages
// (one refcounted prefix): the "query tokens" are the SESSIONS of the batch (q [S][NH][128], one query
// each), every row sees all keys of the shared pages [0, prefix_pages) of the first session's table,
// blockIdx.z-like chunks of those pages go to different CTAs, q is rotated here when the append is
// fused (position n_past[session]), and the result is an un-normalised partial (m, l, acc) per chunk
// in the layout of the decode kernels, merged later with the partial over each session's private pages.
template <bool kPrefix>
__global__ void __launch_bounds__(32 * (kPfWarps + 1), NOVA_PREFILL_CTAS_PER_SM)
attn_prefill_kernel(AttnLaunch a, const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv,
                    int tq, int n_tiles, int prefix_pages, int chunk_pages) {      // both counts in tiles
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long s_full[kPfStages];
    __shared__ __align__(8) unsigned long long s_empty[kPfStages];
    __shared__ int s_abort;

    const int lane = (int)threadIdx.x & 31;
    const int warp = (int)threadIdx.x >> 5;
    const int G = a.n_heads / a.n_kv_heads;
    const int NH = a.n_heads, NKV = a.n_kv_heads, NQ = a.n_q;
    const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const PageGeom geo = page_geom(a.kv_shift);
    const int tpp_mask = (1 << geo.tpp_shift) - 1;
    if (kPrefix) pdl_launch_dependents();      // the split over the private pages shares nothing with this kernel

    // blockIdx.x -> (tile, kv head, session); late tiles (most keys) first
    int bid = (int)blockIdx.x;
    const int tile = n_tiles - 1 - bid % n_tiles;
    bid /= n_tiles;
    const int kvh = bid % NKV;
    const int s = kPrefix ? 0 : bid / NKV;                  // prefix form: rows index sessions, the table is the first one's
    const int chunk = kPrefix ? bid / NKV : 0;
    const int t0 = tile * tq;
    const int t_cnt = NQ - t0 < tq ? NQ - t0 : tq;          // query tokens in this tile
    const int n_past = kPrefix ? 0 : (a.n_past ? a.n_past[s] : a.keys_imm);
    const int keys_tile = kPrefix ? prefix_pages << geo.tile_shift
                                  : n_past + a.keys_add + t0 + t_cnt - 1;   // keys seen by the tile's last query
    // sliding window: the tile's first query sees keys from first_key on, nothing before it matters to any row
    const int first_key = (!kPrefix && a.window > 0) ? n_past + a.keys_add + t0 - a.window : 0;
    const int page_begin = kPrefix ? chunk * chunk_pages : (first_key > 0 ? first_key >> geo.tile_shift : 0);
    const int page_end_all = (keys_tile + geo.tile_keys - 1) >> geo.tile_shift;
    const int page_end = kPrefix && page_begin + chunk_pages < page_end_all ? page_begin + chunk_pages : page_end_all;
    const int n_pages = page_end - page_begin;
    const int32_t* table = a.table_base + (int64_t)(a.slice_ids ? a.slice_ids[s] : s) * a.table_stride;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kPfStages; ++i) {
            mbar_init(smem_u32(&s_full[i]), 1);
            mbar_init(smem_u32(&s_empty[i]), kPfWarps);
        }
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (geo.tile_keys < kTileKeysMax) {      // 8-token pages fill rows 0-7 of a stage only: the other rows must be finite
        for (uint32_t off = threadIdx.x * 16u; off < (uint32_t)(kPfStages * kPfStage); off += blockDim.x * 16u)
            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(stage0 + off), "r"(0u) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    if (n_pages <= 0 || ((page_end + tpp_mask) >> geo.tpp_shift) > a.table_stride) return;

    // ------------------------------------------------------------------ producer warp
    if (warp == kPfWarps) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmk) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmv) : "memory");
        }
        int phys_cur = lane < n_pages ? __ldg(table + ((page_begin + lane) >> geo.tpp_shift)) : 0;
        for (int base = 0; base < n_pages; base += 32) {
            const int nxt = base + 32 + lane;
            const int phys_nxt = nxt < n_pages ? __ldg(table + ((page_begin + nxt) >> geo.tpp_shift)) : 0;
            const int cnt = n_pages - base < 32 ? n_pages - base : 32;
            for (int j = 0; j < cnt; ++j) {
                int phys = __shfl_sync(0xffffffffu, phys_cur, j);
                int ok = 1;
                if (lane == 0) {
                    const uint32_t it = (uint32_t)(base + j);
                    const int stage = (int)(it % kPfStages);
                    const uint32_t round = it / kPfStages;
                    if (round > 0 && !mbar_wait(smem_u32(&s_empty[stage]), (round - 1) & 1, &s_abort)) {
                        if (a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
                        ok = 0;
                    } else {
                        if (phys < 0 || phys >= a.nb) {     // never follow a bad entry; the result is flagged invalid
                            if (a.status) atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
                            phys = 0;
                        }
                        const uint32_t bar = smem_u32(&s_full[stage]);
                        const uint32_t dst = stage0 + (uint32_t)stage * kPfStage;
                        const int c1 = (int)((((int64_t)a.layer0 * a.nb + phys) << geo.kv_shift) + (((page_begin + (int)it) & tpp_mask) << 4));
                        mbar_expect_tx(bar, geo.tile_keys < kTileKeysMax ? kPfStage / 2 : kPfStage);    // 8-row boxes are half the bytes
                        tma_load_3d(dst, &tmk, 0, c1, kvh, bar);
                        tma_load_3d(dst + kPfBox, &tmk, 64, c1, kvh, bar);
                        tma_load_3d(dst + 2 * kPfBox, &tmv, 0, c1, kvh, bar);
                        tma_load_3d(dst + 3 * kPfBox, &tmv, 64, c1, kvh, bar);
                    }
                }
                if (!__shfl_sync(0xffffffffu, ok, 0)) return;
            }
            phys_cur = phys_nxt;
        }
        return;
    }

    // ------------------------------------------------------------------ consumer warps
    const int gq = lane >> 2, t = lane & 3;
    const int lm = lane >> 3, lr = lane & 7;
    const uint32_t k_row = (uint32_t)(((((lm >> 1) << 3) + lr)) * 128);
    const uint32_t v_row = (uint32_t)(((((lm & 1) << 3) + lr)) * 128);
    constexpr float kQScale = kAttnScale * kLog2e;

    // this thread's two tile rows: r0 = 16*warp + gq, r1 = r0 + 8; row -> (query token, head)
    int row_tok[2], row_head[2], row_lim[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = 16 * warp + gq + 8 * h;
        const int tk = r / G, g = r - tk * G;
        row_ok[h] = tk < t_cnt;
        row_tok[h] = t0 + tk;
        row_head[h] = kvh * G + g;
        // last key this row may see; padding rows see everything (their result is dropped)
        row_lim[h] = (row_ok[h] && !kPrefix) ? n_past + a.keys_add + row_tok[h] - 1 : 0x7fffffff;
        // first key of the row's sliding window (keys row_lo .. row_lim are visible)
        row_lo[h] = (row_ok[h] && !kPrefix && a.window > 0) ? row_lim[h] - a.window + 1 : 0;
    }
    uint32_t qa[8][4];
    if (kPrefix && a.fuse_append) {
        // q arrives un-rotated: NeoX pairs (d, d + 64) sit in this thread (k-steps ks and ks + 4); rotate at
        // the session's position with the same fused form as the append kernel, then scale and round.
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int pos = row_ok[h] ? a.n_past[row_tok[h]] : 0;
            const bool rot = row_ok[h] && pos >= 0 && pos < a.rope_rows;
            const float* qp = a.q + ((int64_t)row_tok[h] * NH + row_head[h]) * kHeadDim;
            const float* cr = a.rope_cs + (int64_t)(rot ? pos : 0) * (kHeadDim / 2);
            const float* sr = a.rope_sn + (int64_t)(rot ? pos : 0) * (kHeadDim / 2);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                for (int hlf = 0; hlf < 2; ++hlf) {
                    float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
                    if (row_ok[h]) {
                        x0 = *reinterpret_cast<const float2*>(qp + 16 * ks + 8 * hlf + 2 * t);
                        x1 = *reinterpret_cast<const float2*>(qp + 64 + 16 * ks + 8 * hlf + 2 * t);
                    }
                    if (rot) {
                        const float2 c = *reinterpret_cast<const float2*>(cr + 16 * ks + 8 * hlf + 2 * t);
                        const float2 sn = *reinterpret_cast<const float2*>(sr + 16 * ks + 8 * hlf + 2 * t);
                        const float2 y0 = make_float2(__fmaf_rn(x0.x, c.x, -__fmul_rn(x1.x, sn.x)),
                                                      __fmaf_rn(x0.y, c.y, -__fmul_rn(x1.y, sn.y)));
                        const float2 y1 = make_float2(__fmaf_rn(x0.x, sn.x, __fmul_rn(x1.x, c.x)),
                                                      __fmaf_rn(x0.y, sn.y, __fmul_rn(x1.y, c.y)));
                        x0 = y0;
                        x1 = y1;
                    }
                    qa[ks][2 * hlf + h] = pack_h2(x0.x * kQScale, x0.y * kQScale);
                    qa[ks + 4][2 * hlf + h] = pack_h2(x1.x * kQScale, x1.y * kQScale);
                }
        }
    } else {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
#pragma unroll
            for (int hlf = 0; hlf < 2; ++hlf)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float2 x = make_float2(0.f, 0.f);
                    if (row_ok[h])
                        x = *reinterpret_cast<const float2*>(a.q + (((int64_t)s * NQ + row_tok[h]) * NH + row_head[h]) * kHeadDim +
                                                             16 * ks + 8 * hlf + 2 * t);
                    qa[ks][2 * hlf + h] = pack_h2(x.x * kQScale, x.y * kQScale);     // a0,a1 (k lo) / a2,a3 (k hi)
                }
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[16][4];
#pragma unroll
    for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

    for (int pg = 0; pg < n_pages; ++pg) {
        const int stage = pg % kPfStages;
        const uint32_t round = (uint32_t)pg / kPfStages;
        if (!mbar_wait(smem_u32(&s_full[stage]), round & 1, &s_abort)) {
            if (lane == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
            return;
        }
        const uint32_t sk = stage0 + (uint32_t)stage * kPfStage;
        const uint32_t sv = sk + 2 * kPfBox;
        const int key0 = (page_begin + pg) << geo.tile_shift;
        const int kcount = keys_tile - key0 < geo.tile_keys ? keys_tile - key0 : geo.tile_keys;
        if (kcount < geo.tile_keys) {
            // rows past the tile's last key hold stale bytes: P is 0 there, but 0 * Inf/NaN would poison O.
            // Every warp clears them itself (same zeros) before it reads them.
            for (int i = lane; i < (geo.tile_keys - kcount) * 16; i += 32) {
                const int row = kcount + (i >> 4), c = i & 15;
                const uint32_t addr = sv + (uint32_t)((c >> 3) * kPfBox + row * 128 + ((c & 7) << 4));
                asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(addr), "r"(0u) : "memory");
            }
            __syncwarp();
        }
        float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};      // [n-tile][row r0: 0,1 | row r1: 2,3]
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t b[4];
            const uint32_t chunk = (uint32_t)((2 * ks + (lm & 1)) & 7);
            ldsm_x4(b, sk + (uint32_t)((ks >> 2) * kPfBox) + k_row + ((chunk ^ (uint32_t)lr) << 4));
            mma_full(sc[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
            mma_full(sc[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
        }
        // causal mask: key index of sc[nt][2h + i] is key0 + 8 nt + 2t + i
        uint32_t pa[4];
        bool rescale = false;
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float v[4] = {sc[0][2 * h], sc[0][2 * h + 1], sc[1][2 * h], sc[1][2 * h + 1]};
            const int kbase = key0 + 2 * t;
            // visible: inside the row's causal range (and window) and a real key of this tile
            const int hi_k = row_lim[h] < key0 + kcount - 1 ? row_lim[h] : key0 + kcount - 1;
            if (kbase > hi_k || kbase < row_lo[h]) v[0] = -INFINITY;
            if (kbase + 1 > hi_k || kbase + 1 < row_lo[h]) v[1] = -INFINITY;
            if (kbase + 8 > hi_k || kbase + 8 < row_lo[h]) v[2] = -INFINITY;
            if (kbase + 9 > hi_k || kbase + 9 < row_lo[h]) v[3] = -INFINITY;
            float mx = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float mn = fmaxf(m[h], mx);
            const float ms = mn == -INFINITY ? 0.f : mn;       // nothing visible yet: keep exp arguments finite
            corr[h] = ex2(m[h] - ms);
            m[h] = mn;
            const uint32_t p0 = pack_h2(ex2(v[0] - ms), ex2(v[1] - ms));
            const uint32_t p1 = pack_h2(ex2(v[2] - ms), ex2(v[3] - ms));
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&p0));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&p1));
            l[h] = fmaf(l[h], corr[h], (f0.x + f0.y) + (f1.x + f1.y));
            pa[h] = p0;          // a0 (row r0, keys 2t..) / a1 (row r1)
            pa[2 + h] = p1;      // a2 (row r0, keys 8+2t..) / a3 (row r1)
            rescale = rescale || corr[h] != 1.f;
        }
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
        }
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {
            uint32_t b[4];
            const uint32_t chunk = (uint32_t)((2 * jp + (lm >> 1)) & 7);
            ldsm_x4_t(b, sv + (uint32_t)((jp >> 2) * kPfBox) + v_row + ((chunk ^ (uint32_t)lr) << 4));
            mma_full(o[2 * jp], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
            mma_full(o[2 * jp + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
        }
        if (kcount < geo.tile_keys) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&s_empty[stage]));
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float lh = l[h];
        lh += __shfl_xor_sync(0xffffffffu, lh, 1);
        lh += __shfl_xor_sync(0xffffffffu, lh, 2);
        if (!row_ok[h]) continue;
        if (kPrefix) {
            // the chunk partials are re-used by every layer: the previous layer's final merge may still read them
            if (h == 0 || !row_ok[0]) pdl_wait();
            float* op = a.out_part + (((int64_t)chunk * NQ + row_tok[h]) * NH + row_head[h]) * kPartW;
            if (t == 0) { op[0] = m[h] * (1.f / kLog2e); op[1] = lh; }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                *reinterpret_cast<float2*>(op + 2 + 8 * j + 2 * t) = make_float2(o[j][2 * h], o[j][2 * h + 1]);
        } else {
            const float inv = lh > 0.f ? 1.f / lh : 0.f;
            float* op = a.out + (((int64_t)s * NQ + row_tok[h]) * NH + row_head[h]) * kHeadDim;
#pragma unroll
            for (int j = 0; j < 16; ++j)
                *reinterpret_cast<float2*>(op + 8 * j + 2 * t) = make_float2(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
    }
}

}  // namespace

// Tokens per tile: as many whole query tokens as fit the 64-row tile.
int attn_prefill_tile_tokens(int n_heads, int n_kv_heads) { return 64 / (n_heads / n_kv_heads); }

int launch_attn_prefill(const AttnLaunch& a, cudaStream_t s) {
    if (!a.tmap_k1 || !a.tmap_v1 || a.n_q < 1 || a.n_layers != 1) return NOVA_ERR_UNSUPPORTED;
    if (a.n_heads % a.n_kv_heads || a.n_heads / a.n_kv_heads > 16) return NOVA_ERR_UNSUPPORTED;
    if (a.n_sessions <= 0) return NOVA_OK;
    static bool attr_set[64] = {};
    int dev = 0;
    NOVA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const int tq = attn_prefill_tile_tokens(a.n_heads, a.n_kv_heads);
    const int n_tiles = (a.n_q + tq - 1) / tq;
    const long long ctas = (long long)n_tiles * a.n_kv_heads * a.n_sessions;
    if (ctas > 0x7fffffffLL) return NOVA_ERR_TOO_LARGE;
    const CUtensorMap* tk = static_cast<const CUtensorMap*>(a.tmap_k1);
    const CUtensorMap* tv = static_cast<const CUtensorMap*>(a.tmap_v1);
    attn_prefill_kernel<false><<<(unsigned)ctas, 32 * (kPfWarps + 1), kPfSmem, s>>>(a, *tk, *tv, tq, n_tiles, 0, 0);
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

// Chunks of the shared prefix for a batch of n_sessions decode queries: enough CTAs for two per SM.
int attn_prefix_chunks(int n_sessions, int n_heads, int n_kv_heads, int prefix_pages, int* chunk_pages) {
    const int tq = attn_prefill_tile_tokens(n_heads, n_kv_heads);
    const int n_tiles = (n_sessions + tq - 1) / tq;
    int chunks = (2 * sm_count() + n_tiles * n_kv_heads - 1) / (n_tiles * n_kv_heads);
    if (chunks > prefix_pages / 4) chunks = prefix_pages / 4;          // at least four pages per CTA
    if (chunks < 1) chunks = 1;
    const int per = (prefix_pages + chunks - 1) / chunks;
    if (chunk_pages) *chunk_pages = per;
    return (prefix_pages + per - 1) / per;
}

// Partials of every (session, head) row over the shared pages [0, prefix_pages) of the batch's first session:
// a.out_part [chunks][n_sessions][NH][130], a.q [n_sessions][NH][128] (un-rotated when a.fuse_append), one layer.
int launch_attn_prefix(const AttnLaunch& a_in, int prefix_pages, cudaStream_t s) {
    if (!a_in.tmap_k1 || !a_in.tmap_v1 || a_in.n_layers != 1 || !a_in.out_part || prefix_pages < 1) return NOVA_ERR_UNSUPPORTED;
    if (a_in.n_heads % a_in.n_kv_heads || a_in.n_heads / a_in.n_kv_heads > 16) return NOVA_ERR_UNSUPPORTED;
    if (a_in.fuse_append && (!a_in.n_past || !a_in.rope_cs || !a_in.rope_sn)) return NOVA_ERR_INVALID;
    if (a_in.n_sessions <= 0) return NOVA_OK;
    static bool attr_set[64] = {};
    int dev = 0;
    NOVA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPfSmem));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    AttnLaunch a = a_in;
    a.n_q = a_in.n_sessions;             // the sessions are the query rows of one pseudo-session
    int chunk_pages = 0;
    const int chunks = attn_prefix_chunks(a_in.n_sessions, a.n_heads, a.n_kv_heads, prefix_pages, &chunk_pages);
    const int tq = attn_prefill_tile_tokens(a.n_heads, a.n_kv_heads);
    const int n_tiles = (a.n_q + tq - 1) / tq;
    const long long ctas = (long long)n_tiles * a.n_kv_heads * chunks;
    const CUtensorMap* tk = static_cast<const CUtensorMap*>(a.tmap_k1);
    const CUtensorMap* tv = static_cast<const CUtensorMap*>(a.tmap_v1);
    const cudaError_t le = launch_kernel_pdl(attn_prefill_kernel<true>, dim3((unsigned)ctas), dim3(32 * (kPfWarps + 1)), (size_t)kPfSmem, s,
                                             a.pdl != 0, a, *tk, *tv, tq, n_tiles, prefix_pages, chunk_pages);
    if (le != cudaSuccess) {
        set_cuda_error(le, "prefix attention launch");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
