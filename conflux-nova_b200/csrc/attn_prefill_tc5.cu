// attn_prefill_tc5.cu — paged prefill attention on the fifth-generation tensor cores (tcgen05 + tensor memory).
// Same contract as attn_prefill.cu (replaces flash_paged_kernel, src/kernel/attn.cu:292-357 of the reference, causal
// and sliding-window), built for a contraction-bound shape: the scores S = Q.K^T and the outputs O += P.V are
// tcgen05.mma instructions issued by one thread, their accumulators live in tensor memory, and the 256 threads of
// the softmax warps each own one query row of them.
//
//   * One CTA = (session, kv head, tile of 256 / G query tokens): the (token, head) pairs that share the kv head are
//     the rows of the tile, handled as two halves of M = 128 rows that share every K/V page the CTA brings in (each
//     byte fetched from L2 feeds twice the arithmetic a single half would; with one half per CTA the kernel was bound
//     by those fetches).  Q is converted once to fp16 (scaled by 1/sqrt(128) * log2 e) and laid out in shared memory
//     in the K-major 128-byte-swizzle form the instruction reads (per half, two slabs of 64 dims).
//   * K/V arrive 64 keys at a time (four 16-key tiles of pages) through the same TMA boxes as everywhere else
//     ([64 dims][16 slots][1 kv head], 128-byte swizzle): that layout IS the K-major form for K and the MN-major form
//     for V, so the pages are consumed as they land, without a transpose.  Four stages of 16 KiB K + 16 KiB V: the K
//     part is free again once both halves' scores are computed, the V part once both P.V products are done.
//   * Per 64 keys and half: eight MMAs (M128 N64 K16) fill S in tensor memory (two buffers of 64 columns: the scores
//     of the next 64 keys are computed while the softmax of these runs); the softmax warps read their row with
//     tcgen05.ld, mask (causal / window), keep a running reference maximum that only moves when the row maximum grows
//     by more than 2^8 (so the O accumulator is rescaled rarely) and write P as fp16 back into tensor memory over the
//     scores they just read; four MMAs (M128 N128 K16, A = P from tensor memory) add P.V to O (128 columns).
//   * One CTA per SM: 192 KiB of shared memory and all 512 tensor-memory columns (2 x 2 x 64 of scores, 2 x 128 of
//     outputs).  Each half has its own MMA-issuing warp (one thread cannot issue MMAs of this size as fast as the
//     pipe retires them); one half's softmax overlaps the other half's MMAs.
//   * Every mbarrier wait is bounded (NOVA_ERR_TIMEOUT in the status word); tensor memory is released on every path.
#include "attn_plan.cuh"
#include "mma_common.cuh"

namespace novab {
namespace {

constexpr int kT5Rows = 256;                          // query rows of a CTA
constexpr int kT5Half = 128;                          // rows of one half = M of the MMAs
constexpr int kT5Keys = 64;                           // keys per K/V tile = N of S = Q.K^T
constexpr int kT5Stages = 4;
constexpr int kT5SlabBytes = kT5Keys * 128;           // 64 key rows x 128 B (64 dims): 8 KiB
constexpr int kT5QSlabBytes = kT5Half * 128;          // 128 query rows x 128 B: 16 KiB
constexpr int kT5QBytes = 4 * kT5QSlabBytes;          // half 0: dims 0-63 | 64-127, half 1: the same
constexpr int kT5StageBytes = 4 * kT5SlabBytes;       // K dims lo | K dims hi | V dims lo | V dims hi: 32 KiB
constexpr int kT5OffStage = kT5QBytes;
constexpr int kT5OffBar = kT5OffStage + kT5Stages * kT5StageBytes;
constexpr int kT5Smem = kT5OffBar + 256;              // 196864 B: one CTA per SM
constexpr int kT5TmemCols = 512;                      // S of half h, buffer b: columns 128h + 64b (P overlays the first 32
                                                      // of them); O of half h: columns 256 + 128h
constexpr uint32_t kT5ColO = 256;
constexpr float kRescaleStep = 8.f;                   // the reference maximum moves only when the row maximum grew by more (log2 units)

// Instruction descriptors (kind::f16): fp32 accumulate (bit 4), fp16 A and B (formats 0), N >> 3 at bit 17,
// M >> 4 at bit 24; bit 16 = B is MN-major (V: the 64 dims of a key row are contiguous).
constexpr uint32_t kIdescS = (1u << 4) | ((uint32_t)(kT5Keys >> 3) << 17) | ((uint32_t)(kT5Half >> 4) << 24);
constexpr uint32_t kIdescPV = (1u << 4) | (1u << 16) | ((uint32_t)(kHeadDim >> 3) << 17) | ((uint32_t)(kT5Half >> 4) << 24);

// Shared-memory matrix descriptor, 128-byte swizzle: start address, leading / stride byte offsets (all >> 4),
// descriptor version 1 (bit 46), layout type 2 = SWIZZLE_128B (bits 61-63).  Atoms are 8 rows x 128 B = 1024 B.
// The issuing thread is one dependent instruction stream, so what it computes per MMA is what paces the tensor
// pipe: the descriptor is split into a constant high word and a low word (address and leading offset, both >> 4) that
// moves by a compile-time constant from one MMA to the next.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);      // stride 1024 B, version 1, SWIZZLE_128B
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t umma_desc_of(uint32_t lo) { return ((uint64_t)kDescHi << 32) | (uint64_t)lo; }
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// The same with the A operand in tensor memory (M = 128: row r in lane r, two fp16 of consecutive K per 32-bit column).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t"
        "}\n" ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// One lane of a converged warp (the same one every time for a full mask).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive columns of this thread's tensor-memory lane (the warp's 32 lanes = 32 rows of the tile)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Hand-overs between the warps of a CTA last a fraction of a microsecond: poll a while before reading the clock
// (reading it costs more than such a wait lasts), then fall back to the bounded wait.
__device__ __forceinline__ bool t5_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
        if (mbar_try(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag);
}

constexpr int kT5Threads = 352;       // 8 softmax warps (4 per half), an MMA-issuing warp per half, the page-copy warp

#ifdef NOVA_TIMELINE       // profiling build: cycles spent inside a wait are added to a counter
#define T5_TIMED(acc, expr) [&]() { const long long t_ = clock64(); const bool r_ = (expr); acc += clock64() - t_; return r_; }()
#else
#define T5_TIMED(acc, expr) (expr)
#endif

// kPrefix = true is the shared-prefix form used by decode steps of sessions that share their first pages: the tile
// rows are (session, head) pairs - each session's single query - the keys are chunk `bid / (row tiles * NKV)` of the
// first prefix_pages 16-key tiles of the FIRST session's table, nothing is masked, q is rotated on the way in when
// the append is fused, and the result is an un-normalised partial row per chunk (m, l, acc) for the merge kernel.
template <bool kPrefix>
__global__ void __launch_bounds__(kT5Threads, 1)
attn_prefill_tc5_kernel(AttnLaunch a, const __grid_constant__ CUtensorMap tmk, const __grid_constant__ CUtensorMap tmv, int tq,
                        int n_qtiles, int prefix_pages, int chunk_pages) {
    // No static shared memory and no alignment attribute: the dynamic region then starts at the front of the CTA's
    // window, which is 1024-byte aligned as the swizzled tiles need.  The kernel checks that and reports
    // NOVA_ERR_UNSUPPORTED otherwise.
    extern __shared__ unsigned char smem_raw[];
    uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(smem_raw + kT5OffBar + 224);
    volatile int& s_abort = *reinterpret_cast<volatile int*>(smem_raw + kT5OffBar + 228);

    const int lane = (int)threadIdx.x & 31;
    // (a shuffle result is warp-uniform for the compiler: the issuing warps then keep descriptors in uniform registers)
    const int warp = __shfl_sync(0xffffffffu, (int)threadIdx.x >> 5, 0);
    const int G = a.n_heads / a.n_kv_heads;
    const int NH = a.n_heads, NKV = a.n_kv_heads, NQ = a.n_q;
    const PageGeom geo = page_geom(a.kv_shift);            // 16-key tiles (pages of 16, 32 or 64 tokens)
    const int tpp_mask = (1 << geo.tpp_shift) - 1;
    const uint32_t base = smem_u32(smem_raw);

    // blockIdx.x -> (query tile, kv head, session); late tiles (most keys) first
    int bid = (int)blockIdx.x;
    const int qtile = n_qtiles - 1 - bid % n_qtiles;
    bid /= n_qtiles;
    const int kvh = bid % NKV;
    // prefix form: rows index sessions, the table is the first one's; prefill: sessions in the host's order (longest first)
    const int s = kPrefix ? 0 : (a.n_order > 0 && bid / NKV < a.n_order ? (int)a.sess_order[bid / NKV] : bid / NKV);
    const int chunk = kPrefix ? bid / NKV : 0;
    const int t0 = qtile * tq;
    const int t_cnt = NQ - t0 < tq ? NQ - t0 : tq;
    const int n_past = kPrefix ? 0 : (a.n_past ? a.n_past[s] : a.keys_imm);
    const int first_key = (!kPrefix && a.window > 0) ? n_past + a.keys_add + t0 - a.window : 0;   // nothing before it is visible to any row
    const int page_begin = kPrefix ? chunk * chunk_pages : (first_key > 0 ? first_key >> 4 : 0);   // in 16-key tiles
    const int page_end = kPrefix ? (page_begin + chunk_pages < prefix_pages ? page_begin + chunk_pages : prefix_pages)
                                 : (n_past + a.keys_add + t0 + t_cnt - 1 + 15) >> 4;
    const int keys_all = kPrefix ? page_end << 4 : n_past + a.keys_add + t0 + t_cnt - 1;   // keys seen by the tile's last query
    const int n_pages = page_end - page_begin;
    const int n_tiles = (n_pages + 3) >> 2;                             // 64-key tiles
    const int32_t* table = a.table_base + (int64_t)(a.slice_ids ? a.slice_ids[s] : s) * a.table_stride;

    // barriers (8 bytes each): K landed [4 stages], V landed [4], K part free [4], V part free [4], scores ready
    // [half][buffer], P written [half][buffer] (the half's 128 threads), P.V done [half][buffer].
    // Every waiter waits for a phase whose successor on the same barrier cannot complete without that waiter's own next
    // action, so a parity can never be mistaken for a later one.  (That is why "P written" has a barrier per buffer:
    // a half's softmax may finish tile i + 1, whose scores are computed ahead, before the issuing thread has looked at
    // tile i's barrier; tile i + 2's scores are only issued after it has.)
    const uint32_t bar_kfull = base + kT5OffBar, bar_vfull = bar_kfull + 32, bar_kfree = bar_kfull + 64, bar_vfree = bar_kfull + 96,
                   bar_sready = bar_kfull + 128, bar_pready = bar_kfull + 160, bar_pvdone = bar_kfull + 192;
    if (kPrefix) pdl_launch_dependents();      // the split over the private pages shares nothing with this kernel
    if (threadIdx.x == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(bar_kfull + 8u * (uint32_t)i, 1);
        for (int i = 0; i < 8; ++i) mbar_init(bar_kfree + 8u * (uint32_t)i, 2);        // both halves' issuers release a stage
        for (int i = 0; i < 4; ++i) mbar_init(bar_sready + 8u * (uint32_t)i, 1);
        for (int i = 0; i < 4; ++i) mbar_init(bar_pready + 8u * (uint32_t)i, kT5Half);
        for (int i = 0; i < 4; ++i) mbar_init(bar_pvdone + 8u * (uint32_t)i, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
#ifdef NOVA_TIMELINE       // which SM ran this CTA, and when
    if (a.timeline && threadIdx.x == 0 && blockIdx.x < (kPrefix ? 148 : 1700)) {
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        a.timeline[(size_t)blockIdx.x * 4 + 0] = now_ns();
        a.timeline[(size_t)blockIdx.x * 4 + 1] = smid;
    }
#endif
    const bool bad_layout = (base & 1023u) != 0 || n_pages <= 0 || ((page_end + tpp_mask) >> geo.tpp_shift) > a.table_stride;
    if (bad_layout) {                 // uniform over the CTA: nothing has been allocated yet
        if (threadIdx.x == 0 && a.status && n_pages > 0) atomicCAS(a.status, 0, (base & 1023u) ? NOVA_ERR_UNSUPPORTED : NOVA_ERR_BAD_TABLE);
        return;
    }
    if (warp == 0) {                  // tensor memory: all 512 columns (the CTA has the SM to itself), released below on every path
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"((uint32_t)kT5TmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, s_tmem_base, 0);
    bool failed = false;

    // Page copies: eight lanes of the copy warp, lane = (K or V, page j of the tile's four).  A lane brings page
    // 4i + j of the CTA's range into stage i & 3 (two boxes: dims 0-63 and 64-127) and reads its own block-table
    // entries two tiles ahead.  Stage layout: K dims lo | K dims hi | V dims lo | V dims hi, 8 KiB each; the first lane
    // of each group posts the byte count (the other lanes' bytes may land before it: the phase cannot complete
    // without that arrival).
    const int cp_j = lane & 3, cp_which = (lane >> 2) & 1;
    auto load_page = [&](int i, int ph) {
        const int stage = i & (kT5Stages - 1);
        const uint32_t dst = base + kT5OffStage + (uint32_t)stage * kT5StageBytes + (uint32_t)cp_which * 2u * kT5SlabBytes + (uint32_t)cp_j * 2048u;
        const uint32_t bar = (cp_which ? bar_vfull : bar_kfull) + 8u * (uint32_t)stage;
        const int p0 = 4 * i, cnt = n_pages - p0 < 4 ? n_pages - p0 : 4;
        if (cp_j == 0) mbar_expect_tx(bar, (uint32_t)cnt * 4096u);
        if (cp_j < cnt) {
            if (ph < 0 || ph >= a.nb) {            // never follow a bad entry; the result is flagged invalid
                if (a.status) atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
                ph = 0;
            }
            const int c1 = (int)((((int64_t)a.layer0 * a.nb + ph) << geo.kv_shift) + (((page_begin + p0 + cp_j) & tpp_mask) << 4));
            const CUtensorMap* tm = cp_which ? &tmv : &tmk;
            tma_load_3d(dst, tm, 0, c1, kvh, bar);
            tma_load_3d(dst + kT5SlabBytes, tm, 64, c1, kvh, bar);
        }
    };
    auto fetch_phys = [&](int i) -> int {       // this lane's block-table entry of tile i (0 beyond the range)
        const int p = 4 * i + cp_j;
        return p < n_pages ? __ldg(table + ((page_begin + p) >> geo.tpp_shift)) : 0;
    };
    int ph_a = 0, ph_b = 0;                     // entries of the next two tiles
    if (warp == 10 && lane < 8) {
        // ------------------------------------------------------------- every stage is filled at once
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmk) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmv) : "memory");
        }
        int e[kT5Stages];
#pragma unroll
        for (int t = 0; t < kT5Stages; ++t) e[t] = fetch_phys(t);
        ph_a = fetch_phys(kT5Stages);
        ph_b = fetch_phys(kT5Stages + 1);
#pragma unroll
        for (int t = 0; t < kT5Stages; ++t)
            if (t < n_tiles) load_page(t, e[t]);
    }
    // ---- Q -> shared memory (softmax threads: one row each), then everybody meets once
    const int row = (int)threadIdx.x;                       // tile row of a softmax thread
    const int half = row >> 7, hrow = row & (kT5Half - 1);
    int row_tok = 0, row_head = 0, row_lim = -1, row_lo = 0;
    bool row_ok = false;
    if (warp < 8) {
        const int tk = row / G, g = row - tk * G;
        row_ok = tk < t_cnt && tk < tq;
        row_tok = t0 + tk;
        row_head = kvh * G + g;
        row_lim = kPrefix ? 0x7fffffff : (row_ok ? n_past + a.keys_add + row_tok - 1 : -1);          // last visible key of the row
        row_lo = (!kPrefix && row_ok && a.window > 0) ? row_lim - a.window + 1 : 0;
        constexpr float kQScale = kAttnScale * kLog2e;
        const float* qp = a.q + (((int64_t)s * NQ + row_tok) * NH + row_head) * kHeadDim;
        if (kPrefix && a.fuse_append) {
            // q arrives un-rotated: rotate the NeoX pairs (d, d + 64) at the session's position with the same fused
            // form as the append kernel, then scale and round
            const int pos = row_ok ? a.n_past[row_tok] : 0;
            const bool rot = row_ok && pos >= 0 && pos < a.rope_rows;
            const float* cr = a.rope_cs + (int64_t)(rot ? pos : 0) * (kHeadDim / 2);
            const float* sr = a.rope_sn + (int64_t)(rot ? pos : 0) * (kHeadDim / 2);
#pragma unroll 4
            for (int c = 0; c < 8; ++c) {                  // dims 8c .. 8c+7 and their partners 64 + 8c ..
                float x0[8], x1[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) x0[e] = x1[e] = 0.f;
                if (row_ok) {
                    *reinterpret_cast<float4*>(x0) = *reinterpret_cast<const float4*>(qp + 8 * c);
                    *reinterpret_cast<float4*>(x0 + 4) = *reinterpret_cast<const float4*>(qp + 8 * c + 4);
                    *reinterpret_cast<float4*>(x1) = *reinterpret_cast<const float4*>(qp + 64 + 8 * c);
                    *reinterpret_cast<float4*>(x1 + 4) = *reinterpret_cast<const float4*>(qp + 64 + 8 * c + 4);
                }
                if (rot) {
                    float cs[8], sn[8];
                    *reinterpret_cast<float4*>(cs) = *reinterpret_cast<const float4*>(cr + 8 * c);
                    *reinterpret_cast<float4*>(cs + 4) = *reinterpret_cast<const float4*>(cr + 8 * c + 4);
                    *reinterpret_cast<float4*>(sn) = *reinterpret_cast<const float4*>(sr + 8 * c);
                    *reinterpret_cast<float4*>(sn + 4) = *reinterpret_cast<const float4*>(sr + 8 * c + 4);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float y0 = __fmaf_rn(x0[e], cs[e], -__fmul_rn(x1[e], sn[e]));
                        const float y1 = __fmaf_rn(x0[e], sn[e], __fmul_rn(x1[e], cs[e]));
                        x0[e] = y0;
                        x1[e] = y1;
                    }
                }
                const uint32_t sw = (uint32_t)(hrow * 128 + ((c ^ (hrow & 7)) << 4));
                const uint32_t a0 = base + (uint32_t)(2 * half) * kT5QSlabBytes + sw, a1 = a0 + kT5QSlabBytes;
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a0), "r"(pack_h2(x0[0] * kQScale, x0[1] * kQScale)),
                             "r"(pack_h2(x0[2] * kQScale, x0[3] * kQScale)), "r"(pack_h2(x0[4] * kQScale, x0[5] * kQScale)),
                             "r"(pack_h2(x0[6] * kQScale, x0[7] * kQScale))
                             : "memory");
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a1), "r"(pack_h2(x1[0] * kQScale, x1[1] * kQScale)),
                             "r"(pack_h2(x1[2] * kQScale, x1[3] * kQScale)), "r"(pack_h2(x1[4] * kQScale, x1[5] * kQScale)),
                             "r"(pack_h2(x1[6] * kQScale, x1[7] * kQScale))
                             : "memory");
            }
        } else {
#pragma unroll 4
        for (int c = 0; c < 16; ++c) {                     // 16 chunks of 8 dims
            float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
            if (row_ok) {
                x0 = *reinterpret_cast<const float4*>(qp + 8 * c);
                x1 = *reinterpret_cast<const float4*>(qp + 8 * c + 4);
            }
            const uint32_t w0 = pack_h2(x0.x * kQScale, x0.y * kQScale), w1 = pack_h2(x0.z * kQScale, x0.w * kQScale);
            const uint32_t w2 = pack_h2(x1.x * kQScale, x1.y * kQScale), w3 = pack_h2(x1.z * kQScale, x1.w * kQScale);
            const uint32_t addr = base + (uint32_t)((2 * half + (c >> 3)) * kT5QSlabBytes + hrow * 128 + (((c & 7) ^ (hrow & 7)) << 4));
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
        }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
#ifdef NOVA_TIMELINE
    if (kPrefix && a.timeline && threadIdx.x == 0 && blockIdx.x < 148) a.timeline[(size_t)blockIdx.x * 4 + 1] = now_ns();   // q staged
#endif

    if (warp == 10) {
        // ------------------------------------------------------------- page copies, stage by stage
        if (lane < 8) {
            for (int t = kT5Stages; t < n_tiles; ++t) {
                const int stage = t & (kT5Stages - 1);
                const uint32_t parity = (uint32_t)((t >> 2) - 1) & 1u;      // the stage's previous use (tile t - 4)
                const int ph_c = fetch_phys(t + 2);
                // the K part is free once both halves' scores of tile t - 4 are computed, the V part once both P.V are
                if (!t5_wait((cp_which ? bar_vfree : bar_kfree) + 8u * (uint32_t)stage, parity, &s_abort)) break;
                load_page(t, ph_a);
                ph_a = ph_b;
                ph_b = ph_c;
            }
        }
        __syncwarp();
    } else if (warp >= 8) {
        // ------------------------------------------------------------- MMA issue: one warp per half, one elected lane
        // A thread issues an MMA every ~80 cycles at best, more than a 64-key MMA takes: two issuers keep the pipe
        // fed.  The whole warp runs the loop (uniform control flow and operands); one elected lane issues.  MMAs of one
        // issuer execute in order, which is what the overlay of P on S relies on; the halves share only the stages.
        const int h = warp - 8;
#ifdef NOVA_TIMELINE
        long long w_p = 0, w_v = 0, w_k = 0, w_is = 0, c0 = clock64();
#else
        int w_p = 0, w_v = 0, w_k = 0;
        (void)w_p; (void)w_v; (void)w_k;
#endif
        const uint32_t q_lo0 = umma_desc_lo(base + (uint32_t)(2 * h) * kT5QSlabBytes, 16u), k_lo0 = umma_desc_lo(base + kT5OffStage, 16u),
                       v_lo0 = umma_desc_lo(base + kT5OffStage + 2u * kT5SlabBytes, (uint32_t)kT5SlabBytes);
        const uint32_t col_s = tmem + 128u * (uint32_t)h, col_o = tmem + kT5ColO + 128u * (uint32_t)h;
        // S_h(t) = Q_h.K(t)^T into score buffer t & 1: eight K-steps of 16 dims (slab j >> 2 = dims 0-63 | 64-127; a
        // step moves 32 bytes inside the swizzled 128-byte row)
        auto issue_s = [&](int t) -> bool {
            const int stage = t & (kT5Stages - 1);
            const uint32_t k_lo = k_lo0 + (uint32_t)stage * (kT5StageBytes >> 4);
            const uint32_t d_s = col_s + 64u * (uint32_t)(t & 1);
            if (!__all_sync(0xffffffffu, T5_TIMED(w_k, t5_wait(bar_kfull + 8u * (uint32_t)stage, (uint32_t)(t >> 2) & 1u, &s_abort)))) return false;
            tc_fence_after();
#ifdef NOVA_TIMELINE
            const long long ti = clock64();
#endif
            if (elect_one()) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    umma_f16(d_s, umma_desc_of(q_lo0 + (uint32_t)((j >> 2) * (kT5QSlabBytes >> 4) + (j & 3) * 2)),
                             umma_desc_of(k_lo + (uint32_t)((j >> 2) * (kT5SlabBytes >> 4) + (j & 3) * 2)), kIdescS, j > 0 ? 1u : 0u);
                umma_commit(bar_sready + 8u * (uint32_t)(2 * h + (t & 1)));
                umma_commit(bar_kfree + 8u * (uint32_t)stage);
            }
            __syncwarp();
#ifdef NOVA_TIMELINE
            w_is += clock64() - ti;
#endif
            return true;
        };
        failed = !issue_s(0);
        for (int i = 0; i < n_tiles && !failed; ++i) {
            const int stage = i & (kT5Stages - 1);
            const uint32_t v_lo = v_lo0 + (uint32_t)stage * (kT5StageBytes >> 4);
            const uint32_t p_col = col_s + 64u * (uint32_t)(i & 1);
            const uint32_t acc0 = i > 0 ? 1u : 0u;
            // The scores of the NEXT 64 keys first (their buffer was read two tiles ago): they are computed while the
            // softmax warps work on tile i and are waiting for them when those warps come back.
            if (i + 1 < n_tiles && !issue_s(i + 1)) { failed = true; break; }
            if (!__all_sync(0xffffffffu, T5_TIMED(w_v, t5_wait(bar_vfull + 8u * (uint32_t)stage, (uint32_t)(i >> 2) & 1u, &s_abort)))) { failed = true; break; }
            // P_h(i) is written (the half's softmax has read S_h(i))
            if (!__all_sync(0xffffffffu, T5_TIMED(w_p, t5_wait(bar_pready + 8u * (uint32_t)(2 * h + (i & 1)), (uint32_t)(i >> 1) & 1u, &s_abort)))) { failed = true; break; }
            tc_fence_after();
            if (elect_one()) {
                // O_h += P_h.V: four K-steps of 16 keys; P is read from tensor memory (16 keys = 8 columns); V is
                // MN-major: 16 key rows = two 1024-byte atoms (stride), the two halves of the 128 dims are a slab apart
                // (leading offset)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    umma_f16_ts(col_o, p_col + (uint32_t)(8 * j), umma_desc_of(v_lo + (uint32_t)(j * (2048 >> 4))), kIdescPV, j > 0 ? 1u : acc0);
                umma_commit(bar_pvdone + 8u * (uint32_t)(2 * h + (i & 1)));
                umma_commit(bar_vfree + 8u * (uint32_t)stage);
            }
            __syncwarp();
        }
        if (failed && lane == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
#ifdef NOVA_TIMELINE
        if (a.timeline && blockIdx.x < (kPrefix ? 148 : 1700) && h == 0 && lane == 0) {       // cycles: total | K wait | P wait | V wait
            unsigned long long* t = a.timeline + (kPrefix ? 148 : 1700) * 4 + (size_t)blockIdx.x * 4;
            t[0] = (unsigned long long)(clock64() - c0);
            t[1] = (unsigned long long)w_k;
            t[2] = (unsigned long long)w_p;
            t[3] = (unsigned long long)w_v;
            a.timeline[(size_t)blockIdx.x * 4 + 3] = (unsigned long long)w_is;      // issuing the score MMAs
        }
#endif
    } else {
        // ------------------------------------------------------------- softmax warps: thread = one row of S and O
        const uint32_t t_lane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);  // this warp's 32 lanes of tensor memory
        const uint32_t col_s = 128u * (uint32_t)half, col_o = kT5ColO + 128u * (uint32_t)half;
        const uint32_t my_sready = bar_sready + 16u * (uint32_t)half, my_pvdone = bar_pvdone + 16u * (uint32_t)half;
        float m_ref = -INFINITY, l = 0.f;
#ifdef NOVA_TIMELINE
        long long x_s = 0, x_pv = 0, x0 = clock64();
#else
        int x_s = 0, x_pv = 0;
        (void)x_s; (void)x_pv;
#endif
        for (int i = 0; i < n_tiles; ++i) {
            // (the warp decides together: what follows is warp-collective)
            if (!__all_sync(0xffffffffu, T5_TIMED(x_s, t5_wait(my_sready + 8u * (uint32_t)(i & 1), (uint32_t)(i >> 1) & 1u, &s_abort)))) { failed = true; break; }
            tc_fence_after();
            uint32_t sv[2][32];
            tmem_ld32(t_lane + col_s + 64u * (uint32_t)(i & 1), sv[0]);
            tmem_ld32(t_lane + col_s + 64u * (uint32_t)(i & 1) + 32, sv[1]);
            tmem_wait_ld();
            const int key0 = (page_begin + 4 * i) << 4;
            const int kcount = keys_all - key0 < kT5Keys ? keys_all - key0 : kT5Keys;     // real keys in this tile
            const int hi_k = (row_lim < key0 + kcount - 1 ? row_lim : key0 + kcount - 1) - key0;   // last visible column
            const int lo_k = row_lo - key0;                                                        // first visible column
            float mx = -INFINITY;
            if (__all_sync(0xffffffffu, hi_k >= kT5Keys - 1 && lo_k <= 0)) {      // every key of the tile is visible to the warp's rows
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; ++c) mx = fmaxf(mx, __uint_as_float(sv[h][c]));
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int col = 32 * h + c;
                        float v = __uint_as_float(sv[h][c]);
                        v = (col <= hi_k && col >= lo_k) ? v : -INFINITY;
                        sv[h][c] = __float_as_uint(v);
                        mx = fmaxf(mx, v);
                    }
            }
            // reference maximum: moves only when the row maximum outgrew it by more than kRescaleStep
            float scale = 1.f;
            if (mx > m_ref + kRescaleStep || (m_ref == -INFINITY && mx > -INFINITY)) {
                scale = m_ref == -INFINITY ? 0.f : ex2(m_ref - mx);
                m_ref = mx;
            }
            const float ms = m_ref == -INFINITY ? 0.f : m_ref;          // nothing visible yet: keep exp arguments finite
            uint32_t pk[32];
            float psum = 0.f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                const int h = c >> 4, cc = (2 * c) & 31;
                const float e0 = ex2(__uint_as_float(sv[h][cc]) - ms), e1 = ex2(__uint_as_float(sv[h][cc + 1]) - ms);
                psum += e0 + e1;
                pk[c] = pack_h2(e0, e1);                                 // keys 2c, 2c+1 of the tile
            }
            l = fmaf(l, scale, psum);
            if (i > 0 && __any_sync(0xffffffffu, scale != 1.f)) {
                // O is rescaled between two P.V products: the previous one must be done (the one before it is, since
                // these scores were computed after it, so the barrier's parity cannot be mistaken)
                if (!__all_sync(0xffffffffu, T5_TIMED(x_pv, t5_wait(my_pvdone + 8u * (uint32_t)((i - 1) & 1), (uint32_t)((i - 1) >> 1) & 1u, &s_abort)))) { failed = true; break; }
                tc_fence_after();
#pragma unroll 1
                for (int cc = 0; cc < 4; ++cc) {
                    uint32_t ov[32];
                    tmem_ld32(t_lane + col_o + 32u * (uint32_t)cc, ov);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * scale);
                    tmem_st32(t_lane + col_o + 32u * (uint32_t)cc, ov);
                }
                tmem_wait_st();
            }
            // P (fp16) over the first 32 columns of the scores just read: the products issued before the next scores
            // land in this buffer (tile i + 2) include the P.V that reads it
            tmem_st32(t_lane + col_s + 64u * (uint32_t)(i & 1), pk);
            tmem_wait_st();
            if (kcount < kT5Keys) {
                // key rows past the last real key hold stale bytes: their weights are 0, but 0 * Inf/NaN would poison O.
                // The V rows of this tile must have landed first (the copy of a partly filled page brings such rows too).
                // Each half does it before its own P.V (the two write the same zeros).
                if (!__all_sync(0xffffffffu, t5_wait(bar_vfull + 8u * (uint32_t)(i & (kT5Stages - 1)), (uint32_t)(i >> 2) & 1u, &s_abort))) { failed = true; break; }
                const uint32_t st_addr = base + kT5OffStage + (uint32_t)(i & (kT5Stages - 1)) * kT5StageBytes + 2u * kT5SlabBytes;
                for (int e = hrow; e < (kT5Keys - kcount) * 16; e += kT5Half) {
                    const int r = kcount + (e >> 4), c = e & 15;
                    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(st_addr + (uint32_t)((c >> 3) * kT5SlabBytes + r * 128 + ((c & 7) << 4))),
                                 "r"(0u)
                                 : "memory");
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            tc_fence_before();
            mbar_arrive(bar_pready + 8u * (uint32_t)(2 * half + (i & 1)));
        }
#ifdef NOVA_TIMELINE
        if (a.timeline && threadIdx.x == 0 && blockIdx.x < (kPrefix ? 148 : 1700)) {       // cycles: softmax loop total | score wait | P.V wait | tiles
            unsigned long long* t = a.timeline + (kPrefix ? 148 : 1700) * 8 + (size_t)blockIdx.x * 4;
            t[0] = (unsigned long long)(clock64() - x0);
            t[1] = (unsigned long long)x_s;
            t[2] = (unsigned long long)x_pv;
            t[3] = (unsigned long long)n_tiles;
        }
#endif
        if (!failed && !__all_sync(0xffffffffu, t5_wait(my_pvdone + 8u * (uint32_t)((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1u, &s_abort))) failed = true;
        if (failed && lane == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_TIMEOUT);
        if (kPrefix) {
            // Partial rows (m, l, acc[128]) leave through shared memory: a thread owns a row, but the rows of a token
            // are one contiguous run of G * 130 floats in the result, which the 256 threads then write together.
            // Every MMA and page copy of the CTA is done once both halves are here (a failed wait has set the status
            // word and passes through), so the staging area may start at the front of the shared memory.
            asm volatile("bar.sync 1, 256;" ::: "memory");
            tc_fence_after();
            float* stage_rows = reinterpret_cast<float*>(smem_raw);
            float* srow = stage_rows + row * kPartW;
            *reinterpret_cast<float2*>(srow) = make_float2(m_ref * (1.f / kLog2e), l);
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t ov[32];
                tmem_ld32(t_lane + col_o + 32u * (uint32_t)cc, ov);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 32; c += 2)
                    *reinterpret_cast<float2*>(srow + 2 + 32 * cc + c) = make_float2(__uint_as_float(ov[c]), __uint_as_float(ov[c + 1]));
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
#ifdef NOVA_TIMELINE
            if (a.timeline && threadIdx.x == 0 && blockIdx.x < 148) a.timeline[148 * 8 + (size_t)blockIdx.x * 4 + 2] = now_ns();   // loop done
#endif
            // the chunk partials are re-used by every layer: the previous layer's final merge may still read them
            pdl_wait();
#ifdef NOVA_TIMELINE
            if (a.timeline && threadIdx.x == 0 && blockIdx.x < 148) a.timeline[148 * 8 + (size_t)blockIdx.x * 4 + 3] = now_ns();   // dependency met
#endif
            const int seg = G * kPartW;                      // floats of one token's rows (even)
            const int total = (t_cnt < tq ? t_cnt : tq) * seg;
            float* const obase = a.out_part + (((int64_t)chunk * NQ + t0) * NH + kvh * G) * kPartW;
            const int64_t tok_stride = (int64_t)NH * kPartW;
            int e = 2 * (int)threadIdx.x, tk = e / seg, r = e - tk * seg;       // float e of the staged rows = token tk, offset r
            for (; e < total; e += 2 * kT5Rows) {
                *reinterpret_cast<float2*>(obase + tk * tok_stride + r) = *reinterpret_cast<const float2*>(stage_rows + e);
                r += 2 * kT5Rows;
                while (r >= seg) { r -= seg; ++tk; }
            }
        } else if (!failed) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            float* op = a.out + (((int64_t)s * NQ + row_tok) * NH + row_head) * kHeadDim;
#pragma unroll 1
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t ov[32];
                tmem_ld32(t_lane + col_o + 32u * (uint32_t)cc, ov);
                tmem_wait_ld();
                if (row_ok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 4)
                        *reinterpret_cast<float4*>(op + 32 * cc + c) =
                            make_float4(__uint_as_float(ov[c]) * inv, __uint_as_float(ov[c + 1]) * inv, __uint_as_float(ov[c + 2]) * inv,
                                        __uint_as_float(ov[c + 3]) * inv);
                }
            }
        }
    }
    // ---- release the tensor memory (every path of every thread ends here)
    tc_fence_before();
    __syncthreads();
#ifdef NOVA_TIMELINE
    if (a.timeline && threadIdx.x == 0 && blockIdx.x < (kPrefix ? 148 : 1700)) a.timeline[(size_t)blockIdx.x * 4 + 2] = now_ns();
#endif
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)kT5TmemCols) : "memory");
}

}  // namespace

// Query tokens per CTA of the tcgen05 prefill: as many whole tokens as fit the 256-row tile.
int attn_prefill_tc5_tile_tokens(int n_heads, int n_kv_heads) { return kT5Rows / (n_heads / n_kv_heads); }

bool attn_prefill_tc5_supports(const AttnLaunch& a) {
    const int kvs = a.kv_shift ? a.kv_shift : kKvShift;
    return a.tmap_k1 && a.tmap_v1 && a.n_layers == 1 && a.n_q >= 1 && kvs >= 4 && a.n_heads % a.n_kv_heads == 0 &&
           a.n_heads / a.n_kv_heads <= kT5Rows;
}

namespace {
int t5_set_attributes() {
    static bool attr_set[64] = {};
    int dev = 0;
    NOVA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        // 192 KiB per CTA: the whole shared-memory carve-out
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kT5Smem));
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_tc5_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kT5Smem));
        NOVA_CUDA_TRY(cudaFuncSetAttribute(attn_prefill_tc5_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                           cudaSharedmemCarveoutMaxShared));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    return NOVA_OK;
}
}  // namespace

int launch_attn_prefill_tc5(const AttnLaunch& a, cudaStream_t s) {
    if (!attn_prefill_tc5_supports(a)) return NOVA_ERR_UNSUPPORTED;
    if (a.n_sessions <= 0) return NOVA_OK;
    const int rc = t5_set_attributes();
    if (rc != NOVA_OK) return rc;
    const int tq = attn_prefill_tc5_tile_tokens(a.n_heads, a.n_kv_heads);
    const int n_qtiles = (a.n_q + tq - 1) / tq;
    const long long ctas = (long long)n_qtiles * a.n_kv_heads * a.n_sessions;
    if (ctas > 0x7fffffffLL) return NOVA_ERR_TOO_LARGE;
    const CUtensorMap* tk = static_cast<const CUtensorMap*>(a.tmap_k1);
    const CUtensorMap* tv = static_cast<const CUtensorMap*>(a.tmap_v1);
    attn_prefill_tc5_kernel<false><<<(unsigned)ctas, kT5Threads, kT5Smem, s>>>(a, *tk, *tv, tq, n_qtiles, 0, 0);
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

// Chunks of the shared prefix (prefix_pages 16-key tiles) for the tcgen05 prefix launch: whole 64-key tiles per chunk,
// at least four of them, and about a third of the SMs in all - the split over the private pages runs beside it.
int attn_prefix_tc5_chunks(int n_sessions, int n_heads, int n_kv_heads, int prefix_pages, int* chunk_pages) {
    const int tq = attn_prefill_tc5_tile_tokens(n_heads, n_kv_heads);
    const int n_rt = (n_sessions + tq - 1) / tq;
#ifndef NOVA_T5_PREFIX_EIGHTHS
#define NOVA_T5_PREFIX_EIGHTHS 4
#endif
    int chunks = (sm_count() * NOVA_T5_PREFIX_EIGHTHS / 8) / (n_rt * n_kv_heads);
    if (chunks > prefix_pages / 8) chunks = prefix_pages / 8;
    if (chunks < 1) chunks = 1;
    int per = (prefix_pages + chunks - 1) / chunks;
    per = (per + 3) & ~3;
    if (chunk_pages) *chunk_pages = per;
    return (prefix_pages + per - 1) / per;
}

// Partials of every (session, head) row over the shared pages [0, prefix_pages) (in 16-key tiles) of the batch's
// first session: a.out_part [chunks][n_sessions][NH][130], a.q [n_sessions][NH][128] (un-rotated when a.fuse_append),
// one layer.  The tcgen05 counterpart of launch_attn_prefix.
int launch_attn_prefix_tc5(const AttnLaunch& a_in, int prefix_pages, cudaStream_t s) {
    if (a_in.n_sessions <= 0) return NOVA_OK;
    AttnLaunch a = a_in;
    a.n_q = a_in.n_sessions;             // the sessions are the query rows of one pseudo-session
    if (!attn_prefill_tc5_supports(a) || !a.out_part || prefix_pages < 1) return NOVA_ERR_UNSUPPORTED;
    if (a.fuse_append && (!a.n_past || !a.rope_cs || !a.rope_sn)) return NOVA_ERR_INVALID;
    const int rc = t5_set_attributes();
    if (rc != NOVA_OK) return rc;
    int chunk_pages = 0;
    const int chunks = attn_prefix_tc5_chunks(a_in.n_sessions, a.n_heads, a.n_kv_heads, prefix_pages, &chunk_pages);
    const int tq = attn_prefill_tc5_tile_tokens(a.n_heads, a.n_kv_heads);
    const int n_rt = (a.n_q + tq - 1) / tq;
    const long long ctas = (long long)n_rt * a.n_kv_heads * chunks;
    const CUtensorMap* tk = static_cast<const CUtensorMap*>(a.tmap_k1);
    const CUtensorMap* tv = static_cast<const CUtensorMap*>(a.tmap_v1);
    const cudaError_t le = launch_kernel_pdl(attn_prefill_tc5_kernel<true>, dim3((unsigned)ctas), dim3(kT5Threads), (size_t)kT5Smem, s,
                                             a.pdl != 0, a, *tk, *tv, tq, n_rt, prefix_pages, chunk_pages);
    if (le != cudaSuccess) {
        set_cuda_error(le, "prefix attention launch (tcgen05)");
        return NOVA_ERR_CUDA;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
