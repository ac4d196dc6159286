// common.cuh — shared declarations of the sm_100a paged-KV decode library.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <atomic>
#include <cstdint>
#include <cstdio>

#include "../../include/nova_b200.h"

namespace novab {

constexpr int kHeadDim = 128;   // the only head_dim built (every model of the reference uses 128)
constexpr int kKvBlock = 16;    // tokens per page by default (the reference's default NOVA_KV_BLOCK)
constexpr int kKvShift = 4;
// Pages of 8, 16, 32 or 64 tokens (NOVA_KV_BLOCK, code/graph/kv_pool_cfg.h:12-26) are a runtime property of a
// launch: kv_shift = log2(tokens per page).  The kernels stream TILES of kTileKeys = min(16, page) keys: a page of
// 32 or 64 tokens is 2 or 4 tiles that share one block-table entry, a page of 8 tokens is one half-filled tile.
constexpr int kTileKeysMax = 16;
inline int kv_shift_of_block(int kv_block) { return kv_block == 8 ? 3 : kv_block == 16 ? 4 : kv_block == 32 ? 5 : kv_block == 64 ? 6 : -1; }
constexpr int kPartW = kHeadDim + 2;   // partial row handed to callers: m, l, acc[128]  (src/kernel/attn.cu:150-158)
constexpr int kSlotW = kHeadDim + 4;   // the same row inside the split-K scratch: m, l, 2 pad, acc[128] (acc 16-byte aligned)
// 1/sqrt(128), the literal the reference uses (src/kernel/attn.cu:21)
constexpr float kAttnScale = 0.08838834764831845f;
constexpr float kLog2e = 1.4426950408889634f;

// ---- error plumbing -------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char* what);
void count_launch(int n = 1);
int sm_count();                  // multiprocessors of the current device
constexpr int kMaxSms = 256;     // upper bound used to size per-SM scratch (partial slots)
constexpr int kTimelineCtas = 148;   // CTAs per record of the profiling build's time stamps (NOVA_TIMELINE)

// Launch with or without the programmatic-stream-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Device side of the above (no-ops when the launch did not carry the attribute).
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

#define NOVA_CUDA_TRY(expr)                                   \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) {                              \
            ::novab::set_cuda_error(_e, #expr);               \
            return NOVA_ERR_CUDA;                             \
        }                                                     \
    } while (0)

#define NOVA_LAUNCH_CHECK()                                   \
    do {                                                      \
        cudaError_t _e = cudaGetLastError();                  \
        if (_e != cudaSuccess) {                              \
            ::novab::set_cuda_error(_e, "kernel launch");     \
            return NOVA_ERR_CUDA;                             \
        }                                                     \
        ::novab::count_launch();                              \
    } while (0)

// ---- KV element access ----------------------------------------------------------------
template <typename T> struct KvTraits;
template <> struct KvTraits<float> {
    static constexpr int kDtype = NOVA_KV_F32;
    __device__ static __forceinline__ float load(const float* p) { return *p; }
    __device__ static __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct KvTraits<__half> {
    static constexpr int kDtype = NOVA_KV_F16;
    __device__ static __forceinline__ float load(const __half* p) { return __half2float(*p); }
    __device__ static __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};

// ---- attention launch description (shared by the SIMT and tensor-core kernels) ---------
//
// Work is cut stream-K style.  A "row" is one (layer, session, kv-head group): its pages
// are ceil(n_keys/16).  All pages of all rows of the launch form one line of P pages; CTA c
// owns [floor(c*P/C), floor((c+1)*P/C)).  A CTA whose range crosses a row boundary produces
// one partial per row it touches; the (CTA, row) pairs form a chain, so `c + row` names a
// unique partial slot.  A row that one CTA covers alone is normalised and written at once; the
// others are merged, in CTA order, by the combine kernel that follows the split kernel
// (the reference's split + combine pair, src/kernel/attn.cu:498-512).
struct AttnLaunch {
    const void* pool_k;          // [L][NB][page tokens][NKV][128]
    const void* pool_v;
    int32_t kv_shift;            // log2(tokens per page): 3..6; 0 is read as 4 (16-token pages)
    int32_t window;              // prefill only: > 0 = sliding window, query at position p sees keys (p - window, p]
    int32_t n_order;             // tcgen05 prefill only: > 0 = the CTAs take the sessions in the order sess_order[0..n_order)
    unsigned char sess_order[64];   //   (longest context first, so that the last CTAs of the launch are the short ones)
    const int32_t* table_base;   // device block tables, one per slice
    int64_t table_stride;        // entries per slice table (nblocks)
    const int32_t* slice_ids;    // [S] slice of each batch entry; nullptr: entry s uses table_base + s*stride
    const int32_t* n_past;       // [S] device; n_keys = n_past[s] + keys_add; nullptr: n_keys = keys_imm
    int32_t keys_add;
    int32_t keys_imm;
    const float* q;              // [layers][S][NH][128] fp32, already rotated
    float* out;                  // [layers][S][NH][128]
    float* part;                 // partial slots [(C + rows)][heads_per_row][kSlotW]
    int32_t* status;             // device status word (0 ok)
    int32_t n_sessions;
    int32_t n_q;                 // query tokens per session (0/1 = decode).  Query t of session s sees
                                 // n_past[s] + keys_add + t keys (causal prefill); q/out are [layers][S][n_q][NH][128].
                                 // "Unit" below = s * n_q + t, a session as far as the work split is concerned.
    int32_t layer0;              // first layer of the pools this launch reads
    int32_t n_layers;            // layers covered by this launch (1 = per-layer call)
    int32_t nb;                  // physical pages per layer
    int32_t n_heads, n_kv_heads;
    int32_t kv_group;            // kv heads handled by one CTA (<= 4)
    int64_t page_lo, page_hi;    // restrict every session to logical pages [lo, hi) (multi-GPU split); hi<0: all
    int32_t write_partial_only;  // 1: leave un-normalised (m,l,acc) rows in `out_part` instead of `out`
    float* out_part;             // [layers][S][NH][130]
    const void* tmap_k;          // host pointers to the CUtensorMap of each pool (tensor-core kernel only)
    const void* tmap_v;
    const void* tmap_k1;         // the same pools with one kv head per box (prefill kernel)
    const void* tmap_v1;
    // Fused RoPE + append (tensor-core kernel): when fuse_append != 0 the CTA that owns a session's
    // last page rotates k_new at n_past[s], stores k_new/v_new into that page (pool and the staged copy)
    // and every CTA rotates q on the fly; q itself is left as it was.
    int32_t fuse_append;
    void* pool_k_w;              // the pools again, writable
    void* pool_v_w;
    float* k_new;                // [layers][S][NKV][128], rotated in place
    const float* v_new;          // [layers][S][NKV][128]
    const float* rope_cs;        // [rope_rows][64]
    const float* rope_sn;
    int64_t rope_rows;
    // Programmatic dependent launch: 1 = this launch may start while the kernels before it in the
    // stream are still running.  The caller promises that those kernels neither write what this launch
    // reads (pages of earlier steps, tables, n_past, its q/k/v) nor touch what it writes for its own
    // layers (their pages, k rows, outputs); the shared partial-slot scratch is written only after
    // griddepcontrol.wait.  2 = the same early start, but without the promise for q, k_new and v_new: the
    // kernel reads those only after griddepcontrol.wait (tables, positions and page copies still start early).
    int32_t pdl;
    // With pdl: 1 = shape the launch for a chain of one-layer launches that should overlap (the split leaves
    // some SMs without a CTA, the merge uses few CTAs); 0 = only the early start and the late wait.
    int32_t pdl_spare;
    // Work-split weight of starting a row inside a CTA (q fetch, and with the fused append the new
    // token's k/v fetch at the row end next to it), in pages: every row is treated as that many pages
    // longer at its start, so a CTA whose range crosses a row boundary gets fewer real pages.
    int32_t row_setup_pages;
    // Merge kernel only: n_extra more partial rows per (session, head), extra_parts [n_extra][S * NH][130]
    // (one layer), are folded into every row after the split-K slots, and the normalised result goes to
    // `out` although the split kernel ran with write_partial_only (the cascade's final merge).
    const float* extra_parts;
    int32_t n_extra;
    unsigned long long* timeline;   // optional [n_ctas][8] globaltimer stamps (profiling aid), or nullptr
};

constexpr int kMaxRowsSmem = 1024;   // (sessions x kv groups) prefix entries kept in shared memory

// Launchers (defined in attn_simt.cu / attn_mma.cu).  n_ctas == 0 picks a default.
int launch_attn_simt(const AttnLaunch& a, int kv_dtype, int n_ctas, cudaStream_t s);
int launch_attn_mma(const AttnLaunch& a, int kv_dtype, int n_ctas, cudaStream_t s);
int attn_default_ctas_simt(int n_kv_heads);
int attn_default_ctas_mma();
bool attn_mma_built();
int attn_make_tmap(void* out_map, void* pool, int64_t slot_rows, int n_kv_heads, int kv_group, int box_rows, int elem_bytes);
int launch_attn_prefill(const AttnLaunch& a, cudaStream_t s);     // query-tiled tensor-core prefill (n_q >= 1, one layer)
int attn_prefill_tile_tokens(int n_heads, int n_kv_heads);
int launch_attn_prefill_tc5(const AttnLaunch& a, cudaStream_t s);    // the same on tcgen05 + tensor memory (pages of >= 16 tokens)
bool attn_prefill_tc5_supports(const AttnLaunch& a);
int attn_prefix_tc5_chunks(int n_sessions, int n_heads, int n_kv_heads, int prefix_pages, int* chunk_pages);
int launch_attn_prefix_tc5(const AttnLaunch& a, int prefix_pages, cudaStream_t s);   // shared-prefix partials on tcgen05
// Shared-prefix form of the same kernel: decode queries of n_sessions sessions over the shared pages
// [0, prefix_pages) of the first session's table, as partials a.out_part [chunks][n_sessions][NH][130].
int attn_prefix_chunks(int n_sessions, int n_heads, int n_kv_heads, int prefix_pages, int* chunk_pages);
int launch_attn_prefix(const AttnLaunch& a, int prefix_pages, cudaStream_t s);
int launch_attn_combine(const AttnLaunch& a, int n_ctas_split, cudaStream_t s);   // after either split kernel
int attn_split_ctas_simt(const AttnLaunch& a, int n_ctas);
int attn_split_ctas_mma(const AttnLaunch& a, int n_ctas);
int launch_lse_combine(const float* parts, int n_parts, int n_rows, float* out, cudaStream_t s);
constexpr int kMaxPeerRanks = 8;        // ranks of one NVLink domain that can share a long session
constexpr int kLLRowBytes = 16 * (1 + kHeadDim / 2);   // a partial row as 16-byte {value, epoch, value, epoch} words: (m, l) + 128 values
size_t peer_region_bytes(int n_rows);   // bytes one source rank's rows take in an exchange slot
int launch_lse_exchange(const float* part, void* const* slot_base, int n_ranks, int my_rank, int n_rows, long long epoch,
                        unsigned long long timeout_ns, float* out, int32_t* status, cudaStream_t s);
int launch_attn_combine_exchange(const AttnLaunch& a, int n_ctas_split, void* const* slot_base, int n_ranks, int my_rank,
                                 long long epoch, unsigned long long timeout_ns, int32_t* status, cudaStream_t s);

// rope / append / page utilities (rope_append.cu)
int launch_rope_table(float* cs, float* sn, int64_t n_pos, int theta, cudaStream_t s);
struct AppendLaunch {
    void* pool_k; void* pool_v;
    int32_t kv_shift;             // log2(tokens per page); 0 is read as 4
    const int32_t* table_base; int64_t table_stride;
    const int32_t* slice_ids;     // [S] or nullptr (see AttnLaunch)
    const int32_t* n_past;        // [S] device write positions, or nullptr: pos_imm
    int64_t pos_imm;
    float* q; float* k; const float* v;   // [layers][S][n_tok][NH|NKV][128]
    const float* cs; const float* sn; int64_t rope_rows;
    int32_t* status;
    int32_t n_sessions, n_tok, layer0, n_layers, nb, n_heads, n_kv_heads, neox, kv_dtype;
};
int launch_rope_append(const AppendLaunch& a, cudaStream_t s);
struct CowEvent { int32_t src, dst; int32_t* table_entry; };
int launch_cow_copy(void* pool_k, void* pool_v, int n_layers, int nb, size_t page_bytes,
                    const CowEvent* ev, int n_events, cudaStream_t s);
int launch_zero_pages(void* pool_k, void* pool_v, int n_layers, int nb, size_t page_bytes,
                      const int32_t* table_dev, int n_pages, cudaStream_t s);
int launch_advance(int32_t* n_past, int n, cudaStream_t s, int delta = 1);
int launch_synth_normal(float* dst, size_t n, uint64_t key, uint64_t first_index, cudaStream_t s);

}  // namespace novab
