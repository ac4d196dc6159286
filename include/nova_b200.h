/* nova_b200.h — C ABI of the B200 paged-KV decode path.
 *
 * One shared library (libnova_b200.so) exports everything below with C linkage:
 * plain pointers, sizes and integer handles, no C++ or framework types.  Every
 * entry point names the interface of the Conflux Nova reference it replaces
 * (file:line inside the reference project).  Unless stated otherwise a function
 * returns NOVA_OK (0) or a negative NOVA_ERR_* code; nothing here calls abort().
 *
 * Memory model (same as the reference): all device memory of an engine is
 * allocated once at nova_engine_create() and lives until nova_engine_destroy();
 * the host-side block table is the source of truth and its device mirror is
 * refreshed by the call that mutates it.  Launch functions are asynchronous on
 * the stream they are given and never synchronise.
 */
#ifndef NOVA_B200_H_
#define NOVA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
#define NOVA_OK               0
#define NOVA_ERR_INVALID     (-1)  /* bad argument / handle                     */
#define NOVA_ERR_POOL_FULL   (-2)  /* no free page (KvPool::cow_slice's -2)     */
#define NOVA_ERR_NO_SLICE    (-3)  /* KvPool::acquire() would return nullptr    */
#define NOVA_ERR_NO_SESSION  (-4)  /* all session slots in use                  */
#define NOVA_ERR_CUDA        (-5)  /* a CUDA runtime call failed                */
#define NOVA_ERR_BAD_TABLE   (-6)  /* block-table entry outside [0, NB)         */
#define NOVA_ERR_TIMEOUT     (-7)  /* a bounded device-side wait ran out        */
#define NOVA_ERR_UNSUPPORTED (-8)  /* shape / dtype not built into the library  */
#define NOVA_ERR_TOO_LARGE   (-9)  /* size beyond a documented fixed maximum    */
#define NOVA_ERR_BUSY        (-10) /* pages of the slice are still mapped by another session */

const char* nova_status_string(int status);
/* Text of the last CUDA error seen by this thread's calls (empty if none). */
const char* nova_last_cuda_error(void);

/* KV element type of the page pools. */
#define NOVA_KV_F32 0   /* the reference's format (float* pool_k/pool_v, include/nova/model.h:173-174) */
#define NOVA_KV_F16 1   /* IEEE half, value = round-to-nearest-even of the fp32 value */

/* Opaque CUDA stream (cudaStream_t).  NULL = the legacy default stream. */
typedef void* nova_stream_t;

/* --------------------------------------------------------------------- HAL */
/* The reference names these six functions as its device layer
 * (README.md:203 "dev_alloc / dev_free / dev_upload / dev_download / dev_sync /
 * dev_max_alloc") without shipping a header; semantics follow its SYCL
 * Device::alloc/upload/download/zero/sync (code/device/sycl/device.h:143-148):
 * upload/download are synchronous, alloc of 0 bytes returns NULL.
 * All act on the calling thread's current device (dev_select). */
int    dev_select(int device);                              /* cudaSetDevice */
int    dev_count(void);
void*  dev_alloc(size_t bytes);                             /* NULL on failure or bytes==0 */
void   dev_free(void* p);
int    dev_upload(void* dst_dev, const void* src_host, size_t bytes);
int    dev_download(void* dst_host, const void* src_dev, size_t bytes);
int    dev_zero(void* dst_dev, size_t bytes);
int    dev_sync(void);
size_t dev_max_alloc(void);                                 /* free device bytes right now */
void*  dev_host_alloc(size_t bytes);                        /* pinned host memory (model.cpp staging buffer) */
void   dev_host_free(void* p);
/* One dev_alloc allocation shared between the processes of a node (one process per GPU); no counterpart in
 * the reference, which is single-process.  The owner exports a 64-byte handle, a peer opens it and gets a
 * pointer valid in its own kernels (peer access over NVLink is switched on by the open). */
int    dev_ipc_export(void* dev_ptr, void* handle64);
int    dev_ipc_open(const void* handle64, void** dev_ptr);
int    dev_ipc_close(void* dev_ptr);
int    dev_stream_create(nova_stream_t* out);
int    dev_stream_destroy(nova_stream_t s);
int    dev_stream_sync(nova_stream_t s);
/* CUDA events on a stream, for timing on the device (Profiler / scope_cuda.h:73-140 pairs). */
typedef void* nova_event_t;
int    dev_event_create(nova_event_t* out);
int    dev_event_destroy(nova_event_t e);
int    dev_event_record(nova_event_t e, nova_stream_t s);
int    dev_event_sync(nova_event_t e);
int    dev_event_elapsed_ms(nova_event_t start, nova_event_t stop, float* ms);

/* ----------------------------------------------- block-ID protocol (host) */
/* kv_hash_ids  (code/graph/kv_block.h:21-64): ids -> decimal text -> hex of the
 * ASCII bytes -> 64-bit blocks (last one zero-padded) -> fold ends pairwise
 * until one block is left.  Empty input -> 0. */
uint64_t nova_kv_hash_ids(const int32_t* ids, size_t n);
/* kv_hash_text (kv_block.h:67-72): the same over the bytes of a string. */
uint64_t nova_kv_hash_text(const char* bytes, size_t n);
/* kv_hash_hex  (kv_block.h:74-79): 16 upper-case hex digits + NUL into out[17]. */
void     nova_kv_hash_hex(uint64_t v, char* out17);
/* kv_block_id  (kv_block.h:81-83): "{ PPPPPPPPPPPPPPPP . SSSSSSSSSSSSSSSS }" + NUL into out[40]. */
void     nova_kv_block_id(uint64_t prefix, uint64_t suffix, char* out40);

/* BlockRegistry (code/graph/kv_registry.h:26-66). */
typedef struct nova_registry nova_registry;
typedef struct {
    uint64_t prefix, suffix;
    int32_t  session, turn;
    int64_t  pos0, pos1;
} nova_kv_block;
nova_registry* nova_registry_create(void);
void   nova_registry_destroy(nova_registry* r);
void   nova_registry_set_capacity(nova_registry* r, size_t n);     /* kv_registry.h:28 */
size_t nova_registry_capacity(const nova_registry* r);
void   nova_registry_put(nova_registry* r, const nova_kv_block* b); /* :32-36 */
int    nova_registry_find(const nova_registry* r, uint64_t prefix, uint64_t suffix,
                          nova_kv_block* out);                      /* :38-41; 1 found, 0 not */
int    nova_registry_live(const nova_registry* r);                  /* :43 */
int    nova_registry_total(const nova_registry* r);                 /* :44 */

/* ------------------------------------------- host page pool (no device) */
/* KvPool (code/graph/kv_pool.h:68-197) on its own, for callers that keep the
 * reference's split between host bookkeeping and device copies.  Slices are
 * named by the id KvPool hands out (0,1,2,… then LIFO reuse). */
typedef struct nova_pool nova_pool;
nova_pool* nova_pool_create(int kv_block);                          /* kKvBlock: 8/16/32/64 */
void nova_pool_destroy(nova_pool* p);
int  nova_pool_init(nova_pool* p, int n_slices, int64_t ctx);       /* KvPool::init :70-84 */
int  nova_pool_acquire(nova_pool* p);                               /* :90-113; slice id or NOVA_ERR_NO_SLICE */
int  nova_pool_release(nova_pool* p, int slice);                    /* :168-174 */
int  nova_pool_alloc_block(nova_pool* p);                           /* :116-122; page id or -1 */
int  nova_pool_free_block(nova_pool* p, int b);                     /* :123-126 */
int  nova_pool_ref_block(nova_pool* p, int b);                      /* :127 */
int  nova_pool_refcnt(const nova_pool* p, int b);                   /* :128 */
int  nova_pool_attach(nova_pool* p, int dst, int src, int k);       /* :132-138 */
int  nova_pool_attach_prefix(nova_pool* p, int dst, int src, int64_t n_tokens); /* :141-148 */
int  nova_pool_cow_slice(nova_pool* p, int slice, int64_t pos);     /* :153-166; new page, -1 none, -2 full */
int  nova_pool_need_copy(const nova_pool* p, int slice, int* from, int* blk);   /* KvSlice::need_copy_* :57-58 */
int  nova_pool_clear_need_copy(nova_pool* p, int slice);            /* what cow_guard does, model.cpp:176 */
/* No counterpart in the reference.  KvPool::acquire sets the count of every identity page of the slice it
 * hands out to 1 whatever it was (kv_pool.h:100-112).  If a fork still maps pages of a released parent, or
 * cow_slice handed such a page out while the slice was free, the new owner and the old reader would share
 * them unnoticed.  nova_pool_next_slice names the slice the next acquire returns (-1: none);
 * nova_pool_foreign_mappings counts the entries of other live tables that map its identity pages.
 * nova_session_create refuses (NOVA_ERR_BUSY) while that count is not zero. */
int  nova_pool_next_slice(const nova_pool* p);
int  nova_pool_foreign_mappings(const nova_pool* p, int slice);
int  nova_pool_nb_total(const nova_pool* p);
int  nova_pool_nblocks(const nova_pool* p);
int  nova_pool_cow_count(const nova_pool* p);
int  nova_pool_free_blocks(const nova_pool* p);
int  nova_pool_free_slices(const nova_pool* p);
int  nova_pool_used(const nova_pool* p);
int64_t nova_pool_n_past(const nova_pool* p, int slice);
int  nova_pool_set_n_past(nova_pool* p, int slice, int64_t n_past);
/* State dumps for parity diffs; each copies min(cap, size) entries and returns size. */
int  nova_pool_get_table(const nova_pool* p, int slice, int32_t* out, int cap);
int  nova_pool_get_refcnts(const nova_pool* p, int32_t* out, int cap);
int  nova_pool_get_free_list(const nova_pool* p, int32_t* out, int cap);   /* in stack order, back = next */
int  nova_pool_get_free_slices(const nova_pool* p, int32_t* out, int cap);
int  nova_pool_get_live_slices(const nova_pool* p, int32_t* out, int cap); /* ids in slices_ order */

/* ------------------------------------------------------------------ engine */
/* The part of nova::Engine that this path needs (include/nova/model.h:117-179,
 * src/model.cpp:93-96,115-119,171-191): K and V page pools
 * [layer][NB][kv_block][n_kv_heads][head_dim], one block table per slice
 * [n_slices][nblocks] int32, the RoPE cos/sin tables, plus the KvPool and the
 * SessionManager (code/session.h:74-150) that drive them.  The reference fixes
 * the shape at compile time (ModelSpec, include/nova/model/matrix.h:13-53); here
 * it is a runtime descriptor. */
typedef struct nova_engine nova_engine;

typedef struct {
    int32_t n_layers;       /* Model::L                                           */
    int32_t n_heads;        /* Model::NH                                          */
    int32_t n_kv_heads;     /* Model::NKV (NH % NKV == 0)                         */
    int32_t head_dim;       /* Model::HD; 128 only                                */
    int32_t kv_block;       /* kKvBlock = NOVA_KV_BLOCK (code/graph/kv_pool_cfg.h:12-26): 8, 16, 32 or 64 */
    int32_t kv_dtype;       /* NOVA_KV_F32 | NOVA_KV_F16                          */
    int32_t rope_theta;     /* Model::theta (1000000 / 500000 / 10000)            */
    int32_t rope_neox;      /* 1 = pairs (i, i+HD/2) (Qwen2), 0 = (2i, 2i+1)      */
    int32_t n_slices;       /* KvPool::init(n_slices, ctx): slices == max sessions */
    int32_t max_sessions;   /* kMaxSessions: session slots (<= n_slices); 0 = n_slices */
    int64_t ctx;            /* tokens per slice (kMaxCtx)                         */
    int64_t rope_positions; /* rows of the cos/sin tables (kCtx); 0 = ctx         */
    int32_t device;         /* CUDA device ordinal                                */
    int32_t zero_pages;     /* 1 = zero a slice's pages in nova_session_create (session.h:106-118) */
} nova_engine_desc;

int  nova_engine_create(const nova_engine_desc* desc, nova_engine** out);
void nova_engine_destroy(nova_engine* e);
int  nova_engine_desc_get(const nova_engine* e, nova_engine_desc* out);

/* Pool views: Engine::kv_k_base / kv_v_base / kv_table_slot (model.h:135-137),
 * kv_nb / kv_nblocks / kv_width (:140-144), rcs_/rsn_ (model.cpp:115-119). */
void*       nova_kv_k_base(const nova_engine* e);
void*       nova_kv_v_base(const nova_engine* e);
int32_t*    nova_kv_table_slot(const nova_engine* e, int slice);
int         nova_kv_nb(const nova_engine* e);
int         nova_kv_nblocks(const nova_engine* e);
int         nova_kv_width(const nova_engine* e);
size_t      nova_kv_page_bytes(const nova_engine* e);     /* one page of one layer of one pool */
const float* nova_rope_cos(const nova_engine* e);
const float* nova_rope_sin(const nova_engine* e);
nova_pool*  nova_engine_pool(nova_engine* e);             /* the engine's KvPool (kv_pool(), kv_pool.h:199) */

/* SessionManager::create (code/session.h:84-123): lowest free slot, own stream,
 * KvPool::acquire, table upload, page zeroing, stream sync.  Returns the session
 * id (slot) or NOVA_ERR_NO_SESSION / NOVA_ERR_NO_SLICE (the reference exits), or NOVA_ERR_BUSY while
 * the slice that acquire would hand out has pages that another live session still maps (a fork of a
 * destroyed parent, a copy-on-write page): destroy or re-home that session first.  On failure nothing is
 * left allocated.
 * Threading: create and destroy take the engine's lock; every other call that changes the pool (attach,
 * cow, fork, permute, the batch calls) must come from one thread at a time, as in the reference
 * (KvPool is an unsynchronised singleton, kv_pool.h:199). */
int  nova_session_create(nova_engine* e);
int  nova_session_destroy(nova_engine* e, int session);             /* session.h:131-142 */
int  nova_session_live_count(nova_engine* e);                       /* :144 */
int  nova_session_slice(const nova_engine* e, int session);         /* KvSlice::id */
nova_stream_t nova_session_stream(const nova_engine* e, int session); /* Session::ws.s */
int64_t nova_session_n_past(const nova_engine* e, int session);
int  nova_session_set_n_past(nova_engine* e, int session, int64_t n_past);
/* session_attach / session_attach_prefix (session.h:156-163,173-180): host share,
 * whole-table upload on dst's stream, stream sync. */
int  nova_session_attach(nova_engine* e, int dst, int src, int k);
int  nova_session_attach_prefix(nova_engine* e, int dst, int src, int64_t n_tokens);
/* EngineHost::fork (client/src/engine_host.cpp:179-192): a new session that shares ALL of src's cached
 * tokens (session_attach_prefix with n = src's n_past).  Returns the new session id, or an error code
 * (NOVA_ERR_INVALID when src has no tokens, as the reference returns -1). */
int  nova_session_fork(nova_engine* e, int src);
/* Prefix reuse through the block registry (code/graph/kv_registry.h; the reference writes the registry
 * but never consults it, code/INPUT_START.h:35): looks the block {prefix, suffix} up, and when the session
 * that produced it is still alive shares that session's first pos1 tokens with dst
 * (session_attach_prefix).  Returns the number of tokens shared (> 0), 0 when the block is unknown or
 * its session is gone, or an error code. */
int64_t nova_session_attach_block(nova_engine* e, const nova_registry* r, uint64_t prefix, uint64_t suffix, int dst);
/* EngineHost::telemetry (client/src/engine_host.cpp:194-211), the pool part. */
typedef struct nova_telemetry {
    int32_t blocks_total, blocks_free, blocks_shared;   /* shared: refcnt > 1 */
    int32_t cow_count, sessions_live, slices_free;
    uint64_t kv_bytes_cap, kv_bytes_used;               /* both pools, all layers */
} nova_telemetry;
int  nova_engine_telemetry(const nova_engine* e, nova_telemetry* out);
/* session_cow (session.h:166-171) -> Engine::cow_guard (model.cpp:171-191) for every
 * logical block in [pos0, pos0+n): KvPool::cow_slice, then ONE kernel copies the
 * page in all layers of both pools and rewrites the device table entry.  Returns
 * the number of pages copied (>= 0), NOVA_ERR_POOL_FULL where the reference aborts. */
int  nova_session_cow(nova_engine* e, int session, int64_t pos0, int n);
int  nova_session_cow_on(nova_engine* e, int session, int64_t pos0, int n, nova_stream_t s);
/* Harness hook with no counterpart in the reference: re-map a freshly created
 * session's logical blocks onto a permutation of ITS OWN pages
 * (table[b] = slice*nblocks + perm[b]); refcounts are unchanged.  Gives the
 * fragmented block tables that the reference only reaches after COW traffic. */
int  nova_session_permute_pages(nova_engine* e, int session, const int32_t* perm, int n);
/* Re-upload the host table of a session to its device mirror. */
int  nova_session_sync_table(nova_engine* e, int session);

/* ----------------------------------------------------- kernel layer (raw) */
/* Shape of one launch; the reference bakes these into each .cu via Model::. */
typedef struct {
    int32_t n_heads, n_kv_heads, head_dim, kv_block, kv_dtype, rope_neox;
} nova_kv_shape;

/* launch_rope_table (src/kernel/rope.cu:9-18,62-65) for n_pos rows (the
 * reference always builds kCtx = 4096 rows). */
int nova_launch_rope_table(float* cs, float* sn, int64_t n_pos, int32_t head_dim,
                           int32_t theta, nova_stream_t s);

/* launch_rope_batch + launch_kv_store_paged (rope.cu:38-58,67-73; elem.cu:59-76,93-98)
 * fused: rotates q[n][NH][HD] and k[n][NKV][HD] in place at positions pos0..pos0+n-1
 * and scatters the rotated k and v rows into the pools through the block table.
 * q may be NULL (context fill: only k is rotated and k/v stored). */
int nova_launch_rope_append_paged(const nova_kv_shape* sh, void* pool_k, void* pool_v,
                                  const int32_t* table, int layer, int nb, int n, int64_t pos0,
                                  float* q, float* k, const float* v,
                                  const float* cs, const float* sn, nova_stream_t s);

/* launch_attn_decode_paged (src/kernel/attn.cu:197-289,163-191,498-512).
 * scratch: at least nova_attn_scratch_floats(sh) floats (the reference's
 * NH*32*(HD+2), model.cpp:148); split kernel + combine kernel, no other state. */
size_t nova_attn_scratch_floats(const nova_kv_shape* sh);
int nova_launch_attn_decode_paged(const nova_kv_shape* sh, const float* q,
                                  const void* pool_k, const void* pool_v,
                                  const int32_t* table, int layer, int nb, int n_keys,
                                  float* o, float* scratch, nova_stream_t s);

/* No counterpart in the reference.  Which kernel nova_launch_attn_decode_paged runs, process-wide: 0 = SIMT (the
 * default: fp32 arithmetic on the pool's own values), 1 = the tensor-core kernel where it applies (16-token pages,
 * at most 8 query heads per kv head; fp32 pools are rounded to fp16 on their way into the tensor cores, see
 * nova_batch_set_kernel) with the SIMT kernel for everything else.  The launcher keeps one tensor map per pool it
 * has been given (encoded on first use). */
int nova_launcher_set_kernel(int which);

/* No counterpart in the reference.  The same attention as nova_launch_attn_decode_paged for callers
 * that cannot provide scratch memory because they may not allocate on the device at all (an engine
 * whose start-up arena is spoken for and whose operators must not call cudaMalloc, code inside a
 * stream capture, a plug-in host that forbids allocation).  The split-K scratch is a fixed array
 * inside the library's device image; this call performs no cudaMalloc/cudaFree and calls nothing
 * that allocates.
 *   - Limit: n_heads <= nova_attn_static_scratch_max_heads() (64); more returns NOVA_ERR_TOO_LARGE.
 *     The array (1.02 MiB) is held on every GPU that loads the library until the process exits.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 *     that first call outside of any stream capture.
 *   - All calls on a device share the one array: calls whose kernels may overlap on the GPU (other
 *     streams, concurrent host threads) race on it and must be ordered by the caller.  Nothing in
 *     it needs clearing between calls; what a previous call left there is never read. */
size_t nova_attn_static_scratch_max_heads(void);
int nova_launch_attn_decode_paged_static(const nova_kv_shape* sh, const float* q,
                                         const void* pool_k, const void* pool_v,
                                         const int32_t* table, int layer, int nb, int n_keys,
                                         float* o, nova_stream_t s);

/* ------------------------------------------- batched decode over sessions */
/* Engine::decode_batch's hot-path calls (model.cpp:281-289) for any number of
 * sessions in one launch per op.  A batch owns device copies of the sessions'
 * slice ids and write positions, and the scratch of the split-K attention. */
typedef struct nova_batch nova_batch;
int  nova_batch_create(nova_engine* e, const int32_t* sessions, int n, nova_batch** out);
void nova_batch_destroy(nova_batch* b);
int  nova_batch_size(const nova_batch* b);
/* Re-read n_past of every session from the host state into the device array. */
int  nova_batch_sync_positions(nova_batch* b, nova_stream_t s);
/* Select the attention kernel: 0 = SIMT (the default; fp32 arithmetic on the pool's own values), 1 = tensor-core
 * (mma + bulk-copy pipeline).  On fp16 pools 1 applies to every shape and page size.  On fp32 pools - the
 * reference's format - it applies to 16-token pages; the K/V rows are rounded to
 * fp16 in shared memory on their way into the tensor cores (results agree with the exact softmax to about 3e-4
 * relative, values beyond the fp16 range would saturate), the pool itself keeps fp32.  NOVA_ERR_UNSUPPORTED
 * otherwise. */
int  nova_batch_set_kernel(nova_batch* b, int which);
int  nova_batch_get_kernel(const nova_batch* b);
/* For each session s of the batch: session_cow(s, n_past, 1).  One kernel copies
 * all pages that had to be un-shared.  Returns the number of COW copies. */
int  nova_batch_cow(nova_batch* b, nova_stream_t s);
/* RopeKvOp (code/graph/dense.h:75-83) for every session: q [S][NH][HD] and
 * k [S][NKV][HD] rotated in place at n_past[s], k/v appended to the pages. */
int  nova_batch_append(nova_batch* b, int layer, float* q, float* k, const float* v, nova_stream_t s);
/* The same for layers [layer0, layer0 + n_layers) in one launch: q [n][S][NH][HD] (may be NULL: no q to
 * rotate), k/v [n][S][NKV][HD]. */
int  nova_batch_append_layers(nova_batch* b, int layer0, int n_layers, float* q, float* k, const float* v,
                              nova_stream_t s);
/* AttnOp decode branch (dense.h:86-95): n_keys = n_past[s] + 1; out [S][NH][HD]. */
int  nova_batch_attn(nova_batch* b, int layer, const float* q, float* out, nova_stream_t s);
/* RopeKvOp + AttnOp of one layer as one call.  With nova_batch_set_fused_append(b, 1) (tensor-core
 * kernel, NeoX RoPE) both run in ONE launch: the CTA that reads a session's last page rotates k, stores
 * k/v into it and uses them at once; q is rotated in registers and the buffer is left un-rotated.
 * Otherwise it is nova_batch_append followed by nova_batch_attn (q rotated in place).  Callers must
 * not rely on the contents of q afterwards (the reference does not read it after AttnOp either). */
int  nova_batch_set_fused_append(nova_batch* b, int on);
/* Cascade over a shared prefix (kernel 1): when every session of the batch maps its first P logical pages
 * to the same physical pages (sessions forked from one refcounted prefix, code/session.h:173-180) and those
 * pages are full for all of them, a decode step attends these pages ONCE for all sessions (the sessions'
 * queries are the rows of tensor-core tiles), attends each session's own pages as usual, and merges the
 * two by log-sum-exp.  P is re-read from the host tables by every nova_batch_cow (so after a COW or an
 * attach the next step sees the new tables); nova_batch_shared_prefix_pages returns the P in use (0: the
 * plain path).  Results agree with the plain path within the attention tolerance. */
int  nova_batch_set_cascade(nova_batch* b, int on);
int  nova_batch_shared_prefix_pages(const nova_batch* b);
/* Programmatic dependent launch for nova_batch_run_steps / nova_batch_decode_step_host with the fused
 * append: the launches of every layer after the first may start while the previous layer's kernels are
 * still running (consecutive layers overlap on the GPU).  Such a launch streams and processes its pages,
 * appends its layer's new token, and waits (griddepcontrol.wait) only before it writes outputs or
 * partial slots.  Inside these two calls the layer before never produces the next layer's q, k or v and
 * never touches its pages; that is the promise the attribute needs.
 * on = 2: for callers that cannot promise that for q, k and v (an engine computes a layer's q/k/v from the
 * previous layer's attention output): the launches still start early and bring in tables, positions and the
 * first pages, but read q and the new k/v only after the launches before them have finished. */
int  nova_batch_set_pdl(nova_batch* b, int on);
/* Tuning knob of the attention work split: how many pages' worth of time starting a session inside a
 * CTA costs (default 2).  A CTA whose page range crosses a session boundary gets that many fewer pages. */
int  nova_batch_set_row_setup_pages(nova_batch* b, int pages);
/* Tuning knob: CTAs of a tensor-core attention launch (0 = chosen by the library: one per SM, a few fewer in a
 * programmatic chain, half of the SMs when a chained launch has little to stream). */
int  nova_batch_set_split_ctas(nova_batch* b, int n_ctas);
int  nova_batch_append_attn(nova_batch* b, int layer, float* q, float* k, const float* v, float* out,
                            nova_stream_t s);
/* n_past[s] += 1 on host and device (the caller's ++A->n_past, cow_e2e_demo.cpp:64). */
int  nova_batch_advance(nova_batch* b, nova_stream_t s);
/* Prefill (RopeKvOp + AttnOp with n > 1, code/graph/dense.h:75-95; launch_attn_prefill_paged,
 * src/kernel/attn.cu:292-357,514-526): for every session of the batch append n_tokens tokens at
 * n_past.. (k rotated in place, COW guard of the touched pages when layer == 0) and attend causally:
 * query t sees n_past + t + 1 keys.  q/out [S][n_tokens][NH][HD], k/v [S][n_tokens][NKV][HD].
 * n_tokens <= nova_batch_prefill_max_tokens(b) per call; after the last layer call
 * nova_batch_advance_by(b, n_tokens). */
int  nova_batch_prefill_max_tokens(const nova_batch* b);
/* Sliding-window prefill (flash_paged_kernel<true>, src/kernel/attn.cu:317, MaskKind::CausalSWA): a query at
 * position p sees keys (p - window_tokens, p].  0 = plain causal (every model of the reference).  Tensor-core
 * kernel only; nova_batch_prefill returns NOVA_ERR_UNSUPPORTED otherwise. */
int  nova_batch_set_window(nova_batch* b, int window_tokens);
/* Which tensor-core prefill kernel nova_batch_prefill uses: 0 = mma.sync tiles of 64 rows, 1 = tcgen05 tiles of 256
 * rows with the accumulators in tensor memory (fp16 pools, pages of 16 tokens or more; NOVA_ERR_UNSUPPORTED
 * otherwise).  1 is the default: a batch it does not apply to runs the mma.sync tiles.  Both replace
 * flash_paged_kernel (src/kernel/attn.cu:292-357). */
int  nova_batch_set_prefill_kernel(nova_batch* b, int which);
int  nova_batch_prefill(nova_batch* b, int layer, int n_tokens, float* q, float* k, const float* v, float* out,
                        nova_stream_t s);
int  nova_batch_advance_by(nova_batch* b, int n_tokens, nova_stream_t s);
/* All layers at once (inputs of different layers are independent here):
 * q [L][S][NH][HD], k/v [L][S][NKV][HD], out [L][S][NH][HD]; one append launch and
 * one attention launch.  Does not advance. */
int  nova_batch_step_all_layers(nova_batch* b, float* q, float* k, const float* v, float* out,
                                nova_stream_t s);
/* Whole decode step from HOST buffers (layouts as above, pinned or pageable): COW guard, H2D of q/k/v,
 * L x (append, attention), D2H of out, advance.
 * flags bit 0: 1 = one attention launch per layer (engine order), 0 = all layers per launch.
 * flags bit 1: 0 = the call returns when `out` is complete (stream sync); 1 = the call only queues the step and
 *   returns: uploads, kernels and downloads of consecutive steps then overlap (two sets of staging buffers are
 *   used in turn).  The caller keeps q/k/v valid and leaves `out` alone until nova_batch_host_wait() has returned,
 *   and gives every step that is in flight its own `out`. */
int  nova_batch_decode_step_host(nova_batch* b, const float* q, const float* k, const float* v,
                                 float* out, int flags, nova_stream_t s);
/* Blocks until every queued host-buffer step on stream s has delivered its `out`. */
int  nova_batch_host_wait(nova_batch* b, nova_stream_t s);
/* n_steps whole decode steps from DEVICE buffers, issued from native code (no per-launch
 * interpreter cost): per step the COW guard, L x (append, attention) and the advance.
 * Step i reads q + i*q_stride floats (layout [L][S][NH][HD]), k/v + i*kv_stride ([L][S][NKV][HD])
 * and writes out + i*q_stride; a stride of 0 re-uses one buffer set.
 * mode 0: all layers per launch (2 launches + advance per step);
 * mode 1: per-layer launches, the engine's order (2L launches + advance per step);
 * mode 2: as mode 1, captured once into a CUDA graph that is replayed every step on the batch's
 *         fixed staging buffers (inputs are copied in, the result copied out, device to device).
 * attn_ms (may be NULL, modes 0/1): receives the summed CUDA-event time of the attention launches
 * alone; asking for it puts an event pair around each of them. */
int  nova_batch_run_steps(nova_batch* b, int n_steps, float* q, float* k, const float* v, float* out,
                          size_t q_stride, size_t kv_stride, int mode, float* attn_ms, nova_stream_t s);
/* Device status word of the batch (0, or NOVA_ERR_TIMEOUT / NOVA_ERR_BAD_TABLE set by a kernel). */
int  nova_batch_device_status(nova_batch* b);
/* Number of kernels this library has launched since load (all threads). */
uint64_t nova_launch_count(void);

/* Split-K over GPUs for one long session: this rank attends over logical pages
 * [page0, page1) only and leaves un-normalised partials part[S][NH][2+HD] =
 * (m, l, acc) in the reference's layout (attn.cu:150-158).  nova_lse_combine
 * merges n_parts such buffers ([n_parts][S*NH][2+HD], e.g. after an all-gather)
 * in index order with fa_combine_kernel's arithmetic (attn.cu:163-191). */
int  nova_batch_attn_partial(nova_batch* b, int layer, const float* q, int64_t page0, int64_t page1,
                             float* part, nova_stream_t s);
/* The same for layers [layer0, layer0 + n_layers) in one launch: q [n_layers][S][NH][HD],
 * part [n_layers][S][NH][2+HD]. */
int  nova_batch_attn_partial_layers(nova_batch* b, int layer0, int n_layers, const float* q, int64_t page0,
                                    int64_t page1, float* part, nova_stream_t s);
int  nova_lse_combine(const float* parts, int n_parts, int n_rows, int head_dim, float* out,
                      nova_stream_t s);

/* The merge with the exchange folded in (no counterpart in the reference, which scales a long context only
 * inside one GPU).  Every rank owns an exchange buffer of n_slots slots of slot_bytes
 * (>= nova_peer_slot_bytes(n_rows), a multiple of 128), zero-filled once and shared with the other processes of
 * the node through dev_ipc_export / dev_ipc_open.  A rank SENDS its partial rows: the warp that holds a finished
 * row stores it into every peer's buffer (plain stores over NVLink, one way; no multicast), waits - each wait
 * bounded by timeout_ms; on expiry *status (device, may be NULL) becomes NOVA_ERR_TIMEOUT and the row's output is
 * left alone - until the peers' rows have arrived in its own buffer, and merges all ranks' rows in rank order from
 * local memory.  Rows travel as 16-byte words {value, epoch, value, epoch}: a word whose two epoch fields match
 * is complete, so there is no separate flag and no fence.
 * Epochs grow by one per exchange, start at 1 and stay below 2^31; slot = epoch % n_slots and n_slots >= 2 is
 * enough: a rank can be at most one epoch ahead of a peer that is still reading.  peer_base: host array of
 * n_ranks (<= 8) device pointers, entry my_rank being this rank's own buffer.
 *
 * nova_lse_merge_peers: the exchange on its own, called by every rank with the same slot and epoch after the
 * kernels that wrote part [n_rows][2+HD] on stream s; out [n_rows][HD]. */
size_t nova_peer_slot_bytes(int n_rows);
int  nova_lse_merge_peers(const float* part, void* const* peer_base, int n_ranks, int my_rank, size_t slot_bytes, int slot,
                          int n_rows, int64_t epoch, int timeout_ms, float* out, int32_t* status, nova_stream_t s);
/* One whole decode step of the batch's sessions, their pages split over the ranks of a node, issued natively in
 * layer order: per layer the (fused) RoPE+append+attention over this rank's logical pages [page0, page1), then ONE
 * launch that merges the split-K partials of this rank, exchanges the finished rows [S*NH] with the peers in slot
 * (epoch0 + layer) % n_slots and writes out + layer * S*NH*HD; n_past advances at the end.  q/k/v/out are
 * [layers][S][...] as in nova_batch_run_steps.  The caller passes epoch0 = 1, 1 + layers, 1 + 2*layers, ... on every
 * rank.  With the fused append, k is rotated in place only on the rank whose page range holds the new token. */
int  nova_batch_step_partial_peers(nova_batch* b, float* q, float* k, const float* v, int64_t page0, int64_t page1,
                                   void* const* peer_base, int n_ranks, int my_rank, size_t slot_bytes, int n_slots,
                                   int64_t epoch0, int timeout_ms, float* out, int32_t* status, nova_stream_t s);

#ifdef __cplusplus
}
#endif
#endif /* NOVA_B200_H_ */
