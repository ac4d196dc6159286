/* paged_decode_oracle.c — TEST INFRASTRUCTURE: a CPU restatement of the reference's
 * paged-KV decode path, used only as the checker in tests/, in the smoke check and
 * as the timed CPU baseline of bench.py.  The product never links or calls it.
 *
 * Parity status: PINNED.  The integer/state part is checked bit-for-bit against the
 * reference's own host code (oracle/ref_host_shim.cpp, built from the reference
 * tree), the attention against outputs of the reference's own decode attention
 * (src/kernel/sycl/attn.cpp run on the CPU through the reference's SYCL stand-in;
 * fixtures under tests/golden/) and, on a GPU box, against the reference's CUDA
 * kernels compiled unmodified for sm_100a (oracle/ref_gpu_shim.cu).
 *
 * Every function names the reference lines it follows.  Build with
 * -ffp-contract=off: all fused multiply-adds are written out.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_KV_F32 0
#define ORACLE_KV_F16 1

typedef struct {
    int32_t n_layers, n_heads, n_kv_heads, head_dim, kv_block, kv_dtype, rope_neox;
} oracle_shape;

/* ---- fp16 <-> fp32, round-to-nearest-even (what __float2half_rn does) ---- */
static inline float h2f(uint16_t h) {
    _Float16 x;
    memcpy(&x, &h, 2);
    return (float)x;
}
static inline uint16_t f2h(float f) {
    _Float16 x = (_Float16)f;
    uint16_t h;
    memcpy(&h, &x, 2);
    return h;
}
uint16_t oracle_f2h(float f) { return f2h(f); }
float oracle_h2f(uint16_t h) { return h2f(h); }

static inline float kv_load(const void* pool, int dtype, int64_t idx) {
    return dtype == ORACLE_KV_F16 ? h2f(((const uint16_t*)pool)[idx]) : ((const float*)pool)[idx];
}
static inline void kv_store(void* pool, int dtype, int64_t idx, float v) {
    if (dtype == ORACLE_KV_F16) ((uint16_t*)pool)[idx] = f2h(v);
    else ((float*)pool)[idx] = v;
}

/* ---- synthetic inputs: counter-based, integer-only, identical on CPU and GPU ----
 * value(key, i) = (sum of twelve 16-bit fields of three 64-bit hashes - 393210) * 2^-16:
 * Irwin-Hall(12), mean 0, variance 1 - 2^-32, support (-6, 6); every step exact in fp32. */
static inline uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
uint64_t oracle_synth_key(uint64_t seed, uint64_t tensor, uint64_t session, uint64_t layer) {
    uint64_t k = mix64(seed);
    k = mix64(k ^ (tensor * 0xD6E8FEB86659FD93ull));
    k = mix64(k ^ (session * 0xA0761D6478BD642Full));
    k = mix64(k ^ (layer * 0xE7037ED1A0B428DBull));
    return k;
}
static inline float synth_value(uint64_t key, uint64_t i) {
    uint32_t sum = 0;
    for (int r = 0; r < 3; ++r) {
        uint64_t h = mix64(key + 3ull * i + (uint64_t)r);
        sum += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) + (uint32_t)((h >> 32) & 0xFFFF) +
               (uint32_t)(h >> 48);
    }
    return (float)((int32_t)sum - 393210) * (1.0f / 65536.0f);
}
void oracle_synth_normal(float* dst, size_t n, uint64_t key, uint64_t first_index) {
    for (size_t i = 0; i < n; ++i) dst[i] = synth_value(key, first_index + i);
}
uint64_t oracle_mix64(uint64_t x) { return mix64(x); }

/* ---- RoPE tables: rope_table_kernel, src/kernel/rope.cu:9-18 ----
 * Same expression; the host libm is not the GPU's, so GPU parity tests hand the
 * GPU-built table to the functions below instead of this one. */
void oracle_rope_table(float* cs, float* sn, int64_t n_pos, int head_dim, int theta) {
    const int half = head_dim / 2;
    for (int64_t pos = 0; pos < n_pos; ++pos)
        for (int i = 0; i < half; ++i) {
            const float f = exp2f(-(float)i * (1.f / (float)half) * log2f((float)theta));
            const float a = (float)pos * f;
            cs[pos * half + i] = cosf(a);
            sn[pos * half + i] = sinf(a);
        }
}

/* ---- RoPE in place: rope_batch_kernel, src/kernel/rope.cu:38-58 ----
 * `x0*c - x1*s` and `x0*s + x1*c` are compiled by nvcc with one multiply fused:
 * fma_mode 1: fma(x0, c, -(x1*s)) and fma(x0, s, x1*c)   (the form nvcc emits)
 * fma_mode 2: fma(-x1, s, x0*c)   and fma(x1, c, x0*s)
 * fma_mode 0: no fusion. */
static inline void rot_pair(float x0, float x1, float c, float s, int fma_mode, float* r0, float* r1) {
    if (fma_mode == 1) {
        *r0 = fmaf(x0, c, -(x1 * s));
        *r1 = fmaf(x0, s, x1 * c);
    } else if (fma_mode == 2) {
        *r0 = fmaf(-x1, s, x0 * c);
        *r1 = fmaf(x1, c, x0 * s);
    } else {
        *r0 = x0 * c - x1 * s;
        *r1 = x0 * s + x1 * c;
    }
}
void oracle_rope_batch(const oracle_shape* sh, float* q, float* k, int n, int64_t pos0, const float* cs,
                       const float* sn, int fma_mode) {
    const int HD = sh->head_dim, half = HD / 2, NH = sh->n_heads, NKV = sh->n_kv_heads;
    for (int t = 0; t < n; ++t) {
        const int64_t pos = pos0 + t;
        for (int head = 0; head < NH + NKV; ++head) {
            float* base = head < NH ? q + ((int64_t)t * NH + head) * HD
                                    : k + ((int64_t)t * NKV + (head - NH)) * HD;
            for (int i = 0; i < half; ++i) {
                const float c = cs[pos * half + i], s = sn[pos * half + i];
                const int a = sh->rope_neox ? i : 2 * i;
                const int b = sh->rope_neox ? i + half : 2 * i + 1;
                float r0, r1;
                rot_pair(base[a], base[b], c, s, fma_mode, &r0, &r1);
                base[a] = r0;
                base[b] = r1;
            }
        }
    }
}

/* ---- append: kv_store_paged_kernel, src/kernel/elem.cu:59-76 ----
 * pool index = ((layer*nb + table[pos>>shift])*KB + (pos & (KB-1))) * NKV*HD + h*HD + d */
void oracle_kv_store_paged(const oracle_shape* sh, void* pool_k, void* pool_v, const int32_t* table,
                           int layer, int nb, int n, int64_t pos0, const float* k, const float* v) {
    const int HD = sh->head_dim, NKV = sh->n_kv_heads, KB = sh->kv_block;
    int shift = 0;
    while ((1 << shift) < KB) ++shift;
    for (int t = 0; t < n; ++t) {
        const int64_t pos = pos0 + t;
        const int phys = table[pos >> shift];
        const int slot = (int)pos & (KB - 1);
        for (int h = 0; h < NKV; ++h)
            for (int d = 0; d < HD; ++d) {
                const int64_t off = (((int64_t)layer * nb + phys) * KB + slot) * (int64_t)NKV * HD + (int64_t)h * HD + d;
                const int64_t src = ((int64_t)t * NKV + h) * HD + d;
                kv_store(pool_k, sh->kv_dtype, off, k[src]);
                kv_store(pool_v, sh->kv_dtype, off, v[src]);
            }
    }
}

/* RopeKvOp, code/graph/dense.h:75-83: rope_batch then kv_store_paged. */
void oracle_rope_append_paged(const oracle_shape* sh, void* pool_k, void* pool_v, const int32_t* table,
                              int layer, int nb, int n, int64_t pos0, float* q, float* k, const float* v,
                              const float* cs, const float* sn, int fma_mode) {
    oracle_rope_batch(sh, q, k, n, pos0, cs, sn, fma_mode);
    oracle_kv_store_paged(sh, pool_k, pool_v, table, layer, nb, n, pos0, k, v);
}

/* ---- copy-on-write device copy: Engine::cow_guard, src/model.cpp:178-188 ---- */
void oracle_cow_copy(const oracle_shape* sh, void* pool_k, void* pool_v, int nb, int src, int dst) {
    const size_t es = sh->kv_dtype == ORACLE_KV_F16 ? 2 : 4;
    const size_t per = (size_t)sh->kv_block * sh->n_kv_heads * sh->head_dim * es;
    for (int l = 0; l < sh->n_layers; ++l) {
        memcpy((char*)pool_k + ((size_t)l * nb + dst) * per, (char*)pool_k + ((size_t)l * nb + src) * per, per);
        memcpy((char*)pool_v + ((size_t)l * nb + dst) * per, (char*)pool_v + ((size_t)l * nb + src) * per, per);
    }
}

/* ---- decode attention, order-faithful ----
 * fa_split_paged_kernel (src/kernel/attn.cu:197-289) + fa_combine_kernel (:163-191) with the
 * split rule of launch_attn_decode_paged (:498-512): same nsplit/chunk/per-warp quarter, same
 * per-lane fma chain, same shuffle-tree order, same merges.  __expf is stood in for by expf.
 * head_dim must be 128 (4 values per lane). */
static float warp_tree_sum(float v[32]) {   /* warp_sum, attn.cu:29-33: result of lane 0 */
    for (int o = 16; o > 0; o >>= 1)
        for (int i = 0; i < o; ++i) v[i] += v[i + o];
    return v[0];
}

static void attn_head_ref_order(const oracle_shape* sh, const float* qh, const void* pool_k, const void* pool_v,
                                const int32_t* table, int layer, int nb, int n_keys, int kvh, float* out,
                                float* part /* [nsplit][HD+2] */) {
    const int HD = sh->head_dim, NKV = sh->n_kv_heads, KB = sh->kv_block;
    const float scale = HD == 64 ? 0.125f : 0.08838834764831845f;   /* attn.cu:21-22 */
    int shift = 0;
    while ((1 << shift) < KB) ++shift;
    int nsplit = (n_keys + 31) / 32;
    if (nsplit > 32) nsplit = 32;
    if (nsplit < 1) nsplit = 1;
    const int chunk = (n_keys + nsplit - 1) / nsplit;
    const int64_t KW = (int64_t)NKV * HD;

    for (int sp = 0; sp < nsplit; ++sp) {
        float wm[4], wl[4], wacc[4][128];
        const int q4 = (chunk + 3) >> 2;
        for (int w = 0; w < 4; ++w) {
            const int kv0 = sp * chunk + w * q4;
            int kv1 = kv0 + q4;
            if (kv1 > n_keys) kv1 = n_keys;
            if (kv1 > (sp + 1) * chunk) kv1 = (sp + 1) * chunk;
            float m = -INFINITY, l = 0.f;
            float* acc = wacc[w];
            for (int d = 0; d < HD; ++d) acc[d] = 0.f;
            for (int p = kv0; p < kv1; ++p) {
                const int phys = table[p >> shift];
                const int slot = p & (KB - 1);
                const int64_t row = (((int64_t)layer * nb + phys) * KB + slot) * KW + (int64_t)kvh * HD;
                float lanes[32];
                for (int lane = 0; lane < 32; ++lane) {
                    float pd = 0.f;
                    for (int c = 0; c < 4; ++c)
                        pd = fmaf(qh[lane + 32 * c], kv_load(pool_k, sh->kv_dtype, row + lane + 32 * c), pd);
                    lanes[lane] = pd;
                }
                const float qk = warp_tree_sum(lanes) * scale;
                const float mn = fmaxf(m, qk);
                const float corr = expf(m - mn);
                const float pr = expf(qk - mn);
                l = fmaf(l, corr, pr);
                for (int d = 0; d < HD; ++d)
                    acc[d] = fmaf(acc[d], corr, pr * kv_load(pool_v, sh->kv_dtype, row + d));
                m = mn;
            }
            wm[w] = m;
            wl[w] = l;
        }
        float mm = -INFINITY;
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wm[w]);
        float ll = 0.f;
        for (int w = 0; w < 4; ++w)
            if (wl[w] > 0.f) ll = fmaf(wl[w], expf(wm[w] - mm), ll);
        float* o = part + (size_t)sp * (HD + 2);
        o[0] = mm;
        o[1] = ll;
        for (int d = 0; d < HD; ++d) {
            float a = 0.f;
            for (int w = 0; w < 4; ++w) a = fmaf(wacc[w][d], expf(wm[w] - mm), a);
            o[2 + d] = a;
        }
    }
    /* fa_combine_kernel */
    float m = -INFINITY;
    for (int s = 0; s < nsplit; ++s) m = fmaxf(m, part[(size_t)s * (HD + 2)]);
    float l = 0.f;
    for (int s = 0; s < nsplit; ++s) {
        const float ms = part[(size_t)s * (HD + 2)], ls = part[(size_t)s * (HD + 2) + 1];
        if (ls > 0.f) l = fmaf(ls, expf(ms - m), l);
    }
    for (int d = 0; d < HD; ++d) {
        float a = 0.f;
        for (int s = 0; s < nsplit; ++s)
            a = fmaf(part[(size_t)s * (HD + 2) + 2 + d], expf(part[(size_t)s * (HD + 2)] - m), a);
        out[d] = l > 0.f ? a / l : 0.f;
    }
}

/* q [NH][HD] -> o [NH][HD]; every head re-reads its KV head, as the reference does. */
void oracle_attn_decode_paged(const oracle_shape* sh, const float* q, const void* pool_k, const void* pool_v,
                              const int32_t* table, int layer, int nb, int n_keys, float* o) {
    const int HD = sh->head_dim, NH = sh->n_heads, G = NH / sh->n_kv_heads;
    float* part = (float*)malloc(sizeof(float) * 32 * (size_t)(HD + 2));
    for (int h = 0; h < NH; ++h)
        attn_head_ref_order(sh, q + (size_t)h * HD, pool_k, pool_v, table, layer, nb, n_keys, h / G,
                            o + (size_t)h * HD, part);
    free(part);
}

/* ---- decode attention, exact: double-precision softmax as in the reference's own numeric
 * check (tests/sycl_bench.cpp:915-938) ---- */
static void attn_head_f64(const oracle_shape* sh, const float* qh, const void* pool_k, const void* pool_v,
                          const int32_t* table, int layer, int nb, int n_keys, int kvh, float* out) {
    const int HD = sh->head_dim, NKV = sh->n_kv_heads, KB = sh->kv_block;
    const float scale = HD == 64 ? 0.125f : 0.08838834764831845f;
    int shift = 0;
    while ((1 << shift) < KB) ++shift;
    double* sc = (double*)malloc(sizeof(double) * (size_t)(n_keys > 0 ? n_keys : 1));
    double* acc = (double*)malloc(sizeof(double) * (size_t)HD);
    double mx = -1e300;
    for (int p = 0; p < n_keys; ++p) {
        const int64_t row = (((int64_t)layer * nb + table[p >> shift]) * KB + (p & (KB - 1))) * (int64_t)NKV * HD + (int64_t)kvh * HD;
        double a = 0.0;
        for (int d = 0; d < HD; ++d) a += (double)qh[d] * (double)kv_load(pool_k, sh->kv_dtype, row + d);
        sc[p] = a * (double)scale;
        if (sc[p] > mx) mx = sc[p];
    }
    double sum = 0.0;
    for (int d = 0; d < HD; ++d) acc[d] = 0.0;
    for (int p = 0; p < n_keys; ++p) {
        const int64_t row = (((int64_t)layer * nb + table[p >> shift]) * KB + (p & (KB - 1))) * (int64_t)NKV * HD + (int64_t)kvh * HD;
        const double w = exp(sc[p] - mx);
        sum += w;
        for (int d = 0; d < HD; ++d) acc[d] += w * (double)kv_load(pool_v, sh->kv_dtype, row + d);
    }
    for (int d = 0; d < HD; ++d) out[d] = n_keys > 0 ? (float)(acc[d] / sum) : 0.f;
    free(sc);
    free(acc);
}

void oracle_attn_decode_paged_f64(const oracle_shape* sh, const float* q, const void* pool_k, const void* pool_v,
                                  const int32_t* table, int layer, int nb, int n_keys, float* o) {
    const int HD = sh->head_dim, NH = sh->n_heads, G = NH / sh->n_kv_heads;
    /* heads are independent: one thread each (long contexts would otherwise take minutes) */
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < NH; ++h)
        attn_head_f64(sh, q + (size_t)h * HD, pool_k, pool_v, table, layer, nb, n_keys, h / G, o + (size_t)h * HD);
}

/* ---- prefill attention, order-faithful: flash_paged_kernel<SWA>, src/kernel/attn.cu:292-357 ----
 * one warp per (head, query): every lane an fma chain over its 4 dims, the shuffle-tree sum, online
 * softmax over keys start..n_past+qi in order, out = acc / l.  q, o: [n_q][NH][HD].
 * window == 0: the causal instantiation (start = 0).  window > 0: the sliding-window one, attn.cu:317,
 * start = max(0, pos - window + 1); the reference fixes the window at kCtx, here it is a parameter. */
void oracle_attn_prefill_paged(const oracle_shape* sh, const float* q, const void* pool_k, const void* pool_v,
                               const int32_t* table, int layer, int nb, int n_q, int n_past, int window, float* o) {
    const int HD = sh->head_dim, NH = sh->n_heads, NKV = sh->n_kv_heads, KB = sh->kv_block, G = NH / NKV;
    const float scale = HD == 64 ? 0.125f : 0.08838834764831845f;
    int shift = 0;
    while ((1 << shift) < KB) ++shift;
    /* every (query, head) pair is one warp of the kernel and independent of the others */
#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int qi = 0; qi < n_q; ++qi)
        for (int h = 0; h < NH; ++h) {
            const int kvh = h / G;
            const float* qp = q + ((size_t)qi * NH + h) * HD;
            float m = -INFINITY, l = 0.f, acc[128];
            for (int d = 0; d < HD; ++d) acc[d] = 0.f;
            const int pos = n_past + qi;
            const int start = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
            for (int p = start; p <= pos; ++p) {
                const int64_t row = (((int64_t)layer * nb + table[p >> shift]) * KB + (p & (KB - 1))) * (int64_t)NKV * HD + (int64_t)kvh * HD;
                float lanes[32];
                for (int lane = 0; lane < 32; ++lane) {
                    float part = 0.f;
                    for (int t = 0; t < HD / 32; ++t)
                        part = fmaf(qp[lane + 32 * t], kv_load(pool_k, sh->kv_dtype, row + lane + 32 * t), part);
                    lanes[lane] = part;
                }
                const float qk = warp_tree_sum(lanes) * scale;
                const float mn = fmaxf(m, qk);
                const float e = expf(m - mn);
                const float pe = expf(qk - mn);
                l = fmaf(l, e, pe);
                for (int d = 0; d < HD; ++d) acc[d] = fmaf(acc[d], e, pe * kv_load(pool_v, sh->kv_dtype, row + d));
                m = mn;
            }
            const float inv = 1.f / l;
            for (int d = 0; d < HD; ++d) o[((size_t)qi * NH + h) * HD + d] = acc[d] * inv;
        }
}

/* Un-normalised partial over logical pages [page0, page1) of one head set, in the reference's
 * partial layout [m, l, acc[HD]] (attn.cu:150-158), accumulated in double, for checking the
 * multi-GPU split; and the LSE merge of fa_combine_kernel (attn.cu:169-190) over such partials. */
void oracle_attn_partial_f64(const oracle_shape* sh, const float* q, const void* pool_k, const void* pool_v,
                             const int32_t* table, int layer, int nb, int n_keys, int64_t page0, int64_t page1,
                             float* part /* [NH][HD+2] */) {
    const int HD = sh->head_dim, NH = sh->n_heads, NKV = sh->n_kv_heads, KB = sh->kv_block, G = NH / NKV;
    const float scale = HD == 64 ? 0.125f : 0.08838834764831845f;
    int shift = 0;
    while ((1 << shift) < KB) ++shift;
    int64_t p0 = page0 * KB, p1 = page1 * KB;
    if (p1 > n_keys) p1 = n_keys;
    double* acc = (double*)malloc(sizeof(double) * (size_t)HD);
    for (int h = 0; h < NH; ++h) {
        const int kvh = h / G;
        double mx = -INFINITY, sum = 0.0;
        for (int d = 0; d < HD; ++d) acc[d] = 0.0;
        for (int64_t p = p0; p < p1; ++p) {
            const int64_t row = (((int64_t)layer * nb + table[p >> shift]) * KB + (p & (KB - 1))) * (int64_t)NKV * HD + (int64_t)kvh * HD;
            double a = 0.0;
            for (int d = 0; d < HD; ++d) a += (double)q[(size_t)h * HD + d] * (double)kv_load(pool_k, sh->kv_dtype, row + d);
            const double s = a * (double)scale;
            if (s > mx) {
                const double c = exp(mx - s);
                sum *= c;
                for (int d = 0; d < HD; ++d) acc[d] *= c;
                mx = s;
            }
            const double w = exp(s - mx);
            sum += w;
            for (int d = 0; d < HD; ++d) acc[d] += w * (double)kv_load(pool_v, sh->kv_dtype, row + d);
        }
        float* o = part + (size_t)h * (HD + 2);
        o[0] = (float)mx;
        o[1] = (float)sum;
        for (int d = 0; d < HD; ++d) o[2 + d] = (float)acc[d];
    }
    free(acc);
}

void oracle_lse_combine(const float* parts /* [n_parts][n_rows][HD+2] */, int n_parts, int n_rows, int head_dim,
                        float* out /* [n_rows][HD] */) {
    const int W = head_dim + 2;
    for (int r = 0; r < n_rows; ++r) {
        float m = -INFINITY;
        for (int s = 0; s < n_parts; ++s) m = fmaxf(m, parts[((size_t)s * n_rows + r) * W]);
        float l = 0.f;
        for (int s = 0; s < n_parts; ++s) {
            const float ms = parts[((size_t)s * n_rows + r) * W], ls = parts[((size_t)s * n_rows + r) * W + 1];
            if (ls > 0.f) l = fmaf(ls, expf(ms - m), l);
        }
        for (int d = 0; d < head_dim; ++d) {
            float a = 0.f;
            for (int s = 0; s < n_parts; ++s) {
                const float ls = parts[((size_t)s * n_rows + r) * W + 1];
                if (ls > 0.f)
                    a = fmaf(parts[((size_t)s * n_rows + r) * W + 2 + d], expf(parts[((size_t)s * n_rows + r) * W] - m), a);
            }
            out[(size_t)r * head_dim + d] = l > 0.f ? a / l : 0.f;
        }
    }
}

/* ---- one decode step over many sessions: the per-session, per-layer call order of
 * Engine::decode_batch (src/model.cpp:281-289) — rope+store, then attention with
 * n_keys = pos+1 — spread over host threads (OpenMP over layer x session).
 * q [L][S][NH][HD] (rotated in place), k [L][S][NKV][HD] (rotated in place), v, out [L][S][NH][HD];
 * tables [S][table_stride]; pos [S].  exact != 0 selects the double-precision attention. */
void oracle_decode_step(const oracle_shape* sh, void* pool_k, void* pool_v, const int32_t* tables,
                        int64_t table_stride, int nb, int n_sessions, const int64_t* pos, float* q, float* k,
                        const float* v, float* out, const float* cs, const float* sn, int fma_mode, int exact,
                        int layer0, int layer1) {
    const int NH = sh->n_heads, NKV = sh->n_kv_heads, HD = sh->head_dim;
    const int64_t S = n_sessions;
    const int G = NH / NKV;
    /* phase 1: rope + store of every (layer, session); phase 2: attention per (layer, session, head) - the heads
     * of the reference's kernel are independent CTAs, so the order inside each head is untouched */
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int l = layer0; l < layer1; ++l)
        for (int s = 0; s < n_sessions; ++s) {
            float* ql = q + ((int64_t)l * S + s) * NH * HD;
            float* kl = k + ((int64_t)l * S + s) * NKV * HD;
            const float* vl = v + ((int64_t)l * S + s) * NKV * HD;
            const int32_t* tb = tables + (int64_t)s * table_stride;
            oracle_rope_append_paged(sh, pool_k, pool_v, tb, l, nb, 1, pos[s], ql, kl, vl, cs, sn, fma_mode);
        }
#pragma omp parallel for collapse(3) schedule(dynamic, 1)
    for (int l = layer0; l < layer1; ++l)
        for (int s = 0; s < n_sessions; ++s)
            for (int h = 0; h < NH; ++h) {
                const float* qh = q + (((int64_t)l * S + s) * NH + h) * HD;
                float* oh = out + (((int64_t)l * S + s) * NH + h) * HD;
                const int32_t* tb = tables + (int64_t)s * table_stride;
                if (exact) {
                    attn_head_f64(sh, qh, pool_k, pool_v, tb, l, nb, (int)pos[s] + 1, h / G, oh);
                } else {
                    float part[32 * (128 + 2)];
                    attn_head_ref_order(sh, qh, pool_k, pool_v, tb, l, nb, (int)pos[s] + 1, h / G, oh, part);
                }
            }
}

/* Thread count of the parallel loops above; oracle_set_num_threads overrides what the environment
 * (OMP_NUM_THREADS) asked for. */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}
