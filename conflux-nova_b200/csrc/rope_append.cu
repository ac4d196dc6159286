// rope_append.cu — RoPE tables, fused RoPE + paged append, copy-on-write page copies and
// small page utilities.  Replaces rope_table_kernel / rope_batch_kernel
// (src/kernel/rope.cu:9-18,38-58), kv_store_paged_kernel (src/kernel/elem.cu:59-76) and the
// 2*L cudaMemcpyAsync calls of Engine::cow_guard (src/model.cpp:178-190) of the reference.
//
// Page contents must equal the reference's bit for bit, so this file is compiled WITHOUT
// fast-math and the rotation is written with explicit rounding intrinsics in the fused form
// nvcc gives the reference's `x0*c - x1*s` / `x0*s + x1*c`.
#include "common.cuh"

namespace novab {
namespace {

// Same expression as the reference's table kernel, with theta and HALF compile-time
// constants as they are there, so that the compiler folds exactly the same sub-expressions.
template <int THETA, int HALF>
__global__ void rope_table_kernel(float* __restrict__ cs, float* __restrict__ sn, int64_t n_pos) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_pos * HALF) return;
    const int64_t pos = idx / HALF;
    const int i = (int)(idx - pos * HALF);
    const float f = exp2f(-(float)i * (1.f / (float)HALF) * log2f((float)THETA));
    const float a = (float)pos * f;
    cs[idx] = cosf(a);
    sn[idx] = sinf(a);
}

__global__ void rope_table_any_kernel(float* __restrict__ cs, float* __restrict__ sn, int64_t n_pos,
                                      int half, float theta) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_pos * half) return;
    const int64_t pos = idx / half;
    const int i = (int)(idx - pos * half);
    const float f = exp2f(-(float)i * (1.f / (float)half) * log2f(theta));
    const float a = (float)pos * f;
    cs[idx] = cosf(a);
    sn[idx] = sinf(a);
}

// One 64-thread unit per head: q heads and k heads are rotated in place, k and v rows go to
// their page.  grid = (ceil(units/4), n_tok, layers*S), block = 256.
template <typename KvT>
__global__ void __launch_bounds__(256) rope_append_kernel(AppendLaunch a) {
    constexpr int HD = kHeadDim, HALF = HD / 2;
    const int unit = (int)blockIdx.x * 4 + ((int)threadIdx.x >> 6);
    const int i = (int)threadIdx.x & 63;
    const int NH = a.n_heads, NKV = a.n_kv_heads;
    if (unit >= NH + 2 * NKV) return;
    const int t = (int)blockIdx.y;
    const int ls = (int)blockIdx.z;                 // layer_local * S + s
    const int s = ls % a.n_sessions;
    const int layer = a.layer0 + ls / a.n_sessions;
    const int64_t pos = (a.n_past ? (int64_t)a.n_past[s] : a.pos_imm) + t;
    const int64_t tok = (int64_t)ls * a.n_tok + t;

    const bool is_q = unit < NH;
    if (is_q && !a.q) return;                       // KV-only append (context fill): no q to rotate
    const bool is_k = !is_q && unit < NH + NKV;
    const int kvh = is_q ? 0 : (is_k ? unit - NH : unit - NH - NKV);

    int64_t row = -1;   // element offset of this head's row in the pools
    if (!is_q) {
        const int32_t* table = a.table_base + (int64_t)(a.slice_ids ? a.slice_ids[s] : s) * a.table_stride;
        const int kvs = a.kv_shift ? a.kv_shift : kKvShift;
        const int64_t lb = pos >> kvs;
        int phys = -1;
        if (pos >= 0 && lb < a.table_stride) phys = __ldg(table + lb);
        if (phys < 0 || phys >= a.nb) {
            if (i == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_BAD_TABLE);
        } else {
            const int slot = (int)(pos & ((1 << kvs) - 1));
            row = ((((int64_t)layer * a.nb + phys) << kvs) + slot) * (int64_t)NKV * HD + (int64_t)kvh * HD;
        }
    }

    if (is_q || is_k) {
        if (pos < 0 || pos >= a.rope_rows) {
            if (i == 0 && a.status) atomicCAS(a.status, 0, NOVA_ERR_INVALID);
            return;
        }
        const float c = a.cs[pos * HALF + i];
        const float sn = a.sn[pos * HALF + i];
        float* base = is_q ? a.q + (tok * NH + unit) * HD : a.k + (tok * NKV + kvh) * HD;
        const int ia = a.neox ? i : 2 * i;
        const int ib = a.neox ? i + HALF : 2 * i + 1;
        const float x0 = base[ia];
        const float x1 = base[ib];
        const float r0 = __fmaf_rn(x0, c, -__fmul_rn(x1, sn));
        const float r1 = __fmaf_rn(x0, sn, __fmul_rn(x1, c));
        base[ia] = r0;
        base[ib] = r1;
        if (is_k && row >= 0) {
            KvT* pk = static_cast<KvT*>(a.pool_k) + row;
            KvTraits<KvT>::store(pk + ia, r0);
            KvTraits<KvT>::store(pk + ib, r1);
        }
    } else if (row >= 0) {
        const float* src = a.v + (tok * NKV + kvh) * HD;
        KvT* pv = static_cast<KvT*>(a.pool_v) + row;
        KvTraits<KvT>::store(pv + i, src[i]);
        KvTraits<KvT>::store(pv + i + HALF, src[i + HALF]);
    }
}

constexpr int kCowBatch = 32;
struct CowBatch {
    CowEvent ev[kCowBatch];
};

// grid = (layers, 2 pools, events): one page per block, 16-byte copies.
__global__ void __launch_bounds__(256) cow_copy_kernel(char* __restrict__ pool_k, char* __restrict__ pool_v,
                                                       int nb, size_t page_bytes, CowBatch b) {
    const CowEvent e = b.ev[blockIdx.z];
    char* pool = blockIdx.y ? pool_v : pool_k;
    const size_t layer_base = (size_t)blockIdx.x * (size_t)nb;
    const uint4* src = reinterpret_cast<const uint4*>(pool + (layer_base + (size_t)e.src) * page_bytes);
    uint4* dst = reinterpret_cast<uint4*>(pool + (layer_base + (size_t)e.dst) * page_bytes);
    const int n16 = (int)(page_bytes >> 4);
    for (int i = (int)threadIdx.x; i < n16; i += (int)blockDim.x) dst[i] = src[i];
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && e.table_entry) *e.table_entry = e.dst;
}

// grid = (pages, layers, 2 pools)
__global__ void __launch_bounds__(256) zero_pages_kernel(char* __restrict__ pool_k, char* __restrict__ pool_v,
                                                         int nb, size_t page_bytes,
                                                         const int32_t* __restrict__ table) {
    const int phys = table[blockIdx.x];
    if (phys < 0 || phys >= nb) return;
    char* pool = blockIdx.z ? pool_v : pool_k;
    uint4* dst = reinterpret_cast<uint4*>(pool + ((size_t)blockIdx.y * (size_t)nb + (size_t)phys) * page_bytes);
    const int n16 = (int)(page_bytes >> 4);
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int i = (int)threadIdx.x; i < n16; i += (int)blockDim.x) dst[i] = z;
}

__global__ void advance_kernel(int32_t* n_past, int n, int delta) {
    const int i = (int)(blockIdx.x * blockDim.x + threadIdx.x);
    if (i < n) n_past[i] += delta;
}

}  // namespace

int launch_rope_table(float* cs, float* sn, int64_t n_pos, int theta, cudaStream_t s) {
    if (!cs || !sn || n_pos <= 0) return NOVA_ERR_INVALID;
    constexpr int HALF = kHeadDim / 2;
    const int64_t total = n_pos * HALF;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    switch (theta) {
        case 1000000: rope_table_kernel<1000000, HALF><<<blocks, 256, 0, s>>>(cs, sn, n_pos); break;
        case 500000:  rope_table_kernel<500000, HALF><<<blocks, 256, 0, s>>>(cs, sn, n_pos); break;
        case 10000:   rope_table_kernel<10000, HALF><<<blocks, 256, 0, s>>>(cs, sn, n_pos); break;
        default:      rope_table_any_kernel<<<blocks, 256, 0, s>>>(cs, sn, n_pos, HALF, (float)theta); break;
    }
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

int launch_rope_append(const AppendLaunch& a, cudaStream_t s) {
    if (a.n_sessions <= 0 || a.n_tok <= 0 || a.n_layers <= 0) return NOVA_OK;
    const int units = a.n_heads + 2 * a.n_kv_heads;
    const long long z = (long long)a.n_layers * a.n_sessions;
    if (z > 65535 || a.n_tok > 65535) return NOVA_ERR_TOO_LARGE;
    dim3 grid((unsigned)((units + 3) / 4), (unsigned)a.n_tok, (unsigned)z);
    if (a.kv_dtype == NOVA_KV_F16) rope_append_kernel<__half><<<grid, 256, 0, s>>>(a);
    else if (a.kv_dtype == NOVA_KV_F32) rope_append_kernel<float><<<grid, 256, 0, s>>>(a);
    else return NOVA_ERR_UNSUPPORTED;
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

int launch_cow_copy(void* pool_k, void* pool_v, int n_layers, int nb, size_t page_bytes, const CowEvent* ev,
                    int n_events, cudaStream_t s) {
    for (int done = 0; done < n_events; done += kCowBatch) {
        CowBatch b;
        const int n = (n_events - done < kCowBatch) ? n_events - done : kCowBatch;
        for (int i = 0; i < n; ++i) b.ev[i] = ev[done + i];
        dim3 grid((unsigned)n_layers, 2u, (unsigned)n);
        cow_copy_kernel<<<grid, 256, 0, s>>>((char*)pool_k, (char*)pool_v, nb, page_bytes, b);
        NOVA_LAUNCH_CHECK();
    }
    return NOVA_OK;
}

int launch_zero_pages(void* pool_k, void* pool_v, int n_layers, int nb, size_t page_bytes,
                      const int32_t* table_dev, int n_pages, cudaStream_t s) {
    if (n_pages <= 0) return NOVA_OK;
    for (int p0 = 0; p0 < n_pages; p0 += 32768) {   // grid.x is wide; chunked only for tidy launches
        const int n = (n_pages - p0 < 32768) ? n_pages - p0 : 32768;
        dim3 grid((unsigned)n, (unsigned)n_layers, 2u);
        zero_pages_kernel<<<grid, 256, 0, s>>>((char*)pool_k, (char*)pool_v, nb, page_bytes, table_dev + p0);
        NOVA_LAUNCH_CHECK();
    }
    return NOVA_OK;
}

int launch_advance(int32_t* n_past, int n, cudaStream_t s, int delta) {
    if (n <= 0) return NOVA_OK;
    advance_kernel<<<(n + 127) / 128, 128, 0, s>>>(n_past, n, delta);
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab
