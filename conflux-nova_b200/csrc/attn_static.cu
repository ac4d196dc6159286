// attn_static.cu — decode attention for callers that may not allocate device memory.
//
// Some hosts of this library cannot hand the attention its split-K scratch: an engine that follows
// the rule "every device byte comes from the one arena carved up at start-up and operators allocate
// nothing" may have no arena bytes left to spare, and code that runs inside a region where cudaMalloc
// is forbidden (a stream capture, a real-time loop, a sandboxed plug-in) cannot get any.  For them
// this file carries the scratch itself: a fixed array in the library's own device image, present on
// every GPU that loads the library from load time until the process ends.
//
// The price: the size is fixed (see kStaticScratchFloats), and the array is SHARED by every call on
// a device.  Two calls whose kernels can overlap on the GPU (different streams, or threads launching
// at once) would write each other's partial results; callers must keep such calls ordered.
#include <cstring>
#include <limits>

#include "common.cuh"

namespace novab {
namespace {

// Room for 64 query heads x 32 partial rows of (head_dim + 2) floats, the reference's own scratch
// formula (src/model.cpp:148) at its largest head count: 1.02 MiB.
constexpr size_t kStaticMaxHeads = 64;
constexpr size_t kStaticScratchFloats = kStaticMaxHeads * 32 * (size_t)(kHeadDim + 2);
static __device__ __align__(256) float g_attn_scratch[kStaticScratchFloats];

// In host code `g_attn_scratch` is only a handle for the symbol, not an address a kernel can use; the
// device address has to be asked for, once per device, with that device current.
// Host threads that make their first call on a device at the same moment may both look the address up;
// they store the same value, and the atomic keeps that well defined.
std::atomic<float*> g_scratch_addr[64];

int static_scratch_for_current_device(float** out) {
    int dev = -1;
    NOVA_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NOVA_ERR_UNSUPPORTED;
    float* addr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!addr) {
        void* p = nullptr;
        NOVA_CUDA_TRY(cudaGetSymbolAddress(&p, g_attn_scratch));
        if (!p) return NOVA_ERR_CUDA;
        addr = static_cast<float*>(p);
        g_scratch_addr[dev].store(addr, std::memory_order_release);
    }
    *out = addr;
    return NOVA_OK;
}

}  // namespace
}  // namespace novab

using namespace novab;

extern "C" {

size_t nova_attn_static_scratch_max_heads(void) { return kStaticMaxHeads; }

int nova_launch_attn_decode_paged_static(const nova_kv_shape* sh, const float* q, const void* pool_k,
                                         const void* pool_v, const int32_t* table, int layer, int nb, int n_keys,
                                         float* o, nova_stream_t s) {
    if (!sh || !q || !pool_k || !pool_v || !table || !o || layer < 0 || nb <= 0) return NOVA_ERR_INVALID;
    if (sh->head_dim != kHeadDim || kv_shift_of_block(sh->kv_block) < 0) return NOVA_ERR_UNSUPPORTED;
    if (sh->n_kv_heads <= 0 || sh->n_heads % sh->n_kv_heads) return NOVA_ERR_INVALID;
    // The one size the fixed array cannot follow: more query heads than it has rows for.
    if ((size_t)sh->n_heads > kStaticMaxHeads) return NOVA_ERR_TOO_LARGE;
    float* scratch = nullptr;
    const int rc0 = static_scratch_for_current_device(&scratch);
    if (rc0 != NOVA_OK) return rc0;

    AttnLaunch a;
    std::memset(&a, 0, sizeof(a));
    a.pool_k = pool_k;
    a.pool_v = pool_v;
    a.kv_shift = kv_shift_of_block(sh->kv_block);
    a.table_base = table;
    a.table_stride = std::numeric_limits<int32_t>::max();
    a.keys_imm = n_keys;
    a.q = q;
    a.out = o;
    a.part = scratch;
    a.n_sessions = 1;
    a.layer0 = layer;
    a.n_layers = 1;
    a.nb = nb;
    a.n_heads = sh->n_heads;
    a.n_kv_heads = sh->n_kv_heads;
    a.kv_group = sh->n_kv_heads < 4 ? sh->n_kv_heads : 4;
    a.page_lo = 0;
    a.page_hi = -1;
    a.row_setup_pages = 1;
    if (a.n_kv_heads % a.kv_group) return NOVA_ERR_UNSUPPORTED;
    // Every partial slot that the merge reads is written by the split kernel of the same call, so
    // nothing in the array has to start at zero and what an earlier call left behind is never read.
    const int heads_per_row = a.kv_group * (sh->n_heads / sh->n_kv_heads);
    const int rows = sh->n_kv_heads / a.kv_group;
    const size_t have = (size_t)sh->n_heads * 32 * (size_t)(kHeadDim + 2);      // floats this shape may use
    int ctas = (int)(have / ((size_t)heads_per_row * kSlotW)) - rows;
    const int want = attn_default_ctas_simt(sh->n_kv_heads);
    if (ctas > want) ctas = want;
    if (ctas < 1) return NOVA_ERR_UNSUPPORTED;
    const int rc = launch_attn_simt(a, sh->kv_dtype, ctas, (cudaStream_t)s);
    if (rc != NOVA_OK) return rc;
    return launch_attn_combine(a, ctas, (cudaStream_t)s);
}

}  // extern "C"
