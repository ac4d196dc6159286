// synth.cu — synthetic inputs for tests and benchmarks (declared in include/nova_b200_testing.h).
// Not on the decode path: the reference feeds real activations.  Kept in a translation unit of its own so
// that the product kernels carry none of it.
#include "common.cuh"
#include "../../include/nova_b200_testing.h"

namespace novab {
namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// Integer-only Irwin-Hall(12) "normal": the sum of twelve 16-bit hash fields, centred and
// scaled by 2^-16.  Every step is exact in fp32, so host and device agree bit for bit.
__global__ void synth_normal_kernel(float* __restrict__ dst, size_t n, uint64_t key, uint64_t first) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        uint32_t sum = 0;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const uint64_t h = mix64(key + 3ull * (first + i) + (uint64_t)r);
            sum += (uint32_t)(h & 0xFFFF) + (uint32_t)((h >> 16) & 0xFFFF) + (uint32_t)((h >> 32) & 0xFFFF) +
                   (uint32_t)(h >> 48);
        }
        dst[i] = (float)((int32_t)sum - 393210) * (1.0f / 65536.0f);
    }
}

}  // namespace

int launch_synth_normal(float* dst, size_t n, uint64_t key, uint64_t first_index, cudaStream_t s) {
    if (n == 0) return NOVA_OK;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
    synth_normal_kernel<<<(unsigned)blocks, 256, 0, s>>>(dst, n, key, first_index);
    NOVA_LAUNCH_CHECK();
    return NOVA_OK;
}

}  // namespace novab

using namespace novab;

extern "C" {

uint64_t nova_synth_key(uint64_t seed, uint64_t tensor, uint64_t session, uint64_t layer) {
    auto mix = [](uint64_t x) {
        x += 0x9E3779B97F4A7C15ull;
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        return x ^ (x >> 31);
    };
    uint64_t k = mix(seed);
    k = mix(k ^ (tensor * 0xD6E8FEB86659FD93ull));
    k = mix(k ^ (session * 0xA0761D6478BD642Full));
    k = mix(k ^ (layer * 0xE7037ED1A0B428DBull));
    return k;
}

int nova_synth_normal(float* dst_dev, size_t n, uint64_t key, uint64_t first_index, nova_stream_t s) {
    if (!dst_dev && n) return NOVA_ERR_INVALID;
    return launch_synth_normal(dst_dev, n, key, first_index, (cudaStream_t)s);
}

}  // extern "C"
