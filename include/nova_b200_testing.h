/* nova_b200_testing.h — aids for tests, benchmarks and profiling builds of libnova_b200.so.
 *
 * Nothing here is on the decode path and nothing here has a counterpart in the reference, which feeds real
 * activations and profiles with its own CUDA-event scopes (code/scope_cuda.h).  The functions are exported
 * by the same shared library as include/nova_b200.h.
 */
#ifndef NOVA_B200_TESTING_H_
#define NOVA_B200_TESTING_H_

#include "nova_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Synthetic inputs: dst[i] = value(key, first_index + i), an integer-only Irwin-Hall(12) approximation of
 * N(0,1) built from 64-bit hashes, bit-identical on host and device (every step is exact in fp32). */
uint64_t nova_synth_key(uint64_t seed, uint64_t tensor, uint64_t session, uint64_t layer);
int nova_synth_normal(float* dst_dev, size_t n, uint64_t key, uint64_t first_index, nova_stream_t s);

/* In-kernel time stamps of the tensor-core attention launches.  Only a library built with -DNOVA_TIMELINE
 * carries them; any other build returns NOVA_ERR_UNSUPPORTED.  dev_buf = 4 records of 148*12 uint64 in device
 * memory (launch i of the batch writes record i % 4), or NULL to switch off.  Every CTA leaves %globaltimer
 * stamps: [0] start, [1] work split known, [2] first page requested, [3] last page requested, [4] first page
 * landed, [5] last page consumed, [6] results written, [7] the SM it ran on (%smid); after those 148*8 values
 * the first 148 CTAs of the merge kernel leave four values each (start, dependency met, %smid, end; the merge +
 * exchange kernel of nova_batch_step_partial_peers leaves "own row ready" in place of %smid).
 * With the cascade on, four more records follow (launch i's shared-prefix tiles write record 4 + i % 4: per CTA start,
 * %smid, end).  The tcgen05 prefill kernel uses the buffer differently (3 x 1700 x 4 uint64, CTAs beyond 1700 leave nothing):
 * [cta][0..3] = start (ns), %smid, end (ns), cycles spent issuing score MMAs; then per CTA the first issuing warp's
 * cycles (total, K wait, P wait, V wait); then the first softmax thread's (total, score wait, P.V wait, tiles). */
int nova_batch_set_timeline(nova_batch* b, void* dev_buf);

/* The literal drop-in launchers (nova_launch_rope_append_paged, nova_launch_attn_decode_paged) for n sessions of one
 * layer in the reference's call order (per session: RopeKvOp then AttnOp, code/graph/dense.h:75-95), issued from
 * one C call: a loop in an interpreter is bound by the interpreter, not by the GPU.  q / k / v / o rows of session i
 * at i * q_stride / i * kv_stride floats; tables[i] = that session's device block table; pos[i] = its n_past. */
int nova_launch_decode_layer_sessions(const nova_kv_shape* sh, int n, void* pool_k, void* pool_v,
                                      const int32_t* const* tables, int layer, int nb, const int64_t* pos,
                                      float* q, float* k, const float* v, size_t q_stride, size_t kv_stride,
                                      const float* cs, const float* sn, float* o, float* scratch, nova_stream_t s);

#ifdef __cplusplus
}
#endif
#endif /* NOVA_B200_TESTING_H_ */
