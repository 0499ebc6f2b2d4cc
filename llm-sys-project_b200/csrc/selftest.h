/* Test hooks of the library: exported symbols that only the test suite calls.  They are not part of
 * the public interface (include/b200_moe_dsa.h) and may change without notice. */
#pragma once
#include "../../include/b200_moe_dsa.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Tensor-core self check: D[128,N] = A[128,K] * B[N,K]^T through the same shared-memory
 * descriptors the production kernels use.  mode 0: bf16, both operands K-major;
 * mode 1: bf16, B stored [K,N] (MN-major); mode 2: e4m3 K-major; mode 3: bf16 CTA pair. a/b are raw bits. */
B200_API int b200_umma_selftest(int mode, const void* a, const void* b, float* d, int N, int K,
                                b200_stream_t stream);

/* Runs the give-up branch of the bounded device-side waits: one block, two waiters (a spinning one
 * and a sleeping one) on an mbarrier that nobody signals, compiled with a wait limit of 2 ms.
 * Both return, the block records B200_TIMEOUT in the workspace status word (read it with
 * b200_ws_device_status) and exits normally; nothing traps and no wait is unbounded.
 * elapsed_ns [2] (device, may be NULL): nanoseconds each waiter spent before giving up. */
B200_API int b200_wait_selftest(b200_ws* ws, long long* elapsed_ns, b200_stream_t stream);

/* Measurement hook: dense FP8 (e4m3, fp32 accumulate) tensor rate of this GPU with the MMA shape the
 * grouped GEMMs issue, operands resident in shared memory, one issuing thread per CTA, all SMs busy.
 * pair = 0: cta_group::1, 128 x 256 x 32; pair = 1: cta_group::2, 256 x 256 x 32 per CTA pair.
 * Synchronises the stream (timed with CUDA events inside the call); iters K blocks of four MMAs per CTA. */
B200_API int b200_fp8_mma_rate(int pair, int iters, float* tflops, float* ms, b200_stream_t stream);

/* Block-scaled FP8 MMA self check (kind::mxf8f6f4.block_scale): d[128, N] = sum_k a[m,k] 2^(sfa[m,k/32]-127)
 * b[n,k] 2^(sfb[n,k/32]-127); a [128, K] and b [N, K] e4m3 bytes, sfa [128, K/32] and sfb [N, K/32] UE8M0 bytes,
 * N in {128, 256}, K in {128, 256, 384, 512}. */
B200_API int b200_mx_selftest(const void* a, const void* b, const void* sfa, const void* sfb, float* d, int N, int K,
                              b200_stream_t stream);

/* Work split of the tensor-core router logits kernel, checked on the host (no GPU): 0 when every tile's partial
 * sums get consecutive slots in order of d, cover d once and stay within the bound the scratch is sized with. */
B200_API int b200_tc_plan_selftest(int T, int D, int sms, int chain_blocks, int* max_slots_out);

/* The approximate router logits [T, E] of the tensor-core path, for the test that bounds their distance from the
 * fixed-order FMA chains.  chain_blocks: length of the accumulation chains in 128-deep blocks of d (0 = the
 * library's choice, D / 128 = one chain over all of d).  B200_UNSUPPORTED when the shape does not take that path. */
B200_API int b200_moe_gate_logits_tc(const uint8_t* xq, const float* xs, const float* gate_w, float* logits_out,
                                     int T, int E, int D, int chain_blocks, b200_stream_t stream);
/* Number of tokens the last tensor-core routing call on this workspace handed to its exact pass (synchronises
 * the stream); -1 when the last routing call took the exact path for all tokens. */
B200_API int b200_moe_route_last_flagged(b200_ws* ws, b200_stream_t stream, int* n);

/* Maps every peer of an expert-parallel object onto the object's own exchange buffer, so that a single
 * GPU can run the step of "rank 0 of 2": the words of the absent rank never arrive, the bounded waits run
 * out, and the step reports B200_TIMEOUT (results are meaningless; every access stays inside the buffers). */
B200_API int b200_ep_connect_loopback(b200_ep* ep);
/* Phase timeline of expert-parallel steps (events on the launch stream).  enable != 0 switches it on for the
 * following steps; ms[6], when given and the timeline was on, receives the last step's route + plan, dispatch,
 * wait for the senders, local experts, push and combine times. */
B200_API int b200_ep_phase_profile(b200_ep* ep, int enable, float* ms);

#ifdef __cplusplus
}
#endif
