// Internal launch helpers shared by the MoE translation units.
#pragma once
#include "common.cuh"

// Width of one reduction chunk of the FP8 router's logits (see moe_route.cu).
#define MOE_GATE_CHUNK 1024

void b200_count_launch(int n);

int moe_gate_chunks(int D, bool fp8);
int launch_gate_logits(const void* x, const float* xs, const float* wg, float* partials, int T, int E, int D,
                       bool fp8, cudaStream_t stream);
int launch_route_select(const float* partials, int n_chunks, const float* bias, int* ids, float* wts, int* counts,
                        float* logits_out, int T, int E, int K, int scoring, int n_group, int topk_group,
                        float routed_scale, cudaStream_t stream);
// counts_in: the router's per-expert histogram (may be NULL: counted from ids).  trusted: ids come from
// this library's router (an expert appears at most once per token), so the duplicate check is skipped.
int launch_permute(const int* ids, int T, int K, int E, const int* counts_in, bool trusted, int* counts,
                   int* offsets, int* row_pair, cudaStream_t stream);
int check_route_cfg(int T, int E, int K, int D, int scoring, int n_group, int topk_group);

// b200_moe_fp8_experts without the zero-fill of `out` (the caller keeps the rows that receive
// contributions at zero); used by the expert-parallel owner side.
int b200_moe_fp8_experts_accumulate(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                    const float* expert_w, const uint8_t* w1, const float* w1s, const uint8_t* w2,
                                    const float* w2s, float* out, const b200_moe_fp8_config* cfg, bool packed,
                                    cudaStream_t stream);
