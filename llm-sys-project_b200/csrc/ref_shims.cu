// C++ entry points with the reference's own names, signatures and config structs
// (kernels/moe/naive_moe.cuh:9-76, kernels/dsa/naive_dsa.cuh:9-87), so that the
// reference's unmodified tests/ and benchmarks/ drivers link against this library
// instead of naive_moe.cu / naive_dsa.cu.  Each one forwards to the C ABI with the
// per-device default workspace; a non-zero status prints a message and exits, which
// is what the reference's CUDA_CHECK does (utils/cuda_utils.cuh:13-21).
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

struct MoeConfig {     // naive_moe.cuh:9-15
    int num_tokens, num_experts, top_k, hidden_dim, intermediate_dim;
};
struct DsaConfig {     // naive_dsa.cuh:9-17
    int num_queries, num_heads, head_dim_compressed, head_dim_positional, num_selected_kv, page_size,
        total_kv_tokens;
};
using MoEConfig = MoeConfig;
using DSAConfig = DsaConfig;
static_assert(sizeof(MoeConfig) == sizeof(b200_moe_config), "MoeConfig layout");
static_assert(sizeof(DsaConfig) == sizeof(b200_dsa_config), "DsaConfig layout");

#define SHIM_VIS __attribute__((visibility("default")))

static void die_on(int st, const char* what) {
    if (st == B200_OK) return;
    fprintf(stderr, "%s failed: %s (%s)\n", what, b200_status_string(st), b200_last_error_string());
    exit(EXIT_FAILURE);
}
static const b200_moe_config* as_c(const MoeConfig& c) { return reinterpret_cast<const b200_moe_config*>(&c); }
static const b200_dsa_config* as_c(const DsaConfig& c) { return reinterpret_cast<const b200_dsa_config*>(&c); }

// ---- MoE (naive_moe.cuh:27-76) ---------------------------------------------
SHIM_VIS void moe_gate(const float* input, const float* gate_weight, int* expert_indices, float* expert_weights,
                       const MoeConfig& cfg, cudaStream_t stream) {
    die_on(b200_moe_gate_f32(nullptr, input, gate_weight, expert_indices, expert_weights, as_c(cfg), stream),
           "moe_gate");
}
SHIM_VIS void moe_gather(const float* input, const int* expert_indices, const float* /*expert_weights*/,
                         int expert_id, float* gathered, int* token_map, int* count, const MoeConfig& cfg,
                         cudaStream_t stream) {
    die_on(b200_moe_gather_f32(input, expert_indices, expert_id, gathered, token_map, count, as_c(cfg), stream),
           "moe_gather");
}
SHIM_VIS void naive_gemm(const float* A, const float* B, float* C, int M, int N, int K, cudaStream_t stream) {
    die_on(b200_gemm_f32(A, B, C, M, N, K, stream), "naive_gemm");
}
SHIM_VIS void swiglu(const float* gate, const float* up, float* out, int n, cudaStream_t stream) {
    die_on(b200_swiglu_f32(gate, up, out, n, stream), "swiglu");
}
SHIM_VIS void moe_scatter(const float* expert_out, const int* token_map, const float* expert_weights,
                          const int* expert_indices, int expert_id, float* output, int count, const MoeConfig& cfg,
                          cudaStream_t stream) {
    die_on(b200_moe_scatter_f32(expert_out, token_map, expert_weights, expert_indices, expert_id, output, count,
                                as_c(cfg), stream),
           "moe_scatter");
}
SHIM_VIS void moe_forward(const float* input, const float* gate_weight, const float* w1, const float* w2,
                          float* output, const MoeConfig& cfg, cudaStream_t stream) {
    die_on(b200_moe_forward_f32(nullptr, input, gate_weight, w1, w2, output, as_c(cfg), stream), "moe_forward");
}

// ---- DSA (naive_dsa.cuh:31-87) ----------------------------------------------
SHIM_VIS void dsa_kv_gather(const float* kv_cache_compressed, const float* kv_cache_positional, const float* v_cache,
                            const int* sparse_indices, float* gathered_kc, float* gathered_kp, float* gathered_v,
                            const DsaConfig& cfg, cudaStream_t stream) {
    die_on(b200_dsa_kv_gather_f32(kv_cache_compressed, kv_cache_positional, v_cache, sparse_indices, gathered_kc,
                                  gathered_kp, gathered_v, as_c(cfg), stream),
           "dsa_kv_gather");
}
SHIM_VIS void dsa_dot_compressed(const float* q_nope, const float* kc, float* scores, const DsaConfig& cfg,
                                 cudaStream_t stream) {
    die_on(b200_dsa_dot_f32(q_nope, nullptr, kc, nullptr, scores, as_c(cfg), stream), "dsa_dot_compressed");
}
SHIM_VIS void dsa_dot_positional(const float* q_pe, const float* kp, float* scores, const DsaConfig& cfg,
                                 cudaStream_t stream) {
    die_on(b200_dsa_dot_f32(nullptr, q_pe, nullptr, kp, scores, as_c(cfg), stream), "dsa_dot_positional");
}
SHIM_VIS void dsa_dot_fused(const float* q_nope, const float* q_pe, const float* kc, const float* kp, float* scores,
                            const DsaConfig& cfg, cudaStream_t stream) {
    die_on(b200_dsa_dot_f32(q_nope, q_pe, kc, kp, scores, as_c(cfg), stream), "dsa_dot_fused");
}
SHIM_VIS void dsa_softmax(float* scores, const DsaConfig& cfg, cudaStream_t stream) {
    die_on(b200_dsa_softmax_f32(scores, as_c(cfg), stream), "dsa_softmax");
}
SHIM_VIS void dsa_output_proj(const float* attn, const float* v, float* output, const DsaConfig& cfg,
                              cudaStream_t stream) {
    die_on(b200_dsa_output_proj_f32(attn, v, output, as_c(cfg), stream), "dsa_output_proj");
}
SHIM_VIS void dsa_forward(const float* q_nope, const float* q_pe, const float* kv_cache_compressed,
                          const float* kv_cache_positional, const float* v_cache, const int* sparse_indices,
                          float* output, const DsaConfig& cfg, cudaStream_t stream) {
    die_on(b200_dsa_forward_f32(nullptr, q_nope, q_pe, kv_cache_compressed, kv_cache_positional, v_cache,
                                sparse_indices, output, as_c(cfg), stream),
           "dsa_forward");
}
