// Wrapper translation unit around the reference's own tests/test_moe.cu.
// TEST INFRASTRUCTURE ONLY: it compiles the reference's CPU code where it lies
// (path given by -DREF_TEST_MOE=...), renames its main(), and exports the
// file-static CPU reference through a C ABI so fixtures can be generated from
// the reference itself.  No reference source is copied into this repository.
#define main reference_test_moe_main
#include REF_TEST_MOE
#undef main

// The included file's run_test() calls the GPU launcher; the wrapper never
// calls run_test(), so an aborting stub satisfies the linker.
void moe_forward(const float*, const float*, const float*, const float*, float*,
                 const MoeConfig&, cudaStream_t) { abort(); }

extern "C" {
// tests/test_moe.cu:32-140
void ref_cpu_moe_forward(const float* x, const float* wg, const float* w1, const float* w2,
                         int T, int E, int K, int D, int I, int* ids, float* wts, float* out) {
    MoeConfig cfg = {T, E, K, D, I};
    CpuMoeResult r = cpu_moe_forward(x, wg, w1, w2, cfg);
    std::copy(r.expert_indices.begin(), r.expert_indices.end(), ids);
    std::copy(r.expert_weights.begin(), r.expert_weights.end(), wts);
    std::copy(r.output.begin(), r.output.end(), out);
}
// utils/cuda_utils.cuh:56-60
void ref_random_fill(float* data, int n, float lo, float hi) { random_fill(data, n, lo, hi); }
void ref_srand(unsigned s) { srand(s); }
}
