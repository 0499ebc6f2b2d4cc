// Wrapper translation unit around the reference's own tests/test_dsa.cu.
// TEST INFRASTRUCTURE ONLY: see ref_wrap_moe.cpp.  Path given by -DREF_TEST_DSA=...
#define main reference_test_dsa_main
#include REF_TEST_DSA
#undef main

void dsa_forward(const float*, const float*, const float*, const float*, const float*,
                 const int*, float*, const DsaConfig&, cudaStream_t) { abort(); }

extern "C" {
// tests/test_dsa.cu:23-68
void ref_cpu_dsa_forward(const float* qn, const float* qp, const float* kc, const float* kp,
                         const float* v, const int* idx, float* out,
                         int Q, int H, int Dc, int Dp, int S, int P, int N) {
    DsaConfig cfg = {Q, H, Dc, Dp, S, P, N};
    cpu_dsa_forward(qn, qp, kc, kp, v, idx, out, cfg);
}
// tests/test_dsa.cu:73-85
void ref_gen_sparse_indices(int* indices, int Q, int S, int total_kv) {
    gen_sparse_indices(indices, Q, S, total_kv);
}
void ref_dsa_random_fill(float* data, int n, float lo, float hi) { random_fill(data, n, lo, hi); }
void ref_dsa_srand(unsigned s) { srand(s); }
}
