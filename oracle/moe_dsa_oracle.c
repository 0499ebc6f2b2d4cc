/*
 * CPU oracle for the MoE layer and the DSA/MLA sparse decode layer.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests, the
 * smoke test and the benchmark's CPU-baseline leg compare the CUDA library
 * against.  Nothing in the shipped library links, loads or calls it.
 *
 * Parity pinning: the fp32 functions below restate the reference's own CPU
 * code (tests/test_moe.cu, tests/test_dsa.cu) operation by operation and are
 * pinned against outputs of that reference code itself (golden fixtures made
 * by compiling the reference's test files into a wrapper library).  The FP8
 * block-scale, grouped-sigmoid-routing and bf16 functions have no reference
 * counterpart; they extend the same stage order and are pinned against
 * torch.float8_e4m3fn / torch.bfloat16 for the number formats only.
 *
 * Build:  gcc -O2 -std=c11 -fPIC -shared -ffp-contract=off -mfma -fopenmp
 *         (-ffp-contract=off keeps "a*b + c" as two rounded operations, which
 *         is what the reference's x86-64 -O2 build does; explicit fmaf() is
 *         used where a fused operation is part of the definition.)
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* Host threads                                                              */
/* ------------------------------------------------------------------------- */
ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* The reference's input generator: utils/cuda_utils.cuh:56-60 (random_fill), */
/* seeded by srand(42) in tests (tests/test_moe.cu:151) and srand(123) in     */
/* benchmarks (benchmarks/bench_moe.cu:88).  The sequence of rand() calls is  */
/* the seed contract.                                                         */
/* ------------------------------------------------------------------------- */
ORC_API void orc_srand(unsigned seed) { srand(seed); }

ORC_API void orc_rand_fill(float* data, int64_t n, float lo, float hi) {
    for (int64_t i = 0; i < n; i++)
        data[i] = lo + (float)rand() / RAND_MAX * (hi - lo);
}

/* tests/test_dsa.cu:73-85 — partial Fisher-Yates, unique per query, then
 * sorted ascending when `sorted` is non-zero (the reference always sorts). */
static int cmp_int(const void* a, const void* b) {
    int x = *(const int*)a, y = *(const int*)b;
    return (x > y) - (x < y);
}
ORC_API void orc_gen_sparse_indices(int* indices, int Q, int S, int total_kv, int sorted) {
    int* pool = (int*)malloc(sizeof(int) * (size_t)total_kv);
    for (int q = 0; q < Q; q++) {
        for (int i = 0; i < total_kv; i++) pool[i] = i;
        for (int i = 0; i < S; i++) {
            int j = i + rand() % (total_kv - i);
            int t = pool[i]; pool[i] = pool[j]; pool[j] = t;
        }
        if (sorted) qsort(pool, (size_t)S, sizeof(int), cmp_int);
        for (int s = 0; s < S; s++) indices[(size_t)q * S + s] = pool[s];
    }
    free(pool);
}

/* ------------------------------------------------------------------------- */
/* fp32 MoE — tests/test_moe.cu:14-140                                       */
/* ------------------------------------------------------------------------- */

/* tests/test_moe.cu:14-20 */
static void softmax_inplace(float* data, int n) {
    float mx = -FLT_MAX;
    for (int i = 0; i < n; i++) mx = fmaxf(mx, data[i]);
    float s = 0.0f;
    for (int i = 0; i < n; i++) { data[i] = expf(data[i] - mx); s += data[i]; }
    for (int i = 0; i < n; i++) data[i] /= s;
}

/* tests/test_moe.cu:22-24 */
static inline float silu(float x) { return x / (1.0f + expf(-x)); }

/* Routing of the softmax mode: tests/test_moe.cu:39-70 (the device twin is
 * kernels/moe/naive_moe.cu:87-142).  ids/wts come out in replacement-slot
 * order; ties keep the lowest expert id (strict '>' at test_moe.cu:60). */
ORC_API void orc_route_softmax(const float* x, const float* wg, int T, int E, int K, int D,
                               int* ids, float* wts) {
    float* logits = (float*)malloc(sizeof(float) * (size_t)E);
    for (int t = 0; t < T; t++) {
        for (int e = 0; e < E; e++) {
            float sum = 0.0f;
            for (int d = 0; d < D; d++)
                sum += x[(size_t)t * D + d] * wg[(size_t)e * D + d];
            logits[e] = sum;
        }
        softmax_inplace(logits, E);
        int* oi = ids + (size_t)t * K;
        float* ow = wts + (size_t)t * K;
        for (int k = 0; k < K; k++) { oi[k] = -1; ow[k] = -FLT_MAX; }
        for (int e = 0; e < E; e++) {
            float v = logits[e];
            int min_k = 0;
            for (int k = 1; k < K; k++)
                if (ow[k] < ow[min_k]) min_k = k;
            if (v > ow[min_k]) { ow[min_k] = v; oi[min_k] = e; }
        }
        float s = 0.0f;
        for (int k = 0; k < K; k++) s += ow[k];
        if (s > 0.0f) for (int k = 0; k < K; k++) ow[k] /= s;
    }
    free(logits);
}

/* Canonical permutation: experts ascending, tokens ascending inside an expert
 * (the order kernels/moe/naive_moe.cu:153-163 and tests/test_moe.cu:76-81
 * produce, a token counted once per expert).  row_pair[r] = t*K + k of the
 * (token, slot) pair that sorted row r holds; offsets[e] is the exclusive
 * prefix sum of counts. */
ORC_API void orc_permute(const int* ids, int T, int K, int E,
                         int* counts, int* offsets, int* row_pair) {
    int r = 0;
    for (int e = 0; e < E; e++) {
        offsets[e] = r;
        for (int t = 0; t < T; t++) {
            for (int k = 0; k < K; k++) {
                if (ids[(size_t)t * K + k] == e) { row_pair[r++] = t * K + k; break; }
            }
        }
        counts[e] = r - offsets[e];
    }
    offsets[E] = r;
}

/* Expert FFN + combine of tests/test_moe.cu:72-133 for given routing. */
static void moe_experts_f32(const float* x, const float* w1, const float* w2,
                            const int* ids, const float* wts,
                            int T, int E, int K, int D, int I, float* out) {
    memset(out, 0, sizeof(float) * (size_t)T * D);
    int* tmap = (int*)malloc(sizeof(int) * (size_t)T);
    float* g1 = (float*)malloc(sizeof(float) * (size_t)T * 2 * I);
    float* act = (float*)malloc(sizeof(float) * (size_t)T * I);
    float* g2 = (float*)malloc(sizeof(float) * (size_t)T * D);
    for (int e = 0; e < E; e++) {
        int cnt = 0;
        for (int t = 0; t < T; t++)
            for (int k = 0; k < K; k++)
                if (ids[(size_t)t * K + k] == e) { tmap[cnt++] = t; break; }
        if (cnt == 0) continue;
        const float* w1e = w1 + (size_t)e * 2 * I * D;
        const float* w2e = w2 + (size_t)e * D * I;
        for (int m = 0; m < cnt; m++) {
            int t = tmap[m];
            for (int n = 0; n < 2 * I; n++) {
                float sum = 0.0f;
                for (int d = 0; d < D; d++)
                    sum += x[(size_t)t * D + d] * w1e[(size_t)n * D + d];
                g1[(size_t)m * 2 * I + n] = sum;
            }
        }
        for (int m = 0; m < cnt; m++)
            for (int j = 0; j < I; j++) {
                float g = g1[(size_t)m * 2 * I + j];
                float u = g1[(size_t)m * 2 * I + I + j];
                act[(size_t)m * I + j] = silu(g) * u;
            }
        for (int m = 0; m < cnt; m++)
            for (int n = 0; n < D; n++) {
                float sum = 0.0f;
                for (int j = 0; j < I; j++)
                    sum += act[(size_t)m * I + j] * w2e[(size_t)n * I + j];
                g2[(size_t)m * D + n] = sum;
            }
        for (int m = 0; m < cnt; m++) {
            int t = tmap[m];
            float w = 0.0f;
            for (int k = 0; k < K; k++)
                if (ids[(size_t)t * K + k] == e) { w = wts[(size_t)t * K + k]; break; }
            for (int d = 0; d < D; d++)
                out[(size_t)t * D + d] += w * g2[(size_t)m * D + d];
        }
    }
    free(tmap); free(g1); free(act); free(g2);
}

/* Whole layer, tests/test_moe.cu:32-140 (cpu_moe_forward). */
ORC_API void orc_moe_forward_f32(const float* x, const float* wg, const float* w1, const float* w2,
                                 int T, int E, int K, int D, int I,
                                 int* ids, float* wts, float* out) {
    orc_route_softmax(x, wg, T, E, K, D, ids, wts);
    moe_experts_f32(x, w1, w2, ids, wts, T, E, K, D, I, out);
}

/* ------------------------------------------------------------------------- */
/* FP8 e4m3 (finite-only "fn" flavour: max 448, no inf, 0x7f/0xff = NaN)     */
/* ------------------------------------------------------------------------- */
ORC_API float orc_e4m3_decode(uint8_t b) {
    int s = b >> 7, e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);            /* subnormal: m * 2^-3 * 2^-6 */
    else        v = ldexpf((float)(8 + m), e - 10);  /* (1 + m/8) * 2^(e-7)        */
    return s ? -v : v;
}

/* Round to nearest even, saturate to +-448 (what cvt.rn.satfinite.e4m3x2.f32 does). */
ORC_API uint8_t orc_e4m3_encode(float f) {
    uint8_t sign = signbit(f) ? 0x80 : 0;
    if (isnan(f)) return (uint8_t)(sign | 0x7f);
    float a = fabsf(f);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7e);
    if (a < 0.015625f) {                 /* below 2^-6: subnormal grid of 2^-9 */
        float q = nearbyintf(a * 512.0f);            /* exact scaling; ties-to-even */
        return (uint8_t)(sign | (uint8_t)q);         /* q == 8 encodes 2^-6 correctly */
    }
    int ex;
    float fr = frexpf(a, &ex);           /* a = fr * 2^ex, fr in [0.5,1) */
    float q = nearbyintf(fr * 16.0f);    /* 8..16 */
    if (q == 16.0f) { q = 8.0f; ex += 1; }
    int e = ex - 1 + 7;
    int m = (int)q - 8;
    if (e > 15 || (e == 15 && m > 6)) return (uint8_t)(sign | 0x7e);
    return (uint8_t)(sign | (e << 3) | m);
}

ORC_API void orc_e4m3_decode_n(const uint8_t* b, float* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_e4m3_decode(b[i]);
}
ORC_API void orc_e4m3_encode_n(const float* f, uint8_t* out, int64_t n) {
    for (int64_t i = 0; i < n; i++) out[i] = orc_e4m3_encode(f[i]);
}

/* bf16 <-> fp32 (round to nearest even; NaN kept quiet) */
ORC_API uint16_t orc_bf16_encode(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
ORC_API float orc_bf16_decode(uint16_t h) {
    uint32_t u = (uint32_t)h << 16; float f; memcpy(&f, &u, 4); return f;
}

/* Block scale rule shared by both quantisers: scale = amax/448, or 1 for an
 * all-zero block; q = e4m3(x / scale). */
static int g_pow2_scales = 0;
/* Power-of-two scale rule (the UE8M0 scale format; no reference counterpart): the smallest power of two
 * >= amax/448, at least 2^-126, at most 2^127.  Applies to both quantisers and to the requantisation inside the
 * FP8 expert emulation while switched on. */
ORC_API void orc_set_pow2_scales(int on) { g_pow2_scales = on; }
static inline float pow2_ceil(float q) {
    uint32_t u; memcpy(&u, &q, 4);
    uint32_t e = (u >> 23) & 0xFFu;
    if (e == 0) e = 1;
    else if (u & 0x7FFFFFu) e += 1;
    if (e > 254) e = 254;
    u = e << 23;
    float f; memcpy(&f, &u, 4); return f;
}
static inline float block_scale(float amax) {
    if (!(amax > 0.0f)) return 1.0f;
    float q = amax / 448.0f;
    return g_pow2_scales ? pow2_ceil(q) : q;
}

/* Activations: one fp32 scale per 1x128 block of a row.  cols % 128 == 0. */
ORC_API void orc_quant_act_1x128(const float* x, int64_t rows, int cols, uint8_t* q, float* scales) {
    int nb = cols / 128;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; r++)
        for (int b = 0; b < nb; b++) {
            const float* p = x + r * cols + (int64_t)b * 128;
            float amax = 0.0f;
            for (int i = 0; i < 128; i++) amax = fmaxf(amax, fabsf(p[i]));
            float s = block_scale(amax);
            scales[r * nb + b] = s;
            for (int i = 0; i < 128; i++) q[r * cols + (int64_t)b * 128 + i] = orc_e4m3_encode(p[i] / s);
        }
}

/* Weights: one fp32 scale per 128x128 block.  rows % 128 == 0, cols % 128 == 0.
 * scales is [rows/128, cols/128] row-major. */
ORC_API void orc_quant_weight_128x128(const float* w, int64_t rows, int cols, uint8_t* q, float* scales) {
    int64_t rb = rows / 128; int cb = cols / 128;
    #pragma omp parallel for schedule(static)
    for (int64_t br = 0; br < rb; br++)
        for (int bc = 0; bc < cb; bc++) {
            float amax = 0.0f;
            for (int i = 0; i < 128; i++)
                for (int j = 0; j < 128; j++)
                    amax = fmaxf(amax, fabsf(w[(br * 128 + i) * cols + bc * 128 + j]));
            float s = block_scale(amax);
            scales[br * cb + bc] = s;
            for (int i = 0; i < 128; i++)
                for (int j = 0; j < 128; j++) {
                    int64_t o = (br * 128 + i) * cols + bc * 128 + j;
                    q[o] = orc_e4m3_encode(w[o] / s);
                }
        }
}

/* ------------------------------------------------------------------------- */
/* Grouped sigmoid routing (DeepSeek-V3 style; no reference counterpart —    */
/* it extends the top-K of tests/test_moe.cu:50-69 with the same "lowest     */
/* index wins a tie" rule).                                                  */
/*   logit[e] = sum, in order, of the partial sums of 1024-wide chunks of d; */
/*              each partial is an fma chain from 0 over xdeq[d] * wg[e,d],  */
/*              xdeq = e4m3(xq) * xs (the fixed order makes it reproducible) */
/*   s[e]     = (float)(1 / (1 + exp(-(double)logit[e])))                    */
/*   c[e]     = s[e] + bias[e]                                               */
/*   group score = largest + second largest c in the group (E/n_group each)  */
/*   keep topk_group groups (max first, ties -> lowest group)                */
/*   pick K experts among kept groups by c (max first, ties -> lowest id)    */
/*   w[k] = s[id_k] / (sum over slots in order) * routed_scale               */
/* Slot order is rank order (best first).                                    */
/* ------------------------------------------------------------------------- */
#define ORC_GATE_CHUNK 1024
ORC_API void orc_gate_logits_fp8(const uint8_t* xq, const float* xs, const float* wg,
                                 int T, int E, int D, float* logits) {
    int nb = D / 128;
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = orc_e4m3_decode((uint8_t)i);
    #pragma omp parallel
    {
        float* xd = (float*)malloc(sizeof(float) * (size_t)D);
        #pragma omp for schedule(static)
        for (int t = 0; t < T; t++) {
            for (int d = 0; d < D; d++)
                xd[d] = lut[xq[(size_t)t * D + d]] * xs[(size_t)t * nb + d / 128];
            for (int e = 0; e < E; e++) {
                const float* w = wg + (size_t)e * D;
                float total = 0.0f;
                for (int d0 = 0; d0 < D; d0 += ORC_GATE_CHUNK) {
                    int d1 = d0 + ORC_GATE_CHUNK < D ? d0 + ORC_GATE_CHUNK : D;
                    float acc = 0.0f;
                    for (int d = d0; d < d1; d++) acc = fmaf(xd[d], w[d], acc);
                    total = (d0 == 0) ? acc : total + acc;
                }
                logits[(size_t)t * E + e] = total;
            }
        }
        free(xd);
    }
}

ORC_API void orc_route_grouped_from_logits(const float* logits, const float* bias,
                                           int T, int E, int K, int n_group, int topk_group,
                                           float routed_scale, int* ids, float* wts) {
    int gs = E / n_group;
    #pragma omp parallel
    {
        float* s = (float*)malloc(sizeof(float) * (size_t)E);
        float* c = (float*)malloc(sizeof(float) * (size_t)E);
        float* gscore = (float*)malloc(sizeof(float) * (size_t)n_group);
        char* gkeep = (char*)malloc((size_t)n_group);
        char* taken = (char*)malloc((size_t)E);
        #pragma omp for schedule(static)
        for (int t = 0; t < T; t++) {
            for (int e = 0; e < E; e++) {
                float l = logits[(size_t)t * E + e];
                s[e] = (float)(1.0 / (1.0 + exp(-(double)l)));
                c[e] = s[e] + (bias ? bias[e] : 0.0f);
            }
            for (int g = 0; g < n_group; g++) {
                float m1 = -FLT_MAX, m2 = -FLT_MAX; int i1 = -1;
                for (int j = 0; j < gs; j++) if (c[g * gs + j] > m1) { m1 = c[g * gs + j]; i1 = j; }
                for (int j = 0; j < gs; j++) if (j != i1 && c[g * gs + j] > m2) m2 = c[g * gs + j];
                gscore[g] = (gs > 1) ? m1 + m2 : m1;
                gkeep[g] = 0;
            }
            for (int r = 0; r < topk_group; r++) {
                int best = -1; float bv = 0.0f;
                for (int g = 0; g < n_group; g++)
                    if (!gkeep[g] && (best < 0 || gscore[g] > bv)) { best = g; bv = gscore[g]; }
                gkeep[best] = 1;
            }
            memset(taken, 0, (size_t)E);
            float sum = 0.0f;
            for (int k = 0; k < K; k++) {
                int best = -1; float bv = 0.0f;
                for (int e = 0; e < E; e++)
                    if (gkeep[e / gs] && !taken[e] && (best < 0 || c[e] > bv)) { best = e; bv = c[e]; }
                taken[best] = 1;
                ids[(size_t)t * K + k] = best;
                wts[(size_t)t * K + k] = s[best];
                sum += s[best];
            }
            for (int k = 0; k < K; k++)
                wts[(size_t)t * K + k] = wts[(size_t)t * K + k] / sum * routed_scale;
        }
        free(s); free(c); free(gscore); free(gkeep); free(taken);
    }
}

ORC_API void orc_route_grouped(const uint8_t* xq, const float* xs, const float* wg, const float* bias,
                               int T, int E, int K, int D, int n_group, int topk_group,
                               float routed_scale, int* ids, float* wts) {
    float* logits = (float*)malloc(sizeof(float) * (size_t)T * E);
    orc_gate_logits_fp8(xq, xs, wg, T, E, D, logits);
    orc_route_grouped_from_logits(logits, bias, T, E, K, n_group, topk_group, routed_scale, ids, wts);
    free(logits);
}

/* ------------------------------------------------------------------------- */
/* FP8 block-scale expert FFN emulation in fp32 (stage order of              */
/* tests/test_moe.cu:74-133): per 128-deep K block the e4m3 products are     */
/* summed in fp32 and promoted with a_scale*w_scale; SwiGLU; the activation  */
/* is requantised per 1x128 with a fresh scale; second GEMM likewise; times  */
/* the router weight; summed over the token's experts in ascending order.    */
/* Evaluated for the listed tokens only: out_rows[i,:] is the layer output   */
/* of token tokens[i].  w1q [E,2I,D], w1s [E,2I/128,D/128], w2q [E,D,I],      */
/* w2s [E,D/128,I/128].  Optionally returns the requantised activations of   */
/* the first listed token's first (lowest-id) expert for stage checks.       */
/* ------------------------------------------------------------------------- */
static inline float dot128(const float* a, const float* b) {
    float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < 128; i += 8)
        for (int j = 0; j < 8; j++) s[j] += a[i + j] * b[i + j];
    return ((s[0] + s[1]) + (s[2] + s[3])) + ((s[4] + s[5]) + (s[6] + s[7]));
}

ORC_API void orc_moe_fp8_experts(const uint8_t* xq, const float* xs,
                                 const uint8_t* w1q, const float* w1s,
                                 const uint8_t* w2q, const float* w2s,
                                 const int* ids, const float* wts,
                                 int T, int E, int K, int D, int I,
                                 const int* tokens, int n_tokens, float* out_rows) {
    (void)T; (void)E;
    int nbD = D / 128, nbI = I / 128;
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = orc_e4m3_decode((uint8_t)i);
    memset(out_rows, 0, sizeof(float) * (size_t)n_tokens * D);
    #pragma omp parallel
    {
        float* xd = (float*)malloc(sizeof(float) * (size_t)D);
        float* g1 = (float*)malloc(sizeof(float) * (size_t)2 * I);
        float* act = (float*)malloc(sizeof(float) * (size_t)I);
        float* actd = (float*)malloc(sizeof(float) * (size_t)I);
        float* acts = (float*)malloc(sizeof(float) * (size_t)nbI);
        float* wrow = (float*)malloc(sizeof(float) * (size_t)(D > I ? D : I));
        int* order = (int*)malloc(sizeof(int) * (size_t)K);
        #pragma omp for schedule(dynamic, 1)
        for (int it = 0; it < n_tokens; it++) {
            int t = tokens[it];
            float* out = out_rows + (size_t)it * D;
            for (int d = 0; d < D; d++) xd[d] = lut[xq[(size_t)t * D + d]];
            /* experts ascending (the reference's accumulation order, test_moe.cu:74) */
            for (int k = 0; k < K; k++) order[k] = k;
            for (int a = 1; a < K; a++) {
                int v = order[a], b = a - 1;
                while (b >= 0 && ids[(size_t)t * K + order[b]] > ids[(size_t)t * K + v]) { order[b + 1] = order[b]; b--; }
                order[b + 1] = v;
            }
            for (int kk = 0; kk < K; kk++) {
                int k = order[kk];
                int e = ids[(size_t)t * K + k];
                if (e < 0) continue;
                float w = wts[(size_t)t * K + k];
                const uint8_t* w1e = w1q + (size_t)e * 2 * I * D;
                const float* w1se = w1s + (size_t)e * (2 * I / 128) * nbD;
                const uint8_t* w2e = w2q + (size_t)e * D * I;
                const float* w2se = w2s + (size_t)e * (D / 128) * nbI;
                for (int n = 0; n < 2 * I; n++) {
                    const uint8_t* wr = w1e + (size_t)n * D;
                    for (int d = 0; d < D; d++) wrow[d] = lut[wr[d]];
                    float acc = 0.0f;
                    for (int kb = 0; kb < nbD; kb++) {
                        float part = dot128(xd + kb * 128, wrow + kb * 128);
                        float sc = xs[(size_t)t * nbD + kb] * w1se[(size_t)(n / 128) * nbD + kb];
                        acc += part * sc;
                    }
                    g1[n] = acc;
                }
                for (int j = 0; j < I; j++) act[j] = silu(g1[j]) * g1[I + j];
                for (int b = 0; b < nbI; b++) {
                    float amax = 0.0f;
                    for (int i = 0; i < 128; i++) amax = fmaxf(amax, fabsf(act[b * 128 + i]));
                    float s = block_scale(amax);
                    acts[b] = s;
                    for (int i = 0; i < 128; i++) actd[b * 128 + i] = lut[orc_e4m3_encode(act[b * 128 + i] / s)];
                }
                for (int n = 0; n < D; n++) {
                    const uint8_t* wr = w2e + (size_t)n * I;
                    for (int j = 0; j < I; j++) wrow[j] = lut[wr[j]];
                    float acc = 0.0f;
                    for (int kb = 0; kb < nbI; kb++) {
                        float part = dot128(actd + kb * 128, wrow + kb * 128);
                        float sc = acts[kb] * w2se[(size_t)(n / 128) * nbI + kb];
                        acc += part * sc;
                    }
                    out[n] += w * acc;
                }
            }
        }
        free(xd); free(g1); free(act); free(actd); free(acts); free(wrow); free(order);
    }
}

/* Stage check helper: GEMM1 + SwiGLU + requantise for one (token, expert)
 * pair; returns the e4m3 bytes [I] and the scales [I/128]. */
ORC_API void orc_moe_fp8_gemm1_row(const uint8_t* xq_row, const float* xs_row,
                                   const uint8_t* w1e, const float* w1se,
                                   int D, int I, uint8_t* act_q, float* act_s) {
    int nbD = D / 128, nbI = I / 128;
    float lut[256];
    for (int i = 0; i < 256; i++) lut[i] = orc_e4m3_decode((uint8_t)i);
    float* xd = (float*)malloc(sizeof(float) * (size_t)D);
    float* wrow = (float*)malloc(sizeof(float) * (size_t)D);
    float* g1 = (float*)malloc(sizeof(float) * (size_t)2 * I);
    for (int d = 0; d < D; d++) xd[d] = lut[xq_row[d]];
    for (int n = 0; n < 2 * I; n++) {
        for (int d = 0; d < D; d++) wrow[d] = lut[w1e[(size_t)n * D + d]];
        float acc = 0.0f;
        for (int kb = 0; kb < nbD; kb++)
            acc += dot128(xd + kb * 128, wrow + kb * 128) * (xs_row[kb] * w1se[(size_t)(n / 128) * nbD + kb]);
        g1[n] = acc;
    }
    for (int b = 0; b < nbI; b++) {
        float a[128]; float amax = 0.0f;
        for (int i = 0; i < 128; i++) { a[i] = silu(g1[b * 128 + i]) * g1[I + b * 128 + i]; amax = fmaxf(amax, fabsf(a[i])); }
        float s = block_scale(amax);
        act_s[b] = s;
        for (int i = 0; i < 128; i++) act_q[b * 128 + i] = orc_e4m3_encode(a[i] / s);
    }
    free(xd); free(wrow); free(g1);
}

/* ------------------------------------------------------------------------- */
/* DSA / MLA sparse decode — tests/test_dsa.cu:14-68 (cpu_dsa_forward).      */
/* Indices are flat physical token ids; every listed index contributes       */
/* (duplicates twice), order is free.  64-bit offsets (the reference's int   */
/* math overflows once N*Dc reaches 2^31).  Queries run in parallel threads; */
/* each (q,h) is computed exactly as the reference does.                     */
/* ------------------------------------------------------------------------- */
ORC_API void orc_dsa_forward_f32(const float* q_nope, const float* q_pe,
                                 const float* kc, const float* kp, const float* v,
                                 const int* idx, float* out,
                                 int Q, int H, int Dc, int Dp, int S) {
    float scale = 1.0f / sqrtf((float)(Dc + Dp));
    #pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int q = 0; q < Q; q++) {
        for (int h = 0; h < H; h++) {
            float* scores = (float*)malloc(sizeof(float) * (size_t)S);
            const float* qn = q_nope + ((size_t)q * H + h) * Dc;
            const float* qp = q_pe + ((size_t)q * H + h) * Dp;
            for (int s = 0; s < S; s++) {
                int64_t id = idx[(size_t)q * S + s];
                const float* kcr = kc + id * Dc;
                const float* kpr = kp + id * Dp;
                float sum_c = 0.0f, sum_p = 0.0f;
                for (int d = 0; d < Dc; d++) sum_c += qn[d] * kcr[d];
                for (int d = 0; d < Dp; d++) sum_p += qp[d] * kpr[d];
                scores[s] = (sum_c + sum_p) * scale;
            }
            softmax_inplace(scores, S);
            float* o = out + ((size_t)q * H + h) * Dc;
            for (int d = 0; d < Dc; d++) {
                float sum = 0.0f;
                for (int s = 0; s < S; s++) {
                    int64_t id = idx[(size_t)q * S + s];
                    sum += scores[s] * v[id * Dc + d];
                }
                o[d] = sum;
            }
            free(scores);
        }
    }
}

/* bf16 inputs (raw bits), fp32 arithmetic: widen, then the fp32 routine on
 * the selected rows only (the cache can be far larger than host memory
 * wants to hold as fp32).  Row-gathers through idx into compact buffers and
 * rewrites the indices. */
ORC_API void orc_dsa_forward_bf16(const uint16_t* q_nope, const uint16_t* q_pe,
                                  const uint16_t* kc, const uint16_t* kp, const uint16_t* v,
                                  const int* idx, float* out,
                                  int Q, int H, int Dc, int Dp, int S) {
    size_t nq = (size_t)Q * H;
    float* qn = (float*)malloc(sizeof(float) * nq * Dc);
    float* qp = (float*)malloc(sizeof(float) * nq * Dp);
    for (size_t i = 0; i < nq * Dc; i++) qn[i] = orc_bf16_decode(q_nope[i]);
    for (size_t i = 0; i < nq * Dp; i++) qp[i] = orc_bf16_decode(q_pe[i]);
    size_t rows = (size_t)Q * S;
    float* gkc = (float*)malloc(sizeof(float) * rows * Dc);
    float* gkp = (float*)malloc(sizeof(float) * rows * Dp);
    float* gv = (float*)malloc(sizeof(float) * rows * Dc);
    int* gi = (int*)malloc(sizeof(int) * rows);
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        int64_t id = idx[r];
        for (int d = 0; d < Dc; d++) gkc[r * Dc + d] = orc_bf16_decode(kc[id * Dc + d]);
        for (int d = 0; d < Dp; d++) gkp[r * Dp + d] = orc_bf16_decode(kp[id * Dp + d]);
        for (int d = 0; d < Dc; d++) gv[r * Dc + d] = orc_bf16_decode(v[id * Dc + d]);
        gi[r] = (int)r;
    }
    orc_dsa_forward_f32(qn, qp, gkc, gkp, gv, gi, out, Q, H, Dc, Dp, S);
    free(qn); free(qp); free(gkc); free(gkp); free(gv); free(gi);
}

/* Same, but the caller has already gathered the selected rows (row r of the
 * compact buffers belongs to flat pair r = q*S + s). */
ORC_API void orc_dsa_forward_bf16_gathered(const uint16_t* q_nope, const uint16_t* q_pe,
                                           const uint16_t* gkc, const uint16_t* gkp, const uint16_t* gv,
                                           float* out, int Q, int H, int Dc, int Dp, int S) {
    size_t rows = (size_t)Q * S;
    int* gi = (int*)malloc(sizeof(int) * rows);
    for (size_t r = 0; r < rows; r++) gi[r] = (int)r;
    orc_dsa_forward_bf16(q_nope, q_pe, gkc, gkp, gv, gi, out, Q, H, Dc, Dp, S);
    free(gi);
}
