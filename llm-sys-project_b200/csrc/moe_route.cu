// MoE routing and permutation (all data types share these kernels).
//
//   gate_logits_kernel   tokens x experts register-tiled (128 x 128 x 16, 8 x 8 per thread) dot products.  Each logit is
//                        accumulated in a fixed order so the CPU side can reproduce it
//                        bit for bit: chunks of `chunk` consecutive d, each chunk a
//                        sequential chain from 0, chunk partials summed in order.
//                        fp32 inputs use mul-then-add (the reference's arithmetic,
//                        kernels/moe/naive_moe.cu:102-106); FP8 inputs are dequantised
//                        on load and use fused multiply-add.
//   route_select_kernel  one warp per token: scoring + top-K + histogram.
//                        softmax mode follows naive_moe.cu:109-141 step by step;
//                        grouped-sigmoid mode is the DeepSeek-V3 style selection.
//   permute_kernel       one block per expert: stable counting pass producing
//                        counts / exclusive offsets / row -> (token,slot) map
//                        (replaces the E single-thread scans of naive_moe.cu:147-166).
#include <cfloat>

#include "common.cuh"
#include "moe_internal.cuh"
#include "selftest.h"

// ---------------------------------------------------------------------------
// gate logits
// ---------------------------------------------------------------------------
#define GL_TM 128
#define GL_TN 128
#define GL_TK 16
#define GL_LD (GL_TM + 4)

// Block tile 128 tokens x 128 experts, 8 x 8 outputs per thread; every output is still one
// sequential chain over d inside its chunk, so the CPU reproduces it bit for bit.
// VEC: rows are 16-byte aligned and the chunk length is a multiple of 16 (vector loads).
template <bool FP8, bool VEC>
__global__ void __launch_bounds__(256)
gate_logits_kernel(const void* __restrict__ x_, const float* __restrict__ xs, const float* __restrict__ wg,
                   float* __restrict__ partials, int T, int E, int D, int chunk) {
    __shared__ __align__(16) float As[GL_TK][GL_LD];
    __shared__ __align__(16) float Bs[GL_TK][GL_LD];
    const int t0 = blockIdx.x * GL_TM, e0 = blockIdx.y * GL_TN, c = blockIdx.z;
    const int d_begin = c * chunk;
    const int d_end = min(D, d_begin + chunk);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx -> 8 experts, ty -> 8 tokens
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    for (int d0 = d_begin; d0 < d_end; d0 += GL_TK) {
        // ---- stage the token tile (dequantised) and the expert tile, k-major ----
        if (VEC) {
            if (FP8) {
                if (threadIdx.x < GL_TM) {
                    const int t = t0 + threadIdx.x;
                    float v[16];
                    if (t < T) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(x_) +
                                                                          (size_t)t * D + d0);
                        const float sc = xs[(size_t)t * (D / 128) + d0 / 128];
                        const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            __nv_fp8_e4m3 q;
                            q.__x = b[i];
                            v[i] = __fmul_rn(float(q), sc);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; i++) v[i] = 0.0f;
                    }
#pragma unroll
                    for (int i = 0; i < 16; i++) As[i][threadIdx.x] = v[i];
                }
            } else {
#pragma unroll
                for (int rep = 0; rep < 2; rep++) {
                    const int idx = threadIdx.x + rep * 256, r = idx >> 2, kq = (idx & 3) * 4;
                    const int t = t0 + r;
                    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (t < T) v = *reinterpret_cast<const float4*>(static_cast<const float*>(x_) + (size_t)t * D + d0 + kq);
                    As[kq][r] = v.x; As[kq + 1][r] = v.y; As[kq + 2][r] = v.z; As[kq + 3][r] = v.w;
                }
            }
#pragma unroll
            for (int rep = 0; rep < 2; rep++) {
                const int idx = threadIdx.x + rep * 256, r = idx >> 2, kq = (idx & 3) * 4;
                const int e = e0 + r;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (e < E) v = *reinterpret_cast<const float4*>(wg + (size_t)e * D + d0 + kq);
                Bs[kq][r] = v.x; Bs[kq + 1][r] = v.y; Bs[kq + 2][r] = v.z; Bs[kq + 3][r] = v.w;
            }
        } else {
            for (int idx = threadIdx.x; idx < GL_TM * GL_TK; idx += 256) {
                const int r = idx / GL_TK, k = idx % GL_TK, d = d0 + k;
                float xv = 0.0f, wv = 0.0f;
                if (d < d_end) {
                    if (t0 + r < T) {
                        if (FP8) {
                            __nv_fp8_e4m3 q;
                            q.__x = static_cast<const uint8_t*>(x_)[(size_t)(t0 + r) * D + d];
                            xv = __fmul_rn(float(q), xs[(size_t)(t0 + r) * (D / 128) + d / 128]);
                        } else {
                            xv = static_cast<const float*>(x_)[(size_t)(t0 + r) * D + d];
                        }
                    }
                    if (e0 + r < E) wv = wg[(size_t)(e0 + r) * D + d];
                }
                As[k][r] = xv;
                Bs[k][r] = wv;
            }
        }
        __syncthreads();
        const int kmax = min(GL_TK, d_end - d0);
#pragma unroll 4
        for (int k = 0; k < kmax; k++) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[k][ty * 8 + 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 8]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][tx * 8 + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (FP8) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
                    else     acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + ty * 8 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int e = e0 + tx * 8 + j;
            if (e < E) partials[((size_t)c * T + t) * E + e] = acc[i][j];
        }
    }
}

// ---------------------------------------------------------------------------
// selection
// ---------------------------------------------------------------------------
struct ValIdx { float v; int i; };
__device__ __forceinline__ ValIdx better(ValIdx a, ValIdx b) {
    // larger value wins; equal values -> lower index wins; index -1 = empty
    if (b.i < 0) return a;
    if (a.i < 0) return b;
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ __forceinline__ ValIdx warp_argmax(ValIdx x) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ValIdx y;
        y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
        y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
        x = better(x, y);
    }
    return x;
}

// One token's selection, executed by one warp.  s / c: E floats each of this warp's shared memory.
__device__ __forceinline__ void
route_select_row(const float* __restrict__ partials, int n_chunks, const float* __restrict__ bias,
                 int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                 float* __restrict__ logits_out, int T, int E, int K, int scoring, int n_group,
                 int topk_group, float routed_scale, const RouteCert& cert, int row, int t, float* s, float* c,
                 int lane) {
    // logit = the partial sums added in chunk order; the loads of eight chunks are issued together so that their
    // latencies overlap (the adds stay in order)
    if (cert.plan.L > 0) n_chunks = tc_slots_before(cert.plan, row / 128, (row / 128 + 1) * cert.plan.nblk);
    for (int e = lane; e < E; e += 32) {
        float l = 0.0f;
        for (int ch0 = 0; ch0 < n_chunks; ch0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                v[j] = (ch0 + j < n_chunks) ? __ldg(&partials[((size_t)(ch0 + j) * T + row) * E + e]) : 0.0f;
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (ch0 + j < n_chunks) l = (ch0 + j == 0) ? v[j] : __fadd_rn(l, v[j]);
        }
        s[e] = l;
        if (logits_out) logits_out[(size_t)t * E + e] = l;
    }
    __syncwarp();

    int* oi = ids + (size_t)t * K;
    float* ow = wts + (size_t)t * K;

    if (scoring == B200_SCORE_SOFTMAX) {
        // naive_moe.cu:109-141, executed serially by one lane so that every rounding
        // step happens in the reference's order.
        if (lane == 0) {
            float mx = -FLT_MAX;
            for (int e = 0; e < E; e++) mx = fmaxf(mx, s[e]);
            float sum = 0.0f;
            for (int e = 0; e < E; e++) {
                float p = (float)exp((double)__fsub_rn(s[e], mx));   // correctly rounded expf
                s[e] = p;
                sum = __fadd_rn(sum, p);
            }
            for (int e = 0; e < E; e++) s[e] = __fdiv_rn(s[e], sum);
            for (int k = 0; k < K; k++) { c[k] = -FLT_MAX; oi[k] = -1; }   // c[0..K) = slot weights
            for (int e = 0; e < E; e++) {
                float v = s[e];
                int min_k = 0;
                for (int k = 1; k < K; k++)
                    if (c[k] < c[min_k]) min_k = k;
                if (v > c[min_k]) { c[min_k] = v; oi[min_k] = e; }
            }
            float tot = 0.0f;
            for (int k = 0; k < K; k++) tot = __fadd_rn(tot, c[k]);
            for (int k = 0; k < K; k++) {
                ow[k] = (tot > 0.0f) ? __fdiv_rn(c[k], tot) : c[k];
                if (counts && oi[k] >= 0) atomicAdd(&counts[oi[k]], 1);
            }
        }
        return;
    }

    // ---- sigmoid + bias, group-limited top-K ---------------------------------
    // Certification threshold of this token: the tensor core's summation error grows with the size of the sums,
    // so the threshold scales with the root mean square of the token's logits (never below the base value).
    float tau = cert.tau;
    if (cert.tau > 0.0f) {
        float ss = 0.0f;
        for (int e = lane; e < E; e += 32) ss = fmaf(s[e], s[e], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        tau *= fmaxf(1.0f, sqrtf(ss / (float)E));
    }
    for (int e = lane; e < E; e += 32) {
        // exact logits: correctly rounded sigmoid; approximate logits: the fp32 formula (its error, about 1e-7,
        // is far below the threshold that sends a token to the exact pass)
        float sg = (cert.tau > 0.0f) ? __fdividef(1.0f, 1.0f + __expf(-s[e]))
                                     : (float)(1.0 / (1.0 + exp(-(double)s[e])));
        s[e] = sg;
        c[e] = __fadd_rn(sg, bias ? bias[e] : 0.0f);
    }
    __syncwarp();
    const int gs = E / n_group;
    // group scores: lane g (< n_group, n_group <= 32) keeps group g's score
    float my_gscore = -FLT_MAX;
    for (int g = 0; g < n_group; g++) {
        ValIdx b1 = {0.0f, -1};
        for (int j = lane; j < gs; j += 32) b1 = better(b1, ValIdx{c[g * gs + j], j});
        b1 = warp_argmax(b1);
        float sc = b1.v;
        if (gs > 1) {
            ValIdx b2 = {0.0f, -1};
            for (int j = lane; j < gs; j += 32)
                if (j != b1.i) b2 = better(b2, ValIdx{c[g * gs + j], j});
            b2 = warp_argmax(b2);
            sc = __fadd_rn(b1.v, b2.v);
        }
        if (lane == g) my_gscore = sc;
    }
    // keep topk_group groups: bit g of keep_mask
    unsigned keep_mask = 0;
    bool mine_taken = false;
    for (int r = 0; r < topk_group; r++) {
        ValIdx cand = {my_gscore, (lane < n_group && !mine_taken) ? lane : -1};
        cand = warp_argmax(cand);
        keep_mask |= 1u << cand.i;
        if (lane == cand.i) mine_taken = true;
    }
    // Certification (approximate logits only): the smallest gap between the kept and the dropped group scores.
    // A group score is the sum of two selection scores, so its error is twice theirs.
    float min_margin = FLT_MAX;
    if (cert.tau > 0.0f && topk_group < n_group) {
        float kept = (lane < n_group && ((keep_mask >> lane) & 1u)) ? my_gscore : FLT_MAX;
        float dropped = (lane < n_group && !((keep_mask >> lane) & 1u)) ? my_gscore : -FLT_MAX;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kept = fminf(kept, __shfl_xor_sync(0xffffffffu, kept, o));
            dropped = fmaxf(dropped, __shfl_xor_sync(0xffffffffu, dropped, o));
        }
        min_margin = 0.5f * (kept - dropped);
    }
    // top-K experts among kept groups.  Taken experts get c = -inf marker via NaN-free flag array:
    // reuse the sign of s? Keep a separate taken bit by setting c[e] to -FLT_MAX after selection.
    float sum = 0.0f;
    float my_w = 0.0f;      // lane k keeps slot k's unnormalised weight (K <= 32)
    int my_id = -1;
    float prev_v = FLT_MAX;
    const int rounds = (cert.tau > 0.0f) ? K + 1 : K;       // one more round: the best expert that is NOT selected
    for (int k = 0; k < rounds; k++) {
        ValIdx b = {0.0f, -1};
        for (int e = lane; e < E; e += 32)
            if (((keep_mask >> (e / gs)) & 1u) && c[e] != -FLT_MAX) b = better(b, ValIdx{c[e], e});
        b = warp_argmax(b);
        if (cert.tau > 0.0f && b.i >= 0) {
            if (k > 0) min_margin = fminf(min_margin, prev_v - b.v);     // order of the selected, and K-th vs (K+1)-th
            prev_v = b.v;
        }
        if (k == K) break;
        float sv = (b.i >= 0) ? s[b.i] : 0.0f;
        __syncwarp();
        if (lane == 0 && b.i >= 0) c[b.i] = -FLT_MAX;
        __syncwarp();
        sum = __fadd_rn(sum, sv);
        if (lane == k) { my_w = sv; my_id = b.i; }
    }
    // A token whose decisions are not certain at the approximation's accuracy goes on the list of the exact pass
    // (which overwrites its ids / weights and counts it in the histogram).
    const bool uncertain = cert.tau > 0.0f && !(min_margin > tau);
    if (uncertain && lane == 0) cert.flag_list[atomicAdd(cert.flag_n, 1)] = t;
    if (lane < K) {
        oi[lane] = my_id;
        ow[lane] = __fmul_rn(__fdiv_rn(my_w, sum), routed_scale);
        if (counts && my_id >= 0 && !uncertain) atomicAdd(&counts[my_id], 1);
    }
}

// ---------------------------------------------------------------------------
// Grouped sigmoid selection with the token's scores in registers: lane L holds the PER = E / 32 experts
// L * PER .. L * PER + PER - 1, a group is a run of LPG = (E / n_group) / PER lanes (a power of two).  Same
// decisions and the same arithmetic as route_select_row, several times fewer instructions: the group scores of
// all groups are formed at once by a butterfly over each group's lanes, the kept groups by ranking.
// ---------------------------------------------------------------------------
template <int PER>
__device__ __forceinline__ void load_run(const float* p, float* v) {
    if constexpr (PER % 4 == 0) {
#pragma unroll
        for (int j = 0; j < PER; j += 4) {
            const float4 x = __ldg(reinterpret_cast<const float4*>(p + j));
            v[j] = x.x; v[j + 1] = x.y; v[j + 2] = x.z; v[j + 3] = x.w;
        }
    } else if constexpr (PER == 2) {
        const float2 x = __ldg(reinterpret_cast<const float2*>(p));
        v[0] = x.x; v[1] = x.y;
    } else {
#pragma unroll
        for (int j = 0; j < PER; j++) v[j] = __ldg(p + j);
    }
}

template <int PER>
__device__ __forceinline__ void
route_select_row_regs(const float* __restrict__ partials, int n_chunks, const float* __restrict__ bias,
                      int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                      float* __restrict__ logits_out, int T, int E, int K, int n_group, int topk_group,
                      float routed_scale, const RouteCert& cert, int row, int t, int lane) {
    const int e_lo = lane * PER;
    if (cert.plan.L > 0) n_chunks = tc_slots_before(cert.plan, row / 128, (row / 128 + 1) * cert.plan.nblk);
    float lg[PER];
    // logit = the partial sums added in chunk order (loads of four chunks in flight, adds in order)
    for (int ch0 = 0; ch0 < n_chunks; ch0 += 4) {
        float v[4][PER];
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (ch0 + i < n_chunks) load_run<PER>(partials + ((size_t)(ch0 + i) * T + row) * E + e_lo, v[i]);
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (ch0 + i < n_chunks) {
#pragma unroll
                for (int j = 0; j < PER; j++) lg[j] = (ch0 + i == 0) ? v[i][j] : __fadd_rn(lg[j], v[i][j]);
            }
    }
    if (logits_out) {
#pragma unroll
        for (int j = 0; j < PER; j++) logits_out[(size_t)t * E + e_lo + j] = lg[j];
    }
    float tau = cert.tau;
    if (cert.tau > 0.0f) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; j++) ss = fmaf(lg[j], lg[j], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        tau *= fmaxf(1.0f, sqrtf(ss / (float)E));
    }
    float sg[PER], c[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        sg[j] = (cert.tau > 0.0f) ? __fdividef(1.0f, 1.0f + __expf(-lg[j]))
                                  : (float)(1.0 / (1.0 + exp(-(double)lg[j])));
        c[j] = __fadd_rn(sg[j], bias ? bias[e_lo + j] : 0.0f);
    }
    // ---- group scores: best two selection scores of every group ----
    const int gs = E / n_group, lpg = gs / PER, g = lane / lpg;
    ValIdx b1 = {0.0f, -1}, b2 = {0.0f, -1};
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const ValIdx v = {c[j], e_lo + j};
        const ValIdx top = better(b1, v);
        b2 = (top.i == v.i) ? b1 : better(b2, v);
        b1 = top;
    }
    for (int o = 1; o < lpg; o <<= 1) {
        ValIdx o1, o2;
        o1.v = __shfl_xor_sync(0xffffffffu, b1.v, o); o1.i = __shfl_xor_sync(0xffffffffu, b1.i, o);
        o2.v = __shfl_xor_sync(0xffffffffu, b2.v, o); o2.i = __shfl_xor_sync(0xffffffffu, b2.i, o);
        const ValIdx top = better(b1, o1);
        b2 = (top.i == b1.i) ? better(b2, o1) : better(b1, o2);
        b1 = top;
    }
    const float gscore = (gs > 1) ? __fadd_rn(b1.v, b2.v) : b1.v;
    // ---- kept groups: group g stays if fewer than topk_group groups beat it (ties: the lower group wins) ----
    int beaten_by = 0;
    for (int h = 0; h < n_group; h++) {
        const float sh = __shfl_sync(0xffffffffu, gscore, h * lpg);
        beaten_by += (sh > gscore || (sh == gscore && h < g)) ? 1 : 0;
    }
    const bool keep = beaten_by < topk_group;
    float min_margin = FLT_MAX;
    if (cert.tau > 0.0f && topk_group < n_group) {
        float kept = keep ? gscore : FLT_MAX, dropped = keep ? -FLT_MAX : gscore;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            kept = fminf(kept, __shfl_xor_sync(0xffffffffu, kept, o));
            dropped = fmaxf(dropped, __shfl_xor_sync(0xffffffffu, dropped, o));
        }
        min_margin = 0.5f * (kept - dropped);
    }
    // ---- top-K experts among the kept groups, best first ----
    unsigned taken = keep ? 0u : 0xffffffffu;
    float sum = 0.0f, my_w = 0.0f, prev_v = FLT_MAX;
    int my_id = -1;
    const int rounds = (cert.tau > 0.0f) ? K + 1 : K;       // one more round: the best expert that is NOT selected
    for (int k = 0; k < rounds; k++) {
        ValIdx b = {0.0f, -1};
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (!((taken >> j) & 1u)) b = better(b, ValIdx{c[j], e_lo + j});
        b = warp_argmax(b);
        if (cert.tau > 0.0f && b.i >= 0) {
            if (k > 0) min_margin = fminf(min_margin, prev_v - b.v);
            prev_v = b.v;
        }
        if (k == K) break;
        const int owner = (b.i >= 0) ? b.i / PER : 0, slot = (b.i >= 0) ? b.i % PER : 0;
        float mine = 0.0f;
#pragma unroll
        for (int j = 0; j < PER; j++) mine = (j == slot) ? sg[j] : mine;
        float sv = __shfl_sync(0xffffffffu, mine, owner);
        if (b.i < 0) sv = 0.0f;
        if (b.i >= 0 && lane == owner) taken |= 1u << slot;
        sum = __fadd_rn(sum, sv);
        if (lane == k) { my_w = sv; my_id = b.i; }
    }
    const bool uncertain = cert.tau > 0.0f && !(min_margin > tau);
    if (uncertain && lane == 0) cert.flag_list[atomicAdd(cert.flag_n, 1)] = t;
    if (lane < K) {
        ids[(size_t)t * K + lane] = my_id;
        wts[(size_t)t * K + lane] = __fmul_rn(__fdiv_rn(my_w, sum), routed_scale);
        if (counts && my_id >= 0 && !uncertain) atomicAdd(&counts[my_id], 1);
    }
}

// The register path serves: E = 32 * PER with PER in {1, 2, 4, 8}, groups that are whole runs of lanes
// (power-of-two many), K <= 32.
__host__ __device__ inline int route_regs_per(int E, int K, int scoring, int n_group) {
    if (scoring != B200_SCORE_SIGMOID_GROUPED || E % 32 || K > 32 || n_group < 1 || n_group > 32 || E % n_group) return 0;
    const int per = E / 32, gs = E / n_group;
    if (per != 1 && per != 2 && per != 4 && per != 8) return 0;
    if (gs % per) return 0;
    const int lpg = gs / per;
    if (lpg & (lpg - 1)) return 0;
    return per;
}

// smem per warp: E floats (scores s) + E floats (selection scores c).  One warp per row of `partials`, rows
// taken with the grid's stride.  List mode (cert.list): the rows are the tokens of cert.list, in list order, and
// only the first *cert.list_n rows exist (a count known only on the device).
__global__ void __launch_bounds__(128)
route_select_kernel(const float* __restrict__ partials, int n_chunks, const float* __restrict__ bias,
                    int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                    float* __restrict__ logits_out, int T, int E, int K, int scoring, int n_group,
                    int topk_group, float routed_scale, RouteCert cert) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* s = sm + (size_t)warp * 2 * E;
    float* c = s + E;
    const int rows = cert.list ? min(*cert.list_n, T) : T;
    for (int row = blockIdx.x * 4 + warp; row < rows; row += gridDim.x * 4) {
        const int t = cert.list ? cert.list[row] : row;
        route_select_row(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K, scoring, n_group,
                         topk_group, routed_scale, cert, row, t, s, c, lane);
        __syncwarp();
    }
}

// The register path as a kernel of its own (fewer registers than the generic kernel: more resident warps).  Seven
// blocks per SM (72 registers, a few spilled words): 148 x 7 x 4 warps take 4096 tokens in one wave.
template <int PER>
__global__ void __launch_bounds__(128, 7)
route_select_regs_kernel(const float* __restrict__ partials, int n_chunks, const float* __restrict__ bias,
                         int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                         float* __restrict__ logits_out, int T, int E, int K, int n_group, int topk_group,
                         float routed_scale, RouteCert cert) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = cert.list ? min(*cert.list_n, T) : T;
    for (int row = blockIdx.x * 4 + warp; row < rows; row += gridDim.x * 4) {
        const int t = cert.list ? cert.list[row] : row;
        route_select_row_regs<PER>(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K, n_group, topk_group,
                                   routed_scale, cert, row, t, lane);
    }
}

// ---------------------------------------------------------------------------
// permutation
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool pair_selects(const int* __restrict__ ids, int p, int K, int e) {
    if (ids[p] != e) return false;
    int k = p % K, base = p - k;
    for (int j = 0; j < k; j++)
        if (ids[base + j] == e) return false;   // a token counts once per expert (naive_moe.cu:156-161)
    return true;
}

// Per-expert counts of the (token, slot) pairs that select it (ids outside [0,E) and, with CHECK_DUP,
// repeated ids of a token are not counted): shared-memory histogram per block, flushed with atomics.
template <bool CHECK_DUP>
__global__ void __launch_bounds__(256)
pair_histogram_kernel(const int* __restrict__ ids, int TK, int K, int E, int* __restrict__ counts) {
    extern __shared__ int s_hist[];
    for (int i = threadIdx.x; i < E; i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < TK; p += gridDim.x * blockDim.x) {
        const int id = ids[p];
        if (id >= 0 && id < E && (!CHECK_DUP || pair_selects(ids, p, K, id))) atomicAdd(&s_hist[id], 1);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < E; i += blockDim.x)
        if (s_hist[i]) atomicAdd(&counts[i], s_hist[i]);
}

// One block per expert.  The expert's first row (= rows owned by lower experts) comes from the
// per-expert counts (the router's histogram, or pair_histogram_kernel for routing supplied from
// outside); ranks inside the expert are assigned by a block scan over (token, slot) pairs in
// ascending order, four pairs per thread, 4096 pairs per round.
// CHECK_DUP: a token that lists the expert twice counts once (ids supplied from outside).
constexpr int PERMUTE_THREADS = 1024;
template <bool CHECK_DUP>
__global__ void __launch_bounds__(PERMUTE_THREADS)
permute_kernel(const int* __restrict__ ids, int TK, int K, int E, const int* __restrict__ counts_in,
               int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_pair) {
    constexpr int NW = PERMUTE_THREADS / 32;
    __shared__ int warp_sums[NW];
    __shared__ int s_base;
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    auto selects = [&](int p, int id, int want) -> bool {
        if (id != want) return false;
        if (CHECK_DUP) return pair_selects(ids, p, K, want);
        return true;
    };
    int lt = 0;
    for (int i = threadIdx.x; i < e; i += PERMUTE_THREADS) lt += counts_in[i];
    for (int o = 16; o > 0; o >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, o);
    if (lane == 0) warp_sums[warp] = lt;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < NW; w++) tot += warp_sums[w];
        s_base = tot;
    }
    __syncthreads();
    const int base = s_base;
    const bool vec = (TK % 4 == 0) && ((reinterpret_cast<uintptr_t>(ids) & 15) == 0);
    int running = 0;
    for (int p0 = 0; p0 < TK; p0 += PERMUTE_THREADS * 4) {
        const int p = p0 + threadIdx.x * 4;
        int v[4] = {-1, -1, -1, -1};
        if (vec) {
            if (p < TK) {
                const int4 q = *reinterpret_cast<const int4*>(ids + p);
                v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; i++)
                if (p + i < TK) v[i] = ids[p + i];
        }
        bool f[4];
        int c = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) { f[i] = (p + i < TK) && selects(p + i, v[i], e); c += f[i] ? 1 : 0; }
        int incl = c;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        __syncthreads();                      // previous iteration's readers are done
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < NW; w++) {
            int n = warp_sums[w];
            if (w < warp) before += n;
            total += n;
        }
        int pos = base + running + before + incl - c;
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (f[i]) row_pair[pos++] = p + i;
        running += total;
    }
    if (threadIdx.x == 0) {
        counts[e] = running;
        offsets[e] = base;
        if (e == E - 1) offsets[E] = base + running;
    }
}

// FP8 router logits, tuned variant of the kernel above for aligned inputs (rows 16-byte aligned,
// D % 16 == 0, chunk % 16 == 0).  Same arithmetic, hence the same bits: every logit is one fused
// multiply-add chain over the chunk's d in ascending order.  Differences: the token tile is
// 8 * TY rows (TY = 8..16, 16 * TY threads) so that the launcher can pick the height whose tile
// count fills whole waves of resident CTAs, and the next k-tile is fetched into registers while
// the current one is multiplied.
using ptx::pack_f32x2;
using ptx::fma_f32x2;

template <int TY>
__global__ void __launch_bounds__(16 * TY, 512 / (16 * TY))
gate_logits_fp8_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, const float* __restrict__ wg,
                       float* __restrict__ partials, int T, int E, int D, int chunk) {
    constexpr int TM = 8 * TY, NT = 16 * TY, LDA = TM + 4;
    constexpr int BREP = (GL_TN * 4 + NT - 1) / NT;          // float4 loads of the expert tile per thread
    __shared__ __align__(16) float As[GL_TK][LDA];
    __shared__ __align__(16) float Bs[GL_TK][GL_LD];
    const int t0 = blockIdx.x * TM, e0 = blockIdx.y * GL_TN, c = blockIdx.z;
    const int d_begin = c * chunk;
    const int d_end = min(D, d_begin + chunk);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx -> 8 experts, ty -> 8 tokens
    // accumulators as pairs of adjacent experts: one fma.rn.f32x2 does two IEEE fused multiply-adds
    // (same bits as two scalar ones) for one issue slot, and this kernel is bound by issue slots
    unsigned long long acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc2[i][j] = 0ull;

    uint4 a_raw = make_uint4(0, 0, 0, 0);
    float a_sc = 0.0f;
    float4 b_reg[BREP];
    const int nb = D / 128;
    auto fetch = [&](int d0) {
        if (threadIdx.x < TM) {
            const int t = t0 + threadIdx.x;
            if (t < T) {
                a_raw = *reinterpret_cast<const uint4*>(xq + (size_t)t * D + d0);
                a_sc = xs[(size_t)t * nb + d0 / 128];
            } else {
                a_raw = make_uint4(0, 0, 0, 0);
                a_sc = 0.0f;
            }
        }
#pragma unroll
        for (int rep = 0; rep < BREP; rep++) {
            const int idx = threadIdx.x + rep * NT, r = idx >> 2, kq = (idx & 3) * 4;
            b_reg[rep] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < GL_TN * 4 && e0 + r < E) b_reg[rep] = *reinterpret_cast<const float4*>(wg + (size_t)(e0 + r) * D + d0 + kq);
        }
    };
    auto stage = [&]() {
        if (threadIdx.x < TM) {
            const uint8_t* b = reinterpret_cast<const uint8_t*>(&a_raw);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                __nv_fp8_e4m3 q;
                q.__x = b[i];
                As[i][threadIdx.x] = __fmul_rn(float(q), a_sc);
            }
        }
#pragma unroll
        for (int rep = 0; rep < BREP; rep++) {
            const int idx = threadIdx.x + rep * NT, r = idx >> 2, kq = (idx & 3) * 4;
            if (idx < GL_TN * 4) {
                Bs[kq][r] = b_reg[rep].x; Bs[kq + 1][r] = b_reg[rep].y;
                Bs[kq + 2][r] = b_reg[rep].z; Bs[kq + 3][r] = b_reg[rep].w;
            }
        }
    };
    fetch(d_begin);
    for (int d0 = d_begin; d0 < d_end; d0 += GL_TK) {
        stage();
        __syncthreads();
        if (d0 + GL_TK < d_end) fetch(d0 + GL_TK);
#pragma unroll
        for (int k = 0; k < GL_TK; k++) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 8]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[k][ty * 8 + 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][tx * 8]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[k][tx * 8 + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const unsigned long long bb[4] = {pack_f32x2(b0.x, b0.y), pack_f32x2(b0.z, b0.w), pack_f32x2(b1.x, b1.y),
                                              pack_f32x2(b1.z, b1.w)};
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const unsigned long long aa = pack_f32x2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < 4; j++) acc2[i][j] = fma_f32x2(aa, bb[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int t = t0 + ty * 8 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int e = e0 + tx * 8 + j;
            const unsigned long long v = acc2[i][j >> 1];
            const float f = __uint_as_float((j & 1) ? (unsigned)(v >> 32) : (unsigned)(v & 0xffffffffull));
            if (e < E) partials[((size_t)c * T + t) * E + e] = f;
        }
    }
}

// FP8 router logits for decode-sized batches (T <= 32): the register-tiled kernels above would run
// 14 CTAs of mostly padding.  Block = 32 experts x one chunk of d; thread = (expert, token slot);
// every logit is still one fused multiply-add chain over the chunk's d in ascending order, so the
// bits are those of the other kernels.  k-tiles of 128 d are double-buffered in shared memory.
constexpr int GS_E = 32, GS_K = 128, GS_T = 8;
__global__ void __launch_bounds__(GS_E * GS_T)
gate_logits_fp8_small_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, const float* __restrict__ wg,
                             float* __restrict__ partials, int T, int E, int D, int chunk) {
    __shared__ float w_s[2][GS_E][GS_K + 1];
    __shared__ float x_s[2][GS_T][GS_K];
    const int e0 = blockIdx.x * GS_E, c = blockIdx.y;
    const int d_begin = c * chunk, d_end = min(D, d_begin + chunk);
    const int el = threadIdx.x & 31, ts = threadIdx.x >> 5;
    const int nb = D / 128;
    for (int t0 = 0; t0 < T; t0 += GS_T) {
        auto stage = [&](int buf, int d0) {
            // expert tile: 32 rows x 128 floats, coalesced along d; token tile: up to 8 rows, dequantised
            for (int i = threadIdx.x; i < GS_E * GS_K; i += GS_E * GS_T) {
                const int r = i / GS_K, k = i - r * GS_K;
                w_s[buf][r][k] = (e0 + r < E && d0 + k < d_end) ? wg[(size_t)(e0 + r) * D + d0 + k] : 0.0f;
            }
            for (int i = threadIdx.x; i < GS_T * GS_K; i += GS_E * GS_T) {
                const int r = i / GS_K, k = i - r * GS_K, t = t0 + r;
                float v = 0.0f;
                if (t < T && d0 + k < d_end) {
                    __nv_fp8_e4m3 q;
                    q.__x = xq[(size_t)t * D + d0 + k];
                    v = __fmul_rn(float(q), xs[(size_t)t * nb + (d0 + k) / 128]);
                }
                x_s[buf][r][k] = v;
            }
        };
        float acc = 0.0f;
        int buf = 0;
        stage(0, d_begin);
        __syncthreads();
        for (int d0 = d_begin; d0 < d_end; d0 += GS_K) {
            if (d0 + GS_K < d_end) stage(buf ^ 1, d0 + GS_K);
            const int kmax = min(GS_K, d_end - d0);
#pragma unroll 8
            for (int k = 0; k < kmax; k++) acc = __fmaf_rn(x_s[buf][ts][k], w_s[buf][el][k], acc);
            __syncthreads();
            buf ^= 1;
        }
        const int t = t0 + ts, e = e0 + el;
        if (t < T && e < E) partials[((size_t)c * T + t) * E + e] = acc;
        __syncthreads();
    }
}

// The same chains for a list of tokens (the exact pass of the tensor-core router).  Block = 64 threads = 32
// experts x 8 list entries per round x one chunk of d; thread = one expert x four entries, so that one 16-byte
// read of the expert's weights serves sixteen multiply-adds (the entries' activations are warp-wide broadcasts).
// k-tiles of 128 d: the next tile is fetched into registers while the current one is multiplied.  A bounded
// grid walks the list, whose length is known only on the device.
constexpr int GL2_E = 32, GL2_K = 128, GL2_T = 8, GL2_LDW = GL2_K + 4, GL2_THREADS = 64;
__global__ void __launch_bounds__(GL2_THREADS)
gate_logits_fp8_list_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, const float* __restrict__ wg,
                            float* __restrict__ partials, const int* __restrict__ list, const int* __restrict__ list_n,
                            int T, int E, int D, int chunk) {
    __shared__ __align__(16) float w_s[GL2_E][GL2_LDW];
    __shared__ __align__(16) float x_s[GL2_T][GL2_K];
    __shared__ int tok_s[GL2_T];
    const int n = min(*list_n, T);
    const int e0 = blockIdx.x * GL2_E, c = blockIdx.y;
    const int d_begin = c * chunk, d_end = min(D, d_begin + chunk);      // multiples of 128 (D % 128 == 0)
    const int el = threadIdx.x & 31, tg = threadIdx.x >> 5;
    const int nb = D / 128;
    constexpr int WREP = GL2_E * GL2_K / 4 / GL2_THREADS;                 // 16 float4 of the weight tile per thread
    const int xr = threadIdx.x >> 3, xp = threadIdx.x & 7;               // activation tile: entry xr, bytes 16*xp..
    // The block's slab of weights (32 experts x the chunk's d) is walked in eight dependent steps; asking L2 for
    // all of it up front pays the DRAM latency once instead of once per step.
    if (blockIdx.z * GL2_T < n) {
        const int lines_per_row = (d_end - d_begin) / 32;                // 128-byte lines of one expert's chunk
        for (int i = threadIdx.x; i < GL2_E * lines_per_row; i += GL2_THREADS) {
            const int r = i / lines_per_row, l = i - r * lines_per_row;
            if (e0 + r < E)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(wg + (size_t)(e0 + r) * D + d_begin + l * 32));
        }
    }
    for (int i0 = blockIdx.z * GL2_T; i0 < n; i0 += gridDim.z * GL2_T) {
        __syncthreads();
        if (threadIdx.x < GL2_T) tok_s[threadIdx.x] = (i0 + threadIdx.x < n) ? list[i0 + threadIdx.x] : -1;
        __syncthreads();
        const int xt = tok_s[xr];
        const bool x_live = xt >= 0 && xt < T;
        float4 w_reg[WREP];
        uint4 x_raw = make_uint4(0, 0, 0, 0);
        float x_sc = 0.0f;
        auto fetch = [&](int d0) {
#pragma unroll
            for (int rep = 0; rep < WREP; rep++) {
                const int idx = threadIdx.x + rep * GL2_THREADS, r = idx >> 5, kq = (idx & 31) * 4;
                w_reg[rep] = (e0 + r < E) ? __ldg(reinterpret_cast<const float4*>(wg + (size_t)(e0 + r) * D + d0 + kq))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            if (x_live) {
                x_raw = __ldg(reinterpret_cast<const uint4*>(xq + (size_t)xt * D + d0 + xp * 16));
                x_sc = xs[(size_t)xt * nb + d0 / 128];
            }
        };
        auto stage = [&]() {
#pragma unroll
            for (int rep = 0; rep < WREP; rep++) {
                const int idx = threadIdx.x + rep * GL2_THREADS, r = idx >> 5, kq = (idx & 31) * 4;
                *reinterpret_cast<float4*>(&w_s[r][kq]) = w_reg[rep];
            }
            const uint8_t* b = reinterpret_cast<const uint8_t*>(&x_raw);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                __nv_fp8_e4m3 q;
                q.__x = b[i];
                x_s[xr][xp * 16 + i] = x_live ? __fmul_rn(float(q), x_sc) : 0.0f;
            }
        };
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        fetch(d_begin);
        for (int d0 = d_begin; d0 < d_end; d0 += GL2_K) {
            __syncthreads();                      // the previous tile has been read
            stage();
            __syncthreads();
            if (d0 + GL2_K < d_end) fetch(d0 + GL2_K);
#pragma unroll 8
            for (int k = 0; k < GL2_K; k += 4) {
                const float4 w4 = *reinterpret_cast<const float4*>(&w_s[el][k]);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 x4 = *reinterpret_cast<const float4*>(&x_s[tg * 4 + i][k]);
                    acc[i] = __fmaf_rn(x4.x, w4.x, acc[i]);
                    acc[i] = __fmaf_rn(x4.y, w4.y, acc[i]);
                    acc[i] = __fmaf_rn(x4.z, w4.z, acc[i]);
                    acc[i] = __fmaf_rn(x4.w, w4.w, acc[i]);
                }
            }
        }
        const int e = e0 + el;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int li = i0 + tg * 4 + i;
            if (li < n && e < E) partials[((size_t)c * T + li) * E + e] = acc[i];
        }
    }
}

template <int TY>
static int gate_fp8_try(int want_ty, int& blocks_per_sm) {
    if (want_ty != TY) return 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, gate_logits_fp8_kernel<TY>, 16 * TY, 0);
    return 1;
}
template <int TY>
static void gate_fp8_launch(dim3 grid, cudaStream_t stream, const void* x, const float* xs, const float* wg,
                            float* partials, int T, int E, int D, int chunk) {
    gate_logits_fp8_kernel<TY><<<grid, 16 * TY, 0, stream>>>(static_cast<const uint8_t*>(x), xs, wg, partials, T, E, D, chunk);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int moe_gate_chunks(int D, bool fp8) { return fp8 ? ceil_div(D, MOE_GATE_CHUNK) : 1; }

int launch_gate_logits(const void* x, const float* xs, const float* wg, float* partials, int T, int E, int D,
                       bool fp8, cudaStream_t stream) {
    int chunk = fp8 ? MOE_GATE_CHUNK : D;
    const int n_chunks = moe_gate_chunks(D, fp8);
    const bool vec = (D % 16 == 0) && (chunk % 16 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(wg) & 15) == 0);
    if (fp8 && T <= 32 && D % 128 == 0) {
        dim3 grid(ceil_div(E, GS_E), n_chunks);
        gate_logits_fp8_small_kernel<<<grid, GS_E * GS_T, 0, stream>>>(static_cast<const uint8_t*>(x), xs, wg, partials,
                                                                      T, E, D, chunk);
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    if (fp8 && vec) {
        // Pick the token-tile height (8 * TY rows) whose tile count wastes the least of the machine:
        // tiles come in waves of (SMs x resident CTAs); cost ~ waves x rows per tile.
        static int sms = 0;
        static int occ[17] = {0};
        if (!sms) {
            int dev = 0;
            B200_CUDA_TRY(cudaGetDevice(&dev));
            B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            for (int ty = 8; ty <= 16; ty++) {
                int b = 0;
                gate_fp8_try<8>(ty, b) || gate_fp8_try<9>(ty, b) || gate_fp8_try<10>(ty, b) || gate_fp8_try<11>(ty, b) ||
                    gate_fp8_try<12>(ty, b) || gate_fp8_try<13>(ty, b) || gate_fp8_try<14>(ty, b) ||
                    gate_fp8_try<15>(ty, b) || gate_fp8_try<16>(ty, b);
                occ[ty] = b > 0 ? b : 1;
            }
        }
        int best_ty = 16;
        double best_cost = 1e300;
        for (int ty = 16; ty >= 8; ty--) {
            const long long tiles = (long long)ceil_div(T, 8 * ty) * ceil_div(E, GL_TN) * n_chunks;
            const long long slots = (long long)sms * occ[ty];
            const long long waves = (tiles + slots - 1) / slots;
            // a full wave of occ[ty] CTAs of 16*ty threads keeps an SM's FMA pipes busy for ~ occ * ty units of
            // time; when everything fits in one wave an SM works through its ceil(tiles / SMs) CTAs
            const double cost = (tiles <= slots) ? (double)((tiles + sms - 1) / sms) * ty : (double)waves * occ[ty] * ty;
            if (cost < best_cost * 0.999) { best_cost = cost; best_ty = ty; }
        }
        dim3 grid(ceil_div(T, 8 * best_ty), ceil_div(E, GL_TN), n_chunks);
        switch (best_ty) {
            case 8:  gate_fp8_launch<8>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 9:  gate_fp8_launch<9>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 10: gate_fp8_launch<10>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 11: gate_fp8_launch<11>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 12: gate_fp8_launch<12>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 13: gate_fp8_launch<13>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 14: gate_fp8_launch<14>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            case 15: gate_fp8_launch<15>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
            default: gate_fp8_launch<16>(grid, stream, x, xs, wg, partials, T, E, D, chunk); break;
        }
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    dim3 grid(ceil_div(T, GL_TM), ceil_div(E, GL_TN), n_chunks);
    if (fp8) {
        gate_logits_kernel<true, false><<<grid, 256, 0, stream>>>(x, xs, wg, partials, T, E, D, chunk);
    } else {
        if (vec) gate_logits_kernel<false, true><<<grid, 256, 0, stream>>>(x, xs, wg, partials, T, E, D, chunk);
        else     gate_logits_kernel<false, false><<<grid, 256, 0, stream>>>(x, xs, wg, partials, T, E, D, chunk);
    }
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int launch_gate_logits_list(const uint8_t* xq, const float* xs, const float* wg, float* partials, const int* list,
                            const int* list_n, int T, int E, int D, cudaStream_t stream) {
    if (D % 128) return B200_BAD_SHAPE;
    if ((reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wg) & 15)) return B200_BAD_ARG;
    dim3 grid(ceil_div(E, GL2_E), moe_gate_chunks(D, true), min(ceil_div(T, GL2_T), 32));
    gate_logits_fp8_list_kernel<<<grid, GL2_THREADS, 0, stream>>>(xq, xs, wg, partials, list, list_n, T, E, D, MOE_GATE_CHUNK);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int launch_route_select(const float* partials, int n_chunks, const float* bias, int* ids, float* wts, int* counts,
                        float* logits_out, int T, int E, int K, int scoring, int n_group, int topk_group,
                        float routed_scale, cudaStream_t stream, RouteCert cert) {
    size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) {
        B200_CUDA_TRY(cudaFuncSetAttribute(route_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem));
    }
    // list mode: the length of the list is known only on the device; a modest grid walks it with a stride
    const int blocks = cert.list ? min(ceil_div(T, 4), 4 * 148) : ceil_div(T, 4);
    const int per = route_regs_per(E, K, scoring, n_group);
    if (per == 8)
        route_select_regs_kernel<8><<<blocks, 128, 0, stream>>>(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K,
                                                                n_group, topk_group, routed_scale, cert);
    else if (per == 4)
        route_select_regs_kernel<4><<<blocks, 128, 0, stream>>>(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K,
                                                                n_group, topk_group, routed_scale, cert);
    else if (per == 2)
        route_select_regs_kernel<2><<<blocks, 128, 0, stream>>>(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K,
                                                                n_group, topk_group, routed_scale, cert);
    else if (per == 1)
        route_select_regs_kernel<1><<<blocks, 128, 0, stream>>>(partials, n_chunks, bias, ids, wts, counts, logits_out, T, E, K,
                                                                n_group, topk_group, routed_scale, cert);
    else
        route_select_kernel<<<blocks, 128, smem, stream>>>(partials, n_chunks, bias, ids, wts, counts,
                                                           logits_out, T, E, K, scoring, n_group, topk_group,
                                                           routed_scale, cert);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// Minimum decision margin (in selection-score units) a token must show on the approximate logits.  The tensor
// core adds each product into its fp32 accumulator with truncation, so the error of a logit grows with the length
// of the accumulation chain: with chains of at most four 128-deep blocks (moe_route_tc.cu) and unit-variance logits the
// largest |approximate - exact| measured on the full-size router is 2.1e-5 (a single chain over D = 7168: 2.4e-4).
// Assumed bound: 2^-14 = 6.1e-5 per unit of logit rms.  A selection score moves by at most a quarter of the logit
// error (sigmoid), so two scores can close in on each other by 2 * 2^-14 / 4 = 3.05e-5; a token whose smallest
// decision margin is not above that is recomputed exactly.  tests/test_moe_router_tc_gpu.py holds the measured
// error below half of the assumed bound.
constexpr float ROUTE_TC_TAU = 3.06e-5f;

size_t moe_route_scratch_floats(int T, int E, int D) {
    const size_t nch = (size_t)max(moe_gate_chunks(D, true), moe_gate_tc_slots(D));
    size_t n = nch * T * E;                              // partials
    if (moe_gate_tc_supported(T, E, D)) n += 2 * (size_t)E * D + (size_t)T + 64;      // whi, wlo, flag list, counter
    return n + 256;
}

int moe_route_fp8_run(const RouteScratch& rs, const uint8_t* xq, const float* xs, const float* gate_w, const float* bias,
                      int* ids, float* wts, int* counts, float* logits_out, const b200_moe_fp8_config* cfg,
                      int* status, cudaStream_t stream) {
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim;
    if (counts) B200_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * E, stream));
    const int nch = moe_gate_chunks(D, true);
    // Tensor-core path: grouped sigmoid routing, no logits requested (the logits it computes are approximate),
    // a batch large enough to fill 128-token tiles
    const bool tc = rs.whi && !logits_out && cfg->scoring == B200_SCORE_SIGMOID_GROUPED && !(cfg->flags & B200_MOE_EXACT_ROUTER_LOGITS) &&
                    moe_gate_tc_supported(T, E, D) && !((reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(gate_w)) & 15);
    if (!tc) {
        int st = launch_gate_logits(xq, xs, gate_w, rs.partials, T, E, D, true, stream);
        if (st) return st;
        return launch_route_select(rs.partials, nch, bias, ids, wts, counts, logits_out, T, E, K, cfg->scoring,
                                   cfg->n_group, cfg->topk_group, cfg->routed_scale, stream);
    }
    B200_CUDA_TRY(cudaMemsetAsync(rs.flag_n, 0, sizeof(int), stream));
    RouteCert approx;
    int st = launch_gate_logits_tc(xq, xs, gate_w, rs.whi, rs.wlo, rs.partials, T, E, D, status, stream, &approx.plan);
    if (st) return st;
    approx.tau = ROUTE_TC_TAU; approx.flag_list = rs.flag_list; approx.flag_n = rs.flag_n;
    st = launch_route_select(rs.partials, 0, bias, ids, wts, counts, nullptr, T, E, K, cfg->scoring,
                             cfg->n_group, cfg->topk_group, cfg->routed_scale, stream, approx);
    if (st) return st;
    // exact pass over the flagged tokens (usually a few per cent): the fixed-order chains, then the same selection
    st = launch_gate_logits_list(xq, xs, gate_w, rs.partials, rs.flag_list, rs.flag_n, T, E, D, stream);
    if (st) return st;
    RouteCert exact;
    exact.list = rs.flag_list; exact.list_n = rs.flag_n;
    return launch_route_select(rs.partials, nch, bias, ids, wts, counts, nullptr, T, E, K, cfg->scoring, cfg->n_group,
                               cfg->topk_group, cfg->routed_scale, stream, exact);
}

int launch_permute(const int* ids, int T, int K, int E, const int* counts_in, bool trusted, int* counts,
                   int* offsets, int* row_pair, cudaStream_t stream) {
    const int TK = T * K;
    if (!counts_in) {
        // no histogram from the router: count first (all SMs), then every expert's block knows its base
        B200_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * (size_t)E, stream));
        const int blocks = max(1, min((TK + 1023) / 1024, 1184));
        if (trusted) pair_histogram_kernel<false><<<blocks, 256, sizeof(int) * (size_t)E, stream>>>(ids, TK, K, E, counts);
        else         pair_histogram_kernel<true><<<blocks, 256, sizeof(int) * (size_t)E, stream>>>(ids, TK, K, E, counts);
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
        counts_in = counts;       // each block rewrites its own entry with the same value at the end
    }
    if (trusted) permute_kernel<false><<<E, PERMUTE_THREADS, 0, stream>>>(ids, TK, K, E, counts_in, counts, offsets, row_pair);
    else         permute_kernel<true><<<E, PERMUTE_THREADS, 0, stream>>>(ids, TK, K, E, counts_in, counts, offsets, row_pair);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int check_route_cfg(int T, int E, int K, int D, int scoring, int n_group, int topk_group) {
    if (T <= 0 || E <= 0 || K <= 0 || D <= 0) return B200_BAD_SHAPE;
    if (K > E) return B200_BAD_SHAPE;           // the reference would leave -1 ids (never exercised)
    if (E > 4096) return B200_UNSUPPORTED;
    if (scoring == B200_SCORE_SIGMOID_GROUPED) {
        if (n_group <= 0 || n_group > 32 || E % n_group) return B200_BAD_SHAPE;
        if (topk_group <= 0 || topk_group > n_group) return B200_BAD_SHAPE;
        if (K > 32 || K > topk_group * (E / n_group)) return B200_BAD_SHAPE;
    } else if (scoring != B200_SCORE_SOFTMAX) {
        return B200_BAD_ARG;
    }
    return B200_OK;
}

extern "C" {

int b200_moe_gate_f32(b200_ws* ws, const float* x, const float* gate_w, int* expert_ids, float* expert_w,
                      const b200_moe_config* cfg, b200_stream_t stream) {
    if (!x || !gate_w || !expert_ids || !expert_w || !cfg) return B200_BAD_ARG;
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim;
    int st = check_route_cfg(T, E, K, D, B200_SCORE_SOFTMAX, 1, 1);
    if (st) return st;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    WsCarver sz(nullptr);
    sz.take<float>((size_t)T * E);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    float* partials = cv.take<float>((size_t)T * E);
    st = launch_gate_logits(x, nullptr, gate_w, partials, T, E, D, false, stream);
    if (st) return st;
    return launch_route_select(partials, 1, nullptr, expert_ids, expert_w, nullptr, nullptr, T, E, K,
                               B200_SCORE_SOFTMAX, 1, 1, 1.0f, stream);
}

int b200_moe_route_fp8(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w, const float* bias,
                       int* expert_ids, float* expert_w, int* counts, float* logits_out,
                       const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    if (!xq || !xs || !gate_w || !expert_ids || !expert_w || !cfg) return B200_BAD_ARG;
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim;
    int st = check_route_cfg(T, E, K, D, cfg->scoring, cfg->n_group, cfg->topk_group);
    if (st) return st;
    if (D % 128) return B200_BAD_SHAPE;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    auto carve = [&](WsCarver& c, RouteScratch& rs) {
        const bool tc = moe_gate_tc_supported(T, E, D);
        rs.partials = c.take<float>((size_t)max(moe_gate_chunks(D, true), moe_gate_tc_slots(D)) * T * E);
        rs.whi = tc ? c.take<float>((size_t)E * D) : nullptr;
        rs.wlo = tc ? c.take<float>((size_t)E * D) : nullptr;
        rs.flag_list = tc ? c.take<int>((size_t)T) : nullptr;
        rs.flag_n = tc ? c.take<int>(1) : nullptr;
    };
    RouteScratch rs;
    WsCarver sz(nullptr);
    carve(sz, rs);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    carve(cv, rs);
    ws->route_flag_n = nullptr;
    st = moe_route_fp8_run(rs, xq, xs, gate_w, bias, expert_ids, expert_w, counts, logits_out, cfg, ws->d_status, stream);
    if (st == B200_OK && rs.whi && !logits_out && cfg->scoring == B200_SCORE_SIGMOID_GROUPED &&
        !(cfg->flags & B200_MOE_EXACT_ROUTER_LOGITS))
        ws->route_flag_n = rs.flag_n;
    return st;
}

int b200_moe_route_last_flagged(b200_ws* ws, b200_stream_t stream, int* n) {
    if (!n) return B200_BAD_ARG;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    *n = -1;
    if (!ws->route_flag_n) return B200_OK;
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    B200_CUDA_TRY(cudaMemcpy(n, ws->route_flag_n, sizeof(int), cudaMemcpyDeviceToHost));
    return B200_OK;
}

int b200_moe_permute(b200_ws*, const int* expert_ids, int T, int K, int E, int* counts, int* offsets,
                     int* row_pair, b200_stream_t stream) {
    if (!expert_ids || !counts || !offsets || !row_pair) return B200_BAD_ARG;
    if (T <= 0 || K <= 0 || E <= 0) return B200_BAD_SHAPE;
    return launch_permute(expert_ids, T, K, E, nullptr, false, counts, offsets, row_pair, stream);
}

}  // extern "C"
