// MoE routing and permutation (all data types share these kernels).
//
//   gate_logits_kernel   tokens x experts register-tiled dot products.  Each logit is
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

// ---------------------------------------------------------------------------
// gate logits
// ---------------------------------------------------------------------------
#define GL_TM 64
#define GL_TN 64
#define GL_TK 16

template <bool FP8>
__global__ void __launch_bounds__(256)
gate_logits_kernel(const void* __restrict__ x_, const float* __restrict__ xs, const float* __restrict__ wg,
                   float* __restrict__ partials, int T, int E, int D, int chunk) {
    __shared__ float As[GL_TK][GL_TM + 4];
    __shared__ float Bs[GL_TK][GL_TN + 4];
    const int t0 = blockIdx.x * GL_TM, e0 = blockIdx.y * GL_TN, c = blockIdx.z;
    const int d_begin = c * chunk;
    const int d_end = min(D, d_begin + chunk);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // tx -> experts, ty -> tokens
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    const int lr = threadIdx.x >> 2;          // 0..63: row of the tile this thread loads
    const int lk = (threadIdx.x & 3) * 4;     // 0,4,8,12
    for (int d0 = d_begin; d0 < d_end; d0 += GL_TK) {
        {   // tokens
            int t = t0 + lr;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (t < T) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int d = d0 + lk + i;
                    if (d < d_end) {
                        if (FP8) {
                            const uint8_t* xq = static_cast<const uint8_t*>(x_);
                            __nv_fp8_e4m3 q;
                            q.__x = xq[(size_t)t * D + d];
                            v[i] = __fmul_rn(float(q), xs[(size_t)t * (D / 128) + d / 128]);
                        } else {
                            v[i] = static_cast<const float*>(x_)[(size_t)t * D + d];
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) As[lk + i][lr] = v[i];
        }
        {   // experts
            int e = e0 + lr;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (e < E) {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    int d = d0 + lk + i;
                    if (d < d_end) v[i] = wg[(size_t)e * D + d];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; i++) Bs[lk + i][lr] = v[i];
        }
        __syncthreads();
        const int kmax = min(GL_TK, d_end - d0);
        for (int k = 0; k < kmax; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (FP8) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
                    else     acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int t = t0 + ty * 4 + i;
        if (t >= T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int e = e0 + tx * 4 + j;
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

// smem per warp: E floats (scores s) + E floats (selection scores c)
__global__ void __launch_bounds__(128)
route_select_kernel(const float* __restrict__ partials, int n_chunks, const float* __restrict__ bias,
                    int* __restrict__ ids, float* __restrict__ wts, int* __restrict__ counts,
                    float* __restrict__ logits_out, int T, int E, int K, int scoring, int n_group,
                    int topk_group, float routed_scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * 2 * E;
    float* c = s + E;

    for (int e = lane; e < E; e += 32) {
        float l = partials[(size_t)t * E + e];
        for (int ch = 1; ch < n_chunks; ch++) l = __fadd_rn(l, partials[((size_t)ch * T + t) * E + e]);
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
    for (int e = lane; e < E; e += 32) {
        float sg = (float)(1.0 / (1.0 + exp(-(double)s[e])));
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
    // top-K experts among kept groups.  Taken experts get c = -inf marker via NaN-free flag array:
    // reuse the sign of s? Keep a separate taken bit by setting c[e] to -FLT_MAX after selection.
    float sum = 0.0f;
    float my_w = 0.0f;      // lane k keeps slot k's unnormalised weight (K <= 32)
    int my_id = -1;
    for (int k = 0; k < K; k++) {
        ValIdx b = {0.0f, -1};
        for (int e = lane; e < E; e += 32)
            if (((keep_mask >> (e / gs)) & 1u) && c[e] != -FLT_MAX) b = better(b, ValIdx{c[e], e});
        b = warp_argmax(b);
        float sv = (b.i >= 0) ? s[b.i] : 0.0f;
        __syncwarp();
        if (lane == 0 && b.i >= 0) c[b.i] = -FLT_MAX;
        __syncwarp();
        sum = __fadd_rn(sum, sv);
        if (lane == k) { my_w = sv; my_id = b.i; }
    }
    if (lane < K) {
        oi[lane] = my_id;
        ow[lane] = __fmul_rn(__fdiv_rn(my_w, sum), routed_scale);
        if (counts && my_id >= 0) atomicAdd(&counts[my_id], 1);
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

__global__ void __launch_bounds__(256)
permute_kernel(const int* __restrict__ ids, int TK, int K, int E, int* __restrict__ counts,
               int* __restrict__ offsets, int* __restrict__ row_pair) {
    __shared__ int warp_sums[8];
    __shared__ int s_base;
    const int e = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // pass 1: rows owned by lower experts
    int lt = 0;
    for (int p = threadIdx.x; p < TK; p += 256) {
        int id = ids[p];
        if (id >= 0 && id < e && pair_selects(ids, p, K, id)) lt++;
    }
    for (int o = 16; o > 0; o >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, o);
    if (lane == 0) warp_sums[warp] = lt;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < 8; w++) tot += warp_sums[w];
        s_base = tot;
    }
    __syncthreads();
    const int base = s_base;
    // pass 2: stable ranks of this expert's pairs (ascending pair id = ascending token)
    int running = 0;
    for (int p0 = 0; p0 < TK; p0 += 256) {
        int p = p0 + threadIdx.x;
        bool f = (p < TK) && pair_selects(ids, p, K, e);
        unsigned bal = __ballot_sync(0xffffffffu, f);
        __syncthreads();                      // previous iteration's readers are done
        if (lane == 0) warp_sums[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < 8; w++) {
            int v = warp_sums[w];
            if (w < warp) before += v;
            total += v;
        }
        if (f) row_pair[base + running + before + __popc(bal & ((1u << lane) - 1))] = p;
        running += total;
    }
    if (threadIdx.x == 0) {
        counts[e] = running;
        offsets[e] = base;
        if (e == E - 1) offsets[E] = base + running;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int moe_gate_chunks(int D, bool fp8) { return fp8 ? ceil_div(D, MOE_GATE_CHUNK) : 1; }

int launch_gate_logits(const void* x, const float* xs, const float* wg, float* partials, int T, int E, int D,
                       bool fp8, cudaStream_t stream) {
    int chunk = fp8 ? MOE_GATE_CHUNK : D;
    dim3 grid(ceil_div(T, GL_TM), ceil_div(E, GL_TN), moe_gate_chunks(D, fp8));
    if (fp8) gate_logits_kernel<true><<<grid, 256, 0, stream>>>(x, xs, wg, partials, T, E, D, chunk);
    else     gate_logits_kernel<false><<<grid, 256, 0, stream>>>(x, xs, wg, partials, T, E, D, chunk);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int launch_route_select(const float* partials, int n_chunks, const float* bias, int* ids, float* wts, int* counts,
                        float* logits_out, int T, int E, int K, int scoring, int n_group, int topk_group,
                        float routed_scale, cudaStream_t stream) {
    size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) {
        B200_CUDA_TRY(cudaFuncSetAttribute(route_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)smem));
    }
    route_select_kernel<<<ceil_div(T, 4), 128, smem, stream>>>(partials, n_chunks, bias, ids, wts, counts,
                                                              logits_out, T, E, K, scoring, n_group, topk_group,
                                                              routed_scale);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int launch_permute(const int* ids, int T, int K, int E, int* counts, int* offsets, int* row_pair,
                   cudaStream_t stream) {
    permute_kernel<<<E, 256, 0, stream>>>(ids, T * K, K, E, counts, offsets, row_pair);
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
    const int nch = moe_gate_chunks(D, true);
    WsCarver sz(nullptr);
    sz.take<float>((size_t)nch * T * E);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    float* partials = cv.take<float>((size_t)nch * T * E);
    if (counts) B200_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * E, stream));
    st = launch_gate_logits(xq, xs, gate_w, partials, T, E, D, true, stream);
    if (st) return st;
    return launch_route_select(partials, nch, bias, expert_ids, expert_w, counts, logits_out, T, E, K, cfg->scoring,
                               cfg->n_group, cfg->topk_group, cfg->routed_scale, stream);
}

int b200_moe_permute(b200_ws*, const int* expert_ids, int T, int K, int E, int* counts, int* offsets,
                     int* row_pair, b200_stream_t stream) {
    if (!expert_ids || !counts || !offsets || !row_pair) return B200_BAD_ARG;
    if (T <= 0 || K <= 0 || E <= 0) return B200_BAD_SHAPE;
    return launch_permute(expert_ids, T, K, E, counts, offsets, row_pair, stream);
}

}  // extern "C"
