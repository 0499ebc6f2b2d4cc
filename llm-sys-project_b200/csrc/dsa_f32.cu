// DSA / MLA sparse decode, fp32, any shape: ONE kernel does what the reference spreads
// over eight launches and three materialised buffers (kernels/dsa/naive_dsa.cu:435-474):
// the three row gathers (:13-59), the 576-wide fused dot (:208-273), the scale (:321-324),
// the softmax (:278-294, here online) and the output projection (:300-316).
//
// Block = 8 warps = 8 heads of one query.  A tile of up to 32 selected rows (K = [Kc|Kp]
// and V) is staged in shared memory once and reused by the 8 heads; within a warp the
// lane is the row while scoring and the output column while accumulating P*V.
// Offsets are 64-bit; every listed index contributes (duplicates twice), any order.
#include <cfloat>

#include "common.cuh"

void b200_count_launch(int n);

#define DSA_HB 8

template <int NJ>   // output columns per lane: Dc <= 32 * NJ
__global__ void __launch_bounds__(DSA_HB * 32)
dsa_fused_f32_kernel(const float* __restrict__ q_nope, const float* __restrict__ q_pe,
                     const float* __restrict__ kc, const float* __restrict__ kp, const float* __restrict__ v,
                     const int* __restrict__ idx, float* __restrict__ out,
                     int H, int Dc, int Dp, int S, int TS, float scale, int N) {
    extern __shared__ float sm[];
    const int Dk = Dc + Dp;
    const int ldk = Dk | 1;                       // odd row stride: lanes hit distinct banks
    float* qs = sm;                               // [DSA_HB][Dk]
    float* ks = qs + DSA_HB * Dk;                 // [TS][ldk]
    float* vs = ks + (size_t)TS * ldk;            // [TS][Dc]
    float* ps = vs + (size_t)TS * Dc;             // [DSA_HB][32]
    __shared__ long long row_id[32];

    const int q = blockIdx.x;
    const int h0 = blockIdx.y * DSA_HB;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = h0 + warp;
    const bool head_ok = h < H;

    for (int i = threadIdx.x; i < DSA_HB * Dk; i += blockDim.x) {
        int hh = i / Dk, d = i % Dk;
        float val = 0.0f;
        if (h0 + hh < H)
            val = (d < Dc) ? q_nope[((size_t)q * H + h0 + hh) * Dc + d]
                           : q_pe[((size_t)q * H + h0 + hh) * Dp + (d - Dc)];
        qs[i] = val;
    }

    float m = -FLT_MAX, l = 0.0f;
    float acc[NJ];
#pragma unroll
    for (int j = 0; j < NJ; j++) acc[j] = 0.0f;

    for (int s0 = 0; s0 < S; s0 += TS) {
        const int rows = min(TS, S - s0);
        __syncthreads();                          // previous tile fully consumed (and qs visible)
        // an index that is negative or, when the cache size N is given, not below N is an empty entry: it
        // is not read and contributes nothing (the reference reads it unchecked, kernels/dsa/naive_dsa.cu:19-24)
        if (threadIdx.x < rows) {
            const int id = idx[(size_t)q * S + s0 + threadIdx.x];
            row_id[threadIdx.x] = (id < 0 || (N > 0 && id >= N)) ? -1ll : (long long)id;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < rows * Dk; i += blockDim.x) {
            int r = i / Dk, d = i % Dk;
            long long id = row_id[r];
            ks[(size_t)r * ldk + d] = id < 0 ? 0.0f : ((d < Dc) ? kc[id * Dc + d] : kp[id * Dp + (d - Dc)]);
        }
        for (int i = threadIdx.x; i < rows * Dc; i += blockDim.x) {
            int r = i / Dc, d = i % Dc;
            vs[(size_t)r * Dc + d] = row_id[r] < 0 ? 0.0f : v[row_id[r] * Dc + d];
        }
        __syncthreads();

        // scores: lane = row
        float sc = -FLT_MAX;
        const bool row_live = lane < rows && row_id[lane] >= 0;
        if (row_live) {
            const float* kr = ks + (size_t)lane * ldk;
            const float* qr = qs + warp * Dk;
            float sum = 0.0f;
            for (int d = 0; d < Dk; d++) sum = fmaf(qr[d], kr[d], sum);
            sc = sum * scale;
        }
        float tile_max = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, o));
        const float m_new = fmaxf(m, tile_max);
        const float corr = expf(m - m_new);       // first tile: exp(-huge) = 0, acc and l are 0 anyway
        const float p = row_live ? expf(sc - m_new) : 0.0f;
        float psum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
        l = l * corr + psum;
        m = m_new;
        ps[warp * 32 + lane] = p;
        __syncwarp();
        // P*V: lane = output column (d = lane + 32 j)
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            int d = lane + 32 * j;
            if (d < Dc) {
                float a = acc[j] * corr;
                for (int r = 0; r < rows; r++) a = fmaf(ps[warp * 32 + r], vs[(size_t)r * Dc + d], a);
                acc[j] = a;
            }
        }
    }
    if (head_ok) {
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;      // every entry empty: zero row
#pragma unroll
        for (int j = 0; j < NJ; j++) {
            int d = lane + 32 * j;
            if (d < Dc) out[((size_t)q * H + h) * Dc + d] = acc[j] * inv;
        }
    }
}

// ---------------------------------------------------------------------------
// stage kernels (the reference's per-stage launchers)
// ---------------------------------------------------------------------------
__global__ void gather_rows_f32_kernel(const float* __restrict__ src, const int* __restrict__ idx,
                                       float* __restrict__ dst, long long total, int Dm) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < total; i += stride) {
        long long pair = i / Dm;
        int d = (int)(i % Dm);
        dst[i] = src[(long long)idx[pair] * Dm + d];
    }
}

// scores[q,h,s] += q_nope . g_kc + q_pe . g_kp  (either part optional)
__global__ void dot_rows_f32_kernel(const float* __restrict__ qn, const float* __restrict__ qp,
                                    const float* __restrict__ gkc, const float* __restrict__ gkp,
                                    float* scores, int Q, int H, int S, int Dc, int Dp) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = (long long)Q * H * S;
    if (i >= total) return;
    int s = (int)(i % S);
    int h = (int)((i / S) % H);
    int q = (int)(i / ((long long)S * H));
    float sum = 0.0f;
    if (qn && gkc) {
        const float* a = qn + ((size_t)q * H + h) * Dc;
        const float* b = gkc + ((size_t)q * S + s) * Dc;
        for (int d = 0; d < Dc; d++) sum = fmaf(a[d], b[d], sum);
    }
    if (qp && gkp) {
        const float* a = qp + ((size_t)q * H + h) * Dp;
        const float* b = gkp + ((size_t)q * S + s) * Dp;
        for (int d = 0; d < Dp; d++) sum = fmaf(a[d], b[d], sum);
    }
    scores[i] += sum;
}

// one warp per (q,h) row
__global__ void softmax_rows_f32_kernel(float* scores, long long rows, int S) {
    long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (row >= rows) return;
    float* r = scores + row * S;
    float mx = -FLT_MAX;
    for (int s = lane; s < S; s += 32) mx = fmaxf(mx, r[s]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    for (int s = lane; s < S; s += 32) { float e = expf(r[s] - mx); r[s] = e; sum += e; }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float inv = 1.0f / sum;
    for (int s = lane; s < S; s += 32) r[s] *= inv;
}

__global__ void output_proj_f32_kernel(const float* __restrict__ attn, const float* __restrict__ gv,
                                       float* __restrict__ out, int Q, int H, int S, int Dc) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = (long long)Q * H * Dc;
    if (i >= total) return;
    int d = (int)(i % Dc);
    int h = (int)((i / Dc) % H);
    int q = (int)(i / ((long long)Dc * H));
    const float* a = attn + ((size_t)q * H + h) * S;
    const float* vv = gv + (size_t)q * S * Dc + d;
    float sum = 0.0f;
    for (int s = 0; s < S; s++) sum = fmaf(a[s], vv[(size_t)s * Dc], sum);
    out[i] = sum;
}

static int check_dsa(const b200_dsa_config* c) {
    if (!c) return B200_BAD_ARG;
    if (c->num_queries <= 0 || c->num_heads <= 0 || c->head_dim_compressed <= 0 || c->head_dim_positional < 0 ||
        c->num_selected_kv <= 0)
        return B200_BAD_SHAPE;
    return B200_OK;
}

template <int NJ>
static int launch_dsa_f32(const float* qn, const float* qp, const float* kc, const float* kp, const float* v,
                          const int* idx, float* out, const b200_dsa_config* c, size_t smem_limit,
                          cudaStream_t stream) {
    const int Dc = c->head_dim_compressed, Dp = c->head_dim_positional, Dk = Dc + Dp;
    int TS = 32;
    auto need = [&](int ts) {
        return sizeof(float) * ((size_t)DSA_HB * Dk + (size_t)ts * (Dk | 1) + (size_t)ts * Dc + DSA_HB * 32);
    };
    while (TS > 1 && need(TS) > smem_limit) TS >>= 1;
    if (need(TS) > smem_limit) return B200_UNSUPPORTED;
    size_t smem = need(TS);
    B200_CUDA_TRY(cudaFuncSetAttribute(dsa_fused_f32_kernel<NJ>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
    dim3 grid(c->num_queries, ceil_div(c->num_heads, DSA_HB));
    float scale = 1.0f / sqrtf((float)Dk);        // naive_dsa.cu:464
    dsa_fused_f32_kernel<NJ><<<grid, DSA_HB * 32, smem, stream>>>(qn, qp, kc, kp, v, idx, out, c->num_heads, Dc, Dp,
                                                                   c->num_selected_kv, TS, scale, c->total_kv_tokens);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" {

int b200_dsa_forward_f32(b200_ws* ws, const float* q_nope, const float* q_pe, const float* kc, const float* kp,
                         const float* v, const int* idx, float* out, const b200_dsa_config* cfg,
                         b200_stream_t stream) {
    int st = check_dsa(cfg);
    if (st) return st;
    if (!q_nope || !kc || !v || !idx || !out) return B200_BAD_ARG;
    if (cfg->head_dim_positional > 0 && (!q_pe || !kp)) return B200_BAD_ARG;
    if (cfg->num_queries > 0x7fffffff / 1 || ceil_div(cfg->num_heads, DSA_HB) > 65535) return B200_UNSUPPORTED;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    const size_t lim = ws->max_smem_optin - 1024;
    const int Dc = cfg->head_dim_compressed;
    if (Dc <= 32) return launch_dsa_f32<1>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    if (Dc <= 64) return launch_dsa_f32<2>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    if (Dc <= 128) return launch_dsa_f32<4>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    if (Dc <= 256) return launch_dsa_f32<8>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    if (Dc <= 512) return launch_dsa_f32<16>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    if (Dc <= 1024) return launch_dsa_f32<32>(q_nope, q_pe, kc, kp, v, idx, out, cfg, lim, stream);
    return B200_UNSUPPORTED;
}

int b200_dsa_kv_gather_f32(const float* kc, const float* kp, const float* v, const int* idx, float* g_kc, float* g_kp,
                           float* g_v, const b200_dsa_config* cfg, b200_stream_t stream) {
    int st = check_dsa(cfg);
    if (st) return st;
    if (!idx) return B200_BAD_ARG;
    const long long pairs = (long long)cfg->num_queries * cfg->num_selected_kv;
    const int Dc = cfg->head_dim_compressed, Dp = cfg->head_dim_positional;
    auto run = [&](const float* src, float* dst, int Dm) {
        if (!src || !dst || Dm <= 0) return;
        long long total = pairs * Dm;
        long long blocks = (total + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        gather_rows_f32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(src, idx, dst, total, Dm);
        b200_count_launch(1);
    };
    run(kc, g_kc, Dc);
    run(kp, g_kp, Dp);
    run(v, g_v, Dc);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_dsa_dot_f32(const float* q_nope, const float* q_pe, const float* g_kc, const float* g_kp, float* scores,
                     const b200_dsa_config* cfg, b200_stream_t stream) {
    int st = check_dsa(cfg);
    if (st) return st;
    if (!scores) return B200_BAD_ARG;
    long long total = (long long)cfg->num_queries * cfg->num_heads * cfg->num_selected_kv;
    long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_UNSUPPORTED;
    dot_rows_f32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(q_nope, q_pe, g_kc, g_kp, scores, cfg->num_queries,
                                                             cfg->num_heads, cfg->num_selected_kv,
                                                             cfg->head_dim_compressed, cfg->head_dim_positional);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_dsa_softmax_f32(float* scores, const b200_dsa_config* cfg, b200_stream_t stream) {
    int st = check_dsa(cfg);
    if (st) return st;
    if (!scores) return B200_BAD_ARG;
    long long rows = (long long)cfg->num_queries * cfg->num_heads;
    long long blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffffLL) return B200_UNSUPPORTED;
    softmax_rows_f32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(scores, rows, cfg->num_selected_kv);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_dsa_output_proj_f32(const float* attn, const float* g_v, float* out, const b200_dsa_config* cfg,
                             b200_stream_t stream) {
    int st = check_dsa(cfg);
    if (st) return st;
    if (!attn || !g_v || !out) return B200_BAD_ARG;
    long long total = (long long)cfg->num_queries * cfg->num_heads * cfg->head_dim_compressed;
    long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_UNSUPPORTED;
    output_proj_f32_kernel<<<(unsigned)blocks, 256, 0, stream>>>(attn, g_v, out, cfg->num_queries, cfg->num_heads,
                                                                cfg->num_selected_kv, cfg->head_dim_compressed);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"
