// fp32 MoE layer (the reference's own data types): routing + permutation from
// moe_route.cu, then two grouped GEMM launches that cover every expert at once.
//
//   grouped_gemm1_f32  act[r, j] = silu(x_r . W1e[j]) * (x_r . W1e[I+j])   (SwiGLU fused;
//                      replaces tiled_gemm_bt_kernel + swiglu_strided_kernel,
//                      kernels/moe/naive_moe.cu:246-280, :297-310, called per expert at :437-455)
//   grouped_gemm2_f32  out[t, n] += w(t,e) * (act_r . W2e[n])             (router weight and
//                      scatter-add fused; replaces tiled_gemm_bt_kernel + scatter_kernel,
//                      naive_moe.cu:458-468, :315-335)
// Rows are addressed through the row -> (token, slot) map, so no gathered copy of the
// activations is made and the host never learns the per-expert counts.
#include "common.cuh"
#include "moe_internal.cuh"

#define G_TM 32   // rows per tile
#define G_TN 32   // output columns per tile
#define G_TK 32

// grid: (ceil(N/G_TN), ceil(T/G_TM), E); tiles beyond an expert's row count exit at once.
template <int MODE>   // 1: GEMM1 + SwiGLU, 2: GEMM2 + weighted scatter-add
__global__ void __launch_bounds__(256)
grouped_gemm_f32_kernel(const float* __restrict__ a_src,     // MODE 1: x [T,D];  MODE 2: act [rows,I]
                        const float* __restrict__ w,         // MODE 1: W1 [E,2I,D]; MODE 2: W2 [E,D,I]
                        const int* __restrict__ offsets, const int* __restrict__ row_pair,
                        const float* __restrict__ wts, float* __restrict__ dst,
                        int K, int D, int I) {
    const int e = blockIdx.z;
    const int row0 = offsets[e], cnt = offsets[e + 1] - row0;
    const int m0 = blockIdx.y * G_TM;
    if (m0 >= cnt) return;
    const int n0 = blockIdx.x * G_TN;
    const int Kdim = (MODE == 1) ? D : I;      // reduction length
    const int Ncols = (MODE == 1) ? I : D;     // output columns

    __shared__ float As[G_TK][G_TM + 1];
    __shared__ float Bs[(MODE == 1) ? 2 : 1][G_TK][G_TN + 1];
    __shared__ long long a_row_off[G_TM];
    __shared__ int s_tok[G_TM];
    __shared__ float s_w[G_TM];

    if (threadIdx.x < G_TM) {
        int m = m0 + threadIdx.x;
        long long off = -1;
        int tok = 0; float wv = 0.0f;
        if (m < cnt) {
            int pair = row_pair[row0 + m];
            tok = pair / K;
            wv = wts ? wts[pair] : 0.0f;
            off = (MODE == 1) ? (long long)tok * D : (long long)(row0 + m) * I;
        }
        a_row_off[threadIdx.x] = off;
        s_tok[threadIdx.x] = tok;
        s_w[threadIdx.x] = wv;
    }
    __syncthreads();

    const float* we = w + (size_t)e * ((MODE == 1) ? (size_t)2 * I * D : (size_t)D * I);
    const int tx = threadIdx.x & 31;   // output column
    const int ty = threadIdx.x >> 5;   // 0..7 -> rows ty, ty+8, ty+16, ty+24
    float acc[2][4];
#pragma unroll
    for (int h = 0; h < 2; h++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[h][i] = 0.0f;

    for (int k0 = 0; k0 < Kdim; k0 += G_TK) {
        // 256 threads load 32x32 tiles: thread -> (row = tid/8, 4 consecutive k)
        {
            int r = threadIdx.x >> 3, kk = (threadIdx.x & 7) * 4;
            long long off = a_row_off[r];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int k = k0 + kk + i;
                As[kk + i][r] = (off >= 0 && k < Kdim) ? a_src[off + k] : 0.0f;
            }
            int n = n0 + r;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int k = k0 + kk + i;
                bool ok = (n < Ncols) && (k < Kdim);
                Bs[0][kk + i][r] = ok ? we[(size_t)n * Kdim + k] : 0.0f;
                if (MODE == 1) Bs[1][kk + i][r] = ok ? we[(size_t)(I + n) * Kdim + k] : 0.0f;
            }
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < G_TK; k++) {
            float b0 = Bs[0][k][tx];
            float b1 = (MODE == 1) ? Bs[1][k][tx] : 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float a = As[k][ty + 8 * i];
                acc[0][i] = fmaf(a, b0, acc[0][i]);
                if (MODE == 1) acc[1][i] = fmaf(a, b1, acc[1][i]);
            }
        }
        __syncthreads();
    }

    const int n = n0 + tx;
    if (n >= Ncols) return;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int ml = ty + 8 * i;
        if (m0 + ml >= cnt) continue;
        if (MODE == 1) {
            float g = acc[0][i], u = acc[1][i];
            float sg = __fdiv_rn(g, 1.0f + expf(-g));      // silu as naive_moe.cu:308
            dst[(size_t)(row0 + m0 + ml) * I + n] = sg * u;
        } else {
            atomicAdd(&dst[(size_t)s_tok[ml] * D + n], s_w[ml] * acc[0][i]);
        }
    }
}

// ---------------------------------------------------------------------------
// stage kernels (the reference's per-stage launchers; not on the fused path)
// ---------------------------------------------------------------------------
// naive_moe.cu:147-166 semantics, block-parallel: ascending token order kept by a
// ballot scan; rows copied by the whole block.
__global__ void __launch_bounds__(256)
gather_one_expert_kernel(const float* __restrict__ x, const int* __restrict__ ids, int expert, float* gathered,
                         int* token_map, int* count, int T, int K, int D) {
    __shared__ int warp_sums[8];
    __shared__ int s_running;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) s_running = 0;
    __syncthreads();
    for (int t0 = 0; t0 < T; t0 += 256) {
        int t = t0 + threadIdx.x;
        bool f = false;
        if (t < T)
            for (int k = 0; k < K; k++)
                if (ids[(size_t)t * K + k] == expert) { f = true; break; }
        unsigned bal = __ballot_sync(0xffffffffu, f);
        if (lane == 0) warp_sums[warp] = __popc(bal);
        __syncthreads();
        int before = s_running, total = 0;
        for (int w = 0; w < 8; w++) {
            if (w < warp) before += warp_sums[w];
            total += warp_sums[w];
        }
        if (f) token_map[before + __popc(bal & ((1u << lane) - 1))] = t;
        __syncthreads();
        if (threadIdx.x == 0) s_running += total;
        __syncthreads();
    }
    const int cnt = s_running;
    if (threadIdx.x == 0) *count = cnt;
    __threadfence_block();
    __syncthreads();
    for (long long i = threadIdx.x; i < (long long)cnt * D; i += 256) {
        int r = (int)(i / D), d = (int)(i % D);
        gathered[i] = x[(size_t)token_map[r] * D + d];
    }
}

// naive_moe.cu:205-238 (C = A * B, row-major)
__global__ void __launch_bounds__(256) gemm_nn_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                          float* __restrict__ C, int M, int N, int Kd) {
    __shared__ float As[16][17], Bs[16][17];
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    int row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
    float sum = 0.0f;
    for (int k0 = 0; k0 < Kd; k0 += 16) {
        As[ty][tx] = (row < M && k0 + tx < Kd) ? A[(size_t)row * Kd + k0 + tx] : 0.0f;
        Bs[ty][tx] = (k0 + ty < Kd && col < N) ? B[(size_t)(k0 + ty) * N + col] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 16; i++) sum = fmaf(As[ty][i], Bs[i][tx], sum);
        __syncthreads();
    }
    if (row < M && col < N) C[(size_t)row * N + col] = sum;
}

// naive_moe.cu:285-292
__global__ void swiglu_f32_kernel(const float* gate, const float* up, float* out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float g = gate[i];
    out[i] = __fdiv_rn(g, 1.0f + expf(-g)) * up[i];
}

// naive_moe.cu:315-335, any D (grid.y tiles the columns)
__global__ void scatter_f32_kernel(const float* __restrict__ expert_out, const int* __restrict__ token_map,
                                   const float* __restrict__ wts, const int* __restrict__ ids, int expert,
                                   float* out, int count, int K, int D) {
    int i = blockIdx.x;
    int d = blockIdx.y * blockDim.x + threadIdx.x;
    if (i >= count || d >= D) return;
    int t = token_map[i];
    float w = 0.0f;
    for (int k = 0; k < K; k++)
        if (ids[(size_t)t * K + k] == expert) { w = wts[(size_t)t * K + k]; break; }
    atomicAdd(&out[(size_t)t * D + d], w * expert_out[(size_t)i * D + d]);
}

extern "C" {

int b200_moe_forward_f32(b200_ws* ws, const float* x, const float* gate_w, const float* w1, const float* w2,
                         float* out, const b200_moe_config* cfg, b200_stream_t stream) {
    if (!x || !gate_w || !w1 || !w2 || !out || !cfg) return B200_BAD_ARG;
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim,
              I = cfg->intermediate_dim;
    int st = check_route_cfg(T, E, K, D, B200_SCORE_SOFTMAX, 1, 1);
    if (st) return st;
    if (I <= 0) return B200_BAD_SHAPE;
    if (E > 65535 || ceil_div(T, G_TM) > 65535) return B200_UNSUPPORTED;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;

    auto carve = [&](WsCarver& c, float*& partials, int*& ids, float*& wts, int*& counts, int*& offsets,
                     int*& row_pair, float*& act) {
        partials = c.take<float>((size_t)T * E);
        ids = c.take<int>((size_t)T * K);
        wts = c.take<float>((size_t)T * K);
        counts = c.take<int>(E);
        offsets = c.take<int>(E + 1);
        row_pair = c.take<int>((size_t)T * K);
        act = c.take<float>((size_t)T * K * I);
    };
    float *partials, *wts, *act; int *ids, *counts, *offsets, *row_pair;
    WsCarver sz(nullptr);
    carve(sz, partials, ids, wts, counts, offsets, row_pair, act);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    carve(cv, partials, ids, wts, counts, offsets, row_pair, act);

    st = launch_gate_logits(x, nullptr, gate_w, partials, T, E, D, false, stream);
    if (st) return st;
    st = launch_route_select(partials, 1, nullptr, ids, wts, nullptr, nullptr, T, E, K, B200_SCORE_SOFTMAX, 1, 1,
                             1.0f, stream);
    if (st) return st;
    st = launch_permute(ids, T, K, E, nullptr, true, counts, offsets, row_pair, stream);
    if (st) return st;
    B200_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)T * D, stream));   // naive_moe.cu:413
    dim3 g1(ceil_div(I, G_TN), ceil_div(T, G_TM), E);
    grouped_gemm_f32_kernel<1><<<g1, 256, 0, stream>>>(x, w1, offsets, row_pair, nullptr, act, K, D, I);
    dim3 g2(ceil_div(D, G_TN), ceil_div(T, G_TM), E);
    grouped_gemm_f32_kernel<2><<<g2, 256, 0, stream>>>(act, w2, offsets, row_pair, wts, out, K, D, I);
    b200_count_launch(2);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_moe_gather_f32(const float* x, const int* expert_ids, int expert_id, float* gathered, int* token_map,
                        int* count, const b200_moe_config* cfg, b200_stream_t stream) {
    if (!x || !expert_ids || !gathered || !token_map || !count || !cfg) return B200_BAD_ARG;
    gather_one_expert_kernel<<<1, 256, 0, stream>>>(x, expert_ids, expert_id, gathered, token_map, count,
                                                    cfg->num_tokens, cfg->top_k, cfg->hidden_dim);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, b200_stream_t stream) {
    if (!A || !B || !C) return B200_BAD_ARG;
    if (M <= 0 || N <= 0 || K <= 0) return B200_BAD_SHAPE;
    dim3 grid(ceil_div(N, 16), ceil_div(M, 16));
    gemm_nn_f32_kernel<<<grid, 256, 0, stream>>>(A, B, C, M, N, K);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_swiglu_f32(const float* gate, const float* up, float* out, int n, b200_stream_t stream) {
    if (!gate || !up || !out) return B200_BAD_ARG;
    if (n <= 0) return n == 0 ? B200_OK : B200_BAD_SHAPE;
    swiglu_f32_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(gate, up, out, n);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_moe_scatter_f32(const float* expert_out, const int* token_map, const float* expert_w, const int* expert_ids,
                         int expert_id, float* out, int count, const b200_moe_config* cfg, b200_stream_t stream) {
    if (!cfg) return B200_BAD_ARG;
    if (count == 0) return B200_OK;                  // naive_moe.cu:388
    if (!expert_out || !token_map || !expert_w || !expert_ids || !out) return B200_BAD_ARG;
    dim3 grid(count, ceil_div(cfg->hidden_dim, 256));
    scatter_f32_kernel<<<grid, 256, 0, stream>>>(expert_out, token_map, expert_w, expert_ids, expert_id, out, count,
                                                 cfg->top_k, cfg->hidden_dim);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"
