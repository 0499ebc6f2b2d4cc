// Router logits of the FP8 layer on the tensor cores (tcgen05, kind::tf32), for the token counts where the
// fixed-order FMA kernel of moe_route.cu costs a tenth of the layer.
//
// The reference's gate (kernels/moe/naive_moe.cu:87-107) and this library's exact kernels define a logit as
// one fused multiply-add chain over d in a fixed order; a tensor core sums in its own order, so what this
// file computes is an APPROXIMATION of those logits, good to about 2e-5.  The routing decisions stay exact all
// the same: the selection kernel (moe_route.cu) accepts a token only if every decision margin (kept groups,
// the order of the K selected experts, the K-th against the (K+1)-th) is far larger than the approximation
// error, and recomputes the others with the exact kernels.
//
//     logit[t,e] = sum_d (e4m3(xq[t,d]) * xs[t,d/128]) * wg[e,d]
//
// Both factors are fp32 values; tf32 keeps 11 significant bits, so each is split into a high part (the
// fp32 value with its low 13 mantissa bits cleared) and a low part (the exact difference), and the product is
// taken as hi*hi + hi*lo + lo*hi (the dropped lo*lo term and the bits below the low parts are ~2^-22 of
// the product).  Everything accumulates in one 128 x N fp32 TMEM tile across the CTA's whole range of d: no
// per-block rescaling is needed because the activation scale is folded into the A operand.  The tensor core
// truncates when it adds a product into the fp32 accumulator, so the error grows with the length of the chain
// (one chain over d = 7168: 2.4e-4; chains of 512: 2.1e-5): a CTA covers at most four 128-deep blocks of d, and
// the selection kernel adds the CTAs' partial sums with ordinary fp32 additions.
//
//   wsplit_kernel        wg -> (hi, lo), once per call (the weights are a caller-owned buffer that may change)
//   gate_tc_kernel       CTA = 128 tokens x all experts x 512 of d; warps 0-3 dequantise and split the
//                        token rows into the swizzled A tiles (and read the accumulator out at the end), warp
//                        4 fetches the weight tiles by TMA, warp 5 issues the MMAs; two 32-wide stages.
// Every mbarrier wait is bounded; on give-up the CTA flags B200_TIMEOUT and winds down.
#include "common.cuh"
#include "moe_internal.cuh"
#include "selftest.h"
#include "tma_host.cuh"

namespace {

constexpr int TM = 128;              // tokens per CTA (TMEM lanes)
constexpr int KS = 32;               // d per stage: 128 bytes of tf32 = one swizzle row
constexpr int NSTAGE = 2;
constexpr int A_TILE = TM * KS * 4;  // 16384 bytes (hi or lo)
constexpr int TC_THREADS = 192;
constexpr int MAX_N = 256;

struct TcSmem {
    uint64_t a_full[NSTAGE], b_full[NSTAGE], empty[NSTAGE], done;
    uint32_t tmem_base;
    int abort_flag;
};

__global__ void wsplit_kernel(const float* __restrict__ w, float* __restrict__ hi, float* __restrict__ lo, long long n) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) {
        const float x = w[i];
        const float h = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
        hi[i] = h;
        lo[i] = __fsub_rn(x, h);          // exact: the low 13 mantissa bits of x
    }
}

__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// partials[(split * T + t) * E + e] = sum over the split's d of x[t,d] * w[e,d]
__global__ void __launch_bounds__(TC_THREADS, 1)
gate_tc_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo,
               const uint8_t* __restrict__ xq, const float* __restrict__ xs, float* __restrict__ partials, int T, int E,
               int D, int N, int kb_per_split, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_tile = N * KS * 4;                                  // bytes of one weight tile (hi or lo)
    const int stage_bytes = 2 * A_TILE + 2 * b_tile;
    TcSmem* sm = reinterpret_cast<TcSmem*>(base + (size_t)NSTAGE * stage_bytes);
    volatile int* abort_flag = &sm->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * TM, split = blockIdx.y;
    const int nb = D / 128;
    const int kb0 = split * kb_per_split, kb1 = min(nb, kb0 + kb_per_split);
    const int nstages = max(0, kb1 - kb0) * (128 / KS);
    const int d_begin = kb0 * 128;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            ptx::mbar_init(&sm->a_full[s], 128);
            ptx::mbar_init(&sm->b_full[s], 1);
            ptx::mbar_init(&sm->empty[s], 1);
        }
        ptx::mbar_init(&sm->done, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 5) {
        ptx::tmem_alloc(&sm->tmem_base, 256);
        ptx::tmem_relinquish();
    }
    if (warp == 4 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_hi);
        ptx::prefetch_tensormap(&tmap_lo);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (warp < 4) {
        // ===================== A tiles: dequantise, split, swizzle (thread = token row) =====================
        const int r = threadIdx.x;
        const int t = t0 + r;
        const uint8_t* xrow = xq + (size_t)min(t, T - 1) * D;
        const float* srow = xs + (size_t)min(t, T - 1) * nb;
        const bool live = t < T;
        for (int i = 0; i < nstages; i++) {
            const int s = i % NSTAGE;
            const uint32_t par = (uint32_t)((i / NSTAGE) & 1);
            const int d0 = d_begin + i * KS;
            // fetch before waiting for the slot
            const uint4 q0 = *reinterpret_cast<const uint4*>(xrow + d0);
            const uint4 q1 = *reinterpret_cast<const uint4*>(xrow + d0 + 16);
            const float sc = live ? srow[d0 / 128] : 0.0f;
            if (!ptx::mbar_wait(&sm->empty[s], par ^ 1, abort_flag)) goto done;
            {
            const uint32_t a_hi = ptx::smem_u32(base + (size_t)s * stage_bytes) + r * 128;
            const uint32_t a_lo = a_hi + A_TILE;
            const uint32_t words[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int j = 0; j < 8; j++) {                       // 16-byte chunk j = 4 consecutive d
                float h[4], l[4];
#pragma unroll
                for (int b = 0; b < 4; b++) {
                    __nv_fp8_e4m3 q;
                    q.__x = (unsigned char)((words[j] >> (8 * b)) & 0xFF);
                    // the dequantised activation, as the exact kernels form it (rows beyond T: zero)
                    const float x = live ? __fmul_rn(float(q), sc) : 0.0f;
                    h[b] = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
                    l[b] = __fsub_rn(x, h[b]);
                }
                const uint32_t off = (uint32_t)((j ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a_hi + off), "f"(h[0]), "f"(h[1]), "f"(h[2]), "f"(h[3]) : "memory");
                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a_lo + off), "f"(l[0]), "f"(l[1]), "f"(l[2]), "f"(l[3]) : "memory");
            }
            }
            ptx::fence_proxy_async_smem();                      // generic-proxy stores -> visible to the MMA (async proxy)
            ptx::mbar_arrive(&sm->a_full[s]);
        }
        // ---- epilogue: accumulator row -> partial logits ----
        if (!ptx::mbar_wait(&sm->done, 0, abort_flag)) goto done;
        ptx::tc_fence_after();
        {
            const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
            float* dst = partials + ((size_t)split * T + t) * E;
            for (int c0 = 0; c0 < N; c0 += 32) {
                uint32_t v[32];
                if (nstages > 0) {
                    ptx::tmem_ld_32x32(tmem + lane_addr + c0, v);
                    ptx::tc_wait_ld();
                } else {
#pragma unroll
                    for (int k = 0; k < 32; k++) v[k] = 0;
                }
                if (live) {
#pragma unroll
                    for (int k = 0; k < 32; k += 4)
                        if (c0 + k < E)          // E % 4 == 0
                            *reinterpret_cast<float4*>(dst + c0 + k) =
                                make_float4(__uint_as_float(v[k]), __uint_as_float(v[k + 1]), __uint_as_float(v[k + 2]),
                                            __uint_as_float(v[k + 3]));
                }
            }
        }
    } else if (warp == 4) {
        // ===================== weight tiles by TMA =====================
        if (lane == 0) {
            for (int i = 0; i < nstages; i++) {
                const int s = i % NSTAGE;
                const uint32_t par = (uint32_t)((i / NSTAGE) & 1);
                if (!ptx::mbar_wait_relaxed(&sm->empty[s], par ^ 1, abort_flag, 100)) goto done;
                uint8_t* bh = base + (size_t)s * stage_bytes + 2 * A_TILE;
                ptx::mbar_expect_tx(&sm->b_full[s], 2 * b_tile);
                ptx::tma_load_2d(bh, &tmap_hi, &sm->b_full[s], d_begin + i * KS, 0);
                ptx::tma_load_2d(bh + b_tile, &tmap_lo, &sm->b_full[s], d_begin + i * KS, 0);
            }
        }
    } else {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const uint32_t idesc = ptx::make_idesc(2, 2, 0, 0, TM, N);      // tf32 x tf32 -> f32, both K-major
            for (int i = 0; i < nstages; i++) {
                const int s = i % NSTAGE;
                const uint32_t par = (uint32_t)((i / NSTAGE) & 1);
                if (!ptx::mbar_wait(&sm->a_full[s], par, abort_flag)) goto done;
                if (!ptx::mbar_wait(&sm->b_full[s], par, abort_flag)) goto done;
                ptx::tc_fence_after();
                const uint32_t ah = ptx::smem_u32(base + (size_t)s * stage_bytes), al = ah + A_TILE;
                const uint32_t bh = al + A_TILE, bl = bh + b_tile;
#pragma unroll
                for (int kk = 0; kk < KS / 8; kk++) {              // 8 tf32 = 32 bytes of K per MMA
                    const uint64_t dah = ptx::make_smem_desc(ah + kk * 32, 16, 1024, 2);
                    const uint64_t dal = ptx::make_smem_desc(al + kk * 32, 16, 1024, 2);
                    const uint64_t dbh = ptx::make_smem_desc(bh + kk * 32, 16, 1024, 2);
                    const uint64_t dbl = ptx::make_smem_desc(bl + kk * 32, 16, 1024, 2);
                    mma_tf32(tmem, dah, dbh, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                    mma_tf32(tmem, dah, dbl, idesc, 1u);
                    mma_tf32(tmem, dal, dbh, idesc, 1u);
                }
                ptx::tc_commit(&sm->empty[s]);
            }
            ptx::tc_commit(&sm->done);
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 5) ptx::tmem_dealloc(tmem, 256);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(status, B200_TIMEOUT);
}

// Row-major fp32 matrix [rows, cols], tile = box_rows x 32 floats (128 bytes), 128-byte swizzle.
int make_tmap_f32_sw128(CUtensorMap* map, const void* basep, unsigned long long rows, unsigned long long cols,
                        unsigned box_rows) {
    b200_encode_tiled_fn enc = b200_get_encode_tiled();
    if (!enc) return B200_CUDA_ERROR;
    if ((reinterpret_cast<uintptr_t>(basep) & 15) || (cols & 3) || box_rows == 0 || box_rows > 256) return B200_BAD_ARG;
    cuuint64_t gdim[2] = {cols, rows};
    cuuint64_t gstride[1] = {cols * 4};
    cuuint32_t box[2] = {32, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(basep), gdim, gstride, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? B200_OK : B200_CUDA_ERROR;
}

}  // namespace

bool moe_gate_tc_supported(int T, int E, int D) {
    return T >= 256 && E >= 16 && E <= MAX_N && E % 16 == 0 && D % 128 == 0 && D >= 512;
}
static int g_tc_splits_override = 0;      // set only inside b200_moe_gate_logits_tc (test hook)
int moe_gate_tc_splits(int D) {
    if (g_tc_splits_override > 0) return g_tc_splits_override;
    return ceil_div(D / 128, 4);      // chains of at most four 128-deep blocks: the accumulation error grows with the chain
}

// whi / wlo: E * D floats each (workspace); partials: splits * T * E floats.
int launch_gate_logits_tc(const uint8_t* xq, const float* xs, const float* wg, float* whi, float* wlo, float* partials,
                          int T, int E, int D, int* status, cudaStream_t stream) {
    const long long n = (long long)E * D;
    wsplit_kernel<<<592, 256, 0, stream>>>(wg, whi, wlo, n);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    CUtensorMap th, tl;
    int st = make_tmap_f32_sw128(&th, whi, E, D, E);
    if (st) return st;
    st = make_tmap_f32_sw128(&tl, wlo, E, D, E);
    if (st) return st;
    const int N = E;
    const size_t smem = 1024 + (size_t)NSTAGE * (2 * A_TILE + 2 * (size_t)N * KS * 4) + sizeof(TcSmem) + 64;
    static bool attr_done[64] = {false};
    if (b200_first_call_on_device(attr_done))
        B200_CUDA_TRY(cudaFuncSetAttribute(gate_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(1024 + (size_t)NSTAGE * (2 * A_TILE + 2 * (size_t)MAX_N * KS * 4) + sizeof(TcSmem) + 64)));
    const int splits = moe_gate_tc_splits(D);
    const int kbps = ceil_div(D / 128, splits);
    dim3 grid(ceil_div(T, TM), splits);
    gate_tc_kernel<<<grid, TC_THREADS, smem, stream>>>(th, tl, xq, xs, partials, T, E, D, N, kbps, status);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// Test hook: the tensor-core logits as partial sums [splits, T, E] (the caller adds them up and compares with the
// exact chains).  *splits_out > 0 on entry asks for that many partial sums along D (at most D / 128) instead of
// the library's choice; on return it holds the number written.  Not thread-safe (the override is a global).
extern "C" int b200_moe_gate_logits_tc(const uint8_t* xq, const float* xs, const float* gate_w, float* partials_out,
                                       int T, int E, int D, int* splits_out, b200_stream_t stream) {
    if (!xq || !xs || !gate_w || !partials_out || !splits_out) return B200_BAD_ARG;
    if (!moe_gate_tc_supported(T, E, D)) return B200_UNSUPPORTED;
    g_tc_splits_override = (*splits_out > 0 && *splits_out <= D / 128) ? *splits_out : 0;
    b200_ws* ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    WsCarver sz(nullptr);
    sz.take<float>((size_t)E * D);
    sz.take<float>((size_t)E * D);
    int st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    float* whi = cv.take<float>((size_t)E * D);
    float* wlo = cv.take<float>((size_t)E * D);
    *splits_out = moe_gate_tc_splits(D);
    st = launch_gate_logits_tc(xq, xs, gate_w, whi, wlo, partials_out, T, E, D, ws->d_status, stream);
    g_tc_splits_override = 0;
    return st;
}
