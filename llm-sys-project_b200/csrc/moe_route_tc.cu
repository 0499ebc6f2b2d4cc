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
//   gate_tc_kernel       one persistent CTA per SM over an equal share of the (128-token tile, 128-deep block)
//                        units; warps 0-7 dequantise and split the token rows into the swizzled A tiles (rows
//                        fetched one block ahead), warps 8-11 store finished partial sums from one of two TMEM
//                        accumulators while the other one is being multiplied, warp 12 fetches the weight tiles
//                        by TMA, warp 13 issues the MMAs; two 32-wide stages.
// Every mbarrier wait is bounded; on give-up the CTA flags B200_TIMEOUT and winds down.
#include "common.cuh"
#include "moe_internal.cuh"
#include "selftest.h"
#include "tma_host.cuh"
#include <vector>

namespace {

constexpr int TM = 128;              // tokens per tile (TMEM lanes)
constexpr int KS = 32;               // d per stage: 128 bytes of tf32 = one swizzle row
constexpr int NSTAGE = 2;
constexpr int A_TILE = TM * KS * 4;  // 16384 bytes (hi or lo)
constexpr int TC_THREADS = 448;      // warps 0-7 convert, 8-11 read accumulators out, 12 TMA, 13 MMA
constexpr int MAX_N = 256;
constexpr int TC_CHAIN = 4;          // longest accumulation chain, in 128-deep blocks

struct TcSmem {
    uint64_t a_full[NSTAGE], b_full[NSTAGE], empty[NSTAGE], acc_full[2], acc_empty[2];
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

// Persistent CTA over the units [blockIdx.x * L, (blockIdx.x + 1) * L) of the plan (moe_internal.cuh).  Two
// 256-column accumulators in TMEM alternate between pieces, so that a finished piece is stored while the next
// one is multiplied.
__global__ void __launch_bounds__(TC_THREADS, 1)
gate_tc_kernel(const __grid_constant__ CUtensorMap tmap_hi, const __grid_constant__ CUtensorMap tmap_lo,
               const uint8_t* __restrict__ xq, const float* __restrict__ xs, float* __restrict__ partials, int T, int E,
               int D, int N, TcPlan plan, int n_units, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int b_tile = N * KS * 4;                                  // bytes of one weight tile (hi or lo)
    const int stage_bytes = 2 * A_TILE + 2 * b_tile;
    TcSmem* sm = reinterpret_cast<TcSmem*>(base + (size_t)NSTAGE * stage_bytes);
    volatile int* abort_flag = &sm->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = plan.nblk;
    const int u0 = blockIdx.x * plan.L, u1 = min(n_units, u0 + plan.L);
    constexpr int SPB = 128 / KS;                                   // stages per 128-deep block

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTAGE; s++) {
            ptx::mbar_init(&sm->a_full[s], 256);
            ptx::mbar_init(&sm->b_full[s], 1);
            ptx::mbar_init(&sm->empty[s], 1);
        }
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(&sm->acc_full[s], 1);
            ptx::mbar_init(&sm->acc_empty[s], 128);
        }
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 13) {
        ptx::tmem_alloc(&sm->tmem_base, 512);
        ptx::tmem_relinquish();
    }
    if (warp == 12 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_hi);
        ptx::prefetch_tensormap(&tmap_lo);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (warp < 8) {
        // ===================== A tiles: dequantise, split, swizzle =====================
        // Two threads per token row, 16 of a stage's 32 d each; the row's bytes of one 128-deep block are fetched
        // one block ahead of their conversion.  (With one thread per row the conversion of a stage took nearly as
        // long as its MMAs, and with two stages the two do not overlap fully.)
        const int r = threadIdx.x & 127, half = threadIdx.x >> 7;
        uint4 nxt[SPB];
        float nxt_sc = 0.0f;
        bool nxt_live = false;
        auto fetch = [&](int u) {
            const int tile = u / nb, kb = u - tile * nb;
            const int t = tile * TM + r;
            nxt_live = t < T;
            const uint8_t* src = xq + (size_t)min(t, T - 1) * D + (size_t)kb * 128 + half * 16;
#pragma unroll
            for (int j = 0; j < SPB; j++) nxt[j] = __ldg(reinterpret_cast<const uint4*>(src + j * KS));
            nxt_sc = nxt_live ? xs[(size_t)t * nb + kb] : 0.0f;
        };
        if (u0 < u1) fetch(u0);
        int i = 0;
        for (int u = u0; u < u1; u++) {
            uint4 cur[SPB];
#pragma unroll
            for (int j = 0; j < SPB; j++) cur[j] = nxt[j];
            const float sc = nxt_sc;
            const bool live = nxt_live;
            if (u + 1 < u1) fetch(u + 1);
#pragma unroll
            for (int q4 = 0; q4 < SPB; q4++, i++) {
                const int s = i % NSTAGE;
                const uint32_t par = (uint32_t)((i / NSTAGE) & 1);
                if (!ptx::mbar_wait(&sm->empty[s], par ^ 1, abort_flag)) goto done;
                const uint32_t a_hi = ptx::smem_u32(base + (size_t)s * stage_bytes) + r * 128;
                const uint32_t a_lo = a_hi + A_TILE;
                const uint32_t words[4] = {cur[q4].x, cur[q4].y, cur[q4].z, cur[q4].w};
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {                    // 16-byte chunk j = 4 consecutive d
                    const int j = half * 4 + jj;
                    float h[4], l[4];
#pragma unroll
                    for (int b = 0; b < 4; b++) {
                        __nv_fp8_e4m3 q;
                        q.__x = (unsigned char)((words[jj] >> (8 * b)) & 0xFF);
                        // the dequantised activation, as the exact kernels form it (rows beyond T: zero)
                        const float x = live ? __fmul_rn(float(q), sc) : 0.0f;
                        h[b] = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
                        l[b] = __fsub_rn(x, h[b]);
                    }
                    const uint32_t off = (uint32_t)((j ^ (r & 7)) << 4);
                    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a_hi + off), "f"(h[0]), "f"(h[1]), "f"(h[2]), "f"(h[3]) : "memory");
                    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a_lo + off), "f"(l[0]), "f"(l[1]), "f"(l[2]), "f"(l[3]) : "memory");
                }
                ptx::fence_proxy_async_smem();                      // generic-proxy stores -> visible to the MMA (async proxy)
                ptx::mbar_arrive(&sm->a_full[s]);
            }
        }
    } else if (warp < 12) {
        // ===================== accumulators -> partial sums (thread = token row of the tile) =====================
        const int ew = warp - 8;                                    // = warp % 4: the TMEM lanes this warp may read
        const uint32_t lane_addr = (uint32_t)(ew * 32) << 16;
        int pc = 0;
        for (int u = u0; u < u1; pc++) {
            const int tile = u / nb, kb = u - tile * nb;
            const int len = min(plan.ch, min(nb - kb, u1 - u));
            const int slot = tc_slots_before(plan, tile, u);
            const int buf = pc & 1;
            if (!ptx::mbar_wait(&sm->acc_full[buf], (uint32_t)((pc >> 1) & 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            const int t = tile * TM + ew * 32 + lane;
            float* dst = partials + ((size_t)slot * T + min(t, T - 1)) * E;
            for (int c0 = 0; c0 < N; c0 += 32) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(tmem + lane_addr + buf * 256 + c0, v);
                ptx::tc_wait_ld();
                if (t < T) {
#pragma unroll
                    for (int k = 0; k < 32; k += 4)
                        if (c0 + k < E)          // E % 4 == 0
                            *reinterpret_cast<float4*>(dst + c0 + k) =
                                make_float4(__uint_as_float(v[k]), __uint_as_float(v[k + 1]), __uint_as_float(v[k + 2]),
                                            __uint_as_float(v[k + 3]));
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(&sm->acc_empty[buf]);
            u += len;
        }
    } else if (warp == 12) {
        // ===================== weight tiles by TMA =====================
        if (lane == 0) {
            int i = 0;
            for (int u = u0; u < u1; u++) {
                const int kb = u % nb;
                for (int q4 = 0; q4 < SPB; q4++, i++) {
                    const int s = i % NSTAGE;
                    const uint32_t par = (uint32_t)((i / NSTAGE) & 1);
                    if (!ptx::mbar_wait_relaxed(&sm->empty[s], par ^ 1, abort_flag, 100)) goto done;
                    uint8_t* bh = base + (size_t)s * stage_bytes + 2 * A_TILE;
                    ptx::mbar_expect_tx(&sm->b_full[s], 2 * b_tile);
                    ptx::tma_load_2d(bh, &tmap_hi, &sm->b_full[s], kb * 128 + q4 * KS, 0);
                    ptx::tma_load_2d(bh + b_tile, &tmap_lo, &sm->b_full[s], kb * 128 + q4 * KS, 0);
                }
            }
        }
    } else {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const uint32_t idesc = ptx::make_idesc(2, 2, 0, 0, TM, N);      // tf32 x tf32 -> f32, both K-major
            int i = 0, pc = 0;
            for (int u = u0; u < u1; pc++) {
                const int kb = u % nb;
                const int len = min(plan.ch, min(nb - kb, u1 - u));
                const int buf = pc & 1;
                if (!ptx::mbar_wait(&sm->acc_empty[buf], (uint32_t)(((pc >> 1) & 1) ^ 1), abort_flag)) goto done;
                ptx::tc_fence_after();
                const uint32_t acc = tmem + buf * 256;
                for (int st = 0; st < len * SPB; st++, i++) {
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
                        mma_tf32(acc, dah, dbh, idesc, (st > 0 || kk > 0) ? 1u : 0u);
                        mma_tf32(acc, dah, dbl, idesc, 1u);
                        mma_tf32(acc, dal, dbh, idesc, 1u);
                    }
                    ptx::tc_commit(&sm->empty[s]);
                }
                ptx::tc_commit(&sm->acc_full[buf]);
                u += len;
            }
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 13) ptx::tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(status, B200_TIMEOUT);
}

// Sum of a token's slots in order: the approximate logits themselves (test hook only).
__global__ void tc_sum_kernel(const float* __restrict__ partials, float* __restrict__ logits, int T, int E, TcPlan plan) {
    const int t = blockIdx.x;
    const int n = tc_slots_before(plan, t / TM, (t / TM + 1) * plan.nblk);
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float l = partials[(size_t)t * E + e];
        for (int s = 1; s < n; s++) l = __fadd_rn(l, partials[((size_t)s * T + t) * E + e]);
        logits[(size_t)t * E + e] = l;
    }
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
static int g_tc_chain_override = 0;      // set only inside b200_moe_gate_logits_tc (test hook)
static int tc_chain() { return g_tc_chain_override > 0 ? g_tc_chain_override : TC_CHAIN; }
// A CTA never takes fewer than TC_CHAIN units, so a tile is cut by at most nblk / TC_CHAIN range boundaries on top
// of its own nblk / TC_CHAIN chains.
int moe_gate_tc_slots(int D) { return 2 * ceil_div(D / 128, TC_CHAIN) + 1; }

// whi / wlo: E * D floats each (workspace); partials: moe_gate_tc_slots(D) * T * E floats.
int launch_gate_logits_tc(const uint8_t* xq, const float* xs, const float* wg, float* whi, float* wlo, float* partials,
                          int T, int E, int D, int* status, cudaStream_t stream, TcPlan* plan_out) {
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
    static int sm_count[64] = {0};
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (b200_first_call_on_device(attr_done)) {
        B200_CUDA_TRY(cudaFuncSetAttribute(gate_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(1024 + (size_t)NSTAGE * (2 * A_TILE + 2 * (size_t)MAX_N * KS * 4) + sizeof(TcSmem) + 64)));
        B200_CUDA_TRY(cudaDeviceGetAttribute(&sm_count[dev & 63], cudaDevAttrMultiProcessorCount, dev));
    }
    TcPlan plan;
    plan.nblk = D / 128;
    plan.ch = min(tc_chain(), plan.nblk);
    const long long units = (long long)ceil_div(T, TM) * plan.nblk;
    if (units > 0x3fffffff) return B200_UNSUPPORTED;
    const int sms = max(1, sm_count[dev & 63]);
    plan.L = max((int)((units + sms - 1) / sms), plan.ch);         // one CTA per SM, never below one whole chain
    const int grid = (int)((units + plan.L - 1) / plan.L);
    gate_tc_kernel<<<grid, TC_THREADS, smem, stream>>>(th, tl, xq, xs, partials, T, E, D, N, plan, (int)units, status);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    *plan_out = plan;
    return B200_OK;
}

// Test hook (host only, no GPU needed): walks the work split of T tokens x D on `sms` CTAs exactly as the kernel's
// roles do and checks that every tile's pieces get the slots 0 .. n-1 in order of d, cover its blocks once, and
// stay within the bound the scratch is sized with.  Returns 0 when consistent, a positive code otherwise;
// *max_slots_out receives the largest number of slots of a tile.
extern "C" int b200_tc_plan_selftest(int T, int D, int sms, int chain_blocks, int* max_slots_out) {
    if (T <= 0 || D <= 0 || D % 128 || sms <= 0 || chain_blocks < 0) return B200_BAD_ARG;
    TcPlan plan;
    plan.nblk = D / 128;
    plan.ch = min(chain_blocks > 0 ? chain_blocks : TC_CHAIN, plan.nblk);
    const int ntile = ceil_div(T, TM);
    const long long units = (long long)ntile * plan.nblk;
    plan.L = max((int)((units + sms - 1) / sms), plan.ch);
    const int grid = (int)((units + plan.L - 1) / plan.L);
    std::vector<int> next_slot(ntile, 0), next_kb(ntile, 0);
    for (int c = 0; c < grid; c++) {
        const int u0 = c * plan.L;
        const long long end = (long long)u0 + plan.L;
        const int u1 = (int)(end < units ? end : units);
        for (int u = u0; u < u1;) {
            const int tile = u / plan.nblk, kb = u - tile * plan.nblk;
            const int len = min(plan.ch, min(plan.nblk - kb, u1 - u));
            if (tc_slots_before(plan, tile, u) != next_slot[tile]) return 101;      // slots count up in order of d
            if (kb != next_kb[tile]) return 102;                                    // blocks covered once, in order
            next_slot[tile]++;
            next_kb[tile] += len;
            u += len;
        }
    }
    int mx = 0;
    for (int t = 0; t < ntile; t++) {
        if (next_kb[t] != plan.nblk) return 103;
        if (tc_slots_before(plan, t, (t + 1) * plan.nblk) != next_slot[t]) return 104;     // what the selection kernel adds up
        mx = max(mx, next_slot[t]);
    }
    if (mx > 2 * ceil_div(plan.nblk, plan.ch) + 1) return 105;                      // the bound of moe_gate_tc_slots
    if (max_slots_out) *max_slots_out = mx;
    return 0;
}

// Test hook: the tensor-core logits [T, E] (a token's partial sums added in slot order).  chain_blocks > 0 asks
// for accumulation chains of that many 128-deep blocks instead of the library's choice (D / 128: one chain over
// all of d, which shows how the tensor core's accumulation error grows with the chain).  Not thread-safe (the
// override is a global).
extern "C" int b200_moe_gate_logits_tc(const uint8_t* xq, const float* xs, const float* gate_w, float* logits_out,
                                       int T, int E, int D, int chain_blocks, b200_stream_t stream) {
    if (!xq || !xs || !gate_w || !logits_out) return B200_BAD_ARG;
    if (!moe_gate_tc_supported(T, E, D)) return B200_UNSUPPORTED;
    if (chain_blocks < 0 || chain_blocks > D / 128) return B200_BAD_ARG;
    b200_ws* ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    // chains longer than the default need no more slots than the default's bound
    const size_t slots = (size_t)max(moe_gate_tc_slots(D), 2 * ceil_div(D / 128, max(1, chain_blocks)) + 1);
    WsCarver sz(nullptr);
    sz.take<float>((size_t)E * D);
    sz.take<float>((size_t)E * D);
    sz.take<float>(slots * T * E);
    int st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    float* whi = cv.take<float>((size_t)E * D);
    float* wlo = cv.take<float>((size_t)E * D);
    float* partials = cv.take<float>(slots * T * E);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    TcPlan plan;
    g_tc_chain_override = chain_blocks;
    st = launch_gate_logits_tc(xq, xs, gate_w, whi, wlo, partials, T, E, D, ws->d_status, s, &plan);
    g_tc_chain_override = 0;
    if (st) return st;
    tc_sum_kernel<<<T, 128, 0, s>>>(partials, logits_out, T, E, plan);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
