// DSA / MLA sparse decode on bf16 inputs for sm_100a: one fused kernel replaces the reference's
// eight launches (kernels/dsa/naive_dsa.cu:435-474) — the three row gathers (:13-59), the 576-wide
// dot (:208-273), scale (:321-324), softmax (:278-294) and output projection (:300-316) — with the
// scores and the attention matrix never leaving the SM.
//
// Work split: CTA = (query, half of the 512 output columns, range of the selected rows).
// All 128 heads form the M dimension of the MMAs:
//     S[128 heads, 32 rows]  = Q[128, 576] * K_tile[32, 576]^T      (tcgen05.mma kind::f16, N = 32)
//     O[128 heads, 256 cols] += P[128, 32] * V_tile[32, 256]        (N = 256, V read MN-major)
// with S and O in tensor memory (O: 256 columns, S: 2 x 32 columns).
//
// Shared memory (all operands in the canonical UMMA layouts, 128-byte swizzle unless noted):
//     Q   9 blocks of [128 heads x 128 B]   resident for the CTA's lifetime        147456 B
//     K   ring of 9 slots [32 rows x 128 B] (slot c = dims 64c..64c+63 of a row)     36864 B
//     V   2 buffers of 4 chunks [32 rows x 128 B] (chunk = 64 output columns)        32768 B
//     P   [128 x 32] bf16, unswizzled 8x16-byte core matrices, chunk-major             8192 B
// Warp roles: warps 0-3 softmax (thread = head = TMEM lane), warp 4 MMA issuer, warps 5-8
// gather producers (16-byte cp.async straight from the flat caches through the index list,
// with the swizzle applied to the destination address).  K slots are refilled as soon as the
// MMAs that read them retire, so the row stream never waits for a whole tile.
// The online softmax keeps a per-head running maximum and rescales O only when the maximum
// grows by more than 2^8 (the factor is carried in P and in the running sum instead).
// Every mbarrier wait is bounded; on give-up the CTA flags B200_TIMEOUT and winds down.
#include <cfloat>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "dsa_index.cuh"

void b200_count_launch(int n);
void b200_set_last_error_text(const char* text);

namespace {

constexpr int HEADS = 128, DC = 512, DP = 64, TKV = 32, DVH = 256;
constexpr int KBLK = 9;
constexpr int Q_BLK_BYTES = HEADS * 128;          // 16384
constexpr int Q_BYTES = KBLK * Q_BLK_BYTES;       // 147456
constexpr int KSLOT_BYTES = TKV * 128;            // 4096
constexpr int K_BYTES = KBLK * KSLOT_BYTES;       // 36864
constexpr int VCHUNK_BYTES = TKV * 128;           // 4096
constexpr int V_BYTES = 4 * VCHUNK_BYTES;         // 16384
constexpr int P_BYTES = HEADS * TKV * 2;          // 8192
constexpr int P_CHUNK_BYTES = HEADS * 16;         // 2048
constexpr int DSA_THREADS = 288;
constexpr int UNITS = 10;                         // 9 K slots + 1 V buffer per tile
constexpr int LAG = 6;                            // cp.async groups kept in flight per thread
constexpr uint32_t O_COL = 0, S_COL = 256;

struct DsaSmem {
    uint64_t q_full;
    uint64_t k_full[KBLK], k_empty[KBLK];
    uint64_t v_full[2], v_empty[2];
    uint64_t s_full[2], s_empty[2];
    uint64_t p_full, p_empty, o_done;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr size_t DSA_SMEM_BYTES = 1024 + Q_BYTES + K_BYTES + 2 * V_BYTES + P_BYTES + sizeof(DsaSmem);

struct DsaParams {
    const __nv_bfloat16 *q_nope, *q_pe, *kc, *kp, *v;
    DsaIndex ix;
    float* out;        // [Q, H, 512]
    float* part_o;     // [Q, NS, 128, 512]   (NS > 1)
    float* part_ml;    // [Q, NS, 128, 2]     log2-domain max, running sum
    int* status;
    int H, S, NS, tiles_per_split;
    float sl2;         // log2(e) / sqrt(Dc + Dp)
};

__global__ void __launch_bounds__(DSA_THREADS, 1) dsa_decode_bf16_kernel(const DsaParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = base;
    uint8_t* sK = sQ + Q_BYTES;
    uint8_t* sV = sK + K_BYTES;
    uint8_t* sP = sV + 2 * V_BYTES;
    DsaSmem* sm = reinterpret_cast<DsaSmem*>(sP + P_BYTES);
    volatile int* abort_flag = &sm->abort_flag;

    const int hv = blockIdx.x, sp = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt_total = p.S / TKV;
    const int t_begin = sp * p.tiles_per_split;
    const int t_end = min(nt_total, t_begin + p.tiles_per_split);
    const int nt = max(0, t_end - t_begin);

    if (threadIdx.x == 0) {
        ptx::mbar_init(&sm->q_full, 128);
        for (int c = 0; c < KBLK; c++) { ptx::mbar_init(&sm->k_full[c], 128); ptx::mbar_init(&sm->k_empty[c], 1); }
        for (int i = 0; i < 2; i++) {
            ptx::mbar_init(&sm->v_full[i], 128);
            ptx::mbar_init(&sm->v_empty[i], 1);
            ptx::mbar_init(&sm->s_full[i], 1);
            ptx::mbar_init(&sm->s_empty[i], 128);
        }
        ptx::mbar_init(&sm->p_full, 128);
        ptx::mbar_init(&sm->p_empty, 1);
        ptx::mbar_init(&sm->o_done, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 4) {
        ptx::tmem_alloc(&sm->tmem_base, 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (warp >= 5) {
        // ===================== gather producers (128 threads) =====================
        const int pt = threadIdx.x - 160;
        // Q: 128 rows x 72 sixteen-byte chunks; rows >= H are zero
        for (int i = pt; i < HEADS * 72; i += 128) {
            const int r = i / 72, ch = i - r * 72;
            const uint32_t dst = ptx::smem_u32(sQ) + (ch >> 3) * Q_BLK_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            if (r < p.H) {
                const __nv_bfloat16* src = (ch < 64) ? p.q_nope + ((size_t)b * p.H + r) * DC + ch * 8
                                                     : p.q_pe + ((size_t)b * p.H + r) * DP + (ch - 64) * 8;
                ptx::cp_async_16(dst, src);
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(&sm->q_full);

        const int total_units = nt * UNITS;
        long long kid[2] = {0, 0}, vid[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        auto bar_of = [&](int u) -> uint64_t* {
            int j = u / UNITS, c = u - j * UNITS;
            return (c < KBLK) ? &sm->k_full[c] : &sm->v_full[j & 1];
        };
        for (int u = 0; u < total_units; u++) {
            const int j = u / UNITS, c = u - j * UNITS;
            if (c == 0) {
                const int s0 = (t_begin + j) * TKV;
                kid[0] = dsa_resolve(p.ix, b, s0 + (pt >> 3));
                kid[1] = dsa_resolve(p.ix, b, s0 + (pt >> 3) + 16);
#pragma unroll
                for (int x = 0; x < 8; x++) vid[x] = dsa_resolve(p.ix, b, s0 + (pt >> 5) + 4 * x);
            }
            if (c < KBLK) {
                if (!ptx::mbar_wait(&sm->k_empty[c], (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
                const uint32_t slot = ptx::smem_u32(sK) + c * KSLOT_BYTES;
                const int j16 = pt & 7;
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    const int r = (pt >> 3) + 16 * x;
                    const uint32_t dst = slot + r * 128 + ((j16 ^ (r & 7)) << 4);
                    if (kid[x] >= 0) {
                        const __nv_bfloat16* src = (c < 8) ? p.kc + kid[x] * DC + c * 64 + j16 * 8
                                                           : p.kp + kid[x] * DP + j16 * 8;
                        ptx::cp_async_16(dst, src);
                    } else {        // empty entry: zero row, its score is masked by the softmax threads
                        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
                    }
                }
            } else {
                const int vb = j & 1;
                if (!ptx::mbar_wait(&sm->v_empty[vb], (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) goto done;
                const uint32_t vbase = ptx::smem_u32(sV) + vb * V_BYTES;
                const int j32 = pt & 31, cc = j32 >> 3, j16 = j32 & 7;
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int r = (pt >> 5) + 4 * x;
                    const uint32_t dst = vbase + cc * VCHUNK_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((j16 ^ (r & 7)) << 4);
                    if (vid[x] >= 0) ptx::cp_async_16(dst, p.v + vid[x] * DC + hv * DVH + j32 * 8);
                    else asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
                }
            }
            ptx::cp_async_commit();
            if (u >= LAG) {
                ptx::cp_async_wait<LAG>();
                ptx::fence_proxy_async_smem();
                ptx::mbar_arrive(bar_of(u - LAG));
            }
        }
        ptx::cp_async_wait<0>();
        ptx::fence_proxy_async_smem();
        for (int u = max(0, total_units - LAG); u < total_units; u++) ptx::mbar_arrive(bar_of(u));
    } else if (warp == 4) {
        // ===================== MMA issuer =====================
        if (lane == 0 && nt > 0) {
            constexpr uint32_t idesc_qk = ptx::make_idesc(1, 1, 0, 0, HEADS, TKV);
            constexpr uint32_t idesc_pv = ptx::make_idesc(1, 1, 0, 1, HEADS, DVH);
            const uint32_t q_addr = ptx::smem_u32(sQ), k_addr = ptx::smem_u32(sK), v_addr = ptx::smem_u32(sV),
                           p_addr = ptx::smem_u32(sP);
            auto issue_pv = [&](int i) -> bool {
                const int vb = i & 1;
                if (!ptx::mbar_wait(&sm->p_full, (uint32_t)(i & 1), abort_flag)) return false;
                if (!ptx::mbar_wait(&sm->v_full[vb], (uint32_t)((i >> 1) & 1), abort_flag)) return false;
                ptx::tc_fence_after();
#pragma unroll
                for (int k2 = 0; k2 < 2; k2++) {
                    uint64_t ad = ptx::make_smem_desc(p_addr + k2 * 2 * P_CHUNK_BYTES, P_CHUNK_BYTES, 128, 0);
                    uint64_t bd = ptx::make_smem_desc(v_addr + vb * V_BYTES + k2 * 2048, VCHUNK_BYTES, 1024, 2);
                    ptx::mma_f16(tmem + O_COL, ad, bd, idesc_pv, (i > 0 || k2 > 0) ? 1u : 0u);
                }
                ptx::tc_commit(&sm->v_empty[vb]);
                ptx::tc_commit(&sm->p_empty);
                return true;
            };
            if (!ptx::mbar_wait(&sm->q_full, 0, abort_flag)) goto done;
            for (int j = 0; j < nt; j++) {
                const int sb = j & 1;
                if (!ptx::mbar_wait(&sm->s_empty[sb], (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) goto done;
                for (int c = 0; c < KBLK; c++) {
                    if (!ptx::mbar_wait(&sm->k_full[c], (uint32_t)(j & 1), abort_flag)) goto done;
                    ptx::tc_fence_after();
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        uint64_t ad = ptx::make_smem_desc(q_addr + c * Q_BLK_BYTES + k4 * 32, 16, 1024, 2);
                        uint64_t bd = ptx::make_smem_desc(k_addr + c * KSLOT_BYTES + k4 * 32, 16, 1024, 2);
                        ptx::mma_f16(tmem + S_COL + sb * TKV, ad, bd, idesc_qk, (c > 0 || k4 > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(&sm->k_empty[c]);
                }
                ptx::tc_commit(&sm->s_full[sb]);
                if (j > 0 && !issue_pv(j - 1)) goto done;
            }
            if (!issue_pv(nt - 1)) goto done;
            ptx::tc_commit(&sm->o_done);
        }
    } else {
        // ===================== softmax / correction / epilogue (warps 0-3) =====================
        const int h = threadIdx.x;                                   // head = TMEM lane
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float m = -1e30f, l = 0.0f;
        const float thr = 8.0f / p.sl2;                              // 2^8 in raw-score units
        // which of the tile's 32 rows are empty entries (one bit per row), looked up one tile ahead
        // (the entry is fetched during the previous tile and only looked at here, so its latency is hidden)
        int ent_n = (nt > 0) ? dsa_resolve(p.ix, b, t_begin * TKV + lane) : -1;
        for (int j = 0; j < nt; j++) {
            const int sb = j & 1;
            const unsigned mask = __ballot_sync(0xffffffffu, ent_n >= 0);
            if (j + 1 < nt) ent_n = dsa_resolve(p.ix, b, (t_begin + j + 1) * TKV + lane);
            if (!ptx::mbar_wait(&sm->s_full[sb], (uint32_t)((j >> 1) & 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem + lane_addr + S_COL + sb * TKV, r);
            ptx::tc_wait_ld();
            ptx::tc_fence_before();
            ptx::mbar_arrive(&sm->s_empty[sb]);
            if (mask != 0xffffffffu) {
#pragma unroll
                for (int i = 0; i < 32; i++) r[i] = ((mask >> i) & 1u) ? r[i] : 0xff800000u;     // -inf
            }
            float tmax = -FLT_MAX;
#pragma unroll
            for (int i = 0; i < 32; i++) tmax = fmaxf(tmax, __uint_as_float(r[i]));
            const bool need = tmax > m + thr;
            const float m_new = need ? tmax : m;
            const float corr = need ? exp2f((m - m_new) * p.sl2) : 1.0f;
            float rowsum = 0.0f;
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; i++) {
                float p0 = exp2f((__uint_as_float(r[2 * i]) - m_new) * p.sl2);
                float p1 = exp2f((__uint_as_float(r[2 * i + 1]) - m_new) * p.sl2);
                rowsum += p0 + p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[i] = *reinterpret_cast<uint32_t*>(&h2);
            }
            // P buffer free and O quiescent once the previous tile's P*V has retired
            if (!ptx::mbar_wait(&sm->p_empty, (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c0 = 0; c0 < DVH; c0 += 32) {
                    uint32_t o[32];
                    ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                    ptx::tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    ptx::tmem_st_32x32(tmem + lane_addr + O_COL + c0, o);
                }
                ptx::tc_wait_st();
            }
            // P row h: chunk ch (8 kv = 16 B) at ch*2048 + h*16
#pragma unroll
            for (int ch = 0; ch < 4; ch++) {
                const uint32_t dst = ptx::smem_u32(sP) + ch * P_CHUNK_BYTES + h * 16;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * ch]),
                             "r"(pk[4 * ch + 1]), "r"(pk[4 * ch + 2]), "r"(pk[4 * ch + 3])
                             : "memory");
            }
            ptx::fence_proxy_async_smem();
            ptx::tc_fence_before();
            ptx::mbar_arrive(&sm->p_full);
            l = l * corr + rowsum;
            m = m_new;
        }
        if (nt > 0) {
            if (!ptx::mbar_wait(&sm->o_done, 0, abort_flag)) goto done;
            ptx::tc_fence_after();
        }
        const bool direct = (p.NS == 1);
        const float inv = (direct && l > 0.0f) ? 1.0f / l : 1.0f;
        float* dst = direct ? p.out + ((size_t)b * p.H + h) * DC + hv * DVH
                            : p.part_o + (((size_t)b * p.NS + sp) * HEADS + h) * DC + hv * DVH;
#pragma unroll 1
        for (int c0 = 0; c0 < DVH; c0 += 32) {
            uint32_t o[32];
            if (nt > 0) {
                ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                ptx::tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = 0;
            }
            if (h < p.H || !direct) {
                float4* d4 = reinterpret_cast<float4*>(dst + c0);
#pragma unroll
                for (int i = 0; i < 8; i++)
                    d4[i] = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                        __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
            }
        }
        if (!direct && hv == 0) {
            float* ml = p.part_ml + (((size_t)b * p.NS + sp) * HEADS + h) * 2;
            ml[0] = (nt > 0) ? m * p.sl2 : -1e30f;
            ml[1] = l;
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 4) ptx::tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(p.status, B200_TIMEOUT);
}

// out[q,h,:] = sum_sp O_sp * 2^(m_sp - M) / sum_sp l_sp * 2^(m_sp - M)
__global__ void __launch_bounds__(128) dsa_merge_kernel(const float* __restrict__ part_o,
                                                        const float* __restrict__ part_ml, float* __restrict__ out,
                                                        int H, int NS) {
    const int b = blockIdx.y, h = blockIdx.x;
    float M = -1e30f;
    for (int s = 0; s < NS; s++) M = fmaxf(M, part_ml[(((size_t)b * NS + s) * HEADS + h) * 2]);
    float L = 0.0f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < NS; s++) {
        const float* ml = part_ml + (((size_t)b * NS + s) * HEADS + h) * 2;
        const float w = exp2f(ml[0] - M);
        L += ml[1] * w;
        const float4 o = reinterpret_cast<const float4*>(part_o + (((size_t)b * NS + s) * HEADS + h) * DC)[threadIdx.x];
        acc.x += o.x * w; acc.y += o.y * w; acc.z += o.z * w; acc.w += o.w * w;
    }
    const float inv = L > 0.0f ? 1.0f / L : 0.0f;        // a query whose entries are all empty gets zeros
    reinterpret_cast<float4*>(out + ((size_t)b * H + h) * DC)[threadIdx.x] =
        make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

}  // namespace

int b200_launch_dsa_pair(const void* q_nope, const void* q_pe, const void* kc, const void* kp, const void* v,
                         const DsaIndex& ix, float* out, float* part_o, float* part_ml, int* status, int Q, int H, int S,
                         int NS, int tiles_per_split, int tile_rows, cudaStream_t stream);

namespace {

int check_dsa_bf16(const void* q_nope, const void* q_pe, const void* kc, const void* kp, const void* v, const int* idx,
                   const float* out, const b200_dsa_config* cfg) {
    if (!cfg) return B200_BAD_ARG;
    if (!q_nope || !q_pe || !kc || !kp || !v || !idx || !out) return B200_BAD_ARG;
    const int Q = cfg->num_queries, H = cfg->num_heads, S = cfg->num_selected_kv;
    if (Q <= 0 || H <= 0 || S <= 0) return B200_BAD_SHAPE;
    if (cfg->head_dim_compressed != DC || cfg->head_dim_positional != DP) return B200_UNSUPPORTED;
    if (H > HEADS) return B200_UNSUPPORTED;
    if (S % TKV) return B200_BAD_SHAPE;
    const uintptr_t align = reinterpret_cast<uintptr_t>(q_nope) | reinterpret_cast<uintptr_t>(q_pe) |
                            reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(kp) |
                            reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out);
    if (align & 15) return B200_BAD_ARG;
    return B200_OK;
}

// Workspace-backed decode on a resolved row selection.
int dsa_bf16_impl(b200_ws* ws, const uint16_t* q_nope, const uint16_t* q_pe, const uint16_t* kc, const uint16_t* kp,
                  const uint16_t* v, const DsaIndex& ix, float* out, const b200_dsa_config* cfg, cudaStream_t stream) {
    const int Q = cfg->num_queries, H = cfg->num_heads, S = cfg->num_selected_kv;
    if (Q > 65535) return B200_UNSUPPORTED;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;

    // The CTA-pair kernels take every shape with S % 64 == 0 (128-row tiles when S % 128 == 0, else
    // 64-row tiles); the single-CTA kernel (32-row tiles) takes the rest.
    const bool use_pair = (S % 64 == 0);
    const int pair_tile = (S % 128 == 0) ? 128 : 64;
    // split the selected rows so that the grid covers the machine about once
    const int nt_total = S / (use_pair ? pair_tile : TKV);
    int NS = 1;
    if (2 * Q < ws->sm_count) NS = ws->sm_count / (2 * Q);
    if (NS > nt_total) NS = nt_total;
    if (NS > 64) NS = 64;
    if (NS < 1) NS = 1;
    const int tps = ceil_div(nt_total, NS);
    NS = ceil_div(nt_total, tps);

    float *part_o = nullptr, *part_ml = nullptr;
    if (NS > 1) {
        WsCarver sz(nullptr);
        sz.take<float>((size_t)Q * NS * HEADS * DC);
        sz.take<float>((size_t)Q * NS * HEADS * 2);
        int st = b200_ws_ensure(ws, sz.total());
        if (st) return st;
        WsCarver cv(ws->base);
        part_o = cv.take<float>((size_t)Q * NS * HEADS * DC);
        part_ml = cv.take<float>((size_t)Q * NS * HEADS * 2);
    }
    if (use_pair) {
        int st = b200_launch_dsa_pair(q_nope, q_pe, kc, kp, v, ix, out, part_o, part_ml, ws->d_status, Q, H, S, NS, tps,
                                      pair_tile, stream);
        if (st) return st;
        if (NS > 1) {
            dsa_merge_kernel<<<dim3(H, Q), 128, 0, stream>>>(part_o, part_ml, out, H, NS);
            b200_count_launch(1);
            B200_CUDA_TRY(cudaGetLastError());
        }
        return B200_OK;
    }
    static bool attr_done[64] = {false};
    if (b200_first_call_on_device(attr_done)) {
        B200_CUDA_TRY(cudaFuncSetAttribute(dsa_decode_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)DSA_SMEM_BYTES));
    }
    DsaParams p;
    p.q_nope = reinterpret_cast<const __nv_bfloat16*>(q_nope);
    p.q_pe = reinterpret_cast<const __nv_bfloat16*>(q_pe);
    p.kc = reinterpret_cast<const __nv_bfloat16*>(kc);
    p.kp = reinterpret_cast<const __nv_bfloat16*>(kp);
    p.v = reinterpret_cast<const __nv_bfloat16*>(v);
    p.ix = ix; p.out = out; p.part_o = part_o; p.part_ml = part_ml; p.status = ws->d_status;
    p.H = H; p.S = S; p.NS = NS; p.tiles_per_split = tps;
    p.sl2 = 1.4426950408889634f / sqrtf((float)(DC + DP));
    dim3 grid(2, NS, Q);
    dsa_decode_bf16_kernel<<<grid, DSA_THREADS, DSA_SMEM_BYTES, stream>>>(p);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    if (NS > 1) {
        dsa_merge_kernel<<<dim3(H, Q), 128, 0, stream>>>(part_o, part_ml, out, H, NS);
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
}

DsaIndex flat_index(const int* idx, const b200_dsa_config* cfg) {
    DsaIndex ix{};
    ix.idx = idx; ix.S = cfg->num_selected_kv; ix.page = cfg->page_size > 0 ? cfg->page_size : 1;
    ix.N = cfg->total_kv_tokens;        // 0 or negative: rows are not range-checked (the reference never reads it)
    return ix;
}

}  // namespace

extern "C" int b200_dsa_forward_bf16(b200_ws* ws, const uint16_t* q_nope, const uint16_t* q_pe, const uint16_t* kc,
                                     const uint16_t* kp, const uint16_t* v, const int* idx, float* out,
                                     const b200_dsa_config* cfg, b200_stream_t stream) {
    int st = check_dsa_bf16(q_nope, q_pe, kc, kp, v, idx, out, cfg);
    if (st) return st;
    return dsa_bf16_impl(ws, q_nope, q_pe, kc, kp, v, flat_index(idx, cfg), out, cfg, stream);
}

extern "C" int b200_dsa_forward_bf16_paged(b200_ws* ws, const uint16_t* q_nope, const uint16_t* q_pe, const uint16_t* kc,
                                           const uint16_t* kp, const uint16_t* v, const int* positions,
                                           const int* block_table, int max_blocks, const int* seq_of_query,
                                           const int* valid_len, float* out, const b200_dsa_config* cfg,
                                           b200_stream_t stream) {
    int st = check_dsa_bf16(q_nope, q_pe, kc, kp, v, positions, out, cfg);
    if (st) return st;
    if (!block_table || max_blocks <= 0) return B200_BAD_ARG;
    if (cfg->page_size <= 0) return B200_BAD_SHAPE;
    DsaIndex ix = flat_index(positions, cfg);
    ix.block_table = block_table; ix.max_blocks = max_blocks; ix.seq_of_query = seq_of_query; ix.valid_len = valid_len;
    return dsa_bf16_impl(ws, q_nope, q_pe, kc, kp, v, ix, out, cfg, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the bf16 decode call.
//
// Some hosts of this library may not allocate device memory at all once they are running: a
// serving process whose memory pool owns every byte of HBM and forbids cudaMalloc after start-up,
// a plugin loaded into a framework that hands out only the input and output buffers, or a caller
// sitting inside a latency-critical loop where a growing workspace (and the device synchronise
// that growth implies) is unacceptable.  For them the split-KV partial results live in the
// fixed array below instead of the growable workspace.  The array is part of the loaded module:
// every GPU that loads the library holds B200_DSA_STATIC_SCRATCH_BYTES of it until the process
// exits, whether or not this entry point is ever called.
// ---------------------------------------------------------------------------------------------
#define B200_DSA_STATIC_SCRATCH_BYTES (16u << 20)
#define B200_DSA_STATIC_MAX_QUERIES 65535          // one grid row per query
static __device__ __align__(256) unsigned char g_dsa_static_scratch[B200_DSA_STATIC_SCRATCH_BYTES];

namespace {
// Device address of the array per device.  In host code the array's name is only a handle for
// the runtime, not a device pointer, so the address is asked for once per device (with that
// device current) and cached.
unsigned char* g_static_scratch_addr[64] = {nullptr};
int g_static_sm_count[64] = {0};

int static_scratch_setup(int dev) {
    if (g_static_scratch_addr[dev]) return B200_OK;
    void* p = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_dsa_static_scratch));
    if (!p) return B200_CUDA_ERROR;
    int sms = 0;
    B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    B200_CUDA_TRY(cudaFuncSetAttribute(dsa_decode_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)DSA_SMEM_BYTES));
    g_static_sm_count[dev] = sms;
    g_static_scratch_addr[dev] = static_cast<unsigned char*>(p);
    return B200_OK;
}
}  // namespace

extern "C" int b200_dsa_forward_bf16_static(const uint16_t* q_nope, const uint16_t* q_pe, const uint16_t* kc,
                                            const uint16_t* kp, const uint16_t* v, const int* idx, float* out,
                                            const b200_dsa_config* cfg, int* device_status,
                                            b200_stream_t stream) {
    if (!cfg) return B200_BAD_ARG;
    if (!q_nope || !q_pe || !kc || !kp || !v || !idx || !out || !device_status) return B200_BAD_ARG;
    const int Q = cfg->num_queries, H = cfg->num_heads, S = cfg->num_selected_kv;
    if (Q <= 0 || H <= 0 || S <= 0) return B200_BAD_SHAPE;
    if (cfg->head_dim_compressed != DC || cfg->head_dim_positional != DP) return B200_UNSUPPORTED;
    if (H > HEADS) return B200_UNSUPPORTED;
    if (S % TKV) return B200_BAD_SHAPE;
    if (Q > B200_DSA_STATIC_MAX_QUERIES) {
        char msg[160];
        snprintf(msg, sizeof(msg), "b200_dsa_forward_bf16_static: %d queries in one call, the limit is %d; split the batch",
                 Q, B200_DSA_STATIC_MAX_QUERIES);
        b200_set_last_error_text(msg);
        return B200_UNSUPPORTED;
    }
    const uintptr_t align = reinterpret_cast<uintptr_t>(q_nope) | reinterpret_cast<uintptr_t>(q_pe) |
                            reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(kp) |
                            reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out);
    if (align & 15) return B200_BAD_ARG;
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B200_UNSUPPORTED;
    int st = static_scratch_setup(dev);      // first call on a device: not inside a stream capture
    if (st) return st;
    unsigned char* scratch = g_static_scratch_addr[dev];

    // Work split: as many row ranges per query as fill the machine about once, but never more than
    // the built-in array holds partial results for (one (query, range) slot = 128 x 512 fp32 outputs +
    // 128 (max, sum) pairs = 257 KiB).  With one range per query no scratch is needed at all, so every
    // shape the kernel supports is accepted; a large batch simply runs with fewer, longer ranges.
    const int nt_total = S / TKV;
    int NS = 1;
    if (2 * Q < g_static_sm_count[dev]) NS = g_static_sm_count[dev] / (2 * Q);
    if (NS > nt_total) NS = nt_total;
    if (NS > 64) NS = 64;
    const size_t slot_bytes = (size_t)HEADS * DC * sizeof(float) + (size_t)HEADS * 2 * sizeof(float);
    const size_t max_slots = (B200_DSA_STATIC_SCRATCH_BYTES - 512) / slot_bytes;      // 63
    if ((size_t)Q * NS > max_slots) NS = (int)(max_slots / (size_t)Q);
    if (NS < 1) NS = 1;
    const int tps = ceil_div(nt_total, NS);
    NS = ceil_div(nt_total, tps);

    // layout inside the array: [0,256) status word | partial (max,sum) pairs | partial outputs
    const size_t ml_bytes = ((size_t)Q * NS * HEADS * 2 * sizeof(float) + 255) & ~size_t(255);
    const size_t o_bytes = (size_t)Q * NS * HEADS * DC * sizeof(float);
    const size_t need = (NS > 1) ? 256 + ml_bytes + o_bytes : 256;
    if (need > B200_DSA_STATIC_SCRATCH_BYTES) {      // cannot happen after the clamp above; kept as a guard
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "b200_dsa_forward_bf16_static: %d queries x %d splits need %zu bytes of scratch, the built-in "
                 "array holds %u",
                 Q, NS, need, (unsigned)B200_DSA_STATIC_SCRATCH_BYTES);
        b200_set_last_error_text(msg);
        return B200_UNSUPPORTED;
    }
    int* status_word = device_status;
    // the status word must start at zero; the partial results are fully rewritten by the decode
    // kernel before the merge kernel reads them, so stale contents of earlier calls do not matter
    B200_CUDA_TRY(cudaMemsetAsync(status_word, 0, sizeof(int), stream));

    DsaParams p;
    p.q_nope = reinterpret_cast<const __nv_bfloat16*>(q_nope);
    p.q_pe = reinterpret_cast<const __nv_bfloat16*>(q_pe);
    p.kc = reinterpret_cast<const __nv_bfloat16*>(kc);
    p.kp = reinterpret_cast<const __nv_bfloat16*>(kp);
    p.v = reinterpret_cast<const __nv_bfloat16*>(v);
    p.ix = flat_index(idx, cfg); p.out = out; p.status = status_word;
    p.part_ml = reinterpret_cast<float*>(scratch + 256);
    p.part_o = reinterpret_cast<float*>(scratch + 256 + ml_bytes);
    p.H = H; p.S = S; p.NS = NS; p.tiles_per_split = tps;
    p.sl2 = 1.4426950408889634f / sqrtf((float)(DC + DP));
    dsa_decode_bf16_kernel<<<dim3(2, NS, Q), DSA_THREADS, DSA_SMEM_BYTES, stream>>>(p);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    if (NS > 1) {
        dsa_merge_kernel<<<dim3(H, Q), 128, 0, stream>>>(p.part_o, p.part_ml, out, H, NS);
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
    }
    return B200_OK;
}
