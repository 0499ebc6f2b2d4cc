// DSA / MLA sparse decode on bf16 inputs, CTA-pair version (tcgen05 cta_group::2).
//
// Same computation as dsa_decode_bf16_kernel (the fused replacement of kernels/dsa/naive_dsa.cu:435-474),
// re-cut so that a 64-row tile of selected K/V rows can be double-buffered next to a resident Q:
// two CTAs of a cluster work on one (query, row-range) item.  Every MMA spans the pair:
//     S[128 heads, 64 rows]   = Q * K_tile^T        M = 128 (64 heads per CTA), N = 64 (32 rows per CTA)
//     O[128 heads, 512 cols] += P * V_tile          two MMAs of N = 256 (128 columns per CTA each; CTA r
//                                                   supplies and owns output columns [256 r, 256 r + 256))
// so each CTA keeps only its 64 heads of Q (72 KB), gathers only half of the K rows (32 x 1152 B) and
// half of the V columns (64 x 512 B) per tile, and nothing is computed or fetched twice.
// TMEM per CTA: O 256 columns (lanes 0-63: first 128 columns of each 256-wide MMA, lanes 64-127: the
// other 128), S 2 x 32 columns (lanes 0-63: tile rows 0-31, lanes 64-127: rows 32-63).
// The leader CTA (cluster rank 0) issues all MMAs.  Producers and softmax threads signal barriers of their
// own CTA only; one relay thread in the peer forwards each completed barrier to a twin in the leader
// through the cluster address space, and tcgen05.commit signals each CTA in turn.
// Every wait is bounded.
#include <cfloat>

#include "common.cuh"
#include "dsa_index.cuh"

void b200_count_launch(int n);

namespace pair {

constexpr int HEADS = 128, HPC = 64, DC = 512, DP = 64, TKV = 64, KROWS = 32;
constexpr int KBLK = 9;
constexpr int Q_BLK_BYTES = HPC * 128;             // 8192
constexpr int Q_BYTES = KBLK * Q_BLK_BYTES;        // 73728
constexpr int KSLOT_BYTES = KROWS * 128;           // 4096
constexpr int K_STAGE_BYTES = KBLK * KSLOT_BYTES;  // 36864
constexpr int VCHUNK_BYTES = TKV * 128;            // 8192  (64 rows x 64 columns)
constexpr int V_STAGE_BYTES = 4 * VCHUNK_BYTES;    // 32768
constexpr int P_CHUNK_BYTES = HPC * 16;            // 1024
constexpr int P_BYTES = 8 * P_CHUNK_BYTES;         // 8192
constexpr int THREADS = 288;                       // warps 0-3 softmax, 4 MMA/relay, 5-8 gather
constexpr uint32_t O_COL = 0, S_COL = 256;

struct Smem {
    // filled by the CTA's own threads (128 arrivals each)
    uint64_t q_full;
    uint64_t k_full[2];
    uint64_t v_full[2];
    uint64_t s_empty[2];
    uint64_t p_full;
    // twins in the leader, one arrival per use from the peer CTA's relay thread:
    // qk_peer[st]: peer's Q (first use), S buffer and K stage are ready; pv_peer[st]: peer's P and V stage
    uint64_t qk_peer[2];
    uint64_t pv_peer[2];
    // signalled by tcgen05.commit in both CTAs
    uint64_t k_empty[2];
    uint64_t v_empty[2];
    uint64_t s_full[2];
    uint64_t p_empty;
    uint64_t o_done;
    uint64_t mx_bar;                     // local, 128
    uint32_t tmem_base;
    int abort_flag;
    float xchg[2][128];
};
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + 2 * K_STAGE_BYTES + 2 * V_STAGE_BYTES + P_BYTES + sizeof(Smem);

struct Params {
    const __nv_bfloat16 *q_nope, *q_pe, *kc, *kp, *v;
    DsaIndex ix;
    float *out, *part_o, *part_ml;
    int* status;
    int H, S, NS, tiles_per_split;
    float sl2;
};

__device__ __forceinline__ void zero16(uint32_t smem_addr) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(smem_addr), "r"(0) : "memory");
}
// 16 bytes of a selected row into shared memory, or zeros for an empty entry (row < 0)
__device__ __forceinline__ void fetch16(uint32_t smem_addr, const __nv_bfloat16* base, long long row, int row_elems,
                                        int elem_off) {
    if (row >= 0) ptx::cp_async_16(smem_addr, base + row * row_elems + elem_off);
    else          zero16(smem_addr);
}

// ---- cluster-scope helpers --------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on the mbarrier at the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ void mbar_arrive_cta(uint64_t* bar, uint32_t rank) {
    asm volatile(
        "{\n\t.reg .b32 ra;\n\t"
        "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
        "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra];\n\t}"
        ::"r"(ptx::smem_u32(bar)), "r"(rank)
        : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(ptx::smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    uint64_t t0 = 0;                       // the clock is read every 1024 failed polls only (see ptx::mbar_wait)
    uint32_t it = 0;
    while (!mbar_try_wait_cluster(bar, parity)) {
        if (((++it) & 1023u) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > B200_WAIT_LIMIT_NS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// one arrival on the mbarrier at this offset in both CTAs of the pair once all MMAs issued so far
// have retired (two commits, each addressed through the cluster window to one CTA)
__device__ __forceinline__ void commit_both(uint64_t* bar) {
    asm volatile(
        "{\n\t.reg .b32 r0, r1;\n\t"
        "mapa.shared::cluster.u32 r0, %0, 0;\n\t"
        "mapa.shared::cluster.u32 r1, %0, 1;\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [r0];\n\t"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [r1];\n\t}"
        ::"r"(ptx::smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void mma2_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}


__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1) dsa_decode_pair_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = base;
    uint8_t* sK = sQ + Q_BYTES;
    uint8_t* sV = sK + 2 * K_STAGE_BYTES;
    uint8_t* sP = sV + 2 * V_STAGE_BYTES;
    Smem* sm = reinterpret_cast<Smem*>(sP + P_BYTES);
    volatile int* abort_flag = &sm->abort_flag;

    const uint32_t rank = cluster_rank();          // 0 = leader
    const int sp = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt_total = p.S / TKV;
    const int t_begin = sp * p.tiles_per_split;
    const int nt = max(0, min(nt_total, t_begin + p.tiles_per_split) - t_begin);

    if (threadIdx.x == 0) {
        ptx::mbar_init(&sm->q_full, 128);
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(&sm->k_full[s], 128);
            ptx::mbar_init(&sm->v_full[s], 128);
            ptx::mbar_init(&sm->s_empty[s], 128);
            ptx::mbar_init(&sm->qk_peer[s], 1);
            ptx::mbar_init(&sm->pv_peer[s], 1);
            ptx::mbar_init(&sm->k_empty[s], 1);
            ptx::mbar_init(&sm->v_empty[s], 1);
            ptx::mbar_init(&sm->s_full[s], 1);
        }
        ptx::mbar_init(&sm->p_full, 128);
        ptx::mbar_init(&sm->p_empty, 1);
        ptx::mbar_init(&sm->o_done, 1);
        ptx::mbar_init(&sm->mx_bar, 128);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc2(&sm->tmem_base, 512);
        tmem_relinquish2();
    }
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync_all();                            // peer's barriers are initialised before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (warp >= 5) {
        // ===================== gather producers (128 threads per CTA) =====================
        const int pt = threadIdx.x - 160;
        // Q: this CTA's 64 heads x 72 sixteen-byte chunks; heads >= H are zero
        for (int i = pt; i < HPC * 72; i += 128) {
            const int r = i / 72, ch = i - r * 72;
            const int h = (int)rank * HPC + r;
            const uint32_t dst = ptx::smem_u32(sQ) + (ch >> 3) * Q_BLK_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            if (h < p.H) {
                const __nv_bfloat16* src = (ch < 64) ? p.q_nope + ((size_t)b * p.H + h) * DC + ch * 8
                                                     : p.q_pe + ((size_t)b * p.H + h) * DP + (ch - 64) * 8;
                ptx::cp_async_16(dst, src);
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(&sm->q_full);

        // Row ids of the next tile are fetched one tile ahead; the copies of a unit signal its
        // barrier by themselves when they land, so this thread never waits for data and up to two
        // whole tiles (both stages) are in flight.
        // DRAM serves 1 KB of a row fetched in one go at more than twice the rate of the same bytes
        // fetched as scattered 128-byte pieces, so a warp instruction always covers 512 contiguous bytes
        // of one row and the two halves of a Kc row are issued back to back.  Warp w of the four gather
        // warps owns K rows 8w..8w+7 and V rows w, w+4, ...; row ids are fetched one tile ahead.
        const int gw = pt >> 5;                                   // gather warp 0..3
        auto load_ids = [&](int j, long long (&k8)[8], long long (&kp2)[2], long long (&v16)[16]) {
            if (j < nt) {
                const int s0 = (t_begin + j) * TKV;
#pragma unroll
                for (int x = 0; x < 8; x++) k8[x] = dsa_resolve(p.ix, b, s0 + (int)rank * KROWS + 8 * gw + x);
                kp2[0] = dsa_resolve(p.ix, b, s0 + (int)rank * KROWS + 8 * gw + (lane >> 3));
                kp2[1] = dsa_resolve(p.ix, b, s0 + (int)rank * KROWS + 8 * gw + (lane >> 3) + 4);
#pragma unroll
                for (int x = 0; x < 16; x++) v16[x] = dsa_resolve(p.ix, b, s0 + gw + 4 * x);
            }
        };
        long long kid[8], kpid[2] = {0, 0}, vid[16], kid_n[8], kpid_n[2] = {0, 0}, vid_n[16];
#pragma unroll
        for (int x = 0; x < 16; x++) { vid[x] = 0; vid_n[x] = 0; }
#pragma unroll
        for (int x = 0; x < 8; x++) { kid[x] = 0; kid_n[x] = 0; }
        load_ids(0, kid_n, kpid_n, vid_n);
        for (int j = 0; j < nt; j++) {
            const int st = j & 1;
            const uint32_t par = (uint32_t)(((j >> 1) & 1) ^ 1);
#pragma unroll
            for (int x = 0; x < 8; x++) kid[x] = kid_n[x];
            kpid[0] = kpid_n[0]; kpid[1] = kpid_n[1];
#pragma unroll
            for (int x = 0; x < 16; x++) vid[x] = vid_n[x];
            load_ids(j + 1, kid_n, kpid_n, vid_n);
            if (!ptx::mbar_wait(&sm->k_empty[st], par, abort_flag)) goto done;
            {
                const uint32_t kst = ptx::smem_u32(sK) + st * K_STAGE_BYTES;
                // Kc: row r = 8 gw + x, 16-byte chunk ch = lane (+32): slot ch/8, position (ch%8) ^ (r%8)
#pragma unroll
                for (int x = 0; x < 8; x++) {
                    const int r = 8 * gw + x;
#pragma unroll
                    for (int hf = 0; hf < 2; hf++) {
                        const int ch = lane + 32 * hf;
                        fetch16(kst + (ch >> 3) * KSLOT_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4), p.kc, kid[x], DC, ch * 8);
                    }
                }
                // Kp (128 bytes per row, slot 8): four rows per instruction
#pragma unroll
                for (int x = 0; x < 2; x++) {
                    const int r = 8 * gw + (lane >> 3) + 4 * x, j16 = lane & 7;
                    fetch16(kst + 8 * KSLOT_BYTES + r * 128 + ((j16 ^ (r & 7)) << 4), p.kp, kpid[x], DP, j16 * 8);
                }
            }
            __threadfence_block();                 // zero-filled rows of empty entries are written before the arrival
            ptx::cp_async_arrive_noinc(&sm->k_full[st]);
            {
                if (!ptx::mbar_wait(&sm->v_empty[st], par, abort_flag)) goto done;
                const uint32_t vbase = ptx::smem_u32(sV) + st * V_STAGE_BYTES;
                // this CTA's 512 contiguous bytes of a V row: columns [256 rank, 256 rank + 256);
                // 64-column chunk q = lane / 8 (MMA q/2, half q%2)
                const int q = lane >> 3, v16 = lane & 7;
                const uint32_t chunk = vbase + q * VCHUNK_BYTES;
#pragma unroll
                for (int x = 0; x < 16; x++) {
                    const int r = gw + 4 * x;
                    fetch16(chunk + (r >> 3) * 1024 + (r & 7) * 128 + ((v16 ^ (r & 7)) << 4), p.v, vid[x], DC,
                            256 * (int)rank + lane * 8);
                }
                __threadfence_block();
                ptx::cp_async_arrive_noinc(&sm->v_full[st]);
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();           // nothing of this thread is in flight when the CTA winds down
    } else if (warp == 4) {
        // ===================== MMA issuer (leader) / barrier relay (peer) =====================
        // Both threads walk the same sequence of waits.  The peer's thread forwards each completed
        // local barrier to its twin in the leader; the leader waits for its own barrier and the twin.
        if (lane == 0 && nt > 0) {
            const bool leader = (rank == 0);
            constexpr uint32_t idesc_qk = ptx::make_idesc(1, 1, 0, 0, HEADS, TKV);
            constexpr uint32_t idesc_pv = ptx::make_idesc(1, 1, 0, 1, HEADS, 256);
            const uint32_t q_addr = ptx::smem_u32(sQ), k_addr = ptx::smem_u32(sK), v_addr = ptx::smem_u32(sV),
                           p_addr = ptx::smem_u32(sP);
            // The data behind the local barriers was written through the generic proxy (cp.async,
            // st.shared) and is read by the tensor core through the async proxy: fence after waiting.
            auto forward_or_wait = [&](uint64_t* peer, uint32_t par_peer) -> bool {
                ptx::fence_proxy_async_smem();
                if (leader) return mbar_wait_cluster(peer, par_peer, abort_flag);
                mbar_arrive_cta(peer, 0);
                return true;
            };
            auto issue_pv = [&](int i) -> bool {
                const int st = i & 1;
                const uint32_t par = (uint32_t)((i >> 1) & 1);
                if (!ptx::mbar_wait(&sm->p_full, (uint32_t)(i & 1), abort_flag)) return false;
                if (!ptx::mbar_wait(&sm->v_full[st], par, abort_flag)) return false;
                if (!forward_or_wait(&sm->pv_peer[st], par)) return false;
                if (!leader) return true;
                ptx::tc_fence_after();
#pragma unroll
                for (int inst = 0; inst < 2; inst++) {
#pragma unroll
                    for (int ks = 0; ks < 4; ks++) {
                        uint64_t ad = ptx::make_smem_desc(p_addr + ks * 2 * P_CHUNK_BYTES, P_CHUNK_BYTES, 128, 0);
                        uint64_t bd = ptx::make_smem_desc(v_addr + st * V_STAGE_BYTES + 2 * inst * VCHUNK_BYTES + ks * 2048,
                                                          VCHUNK_BYTES, 1024, 2);
                        mma2_f16(tmem + O_COL + 128 * inst, ad, bd, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                    }
                }
                commit_both(&sm->v_empty[st]);
                commit_both(&sm->p_empty);
                return true;
            };
            if (!ptx::mbar_wait(&sm->q_full, 0, abort_flag)) goto done;
            for (int j = 0; j < nt; j++) {
                const int st = j & 1;                           // K stage and S buffer of this tile
                const uint32_t par = (uint32_t)((j >> 1) & 1);
                if (!ptx::mbar_wait(&sm->s_empty[st], par ^ 1, abort_flag)) goto done;   // passes at once on first use
                if (!ptx::mbar_wait(&sm->k_full[st], par, abort_flag)) goto done;
                if (!forward_or_wait(&sm->qk_peer[st], par)) goto done;
                if (leader) {
                    ptx::tc_fence_after();
#pragma unroll
                    for (int c = 0; c < KBLK; c++) {
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            uint64_t ad = ptx::make_smem_desc(q_addr + c * Q_BLK_BYTES + k4 * 32, 16, 1024, 2);
                            uint64_t bd = ptx::make_smem_desc(k_addr + st * K_STAGE_BYTES + c * KSLOT_BYTES + k4 * 32,
                                                              16, 1024, 2);
                            mma2_f16(tmem + S_COL + st * 32, ad, bd, idesc_qk, (c > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    commit_both(&sm->k_empty[st]);
                    commit_both(&sm->s_full[st]);
                }
                if (j > 0 && !issue_pv(j - 1)) goto done;
            }
            if (!issue_pv(nt - 1)) goto done;
            if (leader) commit_both(&sm->o_done);
        }
    } else {
        // ===================== softmax / correction / epilogue (warps 0-3 of each CTA) =====================
        const int t = threadIdx.x;                       // TMEM lane
        const int hl = t & 63, hh = t >> 6;              // local head, column half held by this lane
        const int head = (int)rank * HPC + hl;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float m = -1e30f, l = 0.0f;
        const float thr = 8.0f / p.sl2;
        // which of this lane's 32 score columns (tile rows 32 hh .. +31) are empty entries: one bit per row,
        // looked up one tile ahead
        // (the entry is fetched during the previous tile and only looked at here, so its latency is hidden)
        int ent_n = (nt > 0) ? dsa_resolve(p.ix, b, t_begin * TKV + 32 * hh + lane) : -1;
        for (int j = 0; j < nt; j++) {
            const int sb = j & 1;
            const unsigned mask = __ballot_sync(0xffffffffu, ent_n >= 0);
            if (j + 1 < nt) ent_n = dsa_resolve(p.ix, b, (t_begin + j + 1) * TKV + 32 * hh + lane);
            if (!ptx::mbar_wait(&sm->s_full[sb], (uint32_t)((j >> 1) & 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem + lane_addr + S_COL + sb * 32, r);
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
            // the other half of this head's 64 scores lives in lane t ^ 64
            sm->xchg[sb][t] = tmax;
            ptx::mbar_arrive(&sm->mx_bar);
            if (!ptx::mbar_wait(&sm->mx_bar, (uint32_t)(j & 1), abort_flag)) goto done;
            tmax = fmaxf(tmax, sm->xchg[sb][t ^ 64]);
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
            if (!ptx::mbar_wait(&sm->p_empty, (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c0 = 0; c0 < 256; c0 += 32) {
                    uint32_t o[32];
                    ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                    ptx::tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    ptx::tmem_st_32x32(tmem + lane_addr + O_COL + c0, o);
                }
                ptx::tc_wait_st();
            }
            // P[hl, 32*hh + 0..31]: 16-byte chunk ch = 4*hh + q at ch*1024 + hl*16
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t dst = ptx::smem_u32(sP) + (4 * hh + q) * P_CHUNK_BYTES + hl * 16;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * q]), "r"(pk[4 * q + 1]),
                             "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
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
        // total row sum = this lane's half + the partner lane's half
        sm->xchg[nt & 1][t] = l;
        ptx::mbar_arrive(&sm->mx_bar);
        if (!ptx::mbar_wait(&sm->mx_bar, (uint32_t)(nt & 1), abort_flag)) goto done;
        l += sm->xchg[nt & 1][t ^ 64];
        const bool direct = (p.NS == 1);
        const float inv = (direct && l > 0.0f) ? 1.0f / l : 1.0f;
        float* row = direct ? p.out + ((size_t)b * p.H + head) * DC
                            : p.part_o + (((size_t)b * p.NS + sp) * HEADS + head) * DC;
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            if (nt > 0) {
                ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                ptx::tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = 0;
            }
            // TMEM column c0 of this lane = output column 256*hh + c0 (lanes 64-127 hold the peer's V columns)
            if (head < p.H || !direct) {
                float4* d4 = reinterpret_cast<float4*>(row + 256 * hh + c0);
#pragma unroll
                for (int i = 0; i < 8; i++)
                    d4[i] = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                        __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
            }
        }
        if (!direct && hh == 0) {
            float* ml = p.part_ml + (((size_t)b * p.NS + sp) * HEADS + head) * 2;
            ml[0] = (nt > 0) ? m * p.sl2 : -1e30f;
            ml[1] = l;
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync_all();                  // the pair's MMAs and TMEM reads are over in both CTAs
    if (warp == 4) tmem_dealloc2(tmem, 512);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(p.status, B200_TIMEOUT);
}


// =================================================================================================
// 128-row tiles.  tcgen05.mma has a minimum issue interval of a few tens of nanoseconds whatever its
// shape, so the 36 K-steps of Q K^T cost the same for 64 rows as for 128: with 64-row tiles the tensor
// pipe, not HBM, bounded the kernel.  Here a tile is 128 selected rows (N = 128 for Q K^T, eight
// K-steps per P V half), which leaves room for one K stage (72 KB) and one V stage (64 KB) per CTA next
// to Q (72 KB) and P (16 KB).  The K stage refills while P V of the previous tile and the softmax run,
// the V stage while Q K^T of the next tile runs; K and V have their own gather warps so that neither
// waits behind the other's free-slot barrier.
namespace t128 {

constexpr int TKV = 128, KROWS = 64;
constexpr int KSLOT_BYTES = KROWS * 128;           // 8192: 64 rows of one 128-byte column block
constexpr int K_STAGE_BYTES = KBLK * KSLOT_BYTES;  // 73728
constexpr int VCHUNK_BYTES = TKV * 128;            // 16384 (128 rows x 64 columns)
constexpr int V_STAGE_BYTES = 4 * VCHUNK_BYTES;    // 65536
constexpr int P_BYTES = 16 * P_CHUNK_BYTES;        // 16384
constexpr uint32_t S_COL = 256;                    // two score buffers of 64 columns
constexpr int NKW = 4, NVW = 4;                    // gather warps for K rows and for V rows
constexpr int NPROD = 32 * (NKW + NVW);
constexpr int THREADS128 = 160 + NPROD;            // warps 0-3 softmax, 4 MMA/relay, then K and V gather warps

struct Smem {
    uint64_t q_full;          // all gather threads
    uint64_t k_full, v_full;  // the K gather threads, the V gather threads
    uint64_t s_empty[2];      // 128 softmax threads
    uint64_t p_full;          // 128 softmax threads
    uint64_t qk_peer, pv_peer;   // twins in the leader: one arrival per tile from the peer's relay thread
    uint64_t k_empty, v_empty, s_full[2], p_empty, o_done;   // tcgen05.commit, both CTAs
    uint64_t mx_bar;          // 128 softmax threads
    uint32_t tmem_base;
    int abort_flag;
    float xchg[2][128];
};
constexpr size_t SMEM_BYTES = 1024 + Q_BYTES + K_STAGE_BYTES + V_STAGE_BYTES + P_BYTES + sizeof(Smem);
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS128, 1) dsa_decode_pair128_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = base;
    uint8_t* sK = sQ + Q_BYTES;
    uint8_t* sV = sK + K_STAGE_BYTES;
    uint8_t* sP = sV + V_STAGE_BYTES;
    Smem* sm = reinterpret_cast<Smem*>(sP + P_BYTES);
    volatile int* abort_flag = &sm->abort_flag;

    const uint32_t rank = cluster_rank();          // 0 = leader
    const int sp = blockIdx.y, b = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nt_total = p.S / TKV;
    const int t_begin = sp * p.tiles_per_split;
    const int nt = max(0, min(nt_total, t_begin + p.tiles_per_split) - t_begin);

    if (threadIdx.x == 0) {
        ptx::mbar_init(&sm->q_full, NPROD);
        ptx::mbar_init(&sm->k_full, 32 * NKW);
        ptx::mbar_init(&sm->v_full, 32 * NVW);
        for (int s = 0; s < 2; s++) {
            ptx::mbar_init(&sm->s_empty[s], 128);
            ptx::mbar_init(&sm->s_full[s], 1);
        }
        ptx::mbar_init(&sm->p_full, 128);
        ptx::mbar_init(&sm->qk_peer, 1);
        ptx::mbar_init(&sm->pv_peer, 1);
        ptx::mbar_init(&sm->k_empty, 1);
        ptx::mbar_init(&sm->v_empty, 1);
        ptx::mbar_init(&sm->p_empty, 1);
        ptx::mbar_init(&sm->o_done, 1);
        ptx::mbar_init(&sm->mx_bar, 128);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 4) {
        tmem_alloc2(&sm->tmem_base, 512);
        tmem_relinquish2();
    }
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync_all();                            // peer's barriers are initialised before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    // Launched with programmatic stream serialisation: everything above overlaps the tail of the
    // previous kernel in the stream; nothing below reads or writes global memory before that kernel
    // has completed.  (Both instructions are no-ops under an ordinary launch.)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp >= 5) {
        // ===================== gather producers: NKW warps for K rows, NVW warps for V rows =====================
        const int pt = threadIdx.x - 160;
        // Q: this CTA's 64 heads x 72 sixteen-byte chunks; heads >= H are zero
        for (int i = pt; i < HPC * 72; i += NPROD) {
            const int r = i / 72, ch = i - r * 72;
            const int h = (int)rank * HPC + r;
            const uint32_t dst = ptx::smem_u32(sQ) + (ch >> 3) * Q_BLK_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            if (h < p.H) {
                const __nv_bfloat16* src = (ch < 64) ? p.q_nope + ((size_t)b * p.H + h) * DC + ch * 8
                                                     : p.q_pe + ((size_t)b * p.H + h) * DP + (ch - 64) * 8;
                ptx::cp_async_16(dst, src);
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0) : "memory");
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(&sm->q_full);

        // A warp instruction always covers 512 contiguous bytes of one row (DRAM serves such pieces at
        // more than twice the rate of scattered 128-byte ones).  Each lane fetches the ids of the rows
        // its warp owns one tile ahead and hands them round by shuffle; the copies of a tile signal its
        // barrier by themselves when they land, so these threads never wait for data.
        const int s_begin = t_begin * TKV;
        if (pt < 32 * NKW) {
            constexpr int RPW = KROWS / NKW;                      // K rows per warp
            const int kw = pt >> 5;                               // rows RPW kw .. RPW kw + RPW - 1 of this CTA's 64
            const int my = (int)rank * KROWS + RPW * kw + (lane % RPW);
            int id_n = (nt > 0) ? dsa_resolve(p.ix, b, s_begin + my) : -1;
            const uint32_t kst = ptx::smem_u32(sK);
            for (int j = 0; j < nt; j++) {
                const int id = id_n;
                if (j + 1 < nt) id_n = dsa_resolve(p.ix, b, s_begin + (j + 1) * TKV + my);
                if (!ptx::mbar_wait(&sm->k_empty, (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
                // Kc: row r, 16-byte chunk ch = lane (+32): slot ch/8, position (ch%8) ^ (r%8)
                if (__all_sync(0xffffffffu, id >= 0)) {
                    // every row of this warp is live (the usual case): copies only, no per-row test
#pragma unroll 8
                    for (int x = 0; x < RPW; x++) {
                        const size_t rid = (size_t)__shfl_sync(0xffffffffu, id, x);
                        const int r = RPW * kw + x;
#pragma unroll
                        for (int hf = 0; hf < 2; hf++) {
                            const int ch = lane + 32 * hf;
                            ptx::cp_async_16(kst + (ch >> 3) * KSLOT_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4),
                                             p.kc + rid * DC + ch * 8);
                        }
                    }
                    // Kp (128 bytes per row, slot 8): four rows per instruction
#pragma unroll
                    for (int x = 0; x < RPW / 4; x++) {
                        const int rr = 4 * x + (lane >> 3), j16 = lane & 7;
                        const size_t rid = (size_t)__shfl_sync(0xffffffffu, id, rr);
                        const int r = RPW * kw + rr;
                        ptx::cp_async_16(kst + 8 * KSLOT_BYTES + r * 128 + ((j16 ^ (r & 7)) << 4), p.kp + rid * DP + j16 * 8);
                    }
                } else {
#pragma unroll 4
                    for (int x = 0; x < RPW; x++) {
                        const long long rid = __shfl_sync(0xffffffffu, id, x);
                        const int r = RPW * kw + x;
#pragma unroll
                        for (int hf = 0; hf < 2; hf++) {
                            const int ch = lane + 32 * hf;
                            fetch16(kst + (ch >> 3) * KSLOT_BYTES + r * 128 + (((ch & 7) ^ (r & 7)) << 4), p.kc, rid, DC, ch * 8);
                        }
                    }
#pragma unroll
                    for (int x = 0; x < RPW / 4; x++) {
                        const int rr = 4 * x + (lane >> 3), j16 = lane & 7;
                        const long long rid = __shfl_sync(0xffffffffu, id, rr);
                        const int r = RPW * kw + rr;
                        fetch16(kst + 8 * KSLOT_BYTES + r * 128 + ((j16 ^ (r & 7)) << 4), p.kp, rid, DP, j16 * 8);
                    }
                    __threadfence_block();         // zero-filled rows are written before the arrival
                }
                ptx::cp_async_arrive_noinc(&sm->k_full);
                // pull the next tile's rows into L2 while this tile is on its way
                if (j + 1 < nt && lane < RPW && id_n >= 0) {
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.kc + (size_t)id_n * DC), "r"(DC * 2) : "memory");
                    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.kp + (size_t)id_n * DP), "r"(DP * 2) : "memory");
                }
            }
        } else {
            constexpr int VPW = TKV / NVW;                        // V rows per warp (32 or 64)
            const int vw = (pt - 32 * NKW) >> 5;                  // V rows vw, vw + NVW, ... of the tile's 128
            const int my0 = vw + NVW * lane, my1 = (VPW > 32) ? vw + NVW * (lane + 32) : my0;
            int id0_n = -1, id1_n = -1;
            if (nt > 0) { id0_n = dsa_resolve(p.ix, b, s_begin + my0); id1_n = dsa_resolve(p.ix, b, s_begin + my1); }
            // this CTA's 512 contiguous bytes of a V row: columns [256 rank, 256 rank + 256);
            // 64-column chunk q = lane / 8 (MMA q/2, half q%2)
            const int q = lane >> 3, v16 = lane & 7;
            const uint32_t chunk = ptx::smem_u32(sV) + q * VCHUNK_BYTES;
            for (int j = 0; j < nt; j++) {
                const int id0 = id0_n, id1 = id1_n;
                if (j + 1 < nt) {
                    id0_n = dsa_resolve(p.ix, b, s_begin + (j + 1) * TKV + my0);
                    id1_n = dsa_resolve(p.ix, b, s_begin + (j + 1) * TKV + my1);
                }
                if (!ptx::mbar_wait(&sm->v_empty, (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
                if (__all_sync(0xffffffffu, (id0 >= 0) && (id1 >= 0))) {
#pragma unroll 8
                    for (int x = 0; x < VPW; x++) {
                        const size_t rid = (size_t)__shfl_sync(0xffffffffu, (x < 32) ? id0 : id1, x & 31);
                        const int r = vw + NVW * x;
                        ptx::cp_async_16(chunk + (r >> 3) * 1024 + (r & 7) * 128 + ((v16 ^ (r & 7)) << 4),
                                         p.v + rid * DC + 256 * (int)rank + lane * 8);
                    }
                } else {
#pragma unroll 4
                    for (int x = 0; x < VPW; x++) {
                        const long long rid = __shfl_sync(0xffffffffu, (x < 32) ? id0 : id1, x & 31);
                        const int r = vw + NVW * x;
                        fetch16(chunk + (r >> 3) * 1024 + (r & 7) * 128 + ((v16 ^ (r & 7)) << 4), p.v, rid, DC,
                                256 * (int)rank + lane * 8);
                    }
                    __threadfence_block();
                }
                ptx::cp_async_arrive_noinc(&sm->v_full);
                if (j + 1 < nt) {
                    if (id0_n >= 0)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.v + (size_t)id0_n * DC + 256 * (int)rank), "r"(512) : "memory");
                    if (VPW > 32 && id1_n >= 0)
                        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.v + (size_t)id1_n * DC + 256 * (int)rank), "r"(512) : "memory");
                }
            }
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();           // nothing of this thread is in flight when the CTA winds down
    } else if (warp == 4) {
        // ===================== MMA issuer (leader) / barrier relay (peer) =====================
        if (lane == 0 && nt > 0) {
            const bool leader = (rank == 0);
            constexpr uint32_t idesc_qk = ptx::make_idesc(1, 1, 0, 0, HEADS, TKV);
            constexpr uint32_t idesc_pv = ptx::make_idesc(1, 1, 0, 1, HEADS, 256);
            const uint32_t q_addr = ptx::smem_u32(sQ), k_addr = ptx::smem_u32(sK), v_addr = ptx::smem_u32(sV),
                           p_addr = ptx::smem_u32(sP);
            auto forward_or_wait = [&](uint64_t* peer, uint32_t par_peer) -> bool {
                ptx::fence_proxy_async_smem();
                if (leader) return mbar_wait_cluster(peer, par_peer, abort_flag);
                mbar_arrive_cta(peer, 0);
                return true;
            };
            auto issue_pv = [&](int i) -> bool {
                const uint32_t par = (uint32_t)(i & 1);
                if (!ptx::mbar_wait(&sm->p_full, par, abort_flag)) return false;
                if (!ptx::mbar_wait(&sm->v_full, par, abort_flag)) return false;
                if (!forward_or_wait(&sm->pv_peer, par)) return false;
                if (!leader) return true;
                ptx::tc_fence_after();
#pragma unroll
                for (int inst = 0; inst < 2; inst++) {
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        uint64_t ad = ptx::make_smem_desc(p_addr + ks * 2 * P_CHUNK_BYTES, P_CHUNK_BYTES, 128, 0);
                        uint64_t bd = ptx::make_smem_desc(v_addr + 2 * inst * VCHUNK_BYTES + ks * 2048, VCHUNK_BYTES, 1024, 2);
                        mma2_f16(tmem + O_COL + 128 * inst, ad, bd, idesc_pv, (i > 0 || ks > 0) ? 1u : 0u);
                    }
                }
                commit_both(&sm->v_empty);
                commit_both(&sm->p_empty);
                return true;
            };
            if (!ptx::mbar_wait(&sm->q_full, 0, abort_flag)) goto done;
            for (int j = 0; j < nt; j++) {
                const int sb = j & 1;
                if (!ptx::mbar_wait(&sm->s_empty[sb], (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) goto done;
                if (!ptx::mbar_wait(&sm->k_full, (uint32_t)(j & 1), abort_flag)) goto done;
                if (!forward_or_wait(&sm->qk_peer, (uint32_t)(j & 1))) goto done;
                if (leader) {
                    ptx::tc_fence_after();
#pragma unroll
                    for (int c = 0; c < KBLK; c++) {
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            uint64_t ad = ptx::make_smem_desc(q_addr + c * Q_BLK_BYTES + k4 * 32, 16, 1024, 2);
                            uint64_t bd = ptx::make_smem_desc(k_addr + c * KSLOT_BYTES + k4 * 32, 16, 1024, 2);
                            mma2_f16(tmem + S_COL + sb * 64, ad, bd, idesc_qk, (c > 0 || k4 > 0) ? 1u : 0u);
                        }
                    }
                    commit_both(&sm->k_empty);
                    commit_both(&sm->s_full[sb]);
                }
                if (j > 0 && !issue_pv(j - 1)) goto done;
            }
            if (!issue_pv(nt - 1)) goto done;
            if (leader) commit_both(&sm->o_done);
        }
    } else {
        // ===================== softmax / correction / epilogue (warps 0-3 of each CTA) =====================
        const int t = threadIdx.x;                       // TMEM lane
        const int hl = t & 63, hh = t >> 6;              // local head, half of the tile / of the columns held here
        const int head = (int)rank * HPC + hl;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        float m = -1e30f, l = 0.0f;
        const float thr = 8.0f / p.sl2;
        // which of this lane's 64 score columns (tile rows 64 hh .. +63) are empty entries: one bit per row,
        // looked up one tile ahead (two index loads per lane and tile)
        // (the entries are fetched during the previous tile and only looked at here, so their latency is hidden)
        int e0_n = -1, e1_n = -1;
        if (nt > 0) {
            e0_n = dsa_resolve(p.ix, b, t_begin * TKV + 64 * hh + lane);
            e1_n = dsa_resolve(p.ix, b, t_begin * TKV + 64 * hh + 32 + lane);
        }
        for (int j = 0; j < nt; j++) {
            const int sb = j & 1;
            const unsigned mlo = __ballot_sync(0xffffffffu, e0_n >= 0), mhi = __ballot_sync(0xffffffffu, e1_n >= 0);
            if (j + 1 < nt) {
                e0_n = dsa_resolve(p.ix, b, (t_begin + j + 1) * TKV + 64 * hh + lane);
                e1_n = dsa_resolve(p.ix, b, (t_begin + j + 1) * TKV + 64 * hh + 32 + lane);
            }
            if (!ptx::mbar_wait(&sm->s_full[sb], (uint32_t)((j >> 1) & 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            uint32_t r[64];
            ptx::tmem_ld_32x64(tmem + lane_addr + S_COL + sb * 64, r);
            ptx::tc_wait_ld();
            ptx::tc_fence_before();
            ptx::mbar_arrive(&sm->s_empty[sb]);
            if ((mlo & mhi) != 0xffffffffu) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    r[i] = ((mlo >> i) & 1u) ? r[i] : 0xff800000u;              // -inf
                    r[32 + i] = ((mhi >> i) & 1u) ? r[32 + i] : 0xff800000u;
                }
            }
            float tmax = -FLT_MAX;
#pragma unroll
            for (int i = 0; i < 64; i++) tmax = fmaxf(tmax, __uint_as_float(r[i]));
            // the other half of this head's 128 scores lives in lane t ^ 64
            sm->xchg[sb][t] = tmax;
            ptx::mbar_arrive(&sm->mx_bar);
            if (!ptx::mbar_wait(&sm->mx_bar, (uint32_t)(j & 1), abort_flag)) goto done;
            tmax = fmaxf(tmax, sm->xchg[sb][t ^ 64]);
            const bool need = tmax > m + thr;
            const float m_new = need ? tmax : m;
            const float corr = need ? exp2f((m - m_new) * p.sl2) : 1.0f;
            float rowsum = 0.0f;
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; i++) {
                float p0 = exp2f((__uint_as_float(r[2 * i]) - m_new) * p.sl2);
                float p1 = exp2f((__uint_as_float(r[2 * i + 1]) - m_new) * p.sl2);
                rowsum += p0 + p1;
                __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
                pk[i] = *reinterpret_cast<uint32_t*>(&h2);
            }
            if (!ptx::mbar_wait(&sm->p_empty, (uint32_t)((j & 1) ^ 1), abort_flag)) goto done;
            ptx::tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
                for (int c0 = 0; c0 < 256; c0 += 32) {
                    uint32_t o[32];
                    ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                    ptx::tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    ptx::tmem_st_32x32(tmem + lane_addr + O_COL + c0, o);
                }
                ptx::tc_wait_st();
            }
            // P[hl, 64*hh + 0..63]: 16-byte chunk ch = 8*hh + q at ch*1024 + hl*16
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const uint32_t dst = ptx::smem_u32(sP) + (8 * hh + q) * P_CHUNK_BYTES + hl * 16;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pk[4 * q]), "r"(pk[4 * q + 1]),
                             "r"(pk[4 * q + 2]), "r"(pk[4 * q + 3])
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
        // total row sum = this lane's half + the partner lane's half
        sm->xchg[nt & 1][t] = l;
        ptx::mbar_arrive(&sm->mx_bar);
        if (!ptx::mbar_wait(&sm->mx_bar, (uint32_t)(nt & 1), abort_flag)) goto done;
        l += sm->xchg[nt & 1][t ^ 64];
        const bool direct = (p.NS == 1);
        const float inv = (direct && l > 0.0f) ? 1.0f / l : 1.0f;
        // Rows of this warp: heads 32 (warp & 1) .. +31 of this CTA, output columns 256 hh + [0, 256).
        // Each 32-column chunk goes through a padded staging tile (the K stage is free by now) so that
        // a store instruction writes four full 128-byte lines instead of 32 scattered 16-byte pieces.
        float* wrow0 = direct ? p.out + ((size_t)b * p.H + (int)rank * HPC + 32 * (warp & 1)) * DC
                              : p.part_o + (((size_t)b * p.NS + sp) * HEADS + (int)rank * HPC + 32 * (warp & 1)) * DC;
        const int rows_ok = direct ? max(0, min(32, p.H - ((int)rank * HPC + 32 * (warp & 1)))) : 32;
        float* stg = reinterpret_cast<float*>(sK) + warp * (32 * 36);
#pragma unroll 1
        for (int c0 = 0; c0 < 256; c0 += 32) {
            uint32_t o[32];
            if (nt > 0) {
                ptx::tmem_ld_32x32(tmem + lane_addr + O_COL + c0, o);
                ptx::tc_wait_ld();
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = 0;
            }
            // TMEM column c0 of this lane = output column 256*hh + c0 (lanes 64-127 hold the peer's V columns)
            float4* s4 = reinterpret_cast<float4*>(stg + lane * 36);
#pragma unroll
            for (int i = 0; i < 8; i++)
                s4[i] = make_float4(__uint_as_float(o[4 * i]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                    __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
            __syncwarp();
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int r = 4 * k + (lane >> 3), c4 = lane & 7;
                const float4 v4 = *reinterpret_cast<const float4*>(stg + r * 36 + 4 * c4);
                if (r < rows_ok) *reinterpret_cast<float4*>(wrow0 + (size_t)r * DC + 256 * hh + c0 + 4 * c4) = v4;
            }
            __syncwarp();
        }
        if (!direct && hh == 0) {
            float* ml = p.part_ml + (((size_t)b * p.NS + sp) * HEADS + head) * 2;
            ml[0] = (nt > 0) ? m * p.sl2 : -1e30f;
            ml[1] = l;
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync_all();                  // the pair's MMAs and TMEM reads are over in both CTAs
    if (warp == 4) tmem_dealloc2(tmem, 512);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(p.status, B200_TIMEOUT);
}

}  // namespace t128

}  // namespace pair


// Host side: called by b200_dsa_forward_bf16 with tile_rows = 128 (S % 128 == 0) or 64 (S % 64 == 0);
// tiles_per_split counts tiles of that size.
int b200_launch_dsa_pair(const void* q_nope, const void* q_pe, const void* kc, const void* kp, const void* v,
                         const DsaIndex& ix, float* out, float* part_o, float* part_ml, int* status, int Q, int H, int S,
                         int NS, int tiles_per_split, int tile_rows, cudaStream_t stream) {
    static bool attr_done[64] = {false};
    if (b200_first_call_on_device(attr_done)) {
        B200_CUDA_TRY(cudaFuncSetAttribute(pair::dsa_decode_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)pair::SMEM_BYTES));
        B200_CUDA_TRY(cudaFuncSetAttribute(pair::t128::dsa_decode_pair128_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pair::t128::SMEM_BYTES));
    }
    pair::Params p;
    p.q_nope = static_cast<const __nv_bfloat16*>(q_nope);
    p.q_pe = static_cast<const __nv_bfloat16*>(q_pe);
    p.kc = static_cast<const __nv_bfloat16*>(kc);
    p.kp = static_cast<const __nv_bfloat16*>(kp);
    p.v = static_cast<const __nv_bfloat16*>(v);
    p.ix = ix; p.out = out; p.part_o = part_o; p.part_ml = part_ml; p.status = status;
    p.H = H; p.S = S; p.NS = NS; p.tiles_per_split = tiles_per_split;
    p.sl2 = 1.4426950408889634f / sqrtf((float)(pair::DC + pair::DP));
    if (tile_rows == 128) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2, NS, Q);
        cfg.blockDim = dim3(pair::t128::THREADS128);
        cfg.dynamicSmemBytes = pair::t128::SMEM_BYTES;
        cfg.stream = stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, pair::t128::dsa_decode_pair128_kernel, p));
    } else
        pair::dsa_decode_pair_kernel<<<dim3(2, NS, Q), pair::THREADS, pair::SMEM_BYTES, stream>>>(p);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
