// FP8 (e4m3) block-scale MoE expert path for sm_100a.
//
// Replaces the reference's per-expert host loop (kernels/moe/naive_moe.cu:424-469: gather,
// D2H count + stream sync, GEMM1, SwiGLU, GEMM2, scatter; 5 launches and one host sync per
// expert) with one row-sort pass and two persistent grouped GEMM launches:
//
//   sort_rows_fp8_kernel   expert-sorted copy of the FP8 rows + 1x128 scales, and the
//                          row -> token / router-weight maps.
//   grouped_gemm_fp8<1>    act = requant_1x128( silu(x W1g^T) * (x W1u^T) )   (SwiGLU and
//                          requantisation fused in the epilogue: no fp32 GEMM1 output in HBM)
//   grouped_gemm_fp8<2>    out[token] += w * (act W2^T)                      (router weight and
//                          scatter-add fused in the epilogue)
//   grouped_gemm_fp8<3>    rows[r] = w * (act W2^T), then reduce_rows_kernel sums a token's rows
//                          in ascending expert order (the reference's order, naive_moe.cu:424):
//                          the bit-reproducible alternative to the scatter-add.
//
// GEMM structure (one CTA per SM, 384 threads, tiles 128 x 256 x 128 handed out round-robin,
// expert-major):
//   warp 8       TMA producer: A tile (128 rows x 128 B) and B tile (256 rows x 128 B) per
//                K block into a 4-stage shared-memory ring (128-byte swizzle, K-major).
//   warps 9,10   MMA issuers, one per 256-column TMEM accumulator stage (K blocks alternate between
//                them): 4 x tcgen05.mma kind::f8f6f4 (K = 32 each) per K block, started fresh for
//                every K block.  Everything that waits next to the promotion warps sleeps between
//                polls: a warp that spins takes issue slots from the promotion warps that share
//                its scheduler.
//   warps 0-7    promotion + epilogue: tcgen05.ld the K block's partial sums and fold them
//                into fp32 registers with a_scale[row,kb] * w_scale[nblk,kb] (the scales are
//                arbitrary fp32 values, so the scaling cannot be left to the tensor core).
//                Warp w owns TMEM lanes 32 (w % 4) .. +31 (the tile rows) and accumulator columns
//                128 (w / 4) .. +127: 128 running sums per thread.  (A build with 16 promotion warps
//                and 64 sums each, -DB200_GEMM_PROMO_WARPS=16, measured no faster; neither did packed
//                fma.rn.f32x2 arithmetic, -DB200_GEMM_PACKED_FMA.)
// Every mbarrier wait is bounded; on give-up the CTA flags B200_TIMEOUT and winds down.
#include "common.cuh"
#include "moe_internal.cuh"
#include "tma_host.cuh"

void b200_set_last_error_text(const char* text);

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;            // 16384
constexpr int B_BYTES = BN * BK;            // 32768
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
#ifndef B200_GEMM_PROMO_WARPS
#define B200_GEMM_PROMO_WARPS 8
#endif
constexpr int NUM_PROMO_WARPS = B200_GEMM_PROMO_WARPS;   // 8 or 16; one barrier arrival and one polling lane per warp
constexpr int NQ = NUM_PROMO_WARPS / 4;      // column groups of the accumulator (TMEM lanes fix the row split at 4)
constexpr int QCOLS = BN / NQ;               // accumulator columns per promotion thread
constexpr int GEMM_THREADS = 32 * (NUM_PROMO_WARPS + 4);   // promotion/epilogue warpgroups, then the TMA + MMA warpgroup
constexpr int W_TMA = NUM_PROMO_WARPS, W_MMA0 = NUM_PROMO_WARPS + 1;
constexpr int MAX_E = 1024;
constexpr unsigned ISSUER_SLEEP_NS = 64;
// Register budgets after setmaxnreg.  The registers a warpgroup gives up are the only ones the others can
// take (the pool is what the CTA was launched with: GEMM_THREADS x LAUNCH_REGS), and setmaxnreg.inc waits
// without bound until its request is met, so the two sides must balance:
// promotion threads x (PROMO_REGS - LAUNCH_REGS) <= 128 x (LAUNCH_REGS - AUX_REGS).  The launcher checks
// the compiled register count against this before the first launch.
constexpr int LAUNCH_REGS = (NUM_PROMO_WARPS == 8) ? 168 : 96;
constexpr int PROMO_REGS = (NUM_PROMO_WARPS == 8) ? 232 : 112;
constexpr int AUX_REGS = (NUM_PROMO_WARPS == 8) ? 40 : 32;
// columns per promotion load (two loads in flight)
#ifndef B200_GEMM_PROMO_CH
#define B200_GEMM_PROMO_CH ((B200_GEMM_PROMO_WARPS == 8) ? 32 : 8)
#endif
constexpr int CH = B200_GEMM_PROMO_CH;
constexpr int SW = (NUM_PROMO_WARPS == 8) ? 16 : 8;     // columns per pass of the output transpose
static_assert(NUM_PROMO_WARPS == 8 || NUM_PROMO_WARPS == 16, "promotion warps");
static_assert(QCOLS % (2 * CH) == 0, "promotion chunks");
static_assert(NUM_PROMO_WARPS * (PROMO_REGS - LAUNCH_REGS) <= 4 * (LAUNCH_REGS - AUX_REGS), "setmaxnreg balance");
static_assert(GEMM_THREADS * LAUNCH_REGS <= 65536, "register file");

struct GemmSmem {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t amax_bar[2];
    uint64_t sf_full[STAGES];      // block-scaled kernel only: the stage's scale factors are in shared memory
    uint64_t pair_go;              // single-CTA tiles launched as clusters of two: the neighbour starts its tile
    uint32_t tmem_base;
    int abort_flag;
    int total_tiles;
    int tile_prefix[MAX_E + 1];
    float amax[2][NQ][BM];   // [tile parity][column group][row]
    alignas(16) float stage[NUM_PROMO_WARPS][32][SW + 4];   // per promotion warp: 32 rows x SW columns (+4 pad), output transpose
};

constexpr size_t GEMM_SMEM_BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES + sizeof(GemmSmem);
static_assert(GEMM_SMEM_BYTES <= 232448, "shared memory budget of one CTA");
// block-scaled kernel: per stage one 512-byte scale atom for the 128 rows of A and two for the 256 rows of B
constexpr int SF_BYTES = 1536;
// block-scaled kernel: the accumulator is moved into fp32 registers every MX_FLUSH K blocks.  The tensor core's own
// accumulation over a long chain is less exact than fp32 additions (one chain over K = 7168 put ~1e-4 relative
// error on GEMM1, enough to flip one e4m3 code in a thousand at the requantisation and to push a few outputs of
// the full-size layer past the 1e-2 absolute bound); 32 MMAs per chain keep it near fp32.
constexpr int MX_FLUSH = 8;
constexpr size_t GEMM_MX_SMEM_BYTES = GEMM_SMEM_BYTES + (size_t)STAGES * SF_BYTES;
static_assert(GEMM_MX_SMEM_BYTES <= 232448, "shared memory budget of one CTA (block-scaled kernel)");

struct GemmParams {
    const float* a_scale;      // [rows, nkb]
    const float* w_scale;      // MODE 1: [E, 2I/128, D/128]   MODE 2/3: [E, D/128, I/128]
    const int* offsets;        // [E+1]
    const int* row_tok;        // MODE 2
    const float* row_w;        // MODE 2/3
    uint8_t* act_q;            // MODE 1 out [rows, I]
    float* act_s;              // MODE 1 out [rows, I/128]
    float* out;                // MODE 2 out [T, D]; MODE 3 out [rows, D]
    int* status;
    int E, D, I;
    int packed;                // weights pre-tiled: one contiguous 256 x 128-byte block per (expert, n tile, K block)
    long long total_rows;      // capacity of the sorted row buffers
#ifdef B200_GEMM_TRACE
    long long* trace;          // [8][TRACE_CAP] clock64 stamps of CTA 0's pipeline events (timeline builds only)
    int trace_warp;
#endif
};

#ifdef B200_GEMM_TRACE
constexpr int TRACE_CAP = 512;
long long* g_gemm_trace = nullptr;
int g_gemm_trace_warp = 0;
#define TRACE_STAMP(slot, idx) do { if (p.trace && blockIdx.x == 0 && (idx) < TRACE_CAP) p.trace[(slot) * TRACE_CAP + (idx)] = clock64(); } while (0)
#else
#define TRACE_STAMP(slot, idx) do { } while (0)
#endif

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// ---- CTA-pair (cta_group::2) helpers ------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// Tiles 2i and 2i+1 run on the two CTAs of a cluster at the same time; when an expert has 129..256 rows they are
// the two row tiles of one weight slab.  The slab comes from DRAM once only if both CTAs stream it within the
// time a line stays in L2 (~20 us at full DRAM rate), and without a rendezvous the CTA with the nearly empty row
// tile gains a few microseconds per tile and is a whole tile ahead after some rounds (measured: every second
// row tile re-read from DRAM, 11.7 GB instead of 7.8 GB per GEMM1 launch).  So the two producers meet before
// every tile: each arrives on the neighbour's barrier and waits on its own (bounded).
__device__ __forceinline__ bool pair_rendezvous(uint64_t* own_bar, uint32_t peer_bar_cluster_addr, uint32_t parity,
                                                volatile int* abort_flag) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(peer_bar_cluster_addr) : "memory");
    return ptx::mbar_wait_relaxed(own_bar, parity, abort_flag, 100);
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window)
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(ptx::smem_u32(p)), "r"(rank));
    return r;
}
// Arrival on a barrier of the pair's other CTA.  Relaxed on purpose: what the arrival hands over is a TMEM
// stage whose reads have completed (tcgen05.wait::ld + tcgen05.fence::before_thread_sync), no memory data, and
// a cluster-scope release would first wait for every outstanding global load of the thread (the prefetched
// scales), which put ~1000 cycles into every K block.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
                 "r"(bytes)
                 : "memory");
}
// TMA tile load of one CTA of a pair: data lands in this CTA, completion bytes go to a barrier that may
// live in the pair's other CTA (no multicast: every CTA fetches its own tile)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(ptx::smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
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
// one arrival on the mbarrier at this offset in both CTAs of the pair once all MMAs issued so far have
// retired (two commits, each addressed through the cluster window to one CTA; no multicast qualifier)
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
__device__ __forceinline__ void mma2_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// acc[0..N-1] += v[0..N-1] * s  (B200_GEMM_PACKED_FMA: as N/2 fma.rn.f32x2, same bits)
template <int N>
__device__ __forceinline__ void promote(float* acc, const uint32_t (&v)[N], float s) {
#ifdef B200_GEMM_PACKED_FMA
    const unsigned long long s2 = ptx::pack_f32x2(s, s);
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        const unsigned long long r = ptx::fma_f32x2(ptx::pack_f32x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), s2,
                                                    ptx::pack_f32x2(acc[2 * i], acc[2 * i + 1]));
        ptx::unpack_f32x2(r, acc[2 * i], acc[2 * i + 1]);
    }
#else
#pragma unroll
    for (int i = 0; i < N; i++) acc[i] = fmaf(__uint_as_float(v[i]), s, acc[i]);
#endif
}
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
    if constexpr (N == 8) ptx::tmem_ld_32x8(taddr, r);
    else if constexpr (N == 16) ptx::tmem_ld_32x16(taddr, r);
    else ptx::tmem_ld_32x32(taddr, r);
}

// MODE 1: the tile's 256 accumulator columns are NQ groups [gate j0+g*QCOLS/2 .. | up j0+g*QCOLS/2 ..]
// (j0 = 128 n_tile, QCOLS/2 columns each), so that the gate and the up value of an activation column
// meet in one thread.
// MODE 2/3: plain output columns 256 n_tile .. +255.
//
// PAIR: two CTAs of a cluster (two SMs) work on one tile of 256 rows with tcgen05.mma.cta_group::2: CTA r holds
// rows 128 r .. +127 (its own A tile and accumulator) and HALF of the tile's weight rows (accumulator columns
// 128 r .. +127), so per K block each SM writes and reads 32 KB of shared memory instead of 48 KB, and a
// weight tile crosses L2 -> shared memory once per 256 rows.  Shared-memory bandwidth (TMA fill + MMA operand
// reads: 96 KB per K block for a single-CTA 128 x 256 tile, 768 cycles at 128 B/clk against 546 cycles of
// tensor time) is what bounds the single-CTA kernel.  The leader CTA (rank 0) issues the MMAs; both CTAs'
// loads complete on the leader's `full` barrier, both CTAs' promotion warps release the accumulator stage on
// the leader's `tmem_empty` barrier, and tcgen05.commit signals `empty` / `tmem_full` in both CTAs.
template <int MODE, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const GemmParams p) {
    constexpr int TM = PAIR ? 2 * BM : BM;        // rows of a tile
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    GemmSmem* sm = reinterpret_cast<GemmSmem*>(tiles + (size_t)STAGES * STAGE_BYTES);
    volatile int* abort_flag = &sm->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Kdim = (MODE == 1) ? p.D : p.I;
    const int nkb = Kdim / BK;
    const int NT = (MODE == 1) ? p.I / 128 : p.D / 256;     // N tiles per expert
    const int w_rows = (MODE == 1) ? 2 * p.I : p.D;         // weight rows per expert

    // ---- prologue ---------------------------------------------------------
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;     // 0 = leader
    const bool duo = !PAIR && cluster_nctarank() == 2;        // single-CTA tiles, launched two CTAs to a cluster
    const int pair_count = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;     // tile walkers
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    if (threadIdx.x == 0) {
        // PAIR: the leader's `full` takes one arrive.expect_tx from each CTA's producer, its `tmem_empty` one
        // arrival from every promotion warp of both CTAs
        for (int s = 0; s < STAGES; s++) { ptx::mbar_init(&sm->full[s], PAIR ? 2 : 1); ptx::mbar_init(&sm->empty[s], 1); }
        for (int a = 0; a < 2; a++) {
            ptx::mbar_init(&sm->tmem_full[a], 1);
            ptx::mbar_init(&sm->tmem_empty[a], PAIR ? 2 * NUM_PROMO_WARPS : NUM_PROMO_WARPS);
            ptx::mbar_init(&sm->amax_bar[a], NUM_PROMO_WARPS);
        }
        ptx::mbar_init(&sm->pair_go, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        // tile_prefix[e] = tiles of experts < e (warp scan over the expert counts)
        int running = 0;
        for (int e0 = 0; e0 < p.E; e0 += 32) {
            const int e = e0 + lane;
            int t = 0;
            if (e < p.E) t = ((p.offsets[e + 1] - p.offsets[e] + TM - 1) / TM) * NT;
            int incl = t;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (e < p.E) sm->tile_prefix[e] = running + incl - t;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) { sm->tile_prefix[p.E] = running; sm->total_tiles = running; }
    }
    if (warp == W_MMA0) {
        if (PAIR) { tmem_alloc2(&sm->tmem_base, 512); tmem_relinquish2(); }
        else      { ptx::tmem_alloc(&sm->tmem_base, 512); ptx::tmem_relinquish(); }
    }
    if (warp == W_TMA && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR || duo) cluster_sync_all();      // the peer's barriers are initialised before anyone signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = sm->tmem_base;
    const int total_tiles = sm->total_tiles;

    // tile -> (expert, m_tile, n_tile): expert-major, then n, then m, so the CTAs that run
    // together walk through one expert's weights once.
    auto locate = [&](int tile, int& e, int& m_tile, int& n_tile, int& cnt) {
        int lo = 0, hi = p.E;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (sm->tile_prefix[mid] <= tile) lo = mid; else hi = mid;
        }
        // experts with zero tiles repeat the prefix value; the search lands on the last
        // expert whose prefix is <= tile, which is the one that owns tiles.
        e = lo;
        cnt = p.offsets[e + 1] - p.offsets[e];
        int mt = (cnt + TM - 1) / TM;
        int local = tile - sm->tile_prefix[e];
        n_tile = local / mt;
        m_tile = local - n_tile * mt;
    };

    if (warp >= NUM_PROMO_WARPS) {
        ptx::setmaxnreg_dec<AUX_REGS>();
      if (warp == W_TMA) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            int s = 0; uint32_t ph = 0; int gk = 0; (void)gk;
            uint32_t go_ph = 0;
            const uint32_t peer_go = duo ? map_to_cta(&sm->pair_go, cluster_ctarank() ^ 1u) : 0u;
            for (int tile = walker; tile < total_tiles; tile += pair_count) {
                int e, m_tile, n_tile, cnt;
                locate(tile, e, m_tile, n_tile, cnt);
                if (duo && (tile | 1) < total_tiles) {        // the neighbour has a tile in this pass over the grid too
                    if (!pair_rendezvous(&sm->pair_go, peer_go, go_ph, abort_flag)) goto done;
                    go_ph ^= 1;
                }
                const int row0 = p.offsets[e] + m_tile * TM + (int)crank * BM;
                const long long wrow0 = (long long)e * w_rows;
                for (int kb = 0; kb < nkb; kb++) {
                    if (!ptx::mbar_wait_relaxed(&sm->empty[s], ph ^ 1, abort_flag, 200)) goto done;
                    TRACE_STAMP(6, gk); gk++;
                    uint8_t* a_dst = tiles + (size_t)s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    if (PAIR) {
                        // this CTA's 128 rows of A and its half of the weight tile (accumulator columns
                        // 128 crank .. +127); the bytes are counted on the leader's barrier
                        const uint32_t fbar = map_to_cta(&sm->full[s], 0);
                        mbar_expect_tx_cluster(fbar, A_BYTES + B_BYTES / 2);
                        tma_load_2d_pair(a_dst, &tmap_a, fbar, kb * BK, row0);
                        if (p.packed) {
                            tma_load_2d_pair(b_dst, &tmap_b, fbar, 0, (((e * NT + n_tile) * nkb) + kb) * BN + (int)crank * 128);
                        } else if (MODE == 1) {
                            const int j0 = n_tile * 128 + 64 * (int)crank;
                            tma_load_2d_pair(b_dst, &tmap_b, fbar, kb * BK, (int)(wrow0 + j0));
                            tma_load_2d_pair(b_dst + 8192, &tmap_b, fbar, kb * BK, (int)(wrow0 + p.I + j0));
                        } else {
                            tma_load_2d_pair(b_dst, &tmap_b, fbar, kb * BK, (int)(wrow0 + n_tile * 256 + 128 * (int)crank));
                        }
                    } else {
                        ptx::mbar_expect_tx(&sm->full[s], STAGE_BYTES);
                        ptx::tma_load_2d(a_dst, &tmap_a, &sm->full[s], kb * BK, row0);
                        if (p.packed) {
                            // the tile's K block is one contiguous 32 KB piece of the packed weights
                            ptx::tma_load_2d(b_dst, &tmap_b, &sm->full[s], 0, (((e * NT + n_tile) * nkb) + kb) * BN);
                        } else if (MODE == 1) {
                            // 2 NQ boxes of QCOLS/2 weight rows: group g = [gate j0 + g QCOLS/2 .. | up j0 + g QCOLS/2 ..]
                            const int j0 = n_tile * 128;
#pragma unroll
                            for (int bx = 0; bx < 2 * NQ; bx++)
                                ptx::tma_load_2d(b_dst + bx * (QCOLS / 2) * 128, &tmap_b, &sm->full[s], kb * BK,
                                                 (int)(wrow0 + ((bx & 1) ? p.I : 0) + j0 + (QCOLS / 2) * (bx >> 1)));
                        } else {
                            ptx::tma_load_2d(b_dst, &tmap_b, &sm->full[s], kb * BK, (int)(wrow0 + n_tile * 256));
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
      } else if (warp == W_MMA0 || warp == W_MMA0 + 1) {
        // ===================== MMA issuers =====================
        // Two issuers, one per TMEM stage (K blocks alternate between them).  The thread that issues a
        // K block's MMAs stays tied up until they have run (in the issue of the later ones and in the
        // commits); with a single issuer it came back to look at the other stage's "free" barrier
        // hundreds of cycles after the promotion warps had released it.
        if (lane == 0 && crank == 0) {
            constexpr uint32_t idesc = ptx::make_idesc(0, 0, 0, 0, TM, BN);
            const int role = warp - W_MMA0;                 // the TMEM stage this issuer owns
            int s = 0; uint32_t ph = 0;
            uint32_t acc_ph = 0; long long g = 0;           // g: K blocks since the kernel started
            for (int tile = walker; tile < total_tiles; tile += pair_count) {
                for (int kb = 0; kb < nkb; kb++, g++) {
                    if ((int)(g & 1) == role) {
                        // (waits on barriers that the peer CTA or tcgen05.commit signal need no cluster-scope
                        // acquire: what they hand over is a TMEM stage or TMA-written tiles, not memory data)
                        if (!ptx::mbar_wait_relaxed(&sm->tmem_empty[role], acc_ph ^ 1, abort_flag, ISSUER_SLEEP_NS)) goto done;
                        TRACE_STAMP(0, g);
                        if (!ptx::mbar_wait(&sm->full[s], ph, abort_flag)) goto done;
                        TRACE_STAMP(1, g);
                        ptx::tc_fence_after();
                        const uint32_t a_addr = ptx::smem_u32(tiles + (size_t)s * STAGE_BYTES);
                        const uint32_t b_addr = a_addr + A_BYTES;
                        const uint32_t d_tmem = tmem_base + role * BN;
#pragma unroll
                        for (int k4 = 0; k4 < 4; k4++) {
                            uint64_t ad = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
                            uint64_t bd = ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
                            if (PAIR) mma2_f8(d_tmem, ad, bd, idesc, k4 > 0 ? 1u : 0u);
                            else      ptx::mma_f8(d_tmem, ad, bd, idesc, k4 > 0 ? 1u : 0u);
                        }
                        if (PAIR) {
                            commit_both(&sm->empty[s]);
                            commit_both(&sm->tmem_full[role]);
                        } else {
                            ptx::tc_commit(&sm->empty[s]);          // smem stage reusable once the MMAs have read it
                            ptx::tc_commit(&sm->tmem_full[role]);   // partial sums ready for promotion
                        }
                        TRACE_STAMP(2, g);
                        acc_ph ^= 1;
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
      }
    } else {
        // ===================== promotion + epilogue (warps 0-15) =====================
        ptx::setmaxnreg_inc<PROMO_REGS>();
        // one lane polls the barrier, the warp follows (hundreds of pollers and arrivals per K block on
        // one shared-memory word cost more than the promotion itself)
        auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
            int ok = 1;
            if (lane == 0) ok = ptx::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();
            return ok != 0;
        };
        const int wq = warp >> 2;                         // column group of the accumulator
        const int row = (warp & 3) * 32 + lane;           // TMEM lane = tile row
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        int acc = 0; uint32_t acc_ph = 0;
        int tile_par = 0; uint32_t amax_ph[2] = {0, 0};
        int gp = 0; (void)gp;
#ifdef B200_GEMM_TRACE
        const bool trw = (threadIdx.x == p.trace_warp * 32);
#endif
        const int nkb_w = Kdim / 128;
        // the stage's "free" barrier lives in the leader CTA
        const uint32_t tmem_empty_addr[2] = {PAIR ? map_to_cta(&sm->tmem_empty[0], 0) : 0u,
                                             PAIR ? map_to_cta(&sm->tmem_empty[1], 0) : 0u};
        auto release_stage = [&](int a) {
            if (PAIR && crank != 0) mbar_arrive_cluster(tmem_empty_addr[a]);
            else                    ptx::mbar_arrive(&sm->tmem_empty[a]);
        };
        for (int tile = walker; tile < total_tiles; tile += pair_count) {
            int e, m_tile, n_tile, cnt;
            locate(tile, e, m_tile, n_tile, cnt);
            const int trow0 = m_tile * TM + (int)crank * BM;                       // first row of this CTA inside the expert
            const long long grow = (long long)p.offsets[e] + trow0 + row;         // sorted row
            const bool row_ok = (trow0 + row) < cnt;
            const bool warp_valid = (trow0 + (warp & 3) * 32) < cnt;              // any valid row in this warp's 32
            const float* a_sc = p.a_scale + (grow < p.total_rows ? grow : 0) * nkb;
            const float* w_sc0;
            const float* w_sc1;
            if (MODE == 1) {
                const float* base = p.w_scale + (size_t)e * (2 * p.I / 128) * nkb_w;
                w_sc0 = base + (size_t)n_tile * nkb_w;                     // gate rows' block
                w_sc1 = base + (size_t)(p.I / 128 + n_tile) * nkb_w;       // up rows' block
            } else {
                const float* base = p.w_scale + (size_t)e * (p.D / 128) * nkb_w;
                w_sc0 = base + (size_t)(n_tile * 2 + (wq * QCOLS) / 128) * nkb_w;
                w_sc1 = w_sc0;
            }
            float accv[QCOLS];
#pragma unroll
            for (int i = 0; i < QCOLS; i++) accv[i] = 0.0f;

            // scales of K block kb+1 are fetched while block kb is being promoted
            float sa_n = row_ok ? a_sc[0] : 0.0f, w0_n = w_sc0[0], w1_n = (MODE == 1) ? w_sc1[0] : 0.0f;
            for (int kb = 0; kb < nkb; kb++) {
                const float s0 = sa_n * w0_n;
                const float s1 = (MODE == 1) ? sa_n * w1_n : s0;
                if (kb + 1 < nkb) {
                    sa_n = row_ok ? a_sc[kb + 1] : 0.0f;
                    w0_n = w_sc0[kb + 1];
                    if (MODE == 1) w1_n = w_sc1[kb + 1];
                }
                if (!warp_wait(&sm->tmem_full[acc], acc_ph)) goto done;
#ifdef B200_GEMM_TRACE
                if (trw) TRACE_STAMP(3, gp);
#endif
                if (warp_valid) {
                    // warps whose 32 rows are all padding only hand the stage back
                    ptx::tc_fence_after();
                    const uint32_t t0 = tmem_base + lane_addr + acc * BN + wq * QCOLS;
                    // QCOLS columns in chunks of CH, two loads in flight; columns [0, QCOLS/2) take s0 (MODE 1:
                    // gate), the rest s1 (MODE 1: up)
                    constexpr int NPAIR = QCOLS / (2 * CH);
                    uint32_t ra[CH], rb[CH];
#pragma unroll
                    for (int c = 0; c < NPAIR; c++) {
                        tmem_ld_cols<CH>(t0 + 2 * c * CH, ra);
                        tmem_ld_cols<CH>(t0 + 2 * c * CH + CH, rb);
                        ptx::tc_wait_ld();
                        if (c == NPAIR - 1) {
                            ptx::tc_fence_before();
                            __syncwarp();
                            if (lane == 0) release_stage(acc);   // the stage is in registers now
#ifdef B200_GEMM_TRACE
                            if (trw) TRACE_STAMP(4, gp);
#endif
                        }
                        promote<CH>(accv + 2 * c * CH, ra, (2 * c * CH < QCOLS / 2) ? s0 : s1);
                        promote<CH>(accv + (2 * c + 1) * CH, rb, ((2 * c + 1) * CH < QCOLS / 2) ? s0 : s1);
                    }
                } else {
                    ptx::tc_fence_before();
                    if (lane == 0) release_stage(acc);
                }
#ifdef B200_GEMM_TRACE
                if (trw) TRACE_STAMP(5, gp);
                gp++;
#endif
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
#ifdef B200_GEMM_TRACE
            if (trw) TRACE_STAMP(7, gp / nkb - 1);     // end of the main loop of each tile; epilogue follows
#endif

            if (MODE == 1) {
                // SwiGLU on 32 activation columns, 1x128 requantisation shared with the three other quarters.
                // Fast exp / reciprocal: the result is rounded to e4m3 next, an ulp of fp32 does not matter.
                constexpr int AC = QCOLS / 2;          // activation columns of this thread
                float amax = 0.0f;
                if (warp_valid) {
#pragma unroll
                    for (int i = 0; i < AC; i++) {
                        const float g = accv[i], u = accv[AC + i];
                        const float a = __fdividef(g, 1.0f + __expf(-g)) * u;
                        accv[i] = a;
                        amax = fmaxf(amax, fabsf(a));
                    }
                }
                sm->amax[tile_par][wq][row] = amax;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sm->amax_bar[tile_par]);
                if (!warp_wait(&sm->amax_bar[tile_par], amax_ph[tile_par])) goto done;
                amax_ph[tile_par] ^= 1;
#pragma unroll
                for (int g = 0; g < NQ; g++) amax = fmaxf(amax, sm->amax[tile_par][g][row]);
                if (row_ok) {
                    const float scale = amax > 0.0f ? __fdiv_rn(amax, 448.0f) : 1.0f;
                    const float inv = amax > 0.0f ? __fdiv_rn(448.0f, amax) : 1.0f;
                    uint32_t packed[AC / 4];
#pragma unroll
                    for (int i = 0; i < AC / 4; i++) {
                        const float a0 = accv[4 * i], a1 = accv[4 * i + 1], a2 = accv[4 * i + 2], a3 = accv[4 * i + 3];
                        packed[i] = (uint32_t)__nv_cvt_float_to_fp8(a0 * inv, __NV_SATFINITE, __NV_E4M3) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a1 * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a2 * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a3 * inv, __NV_SATFINITE, __NV_E4M3) << 24);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.act_q + grow * p.I + n_tile * 128 + wq * AC);
#pragma unroll
                    for (int i = 0; i < AC / 16; i++)
                        dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    if (wq == 0) p.act_s[grow * (p.I / 128) + n_tile] = scale;
                }
                tile_par ^= 1;
            } else if (warp_valid) {
                // The accumulator row of a lane is transposed through shared memory SW columns at a time so that
                // one store / red instruction covers 32 / SEGS rows x 16 SEGS contiguous bytes instead of 32 rows
                // x 16 bytes (fewer, larger memory requests).
                const float w = row_ok ? p.row_w[grow] : 0.0f;
                float (*st)[SW + 4] = sm->stage[warp];
                constexpr int SEGS = SW / 4;
                const int sub_row = lane / SEGS, seg = lane % SEGS;
                const int tok = (MODE == 2 && row_ok) ? p.row_tok[grow] : -1;
                // MODE 2: out[token] += w * acc.  MODE 3: rows[sorted row] = w * acc (plain stores).
                const long long grow0 = (long long)p.offsets[e] + trow0 + (warp & 3) * 32;
                const int rows_ok = min(32, cnt - (trow0 + (warp & 3) * 32));
                float* const out_col = p.out + n_tile * 256 + wq * QCOLS;
#pragma unroll
                for (int pass = 0; pass < QCOLS / SW; pass++) {
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < SEGS; q++) {
                        const float* a4 = accv + pass * SW + q * 4;
                        *reinterpret_cast<float4*>(&st[lane][q * 4]) = make_float4(w * a4[0], w * a4[1], w * a4[2], w * a4[3]);
                    }
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < SEGS; k++) {
                        const int r = (32 / SEGS) * k + sub_row;
                        const float4 x4 = *reinterpret_cast<const float4*>(&st[r][seg * 4]);
                        if (MODE == 2) {
                            const int tok_r = __shfl_sync(0xffffffffu, tok, r);
                            if (tok_r >= 0)
                                red_add_v4(out_col + (size_t)tok_r * p.D + pass * SW + seg * 4, x4.x, x4.y, x4.z, x4.w);
                        } else if (r < rows_ok) {
                            *reinterpret_cast<float4*>(out_col + (size_t)(grow0 + r) * p.D + pass * SW + seg * 4) = x4;
                        }
                    }
                }
            }
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR || duo) cluster_sync_all();     // the pair's MMAs, remote arrivals and TMEM reads are over in both CTAs
    if (warp == W_MMA0) {
        if (PAIR) tmem_dealloc2(tmem_base, 512);
        else      ptx::tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(p.status, B200_TIMEOUT);
}

// -------------------------------------------------------------------------------------------------
// The same grouped GEMMs for power-of-two scales (B200_MOE_POW2_SCALES) on the hardware block-scaled MMA
// (tcgen05.mma kind::mxf8f6f4.block_scale, UE8M0 scale = the exponent byte of the fp32 scale): the tensor core
// multiplies every 32-deep slice of a row by its scale itself, so the accumulator of a tile stays in TMEM
// for the whole K loop, nothing is promoted in software and the K-block period is the MMA's own (or the
// weight stream's).  Differences from the kernel above:
//   * warp 10 builds the scale factors of every stage in shared memory: a 512-byte atom for the 128 rows of A
//     (row r -> byte (r % 32) * 16 + (r / 32) * 4 + step, four K = 32 steps of the 128-deep block share the
//     scale) and two atoms for the 256 rows of B (all rows of a 128-column weight block share its scale); it
//     also checks that every scale it sees is a power of two (B200_BAD_SCALE otherwise);
//   * the MMA warp copies the atoms into TMEM (tcgen05.cp 32x128b.warpx4: 4 + 8 columns per stage, at columns
//     256 + 16 stage) and issues the four MMAs of the K block with scale ids 0..3;
//   * ONE 256-column accumulator: the eight epilogue warps add it into registers (128 columns per thread) every
//     MX_FLUSH K blocks and free it at once, so the next segment's (or tile's) MMAs run under the additions and
//     the epilogue;
//   * GEMM1 requantises with a power-of-two scale as well.
// Single-CTA tiles only.
// -------------------------------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmParams p) {
    static_assert(NUM_PROMO_WARPS == 8, "the block-scaled kernel is written for eight epilogue warps");
    constexpr int W_SF = W_MMA0 + 1;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sf_area = tiles + (size_t)STAGES * STAGE_BYTES;
    GemmSmem* sm = reinterpret_cast<GemmSmem*>(sf_area + (size_t)STAGES * SF_BYTES);
    volatile int* abort_flag = &sm->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Kdim = (MODE == 1) ? p.D : p.I;
    const int nkb = Kdim / BK;
    const int NT = (MODE == 1) ? p.I / 128 : p.D / 256;     // N tiles per expert
    const int w_rows = (MODE == 1) ? 2 * p.I : p.D;         // weight rows per expert
    const int walkers = (int)gridDim.x, walker = (int)blockIdx.x;
    const bool duo = cluster_nctarank() == 2;               // launched two CTAs to a cluster

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            ptx::mbar_init(&sm->full[s], 1);
            ptx::mbar_init(&sm->empty[s], 1);
            ptx::mbar_init(&sm->sf_full[s], 1);
        }
        ptx::mbar_init(&sm->pair_go, 1);
        ptx::mbar_init(&sm->tmem_full[0], 1);
        ptx::mbar_init(&sm->tmem_empty[0], NUM_PROMO_WARPS);
        for (int a = 0; a < 2; a++) ptx::mbar_init(&sm->amax_bar[a], NUM_PROMO_WARPS);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        int running = 0;
        for (int e0 = 0; e0 < p.E; e0 += 32) {
            const int e = e0 + lane;
            int t = 0;
            if (e < p.E) t = ((p.offsets[e + 1] - p.offsets[e] + BM - 1) / BM) * NT;
            int incl = t;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            if (e < p.E) sm->tile_prefix[e] = running + incl - t;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) { sm->tile_prefix[p.E] = running; sm->total_tiles = running; }
    }
    if (warp == W_MMA0) { ptx::tmem_alloc(&sm->tmem_base, 512); ptx::tmem_relinquish(); }
    if (warp == W_TMA && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (duo) cluster_sync_all();              // the neighbour's barrier is initialised before anyone signals it
    ptx::tc_fence_after();
    const uint32_t tmem_base = sm->tmem_base;
    const int total_tiles = sm->total_tiles;

    auto locate = [&](int tile, int& e, int& m_tile, int& n_tile, int& cnt) {
        int lo = 0, hi = p.E;
        while (hi - lo > 1) {
            int mid = (lo + hi) >> 1;
            if (sm->tile_prefix[mid] <= tile) lo = mid; else hi = mid;
        }
        e = lo;
        cnt = p.offsets[e + 1] - p.offsets[e];
        int mt = (cnt + BM - 1) / BM;
        int local = tile - sm->tile_prefix[e];
        n_tile = local / mt;
        m_tile = local - n_tile * mt;
    };
    // one lane polls the barrier, the warp follows
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) -> bool {
        int ok = 1;
        if (lane == 0) ok = ptx::mbar_wait(bar, parity, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        __syncwarp();
        return ok != 0;
    };

    if (warp >= NUM_PROMO_WARPS) {
        ptx::setmaxnreg_dec<AUX_REGS>();
      if (warp == W_TMA) {
        // ===================== TMA producer (operand tiles) =====================
        if (lane == 0) {
            int s = 0; uint32_t ph = 0, go_ph = 0;
            const uint32_t peer_go = duo ? map_to_cta(&sm->pair_go, cluster_ctarank() ^ 1u) : 0u;
            for (int tile = walker; tile < total_tiles; tile += walkers) {
                int e, m_tile, n_tile, cnt;
                locate(tile, e, m_tile, n_tile, cnt);
                if (duo && (tile | 1) < total_tiles) {        // the neighbour has a tile in this pass over the grid too
                    if (!pair_rendezvous(&sm->pair_go, peer_go, go_ph, abort_flag)) goto done;
                    go_ph ^= 1;
                }
                const int row0 = p.offsets[e] + m_tile * BM;
                const long long wrow0 = (long long)e * w_rows;
                for (int kb = 0; kb < nkb; kb++) {
                    if (!ptx::mbar_wait_relaxed(&sm->empty[s], ph ^ 1, abort_flag, 200)) goto done;
                    uint8_t* a_dst = tiles + (size_t)s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    ptx::mbar_expect_tx(&sm->full[s], STAGE_BYTES);
                    ptx::tma_load_2d(a_dst, &tmap_a, &sm->full[s], kb * BK, row0);
                    if (p.packed) {
                        ptx::tma_load_2d(b_dst, &tmap_b, &sm->full[s], 0, (((e * NT + n_tile) * nkb) + kb) * BN);
                    } else if (MODE == 1) {
                        const int j0 = n_tile * 128;
#pragma unroll
                        for (int bx = 0; bx < 2 * NQ; bx++)
                            ptx::tma_load_2d(b_dst + bx * (QCOLS / 2) * 128, &tmap_b, &sm->full[s], kb * BK,
                                             (int)(wrow0 + ((bx & 1) ? p.I : 0) + j0 + (QCOLS / 2) * (bx >> 1)));
                    } else {
                        ptx::tma_load_2d(b_dst, &tmap_b, &sm->full[s], kb * BK, (int)(wrow0 + n_tile * 256));
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
      } else if (warp == W_MMA0) {
        // ===================== scale copies + MMAs =====================
        if (lane == 0) {
            int s = 0; uint32_t ph = 0, tph = 0;
            for (int tile = walker; tile < total_tiles; tile += walkers) {
              for (int kb0 = 0; kb0 < nkb; kb0 += MX_FLUSH) {
                // the epilogue warps have added the previous segment (or tile) into their registers
                if (!ptx::mbar_wait(&sm->tmem_empty[0], tph ^ 1, abort_flag)) goto done;
                ptx::tc_fence_after();
                const int kb1 = min(nkb, kb0 + MX_FLUSH);
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!ptx::mbar_wait(&sm->full[s], ph, abort_flag)) goto done;
                    if (!ptx::mbar_wait(&sm->sf_full[s], ph, abort_flag)) goto done;
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(tiles + (size_t)s * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
                    const uint32_t sf_addr = ptx::smem_u32(sf_area + (size_t)s * SF_BYTES);
                    const uint32_t tsfa = tmem_base + BN + 16 * s, tsfb = tsfa + 4;
                    ptx::tmem_cp_32x128b_warpx4(tsfa, ptx::make_smem_desc(sf_addr, 16, 128, 0));
                    ptx::tmem_cp_32x128b_warpx4(tsfb, ptx::make_smem_desc(sf_addr + 512, 16, 128, 0));
                    ptx::tmem_cp_32x128b_warpx4(tsfb + 4, ptx::make_smem_desc(sf_addr + 1024, 16, 128, 0));
#pragma unroll
                    for (int k4 = 0; k4 < 4; k4++) {
                        const uint64_t ad = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
                        const uint64_t bd = ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
                        ptx::mma_mxf8(tmem_base, ad, bd, ptx::make_idesc_mx(BM, BN, k4, k4), tsfa, tsfb,
                                      (kb > kb0 || k4 > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(&sm->empty[s]);          // operand tiles, scale atoms and their TMEM copies reusable
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                ptx::tc_commit(&sm->tmem_full[0]);
                tph ^= 1;
              }
            }
        }
      } else if (warp == W_SF) {
        // ===================== scale factors of every stage =====================
        int s = 0; uint32_t ph = 0;
        uint32_t bad = 0;
        auto expo = [&](float f) -> uint32_t {
            const uint32_t b = __float_as_uint(f);
            bad |= (b & 0x807FFFFFu) | (((b >> 23) == 0u) ? 1u : 0u);     // sign, mantissa bits, zero / denormal
            return ((b >> 23) & 0xFFu) * 0x01010101u;                    // the UE8M0 byte, once per K = 32 step
        };
        const int nkb_w = Kdim / 128;
        for (int tile = walker; tile < total_tiles; tile += walkers) {
            int e, m_tile, n_tile, cnt;
            locate(tile, e, m_tile, n_tile, cnt);
            const float* a_sc[4];
            bool ok[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int r = m_tile * BM + lane + 32 * q;
                ok[q] = r < cnt;
                a_sc[q] = p.a_scale + (size_t)(ok[q] ? (long long)p.offsets[e] + r : 0) * nkb;
            }
            const float* w_sc0;
            const float* w_sc1;
            if (MODE == 1) {
                const float* base = p.w_scale + (size_t)e * (2 * p.I / 128) * nkb_w;
                w_sc0 = base + (size_t)n_tile * nkb_w;                     // gate rows' block
                w_sc1 = base + (size_t)(p.I / 128 + n_tile) * nkb_w;       // up rows' block
            } else {
                const float* base = p.w_scale + (size_t)e * (p.D / 128) * nkb_w;
                w_sc0 = base + (size_t)(n_tile * 2) * nkb_w;               // columns 0..127 of the tile
                w_sc1 = w_sc0 + nkb_w;                                     // columns 128..255
            }
            float an[4], w0n = w_sc0[0], w1n = w_sc1[0];
#pragma unroll
            for (int q = 0; q < 4; q++) an[q] = ok[q] ? a_sc[q][0] : 1.0f;
            for (int kb = 0; kb < nkb; kb++) {
                const float a0 = an[0], a1 = an[1], a2 = an[2], a3 = an[3], w0 = w0n, w1 = w1n;
                if (kb + 1 < nkb) {
#pragma unroll
                    for (int q = 0; q < 4; q++) an[q] = ok[q] ? a_sc[q][kb + 1] : 1.0f;
                    w0n = w_sc0[kb + 1];
                    w1n = w_sc1[kb + 1];
                }
                if (!warp_wait(&sm->empty[s], ph ^ 1)) goto done;
                const uint32_t sfp = ptx::smem_u32(sf_area + (size_t)s * SF_BYTES) + lane * 16;
                const uint32_t g = expo(w0), u = expo(w1);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sfp), "r"(expo(a0)), "r"(expo(a1)), "r"(expo(a2)), "r"(expo(a3)) : "memory");
                if (MODE == 1) {
                    // accumulator columns [gate 64 | up 64 | gate 64 | up 64]
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sfp + 512), "r"(g), "r"(g), "r"(u), "r"(u) : "memory");
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sfp + 1024), "r"(g), "r"(g), "r"(u), "r"(u) : "memory");
                } else {
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sfp + 512), "r"(g), "r"(g), "r"(g), "r"(g) : "memory");
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sfp + 1024), "r"(u), "r"(u), "r"(u), "r"(u) : "memory");
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sm->sf_full[s]);
                if (++s == STAGES) { s = 0; ph ^= 1; }
            }
        }
        if (__any_sync(0xffffffffu, bad != 0) && lane == 0) atomicExch(p.status, B200_BAD_SCALE);
      }
    } else {
        // ===================== epilogue (warps 0-7) =====================
        ptx::setmaxnreg_inc<PROMO_REGS>();
        const int wq = warp >> 2;                         // column half of the accumulator
        const int row = (warp & 3) * 32 + lane;           // TMEM lane = tile row
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        uint32_t fph = 0;
        int tile_par = 0; uint32_t amax_ph[2] = {0, 0};
        for (int tile = walker; tile < total_tiles; tile += walkers) {
            int e, m_tile, n_tile, cnt;
            locate(tile, e, m_tile, n_tile, cnt);
            const int trow0 = m_tile * BM;
            const long long grow = (long long)p.offsets[e] + trow0 + row;         // sorted row
            const bool row_ok = (trow0 + row) < cnt;
            const bool warp_valid = (trow0 + (warp & 3) * 32) < cnt;              // any valid row in this warp's 32
            float accv[QCOLS];
#pragma unroll
            for (int i = 0; i < QCOLS; i++) accv[i] = 0.0f;
            for (int kb0 = 0; kb0 < nkb; kb0 += MX_FLUSH) {
                if (!warp_wait(&sm->tmem_full[0], fph)) goto done;
                fph ^= 1;
                ptx::tc_fence_after();
                if (warp_valid) {
                    const uint32_t t0 = tmem_base + lane_addr + wq * QCOLS;
#pragma unroll
                    for (int c = 0; c < QCOLS / 32; c++) {
                        uint32_t r[32];
                        ptx::tmem_ld_32x32(t0 + 32 * c, r);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) accv[32 * c + i] += __uint_as_float(r[i]);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sm->tmem_empty[0]);  // the segment is in registers: the MMAs may go on
            }

            if (MODE == 1) {
                constexpr int AC = QCOLS / 2;          // activation columns of this thread
                float amax = 0.0f;
                if (warp_valid) {
#pragma unroll
                    for (int i = 0; i < AC; i++) {
                        const float g = accv[i], u = accv[AC + i];
                        const float a = __fdividef(g, 1.0f + __expf(-g)) * u;
                        accv[i] = a;
                        amax = fmaxf(amax, fabsf(a));
                    }
                }
                sm->amax[tile_par][wq][row] = amax;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&sm->amax_bar[tile_par]);
                if (!warp_wait(&sm->amax_bar[tile_par], amax_ph[tile_par])) goto done;
                amax_ph[tile_par] ^= 1;
#pragma unroll
                for (int g = 0; g < NQ; g++) amax = fmaxf(amax, sm->amax[tile_par][g][row]);
                if (row_ok) {
                    // power-of-two scale: the reciprocal is exact
                    const float scale = amax > 0.0f ? ptx::pow2_scale_bits(__fdiv_rn(amax, 448.0f)) : 1.0f;
                    const float inv = __fdiv_rn(1.0f, scale);
                    uint32_t packed[AC / 4];
#pragma unroll
                    for (int i = 0; i < AC / 4; i++) {
                        const float a0 = accv[4 * i], a1 = accv[4 * i + 1], a2 = accv[4 * i + 2], a3 = accv[4 * i + 3];
                        packed[i] = (uint32_t)__nv_cvt_float_to_fp8(a0 * inv, __NV_SATFINITE, __NV_E4M3) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a1 * inv, __NV_SATFINITE, __NV_E4M3) << 8) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a2 * inv, __NV_SATFINITE, __NV_E4M3) << 16) |
                                    ((uint32_t)__nv_cvt_float_to_fp8(a3 * inv, __NV_SATFINITE, __NV_E4M3) << 24);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(p.act_q + grow * p.I + n_tile * 128 + wq * AC);
#pragma unroll
                    for (int i = 0; i < AC / 16; i++)
                        dst[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
                    if (wq == 0) p.act_s[grow * (p.I / 128) + n_tile] = scale;
                }
                tile_par ^= 1;
            } else if (warp_valid) {
                const float w = row_ok ? p.row_w[grow] : 0.0f;
                float (*st)[SW + 4] = sm->stage[warp];
                constexpr int SEGS = SW / 4;
                const int sub_row = lane / SEGS, seg = lane % SEGS;
                const int tok = (MODE == 2 && row_ok) ? p.row_tok[grow] : -1;
                const long long grow0 = (long long)p.offsets[e] + trow0 + (warp & 3) * 32;
                const int rows_ok = min(32, cnt - (trow0 + (warp & 3) * 32));
                float* const out_col = p.out + n_tile * 256 + wq * QCOLS;
#pragma unroll
                for (int pass = 0; pass < QCOLS / SW; pass++) {
                    __syncwarp();
#pragma unroll
                    for (int q = 0; q < SEGS; q++) {
                        const float* a4 = accv + pass * SW + q * 4;
                        *reinterpret_cast<float4*>(&st[lane][q * 4]) = make_float4(w * a4[0], w * a4[1], w * a4[2], w * a4[3]);
                    }
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < SEGS; k++) {
                        const int r = (32 / SEGS) * k + sub_row;
                        const float4 x4 = *reinterpret_cast<const float4*>(&st[r][seg * 4]);
                        if (MODE == 2) {
                            const int tok_r = __shfl_sync(0xffffffffu, tok, r);
                            if (tok_r >= 0)
                                red_add_v4(out_col + (size_t)tok_r * p.D + pass * SW + seg * 4, x4.x, x4.y, x4.z, x4.w);
                        } else if (r < rows_ok) {
                            *reinterpret_cast<float4*>(out_col + (size_t)(grow0 + r) * p.D + pass * SW + seg * 4) = x4;
                        }
                    }
                }
            }
        }
    }
done:
    ptx::tc_fence_before();
    __syncthreads();
    if (duo) cluster_sync_all();              // no remote arrival is in flight towards a CTA that has left
    if (warp == W_MMA0) ptx::tmem_dealloc(tmem_base, 512);
    if (threadIdx.x == 0 && sm->abort_flag) atomicExch(p.status, B200_TIMEOUT);
}

// Deterministic combine: out[t,:] = sum over the token's K slots, in ascending expert order (ties cannot
// occur: an expert appears at most once per token), of rows[row_of_pair[t*K+k],:].  One block per token.
__global__ void __launch_bounds__(256)
reduce_rows_kernel(const float* __restrict__ rows, const int* __restrict__ pair_row, const int* __restrict__ ids,
                   int K, int D, float* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ int order[64];
    if (threadIdx.x == 0) {
        // slots sorted by expert id (K <= 64), skipped slots (row < 0) dropped
        int n = 0;
        for (int k = 0; k < K; k++)
            if (pair_row[t * K + k] >= 0) order[n++] = k;
        for (int i = 1; i < n; i++) {
            const int kk = order[i];
            int j = i - 1;
            while (j >= 0 && ids[t * K + order[j]] > ids[t * K + kk]) { order[j + 1] = order[j]; j--; }
            order[j + 1] = kk;
        }
        for (int i = n; i < K; i++) order[i] = -1;
    }
    __syncthreads();
    for (int c = threadIdx.x * 4; c < D; c += blockDim.x * 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i = 0; i < K; i++) {
            const int k = order[i];
            if (k < 0) break;
            const float4 v = *reinterpret_cast<const float4*>(rows + (size_t)pair_row[t * K + k] * D + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + (size_t)t * D + c) = acc;
    }
}

// Expert-sorted copy of the FP8 rows.  One block per sorted row, grid-stride (the number of valid
// rows is only known on the device: slots owned by other ranks are not rows).
__global__ void __launch_bounds__(128)
sort_rows_fp8_kernel(const uint8_t* __restrict__ xq, const float* __restrict__ xs, const int* __restrict__ row_pair,
                     const int* __restrict__ offsets, const float* __restrict__ wts, int E, int K, int D,
                     uint8_t* __restrict__ sq, float* __restrict__ ss, int* __restrict__ row_tok,
                     float* __restrict__ row_w, int* __restrict__ pair_row) {
    const int total = offsets[E];
    const int nb = D / 128;
    for (int r = blockIdx.x; r < total; r += gridDim.x) {
        const int pair = row_pair[r];
        const int tok = pair / K;
        const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)tok * D);
        uint4* dst = reinterpret_cast<uint4*>(sq + (size_t)r * D);
        for (int i = threadIdx.x; i < D / 16; i += blockDim.x) dst[i] = src[i];
        for (int i = threadIdx.x; i < nb; i += blockDim.x) ss[(size_t)r * nb + i] = xs[(size_t)tok * nb + i];
        if (threadIdx.x == 0) {
            row_tok[r] = tok;
            row_w[r] = wts[pair];
            if (pair_row) pair_row[pair] = r;      // deterministic combine: sorted row of (token, slot)
        }
    }
}

// Optional per-kernel timing: CUDA events recorded on the launch stream around the two grouped
// GEMMs (used by the benchmark for the roofline line; off by default).  The record belongs to the
// workspace, so host threads that drive different GPUs (or different workspaces) do not share it.
constexpr int PROF_SLOTS = 256;
}  // namespace
struct b200_gemm_profile {
    bool on = false;
    cudaEvent_t ev[PROF_SLOTS][4];
    long long calls = 0;      // layer calls recorded since profiling was enabled
};
namespace {

__global__ void pack_weights_kernel(int which, const uint8_t* __restrict__ src, uint8_t* __restrict__ packed, int E,
                                    int D, int I, long long chunks) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= chunks) return;
    const int Kdim = which == 1 ? D : I;
    const int nkb = Kdim / 128;
    const int NT = which == 1 ? I / 128 : D / 256;
    const int c16 = (int)(i & 7);
    const int r = (int)((i >> 3) & 255);
    long long t = i >> 11;
    const int kb = (int)(t % nkb); t /= nkb;
    const int nt = (int)(t % NT);
    const int e = (int)(t / NT);
    long long row;
    if (which == 1) {
        // group g of the tile's 256 rows = [gate j0 + g QCOLS/2 .. | up j0 + g QCOLS/2 ..], QCOLS/2 rows each
        const int j0 = nt * 128, g = r / QCOLS, up = (r / (QCOLS / 2)) & 1, rr = r % (QCOLS / 2);
        row = (long long)e * 2 * I + (up ? I : 0) + j0 + (QCOLS / 2) * g + rr;
    } else {
        row = (long long)e * D + nt * 256 + r;
    }
    const uint4 v = *reinterpret_cast<const uint4*>(src + row * Kdim + (long long)kb * 128 + c16 * 16);
    *reinterpret_cast<uint4*>(packed + i * 16) = v;
}

bool g_regs_ok = true;

struct Fp8Scratch {
    RouteScratch route; int* ids; float* wts; int* hist; int* counts; int* offsets; int* row_pair;
    uint8_t* sq; float* ss; int* row_tok; float* row_w; uint8_t* act_q; float* act_s;
    int* pair_row; float* rows;     // deterministic combine only
};

void carve_fp8(WsCarver& c, const b200_moe_fp8_config* cfg, bool with_route, Fp8Scratch& s) {
    const size_t T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim,
                 I = cfg->intermediate_dim;
    const size_t TK = T * K;
    s.route = RouteScratch{};
    if (with_route) {
        const bool tc = moe_gate_tc_supported((int)T, (int)E, (int)D);
        s.route.partials = c.take<float>((size_t)max(moe_gate_chunks((int)D, true), moe_gate_tc_slots((int)D)) * T * E);
        s.route.whi = tc ? c.take<float>(E * D) : nullptr;
        s.route.wlo = tc ? c.take<float>(E * D) : nullptr;
        s.route.flag_list = tc ? c.take<int>(T) : nullptr;
        s.route.flag_n = tc ? c.take<int>(1) : nullptr;
    }
    s.ids = c.take<int>(TK);
    s.wts = c.take<float>(TK);
    s.hist = c.take<int>(E);
    s.counts = c.take<int>(E);
    s.offsets = c.take<int>(E + 1);
    s.row_pair = c.take<int>(TK);
    s.sq = c.take<uint8_t>(TK * D);
    s.ss = c.take<float>(TK * (D / 128));
    s.row_tok = c.take<int>(TK);
    s.row_w = c.take<float>(TK);
    s.act_q = c.take<uint8_t>(TK * I);
    s.act_s = c.take<float>(TK * (I / 128));
    const bool det = (cfg->flags & B200_MOE_DETERMINISTIC) != 0;
    s.pair_row = det ? c.take<int>(TK) : nullptr;
    s.rows = det ? c.take<float>(TK * D) : nullptr;
}

int check_fp8_cfg(const b200_moe_fp8_config* cfg) {
    if (!cfg) return B200_BAD_ARG;
    if (cfg->num_tokens <= 0 || cfg->num_experts <= 0 || cfg->top_k <= 0) return B200_BAD_SHAPE;
    if (cfg->hidden_dim <= 0 || cfg->intermediate_dim <= 0) return B200_BAD_SHAPE;
    if (cfg->hidden_dim % 256 || cfg->intermediate_dim % 128) return B200_BAD_SHAPE;
    if (cfg->num_experts > MAX_E) return B200_UNSUPPORTED;
    if ((cfg->flags & B200_MOE_DETERMINISTIC) && cfg->top_k > 64) return B200_UNSUPPORTED;
    if ((long long)cfg->num_experts * 2 * cfg->intermediate_dim > 0x7fffffffLL) return B200_UNSUPPORTED;
    if ((long long)cfg->num_experts * cfg->hidden_dim > 0x7fffffffLL) return B200_UNSUPPORTED;
    return B200_OK;
}

// permute + sort + GEMM1 (+ GEMM2) on given routing
int run_experts(b200_ws* ws, const Fp8Scratch& s, const uint8_t* xq, const float* xs, const int* ids,
                const float* wts, const int* hist, const uint8_t* w1q, const float* w1s, const uint8_t* w2q, const float* w2s,
                float* out, const b200_moe_fp8_config* cfg, bool do_gemm2, bool packed, cudaStream_t stream,
                bool zero_out = true) {
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim,
              I = cfg->intermediate_dim;
    const long long TK = (long long)T * K;
    // ids from this library's router are trusted (hist given); ids from outside get the duplicate check
    int st = launch_permute(ids, T, K, E, hist, hist != nullptr, s.counts, s.offsets, s.row_pair, stream);
    if (st) return st;
    const bool det = (cfg->flags & B200_MOE_DETERMINISTIC) != 0 && do_gemm2;
    if (det) B200_CUDA_TRY(cudaMemsetAsync(s.pair_row, 0xFF, sizeof(int) * (size_t)TK, stream));
    const unsigned sort_blocks = (unsigned)(TK < (long long)ws->sm_count * 32 ? TK : (long long)ws->sm_count * 32);
    sort_rows_fp8_kernel<<<sort_blocks, 128, 0, stream>>>(xq, xs, s.row_pair, s.offsets, wts, E, K, D, s.sq, s.ss,
                                                           s.row_tok, s.row_w, det ? s.pair_row : nullptr);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());

    static bool attr_done[64] = {false};
    if (b200_first_call_on_device(attr_done)) {
        const void* kernels[9] = {(const void*)grouped_gemm_fp8_kernel<1, false>, (const void*)grouped_gemm_fp8_kernel<2, false>,
                                  (const void*)grouped_gemm_fp8_kernel<3, false>, (const void*)grouped_gemm_fp8_kernel<1, true>,
                                  (const void*)grouped_gemm_fp8_kernel<2, true>, (const void*)grouped_gemm_fp8_kernel<3, true>,
                                  (const void*)grouped_gemm_mx_kernel<1>, (const void*)grouped_gemm_mx_kernel<2>,
                                  (const void*)grouped_gemm_mx_kernel<3>};
        for (int i = 0; i < 9; i++)
            B200_CUDA_TRY(cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)(i < 6 ? GEMM_SMEM_BYTES : GEMM_MX_SMEM_BYTES)));
        // setmaxnreg.inc waits without bound for registers that only setmaxnreg.dec of the same CTA frees:
        // never launch a build whose compiled register count breaks the balance the budgets assume
        for (int i = 0; i < 9; i++) {
            cudaFuncAttributes a{};
            B200_CUDA_TRY(cudaFuncGetAttributes(&a, kernels[i]));
            const int n = a.numRegs;
            if (!(n * GEMM_THREADS <= 65536 && n <= PROMO_REGS && NUM_PROMO_WARPS * (PROMO_REGS - n) <= 4 * (n - AUX_REGS)))
                g_regs_ok = false;
        }
    }
    if (!g_regs_ok) {
        b200_set_last_error_text("grouped GEMM: the compiled register count does not balance the setmaxnreg budgets");
        return B200_UNSUPPORTED;
    }
    b200_gemm_profile* prof = (ws->gemm_prof && ws->gemm_prof->on) ? ws->gemm_prof : nullptr;
    const int slot = prof ? (int)(prof->calls % PROF_SLOTS) : 0;
    // Single-CTA 128-row tiles unless the caller asks for CTA pairs.  Measured on B200 the pair tiles (256 rows,
    // half of the weight tile per SM, a third less shared-memory traffic) are slower at every shape tried
    // (config 3: GEMM1 3.0 vs 2.2 ms; 32 experts x 1024 rows: 1.9 vs 1.3 ms): the K-block period is set by the
    // promotion of the accumulator stage through tcgen05.ld, which is the same per SM in both shapes, not by
    // shared-memory bandwidth, and a pair idles half of its rows on experts with fewer than 129 rows.
    const bool mx = (cfg->flags & B200_MOE_POW2_SCALES) != 0;      // power-of-two scales: hardware block-scaled MMA
    bool pair = (cfg->flags & B200_MOE_CTA_PAIR_TILES) != 0;
    if ((cfg->flags & B200_MOE_SINGLE_CTA_TILES) || mx) pair = false;
    if (ws->sm_count < 2) pair = false;
    const unsigned grid = pair ? (unsigned)(ws->sm_count / 2) * 2 : (unsigned)ws->sm_count;
    auto launch = [&](int mode, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p) -> int {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(grid); lc.blockDim = dim3(GEMM_THREADS); lc.stream = stream;
        lc.dynamicSmemBytes = mx ? GEMM_MX_SMEM_BYTES : GEMM_SMEM_BYTES;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
#ifndef B200_GEMM_CLUSTER2
#define B200_GEMM_CLUSTER2 1
#endif
        // Single-CTA tiles are launched as clusters of two as well: tiles 2i and 2i+1 (the two 128-row tiles of
        // an expert's weight slab when it has 129..256 rows) then run on SMs of one GPC, behind the same L2
        // partition, and the slab comes from DRAM once instead of once per die.
        const bool cluster2 = pair || (B200_GEMM_CLUSTER2 && grid % 2 == 0);
        lc.attrs = attr; lc.numAttrs = cluster2 ? 1 : 0;
        cudaError_t err;
        if (mx) {
            if (mode == 1)      err = cudaLaunchKernelEx(&lc, grouped_gemm_mx_kernel<1>, ta, tb, p);
            else if (mode == 2) err = cudaLaunchKernelEx(&lc, grouped_gemm_mx_kernel<2>, ta, tb, p);
            else                err = cudaLaunchKernelEx(&lc, grouped_gemm_mx_kernel<3>, ta, tb, p);
        } else if (pair) {
            if (mode == 1)      err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<1, true>, ta, tb, p);
            else if (mode == 2) err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<2, true>, ta, tb, p);
            else                err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<3, true>, ta, tb, p);
        } else {
            if (mode == 1)      err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<1, false>, ta, tb, p);
            else if (mode == 2) err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<2, false>, ta, tb, p);
            else                err = cudaLaunchKernelEx(&lc, grouped_gemm_fp8_kernel<3, false>, ta, tb, p);
        }
        b200_count_launch(1);
        B200_CUDA_TRY(err);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    };
    CUtensorMap ta, tb;
    GemmParams p{};
    p.offsets = s.offsets; p.E = E; p.D = D; p.I = I; p.status = ws->d_status; p.total_rows = TK;
#ifdef B200_GEMM_TRACE
    p.trace = g_gemm_trace; p.trace_warp = g_gemm_trace_warp;
#endif

    // GEMM1 (a CTA of a pair fetches half of a weight tile: boxes of 128 rows instead of 256)
    st = b200_make_tmap_u8_sw128(&ta, s.sq, (unsigned long long)TK, D, 128);
    if (st) return st;
    p.packed = packed ? 1 : 0;
    if (packed) st = b200_make_tmap_u8_sw128(&tb, w1q, (unsigned long long)E * 2 * I * (D / 128), 128, pair ? 128 : 256);
    else        st = b200_make_tmap_u8_sw128(&tb, w1q, (unsigned long long)E * 2 * I, D, QCOLS / 2);
    if (st) return st;
    p.a_scale = s.ss; p.w_scale = w1s; p.act_q = s.act_q; p.act_s = s.act_s;
    if (prof) B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][0], stream));
    st = launch(1, ta, tb, p);
    if (st) return st;
    if (prof) B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][1], stream));
    if (!do_gemm2) return B200_OK;

    // GEMM2
    st = b200_make_tmap_u8_sw128(&ta, s.act_q, (unsigned long long)TK, I, 128);
    if (st) return st;
    if (packed) st = b200_make_tmap_u8_sw128(&tb, w2q, (unsigned long long)E * D * (I / 128), 128, pair ? 128 : 256);
    else        st = b200_make_tmap_u8_sw128(&tb, w2q, (unsigned long long)E * D, I, pair ? 128 : 256);
    if (st) return st;
    p.a_scale = s.act_s; p.w_scale = w2s; p.row_tok = s.row_tok; p.row_w = s.row_w;
#ifdef B200_GEMM_TRACE
    if (p.trace) p.trace += 8 * TRACE_CAP;      // second half of the buffer for GEMM2
#endif
    if (det) {
        p.out = s.rows;
        if (prof) B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][2], stream));
        st = launch(3, ta, tb, p);
        if (st) return st;
        reduce_rows_kernel<<<T, 256, 0, stream>>>(s.rows, s.pair_row, ids, K, D, out);
        if (prof) { B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][3], stream)); prof->calls++; }
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    p.out = out;
    if (zero_out) B200_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)T * D, stream));
    if (prof) B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][2], stream));
    st = launch(2, ta, tb, p);
    if (st) return st;
    if (prof) { B200_CUDA_TRY(cudaEventRecord(prof->ev[slot][3], stream)); prof->calls++; }
    return B200_OK;
}

}  // namespace

extern "C" {

#ifdef B200_GEMM_TRACE
// Timeline builds only (-DB200_GEMM_TRACE; never part of the default library): CTA 0 of the next grouped
// GEMM launches fills dev_buf [2][8][512] with clock64 stamps of its pipeline events.
__attribute__((visibility("default"))) void b200_debug_gemm_trace(long long* dev_buf, int warp) {
    g_gemm_trace = dev_buf;
    g_gemm_trace_warp = warp;
}
#endif

int b200_moe_fp8_profile(b200_ws* ws, int enable) {
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    if (!ws->gemm_prof) {
        if (!enable) return B200_OK;
        b200_gemm_profile* pr = new b200_gemm_profile();
        for (int i = 0; i < PROF_SLOTS; i++)
            for (int j = 0; j < 4; j++) B200_CUDA_TRY(cudaEventCreate(&pr->ev[i][j]));
        ws->gemm_prof = pr;
    }
    ws->gemm_prof->on = enable != 0;
    ws->gemm_prof->calls = 0;
    return B200_OK;
}

int b200_moe_fp8_profile_read(b200_ws* ws, float* gemm1_ms, float* gemm2_ms, int* calls) {
    if (!gemm1_ms || !gemm2_ms || !calls) return B200_BAD_ARG;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    const b200_gemm_profile* pr = ws->gemm_prof;
    const int n = pr ? (int)(pr->calls < PROF_SLOTS ? pr->calls : PROF_SLOTS) : 0;
    *calls = n;
    *gemm1_ms = *gemm2_ms = 0.0f;
    if (n == 0) return B200_OK;
    double s1 = 0.0, s2 = 0.0;
    for (int i = 0; i < n; i++) {
        float a = 0.f, b = 0.f;
        B200_CUDA_TRY(cudaEventSynchronize(pr->ev[i][3]));
        B200_CUDA_TRY(cudaEventElapsedTime(&a, pr->ev[i][0], pr->ev[i][1]));
        B200_CUDA_TRY(cudaEventElapsedTime(&b, pr->ev[i][2], pr->ev[i][3]));
        s1 += a; s2 += b;
    }
    *gemm1_ms = (float)(s1 / n);
    *gemm2_ms = (float)(s2 / n);
    return B200_OK;
}

static int experts_impl(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                        const float* expert_w, const uint8_t* w1q, const float* w1s, const uint8_t* w2q,
                        const float* w2s, float* out, const b200_moe_fp8_config* cfg, bool packed,
                        b200_stream_t stream, bool zero_out = true) {
    int st = check_fp8_cfg(cfg);
    if (st) return st;
    if (!xq || !xs || !expert_ids || !expert_w || !w1q || !w1s || !w2q || !w2s || !out) return B200_BAD_ARG;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    Fp8Scratch s;
    WsCarver sz(nullptr);
    carve_fp8(sz, cfg, false, s);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    carve_fp8(cv, cfg, false, s);
    return run_experts(ws, s, xq, xs, expert_ids, expert_w, nullptr, w1q, w1s, w2q, w2s, out, cfg, true, packed, stream,
                       zero_out);
}

}  // extern "C"

// Expert-parallel owner side (moe_ep.cu): `out` already holds zeros in every row that can receive a
// contribution (the push kernel of the previous step cleared what it read), so the scatter-add GEMM2
// runs without the zero-fill pass over the whole row capacity.
int b200_moe_fp8_experts_accumulate(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                    const float* expert_w, const uint8_t* w1, const float* w1s, const uint8_t* w2,
                                    const float* w2s, float* out, const b200_moe_fp8_config* cfg, bool packed,
                                    cudaStream_t stream) {
    if (cfg && (cfg->flags & B200_MOE_DETERMINISTIC)) return B200_UNSUPPORTED;
    return experts_impl(ws, xq, xs, expert_ids, expert_w, w1, w1s, w2, w2s, out, cfg, packed, stream, false);
}

extern "C" {

int b200_moe_fp8_experts(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                         const float* expert_w, const uint8_t* w1q, const float* w1s, const uint8_t* w2q,
                         const float* w2s, float* out, const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    return experts_impl(ws, xq, xs, expert_ids, expert_w, w1q, w1s, w2q, w2s, out, cfg, false, stream);
}

int b200_moe_fp8_experts_packed(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                const float* expert_w, const uint8_t* w1p, const float* w1s, const uint8_t* w2p,
                                const float* w2s, float* out, const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    return experts_impl(ws, xq, xs, expert_ids, expert_w, w1p, w1s, w2p, w2s, out, cfg, true, stream);
}

static int forward_impl(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w, const float* bias,
                        const uint8_t* w1q, const float* w1s, const uint8_t* w2q, const float* w2s, float* out,
                        const b200_moe_fp8_config* cfg, bool packed, b200_stream_t stream) {
    int st = check_fp8_cfg(cfg);
    if (st) return st;
    if (!xq || !xs || !gate_w || !w1q || !w1s || !w2q || !w2s || !out) return B200_BAD_ARG;
    const int T = cfg->num_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim;
    st = check_route_cfg(T, E, K, D, cfg->scoring, cfg->n_group, cfg->topk_group);
    if (st) return st;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    Fp8Scratch s;
    WsCarver sz(nullptr);
    carve_fp8(sz, cfg, true, s);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    carve_fp8(cv, cfg, true, s);
    st = moe_route_fp8_run(s.route, xq, xs, gate_w, bias, s.ids, s.wts, s.hist, nullptr, cfg, ws->d_status, stream);
    if (st) return st;
    ws->route_flag_n = (s.route.whi && cfg->scoring == B200_SCORE_SIGMOID_GROUPED && !(cfg->flags & B200_MOE_EXACT_ROUTER_LOGITS))
                           ? s.route.flag_n : nullptr;
    return run_experts(ws, s, xq, xs, s.ids, s.wts, s.hist, w1q, w1s, w2q, w2s, out, cfg, true, packed, stream);
}

int b200_moe_fp8_forward(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w, const float* bias,
                         const uint8_t* w1q, const float* w1s, const uint8_t* w2q, const float* w2s, float* out,
                         const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    return forward_impl(ws, xq, xs, gate_w, bias, w1q, w1s, w2q, w2s, out, cfg, false, stream);
}

int b200_moe_fp8_forward_packed(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w,
                                const float* bias, const uint8_t* w1p, const float* w1s, const uint8_t* w2p,
                                const float* w2s, float* out, const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    return forward_impl(ws, xq, xs, gate_w, bias, w1p, w1s, w2p, w2s, out, cfg, true, stream);
}

// Weight pre-tiling.  which = 1: w1 [E,2I,D] -> tiles of 256 accumulator rows (gate j0..+63, up j0..+63,
// gate j0+64..+127, up j0+64..+127 for j0 = 128 * n_tile); which = 2: w2 [E,D,I] -> tiles of 256 rows.
// packed[(((e * NT + n_tile) * nkb + kb) * 256 + r) * 128 + b] = src[e][row(n_tile, r)][kb * 128 + b].
int b200_moe_fp8_pack_weights(int which, const uint8_t* src, uint8_t* packed, int E, int D, int I,
                              b200_stream_t stream) {
    if (!src || !packed) return B200_BAD_ARG;
    if (which != 1 && which != 2) return B200_BAD_ARG;
    if (E <= 0 || D <= 0 || I <= 0 || D % 256 || I % 128) return B200_BAD_SHAPE;
    const int Kdim = which == 1 ? D : I;
    const int NT = which == 1 ? I / 128 : D / 256;
    const long long chunks = (long long)E * NT * (Kdim / 128) * 256 * 8;     // 16-byte chunks
    long long blocks = (chunks + 255) / 256;
    if (blocks > 0x7fffffffLL) return B200_UNSUPPORTED;
    pack_weights_kernel<<<(unsigned)blocks, 256, 0, stream>>>(which, src, packed, E, D, I, chunks);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_moe_fp8_gemm1_stage(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                             const uint8_t* w1q, const float* w1s, uint8_t* act_q, float* act_s, int* offsets,
                             int* row_pair, const b200_moe_fp8_config* cfg, b200_stream_t stream) {
    int st = check_fp8_cfg(cfg);
    if (st) return st;
    if (!xq || !xs || !expert_ids || !w1q || !w1s || !act_q || !act_s || !offsets || !row_pair) return B200_BAD_ARG;
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    Fp8Scratch s;
    WsCarver sz(nullptr);
    carve_fp8(sz, cfg, false, s);
    float* dummy_w = sz.take<float>((size_t)cfg->num_tokens * cfg->top_k);
    st = b200_ws_ensure(ws, sz.total());
    if (st) return st;
    WsCarver cv(ws->base);
    carve_fp8(cv, cfg, false, s);
    dummy_w = cv.take<float>((size_t)cfg->num_tokens * cfg->top_k);
    const size_t TK = (size_t)cfg->num_tokens * cfg->top_k;
    B200_CUDA_TRY(cudaMemsetAsync(dummy_w, 0, sizeof(float) * TK, stream));
    B200_CUDA_TRY(cudaMemsetAsync(s.act_q, 0, TK * cfg->intermediate_dim, stream));
    B200_CUDA_TRY(cudaMemsetAsync(s.act_s, 0, sizeof(float) * TK * (cfg->intermediate_dim / 128), stream));
    st = run_experts(ws, s, xq, xs, expert_ids, dummy_w, nullptr, w1q, w1s, nullptr, nullptr, nullptr, cfg, false, false, stream);
    if (st) return st;
    B200_CUDA_TRY(cudaMemcpyAsync(act_q, s.act_q, TK * cfg->intermediate_dim, cudaMemcpyDeviceToDevice, stream));
    B200_CUDA_TRY(cudaMemcpyAsync(act_s, s.act_s, sizeof(float) * TK * (cfg->intermediate_dim / 128),
                                  cudaMemcpyDeviceToDevice, stream));
    B200_CUDA_TRY(cudaMemcpyAsync(offsets, s.offsets, sizeof(int) * (cfg->num_experts + 1),
                                  cudaMemcpyDeviceToDevice, stream));
    B200_CUDA_TRY(cudaMemcpyAsync(row_pair, s.row_pair, sizeof(int) * TK, cudaMemcpyDeviceToDevice, stream));
    return B200_OK;
}

}  // extern "C"
