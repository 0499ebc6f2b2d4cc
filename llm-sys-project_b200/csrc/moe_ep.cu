// Expert-parallel helpers around the collectives (the reference has no multi-GPU path; these serve the
// expert-sharded layer that sits on top of b200_moe_fp8_experts).
//
//   ep_plan_kernel      one block per destination rank (experts placed contiguously or strided over the
//                       ranks): which tokens have at least one selected expert on that rank, in ascending
//                       token order (stable), with their K slots rewritten to the rank's local expert
//                       numbering (-1 and weight 0 for slots owned elsewhere).
//   ep_sum_rows_kernel  out[t] = sum over ranks (in rank order) of the partial row that came back for
//                       (t, rank); no atomics, no zero-fill pass.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

void b200_count_launch(int n);

namespace {

__global__ void __launch_bounds__(1024)
ep_plan_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int T, int K, int epr, int W, int strided,
               const int* __restrict__ owner_map, const int* __restrict__ local_map, int* __restrict__ send_tok, int* __restrict__ pos, int* __restrict__ send_counts,
               int* __restrict__ slot_ids, float* __restrict__ slot_w) {
    __shared__ int warp_sums[32];
    __shared__ int s_base;
    const int r = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // contiguous placement: expert e lives on rank e / epr as local expert e % epr;
    // strided placement: on rank e % W as local expert e / W (spreads runs of hot experts over the ranks);
    // mapped placement: owner_map[e] / local_map[e] (any assignment, e.g. balanced by measured load)
    auto owner = [&](int id) -> int { return owner_map ? owner_map[id] : (strided ? id % W : id / epr); };
    auto local = [&](int id) -> int { return local_map ? local_map[id] : (strided ? id / W : id % epr); };
    auto rank_mask = [&](int t) -> unsigned long long {
        unsigned long long m = 0;
        for (int k = 0; k < K; k++) {
            const int id = ids[(size_t)t * K + k];
            if (id >= 0 && id < epr * W) m |= 1ull << owner(id);
        }
        return m;
    };
    // rows going to lower ranks
    int lower = 0;
    const unsigned long long below = (r == 0) ? 0ull : ((r >= 64) ? ~0ull : ((1ull << r) - 1));
    for (int t = threadIdx.x; t < T; t += blockDim.x) lower += __popcll(rank_mask(t) & below);
    for (int o = 16; o > 0; o >>= 1) lower += __shfl_xor_sync(0xffffffffu, lower, o);
    if (lane == 0) warp_sums[warp] = lower;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) tot += warp_sums[w];
        s_base = tot;
    }
    __syncthreads();
    const int base = s_base;
    int running = 0;
    for (int t0 = 0; t0 < T; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        const bool f = (t < T) && ((rank_mask(t) >> r) & 1ull);
        const unsigned bal = __ballot_sync(0xffffffffu, f);
        const int within = __popc(bal & ((1u << lane) - 1));
        __syncthreads();                      // readers of the previous round are done
        if (lane == 0) warp_sums[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) {
            const int n = warp_sums[w];
            if (w < warp) before += n;
            total += n;
        }
        if (t < T) {
            int p = -1;
            if (f) {
                p = base + running + before + within;
                send_tok[p] = t;
                for (int k = 0; k < K; k++) {
                    const int id = ids[(size_t)t * K + k];
                    const bool mine = id >= 0 && id < epr * W && owner(id) == r;
                    slot_ids[(size_t)p * K + k] = mine ? local(id) : -1;
                    slot_w[(size_t)p * K + k] = mine ? wts[(size_t)t * K + k] : 0.0f;
                }
            }
            pos[(size_t)r * T + t] = p;
        }
        running += total;
    }
    if (threadIdx.x == 0) send_counts[r] = running;
}

template <bool BF16>
__global__ void __launch_bounds__(256)
ep_sum_rows_kernel(const void* __restrict__ back, const int* __restrict__ pos, int W, int T, int D,
                   float* __restrict__ out) {
    const int t = blockIdx.x;
    __shared__ int s_pos[64];
    if (threadIdx.x < W) s_pos[threadIdx.x] = pos[(size_t)threadIdx.x * T + t];
    __syncthreads();
    for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < W; r++) {
            const int p = s_pos[r];
            if (p < 0) continue;
            if (BF16) {
                const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(back) + (size_t)p * D + c);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __bfloat1622float2(h[i]);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                }
            } else {
                const float4* src = reinterpret_cast<const float4*>(static_cast<const float*>(back) + (size_t)p * D + c);
                const float4 a = src[0], b = src[1];
                acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
                acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
            }
        }
        float4* dst = reinterpret_cast<float4*>(out + (size_t)t * D + c);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

}  // namespace

extern "C" {

int b200_ep_plan(const int* expert_ids, const float* expert_w, int T, int K, int experts_per_rank, int world,
                 int strided, const int* owner_map, const int* local_map, int* send_tok, int* pos, int* send_counts,
                 int* slot_ids, float* slot_w, cudaStream_t stream) {
    if (!expert_ids || !expert_w || !send_tok || !pos || !send_counts || !slot_ids || !slot_w) return B200_BAD_ARG;
    if (T <= 0 || K <= 0 || experts_per_rank <= 0) return B200_BAD_SHAPE;
    if (world <= 0 || world > 64) return B200_UNSUPPORTED;
    if ((owner_map == nullptr) != (local_map == nullptr)) return B200_BAD_ARG;
    ep_plan_kernel<<<world, 1024, 0, stream>>>(expert_ids, expert_w, T, K, experts_per_rank, world, strided ? 1 : 0,
                                               owner_map, local_map, send_tok, pos, send_counts, slot_ids, slot_w);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_ep_sum_rows(const void* back, int back_is_bf16, const int* pos, int world, int T, int D, float* out,
                     cudaStream_t stream) {
    if (!back || !pos || !out) return B200_BAD_ARG;
    if (T <= 0 || D <= 0 || D % 8) return B200_BAD_SHAPE;
    if (world <= 0 || world > 64) return B200_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(back) | reinterpret_cast<uintptr_t>(out)) & 15) return B200_BAD_ARG;
    if (back_is_bf16) ep_sum_rows_kernel<true><<<T, 256, 0, stream>>>(back, pos, world, T, D, out);
    else              ep_sum_rows_kernel<false><<<T, 256, 0, stream>>>(back, pos, world, T, D, out);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"

// =================================================================================================
// Expert-parallel layer behind the C ABI: one host thread (process) per GPU, the data plane in this
// library's own kernels over peer memory (CUDA IPC mappings of each rank's receive buffers, NVLink /
// NVSwitch underneath), no host synchronisation and no collective-library call inside a step.
//
// Every rank owns one exchange buffer that all peers map:
//     disp_word[W]   one 64-bit word per source rank: (step << 32) | rows sent       (written by peers)
//     back_word[W]   one 64-bit word per owner rank:  (step << 32) | 1                (written by peers)
//     recv_q/s/id/w  W regions of max_tokens rows: the rows source s dispatched to this rank
//     back           W regions of max_tokens rows: the partial output rows owner o returned, in the order
//                    this rank dispatched them to o
// A step:
//     route + plan                   local kernels (the router's ids/weights, rows per owner rank)
//     ep_dispatch_kernel             every (token, owner) row is stored into the owner's region of this
//                                    rank (FP8 row, 1x128 scales, local slot ids, weights) with plain
//                                    16-byte peer stores; the last block publishes the row counts
//     ep_recv_ready_kernel           owner side: bounded wait for every source's word, rows beyond a
//                                    source's count are marked empty
//     grouped GEMMs                  b200_moe_fp8_experts on the regions (local memory only: the tensor
//                                    maps never cover a peer's memory), per-token partial sums by the
//                                    GEMM2 scatter-add
//     ep_push_kernel                 partial rows -> fp16 relative to the row maximum (or fp32) -> the source
//                                    rank's `back` region (peer stores), clears what it read; the last block
//                                    publishes the back words
//     ep_combine_kernel              source side: bounded wait for every owner's word, then the per-token
//                                    sum in rank order
// A region is reused by the next step only after its reader has finished: a rank dispatches step n+1
// after its own combine of step n, which waits for every owner's push of step n, which follows that
// owner's GEMMs of step n.  Waits give up after wait_limit_ms and set B200_TIMEOUT in the status word;
// every count read from a peer-written word is clamped to the region size, so a step that timed out
// computes garbage but touches no memory outside the buffers.
// =================================================================================================
#include <cstdio>
#include <cstring>
#include <vector>

#include "moe_internal.cuh"
#include "selftest.h"

void b200_set_last_error_text(const char* text);

struct b200_ep {
    b200_ep_config cfg{};
    int E_local = 0;
    b200_ws* ws = nullptr;
    // exchange buffer (peers map it)
    char* xbuf = nullptr;
    size_t xbytes = 0;
    char* peer[64] = {nullptr};      // peer[r] = rank r's exchange buffer in this process's address space
    bool peer_opened[64] = {false};
    bool connected = false;
    // local buffers
    char* lbuf = nullptr;
    int *d_owner = nullptr, *d_local = nullptr;
    int *ids = nullptr, *hist = nullptr, *send_tok = nullptr, *pos = nullptr, *send_counts = nullptr, *slot_ids = nullptr;
    int *recv_counts = nullptr;
    unsigned int* done = nullptr;     // [2] block counters of the dispatch / push kernels
    float *wts = nullptr, *slot_w = nullptr, *y = nullptr;
    RouteScratch route{};
    char** d_peer = nullptr;          // device copy of peer[]
    unsigned int step = 0;
    int sm_count = 0;
    // phase timeline of a step (b200_ep_phase_profile, a test / benchmark hook): events on the launch stream
    bool prof_on = false;
    cudaEvent_t prof_ev[7] = {nullptr};
};

namespace {

struct XLayout {
    size_t disp_word, back_word, recv_q, recv_s, recv_id, recv_w, back, back_scale, total;
};
__host__ __device__ inline XLayout x_layout(int W, int Tm, int K, int D, int back_elem_bytes) {
    XLayout L;
    size_t off = 0;
    auto take = [&](size_t n) { size_t r = off; off = (off + n + 255) & ~size_t(255); return r; };
    L.disp_word = take(8 * (size_t)W);
    L.back_word = take(8 * (size_t)W);
    L.recv_q = take((size_t)W * Tm * D);
    L.recv_s = take((size_t)W * Tm * (D / 128) * 4);
    L.recv_id = take((size_t)W * Tm * K * 4);
    L.recv_w = take((size_t)W * Tm * K * 4);
    L.back = take((size_t)W * Tm * D * back_elem_bytes);
    L.back_scale = take((size_t)W * Tm * 4);
    L.total = off;
    return L;
}

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait for a peer-written word whose upper half carries the step number.  Returns the lower
// half, or -1 after limit_ns without the expected step (the caller records B200_TIMEOUT).
__device__ long long wait_word(const unsigned long long* p, unsigned int step, unsigned long long limit_ns) {
    uint64_t t0 = 0;
    for (unsigned it = 0;; it++) {
        const unsigned long long v = ld_acquire_sys_u64(p);
        if ((unsigned int)(v >> 32) == step) return (long long)(v & 0xffffffffull);
        if ((it & 63u) == 63u) {
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) return -1;
            __nanosleep(100);
        }
    }
}

struct EpDev {
    char* const* peer;      // [W] exchange buffers
    char* self;             // this rank's exchange buffer
    XLayout L;
    int rank, W, Tm, K, D;
    unsigned int step;
    unsigned long long limit_ns;
    int* status;
};

// One block per dispatched row (grid-stride).  Rows are rank-major in send_tok / slot_ids / slot_w.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const EpDev e, const uint8_t* __restrict__ xq, const float* __restrict__ xs,
                   const int* __restrict__ send_tok, const int* __restrict__ send_counts,
                   const int* __restrict__ slot_ids, const float* __restrict__ slot_w, unsigned int* done) {
    __shared__ int s_start[65];
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int r = 0; r < e.W; r++) { s_start[r] = acc; acc += min(max(send_counts[r], 0), e.Tm); }
        s_start[e.W] = acc;
    }
    __syncthreads();
    const int total = s_start[e.W];
    const int nb = e.D / 128;
    for (int i = blockIdx.x; i < total; i += gridDim.x) {
        int r = 0;
        while (i >= s_start[r + 1]) r++;
        const int row = i - s_start[r];
        const int tok = send_tok[i];
        char* dst = e.peer[r];
        const size_t slot = (size_t)e.rank * e.Tm + row;
        const uint4* src = reinterpret_cast<const uint4*>(xq + (size_t)tok * e.D);
        uint4* dq = reinterpret_cast<uint4*>(dst + e.L.recv_q + slot * e.D);
        for (int c = threadIdx.x; c < e.D / 16; c += blockDim.x) dq[c] = src[c];
        float* dsc = reinterpret_cast<float*>(dst + e.L.recv_s) + slot * nb;
        for (int c = threadIdx.x; c < nb; c += blockDim.x) dsc[c] = xs[(size_t)tok * nb + c];
        int* did = reinterpret_cast<int*>(dst + e.L.recv_id) + slot * e.K;
        float* dw = reinterpret_cast<float*>(dst + e.L.recv_w) + slot * e.K;
        for (int c = threadIdx.x; c < e.K; c += blockDim.x) {
            did[c] = slot_ids[(size_t)i * e.K + c];
            dw[c] = slot_w[(size_t)i * e.K + c];
        }
    }
    // the last block to finish publishes the counts: every block's stores are fenced (system scope)
    // before its increment, so the words become visible to the owners after all rows
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(done, 1u) == gridDim.x - 1);
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        for (int r = threadIdx.x; r < e.W; r += blockDim.x) {
            const unsigned long long cnt = (unsigned long long)(s_start[r + 1] - s_start[r]);
            st_release_sys_u64(reinterpret_cast<unsigned long long*>(e.peer[r] + e.L.disp_word) + e.rank,
                               ((unsigned long long)e.step << 32) | cnt);
        }
        if (threadIdx.x == 0) *done = 0;
    }
}

// Owner side, one block per source rank: wait for the source's word, record its row count, mark the
// region's rows beyond the count empty (all slots -1) so that the grouped GEMMs skip them.
__global__ void __launch_bounds__(256)
ep_recv_ready_kernel(const EpDev e, int* __restrict__ recv_counts) {
    __shared__ int s_cnt;
    const int s = blockIdx.x;
    if (threadIdx.x == 0) {
        const long long v = wait_word(reinterpret_cast<const unsigned long long*>(e.self + e.L.disp_word) + s, e.step,
                                      e.limit_ns);
        if (v < 0) atomicExch(e.status, B200_TIMEOUT);
        s_cnt = v < 0 ? 0 : (int)min(v, (long long)e.Tm);
        recv_counts[s] = s_cnt;
    }
    __syncthreads();
    const int cnt = s_cnt;
    int* ids = reinterpret_cast<int*>(e.self + e.L.recv_id) + (size_t)s * e.Tm * e.K;
    for (int i = cnt * e.K + threadIdx.x; i < e.Tm * e.K; i += blockDim.x) ids[i] = -1;
}

// Owner side: partial output rows (fp32 sums over this rank's experts) -> the source rank's `back` region;
// the fp32 rows are cleared for the next step's scatter-add.  HALF: a row travels as fp16 values divided by
// the row's largest magnitude, plus that magnitude (one fp32 per row): 11 significant bits relative to the
// row maximum.  (bf16 rows, 8 bits, broke the 1e-2 absolute bound where a token's partial rows cancel.)
template <bool HALF>
__global__ void __launch_bounds__(256)
ep_push_kernel(const EpDev e, float* __restrict__ y, const int* __restrict__ recv_counts, unsigned int* done) {
    __shared__ int s_start[65];
    __shared__ float s_red[2][8];
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int r = 0; r < e.W; r++) { s_start[r] = acc; acc += min(max(recv_counts[r], 0), e.Tm); }
        s_start[e.W] = acc;
    }
    __syncthreads();
    const int total = s_start[e.W];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int it = 0;
    for (int i = blockIdx.x; i < total; i += gridDim.x, it++) {
        int s = 0;
        while (i >= s_start[s + 1]) s++;
        const int row = i - s_start[s];
        float4* src = reinterpret_cast<float4*>(y + ((size_t)s * e.Tm + row) * e.D);
        char* dst = e.peer[s] + e.L.back;
        const size_t slot = (size_t)e.rank * e.Tm + row;
        if (HALF) {
            // The row stays in registers between the maximum and the conversion (up to 8 float4 per thread: D <=
            // 8192; wider rows read the rest again): one pass over memory, one block barrier per row.
            constexpr int NPT = 8;
            const int nvec = e.D / 4;
            float4 v[NPT];
            float amax = 0.0f;
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                const int c = threadIdx.x + k * 256;
                v[k] = (c < nvec) ? src[c] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < NPT; k++)
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w))));
            for (int c = threadIdx.x + NPT * 256; c < nvec; c += 256) {
                const float4 a = src[c];
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
            }
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            float* red = s_red[it & 1];               // two sets: the next row's writers do not wait for this row's readers
            if (lane == 0) red[warp] = amax;
            __syncthreads();
            amax = red[0];
            for (int w = 1; w < 8; w++) amax = fmaxf(amax, red[w]);
            const float inv = amax > 0.0f ? 1.0f / amax : 0.0f;
            if (threadIdx.x == 0) reinterpret_cast<float*>(e.peer[s] + e.L.back_scale)[slot] = amax;
            uint2* drow = reinterpret_cast<uint2*>(dst + slot * e.D * 2);
#pragma unroll
            for (int k = 0; k < NPT; k++) {
                const int c = threadIdx.x + k * 256;
                if (c < nvec) {
                    src[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                    const __half2 h0 = __floats2half2_rn(v[k].x * inv, v[k].y * inv), h1 = __floats2half2_rn(v[k].z * inv, v[k].w * inv);
                    uint2 u;
                    u.x = *reinterpret_cast<const uint32_t*>(&h0); u.y = *reinterpret_cast<const uint32_t*>(&h1);
                    drow[c] = u;
                }
            }
            for (int c = threadIdx.x + NPT * 256; c < nvec; c += 256) {
                const float4 a = src[c];
                src[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                const __half2 h0 = __floats2half2_rn(a.x * inv, a.y * inv), h1 = __floats2half2_rn(a.z * inv, a.w * inv);
                uint2 u;
                u.x = *reinterpret_cast<const uint32_t*>(&h0); u.y = *reinterpret_cast<const uint32_t*>(&h1);
                drow[c] = u;
            }
        } else {
            for (int c = threadIdx.x; c < e.D / 4; c += blockDim.x) {
                const float4 a = src[c];
                src[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4*>(dst + slot * e.D * 4)[c] = a;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(done, 1u) == gridDim.x - 1);
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        for (int r = threadIdx.x; r < e.W; r += blockDim.x)
            st_release_sys_u64(reinterpret_cast<unsigned long long*>(e.peer[r] + e.L.back_word) + e.rank,
                               ((unsigned long long)e.step << 32) | 1ull);
        if (threadIdx.x == 0) *done = 0;
    }
}

// Source side, one block per token: wait for every owner's word (the first warp polls, one lane per
// owner), then out[t] = sum over owners in rank order of the partial row that came back for (t, owner).
template <bool HALF>
__global__ void __launch_bounds__(256)
ep_combine_kernel(const EpDev e, const int* __restrict__ pos, const int* __restrict__ send_counts, int T,
                  float* __restrict__ out) {
    __shared__ int s_row[64];
    __shared__ float s_scale[64];
    const int t = blockIdx.x;
    if (threadIdx.x < 64) {
        const int r = threadIdx.x;
        int row = -1;
        if (r < e.W) {
            if (wait_word(reinterpret_cast<const unsigned long long*>(e.self + e.L.back_word) + r, e.step, e.limit_ns) < 0)
                atomicExch(e.status, B200_TIMEOUT);
            int start = 0;
            for (int q = 0; q < r; q++) start += min(max(send_counts[q], 0), e.Tm);
            const int p = pos[(size_t)r * T + t];
            if (p >= 0) row = min(max(p - start, 0), e.Tm - 1);
        }
        s_row[r] = row;
        s_scale[r] = (HALF && row >= 0) ? reinterpret_cast<const float*>(e.self + e.L.back_scale)[(size_t)r * e.Tm + row]
                                        : 1.0f;
    }
    __syncthreads();
    // the owners that hold a row of this token, in rank order (the order of the sum)
    __shared__ int s_n;
    __shared__ size_t s_slot[64];
    __shared__ float s_sc[64];
    if (threadIdx.x == 0) {
        int n = 0;
        for (int r = 0; r < e.W; r++)
            if (s_row[r] >= 0) { s_slot[n] = (size_t)r * e.Tm + s_row[r]; s_sc[n] = s_scale[r]; n++; }
        s_n = n;
    }
    __syncthreads();
    const int nv = s_n;
    const char* back = e.self + e.L.back;
    for (int c = threadIdx.x * 8; c < e.D; c += blockDim.x * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // four rows' loads in flight at a time; the additions stay in rank order
        for (int r0 = 0; r0 < nv; r0 += 4) {
            if (HALF) {
                uint4 v[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (r0 + j < nv) v[j] = *reinterpret_cast<const uint4*>(back + (s_slot[r0 + j] * e.D + c) * 2);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (r0 + j < nv) {
                        const __half2* h = reinterpret_cast<const __half2*>(&v[j]);
                        const float sc = s_sc[r0 + j];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const float2 f = __half22float2(h[i]);
                            acc[2 * i] = fmaf(f.x, sc, acc[2 * i]);
                            acc[2 * i + 1] = fmaf(f.y, sc, acc[2 * i + 1]);
                        }
                    }
                }
            } else {
                float4 va[4], vb[4];
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (r0 + j < nv) {
                        const float4* src = reinterpret_cast<const float4*>(back + (s_slot[r0 + j] * e.D + c) * 4);
                        va[j] = src[0]; vb[j] = src[1];
                    }
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (r0 + j < nv) {
                        acc[0] += va[j].x; acc[1] += va[j].y; acc[2] += va[j].z; acc[3] += va[j].w;
                        acc[4] += vb[j].x; acc[5] += vb[j].y; acc[6] += vb[j].z; acc[7] += vb[j].w;
                    }
            }
        }
        float4* dst = reinterpret_cast<float4*>(out + (size_t)t * e.D + c);
        dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

EpDev ep_dev(const b200_ep* ep) {
    EpDev e;
    const b200_ep_config& c = ep->cfg;
    e.peer = ep->d_peer;
    e.self = ep->xbuf;
    e.L = x_layout(c.world, c.max_tokens, c.top_k, c.hidden_dim, (c.flags & B200_EP_COMBINE_F32) ? 4 : 2);
    e.rank = c.rank; e.W = c.world; e.Tm = c.max_tokens; e.K = c.top_k; e.D = c.hidden_dim;
    e.step = ep->step;
    e.limit_ns = (unsigned long long)(c.wait_limit_ms > 0 ? c.wait_limit_ms : 2000) * 1000000ull;
    e.status = ep->ws->d_status;
    return e;
}

}  // namespace

extern "C" {

int b200_ep_create(b200_ep** out, const b200_ep_config* cfg, const int* owner_map, const int* local_map,
                   void* handle_out) {
    if (!out || !cfg || !handle_out) return B200_BAD_ARG;
    if ((owner_map == nullptr) != (local_map == nullptr)) return B200_BAD_ARG;
    const int W = cfg->world, Tm = cfg->max_tokens, E = cfg->num_experts, K = cfg->top_k, D = cfg->hidden_dim,
              I = cfg->intermediate_dim;
    if (W <= 0 || W > 64 || cfg->rank < 0 || cfg->rank >= W) return B200_BAD_ARG;
    if (Tm <= 0 || E <= 0 || K <= 0 || D <= 0 || I <= 0 || E % W || D % 256 || I % 128) return B200_BAD_SHAPE;
    int st = check_route_cfg(Tm, E, K, D, cfg->scoring, cfg->n_group, cfg->topk_group);
    if (st) return st;
    if ((long long)W * Tm * K > 0x7fffffffLL / 2) return B200_UNSUPPORTED;
    if (cfg->flags & B200_MOE_DETERMINISTIC) return B200_UNSUPPORTED;
    b200_ep* ep = new b200_ep();
    ep->cfg = *cfg;
    ep->E_local = E / W;
    st = b200_ws_create(&ep->ws);
    if (st) { delete ep; return st; }
    ep->sm_count = ep->ws->sm_count;
    const XLayout L = x_layout(W, Tm, K, D, (cfg->flags & B200_EP_COMBINE_F32) ? 4 : 2);
    ep->xbytes = L.total;
    B200_CUDA_TRY(cudaMalloc(&ep->xbuf, L.total));
    B200_CUDA_TRY(cudaMemset(ep->xbuf, 0, L.recv_q));           // the words start at step 0
    // local buffers
    const size_t WT = (size_t)W * Tm;
    const int nch = moe_gate_chunks(D, true);
    WsCarver sz(nullptr);
    auto carve = [&](WsCarver& c) {
        ep->d_owner = c.take<int>(E); ep->d_local = c.take<int>(E);
        ep->ids = c.take<int>((size_t)Tm * K); ep->wts = c.take<float>((size_t)Tm * K);
        ep->hist = c.take<int>(E);
        ep->send_tok = c.take<int>(WT); ep->pos = c.take<int>(WT); ep->send_counts = c.take<int>(64);
        ep->slot_ids = c.take<int>(WT * K); ep->slot_w = c.take<float>(WT * K);
        ep->recv_counts = c.take<int>(64);
        ep->done = c.take<unsigned int>(2);
        {
            const bool tc = moe_gate_tc_supported(Tm, E, D);
            const int nparts = nch > moe_gate_tc_slots(D) ? nch : moe_gate_tc_slots(D);
            ep->route.partials = c.take<float>((size_t)nparts * Tm * E);
            ep->route.whi = tc ? c.take<float>((size_t)E * D) : nullptr;
            ep->route.wlo = tc ? c.take<float>((size_t)E * D) : nullptr;
            ep->route.flag_list = tc ? c.take<int>((size_t)Tm) : nullptr;
            ep->route.flag_n = tc ? c.take<int>(1) : nullptr;
        }
        ep->d_peer = c.take<char*>(64);
        ep->y = c.take<float>(WT * D);
    };
    carve(sz);
    B200_CUDA_TRY(cudaMalloc(&ep->lbuf, sz.total()));
    B200_CUDA_TRY(cudaMemset(ep->lbuf, 0, sz.total()));         // y and the block counters start at zero
    WsCarver cv(ep->lbuf);
    carve(cv);
    std::vector<int> own(E), loc(E);
    for (int e = 0; e < E; e++) {
        own[e] = owner_map ? owner_map[e] : e / ep->E_local;
        loc[e] = local_map ? local_map[e] : e % ep->E_local;
        if (own[e] < 0 || own[e] >= W || loc[e] < 0 || loc[e] >= ep->E_local) { b200_ep_destroy(ep); return B200_BAD_ARG; }
    }
    B200_CUDA_TRY(cudaMemcpy(ep->d_owner, own.data(), sizeof(int) * E, cudaMemcpyHostToDevice));
    B200_CUDA_TRY(cudaMemcpy(ep->d_local, loc.data(), sizeof(int) * E, cudaMemcpyHostToDevice));
    // scratch of the owner-side grouped GEMMs at the worst case (every source sends all its tokens)
    {
        const size_t TK = WT * K;
        const size_t need = TK * D + TK * (D / 128) * 4 + TK * I + TK * (I / 128) * 4 + TK * 24 + (size_t)E * 16 + (1 << 20);
        st = b200_ws_ensure(ep->ws, need);
        if (st) { b200_ep_destroy(ep); return st; }
    }
    static_assert(sizeof(cudaIpcMemHandle_t) <= B200_EP_HANDLE_BYTES, "handle size");
    memset(handle_out, 0, B200_EP_HANDLE_BYTES);
    if (W > 1) {
        cudaIpcMemHandle_t h;
        B200_CUDA_TRY(cudaIpcGetMemHandle(&h, ep->xbuf));
        memcpy(handle_out, &h, sizeof(h));
    }
    ep->peer[cfg->rank] = ep->xbuf;
    *out = ep;
    return B200_OK;
}

int b200_ep_connect(b200_ep* ep, const void* handles) {
    if (!ep) return B200_BAD_ARG;
    const int W = ep->cfg.world;
    if (W > 1 && !handles) return B200_BAD_ARG;
    for (int r = 0; r < W; r++) {
        if (r == ep->cfg.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * B200_EP_HANDLE_BYTES, sizeof(h));
        void* p = nullptr;
        B200_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ep->peer[r] = static_cast<char*>(p);
        ep->peer_opened[r] = true;
    }
    B200_CUDA_TRY(cudaMemcpy(ep->d_peer, ep->peer, sizeof(char*) * 64, cudaMemcpyHostToDevice));
    ep->connected = true;
    return B200_OK;
}

int b200_ep_connect_loopback(b200_ep* ep) {
    if (!ep) return B200_BAD_ARG;
    for (int r = 0; r < ep->cfg.world; r++) ep->peer[r] = ep->xbuf;
    B200_CUDA_TRY(cudaMemcpy(ep->d_peer, ep->peer, sizeof(char*) * 64, cudaMemcpyHostToDevice));
    ep->connected = true;
    return B200_OK;
}

int b200_ep_forward(b200_ep* ep, int num_tokens, const uint8_t* xq, const float* xs, const float* gate_w,
                    const float* bias, const uint8_t* w1, const float* w1s, const uint8_t* w2, const float* w2s,
                    int packed, float* out, int* ids_out, float* w_out, b200_stream_t stream) {
    if (!ep || !xq || !xs || !gate_w || !w1 || !w1s || !w2 || !w2s || !out) return B200_BAD_ARG;
    if (!ep->connected) return B200_BAD_ARG;
    const b200_ep_config& c = ep->cfg;
    const int T = num_tokens, W = c.world, K = c.top_k, D = c.hidden_dim, E = c.num_experts;
    if (T <= 0 || T > c.max_tokens) return B200_BAD_SHAPE;
    ep->step++;
    if (ep->step == 0) ep->step = 1;        // 0 is what the words hold before the first step
    auto mark = [&](int i) { if (ep->prof_on) cudaEventRecord(ep->prof_ev[i], stream); };
    mark(0);
    const EpDev e = ep_dev(ep);
    const bool half = !(c.flags & B200_EP_COMBINE_F32);

    // route (replicated router) and plan
    b200_moe_fp8_config rc{};
    rc.num_tokens = T; rc.num_experts = E; rc.top_k = K; rc.hidden_dim = D; rc.intermediate_dim = c.intermediate_dim;
    rc.scoring = c.scoring; rc.n_group = c.n_group; rc.topk_group = c.topk_group; rc.routed_scale = c.routed_scale;
    rc.flags = c.flags & B200_MOE_EXACT_ROUTER_LOGITS;
    RouteScratch rs = ep->route;
    if (!moe_gate_tc_supported(T, E, D)) rs.whi = nullptr;      // this step's batch is too small for the tensor-core router
    int st = moe_route_fp8_run(rs, xq, xs, gate_w, bias, ep->ids, ep->wts, ep->hist, nullptr, &rc, ep->ws->d_status, stream);
    if (st) return st;
    st = b200_ep_plan(ep->ids, ep->wts, T, K, ep->E_local, W, 0, ep->d_owner, ep->d_local, ep->send_tok, ep->pos,
                      ep->send_counts, ep->slot_ids, ep->slot_w, stream);
    if (st) return st;
    if (ids_out) B200_CUDA_TRY(cudaMemcpyAsync(ids_out, ep->ids, sizeof(int) * (size_t)T * K, cudaMemcpyDeviceToDevice, stream));
    if (w_out) B200_CUDA_TRY(cudaMemcpyAsync(w_out, ep->wts, sizeof(float) * (size_t)T * K, cudaMemcpyDeviceToDevice, stream));
    mark(1);

    // dispatch: rows to their owners' regions, then the counts
    const int grid = ep->sm_count * 8;
    ep_dispatch_kernel<<<grid, 256, 0, stream>>>(e, xq, xs, ep->send_tok, ep->send_counts, ep->slot_ids, ep->slot_w,
                                                 ep->done);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());

    mark(2);
    // owner side
    ep_recv_ready_kernel<<<W, 256, 0, stream>>>(e, ep->recv_counts);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    mark(3);
    b200_moe_fp8_config lc{};
    lc.num_tokens = W * c.max_tokens; lc.num_experts = ep->E_local; lc.top_k = K; lc.hidden_dim = D;
    lc.intermediate_dim = c.intermediate_dim; lc.scoring = c.scoring; lc.n_group = 1; lc.topk_group = 1;
    lc.routed_scale = 1.0f; lc.flags = c.flags & B200_MOE_POW2_SCALES;
    st = b200_moe_fp8_experts_accumulate(ep->ws, reinterpret_cast<const uint8_t*>(ep->xbuf + e.L.recv_q),
                                         reinterpret_cast<const float*>(ep->xbuf + e.L.recv_s),
                                         reinterpret_cast<const int*>(ep->xbuf + e.L.recv_id),
                                         reinterpret_cast<const float*>(ep->xbuf + e.L.recv_w), w1, w1s, w2, w2s, ep->y,
                                         &lc, packed != 0, stream);
    if (st) return st;
    mark(4);
    if (half) ep_push_kernel<true><<<grid, 256, 0, stream>>>(e, ep->y, ep->recv_counts, ep->done + 1);
    else      ep_push_kernel<false><<<grid, 256, 0, stream>>>(e, ep->y, ep->recv_counts, ep->done + 1);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());

    mark(5);
    // source side
    if (half) ep_combine_kernel<true><<<T, 256, 0, stream>>>(e, ep->pos, ep->send_counts, T, out);
    else      ep_combine_kernel<false><<<T, 256, 0, stream>>>(e, ep->pos, ep->send_counts, T, out);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    mark(6);
    return B200_OK;
}

// Test / benchmark hook (declared in selftest.h): time the phases of the following steps with events on the launch
// stream.  ms[6] of the last step: route + plan, dispatch, wait for the senders, local experts, push, combine
// (the last one includes the wait for the owners' partial rows).
int b200_ep_phase_profile(b200_ep* ep, int enable, float* ms) {
    if (!ep) return B200_BAD_ARG;
    if (enable && !ep->prof_ev[0])
        for (int i = 0; i < 7; i++) B200_CUDA_TRY(cudaEventCreate(&ep->prof_ev[i]));
    if (ms && ep->prof_on) {
        B200_CUDA_TRY(cudaEventSynchronize(ep->prof_ev[6]));
        for (int i = 0; i < 6; i++) B200_CUDA_TRY(cudaEventElapsedTime(&ms[i], ep->prof_ev[i], ep->prof_ev[i + 1]));
    }
    ep->prof_on = enable != 0;
    return B200_OK;
}

int b200_ep_stats(b200_ep* ep, b200_stream_t stream, int* status, int* send_counts, int* recv_counts) {
    if (!ep) return B200_BAD_ARG;
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    if (status) {
        B200_CUDA_TRY(cudaMemcpy(status, ep->ws->d_status, sizeof(int), cudaMemcpyDeviceToHost));
        if (*status != 0) B200_CUDA_TRY(cudaMemset(ep->ws->d_status, 0, sizeof(int)));
    }
    if (send_counts) B200_CUDA_TRY(cudaMemcpy(send_counts, ep->send_counts, sizeof(int) * ep->cfg.world, cudaMemcpyDeviceToHost));
    if (recv_counts) B200_CUDA_TRY(cudaMemcpy(recv_counts, ep->recv_counts, sizeof(int) * ep->cfg.world, cudaMemcpyDeviceToHost));
    return B200_OK;
}

b200_ws* b200_ep_workspace(b200_ep* ep) { return ep ? ep->ws : nullptr; }

int b200_ep_destroy(b200_ep* ep) {
    if (!ep) return B200_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < 64; r++)
        if (ep->peer_opened[r] && ep->peer[r]) cudaIpcCloseMemHandle(ep->peer[r]);
    if (ep->xbuf) cudaFree(ep->xbuf);
    if (ep->lbuf) cudaFree(ep->lbuf);
    for (int i = 0; i < 7; i++)
        if (ep->prof_ev[i]) cudaEventDestroy(ep->prof_ev[i]);
    if (ep->ws) b200_ws_destroy(ep->ws);
    delete ep;
    return B200_OK;
}

}  // extern "C"
