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
