// Tensor-core self check: one CTA computes D[128,N] = A[128,K] * B[N,K]^T with tcgen05.mma,
// staging the operands through the same shared-memory layouts and descriptors the production
// kernels use.  It exists so that a descriptor or layout mistake shows up as a wrong number in
// a 128 x N matrix instead of as a wrong answer deep inside a fused kernel.
//   mode 0  bf16, A and B K-major, 128-byte swizzle          (DSA: Q and K tiles)
//   mode 1  bf16, A K-major swizzled, B given as [K,N] and staged MN-major, 128-byte swizzle
//                                                          (DSA: V tile, rows = kv, cols = Dv)
//   mode 2  e4m3, A and B K-major, 128-byte swizzle          (MoE grouped GEMMs)
//   mode 3  bf16, A K-major without swizzle (8x16-byte core matrices, chunk-major), B as mode 0
//                                                          (DSA: P tile written by the softmax warps)
#include "common.cuh"
#include "selftest.h"

namespace {

struct SelfSmem {
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};

// elem: bytes per element.  K-major swizzled tile: blocks of 128 bytes along K, each block
// [rows x 128 B]; 16-byte chunk j of row r sits at r*128 + ((j ^ (r & 7)) * 16).
__device__ __forceinline__ uint32_t kmajor_sw128_offset(int r, int kbyte, int rows) {
    int blk = kbyte >> 7, j = (kbyte >> 4) & 7, w = kbyte & 15;
    return (uint32_t)(blk * rows * 128 + r * 128 + ((j ^ (r & 7)) << 4) + w);
}

__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(int mode, const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, float* __restrict__ d,
                     int N, int K, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int esz = (mode == 2) ? 1 : 2;
    const int a_bytes = 128 * K * esz;
    const int b_bytes = N * K * esz;
    uint8_t* sa = base;
    uint8_t* sb = base + ((a_bytes + 1023) & ~1023);
    SelfSmem* sm = reinterpret_cast<SelfSmem*>(sb + ((b_bytes + 1023) & ~1023));
    const int tid = threadIdx.x, warp = tid >> 5;

    if (tid == 0) {
        ptx::mbar_init(&sm->done, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc(&sm->tmem_base, 256);
        ptx::tmem_relinquish();
    }
    // ---- stage A ------------------------------------------------------------------
    const int krow_bytes = K * esz;
    for (int i = tid; i < 128 * krow_bytes / 16; i += 128) {
        int r = i / (krow_bytes / 16), ch = i % (krow_bytes / 16);
        uint4 v = *reinterpret_cast<const uint4*>(a + (size_t)r * krow_bytes + ch * 16);
        uint32_t off;
        if (mode == 3) off = (uint32_t)(ch * (128 * 16) + r * 16);     // chunk-major core matrices
        else           off = kmajor_sw128_offset(r, ch * 16, 128);
        *reinterpret_cast<uint4*>(sa + off) = v;
    }
    // ---- stage B ------------------------------------------------------------------
    if (mode == 1) {
        // b is [K, N] bf16, N contiguous.  MN-major: 64-column chunk c, kv row k:
        // c*(K*128) + (k/8)*1024 + (k%8)*128 + ((j ^ (k&7))*16)
        const int nrow_bytes = N * 2;
        for (int i = tid; i < K * nrow_bytes / 16; i += 128) {
            int k = i / (nrow_bytes / 16), ch = i % (nrow_bytes / 16);
            uint4 v = *reinterpret_cast<const uint4*>(b + (size_t)k * nrow_bytes + ch * 16);
            int c = ch >> 3, j = ch & 7;
            uint32_t off = (uint32_t)(c * (K * 128) + (k >> 3) * 1024 + (k & 7) * 128 + ((j ^ (k & 7)) << 4));
            *reinterpret_cast<uint4*>(sb + off) = v;
        }
    } else {
        for (int i = tid; i < N * krow_bytes / 16; i += 128) {
            int r = i / (krow_bytes / 16), ch = i % (krow_bytes / 16);
            uint4 v = *reinterpret_cast<const uint4*>(b + (size_t)r * krow_bytes + ch * 16);
            *reinterpret_cast<uint4*>(sb + kmajor_sw128_offset(r, ch * 16, N)) = v;
        }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (tid == 0) {
        const uint32_t a_addr = ptx::smem_u32(sa), b_addr = ptx::smem_u32(sb);
        const int kstep_elems = (mode == 2) ? 32 : 16;        // 32 bytes of K per MMA
        const int nsteps = K / kstep_elems;
        uint32_t idesc;
        if (mode == 2) idesc = ptx::make_idesc(0, 0, 0, 0, 128, N);
        else           idesc = ptx::make_idesc(1, 1, 0, mode == 1 ? 1 : 0, 128, N);
        for (int s = 0; s < nsteps; s++) {
            const int kbyte = s * 32;                          // byte offset along K
            uint64_t ad, bd;
            if (mode == 3) ad = ptx::make_smem_desc(a_addr + (kbyte >> 4) * (128 * 16), 128 * 16, 128, 0);
            else ad = ptx::make_smem_desc(a_addr + (kbyte >> 7) * (128 * 128) + (kbyte & 127), 16, 1024, 2);
            if (mode == 1) bd = ptx::make_smem_desc(b_addr + s * 2048, (uint32_t)K * 128, 1024, 2);
            else bd = ptx::make_smem_desc(b_addr + (kbyte >> 7) * (N * 128) + (kbyte & 127), 16, 1024, 2);
            if (mode == 2) ptx::mma_f8(tmem, ad, bd, idesc, s > 0);
            else           ptx::mma_f16(tmem, ad, bd, idesc, s > 0);
        }
        ptx::tc_commit(&sm->done);
    }
    bool ok = ptx::mbar_wait(&sm->done, 0, &sm->abort_flag);
    ptx::tc_fence_after();
    if (ok) {
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        for (int c0 = 0; c0 < N; c0 += 32) {
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem + lane_addr + c0, r);
            ptx::tc_wait_ld();
            for (int i = 0; i < 32; i++)
                if (c0 + i < N) d[(size_t)tid * N + c0 + i] = __uint_as_float(r[i]);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, 256);
    if (tid == 0 && sm->abort_flag) atomicExch(status, B200_TIMEOUT);
}

}  // namespace

extern "C" int b200_umma_selftest(int mode, const void* a, const void* b, float* d, int N, int K,
                                  b200_stream_t stream) {
    if (!a || !b || !d) return B200_BAD_ARG;
    if (mode < 0 || mode > 3) return B200_BAD_ARG;
    const int esz = (mode == 2) ? 1 : 2;
    if (N < 16 || N > 256 || N % 16) return B200_BAD_SHAPE;
    if (mode == 1 && N % 64) return B200_BAD_SHAPE;
    if (K <= 0 || (K * esz) % 128) return B200_BAD_SHAPE;
    b200_ws* ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    size_t smem = 1024 + (((size_t)128 * K * esz + 1023) & ~size_t(1023)) + (((size_t)N * K * esz + 1023) & ~size_t(1023)) +
                  sizeof(SelfSmem) + 64;
    if (smem > ws->max_smem_optin) return B200_UNSUPPORTED;
    B200_CUDA_TRY(cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    umma_selftest_kernel<<<1, 128, smem, stream>>>(mode, static_cast<const uint8_t*>(a),
                                                   static_cast<const uint8_t*>(b), d, N, K, ws->d_status);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// -------------------------------------------------------------------------------------------------
// Tensor-pipe rate of the FP8 MMA the grouped GEMMs use (kind::f8f6f4, e4m3, fp32 accumulate), measured
// with nothing else going on: every CTA (one per SM) keeps one operand stage in shared memory and one
// thread issues `iters` K blocks of four K = 32 MMAs, alternating between two TMEM accumulator stages.
//   pair = 0   cta_group::1, M = 128, N = 256 (A 16 KB + B 32 KB per K block read from shared memory)
//   pair = 1   cta_group::2, M = 256, N = 256: each CTA of a pair supplies its 128 rows of A and half
//              of B (16 KB + 16 KB per K block per SM)
// The operands are whatever the shared memory holds (the rate does not depend on the values).
// -------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ void mma2_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

template <int PAIR>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int iters, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    SelfSmem* sm = reinterpret_cast<SelfSmem*>(base + 49152);
    const int tid = threadIdx.x, warp = tid >> 5;
    uint32_t rank = 0;
    if (PAIR) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    for (int i = tid; i < 49152 / 16; i += 128) reinterpret_cast<uint4*>(base)[i] = make_uint4(0x38383838u, 0x38383838u, 0x38383838u, 0x38383838u);
    if (tid == 0) {
        ptx::mbar_init(&sm->done, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(&sm->tmem_base)), "r"(512) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            ptx::tmem_alloc(&sm->tmem_base, 512);
            ptx::tmem_relinquish();
        }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    if (tid == 0 && rank == 0) {
        const uint32_t a_addr = ptx::smem_u32(base), b_addr = a_addr + 16384;
        constexpr uint32_t idesc = ptx::make_idesc(0, 0, 0, 0, PAIR ? 256 : 128, 256);
        for (int it = 0; it < iters; it++) {
            const uint32_t d = tmem + (it & 1) * 256;
#pragma unroll
            for (int k4 = 0; k4 < 4; k4++) {
                const uint64_t ad = ptx::make_smem_desc(a_addr + k4 * 32, 16, 1024, 2);
                const uint64_t bd = ptx::make_smem_desc(b_addr + k4 * 32, 16, 1024, 2);
                if (PAIR) mma2_f8(d, ad, bd, idesc, k4 > 0);
                else      ptx::mma_f8(d, ad, bd, idesc, k4 > 0);
            }
        }
        if (PAIR) {
            // one arrival in each CTA of the pair once every MMA has retired
            asm volatile(
                "{\n\t.reg .b32 r0, r1;\n\t"
                "mapa.shared::cluster.u32 r0, %0, 0;\n\t"
                "mapa.shared::cluster.u32 r1, %0, 1;\n\t"
                "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [r0];\n\t"
                "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [r1];\n\t}"
                ::"r"(ptx::smem_u32(&sm->done)) : "memory");
        } else {
            ptx::tc_commit(&sm->done);
        }
    }
    ptx::mbar_wait(&sm->done, 0, &sm->abort_flag);
    ptx::tc_fence_after();
    ptx::tc_fence_before();
    __syncthreads();
    if (PAIR) asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 0) {
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
        else      ptx::tmem_dealloc(tmem, 512);
    }
    if (tid == 0 && sm->abort_flag) atomicExch(status, B200_TIMEOUT);
}

}  // namespace

extern "C" int b200_fp8_mma_rate(int pair, int iters, float* tflops, float* ms_out, b200_stream_t stream) {
    if (!tflops || iters <= 0 || iters > (1 << 22)) return B200_BAD_ARG;
    b200_ws* ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    const size_t smem = 1024 + 49152 + sizeof(SelfSmem) + 64;
    cudaEvent_t e0, e1;
    B200_CUDA_TRY(cudaEventCreate(&e0));
    B200_CUDA_TRY(cudaEventCreate(&e1));
    const int grid = pair ? (ws->sm_count / 2) * 2 : ws->sm_count;
    float ms = 0.f;
    for (int rep = 0; rep < 2; rep++) {        // the first launch warms up
        B200_CUDA_TRY(cudaEventRecord(e0, stream));
        if (pair) {
            B200_CUDA_TRY(cudaFuncSetAttribute(mma_rate_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(grid); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr; cfg.numAttrs = 1;
            B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, mma_rate_kernel<1>, iters, ws->d_status));
        } else {
            B200_CUDA_TRY(cudaFuncSetAttribute(mma_rate_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            mma_rate_kernel<0><<<grid, 128, smem, stream>>>(iters, ws->d_status);
        }
        b200_count_launch(1);
        B200_CUDA_TRY(cudaGetLastError());
        B200_CUDA_TRY(cudaEventRecord(e1, stream));
        B200_CUDA_TRY(cudaEventSynchronize(e1));
        B200_CUDA_TRY(cudaEventElapsedTime(&ms, e0, e1));
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    // per CTA and K block: 4 MMAs of 128 (rows of this CTA) x 256 x 32
    const double flops = (double)grid * iters * 4.0 * 2.0 * 128 * 256 * 32;
    *tflops = (float)(flops / (ms * 1e-3) / 1e12);
    if (ms_out) *ms_out = ms;
    return B200_OK;
}
