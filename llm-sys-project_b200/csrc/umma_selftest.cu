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
