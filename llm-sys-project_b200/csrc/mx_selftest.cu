// Self check of the block-scaled FP8 MMA (tcgen05.mma kind::mxf8f6f4.block_scale, UE8M0 scales): one CTA computes
//     D[m, n] = sum_k  A[m, k] * 2^(sfa[m, k/32] - 127)  *  B[n, k] * 2^(sfb[n, k/32] - 127)
// for a 128 x N x K problem with the operand tiles, scale-factor layout, shared-memory -> TMEM scale copies and
// descriptors the power-of-two-scale grouped GEMM uses, so that a mistake in any of them shows up as a wrong number
// in a small matrix.
#include "common.cuh"
#include "selftest.h"

namespace {

struct MxSmem {
    uint64_t done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint32_t kmajor_sw128_off(int r, int kbyte, int rows) {
    int blk = kbyte >> 7, j = (kbyte >> 4) & 7, w = kbyte & 15;
    return (uint32_t)(blk * rows * 128 + r * 128 + ((j ^ (r & 7)) << 4) + w);
}
// byte offset of (row r, K = 32 step j) inside the 512-byte scale atom of 128 rows x 4 steps
__device__ __forceinline__ uint32_t sf_atom_off(int r, int j) { return (uint32_t)((r & 31) * 16 + (r >> 5) * 4 + j); }

__global__ void __launch_bounds__(128, 1)
mx_selftest_kernel(const uint8_t* __restrict__ a, const uint8_t* __restrict__ b, const uint8_t* __restrict__ sfa,
                   const uint8_t* __restrict__ sfb, float* __restrict__ d, int N, int K, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int nkb = K / 128, natom_b = N / 128;
    uint8_t* sa = base;
    uint8_t* sb = sa + 128 * K;
    uint8_t* ssfa = sb + N * K;                       // nkb atoms of 512 bytes
    uint8_t* ssfb = ssfa + nkb * 512;                 // nkb * natom_b atoms
    MxSmem* sm = reinterpret_cast<MxSmem*>(ssfb + nkb * natom_b * 512);
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        ptx::mbar_init(&sm->done, 1);
        sm->abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc(&sm->tmem_base, 512);
        ptx::tmem_relinquish();
    }
    for (int i = tid; i < 128 * K / 16; i += 128) {
        int r = i / (K / 16), ch = i % (K / 16);
        *reinterpret_cast<uint4*>(sa + kmajor_sw128_off(r, ch * 16, 128)) = *reinterpret_cast<const uint4*>(a + (size_t)r * K + ch * 16);
    }
    for (int i = tid; i < N * K / 16; i += 128) {
        int r = i / (K / 16), ch = i % (K / 16);
        *reinterpret_cast<uint4*>(sb + kmajor_sw128_off(r, ch * 16, N)) = *reinterpret_cast<const uint4*>(b + (size_t)r * K + ch * 16);
    }
    const int nsf = K / 32;
    for (int i = tid; i < 128 * nsf; i += 128) {
        int r = i / nsf, s = i % nsf;
        ssfa[(s >> 2) * 512 + sf_atom_off(r, s & 3)] = sfa[(size_t)r * nsf + s];
    }
    for (int i = tid; i < N * nsf; i += 128) {
        int n = i / nsf, s = i % nsf;
        ssfb[((s >> 2) * natom_b + (n >> 7)) * 512 + sf_atom_off(n & 127, s & 3)] = sfb[(size_t)n * nsf + s];
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = sm->tmem_base;

    if (tid == 0) {
        const uint32_t a_addr = ptx::smem_u32(sa), b_addr = ptx::smem_u32(sb);
        const int sf_cols = 4 + 4 * natom_b;          // TMEM columns of one 128-deep block's scales
        for (int kb = 0; kb < nkb; kb++) {
            const uint32_t tsfa = tmem + 256 + kb * sf_cols, tsfb = tsfa + 4;
            ptx::tmem_cp_32x128b_warpx4(tsfa, ptx::make_smem_desc(ptx::smem_u32(ssfa + kb * 512), 16, 128, 0));
            for (int at = 0; at < natom_b; at++)
                ptx::tmem_cp_32x128b_warpx4(tsfb + 4 * at,
                                            ptx::make_smem_desc(ptx::smem_u32(ssfb + (kb * natom_b + at) * 512), 16, 128, 0));
            for (int j = 0; j < 4; j++) {
                const int kbyte = kb * 128 + j * 32;
                const uint64_t ad = ptx::make_smem_desc(a_addr + (kbyte >> 7) * (128 * 128) + (kbyte & 127), 16, 1024, 2);
                const uint64_t bd = ptx::make_smem_desc(b_addr + (kbyte >> 7) * (N * 128) + (kbyte & 127), 16, 1024, 2);
                ptx::mma_mxf8(tmem, ad, bd, ptx::make_idesc_mx(128, N, j, j), tsfa, tsfb, (kb > 0 || j > 0) ? 1u : 0u);
            }
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
            for (int i = 0; i < 32; i++) d[(size_t)tid * N + c0 + i] = __uint_as_float(r[i]);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, 512);
    if (tid == 0 && sm->abort_flag) atomicExch(status, B200_TIMEOUT);
}

}  // namespace

extern "C" int b200_mx_selftest(const void* a, const void* b, const void* sfa, const void* sfb, float* d, int N, int K,
                                b200_stream_t stream) {
    if (!a || !b || !sfa || !sfb || !d) return B200_BAD_ARG;
    if ((N != 128 && N != 256) || K <= 0 || K % 128 || K > 512) return B200_BAD_SHAPE;
    b200_ws* ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    const size_t smem = 1024 + (size_t)128 * K + (size_t)N * K + (size_t)(K / 128) * 512 * (1 + N / 128) + sizeof(MxSmem) + 64;
    if (smem > ws->max_smem_optin) return B200_UNSUPPORTED;
    B200_CUDA_TRY(cudaFuncSetAttribute(mx_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    mx_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(a), static_cast<const uint8_t*>(b), static_cast<const uint8_t*>(sfa),
        static_cast<const uint8_t*>(sfb), d, N, K, ws->d_status);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
