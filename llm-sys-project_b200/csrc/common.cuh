// Shared host/device helpers for the sm_100a MoE / DSA library: status codes,
// the per-device scratch workspace, and thin inline-PTX wrappers (mbarrier,
// TMA, tcgen05/TMEM).  Every device-side wait is bounded: when a wait runs out
// the kernel records B200_TIMEOUT in the workspace status word and winds down
// instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_moe_dsa.h"

#define B200_CUDA_TRY(expr)                                      \
    do {                                                         \
        cudaError_t _e = (expr);                                 \
        if (_e != cudaSuccess) {                                 \
            b200_set_last_cuda_error(_e, __FILE__, __LINE__);    \
            return B200_CUDA_ERROR;                              \
        }                                                        \
    } while (0)

void b200_set_last_cuda_error(cudaError_t e, const char* file, int line);
void b200_count_launch(int n);

// ---------------------------------------------------------------------------
// Workspace: one grow-only device buffer + a device status word.  A call
// carves what it needs from the start of the buffer, so a workspace serves one
// in-flight call at a time (calls on one stream are naturally ordered).
// ---------------------------------------------------------------------------
struct b200_gemm_profile;    // per-workspace event record of the grouped GEMMs (moe_fp8.cu)

struct b200_ws {
    int device = -1;
    char* base = nullptr;
    size_t capacity = 0;
    int* d_status = nullptr;   // device word: 0 = ok, otherwise a B200_* code
    int sm_count = 0;
    size_t max_smem_optin = 0;
    b200_gemm_profile* gemm_prof = nullptr;
    const int* route_flag_n = nullptr;    // device counter of the last tensor-core routing call (NULL: exact path)
};

b200_ws* b200_default_ws();                        // lazily created, one per device
int b200_ws_ensure(b200_ws* ws, size_t bytes);     // grows (cudaMalloc) when too small

struct WsCarver {
    char* p;
    size_t off = 0;
    explicit WsCarver(char* base) : p(base) {}
    template <typename T>
    T* take(size_t n) {
        off = (off + 255) & ~size_t(255);
        T* r = reinterpret_cast<T*>(p ? p + off : nullptr);
        off += n * sizeof(T);
        return r;
    }
    size_t total() const { return (off + 255) & ~size_t(255); }
};

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

#ifdef __CUDACC__
// ---------------------------------------------------------------------------
// Device-side PTX wrappers
// ---------------------------------------------------------------------------
// Function attributes (dynamic shared-memory limits) belong to a device: a process that drives several
// GPUs has to set them once per device, not once per process.  Returns true the first time it is called
// for the current device with a given flag array (64 entries, zero-initialised static storage).
static inline bool b200_first_call_on_device(bool* done_by_device) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
    if (done_by_device[dev]) return false;
    done_by_device[dev] = true;
    return true;
}

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  `abort_flag` is a CTA-shared word any role sets when it gives
// up; every other waiter then leaves too.  Returns false on give-up.
#ifndef B200_WAIT_LIMIT_NS
#define B200_WAIT_LIMIT_NS 2000000000ull   // 2 s
#endif
// Bounded wait.  The clock is not read on the way in: reading %globaltimer takes hundreds of cycles when
// several warps of a scheduler do it at once, and a waiter that is busy reading it notices a completed
// phase that much later.  The deadline starts at the first clock reading (every 1024 failed polls).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t it = 0;
    while (!mbar_try_wait(bar, parity)) {
        if (((++it) & 1023u) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = globaltimer_ns();
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

// Same, for a waiter that can afford to react late (a producer several stages ahead): it sleeps between
// polls so that its polling does not take issue slots from the warps that share its scheduler.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned sleep_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    uint64_t t0 = 0;
    uint32_t it = 0;
    while (!mbar_try_wait(bar, parity)) {
        __nanosleep(sleep_ns);
        if (((++it) & 255u) == 0) {
            if (*abort_flag) return false;
            const uint64_t now = globaltimer_ns();
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

// ---- proxies / fences -------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA (tiled, 2-D; each CTA fetches its own tile) ---------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- cp.async (16-byte, L2 only) ----------------------------------------------
__device__ __forceinline__ void cp_async_16(uint32_t smem_addr, const void* gptr) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
// The mbarrier receives one arrival (counted against its initial count) once all cp.async
// operations this thread has issued so far have completed; the thread itself does not wait.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05 / TMEM -------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {   // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {      // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Commit: the mbarrier gets one arrival when every MMA issued so far by this
// thread has finished (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Block-scaled FP8 MMA (kind::mxf8f6f4): D (+)= (A * SFA) * (B * SFB)^T over K = 32, one UE8M0 scale (2^(byte-127))
// per row of A and per row of B.  The scales live in TMEM: a 32-bit column holds the scale bytes of four
// consecutive K = 32 steps, byte `sf_id` of the instruction descriptor picks the step; rows r of a 128-row
// operand sit on lane r % 32 of column r / 32 (same data in all four lane quadrants).
__device__ __forceinline__ void mma_mxf8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// Power-of-two block scale: the smallest power of two >= amax / 448 (at least 2^-126, at most 2^127; 1 for an
// all-zero block).  Bit arithmetic on the correctly rounded quotient, so that host and device agree exactly.
__host__ __device__ inline float pow2_scale_bits(float quotient) {
    union { float f; uint32_t u; } c;
    c.f = quotient;
    uint32_t e = (c.u >> 23) & 0xFFu;
    if (e == 0) e = 1;
    else if (c.u & 0x7FFFFFu) e += 1;
    if (e > 254) e = 254;
    c.u = e << 23;
    return c.f;
}
// Instruction descriptor of the block-scaled MMA: e4m3 x e4m3, both K-major, UE8M0 scales, fp32 accumulate.
__host__ __device__ constexpr uint32_t make_idesc_mx(uint32_t M, uint32_t N, uint32_t a_sf_id, uint32_t b_sf_id) {
    return (b_sf_id << 4) | ((N >> 3) << 17) | (1u << 23) | ((M >> 4) << 24) | (a_sf_id << 29);
}
// Shared memory -> TMEM: 32 rows x 16 bytes (four core matrices of 8 rows, 128 bytes apart) into 32 lanes x 4
// columns, replicated into all four lane quadrants.  The layout the scale factors of a 128-row operand use.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading /
// stride byte offsets (all >> 4), version 1 at bit 46, swizzle mode at bits 61-63
// (0 none, 2 = 128-byte, 4 = 64-byte, 6 = 32-byte).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_mode) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(swizzle_mode & 7) << 61;
    return d;
}

// Instruction descriptor for kind::f16 / kind::f8f6f4, fp32 accumulate.
// fmt: kind::f16 -> 0 f16, 1 bf16; kind::f8f6f4 -> 0 e4m3, 1 e5m2.
// major: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t a_major,
                                                  uint32_t b_major, uint32_t M, uint32_t N) {
    return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_major << 15) | (b_major << 16) | ((N >> 3) << 17) |
           ((M >> 4) << 24);
}

// TMEM -> registers: 32 lanes x 32 consecutive 32-bit columns (lane = thread).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}


// TMEM -> registers: 32 lanes x 64 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr)
        : "memory");
}

// TMEM -> registers: 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// TMEM -> registers: 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
        : "r"(taddr)
        : "memory");
}

// Two IEEE fp32 fused multiply-adds in one issue slot (same bits as two scalar fmaf).
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b,
                                                        unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// Warpgroup-wide register budget changes (all four warps of the warpgroup execute it).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }

}  // namespace ptx
#endif  // __CUDACC__
