// Test hook for the bounded device-side waits (the reference's only failure behaviour is to print
// and exit(1), utils/cuda_utils.cuh:13-21; here a wait that runs out becomes a status code).
// This translation unit is compiled with a 2 ms wait limit instead of the production 2 s, so that a
// test can let a wait run out: the kernel below waits on an mbarrier nobody arrives at, both kinds of
// waiter give up, and the block reports B200_TIMEOUT exactly as the production kernels do.
#define B200_WAIT_LIMIT_NS 2000000ull
#include "common.cuh"
#include "selftest.h"

namespace {

__global__ void __launch_bounds__(64) wait_selftest_kernel(int* status, long long* elapsed_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_flag = 0;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
        const uint64_t t0 = ptx::globaltimer_ns();
        bool ok;
        if (warp == 0) ok = ptx::mbar_wait(&bar, 0, &abort_flag);                  // spinning waiter
        else           ok = ptx::mbar_wait_relaxed(&bar, 0, &abort_flag, 200);     // sleeping waiter
        const uint64_t t1 = ptx::globaltimer_ns();
        if (elapsed_ns) elapsed_ns[warp] = ok ? -1 : (long long)(t1 - t0);
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicExch(status, B200_TIMEOUT);
}

}  // namespace

extern "C" int b200_wait_selftest(b200_ws* ws, long long* elapsed_ns, b200_stream_t stream) {
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    wait_selftest_kernel<<<1, 64, 0, stream>>>(ws->d_status, elapsed_ns);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}
