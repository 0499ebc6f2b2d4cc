// Library runtime: status strings, last-error text, workspaces, launch counter,
// and the counter-based synthetic-input generators.
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

static thread_local char g_err[512] = "";
static thread_local long long g_launches = 0;

void b200_set_last_cuda_error(cudaError_t e, const char* file, int line) {
    snprintf(g_err, sizeof(g_err), "%s at %s:%d", cudaGetErrorString(e), file, line);
}
void b200_count_launch(int n) { g_launches += n; }
void b200_set_last_error_text(const char* text) { snprintf(g_err, sizeof(g_err), "%s", text); }

extern "C" {

const char* b200_status_string(int s) {
    switch (s) {
        case B200_OK: return "ok";
        case B200_BAD_SHAPE: return "bad shape";
        case B200_UNSUPPORTED: return "unsupported configuration";
        case B200_CUDA_ERROR: return "CUDA error";
        case B200_TIMEOUT: return "device-side wait timed out";
        case B200_NCCL_ERROR: return "NCCL error";
        case B200_BAD_ARG: return "bad argument";
        case B200_BAD_SCALE: return "a scale is not a power of two";
    }
    return "unknown status";
}
const char* b200_last_error_string(void) { return g_err; }

long long b200_launch_count(int reset) {
    long long v = g_launches;
    if (reset) g_launches = 0;
    return v;
}

int b200_ws_create(b200_ws** out) {
    if (!out) return B200_BAD_ARG;
    b200_ws* ws = new b200_ws();
    B200_CUDA_TRY(cudaGetDevice(&ws->device));
    cudaDeviceProp prop;
    B200_CUDA_TRY(cudaGetDeviceProperties(&prop, ws->device));
    ws->sm_count = prop.multiProcessorCount;
    ws->max_smem_optin = prop.sharedMemPerBlockOptin;
    B200_CUDA_TRY(cudaMalloc(&ws->d_status, 256));
    B200_CUDA_TRY(cudaMemset(ws->d_status, 0, 256));
    *out = ws;
    return B200_OK;
}

int b200_ws_destroy(b200_ws* ws) {
    if (!ws) return B200_OK;
    if (ws->base) cudaFree(ws->base);
    if (ws->d_status) cudaFree(ws->d_status);
    delete ws;
    return B200_OK;
}

int b200_ws_reserve(b200_ws* ws, size_t bytes) {
    if (!ws) ws = b200_default_ws();
    if (!ws) return B200_CUDA_ERROR;
    return b200_ws_ensure(ws, bytes);
}

size_t b200_ws_capacity(const b200_ws* ws) { return ws ? ws->capacity : 0; }

int b200_ws_device_status(b200_ws* ws, b200_stream_t stream, int* status) {
    if (!ws) ws = b200_default_ws();
    if (!ws || !status) return B200_BAD_ARG;
    B200_CUDA_TRY(cudaStreamSynchronize(stream));
    B200_CUDA_TRY(cudaMemcpy(status, ws->d_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) B200_CUDA_TRY(cudaMemset(ws->d_status, 0, sizeof(int)));
    return B200_OK;
}

}  // extern "C"

int b200_ws_ensure(b200_ws* ws, size_t bytes) {
    // growth (free + allocate) is serialised; the calls that then use the buffer still have to be
    // ordered by the caller (one in-flight call per workspace)
    static std::mutex grow_mu;
    std::lock_guard<std::mutex> lock(grow_mu);
    if (bytes <= ws->capacity) return B200_OK;
    // Grow-only.  Earlier launches may still read the old buffer: drain first.
    B200_CUDA_TRY(cudaDeviceSynchronize());
    if (ws->base) B200_CUDA_TRY(cudaFree(ws->base));
    ws->base = nullptr;
    ws->capacity = 0;
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    B200_CUDA_TRY(cudaMalloc(&ws->base, want));
    ws->capacity = want;
    return B200_OK;
}

b200_ws* b200_default_ws() {
    static std::mutex mu;
    static b200_ws* table[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!table[dev]) {
        b200_ws* ws = nullptr;
        if (b200_ws_create(&ws) != B200_OK) return nullptr;
        table[dev] = ws;
    }
    return table[dev];
}

// ---------------------------------------------------------------------------
// Synthetic inputs.  value(seed, i): two splitmix64 outputs give eight 16-bit
// uniforms; their integer sum (Irwin-Hall, n = 8) minus its mean, times one
// fp32 factor, approximates N(0, sigma).  Only integer arithmetic and a single
// fp32 multiply are involved, so the host twin produces identical bits.
// ---------------------------------------------------------------------------
__host__ __device__ inline unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__host__ __device__ inline float synth_normal(unsigned long long seed, unsigned long long i, float factor) {
    unsigned long long key = seed * 0xD1342543DE82EF95ull + i;
    unsigned long long a = splitmix64(key), b = splitmix64(key ^ 0xA5A5A5A5A5A5A5A5ull);
    int s = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        s += (int)((a >> (16 * j)) & 0xFFFF);
        s += (int)((b >> (16 * j)) & 0xFFFF);
    }
    return (float)(s - 262140) * factor;   // mean of the sum = 8 * 32767.5
}
// standard deviation of the integer sum: sqrt(8 * (65536^2 - 1) / 12)
#define SYNTH_SD 53510.03113f

__global__ void fill_normal_f32_kernel(float* dst, long long n, unsigned long long seed, float factor) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = synth_normal(seed, (unsigned long long)i, factor);
}
__global__ void fill_normal_bf16_kernel(__nv_bfloat16* dst, long long n, unsigned long long seed, float factor) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long stride = (long long)gridDim.x * blockDim.x;
    for (; i < n; i += stride) dst[i] = __float2bfloat16_rn(synth_normal(seed, (unsigned long long)i, factor));
}

template <bool POW2>
__device__ inline float block_scale_of(float amax) {
    if (!(amax > 0.0f)) return 1.0f;
    const float q = __fdiv_rn(amax, 448.0f);
    return POW2 ? ptx::pow2_scale_bits(q) : q;
}
__device__ inline uint8_t to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// One block per 128x128 weight block: generate, amax, quantise.
template <bool POW2>
__global__ void fill_normal_fp8_w128_kernel(uint8_t* q, float* scales, long long rows, int cols,
                                            unsigned long long seed, float factor) {
    __shared__ float red[32];
    int cb = cols / 128;
    long long blk = blockIdx.x;
    long long br = blk / cb;
    int bc = (int)(blk % cb);
    float vals[64];   // 256 threads x 64 values = 128 x 128
    float amax = 0.0f;
#pragma unroll 4
    for (int j = 0; j < 64; j++) {
        int e = j * 256 + threadIdx.x;
        int r = e >> 7, c = e & 127;
        long long idx = (br * 128 + r) * (long long)cols + bc * 128 + c;
        vals[j] = synth_normal(seed, (unsigned long long)idx, factor);
        amax = fmaxf(amax, fabsf(vals[j]));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int w = 1; w < 8; w++) amax = fmaxf(amax, red[w]);
    float s = block_scale_of<POW2>(amax);
    if (threadIdx.x == 0) scales[blk] = s;
#pragma unroll 4
    for (int j = 0; j < 64; j++) {
        int e = j * 256 + threadIdx.x;
        int r = e >> 7, c = e & 127;
        long long idx = (br * 128 + r) * (long long)cols + bc * 128 + c;
        q[idx] = to_e4m3(__fdiv_rn(vals[j], s));
    }
}

// Quantisers over fp32 inputs.
template <bool POW2>
__global__ void quant_act_1x128_kernel(const float* x, uint8_t* q, float* scales, long long rows, int cols) {
    // one warp per 1x128 block; lane holds 4 consecutive values
    int nb = cols / 128;
    long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    long long total = rows * nb;
    if (gw >= total) return;
    long long r = gw / nb;
    int b = (int)(gw % nb);
    const float4 v = *reinterpret_cast<const float4*>(x + r * cols + (long long)b * 128 + lane * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    float s = block_scale_of<POW2>(amax);
    if (lane == 0) scales[gw] = s;
    uchar4 o4;
    o4.x = to_e4m3(__fdiv_rn(v.x, s));
    o4.y = to_e4m3(__fdiv_rn(v.y, s));
    o4.z = to_e4m3(__fdiv_rn(v.z, s));
    o4.w = to_e4m3(__fdiv_rn(v.w, s));
    *reinterpret_cast<uchar4*>(q + r * cols + (long long)b * 128 + lane * 4) = o4;
}

template <bool POW2>
__global__ void quant_weight_128x128_kernel(const float* w, uint8_t* q, float* scales, long long rows, int cols) {
    __shared__ float red[32];
    int cb = cols / 128;
    long long blk = blockIdx.x;
    long long br = blk / cb;
    int bc = (int)(blk % cb);
    float vals[64];
    float amax = 0.0f;
#pragma unroll 4
    for (int j = 0; j < 64; j++) {
        int e = j * 256 + threadIdx.x;
        int r = e >> 7, c = e & 127;
        vals[j] = w[(br * 128 + r) * (long long)cols + bc * 128 + c];
        amax = fmaxf(amax, fabsf(vals[j]));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
    for (int wi = 1; wi < 8; wi++) amax = fmaxf(amax, red[wi]);
    float s = block_scale_of<POW2>(amax);
    if (threadIdx.x == 0) scales[blk] = s;
#pragma unroll 4
    for (int j = 0; j < 64; j++) {
        int e = j * 256 + threadIdx.x;
        int r = e >> 7, c = e & 127;
        q[(br * 128 + r) * (long long)cols + bc * 128 + c] = to_e4m3(__fdiv_rn(vals[j], s));
    }
}

static int grid_for(long long n, int block, int cap = 148 * 16) {
    long long g = (n + block - 1) / block;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

extern "C" {

int b200_fill_normal_f32(float* dst, long long n, unsigned long long seed, float sigma, b200_stream_t stream) {
    if (!dst || n < 0) return B200_BAD_ARG;
    if (n == 0) return B200_OK;
    fill_normal_f32_kernel<<<grid_for(n, 256), 256, 0, stream>>>(dst, n, seed, sigma / SYNTH_SD);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_fill_normal_bf16(uint16_t* dst, long long n, unsigned long long seed, float sigma, b200_stream_t stream) {
    if (!dst || n < 0) return B200_BAD_ARG;
    if (n == 0) return B200_OK;
    fill_normal_bf16_kernel<<<grid_for(n, 256), 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(dst), n, seed,
                                                                  sigma / SYNTH_SD);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // extern "C"
static int fill_normal_fp8_w128_impl(uint8_t* q, float* scales, long long rows, int cols, unsigned long long seed,
                                     float sigma, bool pow2, b200_stream_t stream) {
    if (!q || !scales) return B200_BAD_ARG;
    if (rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return B200_BAD_SHAPE;
    long long blocks = (rows / 128) * (cols / 128);
    if (blocks > 0x7fffffffLL) return B200_BAD_SHAPE;
    if (pow2) fill_normal_fp8_w128_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(q, scales, rows, cols, seed, sigma / SYNTH_SD);
    else      fill_normal_fp8_w128_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(q, scales, rows, cols, seed, sigma / SYNTH_SD);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

static int quant_act_1x128_impl(const float* x, uint8_t* q, float* scales, long long rows, int cols, bool pow2,
                               b200_stream_t stream) {
    if (!x || !q || !scales) return B200_BAD_ARG;
    if (rows < 0 || cols <= 0 || cols % 128) return B200_BAD_SHAPE;
    if (rows == 0) return B200_OK;
    long long warps = rows * (cols / 128);
    long long blocks = (warps + 7) / 8;
    if (blocks > 0x7fffffffLL) return B200_BAD_SHAPE;
    if (pow2) quant_act_1x128_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(x, q, scales, rows, cols);
    else      quant_act_1x128_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(x, q, scales, rows, cols);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

static int quant_weight_128x128_impl(const float* w, uint8_t* q, float* scales, long long rows, int cols, bool pow2,
                                    b200_stream_t stream) {
    if (!w || !q || !scales) return B200_BAD_ARG;
    if (rows <= 0 || cols <= 0 || rows % 128 || cols % 128) return B200_BAD_SHAPE;
    long long blocks = (rows / 128) * (cols / 128);
    if (blocks > 0x7fffffffLL) return B200_BAD_SHAPE;
    if (pow2) quant_weight_128x128_kernel<true><<<(unsigned)blocks, 256, 0, stream>>>(w, q, scales, rows, cols);
    else      quant_weight_128x128_kernel<false><<<(unsigned)blocks, 256, 0, stream>>>(w, q, scales, rows, cols);
    b200_count_launch(1);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

extern "C" {
int b200_fill_normal_fp8_w128(uint8_t* q, float* scales, long long rows, int cols, unsigned long long seed,
                              float sigma, b200_stream_t stream) {
    return fill_normal_fp8_w128_impl(q, scales, rows, cols, seed, sigma, false, stream);
}
int b200_fill_normal_fp8_w128_pow2(uint8_t* q, float* scales, long long rows, int cols, unsigned long long seed,
                                   float sigma, b200_stream_t stream) {
    return fill_normal_fp8_w128_impl(q, scales, rows, cols, seed, sigma, true, stream);
}
int b200_quant_act_1x128(const float* x, uint8_t* q, float* scales, long long rows, int cols, b200_stream_t stream) {
    return quant_act_1x128_impl(x, q, scales, rows, cols, false, stream);
}
int b200_quant_act_1x128_pow2(const float* x, uint8_t* q, float* scales, long long rows, int cols, b200_stream_t stream) {
    return quant_act_1x128_impl(x, q, scales, rows, cols, true, stream);
}
int b200_quant_weight_128x128(const float* w, uint8_t* q, float* scales, long long rows, int cols,
                              b200_stream_t stream) {
    return quant_weight_128x128_impl(w, q, scales, rows, cols, false, stream);
}
int b200_quant_weight_128x128_pow2(const float* w, uint8_t* q, float* scales, long long rows, int cols,
                                   b200_stream_t stream) {
    return quant_weight_128x128_impl(w, q, scales, rows, cols, true, stream);
}

}  // extern "C"
