/*
 * C ABI of the sm_100a (B200) MoE-layer and DSA/MLA sparse-decode library.
 *
 * Every entry point returns a status code (0 = ok), takes plain device
 * pointers and sizes, works asynchronously on the given CUDA stream and does
 * no host synchronisation.  Scratch memory comes from a workspace handle
 * (NULL selects a lazily created per-device default workspace).  A workspace
 * serves one call at a time: calls that share a workspace (ws = NULL included, and
 * the C++ functions with the reference's names, which use the default workspace)
 * must be ordered by one stream or by events; concurrent streams or host threads
 * need a workspace each (b200_ws_create).  The reference allocates its scratch
 * inside every call (kernels/moe/naive_moe.cu:408-420), so two streams that were
 * independent there share scratch here unless they bring their own workspace.
 *
 * The comment above each declaration names the reference interface it stands
 * in for (file:line in arun-reddy-a/llm-sys-project).
 */
#ifndef B200_MOE_DSA_H
#define B200_MOE_DSA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

typedef struct CUstream_st* b200_stream_t; /* == cudaStream_t */
typedef struct b200_ws b200_ws;

enum b200_status {
    B200_OK = 0,
    B200_BAD_SHAPE = 1,   /* a dimension is zero/negative or breaks a divisibility rule */
    B200_UNSUPPORTED = 2, /* valid request this build has no kernel for */
    B200_CUDA_ERROR = 3,  /* a CUDA runtime/driver call failed; see b200_last_error_string */
    B200_TIMEOUT = 4,     /* a bounded device-side wait ran out (read back by b200_ws_device_status) */
    B200_NCCL_ERROR = 5,
    B200_BAD_ARG = 6,     /* null pointer / misaligned pointer */
    B200_BAD_SCALE = 7    /* B200_MOE_POW2_SCALES: a scale that is not a power of two was met on the device
                           * (read back by b200_ws_device_status; the output is then wrong) */
};

/* kernels/moe/naive_moe.cuh:9-15 (struct MoeConfig) — same five ints, same order. */
typedef struct b200_moe_config {
    int num_tokens;       /* T */
    int num_experts;      /* E */
    int top_k;            /* K */
    int hidden_dim;       /* D */
    int intermediate_dim; /* I */
} b200_moe_config;

/* kernels/dsa/naive_dsa.cuh:9-17 (struct DsaConfig) — same seven ints, same order.
 * The cache is flat [N, D*] and indices are flat physical token ids.  The reference carries page_size and
 * total_kv_tokens without reading them; here total_kv_tokens, when positive, bounds the indices: an index
 * that is negative or not below it is an empty entry that contributes nothing (the reference would read out
 * of bounds).  page_size is used by b200_dsa_forward_bf16_paged only. */
typedef struct b200_dsa_config {
    int num_queries;         /* Q */
    int num_heads;           /* H */
    int head_dim_compressed; /* Dc */
    int head_dim_positional; /* Dp */
    int num_selected_kv;     /* S */
    int page_size;           /* P */
    int total_kv_tokens;     /* N */
} b200_dsa_config;

/* Routing modes of the FP8 layer. */
enum b200_scoring {
    B200_SCORE_SOFTMAX = 0,        /* the reference's gate: softmax over all E, top-K, renormalise */
    B200_SCORE_SIGMOID_GROUPED = 1 /* sigmoid + per-expert bias, group-limited top-K, routed scaling */
};

/* Extended configuration of the FP8 block-scale layer (no reference counterpart;
 * extends MoeConfig, kernels/moe/naive_moe.cuh:9-15). */
typedef struct b200_moe_fp8_config {
    int num_tokens, num_experts, top_k, hidden_dim, intermediate_dim;
    int scoring;        /* enum b200_scoring */
    int n_group;        /* expert groups (E % n_group == 0); 1 = ungrouped */
    int topk_group;     /* groups kept per token */
    float routed_scale; /* factor applied to the normalised weights */
    int flags;          /* bit set of enum b200_moe_flags; 0 = defaults */
} b200_moe_fp8_config;

enum b200_moe_flags {
    /* Sum a token's K expert contributions in ascending expert order with plain fp32 adds (the order of
     * the reference's host loop, kernels/moe/naive_moe.cu:424, and of its CPU code, tests/test_moe.cu:74):
     * GEMM2 writes one weighted row per (token, expert) and a second kernel reduces them, so the output is
     * bit-reproducible from run to run.  Costs T*K*D*4 bytes of workspace and one more pass over them.
     * Without the flag GEMM2 scatter-adds into the output (order varies, results agree to fp32 rounding). */
    B200_MOE_DETERMINISTIC = 1,
    /* Tile shape of the grouped GEMMs: 128-row tiles on single CTAs (the default, and the faster one at every
     * shape measured so far) or 256-row tiles on CTA pairs (tcgen05 cta_group::2; each SM stages half of a
     * weight tile).  Results agree up to the order of the scatter-add. */
    B200_MOE_SINGLE_CTA_TILES = 4,
    B200_MOE_CTA_PAIR_TILES = 8,
    /* Router logits of grouped sigmoid routing.  By default batches of 256 or more tokens (E <= 256, no logits
     * requested) compute them on the tensor cores (tf32 split operands, accumulation chains of 512 d: within
     * about 2e-5 of the fixed-order chains at unit logit scale) and accept a token's routing only when all its
     * decision margins exceed what an error of 2^-14 per unit of the token's logit rms could close; the other
     * tokens (about 2 %) are recomputed with the fixed-order FMA chains.  The expert ids of every token are the
     * ones exact logits give; the weights of accepted tokens agree with the exact ones to ~1e-6.  This flag
     * forces the exact chains for all tokens (as does a non-NULL logits_out of b200_moe_route_fp8). */
    B200_MOE_EXACT_ROUTER_LOGITS = 16,
    /* Every scale (activations, weights) is a power of two, as the *_pow2 quantisers below produce them (the
     * UE8M0 scale format of DeepSeek-V3.1-style checkpoints).  The grouped GEMMs then run on the hardware
     * block-scaled MMA (tcgen05.mma kind::mxf8f6f4.block_scale): the scales are applied inside the tensor core,
     * the accumulator stays in TMEM for the whole K loop and the software promotion per 128-deep K block
     * disappears.  The requantisation between the two GEMMs also takes power-of-two scales.  Same tolerance as the
     * default path against the fp32 emulation with the same scale rule.  Also accepted in b200_ep_config.flags. */
    B200_MOE_POW2_SCALES = 32
};

/* --------------------------------------------------------------------------- */
/* Library / workspace                                                         */
/* --------------------------------------------------------------------------- */
B200_API const char* b200_status_string(int status);
B200_API const char* b200_last_error_string(void); /* text of the last CUDA error seen by this thread */
B200_API int b200_ws_create(b200_ws** ws);          /* on the current device */
B200_API int b200_ws_destroy(b200_ws* ws);
B200_API int b200_ws_reserve(b200_ws* ws, size_t bytes); /* pre-size so timed calls never allocate */
B200_API size_t b200_ws_capacity(const b200_ws* ws);
/* Synchronises `stream`, then reads and clears the device status word. */
B200_API int b200_ws_device_status(b200_ws* ws, b200_stream_t stream, int* status);
/* Number of kernels this library has launched on the calling thread since the last reset. */
B200_API long long b200_launch_count(int reset);

/* --------------------------------------------------------------------------- */
/* MoE layer, fp32 (the reference's data types)                                 */
/* --------------------------------------------------------------------------- */
/* kernels/moe/naive_moe.cuh:73-75 / naive_moe.cu:400-471 (moe_forward): whole layer,
 * output [T,D] is overwritten. */
B200_API int b200_moe_forward_f32(b200_ws* ws, const float* x, const float* gate_w, const float* w1,
                                  const float* w2, float* out, const b200_moe_config* cfg, b200_stream_t stream);
/* naive_moe.cuh:27-29 / naive_moe.cu:341-355 (moe_gate): ids/weights [T,K] in the
 * reference's replacement-slot order; ties keep the lowest expert id. */
B200_API int b200_moe_gate_f32(b200_ws* ws, const float* x, const float* gate_w, int* expert_ids,
                               float* expert_w, const b200_moe_config* cfg, b200_stream_t stream);
/* Replaces the E serial gather scans (naive_moe.cu:147-166, :424-429) by one stable
 * counting pass: counts[E], offsets[E+1] (exclusive prefix sum), row_pair[T*K] where
 * row_pair[r] = t*K+k of the pair in sorted row r (experts ascending, tokens ascending). */
B200_API int b200_moe_permute(b200_ws* ws, const int* expert_ids, int T, int K, int E, int* counts,
                              int* offsets, int* row_pair, b200_stream_t stream);
/* naive_moe.cuh:38-41 / naive_moe.cu:357-366 (moe_gather), one expert. */
B200_API int b200_moe_gather_f32(const float* x, const int* expert_ids, int expert_id, float* gathered,
                                 int* token_map, int* count, const b200_moe_config* cfg, b200_stream_t stream);
/* naive_moe.cuh:44-45 (naive_gemm): C[M,N] = A[M,K] * B[K,N], row-major. */
B200_API int b200_gemm_f32(const float* A, const float* B, float* C, int M, int N, int K, b200_stream_t stream);
/* naive_moe.cuh:50-51 (swiglu): out[i] = silu(gate[i]) * up[i]. */
B200_API int b200_swiglu_f32(const float* gate, const float* up, float* out, int n, b200_stream_t stream);
/* naive_moe.cuh:59-62 / naive_moe.cu:384-395 (moe_scatter): out[token_map[i],:] += w * expert_out[i,:].
 * Unlike the reference (one thread per column, D <= 1024) any D is accepted. */
B200_API int b200_moe_scatter_f32(const float* expert_out, const int* token_map, const float* expert_w,
                                  const int* expert_ids, int expert_id, float* out, int count,
                                  const b200_moe_config* cfg, b200_stream_t stream);

/* --------------------------------------------------------------------------- */
/* MoE layer, FP8 e4m3 block-scale (no reference counterpart; extends           */
/* moe_forward, naive_moe.cu:400-471, to the DeepSeek-V3 data types)            */
/* --------------------------------------------------------------------------- */
/* Quantisers: scale = amax/448 (1 for an all-zero block), q = e4m3_rn_sat(x/scale).
 * Activations: 1x128 blocks, scales [rows, cols/128].  Weights: 128x128 blocks,
 * scales [rows/128, cols/128] (stack experts along rows). */
B200_API int b200_quant_act_1x128(const float* x, uint8_t* q, float* scales, long long rows, int cols,
                                  b200_stream_t stream);
B200_API int b200_quant_weight_128x128(const float* w, uint8_t* q, float* scales, long long rows, int cols,
                                       b200_stream_t stream);
/* The same quantisers with power-of-two scales: scale = the smallest power of two >= amax/448 (at least 2^-126;
 * 1 for an all-zero block), still stored as fp32.  For B200_MOE_POW2_SCALES. */
B200_API int b200_quant_act_1x128_pow2(const float* x, uint8_t* q, float* scales, long long rows, int cols,
                                       b200_stream_t stream);
B200_API int b200_quant_weight_128x128_pow2(const float* w, uint8_t* q, float* scales, long long rows, int cols,
                                            b200_stream_t stream);
/* Router on the dequantised FP8 activations: logits (fp32 fma chain over d), then
 * softmax / top-K as moe_gate, or sigmoid + bias + group-limited top-K.  Also fills
 * counts[E] (tokens per expert; may be NULL). bias may be NULL. logits_out may be NULL. */
B200_API int b200_moe_route_fp8(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w,
                                const float* bias, int* expert_ids, float* expert_w, int* counts,
                                float* logits_out, const b200_moe_fp8_config* cfg, b200_stream_t stream);
/* Whole layer: route, permute, grouped GEMM1 (+SwiGLU +requantise), grouped GEMM2
 * (+router weight +scatter-add).  xq [T,D] e4m3, xs [T,D/128]; w1q [E,2I,D] with
 * scales [E,2I/128,D/128] (rows [0,I) gate, [I,2I) up, naive_moe.cuh:71); w2q [E,D,I]
 * with scales [E,D/128,I/128]; out [T,D] fp32, overwritten.  D % 128 == 0, I % 128 == 0. */
B200_API int b200_moe_fp8_forward(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w,
                                  const float* bias, const uint8_t* w1q, const float* w1s, const uint8_t* w2q,
                                  const float* w2s, float* out, const b200_moe_fp8_config* cfg,
                                  b200_stream_t stream);
/* Same with the routing given (ids/weights [T,K]); ids outside [0,E) are skipped.
 * This is the expert-parallel building block: E counts the local experts. */
B200_API int b200_moe_fp8_experts(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                  const float* expert_w, const uint8_t* w1q, const float* w1s,
                                  const uint8_t* w2q, const float* w2s, float* out,
                                  const b200_moe_fp8_config* cfg, b200_stream_t stream);
/* Weight pre-tiling for the grouped GEMMs (no reference counterpart).  DRAM delivers random 128-byte
 * pieces at well under half the rate of 1 KB+ contiguous pieces, and a row-major weight tile is made of
 * 128-byte pieces 7 KB apart; the packed form stores each (expert, n tile, K block) tile as one
 * contiguous 32 KB block of 256 rows x 128 bytes.  which = 1: w1q [E,2I,D], tile rows for j0 = 128 * n tile:
 * gate j0..+63, up j0..+63, gate j0+64..+127, up j0+64..+127 (gate row j = w1 row j, up row j = w1 row
 * I + j); which = 2: w2q [E,D,I], tile rows = w2 rows 256 * n tile .. +255; packed has the same size.
 * Scales are unchanged.  The *_packed entry points take packed weights and are otherwise identical to
 * b200_moe_fp8_forward / b200_moe_fp8_experts. */
B200_API int b200_moe_fp8_pack_weights(int which, const uint8_t* src, uint8_t* packed, int E, int D, int I,
                                       b200_stream_t stream);
B200_API int b200_moe_fp8_forward_packed(b200_ws* ws, const uint8_t* xq, const float* xs, const float* gate_w,
                                         const float* bias, const uint8_t* w1p, const float* w1s,
                                         const uint8_t* w2p, const float* w2s, float* out,
                                         const b200_moe_fp8_config* cfg, b200_stream_t stream);
B200_API int b200_moe_fp8_experts_packed(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                         const float* expert_w, const uint8_t* w1p, const float* w1s,
                                         const uint8_t* w2p, const float* w2s, float* out,
                                         const b200_moe_fp8_config* cfg, b200_stream_t stream);
/* Stage access for parity tests: runs permute + GEMM1 and copies the requantised
 * activations of sorted rows out (act_q [rows,I], act_s [rows,I/128], rows = T*K upper bound). */
B200_API int b200_moe_fp8_gemm1_stage(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                      const uint8_t* w1q, const float* w1s, uint8_t* act_q, float* act_s,
                                      int* offsets, int* row_pair, const b200_moe_fp8_config* cfg,
                                      b200_stream_t stream);

/* Measurement aid (no reference counterpart): when enabled, CUDA events are recorded on
 * the launch stream around the two grouped GEMM kernels of every FP8 layer call that uses this
 * workspace (enabling resets the record); the read returns the mean device time of GEMM1 and
 * GEMM2 in milliseconds over the recorded calls (at most the last 256) and their number.
 * The record belongs to the workspace: host threads with their own workspaces do not share it. */
B200_API int b200_moe_fp8_profile(b200_ws* ws, int enable);
B200_API int b200_moe_fp8_profile_read(b200_ws* ws, float* gemm1_ms, float* gemm2_ms, int* calls);

/* --------------------------------------------------------------------------- */
/* DSA / MLA sparse decode                                                      */
/* --------------------------------------------------------------------------- */
/* kernels/dsa/naive_dsa.cuh:79-87 / naive_dsa.cu:435-474 (dsa_forward), fp32, one fused
 * kernel (gather + 576-dim dot + scale + online softmax + PV).  Any index order,
 * duplicates allowed; offsets are 64-bit. */
B200_API int b200_dsa_forward_f32(b200_ws* ws, const float* q_nope, const float* q_pe, const float* kc,
                                  const float* kp, const float* v, const int* idx, float* out,
                                  const b200_dsa_config* cfg, b200_stream_t stream);
/* Same layer on bf16 inputs with fp32 accumulation on the tensor cores (tcgen05/TMEM);
 * out [Q,H,Dc] fp32.  Requires H <= 128, Dc == 512, Dp == 64, S % 32 == 0 (S % 128 == 0 runs the
 * fastest kernel, S % 64 == 0 the next), 16-byte aligned pointers. */
B200_API int b200_dsa_forward_bf16(b200_ws* ws, const uint16_t* q_nope, const uint16_t* q_pe,
                                   const uint16_t* kc, const uint16_t* kp, const uint16_t* v, const int* idx,
                                   float* out, const b200_dsa_config* cfg, b200_stream_t stream);
/* Paged front end of the same decode (no reference counterpart: the reference's callers translate
 * positions themselves and pass flat ids, kernels/dsa/naive_dsa.cuh:15-16,28).  positions [Q,S] are logical
 * token positions inside the query's sequence; block_table [num_seqs, max_blocks] maps a sequence's logical
 * page (position / page_size) to a physical page of the cache (row = page * page_size + position %
 * page_size); seq_of_query [Q] names the sequence of each query (NULL: query q reads sequence q);
 * valid_len [Q] (NULL: all S) is the number of leading entries of a query's list that count.  The
 * translation runs inside the gather warps of the decode kernel.  Empty entries — beyond valid_len, a
 * negative position, a negative page, a page index >= max_blocks, a row >= total_kv_tokens — contribute
 * nothing, as if removed from the list; a query with only empty entries gets a zero row. */
B200_API int b200_dsa_forward_bf16_paged(b200_ws* ws, const uint16_t* q_nope, const uint16_t* q_pe,
                                         const uint16_t* kc, const uint16_t* kp, const uint16_t* v,
                                         const int* positions, const int* block_table, int max_blocks,
                                         const int* seq_of_query, const int* valid_len, float* out,
                                         const b200_dsa_config* cfg, b200_stream_t stream);
/* No counterpart in the reference.  Same computation and arguments as b200_dsa_forward_bf16, for
 * callers that must not allocate device memory: processes whose memory pool owns all of HBM and
 * forbids cudaMalloc after start-up, plugins that are only handed input and output buffers, and
 * latency-critical loops that cannot tolerate a workspace that grows (and synchronises the device
 * when it does).  The split-KV partial results go to a 16 MiB array built into the library (every
 * GPU that loads the library holds it until the process exits) instead of the workspace; the call
 * uses no workspace and calls no allocating routine.  The array holds the partial results of 63
 * (query, row range) pairs (257 KiB each: 128 x 512 fp32 outputs + 128 (max, sum) pairs), so a query's
 * rows are split into at most floor(63 / queries) ranges (the workspace-backed call may use more on a
 * small batch); 64 or more queries run one range each and use no scratch.  Every shape the kernel
 * supports is therefore accepted up to 65535 queries per call; more are rejected with
 * B200_UNSUPPORTED and an explanatory b200_last_error_string.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress) and sets the kernel's shared-memory limit, so make
 * that first call outside any stream capture.  All calls on a device share the one array: it keeps the
 * previous call's contents (everything read is rewritten first), and two calls that overlap on the GPU
 * (different streams) race on it.  device_status (required) is a caller-owned device int that the call
 * clears and that receives B200_TIMEOUT should a bounded device-side wait run out. */
B200_API int b200_dsa_forward_bf16_static(const uint16_t* q_nope, const uint16_t* q_pe, const uint16_t* kc,
                                          const uint16_t* kp, const uint16_t* v, const int* idx, float* out,
                                          const b200_dsa_config* cfg, int* device_status, b200_stream_t stream);
/* naive_dsa.cuh:31-37 (dsa_kv_gather) */
B200_API int b200_dsa_kv_gather_f32(const float* kc, const float* kp, const float* v, const int* idx,
                                    float* g_kc, float* g_kp, float* g_v, const b200_dsa_config* cfg,
                                    b200_stream_t stream);
/* naive_dsa.cuh:43-44, :50-51, :55-58 (dsa_dot_compressed / dsa_dot_positional / dsa_dot_fused):
 * scores[q,h,s] += dot(...) on already gathered rows; either half may be NULL. */
B200_API int b200_dsa_dot_f32(const float* q_nope, const float* q_pe, const float* g_kc, const float* g_kp,
                              float* scores, const b200_dsa_config* cfg, b200_stream_t stream);
/* naive_dsa.cuh:62 (dsa_softmax): in place over S per (q,h). */
B200_API int b200_dsa_softmax_f32(float* scores, const b200_dsa_config* cfg, b200_stream_t stream);
/* naive_dsa.cuh:68-69 (dsa_output_proj): out[q,h,d] = sum_s attn[q,h,s] * g_v[q,s,d]. */
B200_API int b200_dsa_output_proj_f32(const float* attn, const float* g_v, float* out, const b200_dsa_config* cfg,
                                      b200_stream_t stream);

/* --------------------------------------------------------------------------- */
/* Expert-parallel helpers (no reference counterpart: the reference is single-GPU). */
/* The expert-sharded layer sends every token once to each rank that owns at least  */
/* one of its selected experts and gets one partial output row back per rank.       */
/* --------------------------------------------------------------------------- */
/* Dispatch plan for `world` ranks owning experts_per_rank experts each: consecutive ones (strided = 0: expert e on
 * rank e / experts_per_rank, local id e % experts_per_rank) or every world-th one (strided = 1: expert e on rank
 * e % world, local id e / world; spreads a run of hot experts over the ranks), or any assignment given by
 * owner_map / local_map [world * experts_per_rank] (both NULL or both set; they override `strided`). From the
 * routing (ids/weights [T,K], global ids) it writes, rank-major and ascending in token inside a
 * rank: send_tok [<= world*T] token of each dispatched row; slot_ids / slot_w [<= world*T, K] the
 * row's K slots in the destination's local numbering (-1 / 0 for slots owned elsewhere);
 * send_counts [world]; pos [world, T] the dispatched row of (rank, token) or -1. */
B200_API int b200_ep_plan(const int* expert_ids, const float* expert_w, int T, int K, int experts_per_rank,
                          int world, int strided, const int* owner_map, const int* local_map, int* send_tok, int* pos, int* send_counts, int* slot_ids, float* slot_w,
                          b200_stream_t stream);
/* out[t,:] = sum over ranks r with pos[r,t] >= 0, in rank order, of back[pos[r,t],:]; out [T,D] fp32 is
 * overwritten; back holds fp32 rows or, with back_is_bf16 != 0, bf16 rows.  D % 8 == 0. */
B200_API int b200_ep_sum_rows(const void* back, int back_is_bf16, const int* pos, int world, int T, int D,
                              float* out, b200_stream_t stream);

/* Expert-parallel FP8 layer as one object per GPU (no reference counterpart: the reference is single-GPU;
 * the loop being sharded is kernels/moe/naive_moe.cu:424-469).  One host thread or process per GPU.  The
 * data plane is this library's own kernels over peer memory: every rank allocates an exchange buffer,
 * the ranks swap its 64-byte handles out of band (any transport: a file, MPI, torch.distributed) and map
 * each other's buffers; a step then runs without host synchronisation and without a collective call:
 * rows are dispatched with peer stores, owners wait (bounded) on per-source ready words, the grouped
 * GEMMs read local memory only, partial output rows go back with peer stores.  Ranks must call
 * b200_ep_forward the same number of times (a step is a collective).  A wait that runs out sets
 * B200_TIMEOUT in the status word (b200_ep_stats) and the step's output is then undefined; nothing hangs. */
typedef struct b200_ep b200_ep;
#define B200_EP_HANDLE_BYTES 64
enum b200_ep_flags {
    /* partial rows travel back as fp32 (twice the combine bytes).  Default: fp16 values relative to the row's
     * largest magnitude plus that magnitude, i.e. 11 significant bits against the row maximum */
    B200_EP_COMBINE_F32 = 2
    /* B200_MOE_EXACT_ROUTER_LOGITS and B200_MOE_POW2_SCALES (enum b200_moe_flags; their values do not collide with
     * the one above) may be set as well and mean what they mean for the single-GPU layer. */
};
typedef struct b200_ep_config {
    int rank, world;      /* this rank, number of ranks (<= 64); rank g holds num_experts / world experts */
    int max_tokens;       /* upper bound of tokens per rank and step */
    int num_experts;      /* global E */
    int top_k, hidden_dim, intermediate_dim;
    int scoring, n_group, topk_group;   /* as b200_moe_fp8_config */
    float routed_scale;
    int flags;            /* enum b200_ep_flags */
    int wait_limit_ms;    /* bound of every device-side wait for a peer; 0 = 2000 */
} b200_ep_config;
/* Allocates the buffers on the current device.  owner_map / local_map [num_experts] (host arrays, both or
 * neither): expert e lives on rank owner_map[e] as its local expert local_map[e]; NULL = consecutive blocks.
 * handle_out receives B200_EP_HANDLE_BYTES bytes to hand to every other rank. */
B200_API int b200_ep_create(b200_ep** ep, const b200_ep_config* cfg, const int* owner_map, const int* local_map,
                            void* handle_out);
/* handles: world * B200_EP_HANDLE_BYTES bytes, rank-major (this rank's own entry is ignored; may be NULL
 * when world == 1).  Call once, after every rank has created its object. */
B200_API int b200_ep_connect(b200_ep* ep, const void* handles);
/* One layer step for this rank's num_tokens tokens (<= max_tokens): xq [T,D] e4m3 + xs [T,D/128]; the
 * replicated router (gate_w [E,D], bias [E] or NULL); this rank's experts w1 [E/world,2I,D] + w1s, w2
 * [E/world,D,I] + w2s in local order (packed != 0: pre-tiled by b200_moe_fp8_pack_weights); out [T,D] fp32,
 * overwritten.  ids_out / w_out [T,K] (optional) receive the routing (global expert ids). */
B200_API int b200_ep_forward(b200_ep* ep, int num_tokens, const uint8_t* xq, const float* xs, const float* gate_w,
                             const float* bias, const uint8_t* w1, const float* w1s, const uint8_t* w2,
                             const float* w2s, int packed, float* out, int* ids_out, float* w_out,
                             b200_stream_t stream);
/* Synchronises `stream`; status (optional) receives and clears the device status word; send_counts /
 * recv_counts [world] (optional) the rows this rank sent to / received from each rank in the last step. */
B200_API int b200_ep_stats(b200_ep* ep, b200_stream_t stream, int* status, int* send_counts, int* recv_counts);
/* The object's own workspace (scratch of its grouped GEMMs, status word): for b200_moe_fp8_profile and
 * b200_ws_device_status.  Owned by the object. */
B200_API b200_ws* b200_ep_workspace(b200_ep* ep);
B200_API int b200_ep_destroy(b200_ep* ep);

/* --------------------------------------------------------------------------- */
/* Synthetic inputs (stand in for utils/cuda_utils.cuh:56-60 random_fill at      */
/* sizes a host loop cannot fill): counter-based, value i depends only on        */
/* (seed, i); identical bits to the host twin in the Python package.             */
/* --------------------------------------------------------------------------- */
B200_API int b200_fill_normal_f32(float* dst, long long n, unsigned long long seed, float sigma,
                                  b200_stream_t stream);
B200_API int b200_fill_normal_bf16(uint16_t* dst, long long n, unsigned long long seed, float sigma,
                                   b200_stream_t stream);
/* Generates N(0,sigma) values block by block and quantises them on the fly
 * (weights: 128x128 blocks; activations: 1x128) without an fp32 copy in memory. */
B200_API int b200_fill_normal_fp8_w128(uint8_t* q, float* scales, long long rows, int cols,
                                       unsigned long long seed, float sigma, b200_stream_t stream);
B200_API int b200_fill_normal_fp8_w128_pow2(uint8_t* q, float* scales, long long rows, int cols,
                                       unsigned long long seed, float sigma, b200_stream_t stream);   /* power-of-two scales */

#ifdef __cplusplus
}
#endif
#endif /* B200_MOE_DSA_H */
