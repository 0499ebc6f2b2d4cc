// Internal launch helpers shared by the MoE translation units.
#pragma once
#include "common.cuh"

// Width of one reduction chunk of the FP8 router's logits (see moe_route.cu).
#define MOE_GATE_CHUNK 1024

void b200_count_launch(int n);

int moe_gate_chunks(int D, bool fp8);
int launch_gate_logits(const void* x, const float* xs, const float* wg, float* partials, int T, int E, int D,
                       bool fp8, cudaStream_t stream);
// Selection on approximate logits (tensor-core router): a token is accepted only if every decision margin (kept
// vs dropped group scores, the order of the K selected selection scores, the K-th against the best unselected)
// exceeds tau; the others are appended to flag_list (count in *flag_n) for the exact pass.  tau = 0: exact
// logits, nothing is flagged.  list / list_n: the rows of `partials` are the tokens list[0 .. *list_n) (the exact
// pass over the flagged tokens); results go to the tokens' own slots of ids / wts.
// Work split of the tensor-core logits kernel.  A unit is one 128-token tile x one 128-deep block of d, units are
// numbered tile-major; CTA c owns the units [c * L, (c + 1) * L).  Inside its range a CTA cuts a new partial sum
// ("piece") at every tile boundary and after every `ch` blocks, and stores piece number s of a tile (counted in
// order of d) in slot s: partials[(s * T + t) * E + e].  The selection kernel adds a token's slots in order.
struct TcPlan {
    int L = 0;        // units per CTA (0: no tensor-core partial sums; n_chunks says how many slots to add)
    int nblk = 0;     // 128-deep blocks of d
    int ch = 0;       // longest accumulation chain, in blocks
};
// Pieces of tile `tile` that start before unit `upto` (tile * nblk <= upto <= (tile + 1) * nblk); with
// upto = (tile + 1) * nblk: the number of slots the tile's tokens have.
__host__ __device__ inline int tc_slots_before(const TcPlan& p, int tile, int upto) {
    const int s = tile * p.nblk;
    int n = 0;
    for (int c = s / p.L; c * p.L < upto; c++) {
        const int a = (s > c * p.L) ? s : c * p.L;
        const int b = (upto < (c + 1) * p.L) ? upto : (c + 1) * p.L;
        n += (b - a + p.ch - 1) / p.ch;
    }
    return n;
}
struct RouteCert {
    float tau = 0.0f;
    int* flag_list = nullptr;
    int* flag_n = nullptr;
    const int* list = nullptr;
    const int* list_n = nullptr;
    TcPlan plan;
};
int launch_route_select(const float* partials, int n_chunks, const float* bias, int* ids, float* wts, int* counts,
                        float* logits_out, int T, int E, int K, int scoring, int n_group, int topk_group,
                        float routed_scale, cudaStream_t stream, RouteCert cert = RouteCert());
// Tensor-core router logits (moe_route_tc.cu): approximate, for the certified selection above.
bool moe_gate_tc_supported(int T, int E, int D);
int moe_gate_tc_slots(int D);          // upper bound of the slots per token (sizes `partials`), any T
int launch_gate_logits_tc(const uint8_t* xq, const float* xs, const float* wg, float* whi, float* wlo, float* partials,
                          int T, int E, int D, int* status, cudaStream_t stream, TcPlan* plan_out);
// Exact router logits (the fixed-order FMA chains) for the tokens list[0 .. *list_n): partials[(chunk * T + i) * E + e]
// for list entry i.
int launch_gate_logits_list(const uint8_t* xq, const float* xs, const float* wg, float* partials, const int* list,
                            const int* list_n, int T, int E, int D, cudaStream_t stream);
// Whole routing step of the FP8 layer into caller-provided scratch; picks the tensor-core path when it applies.
struct RouteScratch {
    float* partials;     // max(moe_gate_chunks(D), moe_gate_tc_slots(D)) * T * E floats
    float* whi;          // E * D floats (tensor-core path)
    float* wlo;          // E * D floats
    int* flag_list;      // T ints
    int* flag_n;         // 1 int
};
size_t moe_route_scratch_floats(int T, int E, int D);
int moe_route_fp8_run(const RouteScratch& rs, const uint8_t* xq, const float* xs, const float* gate_w, const float* bias,
                      int* ids, float* wts, int* counts, float* logits_out, const b200_moe_fp8_config* cfg,
                      int* status, cudaStream_t stream);
// counts_in: the router's per-expert histogram (may be NULL: counted from ids).  trusted: ids come from
// this library's router (an expert appears at most once per token), so the duplicate check is skipped.
int launch_permute(const int* ids, int T, int K, int E, const int* counts_in, bool trusted, int* counts,
                   int* offsets, int* row_pair, cudaStream_t stream);
int check_route_cfg(int T, int E, int K, int D, int scoring, int n_group, int topk_group);

// b200_moe_fp8_experts without the zero-fill of `out` (the caller keeps the rows that receive
// contributions at zero); used by the expert-parallel owner side.
int b200_moe_fp8_experts_accumulate(b200_ws* ws, const uint8_t* xq, const float* xs, const int* expert_ids,
                                    const float* expert_w, const uint8_t* w1, const float* w1s, const uint8_t* w2,
                                    const float* w2s, float* out, const b200_moe_fp8_config* cfg, bool packed,
                                    cudaStream_t stream);
