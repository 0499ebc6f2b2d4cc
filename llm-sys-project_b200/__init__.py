"""Host-side mirror of the reference's launcher interface (kernels/moe/naive_moe.cuh,
kernels/dsa/naive_dsa.cuh) over the C ABI of ``lib/libb200moedsa.so``.

Function names, argument order and meaning follow the reference headers; tensors are
torch CUDA tensors (used only as device memory + streams).  There is no CPU fallback:
every call goes to the CUDA library and raises if the library is missing or a call
returns a non-zero status.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200moedsa.so")
_lib = None

(B200_OK, B200_BAD_SHAPE, B200_UNSUPPORTED, B200_CUDA_ERROR, B200_TIMEOUT, B200_NCCL_ERROR,
 B200_BAD_ARG) = range(7)
SCORE_SOFTMAX, SCORE_SIGMOID_GROUPED = 0, 1


class B200Error(RuntimeError):
    def __init__(self, status, what, detail=""):
        self.status = status
        super().__init__(f"{what}: status {status} ({detail})")


class MoeConfig(C.Structure):  # kernels/moe/naive_moe.cuh:9-15
    _fields_ = [(n, C.c_int) for n in ("num_tokens", "num_experts", "top_k", "hidden_dim", "intermediate_dim")]


class DsaConfig(C.Structure):  # kernels/dsa/naive_dsa.cuh:9-17
    _fields_ = [(n, C.c_int) for n in ("num_queries", "num_heads", "head_dim_compressed", "head_dim_positional",
                                       "num_selected_kv", "page_size", "total_kv_tokens")]


class MoeFp8Config(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("num_tokens", "num_experts", "top_k", "hidden_dim", "intermediate_dim",
                                       "scoring", "n_group", "topk_group")] + [("routed_scale", C.c_float),
                                                                                  ("flags", C.c_int)]


MOE_DETERMINISTIC = 1      # MoeFp8Config.flags: fixed-order (experts ascending) combine, bit-reproducible
MOE_SINGLE_CTA_TILES, MOE_CTA_PAIR_TILES = 4, 8      # force the grouped GEMMs' tile shape
MOE_EXACT_ROUTER_LOGITS = 16                         # fixed-order FMA router logits for every token
MOE_POW2_SCALES = 32                                 # all scales are powers of two: hardware block-scaled MMA
BAD_SCALE = 7                                        # device status: a scale was not a power of two


class EpConfig(C.Structure):
    _fields_ = ([(n, C.c_int) for n in ("rank", "world", "max_tokens", "num_experts", "top_k", "hidden_dim",
                                        "intermediate_dim", "scoring", "n_group", "topk_group")]
                + [("routed_scale", C.c_float), ("flags", C.c_int), ("wait_limit_ms", C.c_int)])


MoEConfig, DSAConfig = MoeConfig, DsaConfig

# every symbol include/b200_moe_dsa.h declares
EXPORTED_SYMBOLS = [
    "b200_status_string", "b200_last_error_string", "b200_ws_create", "b200_ws_destroy", "b200_ws_reserve",
    "b200_ws_capacity", "b200_ws_device_status", "b200_launch_count",
    "b200_moe_forward_f32", "b200_moe_gate_f32", "b200_moe_permute", "b200_moe_gather_f32", "b200_gemm_f32",
    "b200_swiglu_f32", "b200_moe_scatter_f32",
    "b200_quant_act_1x128", "b200_quant_weight_128x128", "b200_quant_act_1x128_pow2", "b200_quant_weight_128x128_pow2",
    "b200_moe_route_fp8", "b200_moe_fp8_forward",
    "b200_moe_fp8_experts", "b200_moe_fp8_pack_weights", "b200_moe_fp8_forward_packed",
    "b200_moe_fp8_experts_packed", "b200_moe_fp8_gemm1_stage", "b200_moe_fp8_profile", "b200_moe_fp8_profile_read",
    "b200_dsa_forward_f32", "b200_dsa_forward_bf16", "b200_dsa_forward_bf16_paged", "b200_dsa_forward_bf16_static", "b200_dsa_kv_gather_f32", "b200_dsa_dot_f32",
    "b200_dsa_softmax_f32", "b200_dsa_output_proj_f32",
    "b200_ep_plan", "b200_ep_sum_rows", "b200_ep_create", "b200_ep_connect", "b200_ep_forward", "b200_ep_stats",
    "b200_ep_workspace", "b200_ep_destroy",
    "b200_fill_normal_f32", "b200_fill_normal_bf16", "b200_fill_normal_fp8_w128", "b200_fill_normal_fp8_w128_pow2",
]
# exported for the test suite only (declared in csrc/selftest.h, not in the public header)
TEST_ONLY_SYMBOLS = ["b200_umma_selftest", "b200_wait_selftest", "b200_ep_connect_loopback", "b200_fp8_mma_rate",
                     "b200_moe_gate_logits_tc", "b200_moe_route_last_flagged", "b200_mx_selftest", "b200_ep_phase_profile", "b200_tc_plan_selftest"]


def lib():
    """The loaded CUDA library.  Raises if it has not been built (python llm-sys-project_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python llm-sys-project_b200/build.py` "
                               "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        L.b200_status_string.restype = C.c_char_p
        L.b200_status_string.argtypes = [C.c_int]
        L.b200_last_error_string.restype = C.c_char_p
        L.b200_launch_count.restype = C.c_longlong
        L.b200_launch_count.argtypes = [C.c_int]
        L.b200_ws_capacity.restype = C.c_size_t
        L.b200_ep_workspace.restype = C.c_void_p
        L.b200_ep_workspace.argtypes = [C.c_void_p]
        _lib = L
    return _lib


def _check(st, what):
    if st != 0:
        L = lib()
        raise B200Error(st, what, f"{L.b200_status_string(st).decode()}; {L.b200_last_error_string().decode()}")


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


def _stream(stream=None):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def launch_count(reset=False):
    return int(lib().b200_launch_count(1 if reset else 0))


def device_status(stream=None):
    """Synchronises the stream and returns (and clears) the device-side status word."""
    st = C.c_int(0)
    _check(lib().b200_ws_device_status(None, _stream(stream), C.byref(st)), "b200_ws_device_status")
    return st.value


def ws_reserve(nbytes):
    _check(lib().b200_ws_reserve(None, C.c_size_t(int(nbytes))), "b200_ws_reserve")


# ---------------------------------------------------------------------------
# MoE, fp32 — names as in kernels/moe/naive_moe.cuh:27-76
# ---------------------------------------------------------------------------
def moe_forward(input, gate_weight, w1, w2, output, cfg, stream=None):
    _check(lib().b200_moe_forward_f32(None, _p(input), _p(gate_weight), _p(w1), _p(w2), _p(output), C.byref(cfg),
                                      _stream(stream)), "moe_forward")


def moe_gate(input, gate_weight, expert_indices, expert_weights, cfg, stream=None):
    _check(lib().b200_moe_gate_f32(None, _p(input), _p(gate_weight), _p(expert_indices), _p(expert_weights),
                                   C.byref(cfg), _stream(stream)), "moe_gate")


def moe_permute(expert_indices, T, K, E, counts, offsets, row_pair, stream=None):
    _check(lib().b200_moe_permute(None, _p(expert_indices), T, K, E, _p(counts), _p(offsets), _p(row_pair),
                                  _stream(stream)), "moe_permute")


def moe_gather(input, expert_indices, expert_weights, expert_id, gathered, token_map, count, cfg, stream=None):
    _check(lib().b200_moe_gather_f32(_p(input), _p(expert_indices), int(expert_id), _p(gathered), _p(token_map),
                                     _p(count), C.byref(cfg), _stream(stream)), "moe_gather")


def naive_gemm(A, B, Cm, M, N, K, stream=None):
    _check(lib().b200_gemm_f32(_p(A), _p(B), _p(Cm), M, N, K, _stream(stream)), "naive_gemm")


def swiglu(gate, up, out, n, stream=None):
    _check(lib().b200_swiglu_f32(_p(gate), _p(up), _p(out), n, _stream(stream)), "swiglu")


def moe_scatter(expert_out, token_map, expert_weights, expert_indices, expert_id, output, count, cfg, stream=None):
    _check(lib().b200_moe_scatter_f32(_p(expert_out), _p(token_map), _p(expert_weights), _p(expert_indices),
                                      int(expert_id), _p(output), int(count), C.byref(cfg), _stream(stream)),
           "moe_scatter")


# ---------------------------------------------------------------------------
# MoE, FP8 block-scale
# ---------------------------------------------------------------------------
def quant_act_1x128(x, q, scales, stream=None, pow2=False):
    """pow2: power-of-two scales (for MOE_POW2_SCALES)."""
    rows, cols = x.shape
    fn = lib().b200_quant_act_1x128_pow2 if pow2 else lib().b200_quant_act_1x128
    _check(fn(_p(x), _p(q), _p(scales), C.c_longlong(rows), cols, _stream(stream)), "quant_act_1x128")


def quant_weight_128x128(w, q, scales, stream=None, pow2=False):
    cols = w.shape[-1]
    rows = w.numel() // cols
    fn = lib().b200_quant_weight_128x128_pow2 if pow2 else lib().b200_quant_weight_128x128
    _check(fn(_p(w), _p(q), _p(scales), C.c_longlong(rows), cols, _stream(stream)), "quant_weight_128x128")


def moe_route_fp8(xq, xs, gate_w, bias, expert_ids, expert_w, cfg, counts=None, logits_out=None, stream=None):
    _check(lib().b200_moe_route_fp8(None, _p(xq), _p(xs), _p(gate_w), _p(bias), _p(expert_ids), _p(expert_w),
                                    _p(counts), _p(logits_out), C.byref(cfg), _stream(stream)), "moe_route_fp8")


def moe_fp8_forward(xq, xs, gate_w, bias, w1q, w1s, w2q, w2s, out, cfg, stream=None):
    _check(lib().b200_moe_fp8_forward(None, _p(xq), _p(xs), _p(gate_w), _p(bias), _p(w1q), _p(w1s), _p(w2q),
                                      _p(w2s), _p(out), C.byref(cfg), _stream(stream)), "moe_fp8_forward")


def moe_fp8_experts(xq, xs, expert_ids, expert_w, w1q, w1s, w2q, w2s, out, cfg, stream=None):
    _check(lib().b200_moe_fp8_experts(None, _p(xq), _p(xs), _p(expert_ids), _p(expert_w), _p(w1q), _p(w1s),
                                      _p(w2q), _p(w2s), _p(out), C.byref(cfg), _stream(stream)), "moe_fp8_experts")


def moe_fp8_pack_weights(which, src, packed, E, D, I, stream=None):
    """which = 1: w1q [E,2I,D]; which = 2: w2q [E,D,I].  `packed` is a uint8 buffer of the same size."""
    _check(lib().b200_moe_fp8_pack_weights(int(which), _p(src), _p(packed), E, D, I, _stream(stream)),
           "moe_fp8_pack_weights")


def moe_fp8_forward_packed(xq, xs, gate_w, bias, w1p, w1s, w2p, w2s, out, cfg, stream=None):
    _check(lib().b200_moe_fp8_forward_packed(None, _p(xq), _p(xs), _p(gate_w), _p(bias), _p(w1p), _p(w1s), _p(w2p),
                                             _p(w2s), _p(out), C.byref(cfg), _stream(stream)),
           "moe_fp8_forward_packed")


def moe_fp8_experts_packed(xq, xs, expert_ids, expert_w, w1p, w1s, w2p, w2s, out, cfg, stream=None):
    _check(lib().b200_moe_fp8_experts_packed(None, _p(xq), _p(xs), _p(expert_ids), _p(expert_w), _p(w1p), _p(w1s),
                                             _p(w2p), _p(w2s), _p(out), C.byref(cfg), _stream(stream)),
           "moe_fp8_experts_packed")


def moe_fp8_gemm1_stage(xq, xs, expert_ids, w1q, w1s, act_q, act_s, offsets, row_pair, cfg, stream=None):
    _check(lib().b200_moe_fp8_gemm1_stage(None, _p(xq), _p(xs), _p(expert_ids), _p(w1q), _p(w1s), _p(act_q),
                                          _p(act_s), _p(offsets), _p(row_pair), C.byref(cfg), _stream(stream)),
           "moe_fp8_gemm1_stage")


def ep_plan(expert_ids, expert_w, experts_per_rank, world, send_tok, pos, send_counts, slot_ids, slot_w, strided=False,
            owner_map=None, local_map=None, stream=None):
    T, K = expert_ids.shape
    _check(lib().b200_ep_plan(_p(expert_ids), _p(expert_w), T, K, int(experts_per_rank), int(world),
                              1 if strided else 0, _p(owner_map), _p(local_map), _p(send_tok),
                              _p(pos), _p(send_counts), _p(slot_ids), _p(slot_w), _stream(stream)), "ep_plan")


def ep_sum_rows(back, pos, world, out, stream=None):
    """back [R,D] fp32 or bf16; pos [world,T] int32; out [T,D] fp32."""
    import torch
    T, D = out.shape
    _check(lib().b200_ep_sum_rows(_p(back), 1 if back.dtype == torch.bfloat16 else 0, _p(pos), int(world), T, D,
                                  _p(out), _stream(stream)), "ep_sum_rows")


def moe_fp8_profile(enable, ws=None):
    """ws: a workspace handle (e.g. PeerExpertParallelMoe.workspace()); None = the default workspace."""
    _check(lib().b200_moe_fp8_profile(C.c_void_p(ws), 1 if enable else 0), "moe_fp8_profile")


def moe_fp8_profile_read(ws=None):
    a, b, n = C.c_float(0), C.c_float(0), C.c_int(0)
    _check(lib().b200_moe_fp8_profile_read(C.c_void_p(ws), C.byref(a), C.byref(b), C.byref(n)), "moe_fp8_profile_read")
    return a.value, b.value, n.value


# ---------------------------------------------------------------------------
# DSA — names as in kernels/dsa/naive_dsa.cuh:31-87
# ---------------------------------------------------------------------------
def dsa_forward(q_nope, q_pe, kv_cache_compressed, kv_cache_positional, v_cache, sparse_indices, output, cfg,
                stream=None):
    _check(lib().b200_dsa_forward_f32(None, _p(q_nope), _p(q_pe), _p(kv_cache_compressed), _p(kv_cache_positional),
                                      _p(v_cache), _p(sparse_indices), _p(output), C.byref(cfg), _stream(stream)),
           "dsa_forward")


def dsa_forward_bf16(q_nope, q_pe, kv_cache_compressed, kv_cache_positional, v_cache, sparse_indices, output, cfg,
                     stream=None):
    _check(lib().b200_dsa_forward_bf16(None, _p(q_nope), _p(q_pe), _p(kv_cache_compressed),
                                       _p(kv_cache_positional), _p(v_cache), _p(sparse_indices), _p(output),
                                       C.byref(cfg), _stream(stream)), "dsa_forward_bf16")


def dsa_forward_bf16_paged(q_nope, q_pe, kv_cache_compressed, kv_cache_positional, v_cache, positions, block_table,
                           output, cfg, seq_of_query=None, valid_len=None, stream=None):
    """bf16 decode on logical positions: positions [Q,S] int32 (negative = empty slot), block_table
    [num_seqs, max_blocks] int32 (logical page -> physical page, negative = not mapped), seq_of_query [Q]
    (None: query q reads sequence q), valid_len [Q] (None: all S entries count)."""
    _check(lib().b200_dsa_forward_bf16_paged(None, _p(q_nope), _p(q_pe), _p(kv_cache_compressed),
                                             _p(kv_cache_positional), _p(v_cache), _p(positions), _p(block_table),
                                             int(block_table.shape[1]), _p(seq_of_query), _p(valid_len), _p(output),
                                             C.byref(cfg), _stream(stream)), "dsa_forward_bf16_paged")


def dsa_forward_bf16_static(q_nope, q_pe, kv_cache_compressed, kv_cache_positional, v_cache, sparse_indices, output,
                            cfg, device_status, stream=None):
    """bf16 decode for callers that may not allocate device memory (a pool that owns all of HBM, a
    plugin that only receives its input/output buffers): the split-KV partial results live in a
    16 MiB array built into the library instead of the growable workspace, and the row split is
    limited to what that array holds.  device_status: caller-owned int32 CUDA tensor [1], cleared by
    the call; B200_TIMEOUT lands there if a device-side wait runs out.  Calls share the array; do
    not overlap them."""
    _check(lib().b200_dsa_forward_bf16_static(_p(q_nope), _p(q_pe), _p(kv_cache_compressed),
                                              _p(kv_cache_positional), _p(v_cache), _p(sparse_indices), _p(output),
                                              C.byref(cfg), _p(device_status), _stream(stream)),
           "dsa_forward_bf16_static")


def dsa_kv_gather(kc, kp, v, sparse_indices, g_kc, g_kp, g_v, cfg, stream=None):
    _check(lib().b200_dsa_kv_gather_f32(_p(kc), _p(kp), _p(v), _p(sparse_indices), _p(g_kc), _p(g_kp), _p(g_v),
                                        C.byref(cfg), _stream(stream)), "dsa_kv_gather")


def dsa_dot_compressed(q_nope, kc, scores, cfg, stream=None):
    _check(lib().b200_dsa_dot_f32(_p(q_nope), None, _p(kc), None, _p(scores), C.byref(cfg), _stream(stream)),
           "dsa_dot_compressed")


def dsa_dot_positional(q_pe, kp, scores, cfg, stream=None):
    _check(lib().b200_dsa_dot_f32(None, _p(q_pe), None, _p(kp), _p(scores), C.byref(cfg), _stream(stream)),
           "dsa_dot_positional")


def dsa_dot_fused(q_nope, q_pe, kc, kp, scores, cfg, stream=None):
    _check(lib().b200_dsa_dot_f32(_p(q_nope), _p(q_pe), _p(kc), _p(kp), _p(scores), C.byref(cfg), _stream(stream)),
           "dsa_dot_fused")


def dsa_softmax(scores, cfg, stream=None):
    _check(lib().b200_dsa_softmax_f32(_p(scores), C.byref(cfg), _stream(stream)), "dsa_softmax")


def dsa_output_proj(attn, v, output, cfg, stream=None):
    _check(lib().b200_dsa_output_proj_f32(_p(attn), _p(v), _p(output), C.byref(cfg), _stream(stream)),
           "dsa_output_proj")


# ---------------------------------------------------------------------------
# Synthetic inputs: device generators and their host twin (identical bits)
# ---------------------------------------------------------------------------
_SYNTH_SD = np.float32(53510.03113)


def fill_normal_(t, seed, sigma, stream=None):
    import torch
    n = t.numel()
    if t.dtype == torch.float32:
        _check(lib().b200_fill_normal_f32(_p(t), C.c_longlong(n), C.c_ulonglong(seed), C.c_float(sigma),
                                          _stream(stream)), "fill_normal_f32")
    elif t.dtype == torch.bfloat16:
        _check(lib().b200_fill_normal_bf16(_p(t), C.c_longlong(n), C.c_ulonglong(seed), C.c_float(sigma),
                                           _stream(stream)), "fill_normal_bf16")
    else:
        raise TypeError(t.dtype)
    return t


def fill_normal_fp8_w128_(q, scales, seed, sigma, stream=None, pow2=False):
    cols = q.shape[-1]
    rows = q.numel() // cols
    fn = lib().b200_fill_normal_fp8_w128_pow2 if pow2 else lib().b200_fill_normal_fp8_w128
    _check(fn(_p(q), _p(scales), C.c_longlong(rows), cols, C.c_ulonglong(seed), C.c_float(sigma), _stream(stream)),
           "fill_normal_fp8_w128")


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15))
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def synth_normal_host(seed, start, n, sigma):
    """Host twin of the device generator: values [start, start+n) of stream `seed` as float32."""
    with np.errstate(over="ignore"):
        i = np.arange(start, start + n, dtype=np.uint64)
        key = np.uint64(seed) * np.uint64(0xD1342543DE82EF95) + i
        a = _splitmix64(key)
        b = _splitmix64(key ^ np.uint64(0xA5A5A5A5A5A5A5A5))
        s = np.zeros(n, np.int64)
        for j in range(4):
            s += ((a >> np.uint64(16 * j)) & np.uint64(0xFFFF)).astype(np.int64)
            s += ((b >> np.uint64(16 * j)) & np.uint64(0xFFFF)).astype(np.int64)
    factor = np.float32(sigma) / _SYNTH_SD
    return (s - 262140).astype(np.float32) * factor


def umma_selftest(mode, a, b, d, N, K, stream=None):
    """Test hook: one tensor-core tile through the production shared-memory layouts."""
    _check(lib().b200_umma_selftest(int(mode), _p(a), _p(b), _p(d), int(N), int(K), _stream(stream)),
           "umma_selftest")


def fp8_mma_rate(pair=False, iters=20000, stream=None):
    """Measurement hook: dense FP8 tensor rate (TFLOP/s, milliseconds) of the MMA shape the grouped GEMMs issue,
    operands resident in shared memory (pair: cta_group::2, 256 x 256 x 32 per CTA pair)."""
    tf, ms = C.c_float(0), C.c_float(0)
    _check(lib().b200_fp8_mma_rate(1 if pair else 0, int(iters), C.byref(tf), C.byref(ms), _stream(stream)),
           "fp8_mma_rate")
    return tf.value, ms.value


def mx_selftest(a, b, sfa, sfb, d, stream=None):
    """Test hook: block-scaled FP8 MMA, d[128, N] = sum_k a 2^(sfa-127) b 2^(sfb-127) (e4m3 bytes, UE8M0 bytes)."""
    N, K = b.shape
    _check(lib().b200_mx_selftest(_p(a), _p(b), _p(sfa), _p(sfb), _p(d), N, K, _stream(stream)), "mx_selftest")


def moe_gate_logits_tc(xq, xs, gate_w, chain_blocks=0, stream=None):
    """Test hook: the approximate router logits [T, E] of the tensor-core path.
    chain_blocks: length of the accumulation chains in 128-deep blocks of d (0 = the library's own choice;
    D // 128 = one chain over all of d, which shows how the tensor core's accumulation error grows with the chain)."""
    import torch
    T, D = xq.shape
    E = gate_w.shape[0]
    logits = torch.empty((T, E), dtype=torch.float32, device=xq.device)
    _check(lib().b200_moe_gate_logits_tc(_p(xq), _p(xs), _p(gate_w), _p(logits), T, E, D, int(chain_blocks),
                                         _stream(stream)), "moe_gate_logits_tc")
    return logits


def moe_route_last_flagged(stream=None, ws=None):
    """Tokens the last tensor-core routing call handed to its exact pass (-1: the call took the exact path)."""
    n = C.c_int(0)
    _check(lib().b200_moe_route_last_flagged(C.c_void_p(ws), _stream(stream), C.byref(n)), "moe_route_last_flagged")
    return n.value


def wait_selftest(elapsed_ns, stream=None):
    """Test hook: a one-block kernel waits (bounded, a few milliseconds) on an mbarrier nobody signals,
    gives up, records B200_TIMEOUT in the default workspace's status word and exits.
    elapsed_ns: int64 CUDA tensor [2] receiving the time each of the two waiters spent."""
    _check(lib().b200_wait_selftest(None, _p(elapsed_ns), _stream(stream)), "wait_selftest")


from .ep import (ExpertParallelMoe, PeerExpertParallelMoe, balanced_placement, dispatch_plan,  # noqa: E402,F401
                 expert_owner)
from .hostapi import MoeFp8Layer, DsaDecodeLayer, HostPipeline  # noqa: E402,F401
