"""ctypes bindings of the CPU oracle (``moe_dsa_oracle.c``) and, when built, of
the reference's own CPU code (``_ref/libref_*.so``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke test and by the
benchmark's CPU-baseline / reference arm.  The shipped package never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = {}

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")


def reference_dir():
    """A checkout of the reference project, or None: $B200_REFERENCE_DIR, else a directory named
    ``reference`` beside the repository, else ``baseline/_ref`` inside it."""
    root = os.path.dirname(HERE)
    for p in (os.environ.get("B200_REFERENCE_DIR"), os.path.join(os.path.dirname(root), "reference"),
              os.path.join(root, "baseline", "_ref")):
        if p and os.path.exists(os.path.join(p, "tests", "test_moe.cu")):
            return p
    return None


def build(force=False):
    """Compile liboracle.so (and _ref/ when a reference checkout is present)."""
    so = os.path.join(HERE, "liboracle.so")
    src = os.path.join(HERE, "moe_dsa_oracle.c")
    stale = (not os.path.exists(so)) or os.path.getmtime(so) < os.path.getmtime(src)
    ref = reference_dir()
    if force or stale or (ref is not None and not os.path.exists(os.path.join(HERE, "_ref", "libref_moe.so"))):
        cmd = ["make", "-C", HERE] + ([f"REF={ref}"] if ref else [])
        subprocess.run(cmd, check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is not None:
        return _LIB
    so = os.path.join(HERE, "liboracle.so")
    if not os.path.exists(so):
        build()
    L = C.CDLL(so)
    L.orc_max_threads.restype = C.c_int
    L.orc_set_threads.argtypes = [C.c_int]
    L.orc_srand.argtypes = [C.c_uint]
    L.orc_rand_fill.argtypes = [f32p, C.c_int64, C.c_float, C.c_float]
    L.orc_gen_sparse_indices.argtypes = [i32p, C.c_int, C.c_int, C.c_int, C.c_int]
    L.orc_route_softmax.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, f32p]
    L.orc_permute.argtypes = [i32p, C.c_int, C.c_int, C.c_int, i32p, i32p, i32p]
    L.orc_moe_forward_f32.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 5 + [i32p, f32p, f32p]
    L.orc_e4m3_decode_n.argtypes = [u8p, f32p, C.c_int64]
    L.orc_e4m3_encode_n.argtypes = [f32p, u8p, C.c_int64]
    L.orc_bf16_encode.argtypes = [C.c_float]
    L.orc_bf16_encode.restype = C.c_uint16
    L.orc_set_pow2_scales.argtypes = [C.c_int]
    L.orc_quant_act_1x128.argtypes = [f32p, C.c_int64, C.c_int, u8p, f32p]
    L.orc_quant_weight_128x128.argtypes = [f32p, C.c_int64, C.c_int, u8p, f32p]
    L.orc_gate_logits_fp8.argtypes = [u8p, f32p, f32p, C.c_int, C.c_int, C.c_int, f32p]
    L.orc_route_grouped_from_logits.argtypes = [f32p, C.c_void_p] + [C.c_int] * 5 + [C.c_float, i32p, f32p]
    L.orc_route_grouped.argtypes = [u8p, f32p, f32p, C.c_void_p] + [C.c_int] * 6 + [C.c_float, i32p, f32p]
    L.orc_moe_fp8_experts.argtypes = [u8p, f32p, u8p, f32p, u8p, f32p, i32p, f32p] + [C.c_int] * 5 + [i32p, C.c_int, f32p]
    L.orc_moe_fp8_gemm1_row.argtypes = [u8p, f32p, u8p, f32p, C.c_int, C.c_int, u8p, f32p]
    L.orc_dsa_forward_f32.argtypes = [f32p] * 5 + [i32p, f32p] + [C.c_int] * 5
    L.orc_dsa_forward_bf16.argtypes = [u16p] * 5 + [i32p, f32p] + [C.c_int] * 5
    L.orc_dsa_forward_bf16_gathered.argtypes = [u16p] * 5 + [f32p] + [C.c_int] * 5
    _LIB = L
    return L


def ref(which):
    """The reference's own CPU code ('moe' or 'dsa'), or None when not built."""
    if which in _REF:
        return _REF[which]
    so = os.path.join(HERE, "_ref", f"libref_{which}.so")
    L = None
    if os.path.exists(so):
        try:
            L = C.CDLL(so)
        except OSError:
            L = None
    if L is not None and which == "moe":
        L.ref_cpu_moe_forward.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 5 + [i32p, f32p, f32p]
        L.ref_random_fill.argtypes = [f32p, C.c_int, C.c_float, C.c_float]
        L.ref_srand.argtypes = [C.c_uint]
    if L is not None and which == "dsa":
        L.ref_cpu_dsa_forward.argtypes = [f32p] * 5 + [i32p, f32p] + [C.c_int] * 7
        L.ref_gen_sparse_indices.argtypes = [i32p, C.c_int, C.c_int, C.c_int]
        L.ref_dsa_random_fill.argtypes = [f32p, C.c_int, C.c_float, C.c_float]
        L.ref_dsa_srand.argtypes = [C.c_uint]
    _REF[which] = L
    return L


# ----------------------------------------------------------------------------
# numpy-level helpers
# ----------------------------------------------------------------------------
def max_threads():
    return int(lib().orc_max_threads())


def host_threads():
    """Host cores this process may run on (its affinity mask).  Unlike max_threads() this does not
    follow OMP_NUM_THREADS, which process launchers set to 1 for every rank."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def set_threads(n):
    lib().orc_set_threads(int(n))


def rand_fill(n, lo, hi):
    out = np.empty(int(n), np.float32)
    lib().orc_rand_fill(out, int(n), lo, hi)
    return out


def moe_inputs_reference_style(T, E, K, D, I, seed=42):
    """Inputs exactly as tests/test_moe.cu:151-164 makes them (glibc rand())."""
    L = lib()
    L.orc_srand(seed)
    x = rand_fill(T * D, -0.5, 0.5).reshape(T, D)
    wg = rand_fill(E * D, -0.5, 0.5).reshape(E, D)
    w1 = rand_fill(E * 2 * I * D, -0.1, 0.1).reshape(E, 2 * I, D)
    w2 = rand_fill(E * D * I, -0.1, 0.1).reshape(E, D, I)
    return x, wg, w1, w2


def dsa_inputs_reference_style(Q, H, Dc, Dp, S, P, N, seed=42, sorted_idx=True):
    """Inputs exactly as tests/test_dsa.cu:101-115 makes them."""
    L = lib()
    L.orc_srand(seed)
    qn = rand_fill(Q * H * Dc, -0.3, 0.3).reshape(Q, H, Dc)
    qp = rand_fill(Q * H * Dp, -0.3, 0.3).reshape(Q, H, Dp)
    kc = rand_fill(N * Dc, -0.3, 0.3).reshape(N, Dc)
    kp = rand_fill(N * Dp, -0.3, 0.3).reshape(N, Dp)
    v = rand_fill(N * Dc, -0.3, 0.3).reshape(N, Dc)
    idx = np.empty((Q, S), np.int32)
    L.orc_gen_sparse_indices(idx, Q, S, N, 1 if sorted_idx else 0)
    return qn, qp, kc, kp, v, idx


def route_softmax(x, wg, K):
    T, D = x.shape
    E = wg.shape[0]
    ids = np.empty((T, K), np.int32)
    wts = np.empty((T, K), np.float32)
    lib().orc_route_softmax(np.ascontiguousarray(x), np.ascontiguousarray(wg), T, E, K, D, ids, wts)
    return ids, wts


def permute(ids, E):
    T, K = ids.shape
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    row_pair = np.full(T * K, -1, np.int32)
    lib().orc_permute(np.ascontiguousarray(ids), T, K, E, counts, offsets, row_pair)
    return counts, offsets, row_pair[: offsets[E]]


def moe_forward_f32(x, wg, w1, w2, K):
    T, D = x.shape
    E = wg.shape[0]
    I = w2.shape[2]
    ids = np.empty((T, K), np.int32)
    wts = np.empty((T, K), np.float32)
    out = np.empty((T, D), np.float32)
    lib().orc_moe_forward_f32(np.ascontiguousarray(x), np.ascontiguousarray(wg), np.ascontiguousarray(w1),
                              np.ascontiguousarray(w2), T, E, K, D, I, ids, wts, out)
    return ids, wts, out


def e4m3_decode(b):
    b = np.ascontiguousarray(b, np.uint8)
    out = np.empty(b.shape, np.float32)
    lib().orc_e4m3_decode_n(b.reshape(-1), out.reshape(-1), b.size)
    return out


def e4m3_encode(f):
    f = np.ascontiguousarray(f, np.float32)
    out = np.empty(f.shape, np.uint8)
    lib().orc_e4m3_encode_n(f.reshape(-1), out.reshape(-1), f.size)
    return out


def bf16_bits(f):
    """fp32 array -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


class pow2_scales:
    """Context manager: block scales are powers of two (the smallest one >= amax/448) in quant_act, quant_weight
    and in the requantisation inside moe_fp8_experts / moe_fp8_gemm1_row while it is active."""

    def __enter__(self):
        lib().orc_set_pow2_scales(1)
        return self

    def __exit__(self, *exc):
        lib().orc_set_pow2_scales(0)
        return False


def quant_act(x):
    x = np.ascontiguousarray(x, np.float32)
    rows, cols = x.shape
    q = np.empty((rows, cols), np.uint8)
    s = np.empty((rows, cols // 128), np.float32)
    lib().orc_quant_act_1x128(x, rows, cols, q, s)
    return q, s


def quant_weight(w):
    """w [..., rows, cols] -> (q same shape uint8, scales [..., rows/128, cols/128])."""
    w = np.ascontiguousarray(w, np.float32)
    lead = w.shape[:-2]
    rows, cols = w.shape[-2:]
    w2 = w.reshape(-1, cols)
    q = np.empty(w2.shape, np.uint8)
    s = np.empty((w2.shape[0] // 128, cols // 128), np.float32)
    lib().orc_quant_weight_128x128(w2, w2.shape[0], cols, q, s)
    return q.reshape(w.shape), s.reshape(lead + (rows // 128, cols // 128))


def gate_logits_fp8(xq, xs, wg):
    T, D = xq.shape
    E = wg.shape[0]
    out = np.empty((T, E), np.float32)
    lib().orc_gate_logits_fp8(xq, xs, np.ascontiguousarray(wg), T, E, D, out)
    return out


def route_grouped(xq, xs, wg, bias, K, n_group, topk_group, routed_scale):
    T, D = xq.shape
    E = wg.shape[0]
    ids = np.empty((T, K), np.int32)
    wts = np.empty((T, K), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32).ctypes.data
    lib().orc_route_grouped(xq, xs, np.ascontiguousarray(wg), b, T, E, K, D, n_group, topk_group,
                            routed_scale, ids, wts)
    return ids, wts


def route_grouped_from_logits(logits, bias, K, n_group, topk_group, routed_scale):
    T, E = logits.shape
    ids = np.empty((T, K), np.int32)
    wts = np.empty((T, K), np.float32)
    b = None if bias is None else np.ascontiguousarray(bias, np.float32).ctypes.data
    lib().orc_route_grouped_from_logits(np.ascontiguousarray(logits), b, T, E, K, n_group, topk_group,
                                        routed_scale, ids, wts)
    return ids, wts


def moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, ids, wts, tokens):
    T, D = xq.shape
    E, _, I = w2q.shape
    K = ids.shape[1]
    tokens = np.ascontiguousarray(tokens, np.int32)
    out = np.empty((len(tokens), D), np.float32)
    lib().orc_moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, np.ascontiguousarray(ids), np.ascontiguousarray(wts),
                              T, E, K, D, I, tokens, len(tokens), out)
    return out


def moe_fp8_gemm1_row(xq_row, xs_row, w1e, w1se):
    D = xq_row.shape[0]
    I = w1e.shape[0] // 2
    q = np.empty(I, np.uint8)
    s = np.empty(I // 128, np.float32)
    lib().orc_moe_fp8_gemm1_row(np.ascontiguousarray(xq_row), np.ascontiguousarray(xs_row),
                                np.ascontiguousarray(w1e), np.ascontiguousarray(w1se), D, I, q, s)
    return q, s


def dsa_forward_f32(qn, qp, kc, kp, v, idx):
    Q, H, Dc = qn.shape
    Dp = qp.shape[2]
    S = idx.shape[1]
    out = np.empty((Q, H, Dc), np.float32)
    lib().orc_dsa_forward_f32(*(np.ascontiguousarray(a, np.float32) for a in (qn, qp, kc, kp, v)),
                              np.ascontiguousarray(idx, np.int32), out, Q, H, Dc, Dp, S)
    return out


def dsa_forward_bf16(qn, qp, kc, kp, v, idx):
    """Inputs are bf16 bit patterns (uint16 arrays)."""
    Q, H, Dc = qn.shape
    Dp = qp.shape[2]
    S = idx.shape[1]
    out = np.empty((Q, H, Dc), np.float32)
    lib().orc_dsa_forward_bf16(*(np.ascontiguousarray(a, np.uint16) for a in (qn, qp, kc, kp, v)),
                               np.ascontiguousarray(idx, np.int32), out, Q, H, Dc, Dp, S)
    return out


def dsa_forward_bf16_gathered(qn, qp, gkc, gkp, gv, S):
    Q, H, Dc = qn.shape
    Dp = qp.shape[2]
    out = np.empty((Q, H, Dc), np.float32)
    lib().orc_dsa_forward_bf16_gathered(*(np.ascontiguousarray(a, np.uint16) for a in (qn, qp, gkc, gkp, gv)),
                                        out, Q, H, Dc, Dp, S)
    return out
