"""Generates tests/golden/*.npz from the reference's OWN CPU code.

Run in a container that has the reference checkout (``make -C oracle`` builds
``oracle/_ref/libref_{moe,dsa}.so`` from the reference's tests/test_moe.cu and
tests/test_dsa.cu where they lie).  For each of the reference's 13 MoE and 14
DSA cases (tests/test_moe.cu:203-267, tests/test_dsa.cu:161-230) it seeds
srand(42), fills the inputs in the reference's order through the reference's
random_fill / gen_sparse_indices, runs cpu_moe_forward / cpu_dsa_forward and
stores the outputs plus float64 checksums of the inputs (so a test can tell a
libc rand() mismatch from a kernel bug).  Inputs are not stored: they are
regenerated from the seed.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

MOE_CASES = {  # name: (T, E, K, D, I, tol)
    "small": (4, 4, 2, 64, 128, 1e-3), "medium": (32, 8, 2, 128, 256, 1e-3),
    "large": (64, 8, 2, 256, 512, 1e-2), "topk4": (16, 8, 4, 128, 256, 1e-2),
    "single_token": (1, 4, 2, 64, 128, 1e-3), "single_expert": (8, 1, 1, 64, 128, 1e-3),
    "topk1": (32, 16, 1, 128, 256, 1e-2), "wide_ffn": (16, 4, 2, 64, 512, 1e-2),
    "narrow_ffn": (16, 4, 2, 256, 64, 1e-2), "sparse_routing": (4, 16, 2, 128, 256, 1e-3),
    "many_tokens": (128, 8, 2, 128, 256, 1e-2), "full_routing": (8, 4, 4, 64, 128, 1e-3),
    "stress": (64, 16, 2, 512, 1024, 5e-2),
}
DSA_CASES = {  # name: (Q, H, Dc, Dp, S, P, N, tol)
    "tiny": (2, 2, 32, 8, 16, 8, 64, 1e-3), "small": (4, 4, 64, 16, 64, 16, 256, 1e-3),
    "medium": (8, 8, 128, 32, 128, 32, 512, 1e-2), "large": (4, 4, 128, 32, 256, 64, 1024, 1e-2),
    "single_query": (1, 4, 64, 16, 32, 8, 128, 1e-3), "single_head": (4, 1, 64, 16, 64, 16, 256, 1e-3),
    "minimal_s": (4, 4, 64, 16, 4, 4, 256, 1e-3), "pos_heavy": (4, 4, 32, 64, 64, 16, 256, 1e-3),
    "tiny_dp": (4, 4, 128, 4, 64, 16, 256, 1e-2), "many_heads": (4, 32, 64, 16, 64, 16, 256, 1e-2),
    "many_queries": (32, 4, 64, 16, 64, 16, 512, 1e-2), "full_cache": (4, 4, 64, 16, 128, 16, 128, 1e-3),
    "large_cache": (4, 4, 128, 32, 128, 64, 4096, 1e-2), "stress": (16, 16, 128, 32, 256, 64, 2048, 5e-2),
}


def main():
    rm, rd = oracle.ref("moe"), oracle.ref("dsa")
    if rm is None or rd is None:
        sys.exit("oracle/_ref not built: run `make -C oracle` where the reference checkout exists")
    out = {}
    for name, (T, E, K, D, I, tol) in MOE_CASES.items():
        rm.ref_srand(42)
        x = np.empty(T * D, np.float32); rm.ref_random_fill(x, x.size, -0.5, 0.5)
        wg = np.empty(E * D, np.float32); rm.ref_random_fill(wg, wg.size, -0.5, 0.5)
        w1 = np.empty(E * 2 * I * D, np.float32); rm.ref_random_fill(w1, w1.size, -0.1, 0.1)
        w2 = np.empty(E * D * I, np.float32); rm.ref_random_fill(w2, w2.size, -0.1, 0.1)
        ids = np.empty(T * K, np.int32); wts = np.empty(T * K, np.float32); o = np.empty(T * D, np.float32)
        rm.ref_cpu_moe_forward(x, wg, w1, w2, T, E, K, D, I, ids, wts, o)
        out[f"moe/{name}/cfg"] = np.array([T, E, K, D, I], np.int32)
        out[f"moe/{name}/tol"] = np.float32(tol)
        out[f"moe/{name}/ids"] = ids.reshape(T, K)
        out[f"moe/{name}/wts"] = wts.reshape(T, K)
        out[f"moe/{name}/out"] = o.reshape(T, D)
        out[f"moe/{name}/insum"] = np.array([x.sum(dtype=np.float64), wg.sum(dtype=np.float64),
                                             w1.sum(dtype=np.float64), w2.sum(dtype=np.float64)])
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "moe_reference_cases.npz"), **out)
    out = {}
    for name, (Q, H, Dc, Dp, S, P, N, tol) in DSA_CASES.items():
        rd.ref_dsa_srand(42)
        mk = lambda n: np.empty(n, np.float32)
        qn, qp, kc, kp, v = mk(Q * H * Dc), mk(Q * H * Dp), mk(N * Dc), mk(N * Dp), mk(N * Dc)
        for a in (qn, qp, kc, kp, v):
            rd.ref_dsa_random_fill(a, a.size, -0.3, 0.3)
        idx = np.empty(Q * S, np.int32); rd.ref_gen_sparse_indices(idx, Q, S, N)
        o = np.zeros(Q * H * Dc, np.float32)
        rd.ref_cpu_dsa_forward(qn, qp, kc, kp, v, idx, o, Q, H, Dc, Dp, S, P, N)
        out[f"dsa/{name}/cfg"] = np.array([Q, H, Dc, Dp, S, P, N], np.int32)
        out[f"dsa/{name}/tol"] = np.float32(tol)
        out[f"dsa/{name}/idx"] = idx.reshape(Q, S)
        out[f"dsa/{name}/out"] = o.reshape(Q, H, Dc)
        out[f"dsa/{name}/insum"] = np.array([a.sum(dtype=np.float64) for a in (qn, qp, kc, kp, v)])
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "dsa_reference_cases.npz"), **out)
    print("wrote", sorted(os.listdir(os.path.join(ROOT, "tests", "golden"))))


if __name__ == "__main__":
    main()
