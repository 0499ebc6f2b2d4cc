"""CPU tests: the oracle against the golden vectors made by the reference's own CPU code,
the number formats against torch, and properties of the restated routing / quantisers."""
import os

import numpy as np
import pytest
import torch

import oracle

GOLD = os.path.join(os.path.dirname(__file__), "golden")
MOE = np.load(os.path.join(GOLD, "moe_reference_cases.npz"))
DSA = np.load(os.path.join(GOLD, "dsa_reference_cases.npz"))
MOE_NAMES = sorted({k.split("/")[1] for k in MOE.files})
DSA_NAMES = sorted({k.split("/")[1] for k in DSA.files})


@pytest.mark.parametrize("name", MOE_NAMES)
def test_moe_oracle_matches_reference_cpu(name):
    T, E, K, D, I = (int(v) for v in MOE[f"moe/{name}/cfg"])
    x, wg, w1, w2 = oracle.moe_inputs_reference_style(T, E, K, D, I)
    insum = np.array([a.sum(dtype=np.float64) for a in (x, wg, w1, w2)])
    assert np.array_equal(insum, MOE[f"moe/{name}/insum"]), "libc rand() sequence differs from the fixture's"
    ids, wts, out = oracle.moe_forward_f32(x, wg, w1, w2, K)
    assert np.array_equal(ids, MOE[f"moe/{name}/ids"])
    assert np.array_equal(wts, MOE[f"moe/{name}/wts"])
    assert np.array_equal(out, MOE[f"moe/{name}/out"])      # bit-exact restatement


@pytest.mark.parametrize("name", DSA_NAMES)
def test_dsa_oracle_matches_reference_cpu(name):
    Q, H, Dc, Dp, S, P, N = (int(v) for v in DSA[f"dsa/{name}/cfg"])
    qn, qp, kc, kp, v, idx = oracle.dsa_inputs_reference_style(Q, H, Dc, Dp, S, P, N)
    assert np.array_equal(idx, DSA[f"dsa/{name}/idx"])
    out = oracle.dsa_forward_f32(qn, qp, kc, kp, v, idx)
    assert np.array_equal(out, DSA[f"dsa/{name}/out"])


def test_reference_anchor_values():
    # values obtained by running the reference CPU code on its "medium" MoE and "small" DSA cases
    out = MOE["moe/medium/out"]
    assert abs(out.sum(dtype=np.float64) - 3.924888641e-01) < 1e-9
    assert list(MOE["moe/medium/ids"][0]) == [0, 4] and list(MOE["moe/medium/ids"][1]) == [0, 7]
    d = DSA["dsa/small/out"]
    assert abs(d.sum(dtype=np.float64) - (-2.286994082)) < 1e-8
    assert list(DSA["dsa/small/idx"][0][:4]) == [0, 10, 12, 17]


def test_e4m3_matches_torch():
    b = np.arange(256, dtype=np.uint8)
    dec = oracle.e4m3_decode(b)
    ref = torch.from_numpy(b.copy()).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    ok = ~np.isnan(ref)
    assert np.array_equal(np.isnan(dec), np.isnan(ref))
    assert np.array_equal(dec[ok], ref[ok])
    rng = np.random.default_rng(0)
    f = np.concatenate([rng.normal(0, 1, 200000), rng.normal(0, 100, 100000), rng.uniform(-0.02, 0.02, 100000),
                        dec[ok], (dec[ok][:-1] + dec[ok][1:]) / 2, [0.0, -0.0, 448.0, -448.0, 464.0, 1e9, -1e9]]
                       ).astype(np.float32)
    enc = oracle.e4m3_encode(f)
    clamped = torch.from_numpy(np.clip(f, -448.0, 448.0))      # torch's CPU cast does not saturate
    ref_enc = clamped.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(enc, ref_enc)


def test_bf16_matches_torch():
    rng = np.random.default_rng(1)
    f = rng.normal(0, 3, 100000).astype(np.float32)
    bits = oracle.bf16_bits(f)
    ref = torch.from_numpy(f).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, ref)
    assert np.array_equal(oracle.bf16_to_f32(bits), torch.from_numpy(f).to(torch.bfloat16).float().numpy())


def test_quantisers_roundtrip_and_scales():
    rng = np.random.default_rng(2)
    x = rng.normal(0, 1, (5, 384)).astype(np.float32)
    x[3, 128:256] = 0.0                                        # all-zero block -> scale 1
    q, s = oracle.quant_act(x)
    assert s.shape == (5, 3) and s[3, 1] == 1.0 and not q[3, 128:256].any()
    amax = np.abs(x.reshape(5, 3, 128)).max(-1)
    assert np.array_equal(s[amax > 0], (amax / np.float32(448.0))[amax > 0])
    deq = oracle.e4m3_decode(q).reshape(5, 3, 128) * s[..., None]
    assert np.abs(deq.reshape(5, 384) - x).max() <= np.abs(x).max() * 2 ** -4     # 3 mantissa bits
    w = rng.normal(0, 0.02, (2, 256, 128)).astype(np.float32)
    wq, ws = oracle.quant_weight(w)
    assert ws.shape == (2, 2, 1)
    assert np.array_equal(ws[1, 0, 0], np.abs(w[1, :128]).max() / np.float32(448.0))
    assert oracle.e4m3_decode(wq).max() == 448.0 or np.abs(oracle.e4m3_decode(wq)).max() == 448.0


def _route_grouped_numpy(logits, bias, K, n_group, topk_group, scale):
    T, E = logits.shape
    gs = E // n_group
    s = (1.0 / (1.0 + np.exp(-logits.astype(np.float64)))).astype(np.float32)
    c = (s + bias).astype(np.float32)
    ids = np.zeros((T, K), np.int32)
    wts = np.zeros((T, K), np.float32)
    for t in range(T):
        g = c[t].reshape(n_group, gs)
        top2 = -np.sort(-g, axis=1)[:, :2]
        gscore = (top2[:, 0] + top2[:, 1]).astype(np.float32)
        keep = np.zeros(n_group, bool)
        for _ in range(topk_group):
            cand = np.where(~keep, gscore, -np.inf)
            keep[int(np.argmax(cand))] = True          # argmax returns the lowest index on ties
        masked = np.where(np.repeat(keep, gs), c[t], -np.inf)
        chosen = []
        for _ in range(K):
            e = int(np.argmax(masked))
            chosen.append(e)
            masked[e] = -np.inf
        ids[t] = chosen
        w = s[t, chosen]
        tot = np.float32(0)
        for v in w:
            tot = np.float32(tot + v)
        wts[t] = (w / tot * np.float32(scale)).astype(np.float32)
    return ids, wts


def test_grouped_routing_oracle_against_numpy():
    rng = np.random.default_rng(3)
    logits = rng.normal(0, 1, (64, 64)).astype(np.float32)
    logits[5, 3] = logits[5, 9]                                  # a tie: lowest id must win
    bias = rng.normal(0, 0.01, 64).astype(np.float32)
    ids, wts = oracle.route_grouped_from_logits(logits, bias, 8, 8, 4, 2.5)
    rid, rw = _route_grouped_numpy(logits, bias, 8, 8, 4, 2.5)
    assert np.array_equal(ids, rid)
    assert np.array_equal(wts, rw)
    assert np.allclose(wts.sum(1), 2.5, rtol=1e-5)
    groups = ids // 8
    assert all(len(set(g)) <= 4 for g in groups)                 # at most topk_group groups per token


def test_permutation_is_canonical():
    rng = np.random.default_rng(4)
    T, K, E = 50, 3, 7
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    counts, offsets, row_pair = oracle.permute(ids, E)
    assert counts.sum() == T * K and offsets[0] == 0 and np.array_equal(np.diff(offsets), counts)
    e_of_row = ids.reshape(-1)[row_pair]
    assert np.all(np.diff(e_of_row) >= 0)                        # experts ascending
    for e in range(E):
        toks = row_pair[offsets[e]:offsets[e + 1]] // K
        assert np.all(np.diff(toks) > 0)                         # tokens ascending, once each
    assert sorted(row_pair.tolist()) == list(range(T * K))


def test_fp8_emulation_consistency():
    """orc_moe_fp8_experts on one token == its own stage helper + a numpy second GEMM."""
    rng = np.random.default_rng(5)
    T, E, K, D, I = 3, 2, 1, 256, 128
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    w1 = rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32)
    w2 = rng.normal(0, 0.05, (E, D, I)).astype(np.float32)
    xq, xs = oracle.quant_act(x)
    w1q, w1s = oracle.quant_weight(w1)
    w2q, w2s = oracle.quant_weight(w2)
    ids = np.array([[1], [0], [1]], np.int32)
    wts = np.array([[0.5], [1.0], [2.0]], np.float32)
    out = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, ids, wts, np.array([2], np.int32))
    aq, asc = oracle.moe_fp8_gemm1_row(xq[2], xs[2], w1q[1], w1s[1])
    act = oracle.e4m3_decode(aq) * np.repeat(asc, 128)
    w2d = oracle.e4m3_decode(w2q[1]) * np.repeat(np.repeat(w2s[1], 128, 0), 128, 1)
    ref = 2.0 * (w2d.astype(np.float64) @ act.astype(np.float64))
    assert np.allclose(out[0], ref, rtol=1e-4, atol=1e-5)
    # against an unquantised fp64 evaluation: within FP8 noise
    g = w1[1].astype(np.float64) @ x[2].astype(np.float64)
    a = g[:I] / (1 + np.exp(-g[:I])) * g[I:]
    full = 2.0 * (w2[1].astype(np.float64) @ a)
    assert np.abs(out[0] - full).max() < 0.2 * np.abs(full).max() + 1e-3


def test_dsa_bf16_oracle_and_duplicates():
    rng = np.random.default_rng(6)
    Q, H, Dc, Dp, S, N = 2, 3, 64, 16, 8, 40
    f = lambda *s: rng.normal(0, 0.5, s).astype(np.float32)
    qn, qp, kc, kp, v = f(Q, H, Dc), f(Q, H, Dp), f(N, Dc), f(N, Dp), f(N, Dc)
    idx = rng.integers(0, N, (Q, S)).astype(np.int32)
    idx[0, 1] = idx[0, 0]                                        # duplicate contributes twice
    out = oracle.dsa_forward_f32(qn, qp, kc, kp, v, idx)
    sc = np.einsum("qhd,qsd->qhs", qn, kc[idx]) + np.einsum("qhd,qsd->qhs", qp, kp[idx])
    sc = sc / np.sqrt(Dc + Dp)
    p = np.exp(sc - sc.max(-1, keepdims=True)); p /= p.sum(-1, keepdims=True)
    assert np.allclose(out, np.einsum("qhs,qsd->qhd", p, v[idx]), atol=1e-5)
    perm = rng.permutation(S)
    assert np.allclose(oracle.dsa_forward_f32(qn, qp, kc, kp, v, idx[:, perm]), out, atol=1e-6)   # order-free
    b = [oracle.bf16_bits(a) for a in (qn, qp, kc, kp, v)]
    ob = oracle.dsa_forward_bf16(*b, idx)
    of = oracle.dsa_forward_f32(*[oracle.bf16_to_f32(a) for a in b], idx)
    assert np.array_equal(ob, of)


def test_pow2_scale_rule():
    """Power-of-two block scales: the smallest power of two >= amax/448, 1 for an all-zero block; the quantised
    values then stay inside the e4m3 range, and the emulation's requantisation follows the same rule."""
    rng = np.random.default_rng(3)
    x = (rng.normal(0, 1, (16, 384)) * np.exp2(rng.integers(-30, 30, (16, 1)))).astype(np.float32)
    x[2, :128] = 0
    x[3, :128] = np.float32(448.0 * 2.0 ** 5) * np.sign(x[3, :128] + 1e-30)       # quotient exactly 2^5
    q0, s0 = oracle.quant_act(x)
    with oracle.pow2_scales():
        q, s = oracle.quant_act(x)
        wq, ws = oracle.quant_weight(x[:, :128].repeat(8, axis=0))
    q1, s1 = oracle.quant_act(x)
    assert np.array_equal(s0, s1) and np.array_equal(q0, q1)             # the switch is off again
    m, _ = np.frexp(s)
    assert np.all(m == 0.5) and np.all(np.frexp(ws)[0] == 0.5)
    assert np.all(s >= s0) and np.all(s < 2 * s0 * (1 + 1e-6))
    assert s[2, 0] == 1.0 and s[3, 0] == 2.0 ** 5
    deq = oracle.e4m3_decode(q) * np.repeat(s, 128, axis=1)
    assert np.all(np.abs(deq - x) <= np.abs(x) * 2.0 ** -4 + np.repeat(s, 128, axis=1) * 2.0 ** -10)
