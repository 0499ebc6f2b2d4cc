"""Router of the FP8 layer on the tensor cores: the logits are approximate (tf32 split operands, the tensor core's
own summation order), the routing is not: a token's ids are accepted only when every decision margin is far larger
than the approximation error, and the remaining tokens are recomputed with the fixed-order FMA chains.  Checked
against the CPU oracle: ids and histogram bit-exact for every token, weights to 2e-5, including inputs built to
sit on decision boundaries."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _route(b200, cuda, xq, xs, wg, bias, K, ng, tg, flags=0):
    T, D = xq.shape
    E = wg.shape[0]
    cfg = b200.MoeFp8Config(T, E, K, D, 128, b200.SCORE_SIGMOID_GROUPED, ng, tg, 2.5, flags)
    ids = torch.full((T, K), -9, dtype=torch.int32, device=cuda)
    wts = torch.zeros((T, K), dtype=torch.float32, device=cuda)
    counts = torch.zeros(E, dtype=torch.int32, device=cuda)
    b200.moe_route_fp8(_dev(xq, cuda), _dev(xs, cuda), _dev(wg, cuda), _dev(bias, cuda), ids, wts, cfg, counts=counts)
    flagged = b200.moe_route_last_flagged()
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    return ids.cpu().numpy(), wts.cpu().numpy(), counts.cpu().numpy(), flagged


def test_tc_logits_stay_within_the_assumed_error(b200, cuda):
    """The certification threshold assumes |approximate - exact logit| <= 2^-14 per unit of logit rms; measured
    here on the router's real shape (E = 256, D = 7168, unit-variance logits) it has to stay below half of that.
    The tensor core truncates when it adds into its accumulator, so the error grows with the chain: one chain over
    all of D is several times worse than the library's chains of four 128-deep blocks."""
    rng = np.random.default_rng(0)
    T, E, D = 512, 256, 7168
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    xq, xs = oracle.quant_act(x)
    ref = oracle.gate_logits_fp8(xq, xs, wg)
    got = b200.moe_gate_logits_tc(_dev(xq, cuda), _dev(xs, cuda), _dev(wg, cuda)).cpu().numpy()
    one = b200.moe_gate_logits_tc(_dev(xq, cuda), _dev(xs, cuda), _dev(wg, cuda), chain_blocks=D // 128).cpu().numpy()
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    err, err_one = np.abs(got - ref).max(), np.abs(one - ref).max()
    print("max |tc - exact| =", err, " one chain:", err_one, " logits rms", ref.std())
    assert err < 2.0 ** -15, err
    assert err_one < 1e-3 and err_one > err


@pytest.mark.parametrize("T,E,K,D,ng,tg", [(512, 256, 8, 7168, 8, 4), (300, 64, 4, 1024, 4, 2), (1024, 128, 6, 2048, 8, 3)])
def test_tc_routing_ids_bit_exact(b200, cuda, T, E, K, D, ng, tg):
    rng = np.random.default_rng(T + E)
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    xq, xs = oracle.quant_act(x)
    ids, wts, counts, flagged = _route(b200, cuda, xq, xs, wg, bias, K, ng, tg)
    oi, ow = oracle.route_grouped(xq, xs, wg, bias, K, ng, tg, 2.5)
    assert 0 <= flagged < T // 2, flagged                 # the tensor-core path ran, and most tokens were certified
    assert np.array_equal(ids, oi)
    assert np.abs(wts - ow).max() <= 2e-5
    assert np.array_equal(counts, np.bincount(oi.reshape(-1), minlength=E))
    # the exact path on request: weights to the last ulps, as for small batches
    ids2, wts2, counts2, flagged2 = _route(b200, cuda, xq, xs, wg, bias, K, ng, tg, b200.MOE_EXACT_ROUTER_LOGITS)
    assert flagged2 == -1
    assert np.array_equal(ids2, oi) and np.abs(wts2 - ow).max() <= 5e-7 and np.array_equal(counts2, counts)


def test_tc_routing_on_decision_boundaries(b200, cuda):
    """Experts that tie exactly (identical gate rows and biases: the lowest index must win), experts one ulp of a
    weight apart, and a bias vector that makes whole groups tie: every such token has to come out as the oracle
    says, whether the certification accepts it or sends it to the exact pass."""
    rng = np.random.default_rng(7)
    T, E, K, D, ng, tg = 512, 256, 8, 2048, 8, 4
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = np.zeros(E, np.float32)
    for a, b in ((5, 6), (40, 41), (100, 131), (200, 250)):       # exact duplicates, inside and across groups
        wg[b] = wg[a]
    for a, b in ((10, 11), (70, 90), (160, 161)):                 # one ulp apart in one weight
        wg[b] = wg[a]
        j = int(rng.integers(0, D))
        wg[b, j] = np.nextafter(wg[b, j], np.float32(1.0))
    wg[32:64] = wg[0:32]                                          # group 1 ties with group 0 as a whole
    xq, xs = oracle.quant_act(x)
    ids, wts, counts, flagged = _route(b200, cuda, xq, xs, wg, bias, K, ng, tg)
    oi, ow = oracle.route_grouped(xq, xs, wg, bias, K, ng, tg, 2.5)
    assert flagged > 0                                            # ties cannot be certified
    assert np.array_equal(ids, oi)
    assert np.abs(wts - ow).max() <= 2e-5
    assert np.array_equal(counts, np.bincount(oi.reshape(-1), minlength=E))


def test_fp8_layer_with_tc_router_against_emulation(b200, cuda):
    """The whole layer at a batch size that takes the tensor-core router."""
    rng = np.random.default_rng(11)
    T, E, K, D, I = 384, 32, 4, 1024, 256
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    xq, xs = oracle.quant_act(x)
    w1q, w1s = oracle.quant_weight(rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32))
    w2q, w2s = oracle.quant_weight(rng.normal(0, 0.05, (E, D, I)).astype(np.float32))
    cfg = b200.MoeFp8Config(T, E, K, D, I, b200.SCORE_SIGMOID_GROUPED, 4, 2, 2.5)
    out = torch.full((T, D), float("nan"), dtype=torch.float32, device=cuda)
    b200.moe_fp8_forward(_dev(xq, cuda), _dev(xs, cuda), _dev(wg, cuda), _dev(bias, cuda), _dev(w1q, cuda), _dev(w1s, cuda),
                         _dev(w2q, cuda), _dev(w2s, cuda), out, cfg)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    assert b200.moe_route_last_flagged() >= 0
    ids, wts = oracle.route_grouped(xq, xs, wg, bias, K, 4, 2, 2.5)
    ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, ids, wts, np.arange(T, dtype=np.int32))
    got = out.cpu().numpy()
    assert not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()
