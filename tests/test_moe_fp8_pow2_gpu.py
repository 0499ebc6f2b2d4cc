"""FP8 MoE layer with power-of-two scales (MOE_POW2_SCALES): the grouped GEMMs run on the hardware block-scaled MMA
(tcgen05.mma kind::mxf8f6f4.block_scale), the tensor core applies the scales itself.  Checked through the C ABI:
the MMA with its scale-factor layout on a small matrix, the *_pow2 quantisers bit-exact against the oracle with the
same scale rule, the GEMM1 + SwiGLU + requantise stage, and the whole layer against the fp32 CPU emulation
(2e-2 relative + 1e-2 absolute), row-major and pre-tiled weights, scatter-add and fixed-order combine; a scale that
is not a power of two is reported in the device status word."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 2e-2, 1e-2


def _dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _layer(rng, T, E, D, I, sigma_w=0.05):
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    # block-dependent magnitudes (never above the unit-scale data the tolerance is stated for), so that
    # neighbouring blocks carry different scale exponents
    w1 = (rng.normal(0, sigma_w, (E, 2 * I, D)) * np.exp2(rng.integers(-3, 1, (E, 1, D)))).astype(np.float32)
    w2 = (rng.normal(0, sigma_w, (E, D, I)) * np.exp2(rng.integers(-3, 1, (E, D, 1)))).astype(np.float32)
    x = (x * np.exp2(rng.integers(-3, 1, (T, 1)))).astype(np.float32)
    with oracle.pow2_scales():
        xq, xs = oracle.quant_act(x)
        w1q, w1s = oracle.quant_weight(w1)
        w2q, w2s = oracle.quant_weight(w2)
    return x, wg, bias, w1, w2, xq, xs, w1q, w1s, w2q, w2s


@pytest.mark.parametrize("N,K", [(256, 128), (128, 256), (256, 512)])
def test_block_scaled_mma_selftest(b200, cuda, N, K):
    """d[m, n] = sum_k a[m,k] 2^(sfa[m,k/32]-127) b[n,k] 2^(sfb[n,k/32]-127) with a different scale for every row
    and every 32-deep slice of both operands."""
    rng = np.random.default_rng(N + K)
    a8 = rng.integers(0, 256, (128, K), dtype=np.uint8) & 0xBF
    b8 = rng.integers(0, 256, (N, K), dtype=np.uint8) & 0xBF
    a8[(a8 & 0x7F) == 0x7F] = 0x38
    b8[(b8 & 0x7F) == 0x7F] = 0x38
    sfa = rng.integers(120, 134, (128, K // 32)).astype(np.uint8)
    sfb = rng.integers(120, 134, (N, K // 32)).astype(np.uint8)
    af = oracle.e4m3_decode(a8).astype(np.float64) * np.repeat(2.0 ** (sfa.astype(np.float64) - 127), 32, axis=1)
    bf = oracle.e4m3_decode(b8).astype(np.float64) * np.repeat(2.0 ** (sfb.astype(np.float64) - 127), 32, axis=1)
    ref = af @ bf.T
    d = torch.full((128, N), float("nan"), dtype=torch.float32, device=cuda)
    b200.mx_selftest(_dev(a8, cuda), _dev(b8, cuda), _dev(sfa, cuda), _dev(sfb, cuda), d)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    got = d.cpu().numpy().astype(np.float64)
    assert np.abs(got - ref).max() <= 2e-6 * np.abs(ref).max()


def test_pow2_quantisers_bit_exact(b200, cuda):
    rng = np.random.default_rng(0)
    x = (rng.normal(0, 1, (37, 512)) * np.exp2(rng.integers(-20, 20, (37, 1)))).astype(np.float32)
    x[5, 128:256] = 0
    x[6, 0:128] = 448.0 * 2.0 ** -3          # amax / 448 is a power of two itself
    q = torch.empty((37, 512), dtype=torch.uint8, device=cuda)
    s = torch.empty((37, 4), dtype=torch.float32, device=cuda)
    b200.quant_act_1x128(_dev(x, cuda), q, s, pow2=True)
    with oracle.pow2_scales():
        oq, os_ = oracle.quant_act(x)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), os_)
    m, _ = np.frexp(os_)
    assert np.all(m == 0.5)                   # every scale is a power of two
    assert os_[6, 0] == 2.0 ** -3
    w = rng.normal(0, 0.02, (3, 256, 384)).astype(np.float32)
    wq = torch.empty(w.shape, dtype=torch.uint8, device=cuda)
    ws = torch.empty((3, 2, 3), dtype=torch.float32, device=cuda)
    b200.quant_weight_128x128(_dev(w, cuda), wq, ws, pow2=True)
    with oracle.pow2_scales():
        oq, os_ = oracle.quant_weight(w)
    assert np.array_equal(wq.cpu().numpy(), oq) and np.array_equal(ws.cpu().numpy(), os_)
    rows, cols = 256, 384
    q = torch.empty((rows, cols), dtype=torch.uint8, device=cuda)
    s = torch.empty((rows // 128, cols // 128), dtype=torch.float32, device=cuda)
    b200.fill_normal_fp8_w128_(q, s, 99, 0.02, pow2=True)
    with oracle.pow2_scales():
        oq, os_ = oracle.quant_weight(b200.synth_normal_host(99, 0, rows * cols, 0.02).reshape(rows, cols))
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy(), os_)


def test_gemm1_swiglu_requant_stage_pow2(b200, cuda):
    rng = np.random.default_rng(1)
    T, E, K, D, I = 40, 4, 2, 512, 256
    x, wg, bias, w1, w2, xq, xs, w1q, w1s, w2q, w2s = _layer(rng, T, E, D, I)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    cfg = b200.MoeFp8Config(T, E, K, D, I, b200.SCORE_SIGMOID_GROUPED, 1, 1, 1.0, b200.MOE_POW2_SCALES)
    act_q = torch.empty((T * K, I), dtype=torch.uint8, device=cuda)
    act_s = torch.empty((T * K, I // 128), dtype=torch.float32, device=cuda)
    offs = torch.empty(E + 1, dtype=torch.int32, device=cuda)
    rp = torch.empty(T * K, dtype=torch.int32, device=cuda)
    b200.moe_fp8_gemm1_stage(_dev(xq, cuda), _dev(xs, cuda), _dev(ids, cuda), _dev(w1q, cuda), _dev(w1s, cuda),
                             act_q, act_s, offs, rp, cfg)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    aq, asc, rp = act_q.cpu().numpy(), act_s.cpu().numpy(), rp.cpu().numpy()
    m, _ = np.frexp(asc)
    assert np.all(m == 0.5)
    bad = 0
    with oracle.pow2_scales():
        for r in range(0, T * K, 3):
            t, k = divmod(int(rp[r]), K)
            oq, osc = oracle.moe_fp8_gemm1_row(xq[t], xs[t], w1q[ids[t, k]], w1s[ids[t, k]])
            # a scale may differ by one binade when the block's amax sits on a power-of-two boundary
            assert np.all((asc[r] == osc) | (asc[r] == 2 * osc) | (2 * asc[r] == osc)), (r, asc[r], osc)
            got = oracle.e4m3_decode(aq[r]) * np.repeat(asc[r], 128)
            ref = oracle.e4m3_decode(oq) * np.repeat(osc, 128)
            step = np.maximum(np.abs(ref), np.repeat(np.maximum(osc, asc[r]), 128) * 2.0 ** -6) * 2.0 ** -3
            assert np.all(np.abs(got - ref) <= step * 1.01)
            bad += int((aq[r] != oq).sum())
    assert bad <= 0.02 * (T * K // 3 + 1) * I, bad


@pytest.mark.parametrize("packed", [False, True])
@pytest.mark.parametrize("T,E,K,D,I,ng,tg", [(48, 8, 2, 256, 128, 4, 2), (300, 16, 4, 512, 384, 4, 2),
                                              (1, 8, 2, 256, 128, 4, 2), (700, 4, 2, 768, 256, 1, 1)])
def test_pow2_layer_against_emulation(b200, cuda, T, E, K, D, I, ng, tg, packed):
    rng = np.random.default_rng(T + E + (1 if packed else 0))
    x, wg, bias, w1, w2, xq, xs, w1q, w1s, w2q, w2s = _layer(rng, T, E, D, I)
    d = {k: _dev(v, cuda) for k, v in dict(xq=xq, xs=xs, wg=wg, bias=bias, w1q=w1q, w1s=w1s, w2q=w2q, w2s=w2s).items()}
    w1d, w2d = d["w1q"], d["w2q"]
    fwd = b200.moe_fp8_forward
    if packed:
        w1d, w2d = torch.empty_like(d["w1q"]), torch.empty_like(d["w2q"])
        b200.moe_fp8_pack_weights(1, d["w1q"], w1d, E, D, I)
        b200.moe_fp8_pack_weights(2, d["w2q"], w2d, E, D, I)
        fwd = b200.moe_fp8_forward_packed
    ids, wts = oracle.route_grouped(xq, xs, wg, bias, K, ng, tg, 2.5)
    with oracle.pow2_scales():
        ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, ids, wts, np.arange(T, dtype=np.int32))
    for extra in (0, b200.MOE_DETERMINISTIC):
        cfg = b200.MoeFp8Config(T, E, K, D, I, b200.SCORE_SIGMOID_GROUPED, ng, tg, 2.5, b200.MOE_POW2_SCALES | extra)
        out = torch.full((T, D), float("nan"), dtype=torch.float32, device=cuda)
        fwd(d["xq"], d["xs"], d["wg"], d["bias"], w1d, d["w1s"], w2d, d["w2s"], out, cfg)
        torch.cuda.synchronize()
        assert b200.device_status() == 0
        got = out.cpu().numpy()
        viol = np.abs(got - ref) > ATOL + RTOL * np.abs(ref)
        assert not viol.any(), (packed, extra, int(viol.sum()), float(np.abs(got - ref).max()), float(np.abs(ref).max()))


def test_scale_that_is_no_power_of_two_is_reported(b200, cuda):
    rng = np.random.default_rng(5)
    T, E, K, D, I = 32, 4, 2, 256, 128
    x, wg, bias, w1, w2, xq, xs, w1q, w1s, w2q, w2s = _layer(rng, T, E, D, I)
    w1s = w1s.copy()
    w1s[0, 0, 0] *= 1.5
    cfg = b200.MoeFp8Config(T, E, K, D, I, b200.SCORE_SIGMOID_GROUPED, 1, 1, 2.5, b200.MOE_POW2_SCALES)
    out = torch.empty((T, D), dtype=torch.float32, device=cuda)
    ids = np.stack([np.array([0, 1 + t % 3]) for t in range(T)]).astype(np.int32)       # expert 0 is used
    wts = np.full((T, K), 0.5, np.float32)
    b200.moe_fp8_experts(_dev(xq, cuda), _dev(xs, cuda), _dev(ids, cuda), _dev(wts, cuda), _dev(w1q, cuda),
                         _dev(w1s, cuda), _dev(w2q, cuda), _dev(w2s, cuda), out, cfg)
    torch.cuda.synchronize()
    assert b200.device_status() == b200.BAD_SCALE          # reading the status word clears it
    assert b200.device_status() == 0
