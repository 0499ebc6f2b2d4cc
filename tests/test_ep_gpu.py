"""Expert-parallel layer on the GPU with a one-rank NCCL group: dispatch, local grouped GEMMs
(K slots per received token) and combine must reproduce the plain single-GPU layer."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist

import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("combine_dtype", [torch.float32, torch.bfloat16])
def test_ep_world1_matches_plain_layer(b200, cuda, combine_dtype):
    rng = np.random.default_rng(11)
    T, E, K, D, I = 96, 16, 4, 512, 256
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    xq, xs = oracle.quant_act(x)
    w1q, w1s = oracle.quant_weight(rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32))
    w2q, w2s = oracle.quant_weight(rng.normal(0, 0.05, (E, D, I)).astype(np.float32))
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    layer = b200.MoeFp8Layer(to(wg), to(bias), to(w1q), to(w1s), to(w2q), to(w2s), K, b200.SCORE_SIGMOID_GROUPED, 4, 2,
                             2.5)
    dxq, dxs = to(xq), to(xs)
    plain = layer.forward(dxq, dxs).cpu().numpy()
    created = False
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", str(29600 + os.getpid() % 300))
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=cuda)
        created = True
    try:
        ep = b200.ExpertParallelMoe(dist.group.WORLD, E, K, layer.route, layer.local_experts,
                                    combine_dtype=combine_dtype)
        out, ids, wts = ep.forward(dxq, dxs)
        torch.cuda.synchronize()
        assert b200.device_status() == 0
        oi, ow = oracle.route_grouped(xq, xs, wg, bias, K, 4, 2, 2.5)
        assert np.array_equal(ids.cpu().numpy(), oi)
        assert ep.last_stats["recv_rows"] == T and ep.recv_pairs() == T * K
        got = out.cpu().numpy()
        if combine_dtype == torch.float32:
            assert np.allclose(got, plain, rtol=1e-4, atol=1e-5)      # same kernels, other summation order
        else:
            assert np.allclose(got, plain, rtol=2.0 ** -8, atol=1e-5)  # partial rows travel as bf16
        ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, oi, ow, np.arange(T, dtype=np.int32))
        assert not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()
    finally:
        if created:
            dist.destroy_process_group()


@pytest.mark.parametrize("strided", [False, True, "mapped"])
@pytest.mark.parametrize("T,K,E,W", [(37, 2, 8, 2), (300, 8, 64, 8), (1500, 4, 48, 4), (5, 3, 6, 1)])
def test_ep_plan_kernel_matches_host_plan(b200, cuda, T, K, E, W, strided):
    """The dispatch-plan kernel and the torch plan used on CPU produce the same rows, bit for bit."""
    rng = np.random.default_rng(T + K)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    wts = rng.uniform(0.1, 1, (T, K)).astype(np.float32)
    epr = E // W
    maps = None
    if strided == "mapped":
        maps = b200.balanced_placement(rng.integers(0, 1000, E), W)
        strided = False
    tok, rank, counts = b200.dispatch_plan(torch.from_numpy(ids), epr, W, strided, maps)
    d_ids, d_w = torch.from_numpy(ids).to(cuda), torch.from_numpy(wts).to(cuda)
    send_tok = torch.full((W * T,), -7, dtype=torch.int32, device=cuda)
    pos = torch.full((W, T), -7, dtype=torch.int32, device=cuda)
    cnt = torch.zeros((W,), dtype=torch.int32, device=cuda)
    sid = torch.full((W * T, K), -7, dtype=torch.int32, device=cuda)
    sw = torch.full((W * T, K), -7.0, dtype=torch.float32, device=cuda)
    b200.ep_plan(d_ids, d_w, epr, W, send_tok, pos, cnt, sid, sw, strided=strided,
                 owner_map=None if maps is None else maps[0].to(cuda), local_map=None if maps is None else maps[1].to(cuda))
    torch.cuda.synchronize()
    assert cnt.cpu().tolist() == counts.tolist()
    Rs = int(counts.sum())
    assert send_tok[:Rs].cpu().tolist() == tok.tolist()
    row_ids = ids[tok.numpy()]
    owner, local = b200.expert_owner(torch.from_numpy(row_ids), epr, W, strided, maps)
    mine = owner.numpy() == rank.numpy()[:, None]
    assert np.array_equal(sid[:Rs].cpu().numpy(), np.where(mine, local.numpy(), -1))
    assert np.array_equal(sw[:Rs].cpu().numpy(), np.where(mine, wts[tok.numpy()], 0.0).astype(np.float32))
    want_pos = np.full((W, T), -1, dtype=np.int32)
    want_pos[rank.numpy(), tok.numpy()] = np.arange(Rs)
    assert np.array_equal(pos.cpu().numpy(), want_pos)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ep_sum_rows_kernel(b200, cuda, dtype):
    rng = np.random.default_rng(5)
    W, T, D = 3, 41, 512
    need = rng.random((W, T)) < 0.6
    Rs = int(need.sum())
    pos = np.full((W, T), -1, dtype=np.int32)
    pos[need] = np.arange(Rs)
    back = torch.from_numpy(rng.normal(0, 1, (Rs, D)).astype(np.float32)).to(dtype)
    out = torch.full((T, D), 9.0, dtype=torch.float32, device=cuda)
    b200.ep_sum_rows(back.to(cuda), torch.from_numpy(pos).to(cuda), W, out)
    want = np.zeros((T, D), dtype=np.float32)
    b32 = back.to(torch.float32).numpy()
    for r in range(W):                      # rank order, fp32 accumulation: bit-exact
        for t in range(T):
            if pos[r, t] >= 0:
                want[t] += b32[pos[r, t]]
    assert np.array_equal(out.cpu().numpy(), want)


def _small_layer(b200, cuda, rng, T, E, K, D, I, ng, tg, pow2=False):
    import contextlib
    x = rng.normal(0, 1, (T, D)).astype(np.float32)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    with (oracle.pow2_scales() if pow2 else contextlib.nullcontext()):
        xq, xs = oracle.quant_act(x)
        w1q, w1s = oracle.quant_weight(rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32))
        w2q, w2s = oracle.quant_weight(rng.normal(0, 0.05, (E, D, I)).astype(np.float32))
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    layer = b200.MoeFp8Layer(to(wg), to(bias), to(w1q), to(w1s), to(w2q), to(w2s), K, b200.SCORE_SIGMOID_GROUPED, ng, tg,
                             2.5, flags=b200.MOE_POW2_SCALES if pow2 else 0)
    return layer, (xq, xs, wg, bias, w1q, w1s, w2q, w2s), to


@pytest.mark.parametrize("pow2", [False, True])
@pytest.mark.parametrize("combine_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("packed", [False, True])
def test_peer_ep_world1_matches_plain_layer_and_oracle(b200, cuda, combine_dtype, packed, pow2):
    """The C-ABI expert-parallel object with one rank: dispatch into its own receive region, grouped GEMMs
    on the region, push and combine; several steps in a row with different token counts (the flag words
    carry the step number, buffers are reused)."""
    rng = np.random.default_rng(17)
    T, E, K, D, I = 96, 16, 4, 512, 256
    layer, (xq, xs, wg, bias, w1q, w1s, w2q, w2s), to = _small_layer(b200, cuda, rng, T, E, K, D, I, 4, 2, pow2)
    if packed:
        layer.pack()
    ep = b200.PeerExpertParallelMoe(None, layer, E, max_tokens=T, combine_dtype=combine_dtype)
    try:
        for Ts in (T, 40, T):
            dxq, dxs = to(xq[:Ts]), to(xs[:Ts])
            plain = layer.forward(dxq, dxs).cpu().numpy()
            out, ids, wts = ep.forward(dxq, dxs)
            status, sent, recv = ep.stats()
            assert status == 0 and sent == [Ts] and recv == [Ts]
            oi, ow = oracle.route_grouped(xq[:Ts], xs[:Ts], wg, bias, K, 4, 2, 2.5)
            assert np.array_equal(ids.cpu().numpy(), oi)
            assert np.abs(wts.cpu().numpy() - ow).max() <= 5e-7
            got = out.cpu().numpy()
            tol = 1e-4 if combine_dtype == torch.float32 else 2.0 ** -10
            assert np.allclose(got, plain, rtol=tol, atol=tol * np.abs(plain).max())   # fp16 is relative to the row maximum
            import contextlib
            with (oracle.pow2_scales() if pow2 else contextlib.nullcontext()):      # the emulation's requantisation rule
                ref = oracle.moe_fp8_experts(xq[:Ts], xs[:Ts], w1q, w1s, w2q, w2s, oi, ow, np.arange(Ts, dtype=np.int32))
            assert not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()
    finally:
        ep.close()
    assert b200.device_status() == 0


def test_peer_ep_absent_rank_times_out_without_hanging(b200, cuda):
    """Rank 0 of a two-rank layer whose peer never shows up (its exchange buffer is mapped onto this
    rank's own, so every access stays in bounds): the words of rank 1 never arrive, the bounded waits of
    the owner side and of the combine run out after wait_limit_ms, the step returns and reports
    B200_TIMEOUT; the next ordinary call works."""
    import time
    rng = np.random.default_rng(23)
    T, E, K, D, I = 64, 16, 4, 512, 256
    layer, (xq, xs, *_), to = _small_layer(b200, cuda, rng, T, E, K, D, I, 4, 2)
    half = b200.MoeFp8Layer(layer.gate_w, layer.bias, layer.w1q[: E // 2].contiguous(), layer.w1s[: E // 2].contiguous(),
                            layer.w2q[: E // 2].contiguous(), layer.w2s[: E // 2].contiguous(), K,
                            b200.SCORE_SIGMOID_GROUPED, 4, 2, 2.5)
    ep = b200.PeerExpertParallelMoe(None, half, E, max_tokens=T, wait_limit_ms=20, loopback=True)
    try:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ep.forward(to(xq), to(xs))
        status, sent, recv = ep.stats()
        wall = time.perf_counter() - t0
        assert status == b200.B200_TIMEOUT
        assert recv[1] == 0 and sum(sent) >= T            # nothing came from the absent rank
        assert wall < 5.0, wall
        assert ep.stats()[0] == 0                          # the read cleared the word
    finally:
        ep.close()
    out = layer.forward(to(xq), to(xs))                    # the context is intact
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and b200.device_status() == 0
