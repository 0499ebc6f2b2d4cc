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
