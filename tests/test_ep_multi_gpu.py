"""Expert-parallel layer on two real GPUs (NCCL): every rank's output must match the CPU oracle of the
unsharded layer on its own tokens, for the three expert placements.  Skipped on a single-GPU machine
(the two-rank plumbing is then covered by the gloo test on CPU and the kernels by the one-rank GPU test)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T, E, K, D, I = 96, 16, 4, 512, 256


def _weights():
    import oracle
    rng = np.random.default_rng(100)
    wg = rng.normal(0, D ** -0.5, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    w1q, w1s = oracle.quant_weight(rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32))
    w2q, w2s = oracle.quant_weight(rng.normal(0, 0.05, (E, D, I)).astype(np.float32))
    return wg, bias, w1q, w1s, w2q, w2s


def _tokens(rank):
    import oracle
    rng = np.random.default_rng(200 + rank)
    return oracle.quant_act(rng.normal(0, 1, (T, D)).astype(np.float32))


def _worker(rank, world, port, placement_name, combine_bf16, ret, impl="nccl"):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from conftest import load_package
    b200 = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        wg, bias, w1q, w1s, w2q, w2s = _weights()
        El = E // world
        if placement_name == "balanced":
            placement = b200.balanced_placement(np.arange(E)[::-1].copy(), world)
            mine = np.zeros(El, dtype=np.int64)
            for e in range(E):
                if int(placement[0][e]) == rank:
                    mine[int(placement[1][e])] = e
        elif placement_name == "strided":
            placement, mine = "strided", np.arange(rank, E, world)
        else:
            placement, mine = "contiguous", np.arange(rank * El, (rank + 1) * El)
        to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        layer = b200.MoeFp8Layer(to(wg), to(bias), to(w1q[mine]), to(w1s[mine]), to(w2q[mine]), to(w2s[mine]), K,
                                 b200.SCORE_SIGMOID_GROUPED, 4, 2, 2.5)
        # 16-bit combine: bf16 rows for the torch.distributed path, row-scaled fp16 rows for the C-ABI object
        cdt = (torch.float16 if impl == "peer" else torch.bfloat16) if combine_bf16 else torch.float32
        xq, xs = _tokens(rank)
        if impl == "peer":
            # the C-ABI object: peer-store data plane, no collective inside a step; three steps in a row
            if placement == "strided":
                placement = (torch.arange(E, dtype=torch.int32) % world, torch.arange(E, dtype=torch.int32) // world)
            ep = b200.PeerExpertParallelMoe(dist.group.WORLD, layer, E, max_tokens=T, placement=placement,
                                            combine_dtype=cdt, wait_limit_ms=5000)
            for _ in range(3):
                out, ids, wts = ep.forward(to(xq), to(xs))
            status, sent, recv = ep.stats()
            status |= b200.device_status()
        else:
            ep = b200.ExpertParallelMoe(dist.group.WORLD, E, K, layer.route, layer.local_experts, placement=placement,
                                        combine_dtype=cdt)
            out, ids, wts = ep.forward(to(xq), to(xs))
            torch.cuda.synchronize()
            status = b200.device_status()
        oi, ow = oracle.route_grouped(xq, xs, wg, bias, K, 4, 2, 2.5)
        ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, oi, ow, np.arange(T, dtype=np.int32))
        got = out.cpu().numpy()
        if impl == "peer":
            # pairs computed on this rank = (token, expert) pairs of ALL ranks whose expert lives here
            mine_set = set(int(e) for e in mine)
            pairs = 0
            for r in range(world):
                tq, ts = _tokens(r)
                ri, _ = oracle.route_grouped(tq, ts, wg, bias, K, 4, 2, 2.5)
                pairs += int(np.isin(ri, list(mine_set)).sum())
            recv_rows_ok = sum(recv) > 0
            ret[rank] = (status, bool(np.array_equal(ids.cpu().numpy(), oi)),
                         bool(recv_rows_ok and not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()), pairs)
            dist.barrier()
            ep.close()
        else:
            ret[rank] = (status, bool(np.array_equal(ids.cpu().numpy(), oi)),
                         bool(not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()), ep.recv_pairs())
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("combine_bf16", [False, True])
@pytest.mark.parametrize("placement", ["contiguous", "strided", "balanced"])
def test_two_gpu_ep_matches_oracle(placement, combine_bf16):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29700 + os.getpid() % 200 + {"contiguous": 0, "strided": 3, "balanced": 6}[placement] + int(combine_bf16)
    mp.spawn(_worker, args=(world, port, placement, combine_bf16, ret), nprocs=world, join=True)
    pairs = 0
    for rank in range(world):
        status, ids_ok, out_ok, recv = ret[rank]
        assert status == 0
        assert ids_ok and out_ok
        pairs += recv
    assert pairs == world * T * K


@pytest.mark.parametrize("combine_bf16", [False, True])
@pytest.mark.parametrize("placement", ["contiguous", "strided", "balanced"])
def test_two_gpu_peer_ep_matches_oracle(placement, combine_bf16):
    """Same check for the C-ABI expert-parallel object (rows and partial rows travel by peer stores into
    mapped exchange buffers; flag words instead of collectives)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29950 + os.getpid() % 40 + {"contiguous": 0, "strided": 3, "balanced": 6}[placement] + int(combine_bf16)
    mp.spawn(_worker, args=(world, port, placement, combine_bf16, ret, "peer"), nprocs=world, join=True)
    pairs = 0
    for rank in range(world):
        status, ids_ok, out_ok, recv = ret[rank]
        assert status == 0
        assert ids_ok and out_ok
        pairs += recv
    assert pairs == world * T * K
