"""Expert-parallel plumbing on CPU: two gloo ranks, oracle-backed routing/expert functions.
The two ranks together must reproduce the single-rank layer on the concatenated tokens."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T, E, K, D, I = 24, 8, 2, 256, 128
BALANCE_COUNTS = [9, 1, 7, 3, 2, 8, 4, 6]       # calibration loads for the balanced-placement case


def _make(seed):
    rng = np.random.default_rng(seed)
    return rng


def _weights():
    import oracle
    rng = np.random.default_rng(100)
    wg = rng.normal(0, 1 / 16, (E, D)).astype(np.float32)
    bias = rng.normal(0, 0.01, E).astype(np.float32)
    w1q, w1s = oracle.quant_weight(rng.normal(0, 0.05, (E, 2 * I, D)).astype(np.float32))
    w2q, w2s = oracle.quant_weight(rng.normal(0, 0.05, (E, D, I)).astype(np.float32))
    return wg, bias, w1q, w1s, w2q, w2s


def _tokens(rank):
    import oracle
    rng = np.random.default_rng(200 + rank)
    return oracle.quant_act(rng.normal(0, 1, (T, D)).astype(np.float32))


def _worker(rank, world, port, ret, placement):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle
    from conftest import load_package
    b200 = load_package()
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    wg, bias, w1q, w1s, w2q, w2s = _weights()
    El = E // world
    if placement == "balanced":
        maps = b200.balanced_placement(np.array(BALANCE_COUNTS), world)
        mine = np.zeros(El, dtype=np.int64)
        for e in range(E):
            if int(maps[0][e]) == rank:
                mine[int(maps[1][e])] = e
        placement = maps
    else:
        mine = slice(rank * El, (rank + 1) * El) if placement == "contiguous" else slice(rank, E, world)

    def route_fn(xq, xs):
        ids, wts = oracle.route_grouped(xq.numpy(), xs.numpy(), wg, bias, K, 4, 2, 2.5)
        return torch.from_numpy(ids), torch.from_numpy(wts)

    def expert_fn(rq, rs, rid, rw):
        R = rq.shape[0]
        ids = rid.numpy().astype(np.int32)
        w = rw.numpy().astype(np.float32)
        valid = ids >= 0
        # slots owned by other ranks: any local expert with weight zero contributes nothing
        ids = np.where(valid, ids, 0).astype(np.int32)
        w = np.where(valid, w, 0.0).astype(np.float32)
        y = oracle.moe_fp8_experts(rq.numpy(), rs.numpy(), np.ascontiguousarray(w1q[mine]), np.ascontiguousarray(w1s[mine]),
                                   np.ascontiguousarray(w2q[mine]), np.ascontiguousarray(w2s[mine]), ids, w, np.arange(R, dtype=np.int32))
        return torch.from_numpy(y)

    ep = b200.ExpertParallelMoe(dist.group.WORLD, E, K, route_fn, expert_fn, placement=placement)
    xq, xs = _tokens(rank)
    out, ids, wts = ep.forward(torch.from_numpy(xq), torch.from_numpy(xs))
    ret[rank] = (out.numpy(), ids.numpy(), ep.recv_pairs(), ep.last_stats["recv_rows"])
    dist.barrier()
    dist.destroy_process_group()


def test_dispatch_plan(b200):
    ids = torch.tensor([[0, 5], [7, 6], [1, 2]], dtype=torch.int32)
    tok, rank, counts = b200.dispatch_plan(ids, 4, 2)
    assert counts.tolist() == [2, 2]                  # token 0 -> both ranks, token 1 -> rank 1, token 2 -> rank 0
    assert tok.tolist() == [0, 2, 0, 1]               # grouped by rank, ascending in token
    assert rank.tolist() == [0, 0, 1, 1]
    tok, rank, counts = b200.dispatch_plan(ids, 4, 2, strided=True)      # even experts on rank 0, odd on rank 1
    assert counts.tolist() == [3, 3]
    assert tok.tolist() == [0, 1, 2, 0, 1, 2]
    owner, local = b200.expert_owner(ids, 4, 2, strided=True)
    assert owner.tolist() == [[0, 1], [1, 0], [1, 0]] and local.tolist() == [[0, 2], [3, 3], [0, 1]]


def test_balanced_placement():
    import torch
    from conftest import load_package
    b200 = load_package()
    counts = [100, 1, 1, 1, 50, 50, 2, 3]
    owner, local = b200.balanced_placement(counts, 2)
    assert sorted(owner.tolist()) == [0] * 4 + [1] * 4                  # equal number of experts per rank
    for g in range(2):
        assert sorted(local[owner == g].tolist()) == [0, 1, 2, 3]       # local ids are a permutation
    load = [sum(c for c, o in zip(counts, owner.tolist()) if o == g) for g in range(2)]
    assert max(load) <= 105                                             # of 208 rows: the hot expert does not share with the next two
    o2, l2 = b200.expert_owner(torch.tensor([[0, 4]]), 4, 2, maps=(owner, local))
    assert o2.tolist() == [[int(owner[0]), int(owner[4])]] and l2.tolist() == [[int(local[0]), int(local[4])]]


@pytest.mark.parametrize("placement", ["contiguous", "strided", "balanced"])
def test_two_rank_ep_matches_single_rank(placement):
    import oracle
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + os.getpid() % 2000 + {"contiguous": 0, "strided": 7, "balanced": 13}[placement]
    mp.spawn(_worker, args=(world, port, ret, placement), nprocs=world, join=True)
    wg, bias, w1q, w1s, w2q, w2s = _weights()
    total_recv = 0
    for rank in range(world):
        xq, xs = _tokens(rank)
        ids, wts = oracle.route_grouped(xq, xs, wg, bias, K, 4, 2, 2.5)
        ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, ids, wts, np.arange(T, dtype=np.int32))
        out, got_ids, pairs, rows = ret[rank]
        assert np.array_equal(got_ids, ids)
        assert np.allclose(out, ref, rtol=1e-5, atol=1e-6)      # only the summation order over slots differs
        assert rows <= world * T                                # a token goes to a rank at most once
        total_recv += pairs
    assert total_recv == world * T * K
