"""Expert-parallel layer on the GPU with a one-rank NCCL group: dispatch, local grouped GEMMs
(one slot per received row) and combine must reproduce the plain single-GPU layer."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist

import oracle

pytestmark = pytest.mark.gpu


def test_ep_world1_matches_plain_layer(b200, cuda):
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
        ep = b200.ExpertParallelMoe(dist.group.WORLD, E, K, layer.route, layer.local_experts)
        out, ids, wts = ep.forward(dxq, dxs)
        torch.cuda.synchronize()
        assert b200.device_status() == 0
        oi, ow = oracle.route_grouped(xq, xs, wg, bias, K, 4, 2, 2.5)
        assert np.array_equal(ids.cpu().numpy(), oi)
        assert ep.last_stats["recv_rows"] == T * K
        got = out.cpu().numpy()
        assert np.allclose(got, plain, rtol=1e-4, atol=1e-5)          # same kernels, other summation order
        ref = oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, oi, ow, np.arange(T, dtype=np.int32))
        assert not (np.abs(got - ref) > 1e-2 + 2e-2 * np.abs(ref)).any()
    finally:
        if created:
            dist.destroy_process_group()
