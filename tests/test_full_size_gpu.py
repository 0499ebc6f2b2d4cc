"""The benchmark's full-size workloads (FP8 MoE layer D=7168 I=2048 E=256 top-8; bf16 decode B=64 H=128
top-2048 over a multi-GB paged cache) checked on the GPU through properties that do not depend on the size:
a token's output does not depend on the rest of its batch, the output scales with the routed scaling
factor, a query's output does not depend on the order of its selected rows or on the other queries; plus the
CPU oracle on sampled tokens for the token counts the workload is swept over (1, 16, 128, 1024, 4096)."""
import os
import sys

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402  (workload builders of the benchmark: synthetic weights, caches and index sets)


@pytest.fixture(scope="module")
def moe_full(b200, cuda):
    need = 40 << 30
    if torch.cuda.get_device_properties(cuda).total_memory < need:
        pytest.skip("needs a 40 GB+ device")
    layer, xq, xs = bench.build_moe(b200, torch, cuda, 1, 0)
    yield layer, xq, xs
    del layer, xq, xs
    torch.cuda.empty_cache()


@pytest.mark.parametrize("T", [1, 16, 128, 1024, 4096])
def test_moe_full_shape_token_sweep_against_oracle(b200, cuda, moe_full, T):
    """Config-3 shape at the swept token counts: ids bit-exact, outputs within the FP8 tolerance on up
    to 16 sampled tokens (all of them for T <= 16)."""
    layer, xq, xs = moe_full
    out = layer.forward(xq[:T].contiguous(), xs[:T].contiguous())
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    c = bench.MOE
    old_T = c["T"]
    try:
        c["T"] = T
        res = bench.moe_cpu_sample(b200, torch, oracle, layer, xq[:T].contiguous(), xs[:T].contiguous(), out,
                                   min(T, 16), oracle.host_threads())
    finally:
        c["T"] = old_T
    ids_dev, _ = layer.route(xq[:T].contiguous(), xs[:T].contiguous())
    assert np.array_equal(ids_dev.cpu().numpy()[res["toks"]], res["ids"])
    assert res["ok"], res["max_abs_err"]


def test_moe_full_size_batch_independence_and_scaling(b200, cuda, moe_full):
    layer, xq, xs = moe_full
    T = xq.shape[0]
    full = layer.forward(xq, xs).clone()
    sub = torch.arange(5, T, 97, device=cuda)                     # 43 tokens spread over the batch
    part = layer.forward(xq.index_select(0, sub), xs.index_select(0, sub))
    ref = full.index_select(0, sub)
    # same per-row arithmetic; only the order of the eight scatter-adds per element may differ
    assert torch.allclose(part, ref, rtol=1e-4, atol=1e-4)
    # doubling the routed scaling factor doubles every router weight exactly, hence every output
    saved = layer.routed_scale
    try:
        layer.routed_scale = 2 * saved
        twice = layer.forward(xq.index_select(0, sub), xs.index_select(0, sub))
    finally:
        layer.routed_scale = saved
    assert torch.allclose(twice, 2 * part, rtol=1e-4, atol=1e-4)
    # row counts of the permutation add up and the expert histogram matches the ids
    ids, wts = layer.route(xq, xs)
    assert int(torch.bincount(ids.reshape(-1).long(), minlength=layer.E).sum()) == T * layer.K
    assert bool((ids.sort(dim=1).values.diff(dim=1) != 0).all())   # no expert twice in a token
    assert torch.allclose(wts.sum(1), torch.full((T,), saved, device=cuda), rtol=1e-5)
    assert b200.device_status() == 0


def test_dsa_full_size_order_and_batch_independence(b200, cuda):
    if torch.cuda.get_device_properties(cuda).total_memory < (40 << 30):
        pytest.skip("needs a 40 GB+ device")
    layer, qn, qp, idx_sets, N, seq = bench.build_dsa(b200, torch, cuda, 77)
    idx = idx_sets[0]
    out = layer.forward(qn, qp, idx).clone()
    assert bool(torch.isfinite(out).all())
    # the selected rows are a set: any order gives the same softmax-weighted sum
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    perm = torch.stack([torch.randperm(idx.shape[1], generator=g, device=cuda) for _ in range(idx.shape[0])])
    shuffled = torch.gather(idx, 1, perm).contiguous()
    out2 = layer.forward(qn, qp, shuffled)
    assert torch.allclose(out, out2, rtol=0, atol=2e-3)
    # a query's output does not depend on its neighbours in the batch (other grid shape, split-KV path)
    few = layer.forward(qn[3:8].contiguous(), qp[3:8].contiguous(), idx[3:8].contiguous())
    assert torch.allclose(out[3:8], few, rtol=0, atol=2e-3)
    # softmax weights are a convex combination: every output lies inside the range of the selected V rows
    rows = layer.v[idx[0].long()].float()                          # [S, Dc]
    lo, hi = rows.min(0).values, rows.max(0).values
    assert bool(((out[0] >= lo - 1e-2) & (out[0] <= hi + 1e-2)).all())
    assert b200.device_status() == 0
    del layer
    torch.cuda.empty_cache()
