"""The allocation-free decode entry point (b200_dsa_forward_bf16_static), for hosts that cannot
call cudaMalloc once running (a memory pool owns the device, or the library is a plugin that is
only given its inputs and outputs).  Its split-KV scratch is an array built into the library.

Checked through the C ABI against the workspace-backed entry point on two calls in a row with
different inputs (the array keeps the first call's contents), plus the size limit.  This file is
named so that pytest collects it last."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _case(rng, Q, H, S, N, dev):
    f = lambda n, s: oracle.bf16_bits(rng.normal(0, s, n).astype(np.float32))
    arrs = [f(Q * H * 512, 1.0).reshape(Q, H, 512), f(Q * H * 64, 1.0).reshape(Q, H, 64), f(N * 512, 0.5).reshape(N, 512),
            f(N * 64, 0.5).reshape(N, 64), f(N * 512, 0.5).reshape(N, 512)]
    idx = np.stack([rng.permutation(N)[:S] for _ in range(Q)]).astype(np.int32)
    dev_arrs = [torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16) for a in arrs]
    return arrs, idx, dev_arrs, torch.from_numpy(idx).to(dev)


def test_static_scratch_entry_matches_workspace_entry(b200, cuda):
    L = b200.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(2024)
    Q, H, S, N = 3, 128, 1024, 4096                    # 16-way split on a 148-SM part: 12.6 MB of partials
    cfg = b200.DsaConfig(Q, H, 512, 64, S, 64, N)
    status = torch.full((1,), 7, dtype=torch.int32, device=cuda)
    for call in range(2):
        arrs, idx, d, didx = _case(rng, Q, H, S, N, cuda)
        ref_out = torch.empty((Q, H, 512), dtype=torch.float32, device=cuda)
        b200.dsa_forward_bf16(*d, didx, ref_out, cfg)
        out = torch.full((Q, H, 512), float("nan"), dtype=torch.float32, device=cuda)
        st = L.b200_dsa_forward_bf16_static(*(C.c_void_p(t.data_ptr()) for t in d), C.c_void_p(didx.data_ptr()),
                                            C.c_void_p(out.data_ptr()), C.byref(cfg), C.c_void_p(status.data_ptr()),
                                            stream)
        assert st == 0, L.b200_last_error_string()
        torch.cuda.synchronize()
        assert int(status.item()) == 0                  # cleared by the call, no device-side wait ran out
        got, want = out.cpu().numpy(), ref_out.cpu().numpy()
        # the two entry points may run different kernels (CTA-pair vs single-CTA): same tolerance as the decode tests
        assert np.abs(got - want).max() < 1e-2, (call, float(np.abs(got - want).max()))
        oracle_out = oracle.dsa_forward_bf16(*arrs, idx)
        assert np.abs(got - oracle_out).max() < 1e-2    # the tolerance the bf16 decode tests use


def test_static_scratch_limit_is_enforced(b200, cuda):
    L = b200.lib()
    rng = np.random.default_rng(7)
    Q, H, S, N = 4, 128, 2048, 4096                    # 4 queries x 16 splits: 16.8 MB > the 16 MiB array
    _, _, d, didx = _case(rng, Q, H, S, N, cuda)
    out = torch.empty((Q, H, 512), dtype=torch.float32, device=cuda)
    cfg = b200.DsaConfig(Q, H, 512, 64, S, 64, N)
    with pytest.raises(b200.B200Error) as ei:
        b200.dsa_forward_bf16_static(*d, didx, out, cfg)
    assert ei.value.status == b200.B200_UNSUPPORTED and "scratch" in str(ei.value)
    # a single-split shape needs no scratch and is accepted whatever its size
    Q2 = 80
    _, _, d2, didx2 = _case(rng, Q2, H, 64, 512, cuda)
    out2 = torch.empty((Q2, H, 512), dtype=torch.float32, device=cuda)
    ref2 = torch.empty_like(out2)
    cfg2 = b200.DsaConfig(Q2, H, 512, 64, 64, 64, 512)
    b200.dsa_forward_bf16_static(*d2, didx2, out2, cfg2)
    b200.dsa_forward_bf16(*d2, didx2, ref2, cfg2)
    torch.cuda.synchronize()
    assert float((out2 - ref2).abs().max()) < 1e-2
