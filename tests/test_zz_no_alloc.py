"""The allocation-free decode entry point (b200_dsa_forward_bf16_static), for hosts that cannot
call cudaMalloc once running (a memory pool owns the device, or the library is a plugin that is
only given its inputs and outputs).  Its split-KV scratch is an array built into the library.

Checked through the C ABI against the workspace-backed entry point on two calls in a row with
different inputs (the array keeps the first call's contents), plus the limits, and that the device's
free memory does not change across a call.  This file is named so that pytest collects it last."""
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


def _call_static(b200, d, didx, out, cfg, status):
    L = b200.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return L.b200_dsa_forward_bf16_static(*(C.c_void_p(t.data_ptr()) for t in d), C.c_void_p(didx.data_ptr()),
                                          C.c_void_p(out.data_ptr()), C.byref(cfg), C.c_void_p(status.data_ptr()),
                                          stream)


@pytest.mark.parametrize("Q,S,N", [(3, 1024, 4096), (1, 2048, 4096), (4, 2048, 4096)])
def test_static_scratch_entry_matches_workspace_entry(b200, cuda, Q, S, N):
    """Two calls in a row with different inputs (the array keeps the first call's contents), each checked
    against the workspace-backed entry point and the CPU oracle.  (1, 2048) and (4, 2048) are small-batch
    decodes at the production top-k, where the row split is cut down to what the built-in array holds
    (63 and 15 ranges instead of 64 and 18)."""
    L = b200.lib()
    rng = np.random.default_rng(2024 + Q)
    H = 128
    cfg = b200.DsaConfig(Q, H, 512, 64, S, 64, N)
    status = torch.full((1,), 7, dtype=torch.int32, device=cuda)
    for call in range(2):
        arrs, idx, d, didx = _case(rng, Q, H, S, N, cuda)
        ref_out = torch.empty((Q, H, 512), dtype=torch.float32, device=cuda)
        b200.dsa_forward_bf16(*d, didx, ref_out, cfg)
        out = torch.full((Q, H, 512), float("nan"), dtype=torch.float32, device=cuda)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        st = _call_static(b200, d, didx, out, cfg, status)
        assert st == 0, L.b200_last_error_string()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # the property the entry point exists for: the call took no device memory (the first call on
        # a device may load the kernel's code, which the driver accounts for outside this figure)
        assert free_after == free_before, (free_before, free_after)
        assert int(status.item()) == 0                  # cleared by the call, no device-side wait ran out
        got, want = out.cpu().numpy(), ref_out.cpu().numpy()
        # the two entry points may run different kernels (CTA-pair vs single-CTA): same tolerance as the decode tests
        assert np.abs(got - want).max() < 1e-2, (call, float(np.abs(got - want).max()))
        oracle_out = oracle.dsa_forward_bf16(*arrs, idx)
        assert np.abs(got - oracle_out).max() < 1e-2    # the tolerance the bf16 decode tests use


def test_static_scratch_limits(b200, cuda):
    L = b200.lib()
    rng = np.random.default_rng(7)
    H = 128
    status = torch.zeros((1,), dtype=torch.int32, device=cuda)
    # more queries than one call takes: rejected before anything is launched or read, with a clear message
    _, _, d, didx = _case(rng, 2, H, 64, 512, cuda)
    out = torch.empty((2, H, 512), dtype=torch.float32, device=cuda)
    with pytest.raises(b200.B200Error) as ei:
        b200.dsa_forward_bf16_static(*d, didx, out, b200.DsaConfig(70000, H, 512, 64, 64, 64, 512), status)
    assert ei.value.status == b200.B200_UNSUPPORTED and "65535" in str(ei.value)
    # the status word is required (nobody else could report a device-side timeout)
    st = L.b200_dsa_forward_bf16_static(*(C.c_void_p(t.data_ptr()) for t in d), C.c_void_p(didx.data_ptr()),
                                        C.c_void_p(out.data_ptr()), C.byref(b200.DsaConfig(2, H, 512, 64, 64, 64, 512)),
                                        None, None)
    assert st == b200.B200_BAD_ARG
    # a large batch runs one row range per query, needs no scratch and is accepted whatever its size
    Q2 = 80
    _, _, d2, didx2 = _case(rng, Q2, H, 64, 512, cuda)
    out2 = torch.empty((Q2, H, 512), dtype=torch.float32, device=cuda)
    ref2 = torch.empty_like(out2)
    cfg2 = b200.DsaConfig(Q2, H, 512, 64, 64, 64, 512)
    b200.dsa_forward_bf16_static(*d2, didx2, out2, cfg2, status)
    b200.dsa_forward_bf16(*d2, didx2, ref2, cfg2)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert float((out2 - ref2).abs().max()) < 1e-2
