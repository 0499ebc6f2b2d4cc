"""GPU parity of the DSA / MLA sparse decode through the C ABI: the reference's 14 fp32 cases
against golden outputs of its own CPU code, config 2 (paged cache, unsorted indices), duplicate
indices, the stage launchers, the tensor-core self checks and the bf16 tcgen05 kernel."""
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DSA = np.load(os.path.join(ROOT, "tests", "golden", "dsa_reference_cases.npz"))
NAMES = sorted({k.split("/")[1] for k in DSA.files})
pytestmark = pytest.mark.gpu


def _dev(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _run(b200, dev, qn, qp, kc, kp, v, idx, P=64):
    Q, H, Dc = qn.shape
    cfg = b200.DsaConfig(Q, H, Dc, qp.shape[2], idx.shape[1], P, kc.shape[0])
    out = torch.full((Q, H, Dc), float("nan"), dtype=torch.float32, device=dev)
    b200.dsa_forward(*[_dev(a, dev) for a in (qn, qp, kc, kp, v, idx)], out, cfg)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("name", NAMES)
def test_reference_case(b200, cuda, name):
    Q, H, Dc, Dp, S, P, N = (int(v) for v in DSA[f"dsa/{name}/cfg"])
    tol = float(DSA[f"dsa/{name}/tol"])
    qn, qp, kc, kp, v, idx = oracle.dsa_inputs_reference_style(Q, H, Dc, Dp, S, P, N)
    out = _run(b200, cuda, qn, qp, kc, kp, v, idx, P)
    err = np.abs(out - DSA[f"dsa/{name}/out"]).max()
    assert err < tol and err < 1e-5, err


def test_config2_paged_unsorted(b200, cuda):
    """B=4, H=16, Dc=512, Dp=64, page 64, seq_len 1024, top-k 256: distinct logical positions per
    sequence, left unsorted, mapped through a random page table to flat physical token ids."""
    rng = np.random.default_rng(7)
    B, H, Dc, Dp, S, P, L = 4, 16, 512, 64, 256, 64, 1024
    N = B * L
    qn = b200.synth_normal_host(11, 0, B * H * Dc, 1.0).reshape(B, H, Dc)
    qp = b200.synth_normal_host(12, 0, B * H * Dp, 1.0).reshape(B, H, Dp)
    kc = b200.synth_normal_host(13, 0, N * Dc, 1.0).reshape(N, Dc)
    kp = b200.synth_normal_host(14, 0, N * Dp, 1.0).reshape(N, Dp)
    v = b200.synth_normal_host(15, 0, N * Dc, 1.0).reshape(N, Dc)
    pages = rng.permutation(N // P).reshape(B, L // P)          # block table: sequence b, logical page -> physical page
    idx = np.empty((B, S), np.int32)
    for b in range(B):
        pos = rng.permutation(L)[:S]                            # unsorted, distinct
        idx[b] = pages[b, pos // P] * P + pos % P
    assert not np.all(np.diff(idx, axis=1) > 0)
    ref = oracle.dsa_forward_f32(qn, qp, kc, kp, v, idx)
    out = _run(b200, cuda, qn, qp, kc, kp, v, idx, P)
    assert np.abs(out - ref).max() < 1e-3                       # the reference's tolerance class for this size


def test_duplicates_and_order(b200, cuda):
    rng = np.random.default_rng(8)
    Q, H, Dc, Dp, S, N = 3, 5, 96, 24, 40, 64
    f = lambda *s: rng.normal(0, 0.5, s).astype(np.float32)
    qn, qp, kc, kp, v = f(Q, H, Dc), f(Q, H, Dp), f(N, Dc), f(N, Dp), f(N, Dc)
    idx = rng.integers(0, N, (Q, S)).astype(np.int32)            # with replacement: duplicates count twice
    assert any(len(set(r)) < S for r in idx.tolist())
    ref = oracle.dsa_forward_f32(qn, qp, kc, kp, v, idx)
    out = _run(b200, cuda, qn, qp, kc, kp, v, idx)
    assert np.abs(out - ref).max() < 1e-5
    out2 = _run(b200, cuda, qn, qp, kc, kp, v, idx[:, ::-1].copy())
    assert np.abs(out2 - ref).max() < 1e-5


def test_stage_launchers(b200, cuda):
    """dsa_kv_gather -> dsa_dot_fused (and the unfused pair) -> scale -> dsa_softmax -> dsa_output_proj."""
    Q, H, Dc, Dp, S, P, N = 4, 4, 64, 16, 64, 16, 256
    qn, qp, kc, kp, v, idx = oracle.dsa_inputs_reference_style(Q, H, Dc, Dp, S, P, N)
    cfg = b200.DsaConfig(Q, H, Dc, Dp, S, P, N)
    d = [_dev(a, cuda) for a in (qn, qp, kc, kp, v, idx)]
    gkc = torch.empty((Q, S, Dc), device=cuda); gkp = torch.empty((Q, S, Dp), device=cuda)
    gv = torch.empty((Q, S, Dc), device=cuda)
    b200.dsa_kv_gather(d[2], d[3], d[4], d[5], gkc, gkp, gv, cfg)
    assert np.array_equal(gkc.cpu().numpy(), kc[idx]) and np.array_equal(gv.cpu().numpy(), v[idx])
    s1 = torch.zeros((Q, H, S), device=cuda); s2 = torch.zeros((Q, H, S), device=cuda)
    b200.dsa_dot_fused(d[0], d[1], gkc, gkp, s1, cfg)
    b200.dsa_dot_compressed(d[0], gkc, s2, cfg)
    b200.dsa_dot_positional(d[1], gkp, s2, cfg)
    assert torch.allclose(s1, s2, atol=1e-6)
    s1 *= 1.0 / np.sqrt(Dc + Dp)
    b200.dsa_softmax(s1, cfg)
    out = torch.empty((Q, H, Dc), device=cuda)
    b200.dsa_output_proj(s1, gv, out, cfg)
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - DSA["dsa/small/out"]).max() < 1e-5


def test_reference_test_driver_passes(b200, cuda):
    exe = os.path.join(ROOT, "oracle", "_ref", "drivers", "test_dsa")
    if not os.path.exists(exe):
        pytest.skip("reference driver not built (no reference checkout at build time)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout[-2500:])
    assert r.returncode == 0, r.stdout[-2500:] + r.stderr[-2000:]
    assert "14 / 14 passed" in r.stdout


# ---------------------------------------------------------------------------------------
# tensor-core path
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode,N,K", [(0, 32, 576), (0, 256, 64), (1, 256, 128), (1, 64, 64), (2, 256, 128),
                                      (2, 128, 256), (3, 256, 128), (3, 64, 64)])
def test_umma_selftest(b200, cuda, mode, N, K):
    """D[128,N] = A[128,K] * B[N,K]^T through the production shared-memory layouts/descriptors."""
    rng = np.random.default_rng(100 + mode)
    a = rng.normal(0, 1, (128, K)).astype(np.float32)
    bm = rng.normal(0, 1, (N, K)).astype(np.float32)
    if mode == 2:
        aq, bq = oracle.e4m3_encode(a), oracle.e4m3_encode(bm)
        ref = oracle.e4m3_decode(aq).astype(np.float64) @ oracle.e4m3_decode(bq).astype(np.float64).T
        da, db = _dev(aq, cuda), _dev(bq, cuda)
    else:
        ab, bb = oracle.bf16_bits(a), oracle.bf16_bits(bm)
        ref = oracle.bf16_to_f32(ab).astype(np.float64) @ oracle.bf16_to_f32(bb).astype(np.float64).T
        da = _dev(ab.view(np.int16), cuda)
        db = _dev((bb.T.copy() if mode == 1 else bb).view(np.int16), cuda)     # mode 1: B stored [K,N]
    d = torch.full((128, N), float("nan"), dtype=torch.float32, device=cuda)
    b200.umma_selftest(mode, da, db, d, N, K)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    got = d.cpu().numpy()
    assert np.abs(got - ref).max() <= 1e-3 * max(1.0, np.abs(ref).max()), np.abs(got - ref).max()


def _bf16_case(b200, rng, Q, H, S, N, sigma_kv=0.5):
    Dc, Dp = 512, 64
    f = lambda n, s: rng.normal(0, s, n).astype(np.float32)
    qn = oracle.bf16_bits(f(Q * H * Dc, 1.0)).reshape(Q, H, Dc)
    qp = oracle.bf16_bits(f(Q * H * Dp, 1.0)).reshape(Q, H, Dp)
    kc = oracle.bf16_bits(f(N * Dc, sigma_kv)).reshape(N, Dc)
    kp = oracle.bf16_bits(f(N * Dp, sigma_kv)).reshape(N, Dp)
    v = oracle.bf16_bits(f(N * Dc, sigma_kv)).reshape(N, Dc)
    idx = np.stack([rng.permutation(N)[:S] for _ in range(Q)]).astype(np.int32)
    return qn, qp, kc, kp, v, idx


@pytest.mark.parametrize("Q,H,S,N", [(1, 128, 32, 64), (2, 128, 64, 256), (3, 16, 256, 1024), (4, 128, 2048, 4096),
                                     (80, 128, 128, 512)])
def test_bf16_tensor_core_decode(b200, cuda, Q, H, S, N):
    """bf16 in, fp32 accumulate; oracle = reference CPU algorithm on the bf16-rounded inputs.
    Tolerance 1e-2 absolute (the reference's class for larger cases); P is rounded to bf16 before P*V."""
    rng = np.random.default_rng(Q * 1000 + S)
    qn, qp, kc, kp, v, idx = _bf16_case(b200, rng, Q, H, S, N)
    ref = oracle.dsa_forward_bf16(qn, qp, kc, kp, v, idx)
    cfg = b200.DsaConfig(Q, H, 512, 64, S, 64, N)
    out = torch.full((Q, H, 512), float("nan"), dtype=torch.float32, device=cuda)
    as16 = lambda a: _dev(a.view(np.int16), cuda).view(torch.bfloat16)
    b200.dsa_forward_bf16(as16(qn), as16(qp), as16(kc), as16(kp), as16(v), _dev(idx, cuda), out, cfg)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    err = np.abs(out.cpu().numpy() - ref).max()
    assert err < 1e-2, err


@pytest.mark.parametrize("Q,S,N,entry", [(2, 256, 1024, "ws"), (2, 192, 1024, "ws"), (3, 96, 512, "ws"),
                                         (1, 2048, 4096, "ws"), (5, 1024, 2048, "ws"), (1, 1024, 4096, "static"),
                                         (2, 96, 512, "static")])
def test_bf16_decode_running_max_rescale(b200, cuda, Q, S, N, entry):
    """The online softmax rescales the accumulated output only when a tile's maximum exceeds the running
    maximum by more than 2^8 (about 133 raw score units).  Ordinary data never does that after the first
    tile, so this case makes the scores grow along each query's row list: the K rows get a gain of 1, 8,
    64 by thirds of the cache and every index list is ascending.  Covers the 128-row, 64-row and 32-row
    kernels, split row ranges with their merge (Q = 1, S = 2048) and the built-in-scratch entry point."""
    rng = np.random.default_rng(S + Q)
    qn, qp, kc, kp, v, idx = _bf16_case(b200, rng, Q, 128, S, N)
    gain = np.repeat(np.array([1.0, 8.0, 64.0], np.float32), [N // 3, N // 3, N - 2 * (N // 3)])[:, None]
    kc = oracle.bf16_bits(oracle.bf16_to_f32(kc) * gain)
    kp = oracle.bf16_bits(oracle.bf16_to_f32(kp) * gain)
    idx = np.sort(idx, axis=1).astype(np.int32)
    ref = oracle.dsa_forward_bf16(qn, qp, kc, kp, v, idx)
    cfg = b200.DsaConfig(Q, 128, 512, 64, S, 64, N)
    out = torch.full((Q, 128, 512), float("nan"), dtype=torch.float32, device=cuda)
    as16 = lambda a: _dev(a.view(np.int16), cuda).view(torch.bfloat16)
    args = (as16(qn), as16(qp), as16(kc), as16(kp), as16(v), _dev(idx, cuda), out, cfg)
    if entry == "static":
        status = torch.zeros(1, dtype=torch.int32, device=cuda)
        b200.dsa_forward_bf16_static(*args, status)
    else:
        b200.dsa_forward_bf16(*args)
    torch.cuda.synchronize()
    assert b200.device_status() == 0
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max()
    assert err < 1e-2, err


def test_bf16_rejects_unsupported_shapes(b200, cuda):
    t = torch.zeros(64, dtype=torch.bfloat16, device=cuda)
    i = torch.zeros(64, dtype=torch.int32, device=cuda)
    o = torch.zeros(64, dtype=torch.float32, device=cuda)
    with pytest.raises(b200.B200Error) as ei:
        b200.dsa_forward_bf16(t, t, t, t, t, i, o, b200.DsaConfig(1, 4, 64, 16, 32, 64, 64))
    assert ei.value.status == b200.B200_UNSUPPORTED
    with pytest.raises(b200.B200Error) as ei:
        b200.dsa_forward_bf16(t, t, t, t, t, i, o, b200.DsaConfig(1, 128, 512, 64, 48, 64, 64))
    assert ei.value.status == b200.B200_BAD_SHAPE
