#!/usr/bin/env python
"""Benchmark of the two hot paths on B200.

Headline (the JSON line's `metric`/`value`): FP8 block-scale MoE layer throughput in tokens/s
at T = 4096 tokens per GPU (DeepSeek-V3 shape: D=7168, I=2048, E=256, top-8, 8 groups / top-4,
sigmoid + bias scoring, routed scaling 2.5).  One GPU runs the whole layer (config "C3"); N > 1
GPUs shard the experts (E/N per GPU), keep 4096 tokens per GPU and exchange rows with NCCL
all-to-all (config "C5", Zipf(1.1)-skewed expert load) — weak scaling.
The same line carries, under "dsa", the sparse MLA decode step time at B=64, H=128, Dc=512,
Dp=64, top-2048 over a paged bf16 cache with 8192..131072 tokens per sequence (config "C4");
it shards by batch, so with N > 1 every GPU runs an independent replica.

All inputs are synthetic (seeded counter-based generator, DeepSeek shapes and the value
distributions the configs name); weights are random-initialised.

    python bench.py --gpus 1 --steps 20 --warmup 3
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference        # CPU arm: the oracle port on the host cores
"""
import argparse
import importlib.util
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MOE = dict(T=4096, E=256, K=8, D=7168, I=2048, n_group=8, topk_group=4, routed_scale=2.5)
DSA = dict(B=64, H=128, Dc=512, Dp=64, S=2048, page=64, seq_min=8192, seq_max=131072)
ZIPF_S, ZIPF_BETA = 1.1, 0.08
# --ep-placement "strided": expert e lives on GPU e mod N (a group's 32 experts and a run of hot ones spread over
# all GPUs); "balanced": greedy placement by the expert loads of a calibration batch; "contiguous": blocks of E/N
EP_PLACEMENT = "balanced"
MOE_FLAGS = 0          # --moe-tiles: force the grouped GEMMs' tile shape (4 = single CTA, 8 = CTA pairs)
POW2_SCALES = False    # --pow2-scales: variant run with power-of-two scales
RTOL, ATOL = 2e-2, 1e-2


def load_package():
    name = "llm_sys_project_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg = os.path.join(ROOT, "llm-sys-project_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg, "__init__.py"),
                                                  submodule_search_locations=[pkg])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


# DRAM bytes / algorithmic bytes of the dominant kernels, from the ncu captures summarised under profiles/:
# GEMM1 from a one-pass DRAM-counter capture of a full-size launch (7.93 GB read + written for 7.83 GB; the small
# case agrees), the decode kernel from a small case of the same kernel (traffic grows with the rows fetched)
TRAFFIC_RATIO = {"gemm1": 1.01, "dsa": 1.00}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


_FP8_PEAK = {}


def fp8_peak_tflops(b200=None):
    """Dense FP8 tensor rate of this GPU, measured with the library's own kind::f8f6f4 MMA loop (the shape
    the grouped GEMMs issue, operands resident in shared memory, all SMs busy): a 6 ms burst and a 0.3 s
    run.  The operands are constant bytes, so this is the issue-rate ceiling; real data under the power
    cap runs lower.  Nominal: 4500."""
    if not _FP8_PEAK and b200 is not None:
        burst, _ = b200.fp8_mma_rate(False, 20000)
        long_run, ms = b200.fp8_mma_rate(False, 1000000)
        pair, _ = b200.fp8_mma_rate(True, 20000)
        _FP8_PEAK.update(burst=burst, sustained=long_run, sustained_ms=ms, cta_pair_burst=pair, nominal=4500.0)
    return dict(_FP8_PEAK)


class ClockSampler:
    """Polls NVML (read-only) for SM clock and throttle reasons while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                 "hw_thermal_slowdown": 0x40, "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self.nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
def zipf_bias(E, seed):
    rng = np.random.default_rng(seed)
    rank_of = rng.permutation(E) + 1
    logp = -ZIPF_S * np.log(rank_of.astype(np.float64))
    return (ZIPF_BETA * (logp - logp.mean())).astype(np.float32)


def build_moe(b200, torch, dev, world, rank):
    """Weights of this rank's experts, the replicated router, and this rank's tokens."""
    c = MOE
    E_local = c["E"] // world
    w1q = torch.empty((E_local, 2 * c["I"], c["D"]), dtype=torch.uint8, device=dev)
    w1s = torch.empty((E_local, 2 * c["I"] // 128, c["D"] // 128), dtype=torch.float32, device=dev)
    w2q = torch.empty((E_local, c["D"], c["I"]), dtype=torch.uint8, device=dev)
    w2s = torch.empty((E_local, c["D"] // 128, c["I"] // 128), dtype=torch.float32, device=dev)
    b200.fill_normal_fp8_w128_(w1q, w1s, 1000 + rank, 0.02, pow2=POW2_SCALES)
    b200.fill_normal_fp8_w128_(w2q, w2s, 2000 + rank, 0.02, pow2=POW2_SCALES)
    gate_w = torch.empty((c["E"], c["D"]), dtype=torch.float32, device=dev)
    b200.fill_normal_(gate_w, 3000, c["D"] ** -0.5)
    bias_h = b200.synth_normal_host(3001, 0, c["E"], 0.01)
    if world > 1:
        bias_h = bias_h + zipf_bias(c["E"], 7)
    bias = torch.from_numpy(bias_h).to(dev)
    x = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
    b200.fill_normal_(x, 4000 + rank, 1.0)
    xq = torch.empty((c["T"], c["D"]), dtype=torch.uint8, device=dev)
    xs = torch.empty((c["T"], c["D"] // 128), dtype=torch.float32, device=dev)
    b200.quant_act_1x128(x, xq, xs, pow2=POW2_SCALES)
    del x
    layer = b200.MoeFp8Layer(gate_w, bias, w1q, w1s, w2q, w2s, c["K"], b200.SCORE_SIGMOID_GROUPED, c["n_group"],
                             c["topk_group"], c["routed_scale"], flags=MOE_FLAGS)
    layer.pack()          # pre-tiled weights for the grouped GEMMs (the row-major copy stays for the CPU check)
    return layer, xq, xs


def bench_route_only(b200, torch, dev, args):
    """The routing call alone at the full token count (no expert weights: a few hundred MB on the device), for
    profiler captures of the router kernels.  Prints its own JSON line; not a bench value."""
    c = MOE
    gate_w = torch.empty((c["E"], c["D"]), dtype=torch.float32, device=dev)
    b200.fill_normal_(gate_w, 3000, c["D"] ** -0.5)
    bias = torch.from_numpy(b200.synth_normal_host(3001, 0, c["E"], 0.01)).to(dev)
    x = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
    b200.fill_normal_(x, 4000, 1.0)
    xq = torch.empty((c["T"], c["D"]), dtype=torch.uint8, device=dev)
    xs = torch.empty((c["T"], c["D"] // 128), dtype=torch.float32, device=dev)
    b200.quant_act_1x128(x, xq, xs)
    del x
    ids = torch.zeros((c["T"], c["K"]), dtype=torch.int32, device=dev)
    wts = torch.zeros((c["T"], c["K"]), dtype=torch.float32, device=dev)
    counts = torch.zeros(c["E"], dtype=torch.int32, device=dev)
    cfg = b200.MoeFp8Config(c["T"], c["E"], c["K"], c["D"], c["I"], b200.SCORE_SIGMOID_GROUPED, c["n_group"],
                            c["topk_group"], c["routed_scale"], 0)
    steps = max(1, args.steps)
    for _ in range(max(args.warmup, 3)):
        b200.moe_route_fp8(xq, xs, gate_w, bias, ids, wts, cfg, counts=counts)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        b200.moe_route_fp8(xq, xs, gate_w, bias, ids, wts, cfg, counts=counts)
    e1.record()
    torch.cuda.synchronize()
    assert b200.device_status() == 0, "device-side wait timed out"
    print(json.dumps({"routing_only": True, "tokens": c["T"], "ms_per_call": e0.elapsed_time(e1) / steps, "steps": steps,
                      "exact_pass_tokens": b200.moe_route_last_flagged()}))


def moe_gemm1_bytes(counts):
    """Algorithmic HBM bytes of one GEMM1 launch: FP8 weights + block scales of the active experts,
    the sorted FP8 rows + 1x128 scales read, the requantised activations + scales written."""
    c = MOE
    active = int((counts > 0).sum())
    rows = int(counts.sum())
    w = active * (2 * c["I"] * c["D"] + 4 * (2 * c["I"] // 128) * (c["D"] // 128))
    a = rows * (c["D"] + 4 * c["D"] // 128)
    o = rows * (c["I"] + 4 * c["I"] // 128)
    return w + a + o, active, rows


def moe_layer_bytes(counts):
    """Algorithmic bytes of the whole layer (weights once, x once, router weights, output)."""
    c = MOE
    active = int((counts > 0).sum())
    w = active * (3 * c["D"] * c["I"] + 4 * ((2 * c["I"] // 128) * (c["D"] // 128) + (c["D"] // 128) * (c["I"] // 128)))
    return w + c["T"] * (c["D"] + 4 * c["D"] // 128) + 4 * c["E"] * c["D"] + c["T"] * c["D"] * 4


def _emulate(oracle, *a):
    """oracle.moe_fp8_experts under the scale rule of this run (the requantisation between the GEMMs follows it)."""
    if POW2_SCALES:
        with oracle.pow2_scales():
            return oracle.moe_fp8_experts(*a)
    return oracle.moe_fp8_experts(*a)


def moe_cpu_sample(b200, torch, oracle, layer, xq, xs, out_dev, n_tokens, threads):
    """Oracle (CPU emulation of the same FP8 sequence) on a seeded sample of tokens: parity of the
    GPU output rows and the CPU throughput.  Only the experts the sample uses are copied to the host."""
    c = MOE
    rng = np.random.default_rng(5)
    toks = np.sort(rng.choice(c["T"], n_tokens, replace=False)).astype(np.int32)
    xq_h = xq.index_select(0, torch.from_numpy(toks).to(xq.device).long()).cpu().numpy()
    xs_h = xs.index_select(0, torch.from_numpy(toks).to(xq.device).long()).cpu().numpy()
    wg_h, bias_h = layer.gate_w.cpu().numpy(), layer.bias.cpu().numpy()
    oracle.set_threads(threads)
    t0 = time.perf_counter()
    ids, wts = oracle.route_grouped(xq_h, xs_h, wg_h, bias_h, c["K"], c["n_group"], c["topk_group"], c["routed_scale"])
    t_route = time.perf_counter() - t0
    uniq = np.unique(ids)
    remap = -np.ones(c["E"], np.int32)
    remap[uniq] = np.arange(len(uniq), dtype=np.int32)
    sel = torch.from_numpy(uniq.astype(np.int64)).to(xq.device)
    w1q = layer.w1q.index_select(0, sel).cpu().numpy()
    w1s = layer.w1s.index_select(0, sel).cpu().numpy()
    w2q = layer.w2q.index_select(0, sel).cpu().numpy()
    w2s = layer.w2s.index_select(0, sel).cpu().numpy()
    t0 = time.perf_counter()
    ref = _emulate(oracle, xq_h, xs_h, w1q, w1s, w2q, w2s, remap[ids], wts,
                                 np.arange(n_tokens, dtype=np.int32))
    t_ffn = time.perf_counter() - t0
    got = out_dev.index_select(0, torch.from_numpy(toks).to(xq.device).long()).cpu().numpy()
    gids = None
    err = np.abs(got - ref)
    ok = bool(not (err > ATOL + RTOL * np.abs(ref)).any())
    return {"tokens": int(n_tokens), "seconds": t_route + t_ffn, "ok": ok, "max_abs_err": float(err.max()),
            "ref_absmax": float(np.abs(ref).max()), "ids": ids, "toks": toks, "gids": gids}


def bench_moe_pow2_variant(b200, torch, oracle, layer, dev, args, threads):
    """The same layer, the same seeded values, quantised with power-of-two scales (the UE8M0 scale format) and run
    with MOE_POW2_SCALES: the grouped GEMMs take the hardware block-scaled MMA.  A secondary figure beside the
    headline (whose scales are amax/448 as the emulation of the reference defines them); checked against the CPU
    emulation with the same scale rule on a sample of tokens."""
    c = MOE
    b200.fill_normal_fp8_w128_(layer.w1q, layer.w1s, 1000, 0.02, pow2=True)
    b200.fill_normal_fp8_w128_(layer.w2q, layer.w2s, 2000, 0.02, pow2=True)
    layer.w1p = layer.w2p = None
    layer.pack()
    x = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
    b200.fill_normal_(x, 4000, 1.0)
    xq = torch.empty((c["T"], c["D"]), dtype=torch.uint8, device=dev)
    xs = torch.empty((c["T"], c["D"] // 128), dtype=torch.float32, device=dev)
    b200.quant_act_1x128(x, xq, xs, pow2=True)
    del x
    layer.flags |= b200.MOE_POW2_SCALES
    out = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
    for _ in range(3):
        layer.forward(xq, xs, out)
    torch.cuda.synchronize()
    status = b200.device_status()
    b200.moe_fp8_profile(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        layer.forward(xq, xs, out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    g1_ms, g2_ms, _ = b200.moe_fp8_profile_read()
    b200.moe_fp8_profile(False)
    with oracle.pow2_scales():
        cpu = moe_cpu_sample(b200, torch, oracle, layer, xq, xs, out, min(args.cpu_tokens, 24), threads)
    ids, _ = layer.route(xq, xs)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=c["E"]).cpu().numpy()
    g1_bytes, active, rows = moe_gemm1_bytes(counts)
    hbm, _, which = measured_peaks()
    return {"ms_per_step": ms, "tokens_per_s": c["T"] / (ms * 1e-3), "gemm1_ms": g1_ms, "gemm2_ms": g2_ms,
            "gemm1_hbm_gbs": g1_bytes / (g1_ms * 1e-3) / 1e9 if g1_ms > 0 else None,
            "gemm1_hbm_frac": g1_bytes / (g1_ms * 1e-3) / 1e9 / hbm if g1_ms > 0 else None,
            "gemm_tflops": 6.0 * rows * c["D"] * c["I"] / ((g1_ms + g2_ms) * 1e-3) / 1e12 if g1_ms > 0 else None,
            "device_status": int(status),
            "parity": {"checked_tokens": cpu["tokens"], "ok": cpu["ok"], "max_abs_err": cpu["max_abs_err"],
                       "ref_absmax": cpu["ref_absmax"], "tolerance": f"{RTOL} rel + {ATOL} abs"},
            "note": "power-of-two scales (MOE_POW2_SCALES): tcgen05.mma kind::mxf8f6f4.block_scale, no software "
                    "promotion; not the headline configuration"}


def bench_moe_single(b200, torch, oracle, dev, args, sampler):
    c = MOE
    layer, xq, xs = build_moe(b200, torch, dev, 1, 0)
    out = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
    for _ in range(max(args.warmup, 3)):
        layer.forward(xq, xs, out)
    torch.cuda.synchronize()
    assert b200.device_status() == 0, "device-side wait timed out"
    ids, wts = layer.route(xq, xs)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=c["E"]).cpu().numpy()

    # routing alone (router GEMM + top-K selection + histogram), for its own roofline line
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for _ in range(5):
        layer.route(xq, xs)
    r1.record()
    torch.cuda.synchronize()
    route_ms = r0.elapsed_time(r1) / 5
    route_flagged = b200.moe_route_last_flagged()       # tokens the tensor-core router handed to its exact pass

    b200.moe_fp8_profile(True)
    b200.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        layer.forward(xq, xs, out)
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    launches = b200.launch_count()
    ms = e0.elapsed_time(e1) / args.steps
    g1_ms, g2_ms, ncalls = b200.moe_fp8_profile_read()
    b200.moe_fp8_profile(False)

    # the same layer at the other token counts the workload is swept over (device-resident inputs)
    sweep = {}
    for Ts in (1, 16, 128, 1024):
        if Ts >= c["T"]:
            continue
        xq_s, xs_s = xq[:Ts].contiguous(), xs[:Ts].contiguous()
        out_s = torch.empty((Ts, c["D"]), dtype=torch.float32, device=dev)
        for _ in range(3):
            layer.forward(xq_s, xs_s, out_s)
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(10):
            layer.forward(xq_s, xs_s, out_s)
        s1.record()
        torch.cuda.synchronize()
        ms_s = s0.elapsed_time(s1) / 10
        sweep[str(Ts)] = {"ms_per_step": ms_s, "tokens_per_s": Ts / (ms_s * 1e-3)}
        # small batches are launch-bound from Python: the same call replayed from a CUDA graph
        try:
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                layer.forward(xq_s, xs_s, out_s)
            torch.cuda.current_stream().wait_stream(side)
            with torch.cuda.graph(graph):
                layer.forward(xq_s, xs_s, out_s)
            for _ in range(3):
                graph.replay()
            s0.record()
            for _ in range(10):
                graph.replay()
            s1.record()
            torch.cuda.synchronize()
            sweep[str(Ts)]["ms_per_step_cuda_graph"] = s0.elapsed_time(s1) / 10
            del graph
        except Exception as exc:                      # capture is an extra, never a reason to lose the run
            sweep[str(Ts)]["cuda_graph_error"] = str(exc)[:120]
            torch.cuda.synchronize()

    # end to end through the host-facing layer call: pinned host in, pinned host out, every step.
    # Synchronous call first (one step at a time), then the double-buffered call a serving loop uses:
    # the copies of steps n-1 / n+1 run on their own streams under the kernels of step n.
    xq_h, xs_h = xq.cpu().pin_memory(), xs.cpu().pin_memory()
    out_hs = [torch.empty((c["T"], c["D"]), dtype=torch.float32).pin_memory() for _ in range(2)]
    out_h = out_hs[0]
    for _ in range(2):
        layer.forward_host(xq_h, xs_h, out_h)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        layer.forward_host(xq_h, xs_h, out_h)
    e2e_sync_s = (time.perf_counter() - t0) / args.steps
    for i in range(3):
        tk = layer.forward_host_async(xq_h, xs_h, out_hs[i % 2])
    tk.synchronize()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        tk = layer.forward_host_async(xq_h, xs_h, out_hs[i % 2])
    tk.synchronize()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / args.steps
    # both buffers hold a result of the same input (the scatter-add order differs from run to run)
    e2e_same = bool(torch.allclose(out_hs[0][:64], out_hs[1][:64], rtol=1e-4, atol=1e-5))
    # the step's copies alone (inputs in, result out, on two streams at once, no kernels): the floor the host link
    # sets for the end-to-end step
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        with torch.cuda.stream(s_in):
            xq.copy_(xq_h, non_blocking=True)
            xs.copy_(xs_h, non_blocking=True)
        with torch.cuda.stream(s_out):
            out_hs[i % 2].copy_(out, non_blocking=True)
    torch.cuda.synchronize()
    copy_only_s = (time.perf_counter() - t0) / args.steps

    threads = oracle.host_threads()
    cpu = moe_cpu_sample(b200, torch, oracle, layer, xq, xs, out, args.cpu_tokens, threads)
    hbm, bf16_tf, which = measured_peaks()
    fp8_peak = fp8_peak_tflops(b200)
    pow2 = None
    if not args.skip_pow2:
        try:
            pow2 = bench_moe_pow2_variant(b200, torch, oracle, layer, dev, args, threads)
        except Exception as exc:                          # a secondary figure never costs the headline
            pow2 = {"error": str(exc)[:200]}
            torch.cuda.synchronize()
    g1_bytes, active, rows = moe_gemm1_bytes(counts)
    g2_bytes = (active * (c["D"] * c["I"] + 4 * (c["D"] // 128) * (c["I"] // 128)) + rows * (c["I"] + 4 * c["I"] // 128)
                + c["T"] * c["D"] * 4)
    route_bytes = c["T"] * (c["D"] + 4 * c["D"] // 128) + 4 * c["E"] * c["D"] + 8 * c["T"] * c["K"]
    flops = 6.0 * rows * c["D"] * c["I"] + 2.0 * c["T"] * c["E"] * c["D"]
    res = {
        "value": c["T"] / (ms * 1e-3), "ms_per_step": ms, "gpu_launches": int(launches),
        "e2e": {"value": c["T"] / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": int(xq_h.numel() + xs_h.numel() * 4),
                "d2h_bytes_per_step": int(out_h.numel() * 4), "ms_per_step": e2e_s * 1e3,
                "copies_only_ms_per_step": copy_only_s * 1e3,
                "mode": "double-buffered host pipeline (MoeFp8Layer.forward_host_async): every step copies its "
                        "inputs in and its result out; copies overlap the neighbouring steps' kernels",
                "synchronous_value": c["T"] / e2e_sync_s, "synchronous_ms_per_step": e2e_sync_s * 1e3,
                "results_agree_across_buffers": e2e_same},
        "roofline": {"kernel": "grouped_gemm_fp8<1> (GEMM1+SwiGLU+requant)", "bound": "hbm",
                     "achieved": g1_bytes / (g1_ms * 1e-3) / 1e9 if g1_ms > 0 else None, "peak": hbm, "unit": "GB/s",
                     "frac": (g1_bytes / (g1_ms * 1e-3) / 1e9 / hbm) if g1_ms > 0 else None,
                     "traffic": int(g1_bytes * TRAFFIC_RATIO["gemm1"]),
                     "peak_source": which, "kernel_ms": g1_ms, "algorithmic_bytes": int(g1_bytes),
                     "launches_timed": ncalls},
        "roofline_gemm2": {"kernel": "grouped_gemm_fp8<2> (GEMM2 + router weight + scatter-add)", "bound": "hbm",
                           "achieved": g2_bytes / (g2_ms * 1e-3) / 1e9 if g2_ms > 0 else None, "peak": hbm, "unit": "GB/s",
                           "frac": (g2_bytes / (g2_ms * 1e-3) / 1e9 / hbm) if g2_ms > 0 else None, "kernel_ms": g2_ms,
                           "algorithmic_bytes": int(g2_bytes),
                           "note": "weights + requantised activations read, output written once; the fp32 "
                                   "scatter-add traffic (rows x D x 4 bytes) is implementation traffic"},
        "roofline_routing": {"kernel": "router logits + selection (+ exact pass)", "bound": "hbm",
                             "achieved": route_bytes / (route_ms * 1e-3) / 1e9, "peak": hbm, "unit": "GB/s",
                             "frac": route_bytes / (route_ms * 1e-3) / 1e9 / hbm, "kernel_ms": route_ms,
                             "algorithmic_bytes": int(route_bytes)},
        "kernels": {"gemm1_ms": g1_ms, "gemm2_ms": g2_ms, "other_ms": ms - g1_ms - g2_ms, "token_sweep": sweep,
                    "fp8_peak_tflops_measured": fp8_peak,
                    "pow2_scales_variant": pow2,
                    "gemm_frac_of_measured_fp8_peak": (6.0 * rows * c["D"] * c["I"] / ((g1_ms + g2_ms) * 1e-3) / 1e12
                                                       / fp8_peak["burst"]) if g1_ms > 0 and fp8_peak else None,
                    "layer_bytes": int(moe_layer_bytes(counts)),
                    "layer_hbm_gbs": moe_layer_bytes(counts) / (ms * 1e-3) / 1e9,
                    "layer_tflops": flops / (ms * 1e-3) / 1e12,
                    "gemm_tflops": 6.0 * rows * c["D"] * c["I"] / ((g1_ms + g2_ms) * 1e-3) / 1e12 if g1_ms > 0 else None,
                    "fp8_peak_tflops_nominal": 4500.0,
                    "gemm_frac_of_fp8_peak": (6.0 * rows * c["D"] * c["I"] / ((g1_ms + g2_ms) * 1e-3) / 1e12 / 4500.0)
                                             if g1_ms > 0 else None,
                    "gemm_hbm_bound_note": "11.3 GB of weights for 32768 rows: the weight stream caps both GEMMs at "
                                           "37 % of the FP8 peak at this shape",
                    "routing_ms": route_ms,
                    "routing_algorithmic_bytes": int(c["T"] * (c["D"] + 4 * c["D"] // 128) + 4 * c["E"] * c["D"]
                                                     + 8 * c["T"] * c["K"]),
                    "routing_hbm_gbs": (c["T"] * (c["D"] + 4 * c["D"] // 128) + 4 * c["E"] * c["D"] + 8 * c["T"] * c["K"])
                                       / (route_ms * 1e-3) / 1e9,
                    "routing_fp32_tflops": 2.0 * c["T"] * c["E"] * c["D"] / (route_ms * 1e-3) / 1e12,
                    "routing_exact_pass_tokens": route_flagged,
                    "routing_note": "router logits on the tensor cores (tf32 split operands), ids certified by decision "
                                    "margins, the listed number of tokens recomputed with the fixed-order FMA chains"
                                    if route_flagged >= 0 else "fixed-order fp32 FMA chains on the SIMT pipes",
                    "active_experts": active,
                    "max_tokens_per_expert": int(counts.max()), "mean_tokens_per_expert": float(counts.mean())},
        "cpu_baseline": {"value": cpu["tokens"] / cpu["seconds"], "unit": "tokens/s", "cores": threads, "kind": "port",
                         "sample": f"{cpu['tokens']} seeded tokens of the same workload (routing + 8 experts each) "
                                   f"through the fp32 CPU emulation, {cpu['seconds']:.2f} s"},
        "parity": {"checked_tokens": cpu["tokens"], "ok": cpu["ok"], "max_abs_err": cpu["max_abs_err"],
                   "ref_absmax": cpu["ref_absmax"], "tolerance": f"{RTOL} rel + {ATOL} abs"},
    }
    del layer, xq, xs, out
    torch.cuda.empty_cache()
    return res


def ep_parity_sample(b200, torch, oracle, layer, placement, world, xq, xs, out_dev, ids_dev, n_tokens, threads):
    """Oracle check of the expert-parallel layer on rank 0: a seeded sample of this rank's tokens through
    the CPU emulation.  The experts they use live on other GPUs; their weights are regenerated here from the
    seeds (one owner rank's set at a time into a scratch buffer), so the check needs no communication."""
    c = MOE
    El = c["E"] // world
    rng = np.random.default_rng(5)
    toks = np.sort(rng.choice(c["T"], n_tokens, replace=False)).astype(np.int32)
    sel_t = torch.from_numpy(toks).to(xq.device).long()
    xq_h, xs_h = xq.index_select(0, sel_t).cpu().numpy(), xs.index_select(0, sel_t).cpu().numpy()
    wg_h, bias_h = layer.gate_w.cpu().numpy(), layer.bias.cpu().numpy()
    oracle.set_threads(threads)
    t0 = time.perf_counter()
    ids, wts = oracle.route_grouped(xq_h, xs_h, wg_h, bias_h, c["K"], c["n_group"], c["topk_group"], c["routed_scale"])
    cpu_s = time.perf_counter() - t0
    ids_ok = bool(np.array_equal(ids_dev.index_select(0, sel_t).cpu().numpy(), ids))
    if isinstance(placement, (tuple, list)):
        owner, local = placement[0].numpy().astype(np.int64), placement[1].numpy().astype(np.int64)
    elif placement == "strided":
        owner, local = np.arange(c["E"]) % world, np.arange(c["E"]) // world
    else:
        owner, local = np.arange(c["E"]) // El, np.arange(c["E"]) % El
    uniq = np.unique(ids)
    remap = -np.ones(c["E"], np.int32)
    remap[uniq] = np.arange(len(uniq), dtype=np.int32)
    w1q_h = np.empty((len(uniq), 2 * c["I"], c["D"]), np.uint8)
    w1s_h = np.empty((len(uniq), 2 * c["I"] // 128, c["D"] // 128), np.float32)
    w2q_h = np.empty((len(uniq), c["D"], c["I"]), np.uint8)
    w2s_h = np.empty((len(uniq), c["D"] // 128, c["I"] // 128), np.float32)
    s1q, s1s = torch.empty_like(layer.w1q), torch.empty_like(layer.w1s)
    s2q, s2s = torch.empty_like(layer.w2q), torch.empty_like(layer.w2s)
    for r in sorted(set(owner[uniq].tolist())):
        b200.fill_normal_fp8_w128_(s1q, s1s, 1000 + r, 0.02, pow2=POW2_SCALES)   # the weights rank r generated for itself
        b200.fill_normal_fp8_w128_(s2q, s2s, 2000 + r, 0.02, pow2=POW2_SCALES)
        mine = uniq[owner[uniq] == r]
        sel = torch.from_numpy(local[mine]).to(xq.device)
        dst = remap[mine]
        w1q_h[dst], w1s_h[dst] = s1q.index_select(0, sel).cpu().numpy(), s1s.index_select(0, sel).cpu().numpy()
        w2q_h[dst], w2s_h[dst] = s2q.index_select(0, sel).cpu().numpy(), s2s.index_select(0, sel).cpu().numpy()
    del s1q, s1s, s2q, s2s
    t0 = time.perf_counter()
    ref = _emulate(oracle, xq_h, xs_h, w1q_h, w1s_h, w2q_h, w2s_h, remap[ids], wts,
                                 np.arange(n_tokens, dtype=np.int32))
    cpu_s += time.perf_counter() - t0
    got = out_dev.index_select(0, sel_t).float().cpu().numpy()
    err = np.abs(got - ref)
    viol = err > ATOL + RTOL * np.abs(ref)
    return {"cpu_seconds": cpu_s, "checked_tokens": int(n_tokens), "rank": 0, "ids_bit_equal": ids_ok, "ok": bool(ids_ok and not viol.any()),
            "violations": int(viol.sum()), "max_abs_err": float(err.max()), "ref_absmax": float(np.abs(ref).max()),
            "tolerance": f"{RTOL} rel + {ATOL} abs", "experts_regenerated": int(len(uniq))}


def bench_moe_ep(b200, torch, oracle, dist, dev, args, world, rank, sampler):
    c = MOE
    layer, xq, xs = build_moe(b200, torch, dev, world, rank)
    placement = EP_PLACEMENT
    if EP_PLACEMENT == "balanced":
        # expert loads of a calibration batch (other tokens than the timed ones) decide the placement
        xc = torch.empty((c["T"], c["D"]), dtype=torch.float32, device=dev)
        b200.fill_normal_(xc, 9000 + rank, 1.0)
        cq = torch.empty((c["T"], c["D"]), dtype=torch.uint8, device=dev)
        cs = torch.empty((c["T"], c["D"] // 128), dtype=torch.float32, device=dev)
        b200.quant_act_1x128(xc, cq, cs)
        cal_ids, _ = layer.route(cq, cs)
        cal = torch.bincount(cal_ids.reshape(-1).long(), minlength=c["E"])
        dist.all_reduce(cal)
        placement = b200.balanced_placement(cal.cpu(), world)
        del xc, cq, cs
    peer = args.ep_impl == "peer"
    if peer:
        # the C-ABI object: rows travel by peer stores into mapped exchange buffers, no collective in a step
        pl = placement
        if placement == "strided":
            pl = (torch.arange(c["E"], dtype=torch.int32) % world, torch.arange(c["E"], dtype=torch.int32) // world)
        ep = b200.PeerExpertParallelMoe(dist.group.WORLD, layer, c["E"], c["T"], placement=pl,
                                        combine_dtype=torch.float16)      # fp16 rows relative to the row maximum
        ws_handle = ep.workspace()
    else:
        # the same exchange with torch.distributed (NCCL) all-to-alls around the kernels: the baseline
        # (fp32 partial rows: bf16 ones break the 1e-2 absolute bound where a token's partial rows cancel)
        ep = b200.ExpertParallelMoe(dist.group.WORLD, c["E"], c["K"], layer.route, layer.local_experts,
                                    combine_dtype=torch.float32, placement=placement)
        ws_handle = None
    for _ in range(max(args.warmup, 3)):
        out, ids, _ = ep.forward(xq, xs)
    torch.cuda.synchronize()
    if peer:
        st_w, _, recv_counts = ep.stats()
        assert st_w == 0, "device-side wait timed out"
        recv_tokens = int(sum(recv_counts))
    else:
        recv_tokens = ep.last_stats["recv_rows"]
    assert b200.device_status() == 0, "device-side wait timed out"
    counts = torch.bincount(ids.reshape(-1).long(), minlength=c["E"])
    dist.all_reduce(counts)
    counts = counts.cpu().numpy()
    b200.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        ep.forward(xq, xs)
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    sampler.stop()
    launches = b200.launch_count()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    phases = {}
    b200.moe_fp8_profile(True, ws_handle)
    if not peer:
        ep.profile = True
    else:
        ep.phase_profile(True)
    ep.forward(xq, xs)
    if not peer:
        phases = ep.phase_ms()
        ep.profile = False
    else:
        phases = ep.phase_profile(False)
    g1_ms, g2_ms, _ = b200.moe_fp8_profile_read(ws_handle)
    b200.moe_fp8_profile(False, ws_handle)
    El = c["E"] // world
    if EP_PLACEMENT == "balanced":
        local_counts = counts[placement[0].numpy() == rank]
    else:
        local_counts = counts[rank::world] if EP_PLACEMENT == "strided" else counts[rank * El:(rank + 1) * El]
    g1_bytes, active, rows = moe_gemm1_bytes(local_counts)
    hbm, _, which = measured_peaks()

    # end to end: this rank's tokens from pinned host memory, result back to pinned host memory, every
    # step, through the double-buffered host pipeline (copies overlap the neighbouring steps' kernels)
    xq_h, xs_h = xq.cpu().pin_memory(), xs.cpu().pin_memory()
    out_hs = [torch.empty((c["T"], c["D"]), dtype=torch.float32).pin_memory() for _ in range(2)]
    out_h = out_hs[0]
    pipe = b200.HostPipeline(dev)

    def ep_compute(dq, ds, do):
        o, _, _ = ep.forward(dq, ds)
        do.copy_(o)

    for i in range(3):
        tk = pipe.submit([xq_h, xs_h], out_hs[i % 2], ep_compute)
    tk.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        tk = pipe.submit([xq_h, xs_h], out_hs[i % 2], ep_compute)
    tk.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    te = torch.tensor([(time.perf_counter() - t0) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())
    # the same host pipeline with the copies only (no kernels): what the ranks' shared host memory and PCIe paths
    # allow when all ranks copy at once; e2e close to it means the step is bound by the host side, not by the GPUs
    def copy_only(dq, ds, do):
        return None
    for i in range(2):
        tk = pipe.submit([xq_h, xs_h], out_hs[i % 2], copy_only)
    tk.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        tk = pipe.submit([xq_h, xs_h], out_hs[i % 2], copy_only)
    tk.synchronize()
    torch.cuda.synchronize()
    dist.barrier()
    tc = torch.tensor([(time.perf_counter() - t0) / args.steps], device=dev, dtype=torch.float64)
    dist.all_reduce(tc, op=dist.ReduceOp.MAX)
    copy_only_s = float(tc.item())
    if EP_PLACEMENT == "balanced":
        own = placement[0].numpy()
        per_gpu = np.array([counts[own == g].sum() for g in range(world)])
    else:
        per_gpu = counts.reshape(-1, world).sum(0) if EP_PLACEMENT == "strided" else counts.reshape(world, -1).sum(1)
    rmax_v, rsum_v = float(per_gpu.max()), float(per_gpu.sum())     # (token, expert) pairs computed per GPU
    flops_hot = 6.0 * rmax_v * c["D"] * c["I"]
    flops_rank0 = 6.0 * float(per_gpu[0]) * c["D"] * c["I"]
    fp8_peak = fp8_peak_tflops(b200)
    res = {
        "value": world * c["T"] / (ms * 1e-3), "ms_per_step": ms, "gpu_launches": int(launches),
        "e2e": {"value": world * c["T"] / e2e_s, "unit": "tokens/s",
                "h2d_bytes_per_step": int(world * (xq_h.numel() + xs_h.numel() * 4)),
                "d2h_bytes_per_step": int(world * out_h.numel() * 4), "ms_per_step": e2e_s * 1e3,
                "copies_only_ms_per_step": copy_only_s * 1e3,
                "mode": "double-buffered host pipeline (HostPipeline around ExpertParallelMoe.forward); "
                        "copies_only_ms_per_step = the same pipeline without kernels, all ranks copying at once"},
        # with E / N experts per GPU and ~32 K rows the grouped GEMMs are bound by the tensor pipe, not by HBM
        "roofline": {"kernel": "grouped_gemm_fp8<1> + <2> on rank 0", "bound": "tensor",
                     "achieved": flops_rank0 / ((g1_ms + g2_ms) * 1e-3) / 1e12 if g1_ms > 0 else None,
                     "peak": fp8_peak.get("burst", 4500.0), "unit": "TFLOP/s",
                     "frac": (flops_rank0 / ((g1_ms + g2_ms) * 1e-3) / 1e12 / fp8_peak.get("burst", 4500.0)) if g1_ms > 0 else None,
                     "frac_of_nominal_4500": (flops_rank0 / ((g1_ms + g2_ms) * 1e-3) / 1e12 / 4500.0) if g1_ms > 0 else None,
                     "peak_source": "measured (library's FP8 MMA loop, burst)" if fp8_peak else "nominal",
                     "traffic": int(g1_bytes * TRAFFIC_RATIO["gemm1"]), "kernel_ms": g1_ms + g2_ms,
                     "gemm1_hbm_gbs": g1_bytes / (g1_ms * 1e-3) / 1e9 if g1_ms > 0 else None,
                     "gemm1_hbm_frac": (g1_bytes / (g1_ms * 1e-3) / 1e9 / hbm) if g1_ms > 0 else None,
                     "algorithmic_flops": flops_rank0, "launches_timed": 1},
        "kernels": {"phase_ms_rank0": phases, "gemm1_ms": g1_ms, "gemm2_ms": g2_ms, "rows_per_gpu_max": rmax_v, "rows_per_gpu_mean": rsum_v / world,
                    "ep_impl": args.ep_impl,
                    "rank0_gemm_tflops": flops_rank0 / ((g1_ms + g2_ms) * 1e-3) / 1e12 if g1_ms > 0 else None,
                    "dispatched_tokens_this_gpu": int(recv_tokens),
                    "max_tokens_per_expert": int(counts.max()), "mean_tokens_per_expert": float(counts.mean()),
                    "rows_by_gpu": [int(v) for v in per_gpu],
                    "hot_gpu_gemm_tflops_lower_bound": flops_hot / (ms * 1e-3) / 1e12,
                    "fp8_peak_tflops_nominal": 4500.0, "fp8_peak_tflops_measured": fp8_peak},
    }
    if rank == 0:
        # the timed configuration itself (bf16 combine, this placement, Zipf bias) against the CPU emulation
        out, ids, _ = ep.forward(xq, xs)
        torch.cuda.synchronize()
        threads = oracle.host_threads()
        par = ep_parity_sample(b200, torch, oracle, layer, placement, world, xq, xs, out, ids,
                               min(args.cpu_tokens, 12), threads)
        cpu_s = par.pop("cpu_seconds")
        res["parity"] = par
        res["cpu_baseline"] = {"value": par["checked_tokens"] / cpu_s, "unit": "tokens/s", "cores": threads,
                               "kind": "port",
                               "sample": f"{par['checked_tokens']} seeded tokens of rank 0 (routing + 8 experts each) "
                                         f"through the fp32 CPU emulation, {cpu_s:.2f} s"}
    return res


def build_dsa(b200, torch, dev, seed):
    c = DSA
    rng = np.random.default_rng(seed)
    seq = rng.integers(c["seq_min"], c["seq_max"] + 1, c["B"])
    pages_per_seq = (seq + c["page"] - 1) // c["page"]
    total_pages = int(pages_per_seq.sum())
    N = total_pages * c["page"]
    kc = torch.empty((N, c["Dc"]), dtype=torch.bfloat16, device=dev)
    kp = torch.empty((N, c["Dp"]), dtype=torch.bfloat16, device=dev)
    v = torch.empty((N, c["Dc"]), dtype=torch.bfloat16, device=dev)
    b200.fill_normal_(kc, seed + 1, 0.5)
    b200.fill_normal_(kp, seed + 2, 0.5)
    b200.fill_normal_(v, seed + 3, 0.5)
    qn = torch.empty((c["B"], c["H"], c["Dc"]), dtype=torch.bfloat16, device=dev)
    qp = torch.empty((c["B"], c["H"], c["Dp"]), dtype=torch.bfloat16, device=dev)
    b200.fill_normal_(qn, seed + 4, 1.0)
    b200.fill_normal_(qp, seed + 5, 1.0)
    # block table: physical pages handed out by a random permutation
    page_perm = torch.from_numpy(rng.permutation(total_pages)).to(dev)
    starts = np.concatenate([[0], np.cumsum(pages_per_seq)[:-1]])
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    idx_sets = []
    for _ in range(4):
        idx = torch.empty((c["B"], c["S"]), dtype=torch.int32, device=dev)
        for b in range(c["B"]):
            pos = torch.randperm(int(seq[b]), generator=g, device=dev)[: c["S"]]      # distinct, unsorted
            phys = page_perm[int(starts[b]) + pos // c["page"]] * c["page"] + pos % c["page"]
            idx[b] = phys.to(torch.int32)
        idx_sets.append(idx)
    layer = b200.DsaDecodeLayer(kc, kp, v, c["page"])
    return layer, qn, qp, idx_sets, N, seq


def dsa_bytes():
    c = DSA
    e = 2
    # selected K/V rows and queries in bf16, output in fp32, 32-bit row indices
    return (c["B"] * c["S"] * (2 * c["Dc"] + c["Dp"]) * e + c["B"] * c["H"] * (c["Dc"] + c["Dp"]) * e
            + c["B"] * c["H"] * c["Dc"] * 4 + 4 * c["B"] * c["S"])


def bench_dsa(b200, torch, oracle, dev, args, sampler, do_cpu):
    c = DSA
    layer, qn, qp, idx_sets, N, seq = build_dsa(b200, torch, dev, 77)
    out = torch.empty((c["B"], c["H"], c["Dc"]), dtype=torch.float32, device=dev)
    steps = max(args.steps, 400)      # ~30 ms of decode steps, so that the clock sampler sees the timed region
    for i in range(max(args.warmup, 3)):
        layer.forward(qn, qp, idx_sets[i % 4], out)
    torch.cuda.synchronize()
    assert b200.device_status() == 0, "device-side wait timed out"
    b200.launch_count(reset=True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for i in range(steps):
        layer.forward(qn, qp, idx_sets[i % 4], out)      # a different row set each step: 4 x 285 MB > L2
    e1.record()
    torch.cuda.synchronize()
    sampler.stop()
    launches = b200.launch_count()
    us = e0.elapsed_time(e1) / steps * 1e3
    hbm, bf16_tf, which = measured_peaks()
    nbytes = dsa_bytes()
    res = {"metric": "dsa_decode_us_per_step", "value": us, "unit": "us/step", "higher_is_better": False,
           "steps": steps, "gpu_launches": int(launches), "dtype": "bf16",
           "config": {"workload": f"C4: B={c['B']} H={c['H']} Dc={c['Dc']} Dp={c['Dp']} top-k={c['S']}, paged bf16 "
                                  f"cache, page {c['page']}, seq_len U[{c['seq_min']},{c['seq_max']}] ({N} cache rows), "
                                  "indices unsorted",
                      "l2": f"4 index sets rotate; {c['B'] * c['S'] * (2 * c['Dc'] + c['Dp']) * 2 / 1e6:.0f} MB of rows "
                            "per step > 126 MB L2"},
           "roofline": {"kernel": "dsa_decode_pair128_kernel", "bound": "hbm", "achieved": nbytes / (us * 1e-6) / 1e9,
                        "peak": hbm, "unit": "GB/s", "frac": nbytes / (us * 1e-6) / 1e9 / hbm,
                        "traffic": int(nbytes * TRAFFIC_RATIO["dsa"]),
                        "peak_source": which, "algorithmic_bytes": int(nbytes),
                        "tflops": 2.0 * c["B"] * c["H"] * c["S"] * (2 * c["Dc"] + c["Dp"]) / (us * 1e-6) / 1e12,
                        "frac_of_nominal_8TBs": nbytes / (us * 1e-6) / 8e12}}
    if do_cpu:
        qn_h, qp_h = qn.cpu().pin_memory(), qp.cpu().pin_memory()
        idx_h = [i.cpu().pin_memory() for i in idx_sets]
        out_hs = [torch.empty(out.shape, dtype=torch.float32).pin_memory() for _ in range(2)]
        out_h = out_hs[0]
        for i in range(2):
            layer.forward_host(qn_h, qp_h, idx_h[i], out_h)
        t0 = time.perf_counter()
        for i in range(steps):
            layer.forward_host(qn_h, qp_h, idx_h[i % 4], out_h)
        e2e_sync_us = (time.perf_counter() - t0) / steps * 1e6
        for i in range(3):
            tk = layer.forward_host_async(qn_h, qp_h, idx_h[i % 4], out_hs[i % 2])
        tk.synchronize()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            tk = layer.forward_host_async(qn_h, qp_h, idx_h[i % 4], out_hs[i % 2])
        tk.synchronize()
        torch.cuda.synchronize()
        e2e_us = (time.perf_counter() - t0) / steps * 1e6
        res["e2e"] = {"value": e2e_us, "unit": "us/step",
                      "h2d_bytes_per_step": int(qn_h.numel() * 2 + qp_h.numel() * 2 + idx_h[0].numel() * 4),
                      "d2h_bytes_per_step": int(out_h.numel() * 4),
                      "mode": "double-buffered host pipeline (DsaDecodeLayer.forward_host_async)",
                      "synchronous_value": e2e_sync_us}
        # CPU oracle on a sample of queries (rows gathered on the device, computed on the host)
        nq = args.cpu_queries
        idx = idx_sets[0][:nq].long()
        layer.forward(qn, qp, idx_sets[0], out)
        torch.cuda.synchronize()
        as_u16 = lambda t: t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        gkc = as_u16(layer.kc[idx.reshape(-1)]); gkp = as_u16(layer.kp[idx.reshape(-1)]); gv = as_u16(layer.v[idx.reshape(-1)])
        threads = oracle.host_threads()
        oracle.set_threads(threads)
        t0 = time.perf_counter()
        ref = oracle.dsa_forward_bf16_gathered(as_u16(qn[:nq]), as_u16(qp[:nq]), gkc, gkp, gv, c["S"])
        cpu_s = time.perf_counter() - t0
        err = float(np.abs(out[:nq].cpu().numpy() - ref).max())
        res["cpu_baseline"] = {"value": cpu_s / nq * c["B"] * 1e6, "unit": "us/step", "cores": threads, "kind": "port",
                               "sample": f"{nq} of the 64 queries ({cpu_s:.2f} s), scaled to the batch of 64"}
        res["parity"] = {"checked_queries": nq, "max_abs_err": err, "ok": bool(err < 1e-2), "tolerance": "1e-2 abs"}
    del layer
    torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------------------------
# reference arm: the CPU implementation of the path (oracle port) on the host cores
# ---------------------------------------------------------------------------------------------
def reference_arm(args, world, rank):
    if rank != 0:
        return
    import oracle
    b200 = load_package()
    c = MOE
    threads = oracle.host_threads()      # the affinity mask, not OMP_NUM_THREADS (launchers set that to 1 per rank)
    oracle.set_threads(threads)
    n_tok, n_exp = args.cpu_tokens, 2
    # bounded sample of the same workload: n_tok tokens, their 8 experts mapped onto a pool of n_exp
    # generated experts (the CPU cost per token does not depend on which expert it is)
    def synth(seed, n, sigma, chunk=1 << 22):
        return np.concatenate([b200.synth_normal_host(seed, i, min(chunk, n - i), sigma) for i in range(0, n, chunk)])
    w1 = synth(1000, n_exp * 2 * c["I"] * c["D"], 0.02).reshape(n_exp, 2 * c["I"], c["D"])
    w2 = synth(2000, n_exp * c["D"] * c["I"], 0.02).reshape(n_exp, c["D"], c["I"])
    w1q, w1s = oracle.quant_weight(w1)
    w2q, w2s = oracle.quant_weight(w2)
    del w1, w2
    wg = b200.synth_normal_host(3000, 0, c["E"] * c["D"], c["D"] ** -0.5).reshape(c["E"], c["D"])
    bias = b200.synth_normal_host(3001, 0, c["E"], 0.01)
    x = b200.synth_normal_host(4000, 0, n_tok * c["D"], 1.0).reshape(n_tok, c["D"])
    xq, xs = oracle.quant_act(x)
    times = []
    for step in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        ids, wts = oracle.route_grouped(xq, xs, wg, bias, c["K"], c["n_group"], c["topk_group"], c["routed_scale"])
        oracle.moe_fp8_experts(xq, xs, w1q, w1s, w2q, w2s, (ids % n_exp).astype(np.int32), wts,
                               np.arange(n_tok, dtype=np.int32))
        dt = time.perf_counter() - t0
        if step >= args.warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    val = n_tok / sec
    line = {"impl": "reference", "metric": "fp8_moe_layer_tokens_per_s", "value": val, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": {"workload": "C3: FP8 block-scale MoE, D=7168 I=2048 E=256 top-8 (8 groups/top-4), T=4096; "
                                   f"each step = {n_tok} tokens of it on the host"},
            "cpu_baseline": {"value": val, "unit": "tokens/s", "cores": threads, "kind": "port",
                             "sample": f"{n_tok} tokens per step (routing + 8 experts each), fp32 CPU emulation of "
                                       "the FP8 sequence; the reference's own CPU code is fp32-only and has no "
                                       f"FP8 / grouped-routing path; the tokens' experts are mapped onto a pool of {n_exp} "
                                       "generated experts (88 MB of weights, partly cache-resident, which favours the CPU)"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-dsa", action="store_true")
    ap.add_argument("--skip-moe", action="store_true")
    ap.add_argument("--cpu-tokens", type=int, default=96)
    ap.add_argument("--cpu-queries", type=int, default=16)
    ap.add_argument("--pow2-scales", action="store_true",
                    help="variant run, not the headline: all weights and activations quantised with power-of-two "
                         "scales and the layer run with MOE_POW2_SCALES (hardware block-scaled MMA), at any N")
    ap.add_argument("--skip-pow2", action="store_true",
                    help="skip the secondary measurement of the power-of-two-scale variant of the MoE layer")
    ap.add_argument("--route-only", action="store_true",
                    help="run only the routing call of the MoE layer at the full token count (profiler captures)")
    ap.add_argument("--small", action="store_true",
                    help="profiling-sized case of the same kernels (32 experts, 512 tokens; 16 queries, short caches): "
                         "inputs still exceed L2 but only ~2 GB live on the device; not a bench value")
    ap.add_argument("--moe-tiles", default="auto", choices=["auto", "single", "pair"],
                    help="tile shape of the grouped GEMMs: 128-row tiles on single CTAs, 256-row tiles on CTA pairs, "
                         "or the library's own choice by rows per expert")
    ap.add_argument("--ep-impl", default="peer", choices=["peer", "nccl"],
                    help="expert-parallel data plane (N > 1): 'peer' = the library's own kernels over peer memory "
                         "(b200_ep_*), 'nccl' = torch.distributed all-to-alls around the kernels (the baseline)")
    ap.add_argument("--ep-placement", default="balanced", choices=["balanced", "strided", "contiguous"],
                    help="expert placement of the expert-parallel layer (N > 1)")
    args = ap.parse_args()
    global EP_PLACEMENT, MOE_FLAGS, POW2_SCALES
    EP_PLACEMENT = args.ep_placement
    MOE_FLAGS = {"auto": 0, "single": 4, "pair": 8}[args.moe_tiles]
    POW2_SCALES = bool(args.pow2_scales)
    if POW2_SCALES:
        MOE_FLAGS |= 32          # MOE_POW2_SCALES
        args.skip_pow2 = True
    if args.small:
        MOE.update(T=512, E=32, n_group=4, topk_group=2)
        DSA.update(B=16, seq_min=8192, seq_max=16384)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, world, rank)
        return

    import torch
    import oracle            # the checker for the CPU-baseline / parity leg only
    b200 = load_package()
    b200.lib()               # fail loudly when the CUDA library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    if args.route_only:
        if rank == 0:
            bench_route_only(b200, torch, dev, args)
        return
    sampler = ClockSampler(local_rank)

    if args.skip_moe:
        moe = {"value": None, "ms_per_step": None, "gpu_launches": 0}
    elif world == 1:
        moe = bench_moe_single(b200, torch, oracle, dev, args, sampler)
    else:
        moe = bench_moe_ep(b200, torch, oracle, dist, dev, args, world, rank, sampler)
    clocks = sampler.summary()
    dsa = None
    if not args.skip_dsa:
        s2 = ClockSampler(local_rank)
        dsa = bench_dsa(b200, torch, oracle, dev, args, s2, do_cpu=(rank == 0))
        dsa["clocks"] = s2.summary()
        if world > 1:
            t = torch.tensor([dsa["value"]], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dsa["value"] = float(t.item())
            dsa["replicas"] = world
    if rank == 0:
        c = MOE
        line = {"metric": "fp8_moe_layer_tokens_per_s", "value": moe["value"], "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": moe["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3",
                "data": "synthetic",
                "config": {"workload": ("profiling-sized case, not a bench value: " if args.small else "")
                           + ("VARIANT with power-of-two (UE8M0) scales, not the headline configuration: " if POW2_SCALES else "")
                           + ("C3" if world == 1 else "C5") + f": FP8 block-scale MoE layer, D={c['D']} I={c['I']} "
                           f"E={c['E']} top-{c['K']} ({c['n_group']} groups / top-{c['topk_group']}), sigmoid+bias scoring, "
                           f"routed_scaling 2.5, T={c['T']} per GPU"
                           + ("" if world == 1 else f", experts sharded over {world} GPUs ({EP_PLACEMENT} placement), Zipf(1.1) load"),
                           "tokens_per_gpu": c["T"], "parallelism": "single" if world == 1 else f"ep{world}",
                           "l2": "11.3 GB of FP8 weights stream every step (inputs > 126 MB L2)"},
                "clocks": clocks, "gpu_launches": moe.get("gpu_launches", 0)}
        for k in ("e2e", "roofline", "roofline_gemm2", "roofline_routing", "cpu_baseline", "parity", "kernels"):
            if k in moe:
                line[k] = moe[k]
        if dsa is not None:
            line["dsa"] = dsa
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
