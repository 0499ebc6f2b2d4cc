"""Layer objects a serving loop would hold: weights / caches stay resident in HBM, one
``forward_host`` call moves a step's inputs from pinned host memory, runs the CUDA path and
brings the result back (the end-to-end path the benchmark times).  ``forward_host_async`` is the
same call without the final wait: steps are double-buffered on the device, so the input copy of
step n+1 and the output copy of step n-1 run on their own streams under the kernels of step n
(PCIe traffic, not the kernels, bounds a synchronous call)."""
import torch

from . import (DsaConfig, MoeFp8Config, SCORE_SIGMOID_GROUPED, dsa_forward_bf16, moe_fp8_experts,
               moe_fp8_experts_packed, moe_fp8_forward, moe_fp8_forward_packed, moe_fp8_pack_weights, moe_route_fp8)


class HostPipeline:
    """Double-buffered host <-> device staging around a device computation.

    ``submit(host_inputs, host_output, compute)`` copies the pinned host inputs into the next
    slot's device buffers on a copy-in stream, runs ``compute(*device_inputs, device_output)`` on
    the caller's current stream once they have arrived, and copies the result to ``host_output``
    on a copy-out stream.  A slot is reused only after its previous computation has consumed the
    inputs and its previous output copy has finished (events, no host synchronisation).  The host
    buffers of a step must stay untouched until ``wait(ticket)`` returns."""

    def __init__(self, device, depth=2):
        self.device = device
        self.depth = depth
        self.s_in = torch.cuda.Stream(device=device)
        self.s_out = torch.cuda.Stream(device=device)
        self.slots = {}
        self.turn = 0

    def _slot(self, key, host_inputs, host_output):
        if key not in self.slots:
            mk = lambda h: torch.empty(h.shape, dtype=h.dtype, device=self.device)
            self.slots[key] = [{"in": [mk(h) for h in host_inputs], "out": mk(host_output),
                                "consumed": None, "copied_out": None} for _ in range(self.depth)]
        slot = self.slots[key][self.turn % self.depth]
        self.turn += 1
        return slot

    def submit(self, host_inputs, host_output, compute):
        key = tuple((tuple(h.shape), h.dtype) for h in host_inputs) + (tuple(host_output.shape),)
        slot = self._slot(key, host_inputs, host_output)
        main = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.s_in):
            if slot["consumed"] is not None:
                self.s_in.wait_event(slot["consumed"])         # the slot's previous computation read its inputs
            for d, h in zip(slot["in"], host_inputs):
                d.copy_(h, non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(self.s_in)
        main.wait_event(arrived)
        if slot["copied_out"] is not None:
            main.wait_event(slot["copied_out"])                # the slot's previous result has left the device
        compute(*slot["in"], slot["out"])
        done = torch.cuda.Event()
        done.record(main)
        slot["consumed"] = done
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            host_output.copy_(slot["out"], non_blocking=True)
            left = torch.cuda.Event()
            left.record(self.s_out)
        slot["copied_out"] = left
        return left

    @staticmethod
    def wait(ticket):
        ticket.synchronize()


class MoeFp8Layer:
    """FP8 block-scale MoE layer (extends moe_forward, kernels/moe/naive_moe.cu:400-471)."""

    def __init__(self, gate_w, bias, w1q, w1s, w2q, w2s, top_k, scoring=SCORE_SIGMOID_GROUPED, n_group=8,
                 topk_group=4, routed_scale=2.5, flags=0):
        self.gate_w, self.bias = gate_w, bias
        self.w1q, self.w1s, self.w2q, self.w2s = w1q, w1s, w2q, w2s
        self.E, self.D = gate_w.shape
        self.I = w2q.shape[-1]
        self.K = top_k
        self.scoring, self.n_group, self.topk_group, self.routed_scale = scoring, n_group, topk_group, routed_scale
        self.flags = flags          # MoeFp8Config.flags (MOE_DETERMINISTIC, tile shape overrides)
        self.w1p = self.w2p = None
        self._dev = {}
        self._pipe = None

    def pack(self, free_unpacked=False):
        """Pre-tile the weights (one contiguous 32 KB block per tile and K block) so the grouped GEMMs
        stream them at full DRAM rate.  One-time cost; the results do not change."""
        E_local = self.w1q.shape[0]
        self.w1p = torch.empty_like(self.w1q)
        self.w2p = torch.empty_like(self.w2q)
        moe_fp8_pack_weights(1, self.w1q, self.w1p, E_local, self.D, self.I)
        moe_fp8_pack_weights(2, self.w2q, self.w2p, E_local, self.D, self.I)
        if free_unpacked:
            torch.cuda.current_stream().synchronize()
            self.w1q = self.w2q = None
        return self

    def cfg(self, T, E=None, K=None):
        return MoeFp8Config(T, self.E if E is None else E, self.K if K is None else K, self.D, self.I, self.scoring,
                            self.n_group, self.topk_group, self.routed_scale, self.flags)

    def forward(self, xq, xs, out=None):
        T = xq.shape[0]
        if out is None:
            out = torch.empty((T, self.D), dtype=torch.float32, device=xq.device)
        if self.w1p is not None:
            moe_fp8_forward_packed(xq, xs, self.gate_w, self.bias, self.w1p, self.w1s, self.w2p, self.w2s, out,
                                   self.cfg(T))
        else:
            moe_fp8_forward(xq, xs, self.gate_w, self.bias, self.w1q, self.w1s, self.w2q, self.w2s, out, self.cfg(T))
        return out

    def route(self, xq, xs):
        T = xq.shape[0]
        ids = torch.empty((T, self.K), dtype=torch.int32, device=xq.device)
        wts = torch.empty((T, self.K), dtype=torch.float32, device=xq.device)
        moe_route_fp8(xq, xs, self.gate_w, self.bias, ids, wts, self.cfg(T))
        return ids, wts

    def local_experts(self, rq, rs, rid, rw):
        """Expert FFN for rows already dispatched to this rank: slot k of row r goes through local
        expert rid[r,k] scaled by rw[r,k]; slots with rid < 0 belong to other ranks and are skipped.
        Returns the per-row sum over the valid slots."""
        R, K = rid.shape
        y = torch.empty((R, self.D), dtype=torch.float32, device=rq.device)
        E_local = self.w1s.shape[0]
        if self.w1p is not None:
            moe_fp8_experts_packed(rq, rs, rid, rw, self.w1p, self.w1s, self.w2p, self.w2s, y,
                                   self.cfg(R, E=E_local, K=K))
        else:
            moe_fp8_experts(rq, rs, rid, rw, self.w1q, self.w1s, self.w2q, self.w2s, y, self.cfg(R, E=E_local, K=K))
        return y

    def forward_host(self, xq_host, xs_host, out_host):
        """xq_host/xs_host/out_host: pinned host tensors.  Returns after the result is on the host."""
        T = xq_host.shape[0]
        key = ("moe", T)
        if key not in self._dev:
            dev = self.gate_w.device
            self._dev[key] = (torch.empty(xq_host.shape, dtype=torch.uint8, device=dev),
                              torch.empty(xs_host.shape, dtype=torch.float32, device=dev),
                              torch.empty((T, self.D), dtype=torch.float32, device=dev))
        dq, ds, do = self._dev[key]
        dq.copy_(xq_host, non_blocking=True)
        ds.copy_(xs_host, non_blocking=True)
        self.forward(dq, ds, do)
        out_host.copy_(do, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    def forward_host_async(self, xq_host, xs_host, out_host):
        """Same as forward_host but returns at once with a ticket; `HostPipeline.wait(ticket)` (or
        `ticket.synchronize()`) returns when out_host holds the result.  Consecutive calls overlap their
        host copies with each other's kernels."""
        if self._pipe is None:
            self._pipe = HostPipeline(self.gate_w.device)
        return self._pipe.submit([xq_host, xs_host], out_host, lambda dq, ds, do: self.forward(dq, ds, do))


class DsaDecodeLayer:
    """bf16 sparse MLA decode (dsa_forward, kernels/dsa/naive_dsa.cu:435-474) over caches resident in HBM."""

    def __init__(self, kc, kp, v, page_size=64):
        self.kc, self.kp, self.v = kc, kp, v
        self.page_size = page_size
        self._dev = {}
        self._pipe = None

    def cfg(self, Q, H, S):
        return DsaConfig(Q, H, self.kc.shape[1], self.kp.shape[1], S, self.page_size, self.kc.shape[0])

    def forward(self, q_nope, q_pe, idx, out=None):
        Q, H, _ = q_nope.shape
        if out is None:
            out = torch.empty((Q, H, self.kc.shape[1]), dtype=torch.float32, device=q_nope.device)
        dsa_forward_bf16(q_nope, q_pe, self.kc, self.kp, self.v, idx, out, self.cfg(Q, H, idx.shape[1]))
        return out

    def forward_host(self, qn_host, qp_host, idx_host, out_host):
        key = tuple(qn_host.shape) + tuple(idx_host.shape)
        if key not in self._dev:
            dev = self.kc.device
            self._dev[key] = (torch.empty(qn_host.shape, dtype=torch.bfloat16, device=dev),
                              torch.empty(qp_host.shape, dtype=torch.bfloat16, device=dev),
                              torch.empty(idx_host.shape, dtype=torch.int32, device=dev),
                              torch.empty(out_host.shape, dtype=torch.float32, device=dev))
        dn, dp, di, do = self._dev[key]
        dn.copy_(qn_host, non_blocking=True)
        dp.copy_(qp_host, non_blocking=True)
        di.copy_(idx_host, non_blocking=True)
        self.forward(dn, dp, di, do)
        out_host.copy_(do, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    def forward_host_async(self, qn_host, qp_host, idx_host, out_host):
        """forward_host without the final wait (see MoeFp8Layer.forward_host_async)."""
        if self._pipe is None:
            self._pipe = HostPipeline(self.kc.device)
        return self._pipe.submit([qn_host, qp_host, idx_host], out_host,
                                 lambda dn, dp, di, do: self.forward(dn, dp, di, do))
