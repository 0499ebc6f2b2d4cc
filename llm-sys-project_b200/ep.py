"""Expert-parallel MoE layer: experts are split over the ranks of a torch.distributed process
group, contiguously (rank g owns experts [g*E/W, (g+1)*E/W)) or strided (rank g owns experts
g, g+W, ...); tokens stay on their source rank.  One step is

    route (local kernel)
    -> counts all-to-all
    -> dispatch all-to-all: every token goes ONCE to each rank that owns at least one of its
       selected experts (FP8 row, 1x128 scales, its K slots with local expert ids, -1 for slots
       owned elsewhere, and the router weights)
    -> grouped expert GEMMs on the owner (CUDA library; slots with id -1 are skipped), which
       also sums the owner's contributions per token
    -> combine all-to-all: one partial output row per (token, owner rank)
    -> per-token sum of the partial rows on the source rank.

Sending a token once per owner rank instead of once per selected expert cuts the dispatch
volume by the number of its experts that share a rank, and summing on the owner cuts the
combine volume (the large one: D fp32 per row) by the same factor.

The reference has no multi-GPU path; the oracle for this one is the single-GPU layer on
the concatenated tokens.  The collectives are torch.distributed (NCCL over NVLink on GPUs,
gloo in the CPU tests); the routing and expert computations are injected so that the
host-side plumbing can be exercised without a GPU.
"""
import torch
import torch.distributed as dist


def balanced_placement(counts, world):
    """Greedy load-balanced expert placement from per-expert row counts of a calibration batch: experts
    in descending load go to the least loaded rank that still has room (every rank gets E / world experts).
    Returns (owner [E], local [E]) int32 tensors; rank g's local expert j is the j-th expert assigned to it."""
    counts = torch.as_tensor(counts).to(torch.int64).cpu()
    E = counts.numel()
    cap = E // world
    load = [0] * world
    used = [0] * world
    owner = torch.empty(E, dtype=torch.int32)
    local = torch.empty(E, dtype=torch.int32)
    order = sorted(range(E), key=lambda e: (-int(counts[e]), e))
    for e in order:
        g = min((r for r in range(world) if used[r] < cap), key=lambda r: (load[r], r))
        owner[e], local[e] = g, used[g]
        used[g] += 1
        load[g] += int(counts[e])
    return owner, local


def expert_owner(ids, experts_per_rank, world, strided=False, maps=None):
    """Owner rank and local expert id of global expert ids: contiguous placement (expert e on rank
    e // experts_per_rank), strided (expert e on rank e % world, which spreads runs of hot experts) or
    mapped (maps = (owner [E], local [E]) tensors)."""
    ids = ids.to(torch.int64)
    if maps is not None:
        return maps[0].to(ids.device).to(torch.int64)[ids], maps[1].to(ids.device).to(torch.int64)[ids]
    if strided:
        return ids % world, torch.div(ids, world, rounding_mode="floor")
    owner = torch.div(ids, experts_per_rank, rounding_mode="floor")
    return owner, ids - owner * experts_per_rank


def dispatch_plan(ids, experts_per_rank, world, strided=False, maps=None):
    """ids [T,K] global expert ids -> (send_tok, send_rank, send_counts).

    Row i of the dispatch carries token ``send_tok[i]`` to rank ``send_rank[i]``; rows are
    grouped by destination rank and ascending in token inside a destination.
    ``send_counts[r]`` is the number of rows going to rank r."""
    T, K = ids.shape
    dest, _ = expert_owner(ids, experts_per_rank, world, strided, maps)                    # [T,K]
    need = torch.zeros((world, T), dtype=torch.bool, device=ids.device)
    tok = torch.arange(T, device=ids.device).repeat_interleave(K)
    need[dest.reshape(-1), tok] = True
    flat = need.reshape(-1).nonzero(as_tuple=False).squeeze(1)
    send_rank = torch.div(flat, T, rounding_mode="floor")
    send_tok = flat - send_rank * T
    send_counts = need.sum(dim=1)
    return send_tok, send_rank, send_counts


class ExpertParallelMoe:
    def __init__(self, group, num_experts, top_k, route_fn, expert_fn, combine_dtype=torch.float32,
                 placement="contiguous"):
        """placement: "contiguous" (rank g owns experts [g*E/W, (g+1)*E/W)), "strided" (rank g owns experts
        g, g+W, g+2W, ... in that local order) or a pair (owner [E], local [E]) of int32 tensors, e.g. from
        balanced_placement(); the caller shards the weights accordingly.
        route_fn(xq, xs) -> (ids [T,K] int32, wts [T,K] f32) with global expert ids.
        expert_fn(rq [R,D] u8, rs [R,D/128] f32, rid [R,K] int32 local ids or -1, rw [R,K] f32)
        -> y [R,D] f32: per received row the weighted sum over its valid slots."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if num_experts % self.world:
            raise ValueError("num_experts must be divisible by the world size")
        self.E = num_experts
        self.E_local = num_experts // self.world
        self.K = top_k
        self.route_fn = route_fn
        self.expert_fn = expert_fn
        self.combine_dtype = combine_dtype
        self.maps = None
        if isinstance(placement, (tuple, list)):
            owner, local = placement
            if owner.numel() != num_experts or local.numel() != num_experts:
                raise ValueError("placement maps must have one entry per expert")
            self.maps = (owner.to(torch.int32).contiguous(), local.to(torch.int32).contiguous())
            placement = "mapped"
        elif placement not in ("contiguous", "strided"):
            raise ValueError("placement must be 'contiguous', 'strided' or (owner, local) tensors")
        self.strided = placement == "strided"
        self._dev_maps = None
        self.last_stats = {}
        self._last_rid = None
        self.profile = False          # record CUDA events between the phases of a step (GPU only)
        self._marks = []

    def recv_pairs(self):
        """Number of (token, expert) pairs this rank computed in the last step (synchronises)."""
        return int((self._last_rid >= 0).sum().item())

    def _mark(self, name, ref):
        if self.profile and ref.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks.append((name, ev))

    def phase_ms(self):
        """Milliseconds per phase of the last profiled step (synchronises)."""
        if len(self._marks) < 2:
            return {}
        torch.cuda.synchronize()
        return {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(self._marks[:-1], self._marks[1:])}

    def _a2a(self, send, send_counts, recv_counts):
        out = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        dist.all_to_all_single(out, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.group)
        return out

    def forward(self, xq, xs):
        T, D = xq.shape
        K = self.K
        self._marks = []
        self._mark("start", xq)
        ids, wts = self.route_fn(xq, xs)
        self._mark("route", xq)
        if xq.is_cuda:
            # one kernel: rows per destination rank, their slots in local numbering, row of (rank, token)
            from . import ep_plan
            W = self.world
            send_tok_all = torch.empty((W * T,), dtype=torch.int32, device=xq.device)
            pos = torch.empty((W, T), dtype=torch.int32, device=xq.device)
            send_counts_t = torch.empty((W,), dtype=torch.int32, device=xq.device)
            slot_ids = torch.empty((W * T, K), dtype=torch.int32, device=xq.device)
            slot_w = torch.empty((W * T, K), dtype=torch.float32, device=xq.device)
            if self.maps is not None and self._dev_maps is None:
                self._dev_maps = (self.maps[0].to(xq.device), self.maps[1].to(xq.device))
            om, lm = self._dev_maps if self._dev_maps is not None else (None, None)
            ep_plan(ids, wts, self.E_local, W, send_tok_all, pos, send_counts_t, slot_ids, slot_w, strided=self.strided,
                    owner_map=om, local_map=lm)
            both = torch.empty((2, W), dtype=torch.int32, device=xq.device)
            both[0] = send_counts_t
            dist.all_to_all_single(both[1], send_counts_t, group=self.group)
            both_h = both.tolist()                                   # the step's one host synchronisation
            send_counts, recv_counts = both_h[0], both_h[1]
            Rs = sum(send_counts)
            send_tok = send_tok_all[:Rs]
            send_id, send_w = slot_ids[:Rs], slot_w[:Rs]
        else:
            pos = None
            send_tok, send_rank, send_counts_t = dispatch_plan(ids, self.E_local, self.world, self.strided, self.maps)
            recv_counts_t = torch.empty_like(send_counts_t)
            dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
            send_counts = send_counts_t.tolist()
            recv_counts = recv_counts_t.tolist()
            # the K slots of every dispatched row, in the destination's local numbering
            row_ids = ids.index_select(0, send_tok)
            owner, local = expert_owner(row_ids, self.E_local, self.world, self.strided, self.maps)
            mine = owner == send_rank.unsqueeze(1)
            send_id = torch.where(mine, local, torch.full_like(local, -1)).to(torch.int32)
            send_w = torch.where(mine, wts.index_select(0, send_tok),
                                 torch.zeros((), dtype=wts.dtype, device=wts.device))
        self._mark("plan+counts", xq)
        rq = self._a2a(xq.index_select(0, send_tok), send_counts, recv_counts)
        rs = self._a2a(xs.index_select(0, send_tok), send_counts, recv_counts)
        rid = self._a2a(send_id.contiguous(), send_counts, recv_counts)
        rw = self._a2a(send_w.contiguous(), send_counts, recv_counts)
        self._mark("dispatch", xq)
        R = rq.shape[0]
        self.last_stats = {"recv_rows": R, "send_counts": send_counts, "recv_counts": recv_counts}
        self._last_rid = rid
        if R > 0:
            y = self.expert_fn(rq, rs, rid, rw)
        else:
            y = torch.zeros((0, D), dtype=torch.float32, device=xq.device)
        self._mark("experts", xq)
        y = y.to(self.combine_dtype)
        back = self._a2a(y, recv_counts, send_counts)            # rows come back in dispatch order
        self._mark("combine", xq)
        if pos is not None:
            from . import ep_sum_rows
            out = torch.empty((T, D), dtype=torch.float32, device=xq.device)
            ep_sum_rows(back, pos, self.world, out)
        else:
            out = torch.zeros((T, D), dtype=torch.float32, device=xq.device)
            out.index_add_(0, send_tok, back.to(torch.float32))
        self._mark("sum", xq)
        return out, ids, wts


class PeerExpertParallelMoe:
    """The expert-parallel layer of the C ABI (``b200_ep_*``): same exchange scheme as ExpertParallelMoe,
    but the data plane is the library's own kernels over peer memory (rows are stored straight into the
    owner's receive buffers, partial rows straight back) and a step has no host synchronisation and no
    collective call.  ``group`` is only used once, to hand every rank the 64-byte handles of the other
    ranks' exchange buffers.  The layer's weights are this rank's experts in local order.

    placement: "contiguous" or a pair (owner [E], local [E]) as for ExpertParallelMoe.
    combine_dtype: torch.float16 = partial rows travel as fp16 values relative to the row's largest magnitude
    (plus that magnitude); torch.float32 = as they are."""

    def __init__(self, group, layer, num_experts, max_tokens, placement="contiguous", combine_dtype=torch.float16,
                 wait_limit_ms=0, loopback=False):
        import ctypes as C
        from . import EpConfig, _check, lib
        self._C, self._check, self._lib = C, _check, lib()
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        if loopback:                  # test aid: pretend to be rank 0 of two, with the peer mapped onto this rank
            self.world, self.rank = 2, 0
        self.layer = layer
        self.E, self.K, self.D, self.I = num_experts, layer.K, layer.D, layer.I
        self.max_tokens = max_tokens
        if combine_dtype not in (torch.float16, torch.float32):
            raise ValueError("combine_dtype: torch.float16 (row-scaled, the default) or torch.float32")
        flags = 0 if combine_dtype == torch.float16 else 2
        flags |= int(layer.flags) & (16 | 32)         # exact router logits, power-of-two scales: as for the plain layer
        cfg = EpConfig(self.rank, self.world, max_tokens, num_experts, layer.K, layer.D, layer.I, layer.scoring,
                       layer.n_group, layer.topk_group, layer.routed_scale, flags, int(wait_limit_ms))
        om = lm = None
        if isinstance(placement, (tuple, list)):
            own = placement[0].to(torch.int32).contiguous().cpu().numpy()
            loc = placement[1].to(torch.int32).contiguous().cpu().numpy()
            om, lm = own.ctypes.data_as(C.c_void_p), loc.ctypes.data_as(C.c_void_p)
            self._keep = (own, loc)
        elif placement != "contiguous":
            raise ValueError("placement must be 'contiguous' or (owner, local) tensors")
        self._h = C.c_void_p()
        handle = (C.c_char * 64)()
        _check(self._lib.b200_ep_create(C.byref(self._h), C.byref(cfg), om, lm, handle), "b200_ep_create")
        if loopback:
            _check(self._lib.b200_ep_connect_loopback(self._h), "b200_ep_connect_loopback")
        elif self.world > 1:
            mine = torch.frombuffer(bytearray(handle.raw), dtype=torch.uint8).clone()
            gathered = [None] * self.world
            dist.all_gather_object(gathered, mine.tolist(), group=group)
            allh = bytes(b for h in gathered for b in h)
            _check(self._lib.b200_ep_connect(self._h, allh), "b200_ep_connect")
        else:
            _check(self._lib.b200_ep_connect(self._h, None), "b200_ep_connect")

    def forward(self, xq, xs, out=None, want_routing=True):
        C = self._C
        T = xq.shape[0]
        if out is None:
            out = torch.empty((T, self.D), dtype=torch.float32, device=xq.device)
        ids = wts = None
        if want_routing:
            ids = torch.empty((T, self.K), dtype=torch.int32, device=xq.device)
            wts = torch.empty((T, self.K), dtype=torch.float32, device=xq.device)
        L = self.layer
        packed = L.w1p is not None
        w1, w2 = (L.w1p, L.w2p) if packed else (L.w1q, L.w2q)
        p = lambda t: C.c_void_p(0 if t is None else t.data_ptr())
        self._check(self._lib.b200_ep_forward(self._h, int(T), p(xq), p(xs), p(L.gate_w), p(L.bias), p(w1), p(L.w1s),
                                              p(w2), p(L.w2s), 1 if packed else 0, p(out), p(ids), p(wts),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)), "b200_ep_forward")
        return out, ids, wts

    def stats(self):
        """(status, send_counts, recv_counts) of the last step; synchronises the current stream."""
        C = self._C
        st = C.c_int(0)
        sc, rc = (C.c_int * self.world)(), (C.c_int * self.world)()
        self._check(self._lib.b200_ep_stats(self._h, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(st),
                                            sc, rc), "b200_ep_stats")
        return st.value, list(sc), list(rc)

    def phase_profile(self, enable=True):
        """Benchmark hook: switch the phase timeline on / off; returns the last step's phase times in ms (a dict)
        when it was on."""
        C = self._C
        ms = (C.c_float * 6)()
        self._check(self._lib.b200_ep_phase_profile(self._h, 1 if enable else 0, ms), "b200_ep_phase_profile")
        names = ("route_plan", "dispatch", "wait_senders", "local_experts", "push", "combine_incl_wait")
        return {n: float(v) for n, v in zip(names, ms)}

    def workspace(self):
        """Handle of the object's workspace (for moe_fp8_profile / moe_fp8_profile_read)."""
        return self._lib.b200_ep_workspace(self._h)

    def close(self):
        if self._h:
            self._lib.b200_ep_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
