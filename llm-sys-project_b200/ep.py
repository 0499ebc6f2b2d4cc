"""Expert-parallel MoE layer: experts are split contiguously over the ranks of a
torch.distributed process group (rank g owns experts [g*E/W, (g+1)*E/W)); tokens stay on
their source rank.  One step is

    route (local kernel) -> counts all-to-all -> dispatch all-to-all (FP8 rows, 1x128
    scales, local expert id, router weight) -> grouped expert GEMMs on the owner (CUDA
    library, one "token" per received row, K = 1) -> combine all-to-all -> per-token sum.

The reference has no multi-GPU path; the oracle for this one is the single-GPU layer on
the concatenated tokens.  The collectives are torch.distributed (NCCL over NVLink on GPUs,
gloo in the CPU tests); the routing and expert computations are injected so that the
host-side plumbing can be exercised without a GPU.
"""
import torch
import torch.distributed as dist


def dispatch_plan(ids, experts_per_rank, world):
    """ids [T,K] global expert ids -> (order, send_counts).

    ``order`` lists the (token,slot) pairs t*K+k grouped by destination rank, stable in
    pair order inside a destination; ``send_counts[r]`` is the number of pairs going to r."""
    dest = torch.div(ids.reshape(-1), experts_per_rank, rounding_mode="floor").to(torch.int64)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world)
    return order, send_counts


class ExpertParallelMoe:
    def __init__(self, group, num_experts, top_k, route_fn, expert_fn, combine_dtype=torch.float32):
        """route_fn(xq, xs) -> (ids [T,K] int32, wts [T,K] f32) with global expert ids.
        expert_fn(rq [R,D] u8, rs [R,D/128] f32, re [R] int32 local ids, rw [R] f32) -> y [R,D] f32
        (already multiplied by the router weight)."""
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
        self.last_stats = {}

    def _a2a(self, send, send_counts, recv_counts):
        out = send.new_empty((int(sum(recv_counts)),) + tuple(send.shape[1:]))
        dist.all_to_all_single(out, send, output_split_sizes=recv_counts, input_split_sizes=send_counts,
                               group=self.group)
        return out

    def forward(self, xq, xs):
        T, D = xq.shape
        K = self.K
        ids, wts = self.route_fn(xq, xs)
        order, send_counts_t = dispatch_plan(ids, self.E_local, self.world)
        recv_counts_t = torch.empty_like(send_counts_t)
        dist.all_to_all_single(recv_counts_t, send_counts_t, group=self.group)
        send_counts = send_counts_t.tolist()
        recv_counts = recv_counts_t.tolist()
        pair_tok = torch.div(order, K, rounding_mode="floor")
        flat_ids = ids.reshape(-1)[order]
        send_e = (flat_ids - torch.div(flat_ids, self.E_local, rounding_mode="floor") * self.E_local).to(torch.int32)
        send_w = wts.reshape(-1)[order].contiguous()
        rq = self._a2a(xq.index_select(0, pair_tok), send_counts, recv_counts)
        rs = self._a2a(xs.index_select(0, pair_tok), send_counts, recv_counts)
        re = self._a2a(send_e.contiguous(), send_counts, recv_counts)
        rw = self._a2a(send_w, send_counts, recv_counts)
        R = rq.shape[0]
        self.last_stats = {"recv_rows": R, "send_counts": send_counts, "recv_counts": recv_counts}
        if R > 0:
            y = self.expert_fn(rq, rs, re, rw)
        else:
            y = torch.zeros((0, D), dtype=torch.float32, device=xq.device)
        y = y.to(self.combine_dtype)
        back = self._a2a(y, recv_counts, send_counts)            # rows come back in `order` order
        out = torch.zeros((T, D), dtype=torch.float32, device=xq.device)
        out.index_add_(0, pair_tok, back.to(torch.float32))
        return out, ids, wts
