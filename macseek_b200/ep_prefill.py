"""Expert-parallel MoE prefill: tokens are sharded over the ranks (data parallel), experts are sharded expert-parallel
(rank r holds experts [r E/N, (r+1) E/N)), and one all-to-all dispatches every routed (token, expert) entry to the rank
that holds the expert; the grouped expert GEMMs run there on the received rows (now in local HBM), a second all-to-all
brings the expert outputs back, and every token adds its shared-expert output and its k routed outputs in fixed k order.
Semantics of the reference model's expert-parallel MoE (reference/inference/model.py:865-904) with the reference
kernels' deterministic per-token reduce (src/kernels/quant_moe_prefill.metal:330-344).

The exchange is a real data movement step of this path, so it uses the collective library (torch.distributed
all_to_all_single: NCCL over NVLink on GPUs, gloo in the CPU tests); everything else is rank-local.  An entry travels
as one message: its bf16 row (the prefill's hidden states are bf16), its expert id and its routing weight; expert outputs
come back as f32.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DispatchPlan:
    """Who sends what to whom for one prefill chunk on this rank.  Built from the local tokens' routing only."""

    def __init__(self, ids: torch.Tensor, w: torch.Tensor, n_experts: int, world: int):
        n, k = ids.shape
        per = n_experts // world
        flat_e = ids.reshape(-1).to(torch.int64)
        dest = flat_e // per
        # entries sorted by (destination rank, expert, entry index t * k + kk): the order they travel in
        key = dest * (n_experts * n * k) + flat_e * (n * k) + torch.arange(n * k, device=ids.device)
        self.order = torch.argsort(key)
        self.tok = (self.order // k).to(torch.int64)
        self.expert = flat_e[self.order].to(torch.int32)
        self.weight = w.reshape(-1)[self.order].to(torch.float32)
        self.send_counts = torch.bincount(dest, minlength=world).to(torch.int64)
        self.n, self.k, self.world = n, k, world
        # position of entry (t, kk) in the travel order, for the combine
        self.pos_of_entry = torch.empty(n * k, dtype=torch.int64, device=ids.device)
        self.pos_of_entry[self.order] = torch.arange(n * k, device=ids.device)


def _a2a(out, inp, out_splits, in_splits, group):
    dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=group)


def exchange_counts(plan: DispatchPlan, group=None):
    recv = torch.empty_like(plan.send_counts)
    dist.all_to_all_single(recv, plan.send_counts, group=group)
    return recv


def moe_prefill_ep(X: torch.Tensor, ids: torch.Tensor, w: torch.Tensor, n_experts: int, local_experts, shared_local,
                   Y: torch.Tensor, group=None, stats: dict | None = None):
    """Y[t] += shared(X[t]) + sum_k expert_{ids[t][k]}(X[t]) * w[t][k] for this rank's tokens.

    X [n][dim] (bf16-representable values, any float dtype), ids [n][k] global expert ids, w [n][k] routing weights.
    local_experts(rows_f32 [m][dim], expert_ids int32 [m] (sorted ascending), weights f32 [m]) -> f32 [m][dim]: the routed
    experts resident here applied to the received rows, row i by expert expert_ids[i], scaled by weights[i].
    shared_local(rows_f32 [n][dim]) -> f32 [n][dim] (or None): the replicated shared expert on the local tokens.
    stats (optional) receives the per-rank row counts."""
    world = dist.get_world_size(group)
    plan = DispatchPlan(ids, w, n_experts, world)
    recv_counts = exchange_counts(plan, group)
    sc, rc = plan.send_counts.tolist(), recv_counts.tolist()
    n_recv = int(sum(rc))
    dim = X.shape[1]
    dev = X.device
    # one message per entry: the bf16 row, then the expert id (int32) and the routing weight (f32) -- one all-to-all
    # instead of three
    rb = dim * 2
    send = torch.empty(plan.n * plan.k, rb + 8, dtype=torch.uint8, device=dev)
    send[:, :rb] = X[plan.tok].to(torch.bfloat16).contiguous().view(torch.uint8).reshape(-1, rb)
    send[:, rb:rb + 4] = plan.expert.contiguous().view(torch.uint8).reshape(-1, 4)
    send[:, rb + 4:] = plan.weight.contiguous().view(torch.uint8).reshape(-1, 4)
    recv = torch.empty(n_recv, rb + 8, dtype=torch.uint8, device=dev)
    _a2a(recv, send, rc, sc, group)
    recv_rows = recv[:, :rb].contiguous().view(torch.bfloat16).reshape(n_recv, dim)
    recv_e = recv[:, rb:rb + 4].contiguous().view(torch.int32).reshape(n_recv)
    recv_w = recv[:, rb + 4:].contiguous().view(torch.float32).reshape(n_recv)
    if stats is not None:
        stats["rows_sent"], stats["rows_received"] = int(sum(sc)), n_recv
    # local grouped GEMM over the received rows, expert-sorted (stable: ties keep the arrival order)
    by_expert = torch.argsort(recv_e.to(torch.int64), stable=True)
    z_sorted = local_experts(recv_rows[by_expert].float().contiguous(), recv_e[by_expert].contiguous(),
                             recv_w[by_expert].contiguous())
    z = torch.empty_like(z_sorted)
    z[by_expert] = z_sorted
    # combine: outputs return in the order the entries were sent
    back = torch.empty(plan.n * plan.k, dim, dtype=torch.float32, device=dev)
    _a2a(back, z.contiguous(), sc, rc, group)
    acc = Y
    if shared_local is not None:
        acc += shared_local(X.float().contiguous())
    zk = back[plan.pos_of_entry].reshape(plan.n, plan.k, dim)
    for kk in range(plan.k):                      # fixed k order for every token
        acc += zk[:, kk]
    return Y


class _Buffers:
    """Work buffers that grow on demand and are reused from call to call (the prefill kernels need their scratch zeroed
    once, at allocation, not per call)."""

    def __init__(self):
        self.scratch = None
        self.out = None

    def get(self, scratch_bytes, m, dim, device):
        if self.scratch is None or self.scratch.numel() < scratch_bytes:
            self.scratch = torch.zeros(int(scratch_bytes * 1.25) + 256, dtype=torch.uint8, device=device)
        if self.out is None or self.out.shape[0] < m or self.out.shape[1] != dim:
            self.out = torch.empty(int(m * 1.25) + 1, dim, dtype=torch.float32, device=device)
        out = self.out[:m]
        out.zero_()
        return self.scratch, out


def cuda_local_experts(lw, e):
    """local_experts callback over macseek_b200's grouped prefill kernels for a MoeLayerWeights holding this rank's
    experts: every received row is its own one-entry token."""
    from . import quant as q
    bufs = _Buffers()

    def run(rows, expert_ids, weights):
        m, dim = rows.shape
        if m == 0:
            return torch.zeros(0, dim, dtype=torch.float32, device=rows.device)
        used, counts = torch.unique_consecutive(expert_ids, return_counts=True)
        a = q.MoePrefillArgs(lw.dim, lw.inter)
        a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
        a.n_tokens, a.k_per_token, a.has_shared = m, 1, False
        offs = [0]
        for ex, c in zip(used.tolist(), counts.tolist()):
            s = q.ExpertSlot()
            s.gate, s.up, s.down = lw.expert_views(int(ex))
            a.slots.append(s)
            offs.append(offs[-1] + int(c))
        a.offs = offs
        a.tok = torch.arange(m, dtype=torch.int32, device=rows.device)
        a.wt = weights
        a.slot_of = torch.arange(m, dtype=torch.int32, device=rows.device)
        a.scratch, out = bufs.get(q.moe_prefill_scratch_bytes(m, m, len(a.slots), lw.dim, lw.inter), m, dim, rows.device)
        a.X, a.Y = rows, out
        q.encode_moe_prefill(e, a)
        return out            # valid until this callback's next call; consumed on the same stream before that
    return run


def cuda_shared_expert(lw, e):
    """shared_local callback: the replicated shared expert on the local tokens."""
    from . import quant as q
    bufs = _Buffers()

    def run(rows):
        n, dim = rows.shape
        a = q.MoePrefillArgs(lw.dim, lw.inter)
        a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
        a.n_tokens, a.k_per_token, a.has_shared = n, 1, True
        a.shared = lw.shared
        a.offs = [0]
        a.tok = torch.zeros(1, dtype=torch.int32, device=rows.device)
        a.wt = torch.zeros(1, dtype=torch.float32, device=rows.device)
        a.slot_of = torch.full((n,), -1, dtype=torch.int32, device=rows.device)
        a.scratch, out = bufs.get(q.moe_prefill_scratch_bytes(0, n, 0, lw.dim, lw.inter), n, dim, rows.device)
        a.X, a.Y = rows, out
        q.encode_moe_prefill(e, a)
        return out
    return run
