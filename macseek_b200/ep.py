"""Expert-parallel host logic: which experts a rank holds and how the ranks' routed partial sums are combined.

Experts are split into contiguous ranges, rank r of N holding [r * E / N, (r + 1) * E / N) (the reference model's
`n_local_experts` split, model.py:869-872).  Router, shared expert and every dense/attention weight are replicated, so
all ranks see the same ids and weights; each rank's MoE kernels compute the routed experts it holds into a partial y and
the partials are summed (model.py:903-904).  Nothing here touches the CUDA library: it runs under any
torch.distributed backend.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def expert_range(n_experts: int, world: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the experts resident on `rank`."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank %d outside a world of %d" % (rank, world))
    if n_experts % world:
        raise ValueError("%d experts do not split evenly over %d ranks" % (n_experts, world))
    per = n_experts // world
    return rank * per, (rank + 1) * per


def local_slots(ids, lo: int, hi: int) -> list[int]:
    """Positions k of the router's top-k whose expert ids[k] is resident in [lo, hi) (host mirror of the kernels'
    on-GPU resolution; used by tests and byte models)."""
    return [k for k, e in enumerate(ids) if lo <= int(e) < hi]


def combine_routed(y_part: torch.Tensor, group=None) -> torch.Tensor:
    """Sum the ranks' routed partial outputs in place (one all-reduce of dim floats; 16 KB at dim 4096)."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(y_part, op=dist.ReduceOp.SUM, group=group)
    return y_part
