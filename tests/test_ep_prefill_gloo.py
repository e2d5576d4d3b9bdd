"""Expert-parallel prefill host logic on CPU: gloo ranks shard the tokens, dispatch every routed (token, expert) entry
to the rank holding the expert with all-to-all, apply a simple per-expert map there, bring the outputs back and reduce
per token in fixed k order.  With experts that are plain per-expert matrices the result must equal the single-process
computation exactly (bf16-representable inputs travel losslessly)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

N, DIM, E, K = 96, 32, 8, 3


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _case():
    g = torch.Generator().manual_seed(3)
    X = torch.randn(N, DIM, generator=g).to(torch.bfloat16).float()
    bias = -1.1 * torch.log(torch.arange(1, E + 1, dtype=torch.float32))      # skewed expert popularity
    logits = torch.randn(N, E, generator=g) + bias
    ids = torch.topk(logits, K, dim=1).indices
    w = torch.softmax(torch.gather(logits, 1, ids), dim=1)
    mats = torch.randn(E, DIM, DIM, generator=g) * 0.1
    shared = torch.randn(DIM, DIM, generator=g) * 0.1
    Y0 = torch.randn(N, DIM, generator=g)
    return X, ids, w, mats, shared, Y0


def _reference(X, ids, w, mats, shared, Y0):
    Y = Y0.clone()
    Y += X @ shared.T
    for kk in range(K):
        for t in range(N):
            Y[t] += (mats[ids[t, kk]] @ X[t]) * w[t, kk]
    return Y


def _rank_main(rank, world, port, out):
    from macseek_b200 import ep_prefill
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        X, ids, w, mats, shared, Y0 = _case()
        per_tok, per_exp = N // world, E // world
        sl = slice(rank * per_tok, (rank + 1) * per_tok)

        def local_experts(rows, expert_ids, weights):
            assert torch.all(expert_ids[1:] >= expert_ids[:-1])                        # expert-sorted
            assert torch.all((expert_ids >= rank * per_exp) & (expert_ids < (rank + 1) * per_exp))   # only experts held here
            return torch.stack([(mats[int(e)] @ r) * wt for r, e, wt in zip(rows, expert_ids, weights)]) if len(rows) else rows

        stats = {}
        Y = Y0[sl].clone()
        ep_prefill.moe_prefill_ep(X[sl], ids[sl], w[sl], E, local_experts, lambda r: r @ shared.T, Y, stats=stats)
        got = [torch.zeros_like(Y) for _ in range(world)]
        dist.all_gather(got, Y)
        rows = [None] * world
        dist.all_gather_object(rows, stats["rows_received"])
        if rank == 0:
            out.put((torch.cat(got).numpy(), rows))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 4))
def test_dispatch_combine_equals_single_process(world):
    X, ids, w, mats, shared, Y0 = _case()
    want = _reference(X, ids, w, mats, shared, Y0).numpy()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    got, rows = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sum(rows) == N * K and max(rows) > min(rows)          # every entry went somewhere; the load is skewed
    assert np.max(np.abs(got - want)) <= 1e-5 * np.max(np.abs(want))
