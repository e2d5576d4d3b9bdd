"""Expert-parallel host logic on CPU: two gloo ranks each evaluate (with the oracle) only the routed experts they hold
(rank 0 also the replicated shared expert), sum their partial outputs through macseek_b200.ep.combine_routed, and must
reproduce the single-rank oracle result.  Mirrors what the GPU ranks do per layer (router replicated, one partial per
rank all-reduced and added to the hidden state)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle_lib as ol
import synth

D, I, E, K = 512, 256, 8, 4


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _case():
    G = [synth.random_weights(ol.IQ1_S, I, D, 10 + 3 * e) for e in range(E)]
    U = [synth.random_weights(ol.IQ1_S, I, D, 11 + 3 * e) for e in range(E)]
    Dn = [synth.random_weights(ol.IQ2_XXS, D, I, 12 + 3 * e) for e in range(E)]
    sh = (synth.random_weights(ol.Q8_0, I, D, 900), synth.random_weights(ol.Q8_0, I, D, 901),
          synth.random_weights(ol.Q8_0, D, I, 902))
    x = synth.randn(D, 5)
    y0 = synth.randn(D, 6)
    logits = synth.randn(E, 7)
    return G, U, Dn, sh, x, y0, logits


def _rank_main(rank, world, port, out):
    from macseek_b200 import ep
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = ol.Oracle()
        G, U, Dn, sh, x, y0, logits = _case()
        ids, w = orc.router(logits, np.zeros(E, np.float32), K, score_fn=1, route_scale=1.0)   # replicated
        lo, hi = ep.expert_range(E, world, rank)
        mine = ep.local_slots(ids, lo, hi)
        # routed experts resident here -- and, on rank 0 only, the replicated shared expert -- into a zero partial
        mats = [ids[k] for k in mine]
        gg, uu, dd = [G[m] for m in mats], [U[m] for m in mats], [Dn[m] for m in mats]
        with_shared = rank == 0
        if with_shared:
            gg, uu, dd = gg + [sh[0]], uu + [sh[1]], dd + [sh[2]]
        _, part, _, _ = orc.moe_decode(D, I, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, gg, uu, dd, w[mine] if mine else None,
                                       x, np.zeros(D), has_shared=with_shared)
        t = torch.from_numpy(np.asarray(part, dtype=np.float64))
        ep.combine_routed(t)
        y = np.asarray(y0, dtype=np.float64) + t.numpy()       # every rank adds the combined partial to its hidden state
        gathered = [torch.zeros(D, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(y))
        if rank == 0:
            _, want, mag, _ = orc.moe_decode(D, I, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, [G[i] for i in ids] + [sh[0]],
                                             [U[i] for i in ids] + [sh[1]], [Dn[i] for i in ids] + [sh[2]], w, x, y0,
                                             has_shared=True)
            err = float(np.max(np.abs(y - want) / mag))
            same = all(np.array_equal(gathered[0].numpy(), g.numpy()) for g in gathered)
            covered = sorted(k for r in range(world) for k in ep.local_slots(ids, *ep.expert_range(E, world, r)))
            out.put((err, same, covered == list(range(K))))
    finally:
        dist.destroy_process_group()


def test_expert_range_partitions():
    from macseek_b200 import ep
    for world in (1, 2, 4, 8):
        r = [ep.expert_range(384, world, k) for k in range(world)]
        assert r[0][0] == 0 and r[-1][1] == 384
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        assert all(hi - lo == 384 // world for lo, hi in r)
    with pytest.raises(ValueError):
        ep.expert_range(384, 5, 0)
    with pytest.raises(ValueError):
        ep.expert_range(384, 2, 2)


def test_two_rank_combine_matches_single_rank():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err, same, covered = out.get(timeout=10)
    assert covered, "every routed slot must be owned by exactly one rank"
    assert same, "ranks disagree on the combined output"
    assert err < 1e-12, err


def _exchange_main(rank, world, port, out, skip_rank, skip_epoch):
    """Three epochs of the host exchange; rank `skip_rank` does not publish in epoch `skip_epoch` (None: every rank
    always publishes)."""
    from macseek_b200 import ep
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=60))
    ex = ep.HostExchange(store, world, rank)
    h = torch.zeros(8, dtype=torch.float64)
    statuses = []
    for epoch in range(3):
        part = torch.full((8,), float((rank + 1) * 10 ** epoch), dtype=torch.float32)
        if not (rank == skip_rank and epoch == skip_epoch):
            ex.publish(part)
        st = ex.combine(h, timeout_s=1.0 if skip_rank is not None else 20.0)
        statuses.append(st)
        if st:
            break
    out.put((rank, statuses, h.tolist()))
    # the store's master (rank 0) leaves only after every rank has reported; the others need the store no more once
    # their own report is in (polling it further would race with the master's exit)
    store.add("done", 1)
    while rank == 0 and int(store.add("done", 0)) < world:
        __import__("time").sleep(0.01)


def _run_exchange(world, skip_rank, skip_epoch):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_exchange_main, args=(r, world, port, out, skip_rank, skip_epoch)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(out.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return res


def test_host_exchange_sums_in_rank_order_over_epochs():
    res = _run_exchange(2, None, None)
    for rank, statuses, h in res:
        assert statuses == [0, 0, 0]
        assert h == [3.0 + 30.0 + 300.0] * 8              # (1 + 2) * (1 + 10 + 100), identical on every rank


def test_host_exchange_missing_contribution_sets_status_3_and_returns():
    """Rank 1 skips its contribution in the second epoch: every rank's bounded wait runs out, reports status 3 (the
    device status word's value for an expired peer wait), leaves h as the first epoch made it, and returns."""
    res = _run_exchange(2, 1, 1)
    for rank, statuses, h in res:
        assert statuses == [0, 3]
        assert h == [3.0] * 8
