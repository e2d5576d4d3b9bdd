"""GPU parity of the MoE prefill (grouped expert GEMMs on tcgen05) against the reference's own check
(tests/test_quant_moe_prefill.mm): half-emulated reference error <= 1e-3, pure-F32 reference error <= 5e-3, both
normalised by the summed magnitudes, and run-to-run bit identity.  Routing patterns follow the reference's test
(:70-110): a popular expert that spans several tiles, explicit expert sizes around the tile boundaries, Zipf."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


def r16(a):
    return a.astype(np.float16).astype(np.float64)


SIZES = [1, 1, 2, 15, 16, 17, 31, 32, 33, 47, 48, 49, 63, 64, 65, 100, 129, 200, 300]


def make_routing(kind, n, k, n_exp, seed):
    rng = np.random.default_rng(seed)
    rt = [[] for _ in range(n)]
    if kind == "popular":          # slot 0 -> expert 0 for every token, other slots random distinct
        for t in range(n):
            perm = rng.permutation(np.arange(1, n_exp))
            rt[t] = [0] + [int(v) for v in perm[:k - 1]]
    elif kind == "sizes":          # expert 0 takes every token, the rest have the listed sizes
        for t in range(n):
            rt[t].append(0)
        nxt = 0
        for j in range(1, n_exp):
            for _ in range(SIZES[j - 1]):
                t = nxt
                while len(rt[t]) >= k:
                    t = (t + 1) % n
                rt[t].append(j)
                nxt = (t + 7) % n
    else:                          # Zipf(0.8) popularity, k distinct experts per token
        perm = rng.permutation(n_exp)
        pw = np.zeros(n_exp)
        pw[perm] = 1.0 / np.power(np.arange(1, n_exp + 1), 0.8)
        for t in range(n):
            rt[t] = [int(v) for v in rng.choice(n_exp, size=k, replace=False, p=pw / pw.sum())]
    rw = [[0.1 + 0.2 * ((t * 7 + kk * 3) % 5) / 5 for kk in range(len(rt[t]))] for t in range(n)]
    offs, tok, wt = [0] * (n_exp + 1), [], []
    slot_of = -np.ones(n * k, dtype=np.int32)
    for j in range(n_exp):
        offs[j] = len(tok)
        for t in range(n):
            for kk, e in enumerate(rt[t]):
                if e == j:
                    slot_of[t * k + kk] = len(tok)
                    tok.append(t)
                    wt.append(rw[t][kk])
    offs[n_exp] = len(tok)
    return offs, np.array(tok, np.int32), np.array(wt, np.float32), slot_of


# (gate/up type, down type, shared type, n, k, n_exp, shared, routing, tokens checked (0 = all), dim, inter)
# The first three cases use the reference's layer shape (5120 / 2304); the many-expert routings run on a smaller layer so
# that the CPU reference stays cheap (the contraction still spans 16 / 8 K-blocks and several weight-row tiles).
CASES = [
    (ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 80, 2, 5, True, "popular", 0, 5120, 2304),
    (ol.IQ2_XXS, ol.IQ2_XXS, ol.Q8_0, 70, 2, 4, True, "popular", 0, 5120, 2304),
    (ol.IQ1_S, ol.IQ2_XXS, ol.Q6_K, 40, 3, 4, False, "popular", 0, 5120, 2304),
    (ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 600, 6, 20, True, "sizes", 40, 1024, 512),
    (ol.IQ2_XXS, ol.IQ1_S, ol.Q8_0, 256, 6, 64, True, "zipf", 40, 1024, 512),
    (ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 300, 8, 12, True, "zipf", 30, 4096, 2048),      # the benchmark's layer shape
]


@pytest.mark.parametrize("c", CASES, ids=lambda c: "%s-%s-%s-n%d-k%d-e%d-%s" % (ol.TYPE_NAMES[c[0]], ol.TYPE_NAMES[c[1]], ol.TYPE_NAMES[c[2]], c[3], c[4], c[5], c[7]))
def test_moe_prefill_reference_cases(orc, c):
    from macseek_b200 import quant as q
    from macseek_b200.core import Enc
    gu, dn, sh, n, k, n_exp, shared, kind, n_check, D, I = c
    offs, tok, wt, slot_of = make_routing(kind, n, k, n_exp, 42 + n)
    total = offs[-1]
    ne_all = n_exp + (1 if shared else 0)
    G, U, Dn = [], [], []
    for j in range(ne_all):
        tg, td = (sh, sh) if j == n_exp else (gu, dn)
        G.append(synth.random_weights(tg, I, D, 500 + 3 * j))
        U.append(synth.random_weights(tg, I, D, 501 + 3 * j))
        Dn.append(synth.random_weights(td, D, I, 502 + 3 * j))
    X = synth.randn(n * D, 9).reshape(n, D)
    Y0 = synth.randn(n * D, 10).reshape(n, D)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    a = q.MoePrefillArgs(D, I)
    a.t_gate_up, a.t_down, a.t_shared = gu, dn, sh
    a.n_tokens, a.k_per_token, a.has_shared = n, k, shared
    keep = []
    for j in range(ne_all):
        s = q.ExpertSlot()
        s.gate, s.up, s.down = dev(G[j]), dev(U[j]), dev(Dn[j])
        keep.append(s)
        if j == n_exp:
            a.shared = s
        else:
            a.slots.append(s)
    a.offs = offs
    a.tok, a.wt, a.slot_of = dev(tok), dev(wt), dev(slot_of)
    a.X = dev(X)
    a.scratch = torch.zeros(q.moe_prefill_scratch_bytes(total, n, n_exp, D, I), dtype=torch.uint8, device="cuda")
    e = Enc()
    outs = []
    for _ in range(2):
        a.Y = dev(Y0)
        q.encode_moe_prefill(e, a)
        e.wait()
        outs.append(a.Y.cpu().numpy())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32)), "repeat differs"
    got = outs[0].astype(np.float64)
    # tokens to check
    if n_check <= 0:
        chk = list(range(n))
    else:
        on = np.zeros(n, bool)
        for j in range(n_exp):
            if offs[j + 1] - offs[j] <= 2:
                on[tok[offs[j]:offs[j + 1]]] = True
        for t in (0, 15, 16, 31, 32, 47, 48, 63, 64, 65, 127, 128, 511, 512, 513, n - 1):
            if t < n:
                on[t] = True
        on[np.random.default_rng(1).integers(0, n, n_check)] = True
        chk = [t for t in range(n) if on[t]]
    ci = -np.ones(n, dtype=np.int64)
    ci[chk] = np.arange(len(chk))
    yh = Y0[chk].astype(np.float64)
    yf = yh.copy()
    ym = np.abs(yh)
    for j in range(ne_all):
        if j == n_exp:
            toks, ws = np.array(chk), np.ones(len(chk))
        else:
            ent = [i for i in range(offs[j], offs[j + 1]) if ci[tok[i]] >= 0]
            toks, ws = tok[ent], wt[ent].astype(np.float64)
        if len(toks) == 0:
            continue
        tg, td = (sh, sh) if j == n_exp else (gu, dn)
        wg = orc.dequant(tg, G[j], I * D).reshape(I, D).astype(np.float64)
        wu = orc.dequant(tg, U[j], I * D).reshape(I, D).astype(np.float64)
        wd = orc.dequant(td, Dn[j], I * D).reshape(D, I).astype(np.float64)
        for hv in (0, 1):
            xin = X[toks].astype(np.float64)
            if hv:
                xin = r16(xin)
            g = xin @ (r16(wg) if hv else wg).T
            u = xin @ (r16(wu) if hv else wu).T
            gg = np.minimum(g, 10.0)
            uu = np.clip(u, -10.0, 10.0)
            h = (gg / (1 + np.exp(-gg)) * uu * ws[:, None]).astype(np.float32).astype(np.float64)
            if hv:
                h = r16(h)
            wdd = r16(wd) if hv else wd
            o = h @ wdd.T
            if hv:
                yh[ci[toks]] += o
                ym[ci[toks]] += np.abs(h) @ np.abs(wdd).T
            else:
                yf[ci[toks]] += o
    err_h = float(np.max(np.abs(got[chk] - yh) / (ym + 1e-9)))
    err_f = float(np.max(np.abs(got[chk] - yf) / (ym + 1e-9)))
    assert np.all(np.isfinite(got))
    assert err_h <= 1e-3, (err_h, err_f)
    assert err_f <= 5e-3, (err_h, err_f)
    # tokens the reference check did not look at must at least have moved from Y0 when they have any expert
    assert not np.array_equal(outs[0], Y0)


def test_moe_prefill_edge_cases(orc):
    """Shared expert only (no routed experts); routed only with tokens that have no expert at all (slot_of = -1 keeps
    their rows of Y untouched); zero tokens."""
    from macseek_b200 import quant as q
    from macseek_b200.core import Enc
    D, I, n = 512, 256, 37
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    mats = [synth.random_weights(t, r, c, 800 + i) for i, (t, r, c) in enumerate(
        [(ol.Q8_0, I, D), (ol.Q8_0, I, D), (ol.Q8_0, D, I), (ol.IQ1_S, I, D), (ol.IQ1_S, I, D), (ol.IQ2_XXS, D, I)])]
    X = synth.randn(n * D, 3).reshape(n, D)
    Y0 = synth.randn(n * D, 4).reshape(n, D)

    def ref_expert(g, u, d, tg, td, toks, ws):
        wg = r16(orc.dequant(tg, g, I * D).reshape(I, D).astype(np.float64))
        wu = r16(orc.dequant(tg, u, I * D).reshape(I, D).astype(np.float64))
        wd = r16(orc.dequant(td, d, I * D).reshape(D, I).astype(np.float64))
        xin = r16(X[toks].astype(np.float64))
        gg, uu = np.minimum(xin @ wg.T, 10.0), np.clip(xin @ wu.T, -10.0, 10.0)
        h = r16((gg / (1 + np.exp(-gg)) * uu * ws[:, None]).astype(np.float32).astype(np.float64))
        return h @ wd.T, np.abs(h) @ np.abs(wd).T

    def slot(i0):
        s = q.ExpertSlot()
        s.gate, s.up, s.down = dev(mats[i0]), dev(mats[i0 + 1]), dev(mats[i0 + 2])
        return s
    e = Enc()
    # (1) shared expert only
    a = q.MoePrefillArgs(D, I)
    a.t_gate_up, a.t_down, a.t_shared = ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0
    a.n_tokens, a.k_per_token, a.has_shared = n, 2, True
    a.shared = slot(0)
    a.offs = [0]
    a.slot_of = dev(-np.ones(n * 2, np.int32))
    a.tok, a.wt = dev(np.zeros(1, np.int32)), dev(np.zeros(1, np.float32))
    a.X, a.Y = dev(X), dev(Y0)
    a.scratch = torch.zeros(q.moe_prefill_scratch_bytes(0, n, 0, D, I), dtype=torch.uint8, device="cuda")
    q.encode_moe_prefill(e, a)
    e.wait()
    o, om = ref_expert(mats[0], mats[1], mats[2], ol.Q8_0, ol.Q8_0, np.arange(n), np.ones(n))
    got = a.Y.cpu().numpy().astype(np.float64)
    assert np.max(np.abs(got - (Y0 + o)) / (np.abs(Y0) + om + 1e-9)) <= 1e-3
    # (2) one routed expert for the even tokens only, no shared expert
    toks = np.arange(0, n, 2).astype(np.int32)
    ws = np.full(len(toks), 0.25, np.float32)
    so = -np.ones(n * 2, np.int32)
    so[toks * 2 + 1] = np.arange(len(toks))
    b = q.MoePrefillArgs(D, I)
    b.t_gate_up, b.t_down, b.t_shared = ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0
    b.n_tokens, b.k_per_token, b.has_shared = n, 2, False
    b.slots = [slot(3)]
    b.offs = [0, len(toks)]
    b.tok, b.wt, b.slot_of = dev(toks), dev(ws), dev(so)
    b.X, b.Y = dev(X), dev(Y0)
    b.scratch = torch.zeros(q.moe_prefill_scratch_bytes(len(toks), n, 1, D, I), dtype=torch.uint8, device="cuda")
    q.encode_moe_prefill(e, b)
    e.wait()
    got = b.Y.cpu().numpy()
    odd = np.arange(1, n, 2)
    assert np.array_equal(got[odd].view(np.uint32), Y0[odd].view(np.uint32))          # untouched rows
    o, om = ref_expert(mats[3], mats[4], mats[5], ol.IQ1_S, ol.IQ2_XXS, toks, ws.astype(np.float64))
    assert np.max(np.abs(got[toks].astype(np.float64) - (Y0[toks] + o)) / (np.abs(Y0[toks]) + om + 1e-9)) <= 1e-3
    # (3) zero tokens: nothing happens
    b.n_tokens = 0
    q.encode_moe_prefill(e, b)
    e.wait()


def test_moe_prefill_benchmark_layer_full_size(orc, capsys):
    """The benchmark's prefill configuration at its stated size: 4096 tokens, top-8 of 384 experts (IQ1_S gate/up,
    IQ2_XXS down) + Q8_0 shared expert, dim 4096 / inter 2048, router logits N(0,1) + log-Zipf(1.1) bias over a seeded
    expert permutation (a few experts take thousands of tokens -- the pre-dequantised TMA-fed path -- while most hit
    experts take a handful -- the in-kernel dequantisation path).  Checked as the reference checks its own large case
    (tests/test_quant_moe_prefill.mm:165-177,223): the tokens of experts with at most two entries, tile-boundary tokens
    and a random sample, against the half-emulating (<= 1e-3) and the F32 (<= 5e-3) references; two runs bit-identical."""
    from macseek_b200 import moe_layer as ml, quant as q
    from macseek_b200.core import Enc
    n, D, I, E, K = 4096, 4096, 2048, 384, 8
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    lw = ml.MoeLayerWeights(D, I, E, q.QType.IQ1_S, q.QType.IQ2_XXS, q.QType.Q8_0).randomize(gen)
    perm = torch.randperm(E, device="cuda", generator=gen)
    bias = torch.empty(E, device="cuda")
    bias[perm] = -1.1 * torch.log(torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
    logits = torch.randn(n, E, device="cuda", generator=gen) + bias
    ids = torch.topk(logits, K, dim=1).indices
    w = torch.softmax(torch.gather(logits, 1, ids), dim=1).float()
    flat_e = ids.reshape(-1)
    order = torch.argsort(flat_e, stable=True)              # entries sorted by (expert, token * K + k)
    tok = (order // K).int().contiguous()
    wt = w.reshape(-1)[order].contiguous()
    slot_of = torch.empty(n * K, dtype=torch.int32, device="cuda")
    slot_of[order] = torch.arange(n * K, dtype=torch.int32, device="cuda")
    counts = torch.bincount(flat_e, minlength=E).cpu().numpy()
    used = [e for e in range(E) if counts[e] > 0]
    offs = [0]
    for e in used:
        offs.append(offs[-1] + int(counts[e]))
    cs = np.sort(counts[counts > 0])
    with capsys.disabled():
        print("\n  cfg4 routing: %d experts hit, tokens/expert min %d median %d max %d, %d experts with >= 256 entries"
              % (len(used), cs[0], cs[len(cs) // 2], cs[-1], int((cs >= 256).sum())))
    assert cs[-1] >= 256 and cs[0] < 64            # both weight paths are exercised
    a = q.MoePrefillArgs(D, I)
    a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
    a.n_tokens, a.k_per_token, a.has_shared = n, K, True
    for e in used:
        s = q.ExpertSlot()
        s.gate, s.up, s.down = lw.expert_views(e)
        a.slots.append(s)
    a.shared = lw.shared
    a.offs = offs
    a.tok, a.wt, a.slot_of = tok, wt, slot_of
    a.X = torch.randn(n, D, device="cuda", generator=gen)
    Y0 = torch.randn(n, D, device="cuda", generator=gen)
    a.scratch = torch.zeros(q.moe_prefill_scratch_bytes(offs[-1], n, len(used), D, I), dtype=torch.uint8, device="cuda")
    e_ = Enc()
    outs = []
    for _ in range(2):
        a.Y = Y0.clone()
        q.encode_moe_prefill(e_, a)
        e_.wait()
        outs.append(a.Y.cpu().numpy())
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32)), "repeat differs"
    got = outs[0].astype(np.float64)
    assert np.all(np.isfinite(got))
    # tokens to check
    tok_h, ids_h, w_h = tok.cpu().numpy(), ids.cpu().numpy(), w.cpu().numpy().astype(np.float64)
    chk = set()
    rare = [e for e in used if counts[e] <= 2][:6]
    pos = {e: j for j, e in enumerate(used)}
    for e in rare:
        chk.update(int(t) for t in tok_h[offs[pos[e]]:offs[pos[e] + 1]])
    chk.update((0, 127, 128, n - 1))
    chk.update(int(t) for t in np.random.default_rng(1).integers(0, n, 6))
    chk = sorted(chk)
    X = a.X[chk].cpu().numpy().astype(np.float64)
    yh = Y0[chk].cpu().numpy().astype(np.float64)
    yf = yh.copy()
    ym = np.abs(yh)
    need = sorted({int(e) for t in chk for e in ids_h[t]})
    raw = lambda t: t.cpu().numpy()

    def add_expert(g, u, d, tg, td, rows, ws):
        wg = orc.dequant(tg, raw(g), I * D).reshape(I, D).astype(np.float64)
        wu = orc.dequant(tg, raw(u), I * D).reshape(I, D).astype(np.float64)
        wd = orc.dequant(td, raw(d), I * D).reshape(D, I).astype(np.float64)
        for hv in (0, 1):
            xin = r16(X[rows]) if hv else X[rows]
            g_ = xin @ (r16(wg) if hv else wg).T
            u_ = xin @ (r16(wu) if hv else wu).T
            gg, uu = np.minimum(g_, 10.0), np.clip(u_, -10.0, 10.0)
            h = (gg / (1 + np.exp(-gg)) * uu * ws[:, None]).astype(np.float32).astype(np.float64)
            wdd = r16(wd) if hv else wd
            if hv:
                h = r16(h)
                yh[rows] += h @ wdd.T
                ym[rows] += np.abs(h) @ np.abs(wdd).T
            else:
                yf[rows] += h @ wdd.T
    # the kernel adds the shared expert first, then the routed slots in k order; the reference sums in float64, where the
    # order does not matter at these tolerances
    add_expert(lw.shared.gate, lw.shared.up, lw.shared.down, ol.Q8_0, ol.Q8_0, np.arange(len(chk)), np.ones(len(chk)))
    for e in need:
        rows = np.array([i for i, t in enumerate(chk) if e in ids_h[t]])
        ws = np.array([w_h[chk[i]][list(ids_h[chk[i]]).index(e)] for i in rows])
        g, u, d = lw.expert_views(e)
        add_expert(g, u, d, ol.IQ1_S, ol.IQ2_XXS, rows, ws)
    err_h = float(np.max(np.abs(got[chk] - yh) / (ym + 1e-9)))
    err_f = float(np.max(np.abs(got[chk] - yf) / (ym + 1e-9)))
    with capsys.disabled():
        print("  cfg4 parity on %d tokens / %d experts: half-emulating %.2e (<= 1e-3), F32 %.2e (<= 5e-3)"
              % (len(chk), len(need), err_h, err_f))
    assert err_h <= 1e-3 and err_f <= 5e-3, (err_h, err_f)
