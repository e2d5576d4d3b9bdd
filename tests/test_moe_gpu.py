"""GPU parity of the fused MoE decode and the router against the oracle (designs of the reference's
tests/test_quant_moe.mm and tests/test_arch_router.mm)."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


@pytest.fixture()
def enc():
    from macseek_b200.core import Enc
    return Enc()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


class MoeCase:
    """Experts in one arena at 4-byte (not 16-byte) aligned offsets, shuffled order (tests/test_quant_moe.mm:46-61)."""

    def __init__(self, D, I, gu, down, sh, n_routed, shared, xscale=1.0, seed=0, n_experts=None):
        from macseek_b200 import quant as q
        self.q = q
        self.D, self.I, self.gu, self.down, self.sh, self.n_routed, self.shared = D, I, gu, down, sh, n_routed, shared
        n_mats = n_experts if n_experts is not None else n_routed
        self.n_mats = n_mats
        n_exp = n_mats + (1 if shared else 0)
        self.G, self.U, self.Dn = [], [], []
        for e in range(n_exp):
            is_sh = shared and e == n_mats
            tgu, td = (sh, sh) if is_sh else (gu, down)
            self.G.append(synth.random_weights(tgu, I, D, 100 + e * 3 + seed))
            self.U.append(synth.random_weights(tgu, I, D, 101 + e * 3 + seed))
            self.Dn.append(synth.random_weights(td, D, I, 102 + e * 3 + seed))
        total = sum(g.size + u.size + d.size + 60 for g, u, d in zip(self.G, self.U, self.Dn))
        self.arena = torch.zeros(total + 64, dtype=torch.uint8, device="cuda")
        off = 4
        self.slots = [None] * n_exp
        for e in range(n_exp - 1, -1, -1):
            s = q.ExpertSlot()
            for name, arr in (("down", self.Dn[e]), ("gate", self.G[e]), ("up", self.U[e])):
                self.arena[off:off + arr.size] = dev(arr)
                setattr(s, name, self.arena[off:off + arr.size])
                off += arr.size + 12
            self.slots[e] = s
        self.x = synth.randn(D, 77 + seed, xscale)
        self.y0 = synth.randn(D, 78 + seed)
        self.w = np.array([0.31, 0.22, 0.17, 0.12, 0.1, 0.08, 0.05, 0.03][:max(n_routed, 1)], dtype=np.float32)

    def args(self, ids=None):
        q = self.q
        a = q.MoeDecodeArgs(self.D, self.I)
        a.t_gate_up, a.t_down, a.t_shared = self.gu, self.down, self.sh
        a.n_routed, a.has_shared = self.n_routed, self.shared
        sel = ids if ids is not None else range(self.n_routed)
        for i, e in enumerate(sel):
            a.slot[i] = self.slots[e]
        if self.shared:
            a.shared = self.slots[self.n_mats]
        a.weights = dev(self.w)
        a.x = dev(self.x)
        a.y = dev(self.y0)
        a.scratch = torch.zeros(q.moe_decode_scratch_bytes(self.I, self.n_routed) // 4, device="cuda")
        return a

    def reference(self, orc, ids=None, active=None):
        sel = list(ids if ids is not None else range(self.n_routed))
        keep = [i for i in range(len(sel)) if active is None or active[i]]
        mats = [sel[i] for i in keep] + ([self.n_mats] if self.shared else [])
        w = self.w[keep] if keep else np.zeros(1, np.float32)
        h, y, ymag, hmag = orc.moe_decode(self.D, self.I, self.gu, self.down, self.sh, [self.G[m] for m in mats],
                                          [self.U[m] for m in mats], [self.Dn[m] for m in mats], w, self.x, self.y0,
                                          has_shared=self.shared)
        return keep, h, y, ymag, hmag


def check(orc, case, a, keep, h, y, ymag, hmag):
    hg = a.scratch.cpu().numpy().reshape(case.n_routed + 1, case.I)
    rows = keep + ([case.n_routed] if case.shared else [])
    h_err = 0.0
    for j, r in enumerate(rows):
        h_err = max(h_err, float(np.max(np.abs(hg[r] - h[j]) / hmag[j])))
    y_err = orc.max_norm_err(a.y.cpu().numpy(), y, ymag)
    return h_err, y_err


# the reference's 7 cases (tests/test_quant_moe.mm:22-30): dim 5120, inter 2304, 6 routed
REF_CASES = [
    (ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 6, True, 1.0), (ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 6, True, 1.0),
    (ol.IQ1_S, ol.IQ2_XXS, ol.Q6_K, 6, True, 1.0), (ol.IQ2_XXS, ol.IQ2_XXS, ol.Q6_K, 6, True, 1.0),
    (ol.IQ2_XXS, ol.IQ2_XXS, ol.Q8_0, 3, False, 1.0), (ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 0, True, 1.0),
    (ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 6, True, 40.0),
]


@pytest.mark.parametrize("c", REF_CASES, ids=lambda c: "%s-%s-%s-r%d%s-x%g" % (ol.TYPE_NAMES[c[0]], ol.TYPE_NAMES[c[1]], ol.TYPE_NAMES[c[2]], c[3], "s" if c[4] else "", c[5]))
def test_moe_decode_reference_cases(orc, enc, c):
    case = MoeCase(5120, 2304, *c)
    a = case.args()
    case.q.encode_moe_decode(enc, a)
    enc.wait()
    h_err, y_err = check(orc, case, a, *case.reference(orc))
    assert h_err <= 2e-5 and y_err <= 5e-5, (h_err, y_err)     # the reference's own bounds (test_quant_moe.mm:93)


def test_moe_decode_cfg3_layer(orc, enc):
    # benchmark decode layer: hidden 4096, inter 2048, 8 routed IQ1_S gate/up + IQ2_XXS down, shared Q8_0
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True)
    a = case.args()
    case.q.encode_moe_decode(enc, a)
    enc.wait()
    first = a.y.cpu().numpy().copy()
    h_err, y_err = check(orc, case, a, *case.reference(orc))
    assert h_err <= 2e-5 and y_err <= 5e-5, (h_err, y_err)
    for _ in range(3):       # run-to-run bit identity with dynamic tile scheduling
        a2 = case.args()
        case.q.encode_moe_decode(enc, a2)
        enc.wait()
        assert np.array_equal(bits(a2.y.cpu().numpy()), bits(first))


def test_moe_decode_table_and_parts(orc, enc):
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True)
    q = case.q
    a = case.args()
    q.encode_moe_decode(enc, a)
    enc.wait()
    full = a.y.cpu().numpy().copy()
    table = torch.tensor([[s.gate.data_ptr(), s.up.data_ptr(), s.down.data_ptr()] for s in case.slots[:8]],
                         dtype=torch.int64, device="cuda")
    b = case.args()
    q.encode_moe_decode_table(enc, b, table)
    enc.wait()
    assert np.array_equal(bits(b.y.cpu().numpy()), bits(full))
    # Shared then Routed == All up to the summation order of y (quant.hpp:79-81)
    c = case.args()
    q.encode_moe_decode_table_part(enc, c, table, q.MoePart.Shared)
    q.encode_moe_decode_table_part(enc, c, table, q.MoePart.Routed)
    enc.wait()
    keep, h, y, ymag, hmag = case.reference(orc)
    assert orc.max_norm_err(c.y.cpu().numpy(), y, ymag) <= 5e-5
    # SharedGu then AfterSharedGu == All, bit-identical
    d = case.args()
    q.encode_moe_decode_table_part(enc, d, table, q.MoePart.SharedGu)
    q.encode_moe_decode_table_part(enc, d, table, q.MoePart.AfterSharedGu)
    enc.wait()
    assert np.array_equal(bits(d.y.cpu().numpy()), bits(full))


@pytest.mark.parametrize("world", (1, 2, 4, 8))
def test_moe_decode_ids_expert_parallel_partition(orc, enc, world):
    # 16 resident experts, router picks 8; each "rank" computes the experts in its contiguous range, the shared
    # expert is added once; the sum of the partial y equals the single-GPU result
    n_exp = 16
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True, n_experts=n_exp)
    q = case.q
    ids = np.array([13, 2, 7, 8, 0, 15, 5, 10], dtype=np.int32)
    table = torch.tensor([[s.gate.data_ptr(), s.up.data_ptr(), s.down.data_ptr()] for s in case.slots[:n_exp]],
                         dtype=torch.int64, device="cuda")
    ids_d = dev(ids)
    keep, h, y, ymag, hmag = case.reference(orc, ids=ids)
    total = np.zeros(case.D, dtype=np.float64)
    per = n_exp // world
    for r in range(world):
        a = case.args(ids=ids)
        a.y = torch.zeros(case.D, device="cuda")
        a.has_shared = r == 0
        q.encode_moe_decode_ids(enc, a, table, ids_d, r * per, (r + 1) * per)
        enc.wait()
        total += a.y.cpu().numpy().astype(np.float64)
    got = (total + case.y0).astype(np.float32)
    assert orc.max_norm_err(got, y, ymag) <= 5e-5


def test_moe_argument_errors(enc):
    from macseek_b200._lib import MsbError
    case = MoeCase(512, 256, ol.IQ1_S, ol.IQ1_S, ol.Q6_K, 2, True)
    a = case.args()
    a.t_shared = ol.IQ1_S
    with pytest.raises(MsbError):
        case.q.encode_moe_decode(enc, a)
    a = case.args()
    a.scratch = torch.zeros(16, device="cuda")
    with pytest.raises(MsbError):
        case.q.encode_moe_decode(enc, a)
    a = case.args()
    a.n_routed = 17
    with pytest.raises(MsbError):
        case.q.encode_moe_decode(enc, a)


# ---------------------------------------------------------------- router
@pytest.mark.parametrize("cfg", [(384, 5120, 6, 0, 1.5), (384, 4096, 8, 1, 1.0)], ids=["ref-top6-softplus", "cfg3-top8-sigmoid"])
def test_router_fused_and_topk(orc, enc, cfg):
    from macseek_b200 import arch
    E, dim, k, fn, scale = cfg
    rng = np.random.default_rng(5)
    W = (rng.standard_normal((E, dim)) * 0.02).astype(np.float32)
    bias = (rng.standard_normal(E) * 0.05).astype(np.float32)
    s = arch.Scratch.create(E)
    Wd, bd = dev(W), dev(bias)
    ids = torch.zeros(k, dtype=torch.int32, device="cuda")
    w = torch.zeros(k, dtype=torch.float32, device="cuda")
    bad = 0
    for trial in range(20):
        x = synth.randn(dim, 1000 + trial, 1.0 + trial)
        arch.encode_router_fused(enc, dev(x), Wd, bd, ids, w, s, k, fn, scale)
        enc.wait()
        logits = (W.astype(np.float64) @ x.astype(np.float64))
        got_logits = s.router_logits.cpu().numpy()
        assert np.max(np.abs(got_logits - logits)) <= 1e-4 * (np.abs(W) @ np.abs(x)).max()
        rid, rw = orc.router(got_logits, bias, k, fn, scale)     # selection checked on the device's own logits
        gi, gw = ids.cpu().numpy(), w.cpu().numpy()
        if not np.array_equal(gi, rid):
            # a different pick is accepted only for a near tie (key gap < 1e-5), tests/test_arch_router.mm:21-44
            sc = 1 / (1 + np.exp(-got_logits.astype(np.float64))) if fn else np.sqrt(np.log1p(np.exp(got_logits.astype(np.float64))))
            key = sc + bias
            for a_, b_ in zip(gi, rid):
                assert abs(key[a_] - key[b_]) < 1e-5
            bad += 1
        else:
            assert np.max(np.abs(gw - rw) / rw) <= 1e-5
    assert bad <= 2
    # batch top-k from logits, incl. an exact tie (lowest id first)
    n = 37
    L = (rng.standard_normal((n, E)) * 2).astype(np.float32)
    L[3, 10] = L[3, 200] = 9.0
    L[3, :10] = -5.0          # nothing else of row 3 comes close to the tied pair's key
    b0 = bias.copy(); b0[10] = b0[200] = 0.5
    ids_n = torch.zeros((n, k), dtype=torch.int32, device="cuda")
    w_n = torch.zeros((n, k), dtype=torch.float32, device="cuda")
    arch.encode_router_topk(enc, dev(L), dev(b0), ids_n, w_n, n, k, fn, scale)
    enc.wait()
    for t in range(n):
        rid, rw = orc.router(L[t], b0, k, fn, scale)
        assert np.array_equal(ids_n[t].cpu().numpy(), rid), t
        assert np.max(np.abs(w_n[t].cpu().numpy() - rw) / rw) <= 1e-5
    row3 = list(ids_n[3].cpu().numpy())
    assert 10 in row3 and 200 in row3 and row3.index(10) + 1 == row3.index(200)     # equal keys: lowest id first


def test_route_lists_bit_exact(orc, enc):
    from macseek_b200 import arch
    rng = np.random.default_rng(2)
    for n, k, E in ((1, 6, 384), (5, 6, 384), (600, 6, 384), (4096, 8, 384)):
        ids = np.stack([rng.choice(E, k, replace=False) for _ in range(n)]).astype(np.int32)
        if n > 100:
            ids[:, 0] = 7           # one popular expert
        w = rng.random((n, k)).astype(np.float32)
        L = arch.RouteLists.create(n, k, E)
        for rep in range(2):
            arch.encode_route_lists(enc, dev(ids), dev(w), n, L)
            enc.wait()
            ref = orc.route_lists(ids, w, n, k, E)
            got = (L.counts, L.offsets, L.entry, L.tok, L.w, L.slot_of)
            for g, r, nm in zip(got, ref, ("counts", "offsets", "entry", "tok", "w", "slot_of")):
                gn = g.cpu().numpy()
                assert np.array_equal(gn.view(np.uint32), r.view(np.uint32)), (n, nm)


def test_router_fused_rmsnorm(orc, enc):
    """RMSNorm folded into the router launch: logits of the normalised vector, and the normalised vector itself."""
    from macseek_b200 import arch
    E, dim, k = 384, 4096, 8
    rng = np.random.default_rng(11)
    W = (rng.standard_normal((E, dim)) * 0.02).astype(np.float32)
    gain = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    s = arch.Scratch.create(E)
    Wd, gd = dev(W), dev(gain)
    ids = torch.zeros(k, dtype=torch.int32, device="cuda")
    w = torch.zeros(k, dtype=torch.float32, device="cuda")
    xo = torch.zeros(dim, dtype=torch.float32, device="cuda")
    for trial in range(5):
        h = synth.randn(dim, 2000 + trial, 0.5 + trial)
        arch.encode_router_fused_rmsnorm(enc, dev(h), gd, 1e-6, xo, Wd, None, ids, w, s, k, 1, 1.0)
        enc.wait()
        xn = orc.rmsnorm(h, gain, 1e-6)
        got_x = xo.cpu().numpy()
        assert np.max(np.abs(got_x - xn)) <= 1e-5 * np.max(np.abs(xn))
        logits = W.astype(np.float64) @ xn.astype(np.float64)
        got_logits = s.router_logits.cpu().numpy()
        assert np.max(np.abs(got_logits - logits)) <= 1e-4 * (np.abs(W) @ np.abs(xn)).max()
        rid, rw = orc.router(got_logits, np.zeros(E, np.float32), k, 1, 1.0)
        assert np.array_equal(ids.cpu().numpy(), rid)
        assert np.max(np.abs(w.cpu().numpy() - rw) / rw) <= 1e-5


@pytest.mark.parametrize("types", ((ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, True), (ol.IQ2_XXS, ol.IQ2_XXS, ol.Q6_K, True),
                                   (ol.IQ1_S, ol.IQ1_S, ol.Q8_0, False)),
                         ids=lambda t: "%s-%s-%s%s" % (ol.TYPE_NAMES[t[0]], ol.TYPE_NAMES[t[1]], ol.TYPE_NAMES[t[2]],
                                                      "-s" if t[3] else ""))
def test_moe_decode_ids_normed_matches_two_step(orc, enc, types):
    """The MoE launch that builds RMSNorm(h) * gain itself (and starts before the router ahead of it has finished) gives
    the bits of: fused-norm router -> x, then the plain launch on x.  Repeated back to back, as in a decode step."""
    from macseek_b200 import arch
    gu, dn, sh, shared = types
    n_exp, k, E = 16, 8, 16
    case = MoeCase(4096, 2048, gu, dn, sh, k, shared, n_experts=n_exp, seed=5)
    q = case.q
    table = torch.tensor([[s.gate.data_ptr(), s.up.data_ptr(), s.down.data_ptr()] for s in case.slots[:n_exp]],
                         dtype=torch.int64, device="cuda")
    rng = np.random.default_rng(3)
    W = dev((rng.standard_normal((E, case.D)) * 0.02).astype(np.float32))
    gain = dev((1.0 + 0.1 * rng.standard_normal(case.D)).astype(np.float32))
    s = arch.Scratch.create(E)
    ids = torch.zeros(k, dtype=torch.int32, device="cuda")
    w = torch.zeros(k, dtype=torch.float32, device="cuda")
    xo = torch.zeros(case.D, dtype=torch.float32, device="cuda")
    for trial in range(4):
        h = dev(synth.randn(case.D, 300 + trial, 1.0 + trial))
        outs = []
        for normed in (False, True):
            a = case.args()
            a.weights, a.x = w, xo
            a.y = dev(case.y0)
            arch.encode_router_fused_rmsnorm(enc, h, gain, 1e-6, xo, W, None, ids, w, s, k, 1, 1.0)
            if normed:
                a.x = None
                q.encode_moe_decode_ids_normed(enc, a, table, ids, 0, n_exp, h, gain, 1e-6)
            else:
                q.encode_moe_decode_ids(enc, a, table, ids, 0, n_exp)
            enc.wait()
            outs.append((a.y.cpu().numpy(), a.scratch.cpu().numpy()))
        assert np.array_equal(bits(outs[0][0]), bits(outs[1][0])), trial
        assert np.array_equal(bits(outs[0][1]), bits(outs[1][1])), trial
    # expert-parallel style: no shared expert, only half of the experts resident
    a = case.args()
    a.weights, a.x, a.has_shared = w, None, False
    a.y = torch.zeros(case.D, device="cuda")
    b2 = case.args()
    b2.weights, b2.x, b2.has_shared = w, xo, False
    b2.y = torch.zeros(case.D, device="cuda")
    arch.encode_router_fused_rmsnorm(enc, h, gain, 1e-6, xo, W, None, ids, w, s, k, 1, 1.0)
    q.encode_moe_decode_ids_normed(enc, a, table, ids, 8, 16, h, gain, 1e-6)
    arch.encode_router_fused_rmsnorm(enc, h, gain, 1e-6, xo, W, None, ids, w, s, k, 1, 1.0)
    q.encode_moe_decode_ids(enc, b2, table, ids, 8, 16)
    enc.wait()
    assert np.array_equal(bits(a.y.cpu().numpy()), bits(b2.y.cpu().numpy()))
    from macseek_b200 import _lib
    assert _lib.device_status() == 0
