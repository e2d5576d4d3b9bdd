"""Pins the CPU oracle (oracle/msb_oracle.c): against the committed vectors produced by the reference project's own
code (tests/golden/golden_ref.npz), against the reference's known-answer spots, and -- where the reference checkout
is present -- against the reference routines themselves on larger seeded inputs."""
import os

import numpy as np
import pytest

import oracle_lib as ol

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_ref.npz"))
ALL_TYPES = (ol.F32, ol.F16, ol.BF16, ol.Q8_0, ol.Q5_K, ol.Q6_K, ol.IQ2_XXS, ol.IQ1_S, ol.IQ4_NL, ol.MXFP4)


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


@pytest.fixture(scope="module")
def ref():
    r = ol.Ref.load(build=os.path.isdir("/root/reference/tests/ref"))
    if r is None:
        pytest.skip("reference routines not built (no reference checkout)")
    return r


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("t", ALL_TYPES)
def test_dequant_golden_bit_exact(orc, t):
    out = orc.dequant(t, G["deq_raw_%d" % t], 512)
    assert np.array_equal(bits(out), bits(G["deq_out_%d" % t]))


@pytest.mark.parametrize("name", ["tiny", "iq1s", "iq2", "q5k", "q80", "iq4"])
def test_matvec_golden(orc, name):
    t, rows, cols, groups = [int(v) for v in G["mv_%s_meta" % name]]
    y, mag = orc.matvec(t, G["mv_%s_W" % name], rows, cols, G["mv_%s_x" % name], groups)
    assert np.array_equal(y, G["mv_%s_y" % name])
    assert np.array_equal(mag, G["mv_%s_mag" % name])


def test_router_and_lists_golden(orc):
    ids = np.zeros((4, 6), np.int32); w = np.zeros((4, 6), np.float32)
    for i in range(4):
        ids[i], w[i] = orc.router(G["router_logits"][i], G["router_bias"], 6, 0, 1.5)
    assert np.array_equal(ids, G["router_ids"])
    assert np.array_equal(bits(w), bits(G["router_w"]))
    assert ids[1, 0] == 17 and ids[1, 1] == 300     # equal keys: lowest expert id first
    got = orc.route_lists(ids, w, 4, 6, 384)
    for nm, arr in zip(("counts", "offsets", "entry", "tok", "lw", "slot_of"), got):
        assert np.array_equal(arr, G["lists_" + nm]), nm


def test_rope_and_sims_golden(orc):
    assert np.array_equal(bits(orc.rope_table(6, False)), bits(G["rope_plain"]))
    assert np.array_equal(bits(orc.rope_table(6, True)), bits(G["rope_yarn"]))
    for m in ("fp8_sim", "fp4_sim_e8m0", "fp4_sim_e4m3"):
        assert np.array_equal(bits(orc.sim(m, G["sim_in"])), bits(G["sim_" + m])), m


def test_rounding_known_answers(orc):
    # the reference's spot values (tests/test_attn_units.mm:39-42)
    r8, r4 = orc.lib.orc_round_e4m3, orc.lib.orc_round_e2m1
    assert r8(448) == 448 and r8(2.0 ** -10) == 0 and r8(1.5 * 2.0 ** -10) == 2.0 ** -9 and r8(17) == 16 and r8(19) == 20
    assert r4(0.25) == 0 and r4(0.75) == 1 and r4(2.5) == 2 and r4(5) == 4 and r4(5.5) == 6


def test_e4m3_codec_roundtrip(orc):
    codes = np.arange(256, dtype=np.uint8)
    vals = orc.e4m3_to_f32(codes)
    finite = np.isfinite(vals)
    assert vals[0x7e] == 448 and vals[0x08] == 2.0 ** -6 and vals[0x01] == 2.0 ** -9
    back = orc.f32_to_e4m3(vals[finite])
    ok = (back == codes[finite]) | (vals[finite] == 0)      # +-0 both decode to 0
    assert ok.all()


def test_indexer_golden(orc):
    for actq in (0, 1):
        q, w = orc.index_q(G["idx_q_raw"], G["idx_w_raw"], G["idx_cs"], actq, 32, 128)
        assert np.array_equal(bits(q), bits(G["idx_q_%d" % actq]))
        assert np.array_equal(bits(w), bits(G["idx_w_%d" % actq]))
        sc = orc.index_scores(q, w, G["idx_keys"])
        assert np.array_equal(bits(sc), bits(G["idx_sc_%d" % actq]))


def test_topk_golden(orc):
    sc = G["topk_in"]
    assert np.array_equal(orc.topk_sorted(sc, 8), G["topk_k8"])
    assert np.array_equal(orc.topk_sorted(sc, 64), G["topk_k64"])
    assert 40 in G["topk_k8"] and 3 not in G["topk_k64"]           # +inf pinned, -inf never selected
    assert np.array_equal(orc.candidate_blocks(sc), G["cand_blocks"])


def test_topk_structural_cases(orc):
    # the reference's structural cases (tests/test_attn_units.mm:65-70): n=0, n<k, n=k, all ties
    assert (orc.topk_sorted(np.zeros(0, np.float32), 4) == -1).all()
    assert list(orc.topk_sorted(np.array([3, 1, 2], np.float32), 4)) == [0, 1, 2, -1]
    assert list(orc.topk_sorted(np.full(10, 1.5, np.float32), 4)) == [0, 1, 2, 3]


def test_sparse_attn_and_window_golden(orc):
    q = G["sa_q"].astype(np.float32); rows = G["sa_rows"].astype(np.float32)
    out = orc.sparse_attn(q, G["sa_cs"], rows, G["sa_sinks"])
    assert np.array_equal(bits(out), bits(G["sa_out"]))
    for actq in (0, 1):
        assert np.array_equal(bits(orc.window_row(G["win_kv"], G["win_nw"], G["idx_cs"], actq)),
                              bits(G["win_out_%d" % actq]))


def _hc_inputs():
    import synth
    D = 5120
    return (synth.hashed(4 * D, 1, 4.0), synth.hashed(D, 2, 2.0), np.abs(synth.hashed(24, 6, 2.0)) + 0.05,
            synth.hashed(24 * 4 * D, 3, 0.05), np.array([0.7, 1.3, 0.9], np.float32), synth.hashed(24, 4, 1.0),
            1 + synth.hashed(D, 5, 0.2))


def test_hc_step_golden(orc):
    h_in, x_sub, mix_prev, fn, scale, base, norm_w = _hc_inputs()
    h_out, mix_out, x_out = orc.hc_step(h_in, x_sub, mix_prev, fn, scale, base, norm_w, 5120)
    assert np.array_equal(bits(h_out), bits(G["hc_h_out"]))
    assert np.array_equal(bits(mix_out), bits(G["hc_mix_out"]))
    assert np.array_equal(bits(x_out), bits(G["hc_x_out"]))
    _, mix0, x0 = orc.hc_step(h_in, None, mix_prev, fn, scale, base, norm_w, 5120)
    assert np.array_equal(bits(mix0), bits(G["hc0_mix_out"])) and np.array_equal(bits(x0), bits(G["hc0_x_out"]))


def test_compressor_golden(orc):
    import synth
    cn, kn = 1 + synth.hashed(512, 7, 0.2), 1 + synth.hashed(128, 8, 0.2)
    wk = synth.hashed_bf16(128 * 512, 9, 0.2)
    ckv_in, cg_in = synth.hashed(6 * 512, 10, 3.0), synth.hashed(6 * 512, 11, 4.0)
    for ratio in (1, 2):
        for actq in (0, 1):
            ck, ik = orc.compress_tokens(ratio, ckv_in, cg_in if ratio > 1 else None, cn, wk, kn, actq)
            assert ck.shape[0] == 6 // ratio
            assert np.array_equal(bits(ck), bits(G["cmp_ckv_r%d_q%d" % (ratio, actq)]))
            assert np.array_equal(bits(ik), bits(G["cmp_ikey_r%d_q%d" % (ratio, actq)]))


# ---------------------------------------------------------------- against the reference code itself (when present)
def test_sampling_golden(orc):
    """top-k (ties -> lower index), log-sum-exp, log-softmax against the reference build's outputs; the top-p sampler's
    structural properties (the reference has no stored vectors for it: tests/test_arch_sample.mm:120-135 checks
    frequencies)."""
    sl = G["smp_logits"]
    v, i = orc.topk_desc(sl, 64)
    assert np.array_equal(i, G["smp_topk_i"]) and np.array_equal(v.view(np.uint32), G["smp_topk_v"].view(np.uint32))
    assert list(i[:3]) == [7, 1207, 2407]
    assert abs(orc.logsumexp(sl, 1.0) - G["smp_lse"][0]) < 1e-12 and abs(orc.logsumexp(sl, 1 / 0.7) - G["smp_lse"][1]) < 1e-12
    assert np.array_equal(orc.log_softmax(sl).view(np.uint32), G["smp_log_softmax"].view(np.uint32))
    lse = orc.logsumexp(sl, 1 / 0.7)
    p = np.exp(v.astype(np.float64) / 0.7 - lse)
    keep = int(np.searchsorted(np.cumsum(p), 0.3) + 1)
    N = 20000
    cnt = np.zeros(64)
    for it in range(N):
        tok = orc.sample_top_p(v, i, 64, lse, 0.7, 0.3, (it + 0.5) / N)
        pos = int(np.where(i == tok)[0][0])
        assert pos < keep
        cnt[pos] += 1
    assert np.all(np.abs(cnt[:keep] / N - p[:keep] / p[:keep].sum()) < 1e-3)
    assert orc.sample_top_p(v, i, 64, lse, 0.0, 0.3, 0.9) == i[0]           # temperature 0: greedy
    # Gumbel noise: deterministic per (index, seed, row), different across rows, mean of Gumbel(0,1) = 0.5772
    a = np.array([orc.gumbel(j, 0x1234567, 0) for j in range(20000)])
    assert a[5] == orc.gumbel(5, 0x1234567, 0) and a[5] != orc.gumbel(5, 0x1234567, 1)
    assert abs(a.mean() - 0.5772) < 0.03 and abs(a.var() - np.pi ** 2 / 6) < 0.1


@pytest.mark.parametrize("t", ALL_TYPES)
def test_dequant_vs_reference_1m(orc, ref, t):
    n = 1 << 20                                   # 1M elements per type, as tests/test_quant_ref.mm:97-99
    raw = ref.random_blocks(t, n, 4242 + t)
    assert np.array_equal(bits(orc.dequant(t, raw, n)), bits(ref.dequant(t, raw, n)))
    rng = np.random.default_rng(t)
    raw2 = rng.integers(0, 256, ol.row_bytes(t, 1 << 16), dtype=np.uint8)   # arbitrary bytes, incl. odd scales
    a, b = orc.dequant(t, raw2, 1 << 16), ref.dequant(t, raw2, 1 << 16)
    assert np.array_equal(bits(a), bits(b))


def test_matvec_vs_reference(orc, ref):
    rng = np.random.default_rng(5)
    for t, rows, cols, groups in ((ol.Q6_K, 64, 1280, 1), (ol.Q5_K, 48, 512, 8), (ol.IQ1_S, 40, 2304, 1),
                                  (ol.IQ2_XXS, 32, 4096, 1), (ol.Q8_0, 33, 2304, 1), (ol.BF16, 16, 512, 1),
                                  (ol.IQ4_NL, 24, 1024, 1)):
        W = ref.random_blocks(t, rows * cols, 7 + rows + cols)
        x = rng.standard_normal(cols * groups).astype(np.float32)
        y, mag = orc.matvec(t, W, rows, cols, x, groups, threads=3)
        ry, rmag = ref.matvec(t, W, rows, cols, x, groups)
        assert np.array_equal(y, ry) and np.array_equal(mag, rmag)


def test_router_vs_reference(orc, ref):
    rng = np.random.default_rng(9)
    bias = (rng.standard_normal(384) * 0.2).astype(np.float32)
    for i in range(50):
        logits = (rng.standard_normal(384) * (1 + i % 7)).astype(np.float32)
        a, b = orc.router(logits, bias, 6, 0, 1.5), ref.router(logits, bias)
        assert np.array_equal(a[0], b[0]) and np.array_equal(bits(a[1]), bits(b[1]))


def test_attention_vs_reference(orc, ref):
    rng = np.random.default_rng(11)
    tab = ref.rope_table(1000, True)
    assert np.array_equal(bits(orc.rope_table(1000, True)), bits(tab))
    keys = ref.sim("fp4_sim_e8m0", rng.standard_normal((3000, 128)).astype(np.float32)).reshape(3000, 128)
    q, w = ref.index_q(rng.standard_normal((32, 128)), rng.standard_normal(32), tab[999], 1)
    sc = ref.index_scores(q, w, keys)
    assert np.array_equal(bits(orc.index_scores(q, w, keys)), bits(sc))
    for k in (512, 2048):
        assert np.array_equal(orc.topk_sorted(sc, k), ref.topk_sorted(sc, k))
    sc2 = np.round(sc * 4) / 4                     # many ties
    assert np.array_equal(orc.topk_sorted(sc2, 512), ref.topk_sorted(sc2, 512))
    sc3 = rng.standard_normal(30000).astype(np.float32)
    assert np.array_equal(orc.candidate_blocks(sc3), ref.candidate_blocks(sc3))
