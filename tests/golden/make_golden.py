#!/usr/bin/env python3
"""Generate tests/golden/golden_ref.npz by running the reference project's OWN scalar CPU routines
(oracle/_ref/libmsref.so, compiled from the reference checkout by oracle/Makefile) on small seeded inputs.

Run where the reference checkout is available:   python tests/golden/make_golden.py
The vectors are committed so that the oracle can be pinned where the reference checkout is absent."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402


def main():
    ref = ol.Ref.load()
    if ref is None:
        raise SystemExit("reference checkout not found: cannot generate golden vectors")
    rng = np.random.default_rng(20260101)
    g = {}
    # --- dequant: blocks from the reference's own generator (tests/ref/dequant.cpp:133) + pure random bytes
    for t in (ol.F32, ol.F16, ol.BF16, ol.Q8_0, ol.Q5_K, ol.Q6_K, ol.IQ2_XXS, ol.IQ1_S, ol.IQ4_NL, ol.MXFP4):
        n = 512
        raw = ref.random_blocks(t, n, 1000 + t)
        g["deq_raw_%d" % t] = raw
        g["deq_out_%d" % t] = ref.dequant(t, raw, n)
    # --- matvec (tests/test_quant_matvec.mm seeds: random_blocks(t, rows*cols, 7+rows+cols))
    for name, t, rows, cols, groups in (("tiny", ol.Q6_K, 3, 256, 1), ("iq1s", ol.IQ1_S, 8, 512, 1),
                                        ("iq2", ol.IQ2_XXS, 6, 512, 2), ("q5k", ol.Q5_K, 4, 256, 1),
                                        ("q80", ol.Q8_0, 5, 96, 1), ("iq4", ol.IQ4_NL, 4, 64, 1)):
        W = ref.random_blocks(t, rows * cols, 7 + rows + cols)
        x = rng.standard_normal(cols * groups).astype(np.float32)
        y, mag = ref.matvec(t, W, rows, cols, x, groups)
        g["mv_%s_W" % name] = W
        g["mv_%s_x" % name] = x
        g["mv_%s_y" % name] = y
        g["mv_%s_mag" % name] = mag
        g["mv_%s_meta" % name] = np.array([t, rows, cols, groups], dtype=np.int32)
    # --- router (384 experts, top-6) with a forced tie and large logits
    logits = (rng.standard_normal((4, 384)) * 2).astype(np.float32)
    logits[1, 17] = logits[1, 300] = 12.0
    logits[2, 5] = 30.0
    bias = (rng.standard_normal(384) * 0.1).astype(np.float32)
    bias[17] = bias[300] = 0.0
    ids = np.zeros((4, 6), np.int32); w = np.zeros((4, 6), np.float32)
    for i in range(4):
        ids[i], w[i] = ref.router(logits[i], bias)
    g["router_logits"], g["router_bias"], g["router_ids"], g["router_w"] = logits, bias, ids, w
    names = ("counts", "offsets", "entry", "tok", "lw", "slot_of")
    for nm, arr in zip(names, ref.route_lists(ids, w, 4)):
        g["lists_" + nm] = arr
    # --- rope tables, quant sims
    g["rope_plain"] = ref.rope_table(6, False)
    g["rope_yarn"] = ref.rope_table(6, True)
    xs = (rng.standard_normal(128) * np.exp2(rng.integers(-12, 6, 128))).astype(np.float32)
    xs[32:64] = 0
    g["sim_in"] = xs
    for m in ("fp8_sim", "fp4_sim_e8m0", "fp4_sim_e4m3"):
        g["sim_" + m] = ref.sim(m, xs)
    # --- indexer (32 heads x 128), top-k, candidate blocks
    cs = ref.rope_table(300, True)[257]
    q_raw = rng.standard_normal((32, 128)).astype(np.float32)
    w_raw = rng.standard_normal(32).astype(np.float32)
    keys = ref.sim("fp4_sim_e8m0", rng.standard_normal((48, 128)).astype(np.float32)).reshape(48, 128)
    for actq in (0, 1):
        q, wq = ref.index_q(q_raw, w_raw, cs, actq)
        g["idx_q_%d" % actq], g["idx_w_%d" % actq] = q, wq
        g["idx_sc_%d" % actq] = ref.index_scores(q, wq, keys)
    g["idx_q_raw"], g["idx_w_raw"], g["idx_cs"], g["idx_keys"] = q_raw, w_raw, cs, keys
    sc = rng.standard_normal(60).astype(np.float32)
    sc[10] = sc[20] = sc[30] = 1.25; sc[3] = -np.inf; sc[40] = np.inf
    g["topk_in"] = sc
    g["topk_k8"] = ref.topk_sorted(sc, 8)
    g["topk_k64"] = ref.topk_sorted(sc, 64)
    g["cand_blocks"] = ref.candidate_blocks(sc)
    # --- sparse attention (64 heads x 512, K == V rows), window row
    q = rng.standard_normal((64, 512)).astype(np.float32)
    rows = rng.standard_normal((7, 512)).astype(np.float32)
    sinks = rng.standard_normal(64).astype(np.float32)
    g["sa_q"], g["sa_rows"], g["sa_sinks"], g["sa_cs"] = q.astype(np.float16), rows.astype(np.float16), sinks, cs
    g["sa_out"] = ref.sparse_attn(q.astype(np.float16).astype(np.float32), cs,
                                  rows.astype(np.float16).astype(np.float32), sinks)
    kv = rng.standard_normal(512).astype(np.float32); nw = (1 + 0.1 * rng.standard_normal(512)).astype(np.float32)
    g["win_kv"], g["win_nw"] = kv, nw
    for actq in (0, 1):
        g["win_out_%d" % actq] = ref.window_row(kv, nw, cs, actq)
    # --- hyper-connection step (4 x 5120 streams): inputs are integer-hashed patterns (synth.hashed), only outputs stored
    import synth
    D = 5120
    h_in, x_sub = synth.hashed(4 * D, 1, 4.0), synth.hashed(D, 2, 2.0)
    fn, scale, base = synth.hashed(24 * 4 * D, 3, 0.05), np.array([0.7, 1.3, 0.9], np.float32), synth.hashed(24, 4, 1.0)
    norm_w = 1 + synth.hashed(D, 5, 0.2)
    mix_prev = np.abs(synth.hashed(24, 6, 2.0)) + 0.05
    h_out, mix_out, x_out = ref.hc_step(h_in, x_sub, mix_prev, fn, scale, base, norm_w)
    g["hc_h_out"], g["hc_mix_out"], g["hc_x_out"] = h_out, mix_out, x_out
    _, mix0, x0 = ref.hc_step(h_in, None, mix_prev, fn, scale, base, norm_w)          # layer-0 form: no sublayer output
    g["hc0_mix_out"], g["hc0_x_out"] = mix0, x0
    # --- compressor + index key, ratio 2 and ratio 1, 6 tokens
    cn, kn = 1 + synth.hashed(512, 7, 0.2), 1 + synth.hashed(128, 8, 0.2)
    wk = synth.hashed_bf16(128 * 512, 9, 0.2)
    ckv_in, cg_in = synth.hashed(6 * 512, 10, 3.0), synth.hashed(6 * 512, 11, 4.0)
    for ratio in (1, 2):
        for actq in (0, 1):
            ck, ik = ref.compress_tokens(ratio, ckv_in, cg_in if ratio > 1 else None, cn, wk, kn, actq)
            g["cmp_ckv_r%d_q%d" % (ratio, actq)], g["cmp_ikey_r%d_q%d" % (ratio, actq)] = ck, ik
    # --- sampling head: top-k descending with ties, log-sum-exp at two scales, log-softmax (tests/ref/arch_ref.cpp:199-219)
    sl = (3.0 * synth.hashed(3000, 12, 1.0)).astype(np.float32)
    sl[[7, 1207, 2407]] = 20.0                                   # ties -> lower index first
    g["smp_logits"] = sl
    g["smp_topk_v"], g["smp_topk_i"] = ref.topk_desc(sl, 64)
    g["smp_lse"] = np.array([ref.logsumexp(sl, 1.0), ref.logsumexp(sl, 1.0 / 0.7)], dtype=np.float64)
    g["smp_log_softmax"] = ref.log_softmax(sl)
    out = os.path.join(HERE, "golden_ref.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes,", len(g), "arrays")


if __name__ == "__main__":
    main()
