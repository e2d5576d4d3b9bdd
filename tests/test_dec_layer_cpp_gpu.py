"""The C++ layer-forward surface (include/ms_b200_dec_layer.hpp: ds41::encode_dec_attn_side / encode_dec_moe_ids /
encode_dec_final over attn::State) executed on the GPU for several tokens of a small model with the reference's layer
roles in miniature -- a window-only layer, a ratio-2 KV + index source, a ratio-1 source that also produces candidate
blocks, and an index source that scores only those candidates -- against the same sequence computed with the oracle
(hyper-connection steps, projections, window rows, compressor, indexer, sparse attention, router, MoE)."""
import os
import subprocess
import tempfile

import numpy as np
import pytest

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

DIM, QL, OAR, INTER, NE, TOPK, NTOK = 512, 256, 1024, 256, 16, 4, 6
ROLES = [(-1, -1, 0), (1, 1, 2), (2, 2, 1), (2, 3, 1)]      # (kv source, index source, ratio) per layer
CAND = 2


class Blob:
    def __init__(self):
        self.data = bytearray()
        self.lines = []

    def add(self, layer, name, t, rows, cols, arr):
        b = np.ascontiguousarray(arr).view(np.uint8).reshape(-1).tobytes()
        while len(self.data) % 256:
            self.data.append(0)
        off = len(self.data)
        self.data += b
        self.lines.append("w %d %s %d %d %d %d %d" % (layer, name, t, rows, cols, off, len(b)))
        return off


def build_model(seed=5):
    rng = np.random.default_rng(seed)
    f32 = lambda *s, sc=1.0: (rng.standard_normal(s) * sc).astype(np.float32)
    norm = lambda n: (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
    layers = []
    for l, (ks, isrc, ratio) in enumerate(ROLES):
        w = {}
        qw = lambda t, r, c, s: synth.random_weights(t, r, c, 1000 * l + s)
        w["attn_norm"], w["ffn_norm"], w["q_a_norm"], w["kv_norm"] = norm(DIM), norm(DIM), norm(QL), norm(512)
        w["q_a"], w["kv"] = qw(ol.Q6_K, QL, DIM, 1), qw(ol.Q6_K, 512, DIM, 2)
        # small query weights keep the attention logits O(1): with logits in the tens the softmax against the sink turns
        # the half-precision rounding of q . k into percent-level output differences, which says nothing about the path
        w["q_b"] = synth.random_weights(ol.Q6_K, 64 * 512, QL, 1000 * l + 3, 0.0005, 0.001)
        w["o_a"], w["o_b"] = qw(ol.Q6_K, OAR, 64 * 512 // 8, 4), qw(ol.Q6_K, DIM, OAR, 5)
        w["sinks"] = f32(64)
        if ks == l:
            w["c_kv"] = qw(ol.Q6_K, 512, DIM, 6)
            if ratio > 1:
                w["c_gate"] = qw(ol.Q6_K, 512, DIM, 7)
            w["c_norm"], w["idx_knorm"] = norm(512), norm(128)
            w["idx_k"] = synth.hashed_bf16(128 * 512, 100 + l, 0.2)
        if isrc == l:
            w["idx_qb"], w["idx_proj"] = qw(ol.BF16, 32 * 128, QL, 8), qw(ol.BF16, 32, DIM, 9)
        w["gate_inp"], w["bias"] = f32(NE, DIM, sc=0.05), f32(NE, sc=0.05)
        for nm in ("attn", "ffn"):
            w["hc_%s_fn" % nm] = f32(24, 4 * DIM, sc=0.03)
            w["hc_%s_scale" % nm] = np.array([0.7, 1.1, 0.9], np.float32)
            w["hc_%s_base" % nm] = f32(24, sc=0.5)
        w["sh_gate"], w["sh_up"], w["sh_down"] = qw(ol.Q8_0, INTER, DIM, 10), qw(ol.Q8_0, INTER, DIM, 11), qw(ol.Q8_0, DIM, INTER, 12)
        w["experts"] = [(qw(ol.IQ1_S, INTER, DIM, 20 + 3 * e), qw(ol.IQ1_S, INTER, DIM, 21 + 3 * e),
                         qw(ol.IQ2_XXS, DIM, INTER, 22 + 3 * e)) for e in range(NE)]
        layers.append(w)
    tokens = f32(NTOK, 4, DIM)
    return layers, norm(DIM), tokens


TYPES = {"q_a": (ol.Q6_K, QL, DIM), "kv": (ol.Q6_K, 512, DIM), "q_b": (ol.Q6_K, 64 * 512, QL), "o_a": (ol.Q6_K, OAR, 4096),
         "o_b": (ol.Q6_K, DIM, OAR), "c_kv": (ol.Q6_K, 512, DIM), "c_gate": (ol.Q6_K, 512, DIM), "idx_qb": (ol.BF16, 32 * 128, QL),
         "idx_proj": (ol.BF16, 32, DIM), "sh_gate": (ol.Q8_0, INTER, DIM), "sh_up": (ol.Q8_0, INTER, DIM),
         "sh_down": (ol.Q8_0, DIM, INTER), "idx_k": (ol.BF16, 128, 512), "gate_inp": (ol.F32, NE, DIM)}


def write_files(d, layers, out_norm, tokens):
    b = Blob()
    man = ["cfg %d %d %d %d %d %d %d %d %g %d" % (len(layers), DIM, QL, OAR, INTER, NE, TOPK, 1, 1.0, NTOK)]
    for l, (ks, isrc, ratio) in enumerate(ROLES):
        man.append("roles %d %d %d %d" % (l, ks, isrc, ratio))
    man.append("cand %d" % CAND)
    for l, w in enumerate(layers):
        for name, arr in w.items():
            if name == "experts":
                continue
            t, rows, cols = TYPES.get(name, (ol.F32, 1, arr.size))
            b.add(l, name, t, rows, cols, arr)
        table = np.zeros((NE, 3), np.uint64)
        for e, (g, u, dn) in enumerate(w["experts"]):
            for j, (nm, a) in enumerate((("expg", g), ("expu", u), ("expd", dn))):
                table[e, j] = b.add(l, "%s%d" % (nm, e), ol.IQ1_S, 0, 0, a)
        off = b.add(l, "exptable", 0, 0, 0, table)
        man.append("table %d %d" % (l, off))
    b.add(-1, "out_norm", ol.F32, 1, DIM, out_norm)
    b.add(-1, "tokens", ol.F32, NTOK, 4 * DIM, tokens)
    open(os.path.join(d, "blob"), "wb").write(bytes(b.data))
    open(os.path.join(d, "manifest"), "w").write("\n".join(man + b.lines) + "\n")


def oracle_forward(orc, layers, out_norm, tokens):
    """The sequence of dec_layer.mm:138-313 (without engram / prediction) on the CPU.  Returns per token (x_head, h,
    [router ids per layer]) and the KV sources' cache rows."""
    import ctypes as C
    L = len(layers)
    P = lambda a: a.ctypes.data_as(C.c_void_p)
    plain, yarn = orc.rope_table(256, False), orc.rope_table(256, True)
    mv = lambda w, name, x, groups=1: orc.matvec(TYPES[name][0], w[name], TYPES[name][1], TYPES[name][2], x, groups)[0].astype(np.float32)
    win = [np.zeros((128, 512), np.float32) for _ in range(L)]
    src = {l: {"ckv": [], "ikey": [], "st_kv": np.zeros((max(1, r), 512), np.float32),
               "st_sc": np.full((max(1, r), 512), -np.inf, np.float32)} for l, (ks, _, r) in enumerate(ROLES) if ks == l}
    topk = {}
    cand = np.full(2048, -1, np.int32)
    ident = np.zeros(24, np.float32); ident[0] = 1
    outs = []
    for pos in range(tokens.shape[0]):
        h = tokens[pos].reshape(-1).copy()
        sub, mixA, mixF = None, None, ident
        ids_all = []
        for l, w in enumerate(layers):
            ks, isrc, ratio = ROLES[l]
            cs = (plain if ratio == 0 else yarn)[pos]
            h, mixA, x = orc.hc_step(h, sub, mixF, w["hc_attn_fn"], w["hc_attn_scale"], w["hc_attn_base"], w["attn_norm"], DIM)
            qa, kv = mv(w, "q_a", x), mv(w, "kv", x)
            qrn = orc.rmsnorm(qa, w["q_a_norm"], 1e-20)
            q = mv(w, "q_b", qrn)
            win[l][pos % 128] = orc.window_row(kv, w["kv_norm"], cs, False).astype(np.float16).astype(np.float32)
            if ks == l:
                s = src[l]
                r = max(1, ratio)
                ckv_in = mv(w, "c_kv", x)
                cg = mv(w, "c_gate", x) if ratio > 1 else None
                row_c, row_k = np.zeros(512, np.float32), np.zeros(128, np.float32)
                wk = np.ascontiguousarray(w["idx_k"], dtype=np.uint16)
                if orc.lib.orc_compress_token(r, pos, P(ckv_in), P(cg) if cg is not None else None, P(w["c_norm"]), P(wk),
                                              P(w["idx_knorm"]), P(yarn), 0, 512, 128, P(s["st_kv"]), P(s["st_sc"]), P(row_c), P(row_k)):
                    # the caches hold f16
                    s["ckv"].append(row_c.astype(np.float16).astype(np.float32)); s["ikey"].append(row_k.astype(np.float16).astype(np.float32))
            if isrc == l:
                iw, iq = mv(w, "idx_proj", x), mv(w, "idx_qb", qrn)
                keys = np.array(src[ks]["ikey"], np.float32).reshape(-1, 128)
                n = (pos + 1) // max(1, ROLES[ks][2])
                tk = np.full(512, -1, np.int32)
                if n > 0:
                    qi, wi = orc.index_q(iq.reshape(32, 128), iw, cs, False, 32, 128)
                    sc = orc.index_scores(qi, wi, keys[:n])
                    if l > CAND:
                        m = np.full(n, -np.inf, np.float32)
                        for b in cand[cand >= 0]:
                            m[b * 8:b * 8 + 8] = sc[b * 8:b * 8 + 8]
                        sc = m
                    tk = orc.topk_sorted(sc, 512)
                    if l == CAND:
                        cand = orc.candidate_blocks(sc)
                topk[l] = tk
            rows = [win[l][i] for i in range(min(pos + 1, 128))]
            if ks >= 0 and isrc >= 0:
                rows += [src[ks]["ckv"][i] for i in topk[isrc] if i >= 0]
            aout = orc.sparse_attn(q.reshape(64, 512), cs, np.array(rows, np.float32), w["sinks"])
            oa = mv(w, "o_a", aout.reshape(-1), 8)
            sub = mv(w, "o_b", oa)
            h, mixF, x = orc.hc_step(h, sub, mixA, w["hc_ffn_fn"], w["hc_ffn_scale"], w["hc_ffn_base"], w["ffn_norm"], DIM)
            logits = (w["gate_inp"].astype(np.float64) @ x.astype(np.float64)).astype(np.float32)
            ids, rw = orc.router(logits, w["bias"], TOPK, 1, 1.0)
            ids_all.append((np.array(ids, np.int32), x.copy(), logits.copy(), w["bias"]))
            ex = [w["experts"][i] for i in ids]
            hh, y, ymag, hmag = orc.moe_decode(DIM, INTER, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, [e[0] for e in ex] + [w["sh_gate"]],
                                               [e[1] for e in ex] + [w["sh_up"]], [e[2] for e in ex] + [w["sh_down"]], rw, x,
                                               np.zeros(DIM, np.float32))
            sub = y.astype(np.float32)
        h, _, xh = orc.hc_step(h, sub, mixF, None, None, None, out_norm, DIM)
        outs.append((xh, h, ids_all))
    return outs, src


def test_cpp_layer_forward_matches_oracle():
    orc = ol.Oracle()
    layers, out_norm, tokens = build_model()
    lib_dir = os.path.join(ROOT, "macseek_b200")
    with tempfile.TemporaryDirectory() as d:
        write_files(d, layers, out_norm, tokens)
        exe = os.path.join(d, "run")
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                               os.path.join(ROOT, "tests", "dec_layer_exec.cpp"), "-o", exe, "-L", lib_dir, "-lmacseek_b200",
                               "-Wl,-rpath," + lib_dir, "-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64"])
        subprocess.check_call([exe, os.path.join(d, "manifest"), os.path.join(d, "blob"), os.path.join(d, "out")])
        raw = np.fromfile(os.path.join(d, "out"), dtype=np.uint8)
    want, src = oracle_forward(orc, layers, out_norm, tokens)
    L = len(layers)
    off = 0
    for pos in range(NTOK):
        xh_w, h_w, ids_w = want[pos]
        for l in range(L):
            ids = raw[off:off + 4 * TOPK].view(np.int32); off += 4 * TOPK
            x = raw[off:off + 4 * DIM].view(np.float32); off += 4 * DIM
            ids_o, x_o, logits_o, bias_o = ids_w[l]
            assert np.max(np.abs(x - x_o)) <= 2e-3 * np.max(np.abs(x_o)), (pos, l, np.max(np.abs(x - x_o)), np.max(np.abs(x_o)))
            if sorted(ids.tolist()) != sorted(ids_o.tolist()):
                # a different pick is acceptable only between experts whose keys are a near tie
                key = 1 / (1 + np.exp(-logits_o.astype(np.float64))) + bias_o
                d = set(ids.tolist()) ^ set(ids_o.tolist())
                assert len(d) == 2 and abs(key[list(d)[0]] - key[list(d)[1]]) <= 2e-3, (pos, l, ids, ids_o)
                pytest.skip("router near-tie at token %d layer %d: the two sequences diverge from here" % (pos, l))
        xh = raw[off:off + 4 * DIM].view(np.float32); off += 4 * DIM
        h = raw[off:off + 16 * DIM].view(np.float32); off += 16 * DIM
        assert np.max(np.abs(xh - xh_w)) <= 2e-3 * np.max(np.abs(xh_w)), (pos, np.max(np.abs(xh - xh_w)))
        assert np.max(np.abs(h - h_w)) <= 2e-3 * np.max(np.abs(h_w)), pos
    for l in sorted(src):
        rows = NTOK // max(1, ROLES[l][2])
        ck = raw[off:off + rows * 512 * 2].view(np.float16).astype(np.float32).reshape(rows, 512); off += rows * 512 * 2
        ik = raw[off:off + rows * 128 * 2].view(np.float16).astype(np.float32).reshape(rows, 128); off += rows * 128 * 2
        wc, wk = np.array(src[l]["ckv"], np.float32), np.array(src[l]["ikey"], np.float32)
        assert np.max(np.abs(ck - wc)) <= 3e-3 * np.max(np.abs(wc)), l
        assert np.max(np.abs(ik - wk)) <= 3e-3 * np.max(np.abs(wk)), l
    assert off == raw.size
