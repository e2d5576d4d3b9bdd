"""ctypes bindings of the CPU oracle (oracle/libmsb_oracle.so) and, when it has been built, of the reference
project's own routines (oracle/_ref/libmsref.so).  Test infrastructure: imported by tests/, by bench.py's CPU-baseline
legs and by __graft_entry__.smoke() only."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "libmsb_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libmsref.so")

# ggml type ids (src/kernels/quant_types.hpp:10-12 of the reference)
F32, F16, Q8_0, Q5_K, Q6_K, IQ2_XXS, IQ1_S, IQ4_NL, BF16, MXFP4 = 0, 1, 8, 13, 14, 16, 19, 20, 30, 39
TYPE_NAMES = {F32: "F32", F16: "F16", Q8_0: "Q8_0", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ2_XXS: "IQ2_XXS", IQ1_S: "IQ1_S",
              IQ4_NL: "IQ4_NL", BF16: "BF16", MXFP4: "MXFP4"}
BLOCK = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q8_0: (32, 34), Q5_K: (256, 176), Q6_K: (256, 210),
         IQ2_XXS: (256, 66), IQ1_S: (256, 50), IQ4_NL: (32, 18), MXFP4: (32, 17)}


def row_bytes(t, cols):
    be, bb = BLOCK[t]
    return cols // be * bb


def build_oracle(force=False):
    src = os.path.join(ORACLE_DIR, "msb_oracle.c")
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "oracle"], stdout=subprocess.DEVNULL)
    return ORACLE_SO


def build_ref(reference="/root/reference"):
    """Compile the reference's own CPU routines where its checkout is present; returns the path or None."""
    if os.path.isdir(os.path.join(reference, "tests", "ref")):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "ref", "REF=" + reference], stdout=subprocess.DEVNULL)
    return REF_SO if os.path.exists(REF_SO) else None


def _p(a, ct=C.c_void_p):
    return a.ctypes.data_as(ct)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class MoeArgs(C.Structure):
    _fields_ = [("dim", C.c_int), ("inter", C.c_int), ("n_routed", C.c_int), ("has_shared", C.c_int),
                ("t_gate_up", C.c_int), ("t_down", C.c_int), ("t_shared", C.c_int),
                ("gate", C.c_void_p * 16), ("up", C.c_void_p * 16), ("down", C.c_void_p * 16),
                ("w", C.c_void_p), ("x", C.c_void_p), ("limit", C.c_float), ("threads", C.c_int)]


class Oracle:
    """The C restatement (oracle/msb_oracle.c)."""

    def __init__(self):
        self.lib = C.CDLL(build_oracle())
        L = self.lib
        L.orc_row_bytes.restype = C.c_size_t
        L.orc_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.orc_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.orc_matvec.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int64, C.c_int,
                                 C.c_void_p, C.c_void_p, C.c_int]
        L.orc_max_norm_err.restype = C.c_double
        L.orc_max_norm_err.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.orc_moe_decode.argtypes = [C.POINTER(MoeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        L.orc_router.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
        L.orc_route_lists.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 6
        L.orc_argmax.argtypes = [C.c_void_p, C.c_int]
        L.orc_topk_desc.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_logsumexp.restype = C.c_double
        L.orc_logsumexp.argtypes = [C.c_void_p, C.c_int, C.c_double]
        L.orc_log_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.orc_gumbel.restype = C.c_double
        L.orc_gumbel.argtypes = [C.c_uint32, C.c_uint64, C.c_uint32]
        L.orc_sample_top_p.restype = C.c_uint32
        L.orc_sample_top_p.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_double]
        L.orc_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_double]
        L.orc_rope_table.argtypes = [C.c_int, C.c_int, C.c_void_p]
        for n in ("orc_round_e4m3", "orc_round_e2m1"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        for n in ("orc_fp8_sim", "orc_fp4_sim_e8m0", "orc_fp4_sim_e4m3"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_int]
        L.orc_e4m3_to_f32.restype = C.c_float
        L.orc_e4m3_to_f32.argtypes = [C.c_uint8]
        L.orc_f32_to_e4m3.restype = C.c_uint8
        L.orc_f32_to_e4m3.argtypes = [C.c_float]
        L.orc_index_q.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_index_scores.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.orc_topk_sorted.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.orc_candidate_blocks.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        L.orc_sparse_attn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                      C.c_void_p, C.c_int]
        L.orc_window_row.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        self.threads = L.orc_hardware_threads()

    # ---- quant ----
    def dequant(self, t, raw, n):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        self.lib.orc_dequant_row(t, _p(raw), _p(out), n)
        return out

    def matvec(self, t, W, rows, cols, x, groups=1, threads=None):
        """x: [cols*groups] or [n][cols*groups]; returns (y, mag) float64 of shape [rows] or [n][rows]."""
        W = np.ascontiguousarray(W, dtype=np.uint8)
        x = _f32(x)
        n = 1 if x.ndim == 1 else x.shape[0]
        y = np.zeros((n, rows), dtype=np.float64)
        mag = np.zeros((n, rows), dtype=np.float64)
        self.lib.orc_matvec(t, _p(W), rows, cols, _p(x), n, cols * groups, groups, _p(y), _p(mag),
                            self.threads if threads is None else threads)
        return (y[0], mag[0]) if x.ndim == 1 else (y, mag)

    def max_norm_err(self, got, ref, mag):
        got = _f32(got).ravel()
        ref = np.ascontiguousarray(ref, dtype=np.float64).ravel()
        mag = np.ascontiguousarray(mag, dtype=np.float64).ravel()
        return self.lib.orc_max_norm_err(_p(got), _p(ref), _p(mag), got.size, None)

    def moe_decode(self, dim, inter, t_gu, t_down, t_shared, gate, up, down, w, x, y0, has_shared=True, limit=10.0,
                   threads=None):
        """gate/up/down: lists of uint8 arrays, routed experts first, shared expert last (if has_shared).
        Returns (h [n_exp][inter] f32, y f64, ymag f64, hmag f64)."""
        n_exp = len(gate)
        n_routed = n_exp - (1 if has_shared else 0)
        a = MoeArgs()
        a.dim, a.inter, a.n_routed, a.has_shared = dim, inter, n_routed, int(has_shared)
        a.t_gate_up, a.t_down, a.t_shared = t_gu, t_down, t_shared
        keep = []
        for i in range(n_exp):
            for name, lst in (("gate", gate), ("up", up), ("down", down)):
                arr = np.ascontiguousarray(lst[i], dtype=np.uint8)
                keep.append(arr)
                getattr(a, name)[i] = arr.ctypes.data
        w = _f32(w if n_routed else np.zeros(1))
        x = _f32(x)
        a.w, a.x, a.limit = w.ctypes.data, x.ctypes.data, limit
        a.threads = self.threads if threads is None else threads
        h = np.zeros((n_exp, inter), dtype=np.float32)
        y = np.array(y0, dtype=np.float64).copy()
        ymag = np.abs(y).copy()
        hmag = np.zeros((n_exp, inter), dtype=np.float64)
        self.lib.orc_moe_decode(C.byref(a), _p(h), _p(y), _p(ymag), _p(hmag))
        return h, y, ymag, hmag

    # ---- router ----
    def router(self, logits, bias, k, score_fn=0, route_scale=1.5):
        logits = _f32(logits)
        E = logits.shape[-1]
        bias = _f32(bias)
        ids = np.zeros(k, dtype=np.int32)
        w = np.zeros(k, dtype=np.float32)
        self.lib.orc_router(_p(logits), _p(bias), E, k, score_fn, route_scale, _p(ids), _p(w))
        return ids, w

    def route_lists(self, ids, w, n, k, E):
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        w = _f32(w)
        counts = np.zeros(E, np.uint32); offsets = np.zeros(E + 1, np.uint32)
        entry = np.zeros(n * k, np.uint32); tok = np.zeros(n * k, np.uint32)
        lw = np.zeros(n * k, np.float32); slot_of = np.zeros(n * k, np.uint32)
        self.lib.orc_route_lists(_p(ids), _p(w), n, k, E, _p(counts), _p(offsets), _p(entry), _p(tok), _p(lw), _p(slot_of))
        return counts, offsets, entry, tok, lw, slot_of

    def argmax(self, x):
        x = _f32(x)
        return self.lib.orc_argmax(_p(x), x.size)

    def topk_desc(self, x, k):
        x = _f32(x)
        v, idx = np.empty(k, np.float32), np.empty(k, np.uint32)
        self.lib.orc_topk_desc(_p(x), x.size, k, _p(v), _p(idx))
        return v, idx

    def logsumexp(self, x, scale=1.0):
        x = _f32(x)
        return self.lib.orc_logsumexp(_p(x), x.size, float(scale))

    def log_softmax(self, x):
        x = _f32(x); y = np.empty_like(x)
        self.lib.orc_log_softmax(_p(x), _p(y), x.size)
        return y

    def gumbel(self, i, seed, row=0):
        return self.lib.orc_gumbel(int(i), int(seed), int(row))

    def sample_top_p(self, vals, ids, k, lse, temperature, top_p, u):
        vals = _f32(vals); ids = np.ascontiguousarray(ids, dtype=np.uint32)
        return int(self.lib.orc_sample_top_p(_p(vals), _p(ids), k, lse, temperature, top_p, u))

    def rmsnorm(self, x, w, eps):
        x = _f32(x); y = np.empty_like(x)
        wv = _f32(w) if w is not None else None
        self.lib.orc_rmsnorm(_p(x), _p(wv) if wv is not None else None, _p(y), x.size, eps)
        return y

    # ---- attention ----
    def rope_table(self, max_pos, yarn):
        out = np.empty((max_pos, 32, 2), dtype=np.float32)
        self.lib.orc_rope_table(max_pos, int(yarn), _p(out))
        return out

    def sim(self, name, x):
        x = _f32(x).copy()
        getattr(self.lib, "orc_" + name)(_p(x), x.size)
        return x

    def e4m3_to_f32(self, b):
        b = np.ascontiguousarray(b, dtype=np.uint8)
        lut = np.array([self.lib.orc_e4m3_to_f32(i) for i in range(256)], dtype=np.float32)
        return lut[b]

    def f32_to_e4m3(self, x):
        x = _f32(x)
        return np.array([self.lib.orc_f32_to_e4m3(float(v)) for v in x.ravel()], dtype=np.uint8).reshape(x.shape)

    def index_q(self, q_raw, w_raw, cs, actq, heads, dim):
        q_raw = _f32(q_raw); w_raw = _f32(w_raw); cs = _f32(cs)
        q = np.empty(heads * dim, np.float32); w = np.empty(heads, np.float32)
        self.lib.orc_index_q(_p(q_raw), _p(w_raw), _p(cs), int(actq), heads, dim, _p(q), _p(w))
        return q.reshape(heads, dim), w

    def index_scores(self, q, w, keys, threads=None):
        q = _f32(q); w = _f32(w); keys = _f32(keys)
        heads, dim = q.shape
        n = keys.shape[0]
        sc = np.empty(n, np.float32)
        self.lib.orc_index_scores(_p(q), _p(w), _p(keys), heads, dim, n, _p(sc), self.threads if threads is None else threads)
        return sc

    def topk_sorted(self, sc, k):
        sc = _f32(sc)
        out = np.empty(k, np.int32)
        self.lib.orc_topk_sorted(_p(sc), sc.size, k, _p(out))
        return out

    def candidate_blocks(self, sc, bs=8, cap=2048):
        sc = _f32(sc)
        out = np.empty(cap, np.int32)
        self.lib.orc_candidate_blocks(_p(sc), sc.size, bs, cap, _p(out))
        return out

    def sparse_attn(self, q_raw, cs, rows, sinks, threads=None):
        q_raw = _f32(q_raw); cs = _f32(cs); rows = _f32(rows); sinks = _f32(sinks)
        H, D = q_raw.shape
        out = np.empty((H, D), np.float32)
        self.lib.orc_sparse_attn(_p(q_raw), _p(cs), _p(rows), rows.shape[0], _p(sinks), H, D, _p(out),
                                 self.threads if threads is None else threads)
        return out

    def window_row(self, kv_raw, norm_w, cs, actq):
        kv_raw = _f32(kv_raw)
        out = np.empty_like(kv_raw)
        self.lib.orc_window_row(_p(kv_raw), _p(_f32(norm_w)), _p(_f32(cs)), int(actq), kv_raw.size, _p(out))
        return out


def _opt(a):
    return _p(a) if a is not None else None


def _oracle_hc_step(self, h_in, x_sub, mix_prev, fn, scale, base, norm_w, D, want_x=True):
    """hc_step of one token (arch_ref.cpp:75-95): returns (h_out, mix_out, x_out); parts not asked for are None."""
    h_in = _f32(h_in)
    h_out = np.array(h_in, copy=True)
    mix_out = np.zeros(24, np.float32) if fn is not None else None
    x_out = np.zeros(D, np.float32) if want_x else None
    keep = [_f32(v) if v is not None else None for v in (x_sub, mix_prev, fn, scale, base, norm_w)]
    self.lib.orc_hc_step(_p(h_in), _opt(keep[0]), _p(keep[1]), _opt(keep[2]), _opt(keep[3]), _opt(keep[4]), _opt(keep[5]),
                         D, _p(h_out), _opt(mix_out), _opt(x_out))
    return h_out, mix_out, x_out


def _oracle_compress_tokens(self, ratio, ckv_in, cgate_in, cnorm_w, wk_bf16, knorm_w, actq, D=512, ID=128):
    """Feeds tokens 0 .. n-1 to a fresh source (attn_ref.cpp:116-161): returns (ckv rows [rows][D], ikey rows [rows][ID])."""
    ckv_in = _f32(ckv_in).reshape(-1, D)
    n = ckv_in.shape[0]
    cg = _f32(cgate_in).reshape(-1, D) if cgate_in is not None else None
    tab = self.rope_table(n + 1, True)
    st_kv = np.zeros((ratio, D), np.float32)
    st_sc = np.full((ratio, D), -np.inf, np.float32)
    wk = np.ascontiguousarray(wk_bf16, dtype=np.uint16)
    cn, kn = _f32(cnorm_w), _f32(knorm_w)
    ck, ik = [], []
    row_c, row_k = np.zeros(D, np.float32), np.zeros(ID, np.float32)
    for p in range(n):
        g = np.ascontiguousarray(cg[p]) if cg is not None else None
        x = np.ascontiguousarray(ckv_in[p])
        if self.lib.orc_compress_token(ratio, p, _p(x), _opt(g), _p(cn), wk.ctypes.data_as(C.c_void_p), _p(kn), _p(tab),
                                       int(actq), D, ID, _p(st_kv), _p(st_sc), _p(row_c), _p(row_k)):
            ck.append(row_c.copy()); ik.append(row_k.copy())
    return np.array(ck, np.float32).reshape(-1, D), np.array(ik, np.float32).reshape(-1, ID)


Oracle.hc_step = _oracle_hc_step
Oracle.compress_tokens = _oracle_compress_tokens


class Ref:
    """The reference project's own routines (oracle/_ref/libmsref.so); None-safe: use Ref.load()."""

    @staticmethod
    def load(build=True):
        path = build_ref() if build else (REF_SO if os.path.exists(REF_SO) else None)
        return Ref(path) if path else None

    def __init__(self, path):
        self.lib = C.CDLL(path)
        L = self.lib
        L.msref_dequant_row.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64]
        L.msref_row_bytes.restype = C.c_uint64
        L.msref_row_bytes.argtypes = [C.c_int, C.c_int64]
        L.msref_random_blocks.argtypes = [C.c_int, C.c_int64, C.c_uint32, C.c_float, C.c_void_p]
        L.msref_ref_matvec.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int, C.c_int]
        L.msref_router.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float]
        L.msref_route_lists.argtypes = [C.c_void_p, C.c_void_p, C.c_int] + [C.c_void_p] * 6
        L.msref_rope_table.argtypes = [C.c_int, C.c_int, C.c_void_p]
        for n in ("msref_round_e4m3", "msref_round_e2m1"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        for n in ("msref_fp8_sim", "msref_fp4_sim_e8m0", "msref_fp4_sim_e4m3"):
            getattr(L, n).argtypes = [C.c_void_p, C.c_int]
        L.msref_index_q.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.msref_index_scores.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.msref_topk_sorted.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        L.msref_candidate_blocks.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.msref_sparse_attn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        L.msref_window_row.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        L.msref_argmax.argtypes = [C.c_void_p, C.c_int]
        L.msref_topk.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.msref_logsumexp.restype = C.c_double
        L.msref_logsumexp.argtypes = [C.c_void_p, C.c_int, C.c_double]
        L.msref_log_softmax.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.msref_rmsnorm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_double]
        self.threads = L.msref_hardware_threads()

    def random_blocks(self, t, n, seed, scale=0.01):
        out = np.empty(row_bytes(t, n), dtype=np.uint8)
        self.lib.msref_random_blocks(t, n, seed, scale, _p(out))
        return out

    def dequant(self, t, raw, n):
        raw = np.ascontiguousarray(raw, dtype=np.uint8)
        out = np.empty(n, dtype=np.float32)
        self.lib.msref_dequant_row(t, _p(raw), _p(out), n)
        return out

    def matvec(self, t, W, rows, cols, x, groups=1, threads=1):
        W = np.ascontiguousarray(W, dtype=np.uint8); x = _f32(x)
        y = np.zeros(rows, np.float64); mag = np.zeros(rows, np.float64)
        self.lib.msref_ref_matvec(t, _p(W), rows, cols, _p(x), _p(y), _p(mag), groups, threads)
        return y, mag

    def router(self, logits, bias, route_scale=1.5):
        logits = _f32(logits); bias = _f32(bias)
        ids = np.zeros(6, np.int32); w = np.zeros(6, np.float32)
        self.lib.msref_router(_p(logits), _p(bias), _p(ids), _p(w), route_scale)
        return ids, w

    def route_lists(self, ids, w, n):
        ids = np.ascontiguousarray(ids, dtype=np.int32); w = _f32(w)
        E, k = 384, 6
        counts = np.zeros(E, np.uint32); offsets = np.zeros(E + 1, np.uint32)
        entry = np.zeros(n * k, np.uint32); tok = np.zeros(n * k, np.uint32)
        lw = np.zeros(n * k, np.float32); slot_of = np.zeros(n * k, np.uint32)
        self.lib.msref_route_lists(_p(ids), _p(w), n, _p(counts), _p(offsets), _p(entry), _p(tok), _p(lw), _p(slot_of))
        return counts, offsets, entry, tok, lw, slot_of

    def rope_table(self, max_pos, yarn):
        out = np.empty((max_pos, 32, 2), dtype=np.float32)
        self.lib.msref_rope_table(max_pos, int(yarn), _p(out))
        return out

    def sim(self, name, x):
        x = _f32(x).copy()
        getattr(self.lib, "msref_" + name)(_p(x), x.size)
        return x

    def index_q(self, q_raw, w_raw, cs, actq):
        q_raw = _f32(q_raw); w_raw = _f32(w_raw); cs = _f32(cs)
        q = np.empty(32 * 128, np.float32); w = np.empty(32, np.float32)
        self.lib.msref_index_q(_p(q_raw), _p(w_raw), _p(cs), int(actq), _p(q), _p(w))
        return q.reshape(32, 128), w

    def index_scores(self, q, w, keys):
        q = _f32(q); w = _f32(w); keys = _f32(keys)
        sc = np.empty(keys.shape[0], np.float32)
        self.lib.msref_index_scores(_p(q), _p(w), _p(keys), keys.shape[0], _p(sc))
        return sc

    def topk_sorted(self, sc, k):
        sc = _f32(sc); out = np.empty(k, np.int32)
        self.lib.msref_topk_sorted(_p(sc), sc.size, k, _p(out))
        return out

    def candidate_blocks(self, sc):
        sc = _f32(sc); out = np.empty(2048, np.int32)
        self.lib.msref_candidate_blocks(_p(sc), sc.size, _p(out))
        return out

    def sparse_attn(self, q_raw, cs, rows, sinks):
        q_raw = _f32(q_raw); cs = _f32(cs); rows = _f32(rows); sinks = _f32(sinks)
        out = np.empty((64, 512), np.float32)
        self.lib.msref_sparse_attn(_p(q_raw), _p(cs), _p(rows), rows.shape[0], _p(sinks), _p(out))
        return out

    def window_row(self, kv_raw, norm_w, cs, actq):
        kv_raw = _f32(kv_raw); out = np.empty(512, np.float32)
        self.lib.msref_window_row(_p(kv_raw), _p(_f32(norm_w)), _p(_f32(cs)), int(actq), _p(out))
        return out

    def argmax(self, x):
        x = _f32(x)
        return self.lib.msref_argmax(_p(x), x.size)

    def topk_desc(self, x, k):
        x = _f32(x)
        v, idx = np.empty(k, np.float32), np.empty(k, np.uint32)
        self.lib.msref_topk(_p(x), x.size, k, _p(v), _p(idx))
        return v, idx

    def logsumexp(self, x, scale=1.0):
        x = _f32(x)
        return self.lib.msref_logsumexp(_p(x), x.size, float(scale))

    def log_softmax(self, x):
        x = _f32(x); y = np.empty_like(x)
        self.lib.msref_log_softmax(_p(x), _p(y), x.size)
        return y

    def rmsnorm(self, x, w, eps):
        x = _f32(x); y = np.empty_like(x)
        self.lib.msref_rmsnorm(_p(x), _p(_f32(w)), _p(y), x.size, eps)
        return y

    def hc_step(self, h_in, x_sub, mix_prev, fn, scale, base, norm_w, want_x=True):
        h_in = _f32(h_in)
        h_out = np.array(h_in, copy=True)
        mix_out = np.zeros(24, np.float32) if fn is not None else None
        x_out = np.zeros(5120, np.float32) if want_x else None
        keep = [_f32(v) if v is not None else None for v in (x_sub, mix_prev, fn, scale, base, norm_w)]
        self.lib.msref_hc_step(_p(h_in), _opt(keep[0]), _p(keep[1]), _opt(keep[2]), _opt(keep[3]), _opt(keep[4]),
                               _opt(keep[5]), _p(h_out), _opt(mix_out), _opt(x_out))
        return h_out, mix_out, x_out

    def compress_tokens(self, ratio, ckv_in, cgate_in, cnorm_w, wk_bf16, knorm_w, actq):
        ckv_in = _f32(ckv_in).reshape(-1, 512)
        n = ckv_in.shape[0]
        cg = _f32(cgate_in).reshape(-1, 512) if cgate_in is not None else None
        ck = np.zeros((n, 512), np.float32); ik = np.zeros((n, 128), np.float32)
        wk = np.ascontiguousarray(wk_bf16, dtype=np.uint16)
        self.lib.msref_compress_tokens.restype = C.c_int
        rows = self.lib.msref_compress_tokens(ratio, n, _p(ckv_in), _opt(cg), _p(_f32(cnorm_w)),
                                              wk.ctypes.data_as(C.c_void_p), _p(_f32(knorm_w)), int(actq), _p(ck), _p(ik))
        return ck[:rows], ik[:rows]
