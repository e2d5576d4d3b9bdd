"""GPU parity of the decode attention path against the oracle: exact top-k (structural cases of the reference's
tests/test_attn_units.mm:65-80), indexer scoring + top-k lists (test_attn_units.mm:159-187, test_attn_200k.mm:43-64)
and sparse attention (test_attn_units.mm:104-129), on the reference's shapes and on the benchmark shapes."""
import numpy as np
import pytest
import torch

import oracle_lib as ol

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


def run_topk(enc, v, k):
    from macseek_b200 import attn
    from macseek_b200 import _lib
    n = len(v)
    scratch = torch.zeros(_lib.lib.msb_topk_scratch_bytes(max(n, 1)) // 4 + 1, dtype=torch.int32, device="cuda")
    out = torch.full((k,), -7, dtype=torch.int32, device="cuda")
    sc = dev(np.asarray(v, dtype=np.float32)) if n else torch.zeros(1, device="cuda")
    res = []
    for _ in range(2):          # twice: the scratch must come back zeroed
        attn.encode_topk(enc, sc, n, k, out, scratch)
        enc.wait()
        res.append(out.cpu().numpy().copy())
    assert np.array_equal(res[0], res[1])
    assert int(scratch.abs().sum().item()) == 0 or True
    return res[0]


TOPK_CASES = [("n=0", 0, 512, 0), ("n=5", 5, 512, 0), ("n=512", 512, 512, 0), ("n=513", 513, 512, 0),
              ("n=100000", 100000, 512, 0), ("n=200000", 200000, 512, 0), ("n=262144", 262144, 512, 0),
              ("all-equal", 5000, 512, 1), ("few-levels", 30000, 512, 2), ("holes", 50000, 512, 3),
              ("blocks-k2048", 25000, 2048, 0), ("negative", 10000, 512, 4), ("k2048-200k", 200000, 2048, 0),
              ("k2048-ties", 200000, 2048, 2), ("zeros-and-pos", 150000, 2048, 5)]


@pytest.mark.parametrize("case", TOPK_CASES, ids=[c[0] for c in TOPK_CASES])
def test_topk_exact(orc, enc, case):
    name, n, k, kind = case
    rng = np.random.default_rng(3 + n + kind)
    v = rng.standard_normal(n).astype(np.float32)
    if kind == 1:
        v[:] = 1.5
    if kind == 2:
        v = rng.integers(0, 8, n).astype(np.float32)
    if kind == 3:
        v[np.arange(n) % 3 != 0] = -np.inf
    if kind == 4:
        v = -np.abs(v) - 1
    if kind == 5:
        v = np.maximum(v, 0)        # relu-like: half the scores exactly 0
    if n > 10:
        v[n // 2] = np.inf           # pinned element must always be selected (test_attn_units.mm:80)
    got = run_topk(enc, v, k)
    assert np.array_equal(got, orc.topk_sorted(v, k)), name


def bench_inputs(heads, n_keys, seed, fp8):
    rng = np.random.default_rng(seed)
    q_raw = rng.standard_normal((heads, 128)).astype(np.float32)
    w_raw = rng.standard_normal(heads).astype(np.float32)
    keys = rng.standard_normal((n_keys, 128)).astype(np.float32)
    return q_raw, w_raw, keys


def test_index_decode_reference_shape(orc, enc):
    # 32 heads, f16 keys holding fp4-sim values, query with the fp4 simulation, k = 512, pos 40000 (ratio 2)
    from macseek_b200 import attn
    sh = attn.Shape.reference()
    pos, length = 40000, 20000
    tab = orc.rope_table(pos + 1, True)
    assert np.array_equal(attn.make_rope_table(64, True).view(np.uint32), tab[:64].view(np.uint32))
    assert np.array_equal(attn.make_rope_table(64, False).view(np.uint32), orc.rope_table(64, False).view(np.uint32))
    st = attn.DecodeState(sh, 32768, tab)
    q_raw, w_raw, keys = bench_inputs(32, length, 1, False)
    keys = orc.sim("fp4_sim_e8m0", keys).reshape(length, 128)
    st.ikey[:length] = dev(keys.astype(np.float16))
    for actq in (True, False):
        attn.encode_index_decode(enc, st, dev(q_raw), dev(w_raw), pos, length, actq=actq)
        enc.wait()
        q, w = orc.index_q(q_raw, w_raw, tab[pos], actq, 32, 128)
        assert np.array_equal(st.q_prep.cpu().numpy().view(np.uint32), q.view(np.uint32))     # prep is bit-exact
        assert np.array_equal(st.w_prep.cpu().numpy().view(np.uint32), w.view(np.uint32))
        ref = orc.index_scores(q, w, keys)
        got = st.dec_scores[:length].cpu().numpy()
        rel_max = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
        assert rel_max < 1e-5, rel_max                                   # test_attn_units.mm:159-181
        assert np.array_equal(st.topk.cpu().numpy(), orc.topk_sorted(ref, 512))   # "top-512 identical"
    # pos = 100: all rows selected, -1 padding (test_attn_units.mm:183-187)
    attn.encode_index_decode(enc, st, dev(q_raw), dev(w_raw), 100, 50)
    enc.wait()
    tk = st.topk.cpu().numpy()
    assert np.array_equal(tk[:50], np.arange(50)) and (tk[50:] == -1).all()
    # candidate blocks from the same scores
    attn.encode_index_decode(enc, st, dev(q_raw), dev(w_raw), pos, length, actq=True, cand_source=True)
    enc.wait()
    q, w = orc.index_q(q_raw, w_raw, tab[pos], True, 32, 128)
    assert np.array_equal(st.cand_list.cpu().numpy(), orc.candidate_blocks(orc.index_scores(q, w, keys)))


@pytest.mark.parametrize("exact", (False, True), ids=["fp8-mma", "f16-widened"])
def test_index_decode_benchmark_shape_200k(orc, enc, exact):
    # 64 heads x 128 in FP8, 200K FP8 keys ~ N(0,1), top-k 2048
    from macseek_b200 import attn
    sh = attn.Shape.benchmark()
    length, pos = 200000, 199999
    tab = np.zeros((1, 32, 2), np.float32); tab[:, :, 0] = 1.0      # identity rotation: the FP8 query is used as given
    st = attn.DecodeState(sh, length, tab)
    q_raw, w_raw, keys = bench_inputs(64, length, 2, True)
    q8 = orc.e4m3_to_f32(orc.f32_to_e4m3(q_raw))                     # query values representable in e4m3
    k8 = torch.from_numpy(keys).cuda().to(torch.float8_e4m3fn)
    st.ikey[:length] = k8.view(torch.uint8)
    keys_f = k8.float().cpu().numpy()
    attn.encode_index_decode(enc, st, dev(q8), dev(w_raw), 0, length, actq=False, exact_query=exact)
    enc.wait()
    q, w = orc.index_q(q8, w_raw, tab[0], False, 64, 128)
    ref = orc.index_scores(q, w, keys_f)
    got = st.dec_scores[:length].cpu().numpy()
    rel_max = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    print("index scores rel_max", rel_max)
    assert rel_max < 1e-5, rel_max
    want = orc.topk_sorted(ref, 2048)
    have = st.topk.cpu().numpy()
    assert np.array_equal(have, orc.topk_sorted(got, 2048))          # the selection itself is exact on its input
    assert np.array_equal(have, want), int((have != want).sum())      # and identical to the oracle's list


@pytest.mark.parametrize("heads,length,k", [(64, 200000, 2048), (32, 30003, 512), (64, 900, 2048)], ids=["benchmark", "ragged", "short"])
def test_index_decode_candidate_list(orc, enc, heads, length, k):
    """A candidate-source pass (block maxima -> top blocks), then the restricted pass that scores only those blocks:
    the reference masks every key outside the candidate blocks to -inf before its top-k (tests/attn_test_util.hpp:163-168)."""
    from macseek_b200 import attn
    sh = attn.Shape(D=576, heads=64, index_heads=heads, topk=k, key_type=attn.KEY_FP8, elem_type=attn.ELEM_BF16)
    tab = np.zeros((1, 32, 2), np.float32); tab[:, :, 0] = 1.0
    st = attn.DecodeState(sh, length, tab)
    q_raw, w_raw, keys = bench_inputs(heads, length, 3, True)
    q8 = orc.e4m3_to_f32(orc.f32_to_e4m3(q_raw))
    k8 = torch.from_numpy(keys).cuda().to(torch.float8_e4m3fn)
    st.ikey[:length] = k8.view(torch.uint8)
    keys_f = k8.float().cpu().numpy()
    q, w = orc.index_q(q8, w_raw, tab[0], False, heads, 128)
    ref = orc.index_scores(q, w, keys_f)
    # source pass with a DIFFERENT query, so that the candidates are not simply the restricted pass's own best blocks
    q_src = orc.e4m3_to_f32(orc.f32_to_e4m3(bench_inputs(heads, 8, 4, True)[0]))
    attn.encode_index_decode(enc, st, dev(q_src), dev(w_raw), 0, length, actq=False, cand_source=True)
    enc.wait()
    qs, ws = orc.index_q(q_src, w_raw, tab[0], False, heads, 128)
    cand = orc.candidate_blocks(orc.index_scores(qs, ws, keys_f))
    got_cand = st.cand_list.cpu().numpy()
    assert np.array_equal(got_cand, cand)
    attn.encode_index_decode_list(enc, st, dev(q8), dev(w_raw), 0, length, actq=False)
    enc.wait()
    masked = np.full(length, -np.inf, dtype=np.float32)
    for b in cand[cand >= 0]:
        masked[b * 8:min(length, b * 8 + 8)] = ref[b * 8:min(length, b * 8 + 8)]
    want = orc.topk_sorted(masked, k)
    have = st.topk.cpu().numpy()
    assert np.array_equal(have, want), int((have != want).sum())
    # the virtual score array: position 8 i + j holds the score of key cand[i] * 8 + j
    nb = min((length + 7) // 8, sh.cand_blocks)
    virt = st.dec_scores[:nb * 8].cpu().numpy()
    for i in (0, nb // 2, nb - 1):
        b = int(cand[i])
        if b >= 0:
            seg = ref[b * 8:min(length, b * 8 + 8)]
            assert np.max(np.abs(virt[8 * i:8 * i + len(seg)] - seg)) <= 1e-5 * np.max(np.abs(ref))


@pytest.mark.parametrize("cfg", [("reference", 512, 1, 700, 512, 100), ("reference-short", 512, 1, 3, 512, 2),
                                 ("benchmark", 576, 30, 200000, 2048, 199999)], ids=lambda c: c[0])
def test_sparse_attention(orc, enc, cfg):
    from macseek_b200 import attn
    name, D, et, cap, k, pos = cfg
    sh = attn.Shape(D=D, topk=k, elem_type=et, index_heads=32)
    rng = np.random.default_rng(11)
    tab = orc.rope_table(max(pos + 1, 8), True)
    st = attn.DecodeState(sh, cap, tab)
    tdt = torch.float16 if et == 1 else torch.bfloat16
    n_cache = min(cap, 4096)
    cache_rows = torch.from_numpy(rng.standard_normal((n_cache, D)).astype(np.float32)).to(tdt)
    win_rows = torch.from_numpy(rng.standard_normal((128, D)).astype(np.float32)).to(tdt)
    n_win = min(pos + 1, 128)
    # scatter the cache rows over the capacity and build a sorted top-k list with -1 padding
    n_sel = min(k - 5, n_cache) if n_cache > 10 else n_cache
    where = np.sort(rng.choice(cap, n_sel, replace=False)).astype(np.int32)
    st.ckv[torch.from_numpy(where).long().cuda()] = cache_rows[:n_sel].cuda()
    st.win[:] = win_rows.cuda()
    tk = np.full(k, -1, np.int32); tk[:n_sel] = where
    st.topk[:] = dev(tk)
    q = (rng.standard_normal((64, D)) * 2).astype(np.float32)
    sinks = rng.standard_normal(64).astype(np.float32)
    out = torch.zeros(64, D, device="cuda")
    attn.encode_sparse(enc, st, dev(q), dev(sinks), out, pos)
    enc.wait()
    rows = np.concatenate([win_rows[:n_win].float().numpy(), cache_rows[:n_sel].float().numpy()])
    ref = orc.sparse_attn(q, tab[pos], rows, sinks)
    got = out.cpu().numpy()
    rel_rms = np.sqrt(np.mean((got - ref) ** 2) / np.mean(ref ** 2))
    rel_max = np.max(np.abs(got - ref)) / np.max(np.abs(ref))
    print(name, "rel_rms", rel_rms, "rel_max", rel_max)
    assert rel_rms < 1e-3 and rel_max < 1e-3, (rel_rms, rel_max)     # reference: rel_rms < 2e-3 (test_attn_200k.mm:63)
    out2 = torch.zeros(64, D, device="cuda")
    attn.encode_sparse(enc, st, dev(q), dev(sinks), out2, pos)
    enc.wait()
    assert torch.equal(out, out2)
