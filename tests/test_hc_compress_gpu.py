"""GPU parity of the hyper-connection step (+ Sinkhorn), the KV compressor / index key and the candidate-restricted index
decode on F16 keys against the oracle (tests/ref/arch_ref.cpp:22-95, attn_ref.cpp:116-161, 163-202)."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


@pytest.mark.parametrize("D", (5120, 4096, 512))
@pytest.mark.parametrize("form", ("full", "no_sub", "post_only", "no_x"))
def test_hc_step(orc, D, form):
    from macseek_b200 import arch
    from macseek_b200.core import Enc
    rng = np.random.default_rng(D + len(form))
    h_in = rng.standard_normal(4 * D).astype(np.float32) * 2
    x_sub = rng.standard_normal(D).astype(np.float32) if form != "no_sub" else None
    mix_prev = (np.abs(rng.standard_normal(24)) * 0.5 + 0.05).astype(np.float32)
    has_fn = form != "post_only"
    fn = (rng.standard_normal(24 * 4 * D) * 0.02).astype(np.float32) if has_fn else None
    scale = np.array([0.7, 1.3, 0.9], np.float32)
    base = rng.standard_normal(24).astype(np.float32)
    norm_w = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    want_x = form not in ("post_only", "no_x")
    rh, rm, rx = orc.hc_step(h_in, x_sub, mix_prev, fn, scale if has_fn else None, base if has_fn else None,
                             norm_w if want_x else None, D, want_x=want_x)
    e = Enc()
    scratch = arch.hc_scratch(1)
    h = dev(h_in)
    mix_out = torch.zeros(24, device="cuda")
    x_out = torch.zeros(D, device="cuda")
    for _ in range(2):                    # twice: the scratch counters must come back to zero
        h.copy_(dev(h_in))
        arch.encode_hc_step(e, h, h, dev(x_sub) if x_sub is not None else None, dev(mix_prev), dev(fn) if has_fn else None,
                            dev(scale), dev(base), mix_out if has_fn else None, dev(norm_w), x_out if want_x else None, D,
                            scratch)
        e.wait()
    assert np.max(np.abs(h.cpu().numpy() - rh)) <= 2e-6 * np.max(np.abs(rh))
    if has_fn:
        assert np.max(np.abs(mix_out.cpu().numpy() - rm)) <= 2e-5, (mix_out.cpu().numpy(), rm)
    if want_x:
        assert np.max(np.abs(x_out.cpu().numpy() - rx)) <= 1e-5 * np.max(np.abs(rx))


@pytest.mark.parametrize("ratio", (1, 2))
@pytest.mark.parametrize("actq", (False, True))
@pytest.mark.parametrize("shape", ("reference", "benchmark"))
def test_compress_tokens(orc, ratio, actq, shape):
    from macseek_b200 import attn
    from macseek_b200.core import Enc
    sh = attn.Shape.reference() if shape == "reference" else attn.Shape.benchmark()
    D, ID, n = sh.D, 128, 6
    rng = np.random.default_rng(7 * ratio + D)
    ckv_in = (rng.standard_normal((n, D)) * 2).astype(np.float32)
    cg_in = (rng.standard_normal((n, D)) * 3).astype(np.float32)
    cn = (1 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(ID)).astype(np.float32)
    wk = synth.hashed_bf16(ID * D, 9, 0.2)
    rck, rik = orc.compress_tokens(ratio, ckv_in, cg_in if ratio > 1 else None, cn, wk, kn, actq, D=D, ID=ID)
    st = attn.DecodeState(sh, 64, attn.make_rope_table(64, True), "cuda")
    state = torch.zeros(2, ratio, D, device="cuda")
    state[1].fill_(float("-inf"))
    e = Enc()
    wk_d, cn_d, kn_d = dev(wk), dev(cn), dev(kn)
    for p in range(n):
        attn.encode_compress(e, st, dev(ckv_in[p]), dev(cg_in[p]) if ratio > 1 else None, cn_d, wk_d, kn_d, state, ratio, p, actq)
    e.wait()
    rows = n // ratio
    got_c = st.ckv[:rows].float().cpu().numpy()
    if sh.key_type == attn.KEY_F16:
        got_k = st.ikey[:rows].float().cpu().numpy()
    else:
        got_k = st.ikey[:rows].view(torch.float8_e4m3fn).float().cpu().numpy()
    # storage rounding: f16 rows / keys hold the fp4-simulated values exactly; bf16 rows and e4m3 keys round them
    tol_c = 2e-3 if sh.elem_type == attn.ELEM_F16 else 2 ** -8
    tol_k = 2e-3 if sh.key_type == attn.KEY_F16 else 2 ** -3
    if actq and sh.elem_type == attn.ELEM_F16:
        # values are on a coarse fp4 lattice: all but a few boundary cases must agree exactly
        assert np.mean(got_c == rck) >= 0.995
        assert np.mean(got_k == rik) >= 0.995
    else:
        assert np.max(np.abs(got_c - rck)) <= tol_c * np.max(np.abs(rck))
        if not actq:
            assert np.max(np.abs(got_k - rik)) <= tol_k * np.max(np.abs(rik))


def test_index_decode_list_f16_keys(orc):
    # candidate-restricted decode on the reference's key layout: equals the full scan masked to the candidate blocks
    from macseek_b200 import attn
    from macseek_b200.core import Enc
    sh = attn.Shape.reference()
    length, pos = 40000, 39999
    rng = np.random.default_rng(3)
    st = attn.DecodeState(sh, length, attn.make_rope_table(length + 1, True), "cuda")
    keys = orc.sim("fp4_sim_e8m0", rng.standard_normal((length, 128)).astype(np.float32)).reshape(length, 128)
    st.ikey[:length].copy_(dev(keys.astype(np.float16)))
    iq = rng.standard_normal(32 * 128).astype(np.float32)
    iw = rng.standard_normal(32).astype(np.float32)
    nb = (length + 7) // 8
    cand = np.sort(rng.choice(nb, 2048, replace=False)).astype(np.int32)
    cand[-3:] = -1
    st.cand_list.copy_(dev(cand))
    e = Enc()
    attn.encode_index_decode_list(e, st, dev(iq), dev(iw), pos, length, actq=True)
    e.wait()
    got = st.topk.cpu().numpy()
    cs = st.rope[pos].cpu().numpy()
    q, w = orc.index_q(iq.reshape(32, 128), iw, cs, True, 32, 128)
    sc = orc.index_scores(q, w, keys)
    masked = np.full(length, -np.inf, np.float32)
    for b in cand[cand >= 0]:
        masked[b * 8:min(length, b * 8 + 8)] = sc[b * 8:min(length, b * 8 + 8)]
    want = orc.topk_sorted(masked, sh.topk)
    assert np.array_equal(got, want)
