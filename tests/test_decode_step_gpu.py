"""The decode layer-forward call sequence on a small synthetic model: every stage of layer 0 is checked against the
oracle on the device's own inputs to that stage (so one stage's rounding cannot hide or amplify another's), the whole
step is repeatable bit for bit, and a CUDA-graph replay equals the eager run."""
import numpy as np
import pytest
import torch

import oracle_lib as ol

pytestmark = pytest.mark.gpu


def small_cfg():
    from macseek_b200.dec_layer import DecConfig
    return DecConfig(dim=512, n_layers=2, heads=64, D=576, q_lora=256, o_groups=8, o_a_rows=1024, index_heads=64,
                     topk=512, kv_len=3000, n_experts=16, top_k=4, inter=256, vocab=2048)


def host(t):
    return t.detach().cpu().numpy()


def raw(t):
    return t.detach().cpu().numpy().view(np.uint8).reshape(-1)


def test_layer_stages_against_oracle():
    from macseek_b200.core import Enc
    from macseek_b200.dec_layer import SyntheticModel
    orc = ol.Oracle()
    cfg = small_cfg()
    m = SyntheticModel(cfg, seed=7)
    b, w, st = m.bufs, m.layers[0], m.state[0]
    e = Enc()
    pos = cfg.kv_len - 1
    h0 = torch.randn(cfg.dim, device="cuda")
    b.h.copy_(h0)
    m.encode_dec_attn_side(e, 0, pos)
    e.wait()
    T = 2e-5

    def mv(t, W, rows, cols, x, groups=1):
        return orc.matvec(int(t), raw(W), rows, cols, x, groups)

    x = orc.rmsnorm(host(h0), host(w.attn_norm), cfg.norm_eps)       # the norm itself is fused into the matvecs
    for got, (ry, mag) in ((b.qa, mv(cfg.t_attn, w.wq_a, cfg.q_lora, cfg.dim, x)), (b.kv, mv(cfg.t_attn, w.wkv, cfg.D, cfg.dim, x)),
                           (b.iw, mv(cfg.t_index, w.w_idx_proj, cfg.index_heads, cfg.dim, x))):
        assert orc.max_norm_err(host(got), ry, mag) <= T
    qan = orc.rmsnorm(host(b.qa), host(w.q_norm), cfg.norm_eps)
    ry, mag = mv(cfg.t_attn, w.wq_b, cfg.heads * cfg.D, cfg.q_lora, qan)
    assert orc.max_norm_err(host(b.qfull), ry, mag) <= T
    ry, mag = mv(cfg.t_index, w.w_idx_qb, cfg.index_heads * 128, cfg.q_lora, qan)
    assert orc.max_norm_err(host(b.iq), ry, mag) <= T
    # window row of this token (bf16 storage of the oracle's fp32 row)
    cs = host(m.rope[pos])
    want = torch.from_numpy(orc.window_row(host(b.kv), host(w.kv_norm), cs, False)).to(torch.bfloat16).float().numpy()
    got = st.win[pos % cfg.window].float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= 2 ** -7 * np.max(np.abs(want))
    # indexer: prepared query bit-exact; scores of the e4m3-rounded query against the FP8 keys; top-k on those scores
    q, wq = orc.index_q(host(b.iq).reshape(cfg.index_heads, 128), host(b.iw), cs, False, cfg.index_heads, 128)
    assert np.array_equal(host(st.q_prep).view(np.uint32), q.view(np.uint32))
    q8 = orc.e4m3_to_f32(orc.f32_to_e4m3(q))
    keys = st.ikey[:cfg.kv_len].view(torch.float8_e4m3fn).float().cpu().numpy()
    ref_sc = orc.index_scores(q8, wq, keys)
    dev_sc = host(st.dec_scores[:cfg.kv_len])
    assert np.max(np.abs(dev_sc - ref_sc)) <= 1e-5 * np.max(np.abs(ref_sc))
    topk = host(st.topk)
    assert np.array_equal(topk, orc.topk_sorted(dev_sc, cfg.topk))
    # sparse attention over window + selected rows
    n_win = min(pos + 1, cfg.window)
    rows = np.concatenate([st.win[:n_win].float().cpu().numpy(), st.ckv[torch.from_numpy(topk[topk >= 0]).long().cuda()].float().cpu().numpy()])
    ref = orc.sparse_attn(host(b.qfull).reshape(cfg.heads, cfg.D), cs, rows, host(w.sinks))
    got = host(b.attn_out).reshape(cfg.heads, cfg.D)
    assert np.sqrt(np.mean((got - ref) ** 2) / np.mean(ref ** 2)) < 1e-3
    # output projections; h = h0 + o_b(o_a(attn_out))
    ao = host(b.attn_out)
    ry, mag = mv(cfg.t_attn, w.wo_a, cfg.o_a_rows, cfg.heads * cfg.D // cfg.o_groups, ao, cfg.o_groups)
    assert orc.max_norm_err(host(b.oa), ry, mag) <= T
    ry, mag = mv(cfg.t_attn, w.wo_b, cfg.dim, cfg.o_a_rows, host(b.oa))
    h1 = host(b.h)
    assert orc.max_norm_err(h1, ry + host(h0), mag + np.abs(host(h0))) <= T
    # MoE side
    m.encode_dec_moe(e, 0)
    e.wait()
    xf = host(b.x)
    assert np.allclose(xf, orc.rmsnorm(h1, host(w.ffn_norm), cfg.norm_eps), rtol=1e-5, atol=1e-6)
    ids = host(b.moe.ids)
    logits = host(b.moe.router_scratch.router_logits)
    rid, rw = orc.router(logits, host(w.moe.router_bias), cfg.top_k, cfg.score_fn, cfg.route_scale)
    assert np.array_equal(ids, rid) and np.allclose(host(b.moe.w), rw, rtol=1e-5)
    G, U, Dn = [], [], []
    for eid in ids:
        g_, u_, d_ = w.moe.expert_views(int(eid))
        G.append(raw(g_)); U.append(raw(u_)); Dn.append(raw(d_))
    G.append(raw(w.moe.shared.gate)); U.append(raw(w.moe.shared.up)); Dn.append(raw(w.moe.shared.down))
    hh, y, ymag, hmag = orc.moe_decode(cfg.dim, cfg.inter, int(cfg.t_gate_up), int(cfg.t_down), int(cfg.t_shared), G, U, Dn,
                                       host(b.moe.w), xf, h1)
    assert orc.max_norm_err(host(b.h), y, ymag) <= 5e-5


def test_step_repeatable_and_graph_equals_eager():
    from macseek_b200.core import Enc
    from macseek_b200.dec_layer import SyntheticModel
    cfg = small_cfg()
    m = SyntheticModel(cfg, seed=3)
    b = m.bufs
    h0 = torch.randn(cfg.dim, device="cuda")
    outs = []
    for _ in range(2):
        e = Enc()
        b.h.copy_(h0)
        n = m.forward_token(e)
        e.wait()
        outs.append((b.logits.clone(), int(b.next_id.item())))
    assert n > 0 and torch.equal(outs[0][0], outs[1][0]) and outs[0][1] == outs[1][1]
    assert outs[0][1] == ol.Oracle().argmax(outs[0][0].cpu().numpy())
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            b.h.copy_(h0)
            m.forward_token(Enc(torch.cuda.current_stream()))
        g.replay()
        s.synchronize()
    assert torch.equal(b.logits, outs[0][0])


@pytest.mark.parametrize("world,inter", [(2, 256), (2, 512), (4, 1024)])
def test_expert_parallel_step_equals_single_gpu(world, inter):
    """The whole step under expert parallelism, the ranks' models built side by side on one GPU and encoded layer by
    layer in rank order (so that every partial is stored before a combine is launched): every rank ends with the same
    bits, and with the single-GPU model's token and logits within the MoE tolerance."""
    from macseek_b200 import ep
    from macseek_b200.core import Enc
    from macseek_b200.dec_layer import SyntheticModel
    cfg = small_cfg()
    cfg.inter = inter
    cfg.n_experts = 16
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + world + inter)
    h0 = torch.randn(cfg.dim, device="cuda", generator=gen)
    ref = SyntheticModel(cfg, seed=11)
    e = Enc()
    ref.bufs.h.copy_(h0)
    ref.forward_token(e)
    e.wait()
    comms = ep.EpComm.local(cfg.dim, world)
    try:
        ranks = [SyntheticModel(cfg, seed=11, ep_rank=r, ep_world=world, combine="peer", comm=comms[r]) for r in range(world)]
        # rank r holds exactly the single-GPU model's bytes for its experts
        lo, hi = ranks[1].ep_lo, ranks[1].ep_hi
        g_ref = ref.layers[0].moe.expert_views(lo)[0]
        assert torch.equal(ranks[1].layers[0].moe.expert_views(lo)[0], g_ref)
        pos = cfg.kv_len - 1
        for m in ranks:
            m.bufs.h.copy_(h0)
        for l in range(cfg.n_layers):
            for m in ranks:
                m.encode_dec_attn_side(e, l, pos)
                m.encode_dec_moe_partial(e, l)
            for m in ranks:
                m.encode_dec_moe_combine(e, l)
        for m in ranks:
            m.encode_head(e)
        e.wait()
        for m in ranks[1:]:
            assert torch.equal(m.bufs.logits, ranks[0].bufs.logits)
        a, b = ranks[0].bufs.logits.cpu().numpy(), ref.bufs.logits.cpu().numpy()
        assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(b)), (float(np.max(np.abs(a - b))), float(np.max(np.abs(b))))
        assert int(ranks[0].bufs.next_id.item()) == int(ref.bufs.next_id.item())
    finally:
        for c in comms:
            c.close()
