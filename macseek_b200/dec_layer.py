"""Decode layer-forward call surface on synthetic weights: the order of hot-path calls that the reference's
ds41::encode_dec_attn_side / encode_dec_moe_table / encode_head issue per token (src/model/dec_layer.hpp:107-118,
dec_layer.mm:138-313, ds41.mm:491-503), re-expressed over CUDA streams and HBM-resident expert-parallel experts.

Per layer:  q_a, kv, index-proj matvecs (input RMSNorm fused) -> q_b, index-q_b matvecs (q RMSNorm fused) -> window KV row ->
            indexer scores + exact top-k -> sparse attention -> o_a (block-diagonal) -> o_b (accumulated into h) ->
            rmsnorm -> fused router -> MoE gate/up + down on the experts resident here (-> all-reduce under EP).
What the reference does between these calls and is not on the measured path here (hyper-connection mixing, the
compressor that produces new cache rows, engram) is left out; plain residual adds stand in for the hyper-connections.
"""
import numpy as np
import torch

from . import arch, attn, ep, moe_layer as ml, quant as q, synthetic
from .core import Enc
from .shapes import DecConfig  # noqa: F401  (re-exported)


def attn_shape(c: DecConfig):
    return attn.Shape(D=c.D, heads=c.heads, window=c.window, index_heads=c.index_heads, topk=c.topk,
                      key_type=c.key_type, elem_type=c.elem_type)


class LayerW:
    """Weights of one layer (the reference's ds41::LayerW, dec_layer.hpp:18-50), all device tensors."""

    def __init__(self, cfg: DecConfig, gen, ep_lo, ep_hi, expert_seed):
        dev = gen.device
        c = cfg
        rw = lambda t, rows, cols: synthetic.random_weights(t, rows, cols, gen)
        ones = lambda n: torch.ones(n, dtype=torch.float32, device=dev)
        self.attn_norm, self.q_norm, self.kv_norm, self.ffn_norm = ones(c.dim), ones(c.q_lora), ones(c.D), ones(c.dim)
        # q_a and kv read the same normalised hidden state: their rows are stored back to back and run as one matvec
        self.wq_a_kv = torch.cat([rw(c.t_attn, c.q_lora, c.dim), rw(c.t_attn, c.D, c.dim)])
        nb = synthetic.row_bytes(c.t_attn, c.dim) * c.q_lora
        self.wq_a, self.wkv = self.wq_a_kv[:nb], self.wq_a_kv[nb:]
        self.wq_b = rw(c.t_attn, c.heads * c.D, c.q_lora)
        self.w_idx_proj = rw(c.t_index, c.index_heads, c.dim)
        self.w_idx_qb = rw(c.t_index, c.index_heads * c.index_dim, c.q_lora)
        self.wo_a = rw(c.t_attn, c.o_a_rows, c.heads * c.D // c.o_groups)
        self.wo_b = rw(c.t_attn, c.dim, c.o_a_rows)
        self.sinks = torch.zeros(c.heads, dtype=torch.float32, device=dev).normal_(0, 1, generator=gen)
        self.moe = ml.MoeLayerWeights(c.dim, c.inter, c.n_experts, c.t_gate_up, c.t_down, c.t_shared, ep_lo, ep_hi, dev)
        self.moe.randomize(gen, router_gen=gen, expert_seed=expert_seed)


class DecBufs:
    """Activations of one token (the reference's ds41::DecBufs); everything F32 (SPEC.md:155)."""

    def __init__(self, cfg: DecConfig, device):
        f = lambda n: torch.zeros(n, dtype=torch.float32, device=device)
        c = cfg
        self.h, self.x = f(c.dim), f(c.dim)
        self.qa_kv = f(c.q_lora + c.D)                      # one output buffer of the fused q_a / kv matvec
        self.qa, self.kv, self.qan = self.qa_kv[:c.q_lora], self.qa_kv[c.q_lora:], f(c.q_lora)
        self.qfull, self.attn_out = f(c.heads * c.D), f(c.heads * c.D)
        self.iq, self.iw = f(c.index_heads * c.index_dim), f(c.index_heads)
        self.oa = f(c.o_a_rows)
        self.y_part = f(c.dim)
        self.logits = f(c.vocab)
        self.next_id = torch.zeros(1, dtype=torch.int32, device=device)
        self.moe = ml.MoeLayerBufs(c.dim, c.inter, c.n_experts, c.top_k, device)


class SyntheticModel:
    """All layers resident in HBM: attention/dense weights replicated, experts [ep_rank * E / ep_world, ...) local."""

    def __init__(self, cfg: DecConfig, seed=1234, device="cuda", ep_rank=0, ep_world=1, group=None, combine="peer",
                 comm=None):
        """combine: how the ranks' partial MoE outputs meet when ep_world > 1 -- "peer" (the down kernel stores into
        every rank's exchange buffer over NVLink, ep.EpComm) or "nccl" (one all-reduce per layer).  comm: an existing
        ep.EpComm (tests that run the ranks one after the other on one GPU); otherwise one is built over `group`."""
        self.cfg, self.device, self.ep_rank, self.ep_world, self.group = cfg, device, ep_rank, ep_world, group
        c = cfg
        self.ep_lo, self.ep_hi = ep.expert_range(c.n_experts, ep_world, ep_rank)
        self.s_lo, self.s_hi = ep.shared_range(c.inter, ep_world, ep_rank)
        self.combine = combine if ep_world > 1 else "none"
        self.comm = comm
        if self.combine == "peer" and self.comm is None:
            self.comm = ep.EpComm(c.dim, group)
        gen = torch.Generator(device=device)
        gen.manual_seed(seed)                      # replicated tensors: the same stream on every rank
        rope = attn.make_rope_table(c.kv_len + 1, True)
        self.rope = torch.from_numpy(rope).to(device)
        self.layers, self.state = [], []
        sh = attn_shape(c)
        for l in range(c.n_layers):
            # experts are seeded by (model seed, layer, global expert id): every world size holds the same model
            self.layers.append(LayerW(c, gen, self.ep_lo, self.ep_hi, seed * 64 + l))
            st = attn.DecodeState(sh, c.kv_len, self.rope, device)
            # synthetic caches ~ N(0,1), as the reference fills them for its 200K benches (bench/attn200k.mm:60-66)
            st.ckv.normal_(0, 1, generator=gen)
            st.win.normal_(0, 1, generator=gen)
            if c.key_type == attn.KEY_FP8:
                tmp = torch.empty(st.ikey.shape, dtype=torch.bfloat16, device=device).normal_(0, 1, generator=gen)
                st.ikey.copy_(tmp.to(torch.float8_e4m3fn).view(torch.uint8))
                del tmp
            else:
                st.ikey.normal_(0, 1, generator=gen)
            self.state.append(st)
        self.out_norm = torch.ones(c.dim, dtype=torch.float32, device=device)
        self.w_head = synthetic.random_weights(c.t_head, c.vocab, c.dim, gen)
        self.bufs = DecBufs(c, device)
        self.side_stream = torch.cuda.Stream(device=device)
        self.launches_per_token = 0
        self.ids_log = None      # optional int32 [n_layers][top_k]: every layer's router ids are copied there

    # ------------------------------------------------------------------ one layer
    def encode_dec_attn_side(self, e: Enc, l, pos):
        c, w, b, st = self.cfg, self.layers[l], self.bufs, self.state[l]
        n = 0
        # the input RMSNorms are fused into the activation load of the matvecs that consume them
        q.encode_matvec_rmsnorm(e, c.t_attn, w.wq_a_kv, c.q_lora + c.D, c.dim, b.h, w.attn_norm, c.norm_eps, b.qa_kv); n += 1
        q.encode_matvec_rmsnorm(e, c.t_index, w.w_idx_proj, c.index_heads, c.dim, b.h, w.attn_norm, c.norm_eps, b.iw); n += 1
        q.encode_matvec_rmsnorm(e, c.t_index, w.w_idx_qb, c.index_heads * c.index_dim, c.q_lora, b.qa, w.q_norm,
                                c.norm_eps, b.iq); n += 1
        # The query projection (bandwidth) and the index decode (a latency chain) depend on nothing of each other:
        # q_b runs on a second stream as one small block per SM, under the index decode, and joins before the
        # attention that needs both.
        side = self.side_stream
        side.wait_stream(e.stream)
        q.encode_matvec_rmsnorm_shared(Enc(side), c.t_attn, w.wq_b, c.heads * c.D, c.q_lora, b.qa, w.q_norm, c.norm_eps,
                                       b.qfull); n += 1
        attn.encode_kv_window(e, st, b.kv, w.kv_norm, pos); n += 1
        attn.encode_index_decode(e, st, b.iq, b.iw, pos, c.kv_len, actq=False); n += 2   # tcgen05 scoring (+ prep), selection
        e.stream.wait_stream(side)
        attn.encode_sparse(e, st, b.qfull, w.sinks, b.attn_out, pos); n += 2
        q.encode_matvec(e, c.t_attn, w.wo_a, c.o_a_rows, c.heads * c.D // c.o_groups, b.attn_out, b.oa, False,
                        c.o_groups); n += 1
        q.encode_matvec(e, c.t_attn, w.wo_b, c.dim, c.o_a_rows, b.oa, b.h, True); n += 1     # h += o_b(...)
        return n

    def encode_dec_moe(self, e: Enc, l):
        n = self.encode_dec_moe_partial(e, l)
        return n + self.encode_dec_moe_combine(e, l)

    def encode_dec_moe_partial(self, e: Enc, l):
        """Router + the two MoE kernels on what is resident here.  Single GPU: the result is accumulated into h and
        nothing is left for encode_dec_moe_combine."""
        c, w, b = self.cfg, self.layers[l], self.bufs
        n = 0
        # the FFN RMSNorm (h -> x) runs inside the router launch
        if self.ep_world == 1:
            ml.encode_moe_layer(e, w.moe, b.moe, b.x, b.h, c.score_fn, c.route_scale, norm_in=b.h, norm_w=w.ffn_norm,
                                norm_eps=c.norm_eps); n += 3
            if self.ids_log is not None:
                self.ids_log[l].copy_(b.moe.ids)
            return n
        # expert parallel: the router is replicated (every rank sees the same ids); each rank runs ONE gate/up + down
        # launch pair over the routed experts resident here and its slice of the shared expert
        a = q.MoeDecodeArgs(c.dim, c.inter)
        a.t_gate_up, a.t_down, a.t_shared = c.t_gate_up, c.t_down, c.t_shared
        a.n_routed, a.has_shared, a.shared = c.top_k, True, w.moe.shared
        a.weights, a.x, a.scratch = b.moe.w, b.x, b.moe.moe_scratch
        a.y = b.y_part
        if self.combine == "nccl":
            b.y_part.zero_()     # before the router, which must be the launch directly ahead of the MoE pair
        arch.encode_router_fused_rmsnorm(e, b.h, w.ffn_norm, c.norm_eps, b.x, w.moe.router_w, w.moe.router_bias,
                                         b.moe.ids, b.moe.w, b.moe.router_scratch, c.top_k, c.score_fn,
                                         c.route_scale); n += 1
        # "peer": the down launch stores its partial into every rank's exchange buffer; "nccl": into y_part
        q.encode_moe_decode_ep(e, a, w.moe.table, b.moe.ids, w.moe.expert_lo, w.moe.expert_hi, self.s_lo, self.s_hi,
                               self.comm if self.combine == "peer" else None, b.h, w.ffn_norm, c.norm_eps); n += 2
        if self.ids_log is not None:
            self.ids_log[l].copy_(b.moe.ids)
        return n

    def encode_dec_moe_combine(self, e: Enc, l):
        """h += the sum of the ranks' partial MoE outputs."""
        c, b = self.cfg, self.bufs
        if self.ep_world == 1:
            return 0
        if self.combine == "peer":
            ep.encode_combine(e, self.comm, b.h)
            return 1
        ep.combine_routed(b.y_part, self.group)
        arch.encode_add(e, b.h, b.y_part, c.dim)
        return 2

    def encode_head(self, e: Enc):
        c, b = self.cfg, self.bufs
        q.encode_matvec_rmsnorm(e, c.t_head, self.w_head, c.vocab, c.dim, b.h, self.out_norm, c.norm_eps, b.logits)
        arch.encode_argmax(e, b.logits, 1, c.vocab, b.next_id)
        return 2

    def forward_token(self, e: Enc, pos=None):
        """Encode the whole step for the token whose hidden state is in bufs.h; returns the kernel launch count."""
        pos = self.cfg.kv_len - 1 if pos is None else pos
        n = 0
        for l in range(self.cfg.n_layers):
            n += self.encode_dec_attn_side(e, l, pos)
            n += self.encode_dec_moe(e, l)
        n += self.encode_head(e)
        self.launches_per_token = n
        return n
