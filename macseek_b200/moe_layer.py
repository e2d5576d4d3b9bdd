"""One MoE layer with HBM-resident experts: what replaces the reference's expert slot-arena cache and its per-layer
CPU<->GPU handshake (src/store/experts.hpp, src/model/ds41.mm:596-611, dec_layer.mm:257-313).  All experts of the
layer's local range live in one device arena; a device table maps expert id -> {gate, up, down} addresses, the router
writes the ids on the device and the MoE kernels resolve them there, so a whole token needs no host round trip."""
import torch

from . import arch, quant as q
from . import synthetic
from .core import Enc


class MoeLayerWeights:
    def __init__(self, dim, inter, n_experts, t_gate_up, t_down, t_shared, expert_lo=0, expert_hi=None, device="cuda"):
        self.dim, self.inter, self.n_experts = dim, inter, n_experts
        self.t_gate_up, self.t_down, self.t_shared = q.QType(t_gate_up), q.QType(t_down), q.QType(t_shared)
        self.expert_lo = expert_lo
        self.expert_hi = n_experts if expert_hi is None else expert_hi
        self.device = device
        self.gu_bytes = synthetic.row_bytes(self.t_gate_up, dim) * inter
        self.d_bytes = synthetic.row_bytes(self.t_down, inter) * dim
        self.expert_bytes = 2 * self.gu_bytes + self.d_bytes
        self.router_w = None      # f32 [E][dim]
        self.router_bias = None   # f32 [E]
        self.arena = None         # uint8 [(hi - lo) * expert_bytes]
        self.table = None         # int64 [E][3] device addresses (0 for experts not resident here)
        self.shared = q.ExpertSlot()

    def randomize(self, gen, router_gen=None, expert_seed=None):
        """Fill with seeded synthetic weights.  The router and the shared expert (replicated on every rank) draw from
        router_gen.  With expert_seed every expert draws from its own stream, seeded by its GLOBAL id, so that a rank
        holding experts [lo, hi) holds exactly the bytes the single-GPU model has for them; without it the whole local
        arena comes from gen in one pass (faster, for single-GPU benches)."""
        rg = router_gen if router_gen is not None else gen
        dev = self.device
        E, dim, inter = self.n_experts, self.dim, self.inter
        self.router_w = torch.empty(E, dim, dtype=torch.float32, device=dev).normal_(0, 0.02, generator=rg)
        self.router_bias = torch.zeros(E, dtype=torch.float32, device=dev)
        sg = synthetic.row_bytes(self.t_shared, dim) * inter
        sd = synthetic.row_bytes(self.t_shared, inter) * dim
        self.shared_arena = torch.empty(2 * sg + sd, dtype=torch.uint8, device=dev)
        synthetic.random_weights(self.t_shared, 2 * inter, dim, rg, out=self.shared_arena[:2 * sg])
        synthetic.random_weights(self.t_shared, dim, inter, rg, out=self.shared_arena[2 * sg:])
        self.shared = q.ExpertSlot(self.shared_arena[:sg], self.shared_arena[sg:2 * sg], self.shared_arena[2 * sg:])
        n_local = self.expert_hi - self.expert_lo
        self.arena = torch.empty(n_local * self.expert_bytes, dtype=torch.uint8, device=dev)
        # gate|up of every local expert first, then the down matrices: two uniform regions, filled in place
        gu_all = self.arena[:n_local * 2 * self.gu_bytes]
        d_all = self.arena[n_local * 2 * self.gu_bytes:]
        if expert_seed is None:
            synthetic.random_weights(self.t_gate_up, n_local * 2 * inter, dim, gen, out=gu_all)
            synthetic.random_weights(self.t_down, n_local * dim, inter, gen, out=d_all)
        else:
            eg = torch.Generator(device=dev)
            for i in range(n_local):
                eg.manual_seed(int(expert_seed) * 4096 + self.expert_lo + i)
                synthetic.random_weights(self.t_gate_up, 2 * inter, dim, eg,
                                         out=gu_all[i * 2 * self.gu_bytes:(i + 1) * 2 * self.gu_bytes])
                synthetic.random_weights(self.t_down, dim, inter, eg, out=d_all[i * self.d_bytes:(i + 1) * self.d_bytes])
        self.build_table()
        return self

    def build_table(self):
        n_local = self.expert_hi - self.expert_lo
        base = self.arena.data_ptr()
        d_base = base + n_local * 2 * self.gu_bytes
        t = torch.zeros(self.n_experts, 3, dtype=torch.int64)
        for i in range(n_local):
            e = self.expert_lo + i
            t[e, 0] = base + (2 * i) * self.gu_bytes
            t[e, 1] = base + (2 * i + 1) * self.gu_bytes
            t[e, 2] = d_base + i * self.d_bytes
        self.table = t.to(self.device)

    def expert_views(self, e):
        """(gate, up, down) uint8 views of a resident expert."""
        i = e - self.expert_lo
        n_local = self.expert_hi - self.expert_lo
        g0 = (2 * i) * self.gu_bytes
        d0 = n_local * 2 * self.gu_bytes + i * self.d_bytes
        return (self.arena[g0:g0 + self.gu_bytes], self.arena[g0 + self.gu_bytes:g0 + 2 * self.gu_bytes],
                self.arena[d0:d0 + self.d_bytes])

    def algorithmic_bytes(self, k, local_fraction=1.0):
        """Bytes one token must read from this layer: k routed experts, the shared expert and the router."""
        shared = self.shared_arena.numel()
        return int(k * self.expert_bytes * local_fraction) + shared + self.router_w.numel() * 4


class MoeLayerBufs:
    """Per-stream activations / scratch of the MoE side (the reference's DecBufs rows for the FFN, dec_layer.hpp)."""

    def __init__(self, dim, inter, n_experts, k, device="cuda"):
        self.k = k
        self.ids = torch.zeros(k, dtype=torch.int32, device=device)
        self.w = torch.zeros(k, dtype=torch.float32, device=device)
        self.router_scratch = arch.Scratch.create(n_experts, device)
        self.moe_scratch = torch.zeros(q.moe_decode_scratch_bytes(inter, k) // 4, dtype=torch.float32, device=device)


def encode_moe_layer(e: Enc, lw: MoeLayerWeights, b: MoeLayerBufs, x, y, score_fn, route_scale, add_shared=True,
                     norm_in=None, norm_w=None, norm_eps=0.0):
    """y += MoE(x): fused router, then the two MoE kernels on the experts resident here (ids resolved on the GPU).
    With norm_in, x is first produced as RMSNorm(norm_in) * norm_w inside the router launch."""
    if norm_in is not None:
        arch.encode_router_fused_rmsnorm(e, norm_in, norm_w, norm_eps, x, lw.router_w, lw.router_bias, b.ids, b.w,
                                         b.router_scratch, b.k, score_fn, route_scale)
    else:
        arch.encode_router_fused(e, x, lw.router_w, lw.router_bias, b.ids, b.w, b.router_scratch, b.k, score_fn,
                                 route_scale)
    a = q.MoeDecodeArgs(lw.dim, lw.inter)
    a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
    a.n_routed, a.has_shared = b.k, add_shared
    a.shared = lw.shared
    a.weights, a.x, a.y, a.scratch = b.w, x, y, b.moe_scratch
    if norm_in is not None:
        # the router above is the launch directly before: the gate/up kernel may build x from norm_in on its own
        q.encode_moe_decode_ids_normed(e, a, lw.table, b.ids, lw.expert_lo, lw.expert_hi, norm_in, norm_w, norm_eps)
    else:
        q.encode_moe_decode_ids(e, a, lw.table, b.ids, lw.expert_lo, lw.expert_hi)
