"""Host mirror of the reference's quant module interface (namespace ms::q, src/kernels/quant.hpp): same function
names, argument meaning and preconditions; every call enqueues CUDA work through the C ABI and returns."""
import enum

import torch

from . import _lib
from .core import Enc, ptr
from .shapes import QType  # noqa: F401


def block_elems(t):
    return _lib.lib.msb_block_elems(int(t))


def block_bytes(t):
    return _lib.lib.msb_block_bytes(int(t))


def row_bytes(t, cols):
    return _lib.lib.msb_row_bytes(int(t), cols)


def matvec_supported(t):
    """quant.hpp:17 -- every type of the enum has a matvec here (the reference has none for IQ4_NL)."""
    return int(t) in [int(v) for v in QType]


def encode_dequant(e: Enc, t, W, n, out):
    """out[0..n) fp32 = dequantised raw blocks, bit-identical with the reference's CPU ref::dequant_row."""
    _lib.check(_lib.lib.msb_dequant(int(t), ptr(W), n, ptr(out), e.handle))


def encode_matvec(e: Enc, t, W, rows, cols, x, y, accumulate=False, groups=1):
    """y[rows] (+)= W[rows x cols] . x  (quant.hpp:27-30)."""
    _lib.check(_lib.lib.msb_matvec(int(t), ptr(W), rows, cols, ptr(x), ptr(y), int(accumulate), groups, e.handle))


def encode_matvec_n(e: Enc, t, W, rows, cols, X, Y, n, accumulate=False, groups=1):
    """Y[n x rows] (+)= X[n x cols*groups] . W^T for n in 1..16 (quant.hpp:32-35)."""
    _lib.check(_lib.lib.msb_matvec_n(int(t), ptr(W), rows, cols, ptr(X), ptr(Y), n, int(accumulate), groups, e.handle))


# ---------------------------------------------------------------- MoE decode (quant.hpp:49-85)
kMaxRouted = 16


def matmul_scratch_bytes(t, rows, cols, n, with_x=True):
    return _lib.lib.msb_matmul_scratch_bytes(int(t), rows, cols, n, int(with_x))


def encode_f32_to_f16(e: Enc, X, X16, count):
    """F32 -> half (quant.hpp:43); count % 4 == 0."""
    _lib.check(_lib.lib.msb_f32_to_f16(ptr(X), ptr(X16), count, e.handle))


def encode_matmul_h(e: Enc, t, W, rows, cols, X16, Y, n, accumulate=False, x_stride=0, scratch=None):
    """Prefill: Y[n x rows] (+)= X16[n x cols] . W^T, X16 half with row stride x_stride (quant.hpp:45-46).  scratch:
    matmul_scratch_bytes(t, rows, cols, n, with_x=False) bytes (the reference's module-owned W16)."""
    _lib.check(_lib.lib.msb_matmul_h(int(t), ptr(W), rows, cols, ptr(X16), x_stride, ptr(Y), n, int(accumulate),
                                     ptr(scratch), scratch.numel() * scratch.element_size() if scratch is not None else 0,
                                     e.handle))


def encode_matmul(e: Enc, t, W, rows, cols, X, Y, n, accumulate=False, scratch=None):
    """Prefill: Y[n x rows] (+)= X[n x cols] . W^T with X F32, converted to half internally (quant.hpp:41-42)."""
    _lib.check(_lib.lib.msb_matmul(int(t), ptr(W), rows, cols, ptr(X), ptr(Y), n, int(accumulate), ptr(scratch),
                                   scratch.numel() * scratch.element_size() if scratch is not None else 0, e.handle))


class ExpertSlot:
    """Three raw-block matrices of one expert: gate [inter x dim], up [inter x dim], down [dim x inter]."""

    def __init__(self, gate=None, up=None, down=None):
        self.gate, self.up, self.down = gate, up, down


class MoePart(enum.IntEnum):
    """quant.hpp:83"""
    All = 0
    SharedGu = 1
    AfterSharedGu = 2
    Shared = 3
    Routed = 4
    SharedDown = 5
    GuAll = 6       # not in the reference: the gate/up launch of All alone
    DownAll = 7     # the down launch of All alone


class MoeDecodeArgs:
    """ms::q::MoeDecodeArgs with run-time dim / inter (the reference fixes kExpertDim = 5120, kExpertInter = 2304)."""

    def __init__(self, dim=5120, inter=2304):
        self.dim, self.inter = dim, inter
        self.t_gate_up = QType.IQ1_S
        self.t_down = QType.IQ1_S
        self.n_routed = 6
        self.slot = [ExpertSlot() for _ in range(kMaxRouted)]
        self.weights = None
        self.has_shared = True
        self.t_shared = QType.Q6_K
        self.shared = ExpertSlot()
        self.x = None
        self.y = None
        self.scratch = None
        self.swiglu_limit = 10.0

    def _c(self):
        a = _lib.MoeDecodeArgsC()
        a.dim, a.inter = self.dim, self.inter
        a.t_gate_up, a.t_down, a.t_shared = int(self.t_gate_up), int(self.t_down), int(self.t_shared)
        a.n_routed, a.has_shared = self.n_routed, int(self.has_shared)
        for i in range(min(self.n_routed, kMaxRouted)):
            s = self.slot[i]
            a.slot[i].gate, a.slot[i].up, a.slot[i].down = ptr(s.gate), ptr(s.up), ptr(s.down)
        a.shared.gate, a.shared.up, a.shared.down = ptr(self.shared.gate), ptr(self.shared.up), ptr(self.shared.down)
        a.weights, a.x, a.y = ptr(self.weights), ptr(self.x), ptr(self.y)
        a.scratch = ptr(self.scratch)
        a.scratch_bytes = self.scratch.numel() * self.scratch.element_size() if self.scratch is not None else 0
        a.swiglu_limit = self.swiglu_limit
        return a


def moe_decode_scratch_bytes(inter=2304, max_routed=6):
    return _lib.lib.msb_moe_decode_scratch_bytes(inter, max_routed)


def encode_moe_decode(e: Enc, a: MoeDecodeArgs):
    """Gate+up+SwiGLU for every expert, then down for every expert accumulated into y (quant.hpp:72-74)."""
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode(c, e.handle))


def encode_moe_decode_noalloc(e: Enc, a: MoeDecodeArgs):
    """encode_moe_decode with the library's own static scratch (a.scratch is ignored); no reference counterpart."""
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode_noalloc(c, e.handle))


def encode_moe_decode_table(e: Enc, a: MoeDecodeArgs, table):
    encode_moe_decode_table_part(e, a, table, MoePart.All)


def encode_moe_decode_table_part(e: Enc, a: MoeDecodeArgs, table, part):
    """Routed matrices from `table`: n_routed x 3 device addresses {gate, up, down} (quant.hpp:75-85)."""
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode_table_part(c, ptr(table), int(part), e.handle))


def encode_moe_decode_ids(e: Enc, a: MoeDecodeArgs, expert_table, ids, expert_lo, expert_hi, part=MoePart.All):
    """HBM-resident experts: expert_table [n_experts][3] device addresses, ids = device int32 [n_routed] from the
    router; only experts in [expert_lo, expert_hi) are computed on this GPU."""
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode_ids(c, ptr(expert_table), ptr(ids), expert_lo, expert_hi, int(part), e.handle))


def encode_moe_decode_ids_normed(e: Enc, a: MoeDecodeArgs, expert_table, ids, expert_lo, expert_hi, norm_in, norm_w,
                                 norm_eps, part=MoePart.All):
    """encode_moe_decode_ids on x = RMSNorm(norm_in) * norm_w built inside the gate/up launch (a.x is ignored), which
    then starts on the shared expert while the previous kernel -- the fused-norm router over the same norm_in, by
    contract -- is still selecting.  No reference counterpart."""
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode_ids_normed(c, ptr(expert_table), ptr(ids), expert_lo, expert_hi, int(part),
                                                  ptr(norm_in), ptr(norm_w), norm_eps, e.handle))


def encode_moe_decode_ep(e: Enc, a: MoeDecodeArgs, expert_table, ids, expert_lo, expert_hi, shared_lo, shared_hi,
                         comm=None, norm_in=None, norm_w=None, norm_eps=0.0):
    """Expert-parallel form: the experts in [expert_lo, expert_hi) plus rows [shared_lo, shared_hi) of the shared
    expert.  comm (an ep.EpComm) given: the partial output goes to every rank's exchange buffer for ep.encode_combine;
    comm None: it is accumulated into a.y.  No reference counterpart (model.py:869-904 gives the semantics)."""
    import ctypes as C
    c = a._c()
    _lib.check(_lib.lib.msb_moe_decode_ep(c, ptr(expert_table), ptr(ids), expert_lo, expert_hi, ptr(norm_in), ptr(norm_w),
                                          norm_eps, shared_lo, shared_hi, C.byref(comm.c) if comm is not None else None,
                                          e.handle))


def encode_matvec_rmsnorm(e: Enc, t, W, rows, cols, x, norm_w, eps, y):
    """y = W . (x * rsqrt(mean(x^2) + eps) * norm_w): input RMSNorm fused into the x load (quant.hpp:19-26)."""
    _lib.check(_lib.lib.msb_matvec_rmsnorm(int(t), ptr(W), rows, cols, ptr(x), ptr(norm_w), eps, ptr(y), e.handle))


def encode_matvec_rmsnorm_shared(e: Enc, t, W, rows, cols, x, norm_w, eps, y):
    """encode_matvec_rmsnorm as a launch of one small block per SM, leaving room for another stream's kernels beside
    it (no reference counterpart)."""
    _lib.check(_lib.lib.msb_matvec_rmsnorm_shared(int(t), ptr(W), rows, cols, ptr(x), ptr(norm_w), eps, ptr(y), e.handle))


def moe_prefill_scratch_bytes(total_entries, n_tokens, n_exp, dim=5120, inter=2304):
    return _lib.lib.msb_moe_prefill_scratch_bytes(total_entries, n_tokens, n_exp, dim, inter)


class MoePrefillArgs:
    """ms::q::MoePrefillArgs (quant.hpp:96-116) with dim / inter as fields.  slots: list of ExpertSlot (device tensors),
    offs: host list of n_exp + 1 entry offsets; tok / wt / slot_of / X / Y / scratch: device tensors."""

    def __init__(self, dim=5120, inter=2304):
        self.dim, self.inter = dim, inter
        self.t_gate_up = self.t_down = QType.IQ1_S
        self.t_shared = QType.Q6_K
        self.n_tokens = 0
        self.slots, self.offs = [], [0]
        self.tok = self.wt = self.slot_of = None
        self.k_per_token = 6
        self.has_shared = True
        self.shared = ExpertSlot()
        self.X = self.Y = self.scratch = None
        self.swiglu_limit = 10.0


def encode_moe_prefill(e: Enc, a: MoePrefillArgs):
    """Grouped expert GEMMs of a prefill chunk, Y accumulated (quant.hpp:118)."""
    import ctypes as C
    n_exp = len(a.slots)
    c = _lib.MoePrefillArgsC()
    c.dim, c.inter = a.dim, a.inter
    c.t_gate_up, c.t_down, c.t_shared = int(a.t_gate_up), int(a.t_down), int(a.t_shared)
    c.n_tokens, c.n_exp = a.n_tokens, n_exp
    slots = (_lib.ExpertSlotC * max(n_exp, 1))()
    for j, s in enumerate(a.slots):
        slots[j].gate, slots[j].up, slots[j].down = ptr(s.gate), ptr(s.up), ptr(s.down)
    offs = (C.c_int * (n_exp + 1))(*[int(v) for v in a.offs])
    c.slots, c.offs = slots, offs
    c.tok, c.wt, c.slot_of = ptr(a.tok), ptr(a.wt), ptr(a.slot_of)
    c.k_per_token, c.has_shared = a.k_per_token, int(a.has_shared)
    c.shared.gate, c.shared.up, c.shared.down = ptr(a.shared.gate), ptr(a.shared.up), ptr(a.shared.down)
    c.X, c.Y, c.scratch = ptr(a.X), ptr(a.Y), ptr(a.scratch)
    c.scratch_bytes = a.scratch.numel() * a.scratch.element_size() if a.scratch is not None else 0
    c.swiglu_limit = a.swiglu_limit
    _lib.check(_lib.lib.msb_moe_prefill(C.byref(c), e.handle))
