"""Host mirror of the router part of the reference's arch module (namespace ms::arch, src/kernels/arch.hpp:79-97)."""
import torch

from . import _lib
from .core import Enc, ptr

kExperts, kTopK, kRouteScale = 384, 6, 1.5      # the reference's compile-time shape (arch.hpp:13,16)
from .shapes import SCORE_SQRT_SOFTPLUS, SCORE_SIGMOID  # noqa: E402,F401


class Scratch:
    """Device scratch of the fused router (logits + K-slice partials); the reference's arch::Scratch::router_logits."""

    def __init__(self, n_experts=kExperts, device="cuda"):
        self.n_experts = n_experts
        self.buf = torch.zeros(_lib.lib.msb_router_scratch_bytes(n_experts) // 4, dtype=torch.float32, device=device)

    @property
    def router_logits(self):
        return self.buf[:self.n_experts]

    @staticmethod
    def create(n_experts=kExperts, device="cuda"):
        return Scratch(n_experts, device)


def encode_router_fused(e: Enc, x, W, bias, ids, w, s: Scratch, k=kTopK, score_fn=SCORE_SQRT_SOFTPLUS,
                        route_scale=kRouteScale):
    """Fused F32 matvec (W [E][dim]) + score + bias top-k + normalise * route_scale, one launch (arch.hpp:83)."""
    E, dim = W.shape
    _lib.check(_lib.lib.msb_router_fused(ptr(x), ptr(W), ptr(bias), ptr(ids), ptr(w), ptr(s.buf), s.buf.numel() * 4,
                                         E, dim, k, score_fn, route_scale, e.handle))


def encode_router_fused_rmsnorm(e: Enc, h, norm_w, eps, x_out, W, bias, ids, w, s: Scratch, k=kTopK,
                                score_fn=SCORE_SQRT_SOFTPLUS, route_scale=kRouteScale):
    """encode_rmsnorm(h -> x_out) + encode_router_fused(x_out) in one launch; x_out may be None."""
    E, dim = W.shape
    _lib.check(_lib.lib.msb_router_fused_rmsnorm(ptr(h), ptr(norm_w), eps, ptr(x_out), ptr(W), ptr(bias), ptr(ids),
                                                 ptr(w), ptr(s.buf), s.buf.numel() * 4, E, dim, k, score_fn,
                                                 route_scale, e.handle))


def encode_router_topk(e: Enc, logits, bias, ids, w, n, k=kTopK, score_fn=SCORE_SQRT_SOFTPLUS, route_scale=kRouteScale):
    """From precomputed logits [n][E] (arch.hpp:85)."""
    E = logits.shape[-1]
    _lib.check(_lib.lib.msb_router_topk(ptr(logits), ptr(bias), ptr(ids), ptr(w), n, E, k, score_fn, route_scale, e.handle))


class RouteLists:
    """arch.hpp:87-95: counts u32[E], offsets u32[E+1], entry/tok/slot_of u32[k n], w f32[k n]."""

    def __init__(self, max_tokens, k=kTopK, n_experts=kExperts, device="cuda"):
        self.max_tokens, self.k, self.n_experts = max_tokens, k, n_experts
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.zeros(n_experts, **i32)
        self.offsets = torch.zeros(n_experts + 1, **i32)
        self.entry = torch.zeros(max_tokens * k, **i32)
        self.tok = torch.zeros(max_tokens * k, **i32)
        self.w = torch.zeros(max_tokens * k, dtype=torch.float32, device=device)
        self.slot_of = torch.zeros(max_tokens * k, **i32)

    @staticmethod
    def create(max_tokens, k=kTopK, n_experts=kExperts, device="cuda"):
        return RouteLists(max_tokens, k, n_experts, device)


def encode_route_lists(e: Enc, ids, w, n, L: RouteLists):
    if n > L.max_tokens:
        raise _lib.MsbError("route_lists: %d tokens > capacity %d" % (n, L.max_tokens))
    _lib.check(_lib.lib.msb_route_lists(ptr(ids), ptr(w), n, L.k, L.n_experts, ptr(L.counts), ptr(L.offsets),
                                        ptr(L.entry), ptr(L.tok), ptr(L.w), ptr(L.slot_of), e.handle))


def encode_rmsnorm(e: Enc, x, w, y, rows, dim, eps, in_stride=0, out_stride=0):
    """y = x * rsqrt(mean(x^2) + eps) * w (arch.hpp:128-130)."""
    _lib.check(_lib.lib.msb_rmsnorm(ptr(x), ptr(w), ptr(y), rows, dim, eps, in_stride, out_stride, e.handle))


def encode_argmax(e: Enc, logits, rows, V, out_idx, out_val=None):
    """Greedy argmax per row, ties -> lowest index (arch.hpp:107-112, temperature 0)."""
    for r in range(rows):
        _lib.check(_lib.lib.msb_argmax(ptr(logits, r * V * 4), V, ptr(out_idx, r * 4),
                                       ptr(out_val, r * 4) if out_val is not None else None, e.handle))


def encode_add(e: Enc, y, a, n):
    _lib.check(_lib.lib.msb_add(ptr(y), ptr(a), n, e.handle))


def hc_scratch(n_tokens=1, device="cuda"):
    return torch.zeros(_lib.lib.msb_hc_scratch_bytes(n_tokens) // 4 + 1, dtype=torch.int32, device=device)


def encode_hc_step(e: Enc, h_in, h_out, x_sub, mix_prev, fn, scale, base, mix_out, norm_w, x_out, dim, scratch, n=1):
    """One hyper-connection boundary (arch.hpp:44-77): x_sub / fn / x_out may be None."""
    _lib.check(_lib.lib.msb_hc_step(ptr(h_in), ptr(h_out), ptr(x_sub), ptr(mix_prev), ptr(fn), ptr(scale), ptr(base),
                                    ptr(mix_out), ptr(norm_w), ptr(x_out), dim, n, ptr(scratch),
                                    scratch.numel() * scratch.element_size(), e.handle))


# ---------------------------------------------------------------------------------------------- sampling head
SAMPLE_K = 64


def sample_scratch(rows=1, device="cuda"):
    """Zeroed scratch for encode_argmax_rows / encode_sample_topk (one per stream)."""
    return torch.zeros(_lib.lib.msb_sample_scratch_bytes(rows) // 4 + 4, dtype=torch.int32, device=device)


def encode_argmax_rows(e: Enc, logits, rows, V, out_idx, out_val, scratch, temperature=0.0, seed=0):
    """Per-row argmax, ties -> lowest index; temperature > 0: Gumbel-max sampling keyed by seed (arch.hpp:111-115)."""
    _lib.check(_lib.lib.msb_argmax_rows(ptr(logits), rows, V, ptr(out_idx), ptr(out_val), float(temperature),
                                        int(seed) & 0xFFFFFFFFFFFFFFFF, ptr(scratch),
                                        scratch.numel() * scratch.element_size(), e.handle))


def encode_sample_topk(e: Enc, logits, rows, V, k, temperature, out_v, out_i, out_lse, scratch):
    """Top-k (k <= 64) raw logits + ids per row and the full-row logsumexp(logits / temperature) (arch.hpp:116-119).
    out_v f32 [rows][64], out_i int32 [rows][64], out_lse f32 [rows]."""
    _lib.check(_lib.lib.msb_sample_topk(ptr(logits), rows, V, k, float(temperature), ptr(out_v), ptr(out_i), ptr(out_lse),
                                        ptr(scratch), scratch.numel() * scratch.element_size(), e.handle))


def encode_log_softmax(e: Enc, x, out, rows, V):
    """out = x - logsumexp(x) per row; out may be x (arch.hpp:120-121)."""
    _lib.check(_lib.lib.msb_log_softmax(ptr(x), ptr(out), rows, V, e.handle))


def sample_top_p(vals, ids, k, lse, temperature, top_p, u):
    """Host-side temperature + top-p pick from encode_sample_topk's output (arch.hpp:122-126): vals / ids are host
    sequences of at least k entries."""
    import ctypes as C
    v = (C.c_float * k)(*[float(x) for x in vals[:k]])
    i = (C.c_int * k)(*[int(x) for x in ids[:k]])
    return int(_lib.lib.msb_sample_top_p(v, i, k, float(lse), float(temperature), float(top_p), float(u)))
