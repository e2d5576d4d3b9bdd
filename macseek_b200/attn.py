"""Host mirror of the decode side of the reference's attention module (namespace ms::attn, src/kernels/attn.hpp):
indexer scoring + exact top-k (encode_index_decode) and sparse attention (encode_sparse) over caller-visible caches.

The reference fixes the shapes at compile time (attn.hpp:12-14: D 512, 64 heads, window 128, 32 index heads x 128,
top-k 512); here they are fields of Shape so that the benchmark configuration (row width 576, 64 index heads, FP8
index keys, top-k 2048) runs through the same calls."""
import math

import torch

from . import _lib
from .core import Enc, ptr

from .shapes import KEY_F16, KEY_FP8, ELEM_F16, ELEM_BF16  # noqa: E402,F401


class Shape:
    def __init__(self, D=512, heads=64, window=128, index_heads=32, topk=512, key_type=KEY_F16, elem_type=ELEM_F16,
                 cand_blocks=2048, cand_bs=8):
        self.D, self.heads, self.window = D, heads, window
        self.index_heads, self.index_dim, self.topk = index_heads, 128, topk
        self.key_type, self.elem_type = key_type, elem_type
        self.cand_blocks, self.cand_bs = cand_blocks, cand_bs

    @staticmethod
    def reference():
        return Shape()

    @staticmethod
    def benchmark():
        return Shape(D=576, heads=64, window=128, index_heads=64, topk=2048, key_type=KEY_FP8, elem_type=ELEM_BF16)


def make_rope_table(max_pos, yarn):
    """float32 [max_pos][32][2] (cos, sin): theta 1e4 plain, or theta 1.6e5 with YaRN(16, 65536, 32, 1), with the
    float rounding steps of the reference's attn::make_rope_table / attnref::rope_table (tests/ref/attn_ref.cpp:15-46)."""
    import numpy as np
    dim = 64
    base = 160000.0 if yarn else 10000.0
    f = np.array([np.float32(1.0 / math.pow(base, float(np.float32(2 * i)) / dim)) for i in range(32)], dtype=np.float32)
    if yarn:
        factor, orig, bf, bs = 16.0, 65536.0, 32.0, 1.0
        corr = lambda rot: dim * math.log(orig / (rot * 2 * math.pi)) / (2 * math.log(base))
        low = max(math.floor(corr(bf)), 0.0)
        high = min(math.ceil(corr(bs)), dim - 1.0)
        for i in range(32):
            ramp = np.float32((i - low) / max(high - low, 1e-3))
            ramp = min(max(ramp, np.float32(0)), np.float32(1))
            smooth = np.float32(1.0) - ramp
            f[i] = f[i] / np.float32(factor) * (np.float32(1.0) - smooth) + f[i] * smooth
    p = np.arange(max_pos, dtype=np.float32)[:, None]
    a = (p * f[None, :]).astype(np.float32).astype(np.float64)
    out = np.empty((max_pos, 32, 2), dtype=np.float32)
    out[:, :, 0] = np.cos(a)
    out[:, :, 1] = np.sin(a)
    return out


class DecodeState:
    """Caches and scratch of one sequence for one KV source (the decode-side subset of attn::State, attn.hpp:62-101):
    win (window ring), ckv (compressed KV rows, K == V), ikey (index keys), the current top-k list, work buffers."""

    def __init__(self, shape: Shape, cap, rope_table, device="cuda"):
        s = self.shape = shape
        self.cap = cap
        edt = torch.float16 if s.elem_type == ELEM_F16 else torch.bfloat16
        self.win = torch.zeros(s.window, s.D, dtype=edt, device=device)
        self.ckv = torch.zeros(cap + 128, s.D, dtype=edt, device=device)
        if s.key_type == KEY_F16:
            self.ikey = torch.zeros(cap + 128, s.index_dim, dtype=torch.float16, device=device)
        else:
            self.ikey = torch.zeros(cap + 128, s.index_dim, dtype=torch.uint8, device=device)
        self.rope = rope_table if isinstance(rope_table, torch.Tensor) else torch.from_numpy(rope_table).to(device)
        self.topk = torch.full((s.topk,), -1, dtype=torch.int32, device=device)
        self.dec_scores = torch.zeros(cap + 128, dtype=torch.float32, device=device)
        self.dec_bscores = torch.zeros((cap + 128 + s.cand_bs - 1) // s.cand_bs, dtype=torch.float32, device=device)
        self.cand_list = torch.full((s.cand_blocks,), -1, dtype=torch.int32, device=device)
        self.q_prep = torch.zeros(s.index_heads, s.index_dim, dtype=torch.float32, device=device)
        self.w_prep = torch.zeros(s.index_heads, dtype=torch.float32, device=device)
        self.topk_scratch = torch.zeros(_lib.lib.msb_topk_scratch_bytes(cap + 128) // 4 + 1, dtype=torch.int32, device=device)
        self.sparse_scratch = torch.zeros(_lib.lib.msb_sparse_scratch_bytes(s.window + s.topk, s.heads, s.D) // 4 + 1,
                                          dtype=torch.float32, device=device)


def encode_index_decode(e: Enc, s: DecodeState, iq, iw, pos, length, actq=True, exact_query=False, cand_source=False):
    """Index scores of keys [0, length) for the query at position pos, then the exact top-k into s.topk
    (attn.hpp:121-122).  cand_source: also the block maxima -> top candidate blocks into s.cand_list (layer 20 of the
    reference, attn.mm:227,262-263)."""
    sh = s.shape
    cs = s.rope[pos]
    _lib.check(_lib.lib.msb_index_decode(sh.key_type, ptr(s.ikey), length, ptr(iq), ptr(iw), ptr(cs), int(actq),
                                         sh.index_heads, sh.topk, ptr(s.q_prep), ptr(s.w_prep), ptr(s.dec_scores),
                                         ptr(s.topk), ptr(s.topk_scratch), s.topk_scratch.numel() * 4,
                                         int(exact_query), e.handle))
    if cand_source and length > 0:
        nb = (length + sh.cand_bs - 1) // sh.cand_bs
        _lib.check(_lib.lib.msb_block_max(ptr(s.dec_scores), length, sh.cand_bs, ptr(s.dec_bscores), e.handle))
        _lib.check(_lib.lib.msb_topk(ptr(s.dec_bscores), nb, sh.cand_blocks, ptr(s.cand_list), ptr(s.topk_scratch),
                                     s.topk_scratch.numel() * 4, 0, e.handle))


def encode_index_decode_list(e: Enc, s: DecodeState, iq, iw, pos, length, actq=True):
    """encode_index_decode of a layer that uses candidates (attn.mm:226-229): only the keys of the blocks in s.cand_list
    are scored (F16 or FP8 keys)."""
    sh = s.shape
    cs = s.rope[pos]
    nb = (length + sh.cand_bs - 1) // sh.cand_bs
    _lib.check(_lib.lib.msb_index_decode_list(sh.key_type, ptr(s.ikey), length, ptr(iq), ptr(iw), ptr(cs), int(actq),
                                              sh.index_heads, sh.topk, ptr(s.cand_list), min(nb, sh.cand_blocks),
                                              ptr(s.q_prep), ptr(s.w_prep), ptr(s.dec_scores), ptr(s.topk),
                                              ptr(s.topk_scratch), s.topk_scratch.numel() * 4, e.handle))


def encode_topk(e: Enc, scores, n, k, out, scratch):
    _lib.check(_lib.lib.msb_topk(ptr(scores), n, k, ptr(out), ptr(scratch), scratch.numel() * scratch.element_size(), 0,
                                 e.handle))


def encode_sparse(e: Enc, s: DecodeState, q, sinks, out, pos, n_win=None):
    """Sparse attention of one query over the window rows and the rows listed in s.topk (attn.hpp:128-129)."""
    sh = s.shape
    if n_win is None:
        n_win = min(pos + 1, sh.window)
    _lib.check(_lib.lib.msb_sparse_decode(ptr(q), ptr(s.rope[pos]), ptr(sinks), sh.elem_type, ptr(s.win), n_win,
                                          ptr(s.ckv), ptr(s.topk), sh.topk, sh.heads, sh.D, ptr(out),
                                          ptr(s.sparse_scratch), s.sparse_scratch.numel() * 4, e.handle))


def encode_kv_window(e: Enc, s: DecodeState, kv, norm_w, pos, actq=False):
    """Window KV row of the token at pos into the ring slot pos % window (attn.hpp:113, n == 1)."""
    sh = s.shape
    slot = pos % sh.window
    _lib.check(_lib.lib.msb_kv_window(ptr(kv), ptr(norm_w), ptr(s.rope[pos]), int(actq), sh.D, sh.elem_type,
                                      ptr(s.win[slot]), e.handle))


def encode_compress(e: Enc, s: DecodeState, c_kv, c_gate, c_norm, wk_bf16, k_norm, state, ratio, pos, actq=True):
    """Compressor + index key of the token at pos for this KV source (attn.hpp:118, n == 1): updates `state`
    (f32 [2][ratio][D]) and, when pos completes a group, writes row pos // ratio of s.ckv and s.ikey."""
    sh = s.shape
    cs = s.rope[(pos // ratio) * ratio]
    _lib.check(_lib.lib.msb_compress(ptr(c_kv), ptr(c_gate), ptr(c_norm), ptr(wk_bf16), ptr(k_norm), ptr(cs), ptr(state),
                                     ratio, pos, int(actq), sh.D, sh.index_dim, sh.elem_type, ptr(s.ckv), sh.key_type,
                                     ptr(s.ikey), e.handle))
