"""Seeded synthetic inputs in the shapes and value distributions of the benchmark configurations: uniform random
codes per format, fp16 block scales ~ U(0.01, 0.05), N(0,1) activations."""
import numpy as np

import oracle_lib as ol


def random_weights(t, rows, cols, seed, lo=0.01, hi=0.05):
    """Raw GGUF rows [rows x cols] of type t as a uint8 array: every code bit uniform random, fp16 scales U(lo,hi)."""
    rng = np.random.default_rng(seed)
    be, bb = ol.BLOCK[t]
    n = rows * cols
    nb = n // be
    if t == ol.F32:
        return (rng.standard_normal(n) * 0.02).astype(np.float32).view(np.uint8)
    if t == ol.F16:
        return (rng.standard_normal(n) * 0.02).astype(np.float16).view(np.uint8)
    if t == ol.BF16:
        f = (rng.standard_normal(n) * 0.02).astype(np.float32)
        return (f.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
    raw = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)

    def put_scale(off, div=1.0):
        s = (rng.uniform(lo, hi, nb) / div).astype(np.float16).view(np.uint16)
        raw[:, off] = (s & 0xFF).astype(np.uint8)
        raw[:, off + 1] = (s >> 8).astype(np.uint8)

    if t in (ol.IQ1_S, ol.IQ2_XXS, ol.IQ4_NL):
        put_scale(0)
    elif t == ol.Q8_0:
        put_scale(0, 16.0)
    elif t == ol.Q5_K:
        put_scale(0, 8.0)
        put_scale(2, 4.0)
    elif t == ol.Q6_K:
        put_scale(208, 32.0)
    else:
        raise ValueError(t)
    return raw.reshape(-1)


def randn(n, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(n) * scale).astype(np.float32)


def hashed(n, salt, scale=1.0):
    """n float32 values in scale * [-0.5, 0.5) from integer arithmetic only (no library generator): the same bits on
    every platform and numpy version, so large golden-vector inputs need not be stored."""
    i = np.arange(n, dtype=np.uint64)
    v = (i * np.uint64(2654435761) + np.uint64(salt) * np.uint64(40503) + (i >> np.uint64(7)) * np.uint64(97)) & np.uint64(0xFFFF)
    return ((v.astype(np.float64) / 65536.0 - 0.5) * scale).astype(np.float32)


def hashed_bf16(n, salt, scale=1.0):
    """The same values rounded to bf16 bit patterns (uint16)."""
    f = hashed(n, salt, scale)
    u = f.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return u.astype(np.uint16)
