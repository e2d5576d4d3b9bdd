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
