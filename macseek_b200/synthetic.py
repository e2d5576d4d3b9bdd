"""Seeded synthetic weights generated on the device, in raw GGUF block layouts: every code bit uniform random, fp16
block scales ~ U(0.01, 0.05) (divided per type so that dequantised magnitudes are comparable), as the benchmark
configurations specify.  Used by bench.py and the decode-step driver; parity tests build their inputs on the host."""
import torch

from .shapes import BLOCK as _BLOCK, QType, row_bytes  # noqa: F401

def random_weights(t, rows, cols, gen, lo=0.01, hi=0.05, out=None):
    """uint8 tensor of rows * row_bytes(t, cols) bytes on gen.device."""
    t = QType(t)
    dev = gen.device
    n = rows * cols
    if t == QType.F32:
        w = torch.empty(n, dtype=torch.float32, device=dev).normal_(0, 0.02, generator=gen)
        return w.view(torch.uint8)
    if t == QType.F16:
        return torch.empty(n, dtype=torch.float32, device=dev).normal_(0, 0.02, generator=gen).half().view(torch.uint8)
    if t == QType.BF16:
        return torch.empty(n, dtype=torch.float32, device=dev).normal_(0, 0.02, generator=gen).bfloat16().view(torch.uint8)
    be, bb = _BLOCK[t]
    nb = n // be
    raw = out if out is not None else torch.empty(nb * bb, dtype=torch.uint8, device=dev)
    raw = raw.view(nb, bb)
    raw.random_(0, 256, generator=gen)

    def put(off, div):
        s = torch.empty(nb, dtype=torch.float32, device=dev).uniform_(lo, hi, generator=gen) / div
        raw[:, off:off + 2] = s.half().view(torch.uint8).view(nb, 2)

    if t in (QType.IQ1_S, QType.IQ2_XXS, QType.IQ4_NL):
        put(0, 1.0)
    elif t == QType.Q8_0:
        put(0, 16.0)
    elif t == QType.Q5_K:
        put(0, 8.0)
        put(2, 4.0)
    elif t == QType.Q6_K:
        put(208, 32.0)
    return raw.view(-1)
