"""Host mirror of the reference's quant module interface (namespace ms::q, src/kernels/quant.hpp): same function
names, argument meaning and preconditions; every call enqueues CUDA work through the C ABI and returns."""
import enum

import torch

from . import _lib
from .core import Enc, ptr


class QType(enum.IntEnum):
    """ggml type ids (src/kernels/quant_types.hpp:10-12)."""
    F32 = 0
    F16 = 1
    Q8_0 = 8
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ1_S = 19
    IQ4_NL = 20
    BF16 = 30


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
