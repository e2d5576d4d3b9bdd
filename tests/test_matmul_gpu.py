"""GPU parity of the prefill projection GEMM (tcgen05) against the reference's own check (tests/test_quant_matmul.mm:
half-exact error <= 1e-5 and error against the pure F32 product <= 2e-3, both normalised by sum |w x|), on the
reference's shape list (:17-23) plus larger token counts."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


def r16(a):
    return a.astype(np.float16).astype(np.float64)


# (type, rows, cols, n, accumulate): tests/test_quant_matmul.mm:17-23
REF_CASES = [
    (ol.Q6_K, 1280, 5120, 77, False), (ol.Q5_K, 1024, 1280, 160, True), (ol.Q6_K, 512, 5120, 64, False),
    (ol.Q8_0, 2304, 5120, 33, False), (ol.Q6_K, 640, 8192, 40, False), (ol.IQ1_S, 2304, 5120, 50, False),
    (ol.IQ2_XXS, 5120, 2304, 37, True), (ol.IQ1_S, 300, 2304, 129, False), (ol.BF16, 512, 5120, 48, False),
    (ol.F16, 256, 1280, 70, False), (ol.F32, 384, 5120, 36, False),
    # beyond the reference's list: several token tiles, ragged token count, the benchmark's hidden size
    (ol.Q6_K, 4096, 4096, 515, False), (ol.IQ4_NL, 1056, 1056, 260, True), (ol.Q8_0, 136, 4096, 1, False),
]


@pytest.mark.parametrize("case", REF_CASES, ids=lambda c: "%s-%dx%d-n%d%s" % (ol.TYPE_NAMES[c[0]], c[1], c[2], c[3], "-acc" if c[4] else ""))
def test_matmul_reference_cases(orc, case):
    from macseek_b200 import quant as q
    from macseek_b200.core import Enc
    t, rows, cols, n, acc = case
    W = synth.random_weights(t, rows, cols, 3 + rows)
    X = synth.randn(n * cols, 11 + n).reshape(n, cols)
    Y0 = synth.randn(n * rows, 12).reshape(n, rows)
    wd = orc.dequant(t, W, rows * cols).reshape(rows, cols).astype(np.float64)
    wh = wd if t == ol.F32 else r16(wd)
    sh = r16(X) @ wh.T
    sf = X.astype(np.float64) @ wd.T
    mag = np.abs(X.astype(np.float64)) @ np.abs(wd).T
    base = Y0.astype(np.float64) if acc else 0.0
    if acc:
        mag = mag + np.abs(Y0)
    Wd = torch.from_numpy(W).cuda()
    Xd = torch.from_numpy(X).cuda()
    Yd = torch.from_numpy(Y0.copy()).cuda()
    scratch = torch.zeros(q.matmul_scratch_bytes(t, rows, cols, n), dtype=torch.uint8, device="cuda")
    e = Enc()
    q.encode_matmul(e, t, Wd, rows, cols, Xd, Yd, n, acc, scratch)
    e.wait()
    got = Yd.cpu().numpy().astype(np.float64)
    err_h = float(np.max(np.abs(got - (sh + base)) / (mag + 1e-12)))
    err_f = float(np.max(np.abs(got - (sf + base)) / (mag + 1e-12)))
    assert err_h <= 1e-5, (err_h, err_f)
    assert err_f <= 2e-3, (err_h, err_f)


def test_matmul_h_strided_and_repeatable(orc):
    """encode_f32_to_f16 once, two matmul_h calls on column windows of a wider X16 (x_stride > cols)."""
    from macseek_b200 import quant as q
    from macseek_b200.core import Enc
    rows, cols, n, stride = 768, 1024, 200, 2048
    W = synth.random_weights(ol.Q6_K, rows, cols, 5)
    X = synth.randn(n * stride, 6).reshape(n, stride)
    wd = r16(orc.dequant(ol.Q6_K, W, rows * cols).reshape(rows, cols).astype(np.float64))
    Wd, Xd = torch.from_numpy(W).cuda(), torch.from_numpy(X).cuda()
    X16 = torch.zeros(n, stride, dtype=torch.float16, device="cuda")
    Y = torch.zeros(n, rows, device="cuda")
    scratch = torch.zeros(q.matmul_scratch_bytes(ol.Q6_K, rows, cols, n, False), dtype=torch.uint8, device="cuda")
    e = Enc()
    q.encode_f32_to_f16(e, Xd, X16, n * stride)
    outs = []
    for off in (0, 1024):
        q.encode_matmul_h(e, ol.Q6_K, Wd, rows, cols, X16[:, off:], Y, n, False, stride, scratch)
        e.wait()
        got = Y.cpu().numpy().astype(np.float64)
        xs = X[:, off:off + cols]
        want = r16(xs) @ wd.T
        mag = np.abs(xs.astype(np.float64)) @ np.abs(wd).T
        assert float(np.max(np.abs(got - want) / mag)) <= 1e-5
        outs.append(got.copy())
    q.encode_matmul_h(e, ol.Q6_K, Wd, rows, cols, X16[:, 1024:], Y, n, False, stride, scratch)
    e.wait()
    assert np.array_equal(Y.cpu().numpy().astype(np.float64), outs[1])


def test_matmul_argument_errors():
    from macseek_b200 import _lib, quant as q
    from macseek_b200.core import Enc
    W = torch.zeros(64 * 210, dtype=torch.uint8, device="cuda")
    X = torch.zeros(4, 256, device="cuda")
    Y = torch.zeros(4, 64, device="cuda")
    with pytest.raises(_lib.MsbError, match="scratch"):
        q.encode_matmul(Enc(), ol.Q6_K, W, 64, 256, X, Y, 4, False, torch.zeros(16, dtype=torch.uint8, device="cuda"))
    with pytest.raises(_lib.MsbError, match="shape"):
        q.encode_matmul(Enc(), ol.Q6_K, W, 64, 100, X, Y, 4, False, torch.zeros(1 << 20, dtype=torch.uint8, device="cuda"))
