"""GPU parity of the quant kernels through the C ABI: dequant bit-exact, matvec / matvec_n against the oracle in the
reference's normalised error metric |got - ref| / sum|w x| (tests/quant_test_util.hpp:44-52; the reference's own GPU
tolerance is 2e-5, tests/test_quant_matvec.mm:42)."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu

QUANT_TYPES = (ol.Q8_0, ol.Q5_K, ol.Q6_K, ol.IQ2_XXS, ol.IQ1_S, ol.IQ4_NL)
TOL = 2e-5          # the reference's own bound on |got - ref| / sum_k |w_k x_k| (tests/test_quant_matvec.mm:42)
# The relative bound asked of this path, |got - ref| / |ref| <= 1e-3: taken over the whole output vector (L2 norms) and
# per row for every row whose terms do not cancel (see run_matvec); for cancelling rows the normalised bound above is
# the meaningful one.
REL_TOL = 1e-3


@pytest.fixture(scope="module")
def orc():
    return ol.Oracle()


@pytest.fixture(scope="module")
def q():
    from macseek_b200 import quant
    return quant


@pytest.fixture()
def enc():
    from macseek_b200.core import Enc
    return Enc()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("t", QUANT_TYPES + (ol.F16, ol.BF16, ol.F32))
def test_dequant_bit_exact_1m(orc, q, enc, t):
    n = 1 << 20
    raw = synth.random_weights(t, 1, n, 100 + t)
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    q.encode_dequant(enc, t, dev(raw), n, out)
    enc.wait()
    assert np.array_equal(bits(out.cpu().numpy()), bits(orc.dequant(t, raw, n)))


def test_dequant_golden_vectors(q, enc):
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden_ref.npz"))
    for t in QUANT_TYPES + (ol.F16, ol.BF16, ol.F32):
        out = torch.empty(512, dtype=torch.float32, device="cuda")
        q.encode_dequant(enc, t, dev(G["deq_raw_%d" % t]), 512, out)
        enc.wait()
        assert np.array_equal(bits(out.cpu().numpy()), bits(G["deq_out_%d" % t])), ol.TYPE_NAMES[t]


def run_matvec(orc, q, enc, t, rows, cols, groups=1, acc=False, n=1, seed=0):
    W = synth.random_weights(t, rows, cols, 7 + rows + cols + seed)
    x = synth.randn(n * cols * groups, 99 + cols + seed).reshape(n, cols * groups)
    y0 = synth.randn(n * rows, 5).reshape(n, rows)
    ry, mag = orc.matvec(t, W, rows, cols, x, groups)
    if acc:
        ry = ry + y0
        mag = mag + np.abs(y0)
    Wd, xd, yd = dev(W), dev(x), dev(y0)
    if n == 1:
        q.encode_matvec(enc, t, Wd, rows, cols, xd, yd, acc, groups)
    else:
        q.encode_matvec_n(enc, t, Wd, rows, cols, xd, yd, n, acc, groups)
    enc.wait()
    got = yd.cpu().numpy()
    err = orc.max_norm_err(got, ry, mag)
    # relative error: over the whole output (L2), and row by row where the row's terms do not cancel (|ref| at least 5 %
    # of the summed magnitudes); a row whose terms cancel to ~0 has no meaningful relative error in any arithmetic
    solid = np.abs(ry) >= 0.05 * mag
    rel_rows = float(np.max(np.abs(got - ry)[solid] / np.abs(ry)[solid])) if solid.any() else 0.0
    rel = max(rel_rows, float(np.linalg.norm(got - ry) / (np.linalg.norm(ry) + 1e-30)))
    return err, rel, (Wd, xd, yd)


def test_cfg1_iq1s_4096(orc, q, enc):
    err, rel, _ = run_matvec(orc, q, enc, ol.IQ1_S, 4096, 4096)
    assert err <= TOL, err
    assert rel <= REL_TOL, rel


@pytest.mark.parametrize("t", (ol.Q8_0, ol.Q6_K, ol.Q5_K, ol.IQ4_NL, ol.IQ2_XXS))
@pytest.mark.parametrize("shape", ((4096, 4096), (16384, 4096), (4096, 16384)))
@pytest.mark.parametrize("n", (1, 4))
def test_cfg2_sweep(orc, q, enc, t, shape, n):
    err, rel, _ = run_matvec(orc, q, enc, t, shape[0], shape[1], n=n)
    assert err <= TOL, (ol.TYPE_NAMES[t], shape, n, err)
    assert rel <= REL_TOL, (ol.TYPE_NAMES[t], shape, n, rel)


# the reference's own shape list (tests/test_quant_matvec.mm:14-28): type, rows, cols, groups, accumulate
REF_CASES = [
    (ol.Q6_K, 1280, 5120, 1, False), (ol.Q5_K, 1280, 5120, 1, False), (ol.Q6_K, 32768, 1280, 1, False),
    (ol.Q5_K, 32768, 1280, 1, False), (ol.Q6_K, 512, 5120, 1, False), (ol.Q5_K, 512, 5120, 1, True),
    (ol.Q6_K, 8192, 4096, 8, False), (ol.Q5_K, 8192, 4096, 8, True), (ol.Q6_K, 5120, 8192, 1, False),
    (ol.Q5_K, 5120, 8192, 1, False), (ol.IQ1_S, 2304, 5120, 1, False), (ol.IQ1_S, 5120, 2304, 1, True),
    (ol.IQ2_XXS, 2304, 5120, 1, False), (ol.IQ2_XXS, 5120, 2304, 1, False), (ol.Q6_K, 2304, 5120, 1, False),
    (ol.Q6_K, 5120, 2304, 1, False), (ol.Q8_0, 2304, 5120, 1, False), (ol.Q8_0, 5120, 2304, 1, True),
    (ol.Q6_K, 25600, 6144, 1, False), (ol.F32, 384, 5120, 1, False), (ol.F32, 24, 20480, 1, False),
    (ol.BF16, 512, 5120, 1, False), (ol.BF16, 4096, 1280, 1, False), (ol.BF16, 32, 5120, 1, False),
    (ol.BF16, 128, 512, 1, False), (ol.F16, 1280, 5120, 1, False), (ol.F16, 7, 768, 1, True),
    (ol.Q6_K, 3, 256, 1, False), (ol.IQ4_NL, 33, 1056, 1, False), (ol.Q6_K, 8192, 4608, 8, False),
]


@pytest.mark.parametrize("case", REF_CASES, ids=lambda c: "%s-%dx%d-g%d%s" % (ol.TYPE_NAMES[c[0]], c[1], c[2], c[3], "-acc" if c[4] else ""))
def test_reference_shapes(orc, q, enc, case):
    t, rows, cols, groups, acc = case
    err, rel, _ = run_matvec(orc, q, enc, t, rows, cols, groups, acc)
    assert err <= TOL, err
    assert rel <= REL_TOL, rel


@pytest.mark.parametrize("n", (2, 3, 5, 8, 16))
def test_matvec_n_columns(orc, q, enc, n):
    for t, rows, cols, groups in ((ol.Q6_K, 1280, 5120, 1), (ol.IQ2_XXS, 2304, 5120, 1), (ol.Q5_K, 1024, 4096, 8),
                                  (ol.BF16, 512, 1280, 1)):
        err, rel, _ = run_matvec(orc, q, enc, t, rows, cols, groups, acc=(n % 2 == 1), n=n)
        assert err <= TOL, (ol.TYPE_NAMES[t], n, err)


def test_head_matvec_q6k_129280(orc, q, enc):
    err, rel, _ = run_matvec(orc, q, enc, ol.Q6_K, 129280, 4096)
    assert err <= TOL, err


def test_unaligned_weight_base_and_repeatability(orc, q, enc):
    # weights at a 4-byte (not 16-byte) aligned offset inside an arena, as tests/test_quant_moe.mm:46-56 places them
    rows, cols, t = 2304, 5120, ol.IQ1_S
    W = synth.random_weights(t, rows, cols, 3)
    x = synth.randn(cols, 4)
    arena = torch.zeros(W.size + 64, dtype=torch.uint8, device="cuda")
    outs = []
    for off in (4, 6, 12, 0):
        arena[off:off + W.size] = dev(W)
        y = torch.zeros(rows, device="cuda")
        q.encode_matvec(enc, t, arena[off:], rows, cols, dev(x), y)
        enc.wait()
        outs.append(y.cpu().numpy())
    ry, mag = orc.matvec(t, W, rows, cols, x)
    assert orc.max_norm_err(outs[0], ry, mag) <= TOL
    for o in outs[1:]:
        assert np.array_equal(bits(o), bits(outs[0]))      # run-to-run and placement independent, bit for bit


def test_large_activation_outlier(orc, q, enc):
    # One huge activation in a 32-element unit coarsens the fixed-point step of its 31 neighbours (the unit's step is
    # amax / 32767).  The scheme's worst-case error is sum_units (amax_u / 65534) * sum_{k in u} |w_k|: the result must
    # stay inside that bound row by row, and inside 5e-5 of the summed magnitudes overall.
    rows, cols, t = 512, 4096, ol.Q6_K
    W = synth.random_weights(t, rows, cols, 8)
    x = synth.randn(cols, 9)
    x[100] = 500.0
    x[2000] = -1e-6
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec(enc, t, dev(W), rows, cols, dev(x), y)
    enc.wait()
    ry, mag = orc.matvec(t, W, rows, cols, x)
    got = y.cpu().numpy()
    wabs = np.abs(orc.dequant(t, W, rows * cols).reshape(rows, cols // 32, 32)).sum(axis=2)      # [rows][units]
    step = np.abs(x.reshape(-1, 32)).max(axis=1) / 65534.0                                     # half a step per unit
    bound = wabs @ step + 4e-6 * mag                                                           # + fp32 accumulation
    assert np.all(np.abs(got - ry) <= bound)
    assert orc.max_norm_err(got, ry, mag) <= 5e-5


def test_bad_arguments_fail_loudly(q, enc):
    from macseek_b200._lib import MsbError
    W = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    x = torch.zeros(512, device="cuda")
    y = torch.zeros(8, device="cuda")
    with pytest.raises(MsbError):
        q.encode_matvec(enc, ol.IQ1_S, W, 8, 100, x, y)          # cols not a multiple of the block
    with pytest.raises(MsbError):
        q.encode_matvec(enc, 39, W, 8, 256, x, y)                # MXFP4: no kernel
    with pytest.raises(MsbError):
        q.encode_matvec(enc, ol.Q6_K, W, 9, 256, x, y, False, 2)  # rows % groups


@pytest.mark.parametrize("t", (ol.Q6_K, ol.IQ1_S, ol.BF16, ol.Q8_0))
def test_matvec_rmsnorm_fused(orc, q, enc, t):
    # y = W . (x * rsqrt(mean(x^2) + eps) * norm_w)  (quant.hpp:19-26)
    rows, cols = 1280, 4096
    W = synth.random_weights(t, rows, cols, 21)
    x = synth.randn(cols, 22, 3.0)
    nw = (1 + 0.1 * synth.randn(cols, 23)).astype(np.float32)
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec_rmsnorm(enc, t, dev(W), rows, cols, dev(x), dev(nw), 1e-6, y)
    enc.wait()
    ry, mag = orc.matvec(t, W, rows, cols, orc.rmsnorm(x, nw, 1e-6))
    assert orc.max_norm_err(y.cpu().numpy(), ry, mag) <= TOL


@pytest.mark.parametrize("t,rows,cols", ((ol.Q6_K, 16384, 1024), (ol.Q6_K, 1280, 4096), (ol.Q8_0, 4096, 4096),
                                         (ol.BF16, 512, 2048), (ol.IQ1_S, 1280, 4096), (ol.Q6_K, 96, 16384)))
def test_matvec_rmsnorm_shared_launch(orc, q, enc, t, rows, cols):
    """The launch form that leaves room on every SM for another stream (one small block per SM): same values as the
    oracle; table types and rows too long for the small block take the ordinary launch.  Also run beside work on a
    second stream."""
    W = synth.random_weights(t, rows, cols, 31)
    x = synth.randn(cols, 32, 2.0)
    nw = (1 + 0.1 * synth.randn(cols, 33)).astype(np.float32)
    Wd, xd, nd = dev(W), dev(x), dev(nw)
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec_rmsnorm_shared(enc, t, Wd, rows, cols, xd, nd, 1e-6, y)
    enc.wait()
    ry, mag = orc.matvec(t, W, rows, cols, orc.rmsnorm(x, nw, 1e-6))
    assert orc.max_norm_err(y.cpu().numpy(), ry, mag) <= TOL
    # beside an ordinary launch on another stream
    from macseek_b200.core import Enc
    side = torch.cuda.Stream()
    y2, y3 = torch.zeros(rows, device="cuda"), torch.zeros(rows, device="cuda")
    side.wait_stream(enc.stream)
    q.encode_matvec_rmsnorm_shared(Enc(side), t, Wd, rows, cols, xd, nd, 1e-6, y2)
    q.encode_matvec_rmsnorm(enc, t, Wd, rows, cols, xd, nd, 1e-6, y3)
    enc.stream.wait_stream(side)
    enc.wait()
    assert np.array_equal(y2.cpu().numpy().view(np.uint32), y.cpu().numpy().view(np.uint32))
    assert orc.max_norm_err(y3.cpu().numpy(), ry, mag) <= TOL


# ---- the 16-bit fixed-point activation at its weak spots: heavy tails and a wide dynamic range inside one unit
@pytest.mark.parametrize("t", (ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, ol.Q6_K, ol.Q5_K, ol.IQ4_NL))
def test_heavy_tailed_activation(orc, q, enc, t):
    # Student-t with 3 degrees of freedom: what a residual stream with outlier channels looks like
    rows, cols = 1024, 4096
    W = synth.random_weights(t, rows, cols, 41)
    x = np.random.default_rng(42).standard_t(3, cols).astype(np.float32)
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec(enc, t, dev(W), rows, cols, dev(x), y)
    enc.wait()
    ry, mag = orc.matvec(t, W, rows, cols, x)
    assert orc.max_norm_err(y.cpu().numpy(), ry, mag) <= TOL


@pytest.mark.parametrize("t", (ol.IQ2_XXS, ol.IQ1_S, ol.Q8_0))
def test_activation_spanning_decades_inside_a_unit(orc, q, enc, t):
    # |x| log-uniform over 1e-4 .. 10 within every 32-element unit, as the SwiGLU outputs read by the MoE down projection
    rows, cols = 1024, 2048
    rng = np.random.default_rng(43)
    x = (10.0 ** rng.uniform(-4, 1, cols) * rng.choice([-1.0, 1.0], cols)).astype(np.float32)
    W = synth.random_weights(t, rows, cols, 44)
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec(enc, t, dev(W), rows, cols, dev(x), y)
    enc.wait()
    ry, mag = orc.matvec(t, W, rows, cols, x)
    assert orc.max_norm_err(y.cpu().numpy(), ry, mag) <= TOL
