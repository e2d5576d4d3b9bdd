"""The small per-token kernels between the hot-path calls, alone: msb_rmsnorm (rows, strides, no weight) and msb_add
against numpy, msb_argmax ties."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("rows,dim,in_stride,out_stride,has_w", [(1, 4096, 0, 0, True), (3, 1280, 1536, 0, True),
                                                                  (64, 128, 0, 160, False), (2, 576, 640, 704, True)])
def test_rmsnorm_rows_and_strides(rows, dim, in_stride, out_stride, has_w):
    from macseek_b200 import _lib
    from macseek_b200.core import Enc
    orc = ol.Oracle()
    si, so = in_stride or dim, out_stride or dim
    x = synth.randn(rows * si, 3, 2.5).reshape(rows, si)
    w = (1 + 0.1 * synth.randn(dim, 4)).astype(np.float32) if has_w else None
    y0 = synth.randn(rows * so, 5).reshape(rows, so)
    xd, yd = dev(x), dev(y0)
    wd = dev(w) if has_w else None
    e = Enc()
    _lib.check(_lib.lib.msb_rmsnorm(xd.data_ptr(), wd.data_ptr() if has_w else None, yd.data_ptr(), rows, dim, 1e-6,
                                    in_stride, out_stride, e.handle))
    e.wait()
    got = yd.cpu().numpy()
    for r in range(rows):
        want = orc.rmsnorm(x[r, :dim], w if has_w else np.ones(dim, np.float32), 1e-6)
        assert np.max(np.abs(got[r, :dim] - want)) <= 2e-6 * np.max(np.abs(want))
        assert np.array_equal(got[r, dim:], y0[r, dim:])          # the padding between rows is untouched


@pytest.mark.parametrize("n", (1, 7, 4096, 129280))
def test_add(n):
    from macseek_b200 import arch
    from macseek_b200.core import Enc
    y, a = synth.randn(n, 1), synth.randn(n, 2)
    yd, ad = dev(y), dev(a)
    e = Enc()
    arch.encode_add(e, yd, ad, n)
    e.wait()
    assert np.array_equal(yd.cpu().numpy(), y + a)


def test_argmax_ties_take_the_lowest_index():
    from macseek_b200 import arch
    from macseek_b200.core import Enc
    x = synth.randn(129280, 6)
    x[[70000, 313, 99999]] = 50.0
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    e = Enc()
    arch.encode_argmax(e, dev(x), 1, x.size, out)
    e.wait()
    assert int(out.item()) == 313


@pytest.mark.parametrize("D,elem", [(512, "f16"), (576, "bf16")])
def test_kv_window_row_with_fp8_simulation(D, elem):
    # rmsnorm -> rope -> fp8 (e4m3, power-of-two scale per 32) simulation: on the e4m3 lattice every value equals the
    # oracle's except where the fp32 rounding of the normalised value falls on the other side of a lattice midpoint
    from macseek_b200 import _lib, attn
    from macseek_b200.core import Enc
    orc = ol.Oracle()
    kv = synth.randn(D, 7, 3.0)
    nw = (1 + 0.1 * synth.randn(D, 8)).astype(np.float32)
    cs = attn.make_rope_table(300, True)[257]
    out = torch.zeros(D, dtype=torch.float16 if elem == "f16" else torch.bfloat16, device="cuda")
    e = Enc()
    kd, nd, cd = dev(kv), dev(nw), dev(cs)
    _lib.check(_lib.lib.msb_kv_window(kd.data_ptr(), nd.data_ptr(), cd.data_ptr(), 1, D,
                                      attn.ELEM_F16 if elem == "f16" else attn.ELEM_BF16, out.data_ptr(), e.handle))
    e.wait()
    want = orc.window_row(kv, nw, cs, True)
    got = out.float().cpu().numpy()
    if elem == "bf16":
        want = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
    assert np.mean(got == want) >= 0.99 and np.max(np.abs(got - want)) <= 0.13 * np.max(np.abs(want))
