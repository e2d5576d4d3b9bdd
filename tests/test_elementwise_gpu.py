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
