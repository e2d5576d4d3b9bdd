"""The allocation-free MoE decode entry point (msb_moe_decode_noalloc) against msb_moe_decode, through the C ABI.

Collected last on purpose: it must pass alone and after every other GPU test has used the library."""
import numpy as np
import pytest
import torch

import oracle_lib as ol
from test_moe_gpu import MoeCase, bits

pytestmark = pytest.mark.gpu


def test_noalloc_matches_caller_scratch_twice():
    from macseek_b200 import _lib, quant as q
    from macseek_b200.core import Enc
    _lib.check(_lib.lib.msb_init())
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True, seed=5)
    e = Enc()
    for call in range(2):
        ref_args = case.args()
        q.encode_moe_decode(e, ref_args)
        e.wait()
        want = ref_args.y.cpu().numpy()
        a = case.args()
        a.scratch = None                      # ignored by the entry point under test
        q.encode_moe_decode_noalloc(e, a)
        e.wait()
        got = a.y.cpu().numpy()
        assert np.array_equal(bits(got), bits(want)), "call %d differs" % call
        assert not np.array_equal(bits(got), bits(case.y0))
    assert _lib.device_status() == 0


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from macseek_b200 import _lib, quant as q
    from macseek_b200.core import Enc
    a = q.MoeDecodeArgs(4096, 8192)
    a.t_gate_up, a.t_down, a.t_shared = ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0
    a.n_routed, a.has_shared = 0, False
    a.x = torch.zeros(4096, device="cuda")
    a.y = torch.zeros(4096, device="cuda")
    a.weights = torch.zeros(1, device="cuda")
    with pytest.raises(_lib.MsbError, match="beyond the built-in scratch"):
        q.encode_moe_decode_noalloc(Enc(), a)
