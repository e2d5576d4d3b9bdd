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


def test_noalloc_joint_limit_is_a_clean_refusal():
    """inter 4096 with 8 routed experts is inside the scratch's limits but beyond what the down launch can stage in
    shared memory: MSB_E_LIMIT before anything is enqueued, y untouched."""
    from macseek_b200 import _lib, quant as q
    from macseek_b200.core import Enc
    _lib.check(_lib.lib.msb_init())
    case = MoeCase(512, 4096, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True, seed=6)
    a = case.args()
    a.scratch = None
    before = a.y.clone()
    with pytest.raises(_lib.MsbError, match="down staging does not fit"):
        q.encode_moe_decode_noalloc(Enc(), a)
    torch.cuda.synchronize()
    assert torch.equal(a.y, before)
    assert _lib.device_status() == 0


def test_noalloc_leaves_device_memory_as_it_is():
    """A warm call allocates nothing: the device's free memory is the same before and after."""
    from macseek_b200 import _lib, quant as q
    from macseek_b200.core import Enc
    _lib.check(_lib.lib.msb_init())
    case = MoeCase(4096, 2048, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, 8, True, seed=5)
    e = Enc()
    a = case.args()
    a.scratch = None
    q.encode_moe_decode_noalloc(e, a)         # warm: kernels loaded, attributes set
    e.wait()
    free0 = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        q.encode_moe_decode_noalloc(e, a)
    e.wait()
    assert torch.cuda.mem_get_info()[0] == free0


def test_noalloc_before_init_is_refused():
    """In a fresh process that has not called msb_init() on the device the entry point creates nothing and returns
    MSB_E_DEVICE."""
    import subprocess
    import sys
    code = r'''
import ctypes as C, os, sys
sys.path.insert(0, os.getcwd())
import torch
torch.cuda.init()
x = torch.zeros(4096, device="cuda")
from macseek_b200 import _lib
a = _lib.MoeDecodeArgsC()
a.dim, a.inter, a.n_routed, a.has_shared = 4096, 2048, 0, 0
a.t_gate_up, a.t_down, a.t_shared = 19, 16, 8
a.x, a.y, a.weights = x.data_ptr(), x.data_ptr(), x.data_ptr()
rc = _lib.lib.msb_moe_decode_noalloc(C.byref(a), None)
print("RC", rc, _lib.lib.msb_last_error().decode())
'''
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert "RC -5" in out.stdout and "msb_init() has not run" in out.stdout, out.stdout + out.stderr
