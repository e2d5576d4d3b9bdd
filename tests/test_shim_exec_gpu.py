"""The C++ shim executed, not only compiled: a program built against include/ms_b200_shim.hpp runs ms::q::encode_matvec
and ms::attn::encode_index_decode on the GPU; its outputs must equal, bit for bit, the same calls made through ctypes."""
import os
import subprocess
import tempfile

import numpy as np
import pytest
import torch

import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shim_calls_equal_ctypes_calls():
    from macseek_b200 import attn, quant as q
    from macseek_b200.core import Enc
    rows, cols, length = 1280, 4096, 5000
    W = synth.random_weights(ol.Q6_K, rows, cols, 1)
    x = synth.randn(cols, 2)
    keys = synth.randn(length * 128, 3).astype(np.float16)
    iq, iw = synth.randn(32 * 128, 4), synth.randn(32, 5)
    rope = attn.make_rope_table(4, True)[0].reshape(-1)
    lib_dir = os.path.join(ROOT, "macseek_b200")
    with tempfile.TemporaryDirectory() as d:
        p = lambda n: os.path.join(d, n)
        W.tofile(p("W")); x.tofile(p("x")); keys.tofile(p("k"))
        np.concatenate([iq, iw, rope.astype(np.float32)]).astype(np.float32).tofile(p("qw"))
        subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                               os.path.join(ROOT, "tests", "shim_exec.cpp"), "-o", p("t"), "-L", lib_dir, "-lmacseek_b200",
                               "-Wl,-rpath," + lib_dir, "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"])
        subprocess.check_call([p("t"), str(rows), str(cols), str(length), p("W"), p("x"), p("k"), p("qw"), p("out")])
        out = np.fromfile(p("out"), dtype=np.uint8)
    y_shim = out[:rows * 4].view(np.float32)
    tk_shim = out[rows * 4:].view(np.int32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    e = Enc()
    y = torch.zeros(rows, device="cuda")
    q.encode_matvec(e, q.QType.Q6_K, dev(W), rows, cols, dev(x), y)
    sh = attn.Shape.reference()
    st = attn.DecodeState(sh, length, dev(attn.make_rope_table(4, True)), "cuda")
    st.ikey[:length].copy_(dev(keys).view(st.ikey.dtype).reshape(length, -1))
    attn.encode_index_decode(e, st, dev(iq), dev(iw), 0, length, actq=True)
    e.wait()
    assert np.array_equal(y_shim.view(np.uint32), y.cpu().numpy().view(np.uint32))
    assert np.array_equal(tk_shim, st.topk.cpu().numpy().reshape(-1)[:512])
