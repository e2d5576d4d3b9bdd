"""The attention side over a chunk of tokens (ms::attn::encode_layer with n > 1, include/ms_b200_attn_state.hpp): 150
tokens -- more than the 128-row window ring -- through a KV / index source layer with ratio 2 and a layer that shares its
caches and per-token top-k lists must equal, bit for bit, the same tokens decoded one at a time; the per-token lists are
causal (token t selects only compressed rows that exist at t)."""
import os
import subprocess

import numpy as np
import pytest

import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_chunk_equals_token_by_token(tmp_path):
    n, D, H, IH, ID, K = 150, 512, 64, 32, 128, 512
    d = str(tmp_path)
    lib_dir = os.path.join(ROOT, "macseek_b200")
    exe = os.path.join(d, "attn_chunk_exec")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "attn_chunk_exec.cpp"), "-o", exe, "-L", lib_dir, "-lmacseek_b200",
                           "-Wl,-rpath," + lib_dir, "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"])
    parts = [1 + 0.1 * synth.randn(D, 1), synth.randn(H, 2), 1 + 0.1 * synth.randn(D, 3), 1 + 0.1 * synth.randn(ID, 4)]
    wk = synth.hashed_bf16(ID * D, 5, 0.1)
    per_tok = [synth.randn(n * H * D, 6), synth.randn(n * H * D, 7), synth.randn(n * D, 8, 2.0), synth.randn(n * D, 9, 2.0),
               synth.randn(n * D, 10, 2.0), synth.randn(n * IH * ID, 11), synth.randn(n * IH, 12)]
    with open(os.path.join(d, "blob"), "wb") as f:
        for p in parts:
            f.write(p.astype(np.float32).tobytes())
        f.write(np.ascontiguousarray(wk).tobytes())
        for p in per_tok:
            f.write(p.astype(np.float32).tobytes())
    subprocess.check_call([exe, os.path.join(d, "blob"), os.path.join(d, "out"), str(n)])
    raw = np.fromfile(os.path.join(d, "out"), np.uint8)
    sz = 2 * n * H * D * 4
    A, B = raw[:sz].view(np.float32), raw[sz:2 * sz].view(np.float32)
    lists = raw[2 * sz:2 * sz + n * K * 4].view(np.int32).reshape(n, K)
    rows = raw[2 * sz + n * K * 4:].view(np.uint16).reshape(n // 2, D)
    assert np.isfinite(A).all() and np.array_equal(A.view(np.uint32), B.view(np.uint32))
    assert A.reshape(2, n, -1)[0].std() > 0 and not np.array_equal(A.reshape(2, n, -1)[0], A.reshape(2, n, -1)[1])
    for t in range(n):                              # causal: token t sees the (t + 1) // 2 compressed rows, the rest is -1
        have = (t + 1) // 2
        sel = lists[t][lists[t] >= 0]
        assert len(sel) == min(have, K) and (len(sel) == 0 or sel.max() < have) and len(set(sel.tolist())) == len(sel)
    assert rows.any(axis=1).all()                   # every completed group wrote its compressed row
