"""Expert-parallel weight placement from a GGUF file (include/ms_b200_expert_shard.hpp), executed: a synthetic two-split
model with valid IQ1_S / IQ2_XXS expert blocks is loaded rank by rank (world 1, 2 and 4), each rank runs the MoE decode
kernels over the experts it holds, and the ranks' partial outputs must sum to the oracle's result computed from the
SAME bytes of the file."""
import os
import subprocess

import numpy as np
import pytest

import gguf_synth as gs
import oracle_lib as ol
import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DIM, INTER, E, K, LAYERS = 512, 256, 8, 4, 2


def test_expert_shards_from_file(tmp_path):
    orc = ol.Oracle()
    d = str(tmp_path)
    lib_dir = os.path.join(ROOT, "macseek_b200")
    exe = os.path.join(d, "gguf_exec")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-DWITH_SHARD", "-I", os.path.join(ROOT, "include"), "-I/usr/local/cuda/include",
                           os.path.join(ROOT, "tests", "gguf_exec.cpp"), "-o", exe, "-L", lib_dir, "-lmacseek_b200",
                           "-Wl,-rpath," + lib_dir, "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,/usr/local/cuda/lib64"])
    # stacked expert tensors: expert e of a matrix is rows [e * rows, (e + 1) * rows) of one random-block matrix
    mats = {}

    def stacked(l, k):
        t, rows, cols = (ol.IQ2_XXS, DIM, INTER) if k == 2 else (ol.IQ1_S, INTER, DIM)
        w = synth.random_weights(t, rows * E, cols, 50 + 10 * l + k)
        mats[(l, k)] = w.reshape(E, -1)
        return w
    names = ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")
    kvs = [("general.architecture", gs.STR, "deepseek41"), ("deepseek41.block_count", gs.U32, LAYERS),
           ("deepseek41.expert_count", gs.U32, E)]
    tensors = [[], []]
    for l in range(LAYERS):
        for k in range(3):
            ne = [INTER, DIM, E] if k == 2 else [DIM, INTER, E]
            tensors[l].append(("blk.%d.%s.weight" % (l, names[k]), 16 if k == 2 else 19, ne, stacked(l, k)))
    p1 = os.path.join(d, "m-00001-of-00002.gguf")
    gs.write(p1, kvs, [("pad.weight", 0, [7], np.zeros(28, np.uint8))] + tensors[0])
    gs.write(os.path.join(d, "m-00002-of-00002.gguf"), [], tensors[1])
    # per-layer routing and one input vector
    x = synth.randn(DIM, 3)
    ids = np.array([[1, 6, 2, 5], [7, 0, 3, 4]], np.int32)
    w = np.abs(synth.randn(LAYERS * K, 4)).reshape(LAYERS, K).astype(np.float32) + 0.1
    with open(os.path.join(d, "in.bin"), "wb") as f:
        f.write(np.int32(K).tobytes())
        for l in range(LAYERS):
            f.write(ids[l].tobytes()); f.write(w[l].tobytes())
        f.write(x.tobytes())
    want = []
    for l in range(LAYERS):
        g = [mats[(l, 0)][e] for e in ids[l]]
        u = [mats[(l, 1)][e] for e in ids[l]]
        dn = [mats[(l, 2)][e] for e in ids[l]]
        _, y, mag, _ = orc.moe_decode(DIM, INTER, ol.IQ1_S, ol.IQ2_XXS, ol.Q8_0, g, u, dn, w[l], x, np.zeros(DIM), has_shared=False)
        want.append((y, mag))
    for world in (1, 2, 4):
        total = np.zeros((LAYERS, DIM), np.float64)
        for rank in range(world):
            out = os.path.join(d, "out_%d_%d.bin" % (world, rank))
            msg = subprocess.check_output([exe, "shard", p1, str(rank), str(world), os.path.join(d, "in.bin"), out], text=True)
            assert "experts [%d, %d)" % (rank * E // world, (rank + 1) * E // world) in msg
            part = np.fromfile(out, np.float32).reshape(LAYERS, DIM)
            # a rank that holds none of this layer's experts contributes exactly zero
            for l in range(LAYERS):
                if not any(rank * E // world <= e < (rank + 1) * E // world for e in ids[l]):
                    assert not part[l].any()
            total += part
        for l in range(LAYERS):
            assert orc.max_norm_err(total[l], want[l][0], want[l][1]) <= 5e-5, (world, l)
