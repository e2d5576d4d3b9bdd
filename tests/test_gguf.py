"""The GGUF reader (include/ms_b200_gguf.hpp) on files written by tests/gguf_synth.py: tensor table with absolute
offsets over two splits, every metadata value type incl. nested arrays, a non-default alignment, the expert layout,
split-name expansion, the type-size table against the real model's tensor list (tests/golden/tensor_sizes.json), and
malformed files.  The reference's own test needs the 233 GB model (tests/test_gguf.cpp) and skips without it; its
checks that do not (type sizes, split expansion) are repeated here."""
import json
import os
import subprocess

import numpy as np
import pytest

import gguf_synth as gs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TYPE_ID = {"F32": 0, "F16": 1, "Q8_0": 8, "Q5_K": 13, "Q6_K": 14, "IQ2_XXS": 16, "IQ1_S": 19, "IQ4_NL": 20, "BF16": 30, "MXFP4": 39,
           "Q4_K": 12, "IQ4_XS": 23, "I32": 26}
BLOCK = {"F32": (1, 4), "F16": (1, 2), "BF16": (1, 2), "Q8_0": (32, 34), "Q6_K": (256, 210), "IQ1_S": (256, 50), "IQ2_XXS": (256, 66)}


@pytest.fixture(scope="module")
def exe(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("gguf") / "gguf_exec")
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "gguf_exec.cpp"), "-o", out])
    return out


def nbytes(t, ne):
    b, s = BLOCK[t]
    return int(np.prod(ne)) // b * s


def make_model(d, n_layers=2, n_experts=8, dim=512, inter=256, seed=1):
    """Two splits: metadata + dense tensors + layer 0's experts, then the other layers' experts."""
    rng = np.random.default_rng(seed)
    blob = lambda t, ne: rng.integers(0, 256, nbytes(t, ne), dtype=np.uint8)
    kvs = [("general.architecture", gs.STR, "deepseek41"), ("deepseek41.block_count", gs.U32, n_layers),
           ("deepseek41.expert_count", gs.U32, n_experts), ("deepseek41.expert_weights_norm", gs.BOOL, 1),
           ("deepseek41.expert_weights_scale", gs.F32, 1.5), ("t.i8", gs.I8, -5), ("t.u16", gs.U16, 65535), ("t.i16", gs.I16, -300),
           ("t.i32", gs.I32, -70000), ("t.u64", gs.U64, 2 ** 63 + 5), ("t.i64", gs.I64, -2 ** 40), ("t.f64", gs.F64, 2.5e-9),
           ("t.u8", gs.U8, 200), ("tok.tokens", gs.ARR, (gs.STR, ["<s>", "hello", "wörld", ""])),
           ("tok.types", gs.ARR, (gs.I32, [1, 2, 3, -4])), ("t.floats", gs.ARR, (gs.F32, [0.5, -1.25])),
           ("t.mult", gs.ARR, (gs.I64, [76632096046245, 82619226485591])),
           ("t.nested", gs.ARR, (gs.ARR, [(gs.U8, [1, 2]), (gs.U8, [3])])), ("t.empty", gs.ARR, (gs.U32, []))]
    names = ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")

    def experts(l):
        out = []
        for k, nm in enumerate(names):
            t = "IQ2_XXS" if k == 2 else "IQ1_S"
            ne = [inter, dim, n_experts] if k == 2 else [dim, inter, n_experts]
            out.append(("blk.%d.%s.weight" % (l, nm), TYPE_ID[t], ne, blob(t, ne)))
        return out
    t1 = [("token_embd.weight", TYPE_ID["Q6_K"], [dim, 64], blob("Q6_K", [dim, 64])),
          ("blk.0.attn_norm.weight", TYPE_ID["F32"], [dim], blob("F32", [dim])),
          ("odd.weight", TYPE_ID["Q8_0"], [32, 3, 1, 5], blob("Q8_0", [32, 3, 1, 5]))] + experts(0)
    t2 = [t for l in range(1, n_layers) for t in experts(l)]
    p1, p2 = os.path.join(d, "m-00001-of-00002.gguf"), os.path.join(d, "m-00002-of-00002.gguf")
    o1 = gs.write(p1, kvs, t1, align=64)
    o2 = gs.write(p2, [("general.architecture", gs.STR, "other"), ("split.only", gs.U32, 7)], t2, align=64)
    return p1, [(p1, t1, o1), (p2, t2, o2)], kvs


def test_parse_two_splits(exe, tmp_path):
    p1, splits, kvs = make_model(str(tmp_path))
    out = subprocess.check_output([exe, "parse", p1], text=True).splitlines()
    n_t = sum(len(t) for _, t, _ in splits)
    assert out[0] == "version 3 align 64 splits 2 tensors %d" % n_t
    rows = [ln.split("\t") for ln in out if ln.startswith("T\t")]
    want = []
    inv = {v: k for k, v in TYPE_ID.items()}
    for path, tensors, offs in splits:
        for name, gt, ne, data in tensors:
            want.append(["T", name, inv[gt], "[" + ", ".join(map(str, ne)) + "]", str(len(data)), os.path.basename(path), str(offs[name])])
    assert rows == want
    for path, tensors, offs in splits:                       # offsets honour the alignment and the bytes are where they say
        raw = open(path, "rb").read()
        for name, gt, ne, data in tensors:
            assert offs[name] % 64 == 0 and raw[offs[name]:offs[name] + len(data)] == bytes(data)
    kv = {ln.split("\t")[1]: ln.split("\t")[2] for ln in out if ln.startswith("K\t")}
    assert kv["general.architecture"] == "str:deepseek41"          # first occurrence wins over the second split's
    assert kv["split.only"] == "u:7"
    assert kv["deepseek41.expert_weights_norm"] == "bool:1" and kv["deepseek41.expert_weights_scale"] == "f:1.5"
    assert kv["t.i8"] == "i:-5" and kv["t.u16"] == "u:65535" and kv["t.i16"] == "i:-300" and kv["t.i32"] == "i:-70000"
    assert kv["t.u64"] == "u:%d" % (2 ** 63 + 5) and kv["t.i64"] == "i:%d" % (-2 ** 40) and kv["t.f64"] == "f:2.5e-09"
    assert kv["tok.tokens"] == "arr[4]:<s>,hello,wörld," and kv["tok.types"] == "arr[4]:1,2,3,-4"
    assert kv["t.floats"] == "arr[2]:0.5,-1.25" and kv["t.mult"] == "arr[2]:76632096046245,82619226485591"
    assert kv["t.nested"] == "arr[2]:(arr[2]:1,2),(arr[1]:3)" and kv["t.empty"] == "arr[0]:"
    keys = [ln.split("\t")[1] for ln in out if ln.startswith("K\t")]
    assert keys[:3] == ["general.architecture", "deepseek41.block_count", "deepseek41.expert_count"]     # insertion order
    # expert layout: per-expert stride = tensor bytes / experts, base = the tensor's absolute offset, split index
    lay = [ln.split("\t") for ln in out if ln.startswith("E\t")]
    assert len(lay) == 6
    for _e, l, k, split, base, stride, ln_, tname in lay:
        path, tensors, offs = splits[int(split)]
        name = "blk.%s.%s.weight" % (l, ("ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")[int(k)])
        data = [t for t in tensors if t[0] == name][0][3]
        assert int(base) == offs[name] and int(stride) == len(data) // 8 == int(ln_)
        assert tname == ("IQ2_XXS" if k == "2" else "IQ1_S") and int(split) == (0 if l == "0" else 1)


def test_split_names_and_type_sizes(exe):
    sp = subprocess.check_output([exe, "splits", "/a/b-00002-of-00005.gguf"], text=True).split()
    assert sp == ["/a/b-%05d-of-00005.gguf" % i for i in range(1, 6)]
    assert subprocess.check_output([exe, "splits", "/a/b.gguf"], text=True).split() == ["/a/b.gguf"]
    assert subprocess.check_output([exe, "splits", "/a/b-0002-of-00005.gguf"], text=True).split() == ["/a/b-0002-of-00005.gguf"]
    tb = lambda t, n: subprocess.check_output([exe, "typebytes", str(t), str(n)], text=True).split()
    assert tb(19, 256) == ["IQ1_S", "50"] and tb(16, 256) == ["IQ2_XXS", "66"] and tb(20, 256) == ["IQ4_NL", "144"]
    assert tb(14, 5120) == ["Q6_K", "4200"]
    ids = dict(TYPE_ID)
    for t, n, b in json.load(open(os.path.join(ROOT, "tests", "golden", "tensor_sizes.json"))):
        assert tb(ids[t], n) == [t, str(b)], (t, n)
    assert subprocess.run([exe, "typebytes", "19", "100"], capture_output=True).returncode == 3      # not a whole block


def test_malformed_files_are_refused(exe, tmp_path):
    p1, splits, _ = make_model(str(tmp_path), n_layers=1)
    raw = open(splits[0][0], "rb").read()
    bad = str(tmp_path / "bad.gguf")
    for mutate, msg in ((lambda b: b"GGUX" + b[4:], "bad magic"), (lambda b: b[:4] + b"\x01\0\0\0" + b[8:], "unsupported version"),
                        (lambda b: b[:200], "past the end"), (lambda b: b[:len(b) - 4096], "past the end")):
        open(bad, "wb").write(mutate(raw))
        r = subprocess.run([exe, "parse", bad], capture_output=True, text=True)
        assert r.returncode == 3 and msg in r.stderr, (msg, r.stderr)
    r = subprocess.run([exe, "parse", str(tmp_path / "missing.gguf")], capture_output=True, text=True)
    assert r.returncode == 3 and "cannot open" in r.stderr
