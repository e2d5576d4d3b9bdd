"""The logits dump writer against files written by the reference's own writer (tests/golden/dump_*.logits, made by
tests/golden/make_logits_golden.py with tools/quality.py write_dump): byte-identical output, and the reader returns
what went in."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_logits_golden as mk  # noqa: E402


def test_writer_is_byte_identical_to_the_reference_writer(tmp_path):
    from macseek_b200 import logits_dump as ld
    tokens, logits, ids, vals, lse = mk.inputs()
    full, topk = str(tmp_path / "full.logits"), str(tmp_path / "topk.logits")
    ld.write_full(full, tokens, logits, first_pos=2)
    ld.write_topk(topk, tokens, 50, ids, vals, lse, first_pos=2)
    assert open(full, "rb").read() == open(os.path.join(HERE, "golden", "dump_full.logits"), "rb").read()
    assert open(topk, "rb").read() == open(os.path.join(HERE, "golden", "dump_topk.logits"), "rb").read()


def test_reader_round_trip():
    from macseek_b200 import logits_dump as ld
    tokens, logits, ids, vals, lse = mk.inputs()
    a = ld.read(os.path.join(HERE, "golden", "dump_full.logits"))
    assert a["mode"] == 0 and a["n_vocab"] == 50 and a["first_pos"] == 2 and list(a["tokens"]) == tokens
    assert np.array_equal(a["logits"], logits)
    b = ld.read(os.path.join(HERE, "golden", "dump_topk.logits"))
    assert b["mode"] == 1 and b["k"] == 8 and np.array_equal(b["ids"], ids) and np.array_equal(b["vals"], vals)
    assert np.array_equal(b["lse"], lse)
    # ids are in descending logit order and p = exp(v - lse) is a sub-distribution
    assert np.all(np.diff(b["vals"], axis=1) <= 0) and np.all(np.exp(b["vals"] - b["lse"][:, None]).sum(axis=1) <= 1 + 1e-6)
