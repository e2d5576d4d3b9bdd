#!/usr/bin/env python3
"""Generate tests/golden/dump_full.logits and dump_topk.logits with the reference project's OWN dump writer
(tools/quality.py write_dump, the format's reference writer, docs/modules/oracle.md:49-61) from seeded inputs.

Run where the reference checkout is available:   python tests/golden/make_logits_golden.py <reference checkout>
The two small files are committed; tests/test_logits_dump.py rebuilds the same inputs and compares bytes."""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def inputs():
    """4 positions over a vocabulary of 50, top-8: integer-hashed values (no RNG state to depend on)."""
    i = np.arange(4 * 50, dtype=np.uint64)
    x = ((i * np.uint64(2654435761)) % np.uint64(1000003)).astype(np.float64) / 1000003.0
    logits = ((x - 0.5) * 12.0).astype(np.float32).reshape(4, 50)
    tokens = [3, 17, 42, 8, 29, 11]
    order = np.argsort(-logits, axis=1, kind="stable")[:, :8]
    vals = np.take_along_axis(logits, order, axis=1)
    m = logits.astype(np.float64).max(axis=1)
    lse = (m + np.log(np.exp(logits.astype(np.float64) - m[:, None]).sum(axis=1))).astype(np.float32)
    return tokens, logits, order.astype(np.int32), vals, lse


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else None
    path = os.path.join(ref_root or "", "tools", "quality.py")
    if not os.path.isfile(path):
        raise SystemExit("usage: make_logits_golden.py <reference checkout>")
    spec = importlib.util.spec_from_file_location("ref_quality", path)
    q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(q)
    tokens, logits, ids, vals, lse = inputs()
    q.write_dump(os.path.join(HERE, "dump_full.logits"), tokens, rows=[list(map(float, r)) for r in logits], first_pos=2, n_vocab=50)
    topk_rows = [(float(lse[r]), [int(v) for v in ids[r]], [float(v) for v in vals[r]]) for r in range(4)]
    q.write_dump(os.path.join(HERE, "dump_topk.logits"), tokens, topk_rows=topk_rows, k=8, first_pos=2, n_vocab=50)
    print("wrote dump_full.logits, dump_topk.logits")


if __name__ == "__main__":
    main()
