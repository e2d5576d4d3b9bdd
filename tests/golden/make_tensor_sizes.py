#!/usr/bin/env python3
"""Generate tests/golden/tensor_sizes.json from the reference checkout's docs/tensors.txt (the tensor table of the real
1043-tensor model: name, type, dims, bytes, file, offset): the distinct (type, element count) -> bytes triples, a pin for
the GGUF reader's type-size table on what a real file holds.

Run where the reference checkout is available:   python tests/golden/make_tensor_sizes.py <reference checkout>"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    src = os.path.join(sys.argv[1], "docs", "tensors.txt")
    seen = {}
    for line in open(src):
        col = line.rstrip("\n").split("\t")
        if len(col) != 6:
            continue
        n = 1
        for d in col[2].strip("[]").split(","):
            n *= int(d)
        seen[(col[1], n)] = int(col[3])
    out = sorted([t, n, b] for (t, n), b in seen.items())
    json.dump(out, open(os.path.join(HERE, "tensor_sizes.json"), "w"))
    print(len(out), "distinct (type, elements) pairs")


if __name__ == "__main__":
    main()
