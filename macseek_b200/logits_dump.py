"""The reference's logits dump files (".logits", format v1, docs/modules/oracle.md:49-59; writer in the reference's app
layer src/app/model_cmds.mm:29-35, reader tools/quality.py): what a run writes so that the reference's quality tool can
compare it with another engine's dump.

  char magic[4] = "MSLG"; u32 version = 1; u32 n_tokens; u32 n_vocab; u32 mode (0 full, 1 top-k); u32 k;
  u32 first_pos; u32 n_pos;                                  -- 32-byte header, little-endian
  i32 tokens[n_tokens]
  mode 0: f32 logits[n_pos][n_vocab]                         -- row r = logits after token first_pos + r
  mode 1: per position { f32 lse; f32 pad; i32 ids[k]; f32 logits[k] }   -- ids by descending logit, lse over the FULL row

The top-k form is exactly what arch.encode_sample_topk produces per position (temperature 1).
"""
import struct

import numpy as np

MAGIC = b"MSLG"
VERSION = 1


def write_full(path, tokens, logits, first_pos=0):
    """logits: array [n_pos][n_vocab] (any float type; stored as f32)."""
    lg = np.ascontiguousarray(np.asarray(logits, dtype="<f4"))
    if lg.ndim != 2:
        raise ValueError("logits must be [n_pos][n_vocab]")
    tk = np.ascontiguousarray(np.asarray(tokens, dtype="<i4")).reshape(-1)
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<7I", VERSION, tk.size, lg.shape[1], 0, 0, first_pos, lg.shape[0]))
        f.write(tk.tobytes())
        f.write(lg.tobytes())


def write_topk(path, tokens, n_vocab, ids, vals, lse, first_pos=0):
    """ids int [n_pos][k] (descending logit), vals float [n_pos][k], lse float [n_pos] (log-sum-exp of the full row)."""
    ids = np.ascontiguousarray(np.asarray(ids, dtype="<i4"))
    vals = np.ascontiguousarray(np.asarray(vals, dtype="<f4"))
    lse = np.asarray(lse, dtype="<f4").reshape(-1)
    if ids.ndim != 2 or ids.shape != vals.shape or lse.size != ids.shape[0]:
        raise ValueError("ids / vals must be [n_pos][k] and lse [n_pos]")
    tk = np.ascontiguousarray(np.asarray(tokens, dtype="<i4")).reshape(-1)
    n_pos, k = ids.shape
    with open(path, "wb") as f:
        f.write(MAGIC + struct.pack("<7I", VERSION, tk.size, n_vocab, 1, k, first_pos, n_pos))
        f.write(tk.tobytes())
        for r in range(n_pos):
            f.write(struct.pack("<ff", float(lse[r]), 0.0))
            f.write(ids[r].tobytes())
            f.write(vals[r].tobytes())


def read(path):
    """-> dict(n_vocab, mode, k, first_pos, tokens, and logits [n_pos][n_vocab] (mode 0) or ids / vals / lse (mode 1))."""
    with open(path, "rb") as f:
        b = f.read()
    if b[:4] != MAGIC:
        raise ValueError("not a logits dump")
    version, n_tokens, n_vocab, mode, k, first_pos, n_pos = struct.unpack_from("<7I", b, 4)
    if version != VERSION:
        raise ValueError("unsupported dump version %d" % version)
    off = 32
    tokens = np.frombuffer(b, "<i4", n_tokens, off)
    off += 4 * n_tokens
    out = {"n_vocab": n_vocab, "mode": mode, "k": k, "first_pos": first_pos, "tokens": tokens}
    if mode == 0:
        out["logits"] = np.frombuffer(b, "<f4", n_pos * n_vocab, off).reshape(n_pos, n_vocab)
    else:
        rec = np.frombuffer(b, np.dtype([("lse", "<f4"), ("pad", "<f4"), ("ids", "<i4", (k,)), ("vals", "<f4", (k,))]), n_pos, off)
        out["lse"], out["ids"], out["vals"] = rec["lse"].copy(), rec["ids"].copy(), rec["vals"].copy()
    return out
