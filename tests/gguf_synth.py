"""A GGUF (v3) writer for the tests: typed metadata, tensors laid out at aligned offsets, optional splits.  Follows the
published container layout (magic, version, tensor count, metadata count, metadata, tensor infos, aligned data)."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _s(x):
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def _val(t, v):
    if t == STR:
        return _s(v)
    if t == ARR:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_val(et, i) for i in items)
    return struct.pack(_FMT[t], v)


def write(path, kvs, tensors, align=32, write_align_key=True):
    """kvs: list of (key, type, value) (ARR value = (element type, items)); tensors: list of (name, ggml type id, ne
    list in ggml order, bytes).  Returns {name: absolute offset}."""
    kvs = list(kvs)
    if write_align_key:
        kvs.append(("general.alignment", U32, align))
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kvs))
    for k, t, v in kvs:
        head += _s(k) + struct.pack("<I", t) + _val(t, v)
    rel, infos, cur = {}, b"", 0
    for name, gt, ne, data in tensors:
        rel[name] = cur
        infos += _s(name) + struct.pack("<I", len(ne)) + b"".join(struct.pack("<Q", d) for d in ne) + struct.pack("<IQ", gt, cur)
        cur = (cur + len(data) + align - 1) // align * align
    head += infos
    data_off = (len(head) + align - 1) // align * align
    with open(path, "wb") as f:
        f.write(head + b"\0" * (data_off - len(head)))
        for name, gt, ne, data in tensors:
            f.seek(data_off + rel[name])
            f.write(bytes(data))
        end = data_off + cur
        f.truncate(max(end, f.tell()))
    return {n: data_off + o for n, o in rel.items()}
