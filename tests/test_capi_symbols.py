"""The shared library loads and exports every symbol that include/macseek_b200.h declares (no compute calls)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    ge.build()
    return ctypes.CDLL(os.path.join(ROOT, "macseek_b200", "libmacseek_b200.so"))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "macseek_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msb_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), n


def test_geometry_and_argument_errors(lib):
    lib.msb_row_bytes.restype = ctypes.c_size_t
    lib.msb_row_bytes.argtypes = [ctypes.c_int, ctypes.c_int64]
    lib.msb_last_error.restype = ctypes.c_char_p
    assert lib.msb_row_bytes(19, 4096) == 800 and lib.msb_row_bytes(16, 4096) == 1056
    assert lib.msb_row_bytes(14, 4096) == 3360 and lib.msb_row_bytes(8, 4096) == 4352
    assert lib.msb_block_elems(20) == 32 and lib.msb_block_elems(30) == 1
    # argument checks happen before any CUDA call
    lib.msb_matvec.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                               ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    assert lib.msb_matvec(19, None, 8, 100, None, None, 0, 1, None) == -1      # cols not a multiple of 256
    assert b"bad shape" in lib.msb_last_error()
    assert lib.msb_matvec(99, None, 8, 256, None, None, 0, 1, None) == -2      # unknown type
