"""The C++ host shim (include/ms_b200_shim.hpp: the reference's ms::q / ms::arch / ms::attn call surface over the C
ABI) compiles as plain C++17 and links against the library without a GPU."""
import os
import subprocess
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SRC = r'''
#include "ms_b200_dec_layer.hpp"
int main(int argc, char**) {
  ms::Enc e;
  ms::Buffer W, x, y;
  if (argc > 100) {   // never executed: the calls only have to compile and link
    ms::q::encode_matvec(e, ms::q::QType::IQ1_S, W, 8, 256, x, y);
    ms::q::encode_matvec_n(e, ms::q::QType::Q6_K, W, 8, 256, x, y, 4);
    ms::q::MoeDecodeArgs a;
    ms::q::encode_moe_decode(e, a);
    ms::arch::Scratch s;
    ms::arch::encode_router_fused(e, x, W, x, y, y, s);
    ms::attn::DecodeCaches c;
    ms::attn::encode_index_decode(e, c, x, x, 10, 5);
    ms::attn::encode_sparse(e, c, x, x, y, 10);
    // the reference's own signatures over attn::State (src/kernels/attn.hpp:116-129)
    ms::attn::State st;
    ms::attn::init(st, ms::attn::Options{});
    ms::attn::encode_kv_window(e, st, 3, x, x, 10, 1);
    ms::attn::encode_index_decode(e, st, 2, x, x, 10);
    ms::attn::encode_sparse(e, st, 3, x, x, y, 10, 1, true);
    ms::attn::LayerIO io;
    ms::attn::encode_layer(e, st, io, 10, 1);
    // the layer-forward surface (src/model/dec_layer.hpp:107-118)
    ms::ds41::DecCtx ctx;
    ms::ds41::encode_dec_prologue(e, ctx, x);
    ms::ds41::encode_dec_attn_side(e, ctx, 0, 10);
    ms::ds41::encode_dec_moe_table(e, ctx, 0, ms::q::QType::IQ1_S, ms::q::QType::IQ2_XXS, x);
    e.wait();
  }
  return ms::q::row_bytes(ms::q::QType::IQ1_S, 4096) == 800 ? 0 : 1;
}
'''


def test_shim_compiles_and_links():
    import __graft_entry__ as ge
    ge.build()
    lib_dir = os.path.join(ROOT, "macseek_b200")
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "t.cpp")
        exe = os.path.join(d, "t")
        open(src, "w").write(SRC)
        subprocess.check_call(["g++", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "include"), src, "-o", exe,
                               "-L", lib_dir, "-lmacseek_b200", "-Wl,-rpath," + lib_dir, "-L/usr/local/cuda/lib64",
                               "-Wl,-rpath,/usr/local/cuda/lib64"])
        assert subprocess.call([exe]) == 0
