// Drives include/ms_b200_gguf.hpp (and, built with -DWITH_SHARD, include/ms_b200_expert_shard.hpp) for the tests.
//   gguf_exec parse <file>                      -> the tensor table and every metadata value as text
//   gguf_exec splits <path>                     -> what expand_splits makes of a path
//   gguf_exec typebytes <type id> <elements>    -> type name and byte size
//   gguf_exec shard <file> <rank> <world> <in> <out>
//       loads this rank's experts of every layer to the GPU and, per layer, runs the MoE decode kernels over the routed
//       experts resident here (no shared expert) on the x / ids / weights of <in>; <out> = f32 [n_layers][dim] partials.
//       <in>: i32 k, then per layer { i32 ids[k]; f32 w[k] }, then f32 x[dim].
#include <cinttypes>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#ifdef WITH_SHARD
#include "ms_b200_expert_shard.hpp"
#else
#include "ms_b200_gguf.hpp"
#endif

using namespace ms;

static void print_value(const KvValue& v, int depth = 0) {
  switch (v.type) {
    case KvType::STR: std::printf("str:%s", v.s.c_str()); break;
    case KvType::F32: case KvType::F64: std::printf("f:%.9g", v.f); break;
    case KvType::BOOL: std::printf("bool:%d", (int)v.u); break;
    case KvType::ARR:
      std::printf("arr[%zu]:", v.size());
      for (size_t k = 0; k < v.ai.size(); k++) std::printf("%s%" PRId64, k ? "," : "", v.ai[k]);
      for (size_t k = 0; k < v.af.size(); k++) std::printf("%s%.9g", k ? "," : "", v.af[k]);
      for (size_t k = 0; k < v.as.size(); k++) std::printf("%s%s", k ? "," : "", v.as[k].c_str());
      for (size_t k = 0; k < v.aa.size(); k++) { std::printf("%s(", k ? "," : ""); print_value(v.aa[k], depth + 1); std::printf(")"); }
      break;
    default:
      if (v.type == KvType::U64 || v.type == KvType::U32 || v.type == KvType::U16 || v.type == KvType::U8) std::printf("u:%" PRIu64, v.u);
      else std::printf("i:%" PRId64, v.i);
  }
}

int main(int argc, char** argv) {
  if (argc < 3) return 1;
  try {
    if (!std::strcmp(argv[1], "typebytes")) {      // typebytes <type id> <n elements>
      std::printf("%s %" PRIu64 "\n", type_name((GType)std::atoi(argv[2])), type_bytes((GType)std::atoi(argv[2]), std::strtoull(argv[3], nullptr, 10)));
      return 0;
    }
    if (!std::strcmp(argv[1], "splits")) {
      for (const std::string& p : Gguf::expand_splits(argv[2])) std::printf("%s\n", p.c_str());
      return 0;
    }
    Gguf g{std::string(argv[2])};
    if (!std::strcmp(argv[1], "parse")) {
      std::printf("version %u align %u splits %d tensors %zu\n", g.version(), g.alignment(), g.n_splits(), g.tensors().size());
      for (const TensorInfo& t : g.tensors()) {
        std::printf("T\t%s\t%s\t[", t.name.c_str(), type_name(t.type));
        for (int d = 0; d < t.n_dims; d++) std::printf("%s%" PRId64, d ? ", " : "", t.ne[d]);
        std::printf("]\t%" PRIu64 "\t%s\t%" PRIu64 "\n", t.nbytes, g.basename(t.split).c_str(), t.offset);
      }
      for (const std::string& k : g.keys()) { std::printf("K\t%s\t", k.c_str()); print_value(*g.kv(k)); std::printf("\n"); }
      const ExpertLayout L = ExpertLayout::from_gguf(g);
      for (int l = 0; l < L.n_layers; l++)
        for (int k = 0; k < 3; k++)
          std::printf("E\t%d\t%d\t%d\t%" PRIu64 "\t%" PRIu64 "\t%u\t%s\n", l, k, L.layers[l].mat[k].split, L.layers[l].mat[k].base,
                      L.layers[l].mat[k].stride, L.layers[l].mat[k].len, type_name(L.layers[l].mat[k].type));
      return 0;
    }
#ifdef WITH_SHARD
    if (!std::strcmp(argv[1], "shard") && argc >= 7) {
      const int rank = std::atoi(argv[3]), world = std::atoi(argv[4]);
      const ExpertLayout L = ExpertLayout::from_gguf(g);
      ExpertShard S = ExpertShard::load(g, L, rank, world, (size_t)1 << 16);     // small chunks: several per matrix
      FILE* in = std::fopen(argv[5], "rb");
      if (!in) return 2;
      int k = 0;
      if (std::fread(&k, 4, 1, in) != 1) return 2;
      std::vector<int> ids((size_t)L.n_layers * k);
      std::vector<float> w((size_t)L.n_layers * k);
      for (int l = 0; l < L.n_layers; l++)
        if (std::fread(&ids[(size_t)l * k], 4, k, in) != (size_t)k || std::fread(&w[(size_t)l * k], 4, k, in) != (size_t)k) return 2;
      const int dim = S.layers[0].dim, inter = S.layers[0].inter;
      std::vector<float> x((size_t)dim);
      if (std::fread(x.data(), 4, dim, in) != (size_t)dim) return 2;
      std::fclose(in);
      Device& dev = Device::get();
      Buffer dx = dev.alloc((size_t)dim * 4), dy = dev.alloc((size_t)dim * 4), dids = dev.alloc((size_t)k * 4), dw = dev.alloc((size_t)k * 4);
      Buffer scratch = dev.alloc(q::moe_decode_scratch_bytes(inter, k));
      upload(dx, x.data(), x.size() * 4);
      FILE* out = std::fopen(argv[6], "wb");
      std::vector<float> y((size_t)dim);
      Enc e;
      for (int l = 0; l < L.n_layers; l++) {
        upload(dids, &ids[(size_t)l * k], (size_t)k * 4);
        upload(dw, &w[(size_t)l * k], (size_t)k * 4);
        check(msb_fill_f32((float*)dy.ptr(), 0.f, (size_t)dim, nullptr), "fill");
        q::MoeDecodeArgs a;
        a.dim = dim; a.inter = inter; a.t_gate_up = S.layers[l].t_gate_up; a.t_down = S.layers[l].t_down;
        a.n_routed = k; a.has_shared = false; a.weights = dw; a.x = dx; a.y = dy; a.scratch = scratch;
        q::encode_moe_decode_ids(e, a, S.layers[l].table, dids, S.expert_lo, S.expert_hi);
        e.wait();
        download(y.data(), dy, y.size() * 4);
        std::fwrite(y.data(), 4, y.size(), out);
      }
      std::fclose(out);
      std::printf("shard rank %d/%d experts [%d, %d) %" PRIu64 " device bytes\n", rank, world, S.expert_lo, S.expert_hi, S.bytes);
      S.release();
      return 0;
    }
#endif
  } catch (const std::exception& ex) {
    std::fprintf(stderr, "error: %s\n", ex.what());
    return 3;
  }
  return 1;
}
