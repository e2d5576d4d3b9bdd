"""Per-kernel timing of the decode path's kernels, outside the full decode step.

    python kernel_bench.py matvec Q6_K 129280 4096 [--n 1] [--groups 1]
    python kernel_bench.py moe {router|gu|down|all}
    python kernel_bench.py attn {index|scores|topk|sparse|all} [--kv-len 200000]
    python kernel_bench.py gemm Q6_K 4096 4096 --n 4096
    python kernel_bench.py moe_prefill [--n 4096] [--routing bias|sample]
    torchrun --nproc-per-node N kernel_bench.py moe_prefill_ep     # the same layer expert-parallel, checked against one GPU
    python kernel_bench.py hc               # hyper-connection step and KV compressor
    python kernel_bench.py layer            # cost added by each call of the decode layer, in context
    python kernel_bench.py sweep

Each case builds synthetic weights on the device (several copies, together larger than the 126 MB L2, used in
rotation), records 20 launches into one CUDA graph and times graph replays with CUDA events on the replaying
stream, so that the host's launch cost is not part of the figure.  ``--eager K`` instead issues K plain launches
and exits: the form to put under a profiler, which should see few launches.
"""
from __future__ import annotations

import argparse

import torch

from macseek_b200 import _lib, arch, attn, moe_layer as ml, quant as q, synthetic
from macseek_b200.core import Enc, ptr


def graph_time(fn, n_in_graph: int = 20, reps: int = 10):
    """Median and minimum time (microseconds) of one call of ``fn(i)`` inside a replayed CUDA graph."""
    fn(0)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(n_in_graph):
                fn(i)
        for _ in range(3):
            g.replay()
        s.synchronize()
        ts = []
        for _ in range(reps):
            a = torch.cuda.Event(enable_timing=True)
            b = torch.cuda.Event(enable_timing=True)
            a.record(s)
            g.replay()
            b.record(s)
            s.synchronize()
            ts.append(a.elapsed_time(b) * 1e3 / n_in_graph)
    ts.sort()
    return ts[len(ts) // 2], ts[0]


def run(fn, eager: int):
    if eager:
        for i in range(eager):
            fn(i)
        torch.cuda.synchronize()
        return None
    return graph_time(fn)


def matvec_case(t: q.QType, rows: int, cols: int, n: int = 1, groups: int = 1, eager: int = 0, quiet: bool = False):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(2)
    nbytes = synthetic.row_bytes(t, cols) * rows
    copies = min(max(2, int(600e6 // nbytes)), 20)
    Ws = [synthetic.random_weights(t, rows, cols, gen) for _ in range(copies)]
    x = torch.randn(n, cols * groups, device="cuda")
    y = torch.zeros(n, rows, device="cuda")

    def f(i):
        e = Enc()
        if n == 1:
            q.encode_matvec(e, t, Ws[i % copies], rows, cols, x, y, False, groups)
        else:
            q.encode_matvec_n(e, t, Ws[i % copies], rows, cols, x, y, n, False, groups)

    r = run(f, eager)
    if r and not quiet:
        print(f"matvec {t.name:8s} {rows:6d}x{cols:6d} n={n} g={groups} median {r[0]:8.2f} us min {r[1]:8.2f}"
              f"  {nbytes / r[0] / 1e3:8.1f} GB/s  ({nbytes / 1e6:.1f} MB x{copies})", flush=True)
    if r:
        return {"type": t.name, "rows": rows, "cols": cols, "batch": n, "us": r[0], "bytes": nbytes,
                "gbs": nbytes / r[0] / 1e3, "weight_copies": copies}


def moe_cases(which: str, eager: int = 0, quiet: bool = False):
    """The benchmark MoE layer: 8 of 384 routed experts (IQ1_S gate/up, IQ2_XXS down) + Q8_0 shared expert."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    L = 4
    layers = [ml.MoeLayerWeights(4096, 2048, 384, q.QType.IQ1_S, q.QType.IQ2_XXS, q.QType.Q8_0).randomize(gen)
              for _ in range(L)]
    bufs = ml.MoeLayerBufs(4096, 2048, 384, 8)
    xs = [torch.randn(4096, device="cuda", generator=gen) for _ in range(16)]
    y = torch.zeros(4096, device="cuda")
    idsets = [torch.randperm(384, device="cuda", generator=gen)[:8].int().contiguous() for _ in range(20)]
    bufs.w.fill_(0.125)

    def mk(part):
        def f(i):
            e = Enc()
            lw = layers[i % L]
            a = q.MoeDecodeArgs(4096, 2048)
            a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
            a.n_routed, a.has_shared, a.shared = 8, True, lw.shared
            a.weights, a.x, a.y, a.scratch = bufs.w, xs[i % 16], y, bufs.moe_scratch
            q.encode_moe_decode_ids(e, a, lw.table, idsets[i % 20], 0, 384, part)
        return f

    def router(i):
        e = Enc()
        lw = layers[i % L]
        arch.encode_router_fused(e, xs[i % 16], lw.router_w, lw.router_bias, bufs.ids, bufs.w, bufs.router_scratch,
                                 8, 1, 1.0)

    iq1 = synthetic.row_bytes(q.QType.IQ1_S, 4096) * 2048
    iq2 = synthetic.row_bytes(q.QType.IQ2_XXS, 2048) * 4096
    q8a = synthetic.row_bytes(q.QType.Q8_0, 4096) * 2048
    q8b = synthetic.row_bytes(q.QType.Q8_0, 2048) * 4096
    gu_bytes = 8 * 2 * iq1 + 2 * q8a
    d_bytes = 8 * iq2 + q8b
    cases = {"router": (router, 384 * 4096 * 4), "gu": (mk(q.MoePart.GuAll), gu_bytes),
             "down": (mk(q.MoePart.DownAll), d_bytes), "all": (mk(q.MoePart.All), gu_bytes + d_bytes)}
    out = {}
    for name in (cases if which == "every" else [which]):
        fn, nbytes = cases[name]
        r = run(fn, eager)
        if r:
            out[name] = {"us": r[0], "bytes": nbytes, "gbs": nbytes / r[0] / 1e3}
            if not quiet:
                print(f"moe {name:8s} median {r[0]:8.2f} us  min {r[1]:8.2f} us   {nbytes / r[0] / 1e3:8.1f} GB/s",
                      flush=True)
    return out


def attn_cases(which: str, kv_len: int = 200000, eager: int = 0):
    """The benchmark attention side: 64 x 128 FP8 index heads over kv_len keys, exact top-2048, sparse attention of 64
    heads over 128 window rows + the 2048 selected rows of 576 bf16.  Six KV sources are used in rotation so that the
    keys (25.6 MB per source at 200K) come from HBM, not from L2."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    sh = attn.Shape.benchmark()
    rope = torch.from_numpy(attn.make_rope_table(kv_len + 1, True)).cuda()
    states = []
    for _ in range(6):
        st = attn.DecodeState(sh, kv_len, rope, "cuda")
        st.ckv.normal_(0, 1, generator=gen)
        st.win.normal_(0, 1, generator=gen)
        tmp = torch.empty(st.ikey.shape, dtype=torch.bfloat16, device="cuda").normal_(0, 1, generator=gen)
        st.ikey.copy_(tmp.to(torch.float8_e4m3fn).view(torch.uint8))
        states.append(st)
    iq = torch.randn(sh.index_heads * sh.index_dim, device="cuda", generator=gen)
    iw = torch.randn(sh.index_heads, device="cuda", generator=gen)
    qf = torch.randn(sh.heads * sh.D, device="cuda", generator=gen)
    sinks = torch.randn(sh.heads, device="cuda", generator=gen)
    out = torch.zeros(sh.heads * sh.D, device="cuda")
    pos = kv_len - 1
    for st in states:                      # a valid top-k list and scores in every source
        attn.encode_index_decode(Enc(), st, iq, iw, pos, kv_len, actq=False)
    torch.cuda.synchronize()

    def index(i):
        attn.encode_index_decode(Enc(), states[i % 6], iq, iw, pos, kv_len, actq=False)

    def scores(i):
        st = states[i % 6]
        _lib.check(_lib.lib.msb_index_scores(sh.key_type, ptr(st.ikey), kv_len, ptr(st.q_prep), ptr(st.w_prep),
                                             sh.index_heads, ptr(st.dec_scores), None, 0,
                                             torch.cuda.current_stream().cuda_stream))

    def topk(i):
        st = states[i % 6]
        attn.encode_topk(Enc(), st.dec_scores, kv_len, sh.topk, st.topk, st.topk_scratch)

    def sparse(i):
        attn.encode_sparse(Enc(), states[i % 6], qf, sinks, out, pos)

    key_bytes = kv_len * sh.index_dim
    cases = {"index": (index, key_bytes), "scores": (scores, key_bytes), "topk": (topk, kv_len * 4),
             "sparse": (sparse, (sh.window + sh.topk) * sh.D * 2)}
    for name in (cases if which in ("every", "all") else [which]):
        fn, nbytes = cases[name]
        r = run(fn, eager)
        if r:
            print(f"attn {name:8s} median {r[0]:8.2f} us  min {r[1]:8.2f} us   {nbytes / r[0] / 1e3:8.1f} GB/s",
                  flush=True)


def gemm_case(t: q.QType, rows: int, cols: int, n: int, eager: int = 0):
    """Prefill projection Y[n x rows] = X[n x cols] . W^T: the contraction alone (half weights given) and the whole
    call (weight dequantisation to half + contraction)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(4)
    W = synthetic.random_weights(t, rows, cols, gen)
    W16 = synthetic.random_weights(q.QType.F16, rows, cols, gen)
    X16 = torch.randn(n, cols, device="cuda", generator=gen).half()
    Y = torch.zeros(n, rows, device="cuda")
    scratch = torch.zeros(q.matmul_scratch_bytes(t, rows, cols, n, False), dtype=torch.uint8, device="cuda")
    flop = 2.0 * n * rows * cols

    def dense(i):
        q.encode_matmul_h(Enc(), q.QType.F16, W16, rows, cols, X16, Y, n, False, 0, None)

    def whole(i):
        q.encode_matmul_h(Enc(), t, W, rows, cols, X16, Y, n, False, 0, scratch)

    for name, fn in (("contraction (F16 weights)", dense), ("dequant + contraction (%s)" % t.name, whole)):
        r = run(fn, eager) if eager else graph_time(fn, 4, 5)
        if r:
            print(f"gemm {n}x{rows}x{cols} {name:34s} median {r[0]:9.2f} us   {flop / r[0] / 1e6:8.1f} TFLOP/s", flush=True)


def moe_prefill_case(n: int = 4096, eager: int = 0, routing: str = "bias", quiet: bool = False):
    """The benchmark prefill layer: n tokens, top-8 of 384 experts (IQ1_S gate/up, IQ2_XXS down) + Q8_0 shared expert,
    dim 4096, inter 2048.  routing "bias": logits N(0,1) plus a log-Zipf(1.1) popularity bias over a seeded expert
    permutation (a few experts take most tokens); "sample": top-k drawn without replacement from Zipf(0.8)
    popularities, as the reference's own bench does (bench/qmatmul.mm:135-152: every expert gets some tokens)."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    D, I, E, K = 4096, 2048, 384, 8
    lw = ml.MoeLayerWeights(D, I, E, q.QType.IQ1_S, q.QType.IQ2_XXS, q.QType.Q8_0).randomize(gen)
    perm = torch.randperm(E, device="cuda", generator=gen)
    bias = torch.empty(E, device="cuda")
    bias[perm] = -1.1 * torch.log(torch.arange(1, E + 1, device="cuda", dtype=torch.float32))
    logits = torch.randn(n, E, device="cuda", generator=gen) + bias
    if routing == "sample":
        pw = torch.empty(E, device="cuda")
        pw[perm] = torch.arange(1, E + 1, device="cuda", dtype=torch.float32).pow(-0.8)
        ids = torch.multinomial(pw.expand(n, E), K, replacement=False, generator=gen)
    else:
        ids = torch.topk(logits, K, dim=1).indices                               # [n][K]
    w = torch.softmax(torch.gather(logits, 1, ids), dim=1).float()
    flat_e = ids.reshape(-1)
    order = torch.argsort(flat_e, stable=True)                                   # entries sorted by (expert, token*K+k)
    tok = (order // K).int().contiguous()
    wt = w.reshape(-1)[order].contiguous()
    slot_of = torch.empty(n * K, dtype=torch.int32, device="cuda")
    slot_of[order] = torch.arange(n * K, dtype=torch.int32, device="cuda")
    counts = torch.bincount(flat_e, minlength=E).cpu().tolist()
    used = [e for e in range(E) if counts[e] > 0]
    offs = [0]
    for e in used:
        offs.append(offs[-1] + counts[e])

    def slot_of_expert(ex):
        sl = q.ExpertSlot()
        sl.gate, sl.up, sl.down = lw.expert_views(ex)
        return sl
    a = q.MoePrefillArgs(D, I)
    a.t_gate_up, a.t_down, a.t_shared = lw.t_gate_up, lw.t_down, lw.t_shared
    a.n_tokens, a.k_per_token, a.has_shared = n, K, True
    a.slots = [slot_of_expert(ex) for ex in used]
    a.shared = lw.shared
    a.offs = offs
    a.tok, a.wt, a.slot_of = tok, wt, slot_of
    a.X = torch.randn(n, D, device="cuda", generator=gen)
    a.Y = torch.zeros(n, D, device="cuda")
    a.scratch = torch.zeros(q.moe_prefill_scratch_bytes(offs[-1], n, len(used), D, I), dtype=torch.uint8, device="cuda")
    cs = sorted(counts)
    if not quiet:
        print(f"moe_prefill n={n} routing={routing}: {len(used)} experts hit, tokens/expert min {cs[0]} median {cs[len(cs) // 2]} max {cs[-1]}", flush=True)
    e = Enc()
    for _ in range(2):
        q.encode_moe_prefill(e, a)
    e.wait()
    if eager:
        return
    ts = []
    for _ in range(5):
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        q.encode_moe_prefill(e, a)
        t1.record()
        torch.cuda.synchronize()
        ts.append(t0.elapsed_time(t1))
    ts.sort()
    flop = 2.0 * 3 * D * I * (n * K + n)
    if not quiet:
        print(f"moe_prefill n={n} median {ts[2]:8.3f} ms   {flop / ts[2] / 1e9:8.1f} TFLOP/s (algorithmic 2*3*D*I*(entries+tokens))",
              flush=True)
    return {"tokens": n, "routing": routing, "ms": ts[2], "flop": flop, "tflops": flop / ts[2] / 1e9,
            "experts_hit": len(used), "tokens_per_expert": {"min": cs[0], "median": cs[len(cs) // 2], "max": cs[-1]}}


def moe_prefill_ep_case(n: int = 4096, check: bool = True, quiet: bool = False):
    """The benchmark prefill layer expert-parallel (run under torchrun, one rank per GPU): tokens sharded n / N per rank,
    experts 384 / N per rank, all-to-all dispatch of bf16 rows and all-to-all combine of f32 expert outputs.  With
    check, every rank also holds the whole layer and computes the single-GPU result for ITS tokens to compare with."""
    import torch.distributed as dist
    from macseek_b200 import ep, ep_prefill
    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    D, I, E, K = 4096, 2048, 384, 8
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)                                     # the same routing, inputs and replicated weights on every rank
    lo, hi = ep.expert_range(E, world, rank)
    lw = ml.MoeLayerWeights(D, I, E, q.QType.IQ1_S, q.QType.IQ2_XXS, q.QType.Q8_0, lo, hi, dev).randomize(gen, expert_seed=99)
    perm = torch.randperm(E, device=dev, generator=gen)
    bias = torch.empty(E, device=dev)
    bias[perm] = -1.1 * torch.log(torch.arange(1, E + 1, device=dev, dtype=torch.float32))
    logits = torch.randn(n, E, device=dev, generator=gen) + bias
    ids = torch.topk(logits, K, dim=1).indices
    w = torch.softmax(torch.gather(logits, 1, ids), dim=1).float()
    X = torch.randn(n, D, device=dev, generator=gen).to(torch.bfloat16).float()
    per = n // world
    sl = slice(rank * per, (rank + 1) * per)
    e = Enc()
    run_local, run_shared = ep_prefill.cuda_local_experts(lw, e), ep_prefill.cuda_shared_expert(lw, e)
    stats = {}

    def step():
        Y = torch.zeros(per, D, device=dev)
        ep_prefill.moe_prefill_ep(X[sl], ids[sl], w[sl], E, run_local, run_shared, Y, stats=stats)
        return Y
    Y = step()
    torch.cuda.synchronize()
    ts = []
    for _ in range(3):
        dist.barrier()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        Y = step()
        t1.record()
        torch.cuda.synchronize()
        ts.append(t0.elapsed_time(t1))
    t = torch.tensor([sorted(ts)[1]], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    rows = [None] * world
    dist.all_gather_object(rows, stats["rows_received"])
    out = {"tokens": n, "world": world, "ms": float(t.item()), "rows_received_per_rank": rows,
           "flop": 2.0 * 3 * D * I * (n * K + n)}
    out["tflops"] = out["flop"] / out["ms"] / 1e9
    if check:
        # the whole layer on this rank (experts seeded by global id: the same bytes), this rank's tokens, one GPU
        full = ml.MoeLayerWeights(D, I, E, q.QType.IQ1_S, q.QType.IQ2_XXS, q.QType.Q8_0, 0, E, dev)
        g2 = torch.Generator(device=dev)
        g2.manual_seed(7)
        full.randomize(g2, expert_seed=99)
        Xl, il, wl = X[sl].contiguous(), ids[sl], w[sl]
        flat_e = il.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        counts = torch.bincount(flat_e, minlength=E).cpu().tolist()
        used = [x for x in range(E) if counts[x] > 0]
        a = q.MoePrefillArgs(D, I)
        a.t_gate_up, a.t_down, a.t_shared = full.t_gate_up, full.t_down, full.t_shared
        a.n_tokens, a.k_per_token, a.has_shared, a.shared = per, K, True, full.shared
        offs = [0]
        for ex in used:
            sl_ = q.ExpertSlot()
            sl_.gate, sl_.up, sl_.down = full.expert_views(ex)
            a.slots.append(sl_)
            offs.append(offs[-1] + counts[ex])
        a.offs = offs
        a.tok = (order // K).int().contiguous()
        a.wt = wl.reshape(-1)[order].contiguous()
        a.slot_of = torch.empty(per * K, dtype=torch.int32, device=dev)
        a.slot_of[order] = torch.arange(per * K, dtype=torch.int32, device=dev)
        a.X, a.Y = Xl, torch.zeros(per, D, device=dev)
        a.scratch = torch.zeros(q.moe_prefill_scratch_bytes(offs[-1], per, len(used), D, I), dtype=torch.uint8, device=dev)
        q.encode_moe_prefill(e, a)
        e.wait()
        rel = float((Y - a.Y).abs().max() / a.Y.abs().max())
        r = torch.tensor([rel], dtype=torch.float64, device=dev)
        dist.all_reduce(r, op=dist.ReduceOp.MAX)
        out["max_rel_diff_vs_single_gpu"] = float(r.item())
        out["matches_single_gpu"] = bool(r.item() <= 1e-3)
        del full
    if rank == 0 and not quiet:
        print("moe_prefill_ep", out, flush=True)
    return out


def hc_cases():
    """What the reference's real layer runs besides the benchmark step's calls: the hyper-connection step (twice per
    layer: before the attention side and before the FFN side) and, on KV source layers, the compressor + index key.
    Timed as graphs of 20 dependent launches at the benchmark's hidden size."""
    from macseek_b200 import dec_layer as dl
    D = 4096
    gen = torch.Generator(device="cuda")
    gen.manual_seed(3)
    rnd = lambda *shape, s=1.0: torch.empty(*shape, device="cuda").normal_(0, s, generator=gen)
    h, x_sub, x_out = rnd(4 * D), rnd(D), torch.zeros(D, device="cuda")
    fns = [rnd(24 * 4 * D, s=0.02) for _ in range(8)]                 # 1.5 MB each: rotate so that they come from HBM / L2 in turn
    scale, base, norm_w = torch.tensor([0.7, 1.3, 0.9], device="cuda"), rnd(24), 1 + rnd(D, s=0.1)
    mix_prev, mix_out = rnd(24).abs() + 0.05, torch.zeros(24, device="cuda")
    scratch = arch.hc_scratch(1)

    def hc(i):
        arch.encode_hc_step(Enc(), h, h, x_sub, mix_prev, fns[i % 8], scale, base, mix_out, norm_w, x_out, D, scratch)
    r = graph_time(hc)
    print(f"hc_step dim {D}: median {r[0]:6.2f} us  min {r[1]:6.2f} us per launch", flush=True)
    cfg = dl.DecConfig(n_layers=1, kv_len=4096)
    sh = dl.attn_shape(cfg)
    rope = torch.from_numpy(attn.make_rope_table(4200, True)).cuda()
    st = attn.DecodeState(sh, 4096, rope, "cuda")
    c_kv, c_gate, c_norm = rnd(sh.D), rnd(sh.D), 1 + rnd(sh.D, s=0.1)
    wk = rnd(sh.index_dim * sh.D, s=0.05).to(torch.bfloat16)
    k_norm = 1 + rnd(sh.index_dim, s=0.1)
    for ratio in (1, 2):
        state = torch.zeros(2 * ratio * sh.D, device="cuda")

        def cmp(i, ratio=ratio, state=state):
            attn.encode_compress(Enc(), st, c_kv, c_gate if ratio > 1 else None, c_norm, wk, k_norm, state, ratio, 100 + i, actq=False)
        r = graph_time(cmp)
        print(f"compress ratio {ratio} (row {sh.D}, index key {sh.index_dim}): median {r[0]:6.2f} us  min {r[1]:6.2f} us per launch", flush=True)


def layer_stages(n_layers: int = 8, kv_len: int = 200000):
    """The decode layer in context: CUDA graphs of n_layers layers cut after the first k calls of each layer, k = 1 ..;
    the difference between consecutive cuts is what call k adds per layer with all overlaps as in the real step."""
    from macseek_b200 import dec_layer as dl
    cfg = dl.DecConfig(n_layers=n_layers, kv_len=kv_len)
    model = dl.SyntheticModel(cfg, seed=1234, device=torch.device("cuda", torch.cuda.current_device()))
    limit, count, names = [10 ** 9], [0], []

    def wrap(mod, name):
        f = getattr(mod, name)

        def g(*a, **k):
            count[0] += 1
            if count[0] > limit[0]:
                return None
            if len(names) < count[0]:
                names.append(name)
            return f(*a, **k)
        setattr(mod, name, g)
        return f
    saved = [(mod, nm, wrap(mod, nm)) for mod, nm in (
        (q, "encode_matvec_rmsnorm"), (q, "encode_matvec_rmsnorm_shared"), (q, "encode_matvec"), (attn, "encode_kv_window"), (attn, "encode_index_decode"),
        (attn, "encode_sparse"), (arch, "encode_router_fused_rmsnorm"), (q, "encode_moe_decode_ids"),
        (q, "encode_moe_decode_ids_normed"))]
    stream = torch.cuda.Stream()

    def encode(e):
        for l in range(n_layers):
            count[0] = 0
            model.encode_dec_attn_side(e, l, cfg.kv_len - 1)
            model.encode_dec_moe(e, l)

    def run_cut(lim):
        limit[0] = lim
        with torch.cuda.stream(stream):
            model.bufs.h.normal_(0, 1)
            encode(Enc(stream))
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                encode(Enc(torch.cuda.current_stream()))
            for _ in range(3):
                g.replay()
            stream.synchronize()
            ts = []
            for _ in range(7):
                a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a0.record(stream)
                g.replay()
                a1.record(stream)
                stream.synchronize()
                ts.append(a0.elapsed_time(a1) * 1e3 / n_layers)
            ts.sort()
            return ts[len(ts) // 2]
    try:
        run_cut(10 ** 9)
        prev = 0.0
        for lim in range(1, len(names) + 1):
            t = run_cut(lim)
            print(f"{lim:2d} {names[lim - 1]:28s} cumulative {t:8.2f} us/layer   +{t - prev:7.2f}", flush=True)
            prev = t
    finally:
        for mod, nm, f in saved:
            setattr(mod, nm, f)


def sweep():
    T = q.QType
    moe_cases("every")
    attn_cases("every")
    for t in (T.IQ1_S, T.IQ2_XXS, T.Q8_0, T.Q6_K, T.Q5_K, T.IQ4_NL, T.BF16, T.F32):
        matvec_case(t, 16384, 4096)
    # the decode step's own shapes
    for t, r, c, g in ((T.Q6_K, 1280, 4096, 1), (T.Q6_K, 576, 4096, 1), (T.Q6_K, 36864, 1280, 1),
                       (T.Q6_K, 8192, 4608, 8), (T.Q6_K, 4096, 8192, 1), (T.BF16, 8192, 1280, 1),
                       (T.BF16, 64, 4096, 1), (T.Q6_K, 129280, 4096, 1), (T.Q6_K, 4096, 16384, 1)):
        matvec_case(t, r, c, 1, g)
    matvec_case(T.Q6_K, 16384, 4096, 4)
    matvec_case(T.IQ2_XXS, 16384, 4096, 4)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["matvec", "moe", "attn", "gemm", "moe_prefill", "moe_prefill_ep", "layer", "hc", "sweep"])
    ap.add_argument("args", nargs="*")
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--groups", type=int, default=1)
    ap.add_argument("--kv-len", type=int, default=200000)
    ap.add_argument("--routing", default="bias", choices=["bias", "sample"])
    ap.add_argument("--eager", type=int, default=0, help="issue this many plain launches and exit (no timing)")
    a = ap.parse_args()
    if a.case == "moe_prefill_ep":                      # under torchrun: one rank per GPU
        import os
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
        moe_prefill_ep_case(a.n if a.n > 1 else 4096)
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)
    torch.cuda.set_device(0)
    if a.case == "matvec":
        matvec_case(q.QType[a.args[0]], int(a.args[1]), int(a.args[2]), a.n, a.groups, a.eager)
    elif a.case == "moe":
        moe_cases(a.args[0] if a.args else "every", a.eager)
    elif a.case == "layer":
        layer_stages(8, a.kv_len)
    elif a.case == "hc":
        hc_cases()
    elif a.case == "moe_prefill":
        moe_prefill_case(a.n if a.n > 1 else 4096, a.eager, a.routing)
    elif a.case == "gemm":
        gemm_case(q.QType[a.args[0]], int(a.args[1]), int(a.args[2]), a.n if a.n > 1 else 4096, a.eager)
    elif a.case == "attn":
        attn_cases(a.args[0] if a.args else "every", a.kv_len, a.eager)
    else:
        sweep()
    torch.cuda.synchronize()


if __name__ == "__main__":
    main()
