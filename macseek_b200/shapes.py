"""Type ids, block geometry and the benchmark's shapes as plain Python: nothing here loads the CUDA library, so host-only
tools (the CPU baseline arm of the benchmark, byte models) can import it on a machine without the built library."""
import enum


class QType(enum.IntEnum):
    """ggml type ids (src/kernels/quant_types.hpp:10-12)."""
    F32 = 0
    F16 = 1
    Q8_0 = 8
    Q5_K = 13
    Q6_K = 14
    IQ2_XXS = 16
    IQ1_S = 19
    IQ4_NL = 20
    BF16 = 30


SCORE_SQRT_SOFTPLUS, SCORE_SIGMOID = 0, 1     # router score functions
KEY_F16, KEY_FP8 = 1, 101                     # index-key cache element types
ELEM_F16, ELEM_BF16 = 1, 30                   # KV row element types

# (elements, bytes) of one block (src/kernels/quant_types.hpp:15-34)
BLOCK = {QType.Q8_0: (32, 34), QType.Q5_K: (256, 176), QType.Q6_K: (256, 210), QType.IQ2_XXS: (256, 66),
         QType.IQ1_S: (256, 50), QType.IQ4_NL: (32, 18)}


def row_bytes(t, cols):
    t = QType(t)
    if t == QType.F32:
        return cols * 4
    if t in (QType.F16, QType.BF16):
        return cols * 2
    be, bb = BLOCK[t]
    return cols // be * bb


class DecConfig:
    """Shapes of the synthetic decode step (benchmark configuration: hidden 4096, 43 layers, 64 heads, KV rows of
    512 + 64 rope dims in bf16, 64 x 128 FP8 index heads with top-k 2048 over a 200K KV, 384 experts top-8 + 1 shared,
    expert inter 2048, vocab 129280 with a Q6_K head).  Projection shapes follow the reference's structure
    (tests/dec_synth.hpp:113-132) scaled to this hidden size."""

    def __init__(self, **kw):
        self.dim = 4096
        self.n_layers = 43
        self.heads = 64
        self.D = 576
        self.q_lora = 1280
        self.o_groups = 8
        self.o_a_rows = 8192
        self.window = 128
        self.index_heads = 64
        self.index_dim = 128
        self.topk = 2048
        self.kv_len = 200000
        self.n_experts = 384
        self.top_k = 8
        self.inter = 2048
        self.vocab = 129280
        self.score_fn = SCORE_SIGMOID
        self.route_scale = 1.0
        self.t_attn = QType.Q6_K
        self.t_index = QType.BF16
        self.t_gate_up = QType.IQ1_S
        self.t_down = QType.IQ2_XXS
        self.t_shared = QType.Q8_0
        self.t_head = QType.Q6_K
        self.key_type = KEY_FP8
        self.elem_type = ELEM_BF16
        self.norm_eps = 1e-6
        for k, v in kw.items():
            if not hasattr(self, k):
                raise AttributeError(k)
            setattr(self, k, v)

    # ---- byte model: what one token must read, per layer and for the head
    def layer_bytes(self, local_expert_fraction=1.0):
        rb = row_bytes
        hD = self.heads * self.D
        attn_w = (rb(self.t_attn, self.dim) * (self.q_lora + self.D) + rb(self.t_attn, self.q_lora) * hD
                  + rb(self.t_attn, hD // self.o_groups) * self.o_a_rows + rb(self.t_attn, self.o_a_rows) * self.dim)
        idx_w = rb(self.t_index, self.dim) * self.index_heads + rb(self.t_index, self.q_lora) * self.index_heads * self.index_dim
        keys = self.kv_len * self.index_dim * (1 if self.key_type == KEY_FP8 else 2)
        rows = (self.window + self.topk) * self.D * 2
        expert = 2 * rb(self.t_gate_up, self.dim) * self.inter + rb(self.t_down, self.inter) * self.dim
        shared = 2 * rb(self.t_shared, self.dim) * self.inter + rb(self.t_shared, self.inter) * self.dim
        router = self.n_experts * self.dim * 4
        # under expert parallelism the routed experts AND the shared expert's rows are split over the ranks
        moe = int((self.top_k * expert + shared) * local_expert_fraction) + router
        return {"attn_weights": attn_w, "index_weights": idx_w, "index_keys": keys, "kv_rows": rows, "moe": moe,
                "total": attn_w + idx_w + keys + rows + moe}

    def head_bytes(self):
        return row_bytes(self.t_head, self.dim) * self.vocab
