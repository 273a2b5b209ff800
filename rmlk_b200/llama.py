"""Llama-3.2-shaped decoder graphs written as the op sequence an opset-14 ONNX export produces.

Only ops of the reference's operator set are used (schema/src/op.rs:11-51): the token embedding is a
Gather, RMSNorm is Pow -> ReduceMean -> Add -> Sqrt -> Div -> Mul, RoPE tables come from Range / Cast / Pow /
Div / Mul / Concat / Cos / Sin, rotate_half is Slice / Neg / Concat, the causal mask is ConstantOfShape ->
Trilu -> Equal -> Where, grouped-query attention repeats K/V heads with Unsqueeze / Expand / Reshape,
attention is MatMul -> Mul -> Add -> Softmax -> MatMul, the KV cache grows by Concat on axis 2, and SwiGLU is
Sigmoid / Mul / Mul.  Nothing is fused: every line below is one op node executed by its own backend.

Graph inputs and outputs follow the reference's Llama harness (runtime/tests/e2e_ort/llama.rs:210-261):
`input_ids [B,S]`, `attention_mask [B,T]`, `position_ids [B,S]`, `past_key_values.{l}.{key,value}
[B,kv_heads,P,head_dim]` in; `logits [B,S,vocab]`, `present.{l}.{key,value} [B,kv_heads,T,head_dim]` out,
with an empty past (P = 0) on the first step.

Weights are synthetic (seeded normal, std 0.02; norm weights 1): no checkpoint is involved.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from .graphspec import GraphSpec

F32_MIN = float(np.finfo(np.float32).min)


@dataclass
class LlamaConfig:
    hidden: int = 2048
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 64
    ffn: int = 8192
    vocab: int = 128256
    n_layers: int = 16
    rope_theta: float = 500000.0
    rms_eps: float = 1e-5

    @property
    def params(self) -> int:
        per_layer = (2 * self.hidden * self.n_heads * self.head_dim + 2 * self.hidden * self.n_kv_heads * self.head_dim +
                     3 * self.hidden * self.ffn + 2 * self.hidden)
        return self.n_layers * per_layer + self.vocab * self.hidden + self.hidden

    def kv_bytes_per_token(self) -> int:
        return self.n_layers * 2 * self.n_kv_heads * self.head_dim * 4


LLAMA_1B = LlamaConfig()
LLAMA_1B_ONE_LAYER = LlamaConfig(n_layers=1)


def weight_shapes(cfg: LlamaConfig, with_embedding: bool = True):
    """name -> shape of every initializer (all float32)."""
    q = cfg.n_heads * cfg.head_dim
    kv = cfg.n_kv_heads * cfg.head_dim
    s = {}
    if with_embedding:
        s["embed"] = (cfg.vocab, cfg.hidden)
        s["lm_head"] = (cfg.hidden, cfg.vocab)  # the tied embedding, stored transposed for MatMul as exports do
    for l in range(cfg.n_layers):
        s[f"l{l}.ln1"] = (cfg.hidden,)
        s[f"l{l}.wq"] = (cfg.hidden, q)
        s[f"l{l}.wk"] = (cfg.hidden, kv)
        s[f"l{l}.wv"] = (cfg.hidden, kv)
        s[f"l{l}.wo"] = (q, cfg.hidden)
        s[f"l{l}.ln2"] = (cfg.hidden,)
        s[f"l{l}.wgate"] = (cfg.hidden, cfg.ffn)
        s[f"l{l}.wup"] = (cfg.hidden, cfg.ffn)
        s[f"l{l}.wdown"] = (cfg.ffn, cfg.hidden)
    s["ln_f"] = (cfg.hidden,)
    return s


def make_weights_host(cfg: LlamaConfig, seed: int = 0, with_embedding: bool = True):
    """Seeded synthetic weights on the host (numpy float32): N(0, 0.02), norm weights 1."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in weight_shapes(cfg, with_embedding).items():
        if name == "lm_head":
            continue
        if name.endswith(("ln1", "ln2")) or name == "ln_f":
            w[name] = np.ones(shape, dtype=np.float32)
        else:
            w[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)).astype(np.float32)
    if with_embedding:
        w["lm_head"] = np.ascontiguousarray(w["embed"].T)
    return w


def make_weights_device(cfg: LlamaConfig, seed: int = 0, device="cuda"):
    """The same distribution generated directly in device memory (torch is used only as the allocator and
    random source); returns name -> torch tensor."""
    import torch
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    w = {}
    for name, shape in weight_shapes(cfg).items():
        if name == "lm_head":
            continue
        if name.endswith(("ln1", "ln2")) or name == "ln_f":
            w[name] = torch.ones(shape, dtype=torch.float32, device=device)
        else:
            w[name] = torch.randn(shape, dtype=torch.float32, device=device, generator=gen) * 0.02
    w["lm_head"] = w["embed"].t().contiguous()
    return w


def _rmsnorm(g: GraphSpec, x: str, weight: str, tag: str) -> str:
    """Decomposed RMSNorm: Pow 2 -> ReduceMean(last axis, keepdims) -> Add eps -> Sqrt -> Div -> Mul weight."""
    x2 = g.op("Pow", [x, "two"], f"{tag}.pow")
    var = g.op("ReduceMean", [x2], f"{tag}.mean", axes=[-1], keepdims=1)
    ve = g.op("Add", [var, "eps"], f"{tag}.addeps")
    sd = g.op("Sqrt", [ve], f"{tag}.sqrt")
    xn = g.op("Div", [x, sd], f"{tag}.div")
    return g.op("Mul", [xn, weight], f"{tag}.out")


def _rope(g: GraphSpec, x: str, tag: str) -> str:
    """x * cos + rotate_half(x) * sin with rotate_half = Concat(-x[..., d/2:], x[..., :d/2])."""
    xc = g.op("Mul", [x, "rope.cos4"], f"{tag}.xcos")
    x1 = g.op("Slice", [x, "i0_1", "half_1", "ax3_1"], f"{tag}.lo")
    x2 = g.op("Slice", [x, "half_1", "hd_1", "ax3_1"], f"{tag}.hi")
    nx2 = g.op("Neg", [x2], f"{tag}.neg")
    rot = g.op("Concat", [nx2, x1], f"{tag}.rot", axis=-1)
    xs = g.op("Mul", [rot, "rope.sin4"], f"{tag}.xsin")
    return g.op("Add", [xc, xs], f"{tag}.out")


def build_graph(cfg: LlamaConfig, weights: dict, device_weights: bool = False, with_embedding: bool = True) -> GraphSpec:
    """The whole decoder as one op list.  `weights` maps the names of weight_shapes() to numpy arrays
    (device_weights=False) or torch CUDA tensors (device_weights=True).  With with_embedding=False the graph
    takes `inputs_embeds [B,S,hidden]` instead of input_ids and returns the final hidden state as
    `hidden_out` instead of logits (a single decoder layer as an exported sub-graph)."""
    g = GraphSpec()
    H, NH, NKV, D = cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
    rep = NH // NKV
    for name, shape in weight_shapes(cfg, with_embedding).items():
        w = weights[name]
        assert tuple(w.shape) == tuple(shape), (name, tuple(w.shape), shape)
        (g.const_device if device_weights else g.const)(name, w)

    if with_embedding:
        g.input("input_ids", np.int64, [0, 0])
    else:
        g.input("inputs_embeds", np.float32, [0, 0, H])
    g.input("attention_mask", np.int64, [0, 0])
    g.input("position_ids", np.int64, [0, 0])
    for l in range(cfg.n_layers):
        g.input(f"past_key_values.{l}.key", np.float32, [0, NKV, 0, D])
        g.input(f"past_key_values.{l}.value", np.float32, [0, NKV, 0, D])

    # small constants
    i64 = np.int64
    g.const("two", np.array(2.0, np.float32))
    g.const("eps", np.array(cfg.rms_eps, np.float32))
    g.const("one_f", np.array(1.0, np.float32))
    g.const("zero_f", np.array(0.0, np.float32))
    g.const("min_f", np.array(F32_MIN, np.float32))
    g.const("scale", np.array(1.0 / np.sqrt(D), np.float32))
    g.const("theta", np.array(cfg.rope_theta, np.float32))
    g.const("hd_f", np.array(float(D), np.float32))
    g.const("i0", np.array(0, i64))
    g.const("i1", np.array(1, i64))
    g.const("i2", np.array(2, i64))
    g.const("hd", np.array(D, i64))
    g.const("i0_1", np.array([0], i64))
    g.const("half_1", np.array([D // 2], i64))
    g.const("hd_1", np.array([D], i64))
    g.const("ax3_1", np.array([3], i64))
    g.const("ax0", np.array([0], i64))
    g.const("ax1", np.array([1], i64))
    g.const("ax2", np.array([2], i64))
    g.const("ax01", np.array([0, 1], i64))
    g.const("ax12", np.array([1, 2], i64))
    g.const("shape_q", np.array([0, 0, NH, D], i64))
    g.const("shape_kv", np.array([0, 0, NKV, D], i64))
    g.const("shape_rep", np.array([1, 1, rep, 1, 1], i64))
    g.const("shape_heads", np.array([0, NH, -1, D], i64))
    g.const("shape_merge", np.array([0, 0, NH * D], i64))

    # ---- embedding -------------------------------------------------------------------------------
    if with_embedding:
        x = g.op("Gather", ["embed", "input_ids"], "embed_out", axis=0)          # [B,S,H]
        ids_like = "input_ids"
    else:
        x = "inputs_embeds"
        ids_like = "position_ids"

    # ---- RoPE tables (once per step) -------------------------------------------------------------
    r = g.op("Range", ["i0", "hd", "i2"], "rope.range")                            # [D/2] i64: 0,2,..
    rf = g.op("Cast", [r], "rope.range_f", to=1)
    ex = g.op("Div", [rf, "hd_f"], "rope.exp")
    pw = g.op("Pow", ["theta", ex], "rope.pow")                                    # theta^(2i/D)
    inv = g.op("Div", ["one_f", pw], "rope.inv_freq")                              # [D/2]
    pos_f = g.op("Cast", ["position_ids"], "rope.pos_f", to=1)                     # [B,S]
    pos3 = g.op("Unsqueeze", [pos_f, "ax2"], "rope.pos3")                          # [B,S,1]
    fr = g.op("Mul", [pos3, inv], "rope.freqs")                                    # [B,S,D/2]
    emb = g.op("Concat", [fr, fr], "rope.emb", axis=-1)                            # [B,S,D]
    cos = g.op("Cos", [emb], "rope.cos")
    sin = g.op("Sin", [emb], "rope.sin")
    g.op("Unsqueeze", [cos, "ax1"], "rope.cos4")                                   # [B,1,S,D]
    g.op("Unsqueeze", [sin, "ax1"], "rope.sin4")

    # ---- causal + padding mask (once per step) ---------------------------------------------------
    ids_shape = g.op("Shape", [ids_like], "mask.ids_shape")                        # [2]
    s_len = g.op("Gather", [ids_shape, "i1"], "mask.S", axis=0)                    # scalar
    past_shape = g.op("Shape", ["past_key_values.0.key"], "mask.past_shape")       # [4]
    p_len = g.op("Gather", [past_shape, "i2"], "mask.P", axis=0)
    t_len = g.op("Add", [p_len, s_len], "mask.T")
    s1 = g.op("Unsqueeze", [s_len, "ax0"], "mask.S1")
    t1 = g.op("Unsqueeze", [t_len, "ax0"], "mask.T1")
    st = g.op("Concat", [s1, t1], "mask.ST", axis=0)                               # [2] = [S,T]
    ones = g.op("ConstantOfShape", [st], "mask.ones", value=np.array([1.0], np.float32))
    k_diag = g.op("Add", [p_len, "i1"], "mask.k")                                  # first masked diagonal
    tri = g.op("Trilu", [ones, k_diag], "mask.tri", upper=1)                       # 1 where key pos > query pos
    fut = g.op("Equal", [tri, "one_f"], "mask.future")                             # bool [S,T]
    causal = g.op("Where", [fut, "min_f", "zero_f"], "mask.causal")                # [S,T]
    causal4 = g.op("Unsqueeze", [causal, "ax01"], "mask.causal4")                  # [1,1,S,T]
    am_f = g.op("Cast", ["attention_mask"], "mask.am_f", to=1)                     # [B,T]
    padded = g.op("Equal", [am_f, "zero_f"], "mask.padded")                        # bool [B,T]
    padded4 = g.op("Unsqueeze", [padded, "ax12"], "mask.padded4")                  # [B,1,1,T]
    g.op("Where", [padded4, "min_f", causal4], "mask.full")                        # [B,1,S,T]

    for l in range(cfg.n_layers):
        t = f"l{l}"
        h = _rmsnorm(g, x, f"{t}.ln1", f"{t}.norm1")
        q = g.op("MatMul", [h, f"{t}.wq"], f"{t}.q")
        k = g.op("MatMul", [h, f"{t}.wk"], f"{t}.k")
        v = g.op("MatMul", [h, f"{t}.wv"], f"{t}.v")
        q4 = g.op("Transpose", [g.op("Reshape", [q, "shape_q"], f"{t}.q_r")], f"{t}.q4", perm=[0, 2, 1, 3])    # [B,NH,S,D]
        k4 = g.op("Transpose", [g.op("Reshape", [k, "shape_kv"], f"{t}.k_r")], f"{t}.k4", perm=[0, 2, 1, 3])   # [B,NKV,S,D]
        v4 = g.op("Transpose", [g.op("Reshape", [v, "shape_kv"], f"{t}.v_r")], f"{t}.v4", perm=[0, 2, 1, 3])
        qr = _rope(g, q4, f"{t}.rope_q")
        kr = _rope(g, k4, f"{t}.rope_k")
        kk = g.op("Concat", [f"past_key_values.{l}.key", kr], f"present.{l}.key", axis=2)                        # [B,NKV,T,D]
        vv = g.op("Concat", [f"past_key_values.{l}.value", v4], f"present.{l}.value", axis=2)
        ke = g.op("Expand", [g.op("Unsqueeze", [kk, "ax2"], f"{t}.k_u"), "shape_rep"], f"{t}.k_e")             # [B,NKV,rep,T,D]
        ve = g.op("Expand", [g.op("Unsqueeze", [vv, "ax2"], f"{t}.v_u"), "shape_rep"], f"{t}.v_e")
        kh = g.op("Reshape", [ke, "shape_heads"], f"{t}.k_h")                                                   # [B,NH,T,D]
        vh = g.op("Reshape", [ve, "shape_heads"], f"{t}.v_h")
        kt = g.op("Transpose", [kh], f"{t}.k_t", perm=[0, 1, 3, 2])                                             # [B,NH,D,T]
        sc = g.op("MatMul", [qr, kt], f"{t}.scores")                                                            # [B,NH,S,T]
        sc = g.op("Mul", [sc, "scale"], f"{t}.scaled")
        sc = g.op("Add", [sc, "mask.full"], f"{t}.masked")
        pr = g.op("Softmax", [sc], f"{t}.probs", axis=-1)
        cx = g.op("MatMul", [pr, vh], f"{t}.ctx")                                                               # [B,NH,S,D]
        cx = g.op("Transpose", [cx], f"{t}.ctx_t", perm=[0, 2, 1, 3])
        cx = g.op("Reshape", [cx, "shape_merge"], f"{t}.ctx_m")                                                 # [B,S,H]
        ao = g.op("MatMul", [cx, f"{t}.wo"], f"{t}.attn_out")
        x = g.op("Add", [x, ao], f"{t}.res1")
        h2 = _rmsnorm(g, x, f"{t}.ln2", f"{t}.norm2")
        ga = g.op("MatMul", [h2, f"{t}.wgate"], f"{t}.gate")
        up = g.op("MatMul", [h2, f"{t}.wup"], f"{t}.up")
        sg = g.op("Sigmoid", [ga], f"{t}.sig")
        sl = g.op("Mul", [ga, sg], f"{t}.silu")
        gu = g.op("Mul", [sl, up], f"{t}.gated")
        dn = g.op("MatMul", [gu, f"{t}.wdown"], f"{t}.down")
        x = g.op("Add", [x, dn], f"{t}.res2")
        g.output(kk)
        g.output(vv)

    hf = _rmsnorm(g, x, "ln_f", "norm_f")
    if with_embedding:
        g.op("MatMul", [hf, "lm_head"], "logits")                                                               # [B,S,vocab]
        g.output("logits")
    else:
        g.op("Mul", [hf, "one_f"], "hidden_out")
        g.output("hidden_out")
    return g


def dense_decoder_f64(cfg: LlamaConfig, weights: dict, ids, last_only: bool = True):
    """The decoder written densely in float64 with torch on the weights' device: ids [B,T] -> logits of the last position
    [B,vocab] (or of all positions).  No cache, no op graph, none of this library's kernels: an independent statement of
    what build_graph's op list computes, used by the benchmark to check the logits of the very configuration it times."""
    import torch
    B, T = ids.shape
    f64 = torch.float64

    def W(name):
        return weights[name].to(f64)

    x = W("embed")[ids]
    half = cfg.head_dim // 2
    dev = x.device
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=dev, dtype=f64) / cfg.head_dim))
    ang = torch.arange(T, device=dev, dtype=f64)[:, None] * inv[None, :]
    cos = torch.cos(torch.cat([ang, ang], -1))[None, None]
    sin = torch.sin(torch.cat([ang, ang], -1))[None, None]

    def norm(v, g):
        return v / torch.sqrt((v * v).mean(-1, keepdim=True) + cfg.rms_eps) * g

    def rope(v):
        return v * cos + torch.cat([-v[..., half:], v[..., :half]], -1) * sin

    pos = torch.arange(T, device=dev)
    mask = torch.where(pos[None, :] > pos[:, None], float("-inf"), 0.0).to(f64)
    rep = cfg.n_heads // cfg.n_kv_heads
    for l in range(cfg.n_layers):
        h = norm(x, W(f"l{l}.ln1"))
        q = (h @ W(f"l{l}.wq")).reshape(B, T, cfg.n_heads, cfg.head_dim).transpose(1, 2)
        k = (h @ W(f"l{l}.wk")).reshape(B, T, cfg.n_kv_heads, cfg.head_dim).transpose(1, 2)
        v = (h @ W(f"l{l}.wv")).reshape(B, T, cfg.n_kv_heads, cfg.head_dim).transpose(1, 2)
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        p = torch.softmax(q @ k.transpose(2, 3) / (cfg.head_dim ** 0.5) + mask, -1)
        o = (p @ v).transpose(1, 2).reshape(B, T, cfg.hidden)
        x = x + o @ W(f"l{l}.wo")
        h2 = norm(x, W(f"l{l}.ln2"))
        g = h2 @ W(f"l{l}.wgate")
        x = x + ((g * torch.sigmoid(g)) * (h2 @ W(f"l{l}.wup"))) @ W(f"l{l}.wdown")
    if last_only:
        x = x[:, -1]
    return norm(x, W("ln_f")) @ W("lm_head")


class Decoder:
    """Greedy-decode driver around a ModelInstance, shaped like the reference's harness loop
    (runtime/examples/llama.rs:65-161): feed ids / mask / positions, run, read logits; the KV cache is
    carried on the device from `present.*` to `past_key_values.*`."""

    def __init__(self, cfg: LlamaConfig, spec: GraphSpec, device: int = 0, stream=None, arena_bytes: int = 0):
        from .runtime import ModelInstance
        self.cfg = cfg
        self.inst = ModelInstance(spec.to_runtime(), device=device, stream=stream, arena_bytes=arena_bytes)
        for l in range(cfg.n_layers):
            self.inst.bind(f"present.{l}.key", f"past_key_values.{l}.key")
            self.inst.bind(f"present.{l}.value", f"past_key_values.{l}.value")
        self.context = 0
        self.batch = None

    def reset(self, batch: int):
        """Start new sequences: empty past [B, kv_heads, 0, head_dim]."""
        self.batch = batch
        self.context = 0
        empty = np.zeros((batch, self.cfg.n_kv_heads, 0, self.cfg.head_dim), dtype=np.float32)
        for l in range(self.cfg.n_layers):
            self.inst.set_input(f"past_key_values.{l}.key", empty)
            self.inst.set_input(f"past_key_values.{l}.value", empty)

    def feed(self, input_ids: np.ndarray):
        b, s = input_ids.shape
        t = self.context + s
        self.inst.set_input("input_ids", input_ids.astype(np.int64, copy=False))
        self.inst.set_input("attention_mask", np.ones((b, t), dtype=np.int64))
        self.inst.set_input("position_ids", np.broadcast_to(np.arange(self.context, t, dtype=np.int64), (b, s)))
        self.context = t

    def step(self, input_ids: np.ndarray) -> np.ndarray:
        """One forward pass over `input_ids [B,S]`; returns logits [B,S,vocab] on the host."""
        self.feed(input_ids)
        self.inst.launch()
        return self.inst.read("logits")
