"""Graph builders for the benchmark configurations, written against the Function interface.

Each builder takes a Function-like object (the backend's Function, or any object with the same
methods, e.g. a CPU oracle in the tests) plus already-created parameter values, and returns the
output value(s).  They use only the reference's op vocabulary: Gather, FusedLayerNorm, FusedDense,
FusedAttentionQKVProjection, FusedScaledDotProductAttention, DotGeneral and elementwise ops
(ref mpsgraph/gomlx/function.go), plus FusedRMSNorm for the Llama-style model.

  mlp_forward          configuration "MLP forward, fp32"            x[64,784] -> softmax probabilities [64,10]
  gpt2_forward         GPT-2-small-shaped decoder forward, bf16     ids[B,S] -> logits [B,S,V]
  llama_forward        Llama-style decoder forward (GQA, SwiGLU, RMSNorm, RoPE), bf16
  gpt2_greedy_decode   incremental decoding of the GPT-2-shaped model: one While loop, a KV cache per layer updated in
                       place (DynamicUpdateSlice), greedy next token (ArgMinMax + Gather); ids[B] -> tokens [B, n]
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List

import numpy as np

ACT_NONE, ACT_GELU, ACT_RELU, ACT_SILU, ACT_TANH = 0, 1, 2, 3, 4
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1
C_I32, C_BF16, C_F32 = 3, 6, 7


class _Shape:
    def __init__(self, code, dims):
        self.DType, self.Dimensions = code, list(dims)

    def Rank(self):
        return len(self.Dimensions)


# ------------------------------------------------------------------------------------ MLP ---
def mlp_param_shapes(batch=64, d_in=784, d_hidden=512, d_out=10):
    return [("x", (batch, d_in)), ("w1", (d_in, d_hidden)), ("b1", (d_hidden,)), ("w2", (d_hidden, d_out)), ("b2", (d_out,))]


def mlp_init(seed=0, batch=64, d_in=784, d_hidden=512, d_out=10) -> List[np.ndarray]:
    """x ~ U(-1,1); W ~ N(0, 1/fan_in); biases zero."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1, 1, size=(batch, d_in)).astype(np.float32)
    w1 = (rng.standard_normal((d_in, d_hidden)) / math.sqrt(d_in)).astype(np.float32)
    w2 = (rng.standard_normal((d_hidden, d_out)) / math.sqrt(d_hidden)).astype(np.float32)
    return [x, w1, np.zeros(d_hidden, np.float32), w2, np.zeros(d_out, np.float32)]


def mlp_forward(f, x, w1, b1, w2, b2):
    h = f.FusedDense(x, w1, b1, ACT_RELU)
    logits = f.FusedDense(h, w2, b2, ACT_NONE)
    return f.FusedSoftmax(logits, 1)


# ---------------------------------------------------------------------------------- GPT-2 ---
@dataclass
class GPT2Config:
    layers: int = 12
    d_model: int = 768
    heads: int = 12
    d_ff: int = 3072
    seq: int = 1024
    vocab: int = 50257
    batch: int = 16
    eps: float = 1e-5


def gpt2_param_shapes(c: GPT2Config):
    d = c.d_model
    out = [("ids", (c.batch, c.seq, 1)), ("wte", (c.vocab, d)), ("wpe", (c.seq, d))]
    for i in range(c.layers):
        out += [(f"l{i}.ln1_g", (d,)), (f"l{i}.ln1_b", (d,)), (f"l{i}.wqkv", (d, 3 * d)), (f"l{i}.bq", (d,)), (f"l{i}.bk", (d,)),
                (f"l{i}.bv", (d,)), (f"l{i}.wo", (d, d)), (f"l{i}.bo", (d,)), (f"l{i}.ln2_g", (d,)), (f"l{i}.ln2_b", (d,)),
                (f"l{i}.wfc", (d, c.d_ff)), (f"l{i}.bfc", (c.d_ff,)), (f"l{i}.wproj", (c.d_ff, d)), (f"l{i}.bproj", (d,))]
    out += [("lnf_g", (d,)), ("lnf_b", (d,))]
    return out


def _init_params(shapes, seed, float_dtype, vocab):
    """weights ~ N(0, 0.02); norm gains 1, biases 0; token ids uniform in [0, vocab)."""
    rng = np.random.default_rng(seed)
    arrays = []
    for name, shape in shapes:
        if name == "ids":
            arrays.append(rng.integers(0, vocab, size=shape, dtype=np.int64).astype(np.int32))
        elif name.endswith("_g") or name.endswith(".g"):
            arrays.append(np.ones(shape, np.float32).astype(float_dtype))
        elif name.split(".")[-1].startswith("b") or name.endswith("_b"):
            arrays.append(np.zeros(shape, np.float32).astype(float_dtype))
        elif name in ("rope_cos", "rope_sin"):
            arrays.append(None)  # filled by the caller
        else:
            arrays.append((0.02 * rng.standard_normal(shape, dtype=np.float32)).astype(float_dtype))
    return arrays


def gpt2_init(c: GPT2Config, seed=0, float_dtype=None):
    import ml_dtypes
    return _init_params(gpt2_param_shapes(c), seed, float_dtype or ml_dtypes.bfloat16, c.vocab)


def gpt2_forward(f, c: GPT2Config, dtype_code, *params):
    """Returns logits [B, S, V].  The LM head is tied to the token embedding (contract d with wte's axis 1)."""
    it = iter(params)
    ids, wte, wpe = next(it), next(it), next(it)
    B, S, d, H = c.batch, c.seq, c.d_model, c.heads
    D = d // H
    x = f.Gather(wte, ids, 2, [2], [0], [0], [1, d], False)                       # [B, S, d]
    x = f.Add(x, f.BroadcastInDim(wpe, _Shape(dtype_code, (B, S, d)), [1, 2]))
    for _ in range(c.layers):
        ln1_g, ln1_b, wqkv, bq, bk, bv, wo, bo, ln2_g, ln2_b, wfc, bfc, wproj, bproj = (next(it) for _ in range(14))
        h = f.FusedLayerNorm(x, [-1], c.eps, ln1_g, ln1_b)
        q, k, v = f.FusedAttentionQKVProjection(h, wqkv, bq, bk, bv, d, d)
        q, k, v = (f.Reshape(t, B, S, H, D) for t in (q, k, v))
        a = f.FusedScaledDotProductAttention(q, k, v, None, H, H, LAYOUT_BSHD, 1.0 / math.sqrt(D), True)
        x = f.Add(x, f.FusedDense(f.Reshape(a, B, S, d), wo, bo, ACT_NONE))
        h = f.FusedLayerNorm(x, [-1], c.eps, ln2_g, ln2_b)
        m = f.FusedDense(h, wfc, bfc, ACT_GELU)
        x = f.Add(x, f.FusedDense(m, wproj, bproj, ACT_NONE))
    lnf_g, lnf_b = next(it), next(it)
    x = f.FusedLayerNorm(x, [-1], c.eps, lnf_g, lnf_b)
    return f.DotGeneral(x, [2], None, wte, [1], None)


def gpt2_flops_per_token(c: GPT2Config) -> float:
    d, S = c.d_model, c.seq
    return c.layers * (2 * d * 3 * d + 2 * d * d + 4 * d * c.d_ff + 4 * S * d) + 2 * d * c.vocab  # full S x S attention counted


def closure(f, param_shapes, body):
    """body(c, *params) -> outputs, as a closure of function f: a Function.Closure() with its Parameters and Return on the
    backend; an object with MakeClosure (an eager evaluator such as the tests' CPU oracle) gets a callable instead."""
    if hasattr(f, "MakeClosure"):
        return f.MakeClosure(param_shapes, body)
    c = f.Closure()
    params = [c.Parameter(f"p{i}", s) for i, s in enumerate(param_shapes)]
    c.Return(list(body(c, *params)), None)
    return c


def gpt2_decode_param_shapes(c: GPT2Config):
    """The forward's parameters with the token ids replaced by one start token per batch entry."""
    return [("ids", (c.batch, 1, 1))] + gpt2_param_shapes(c)[1:]


def _const_i32(g, v):
    return g.Constant(np.array([v], dtype=np.int32))


def gpt2_decode_step(g, c: GPT2Config, dtype_code, weights, t, tok, out, caches):
    """One decoding step at position t (int32 scalar): the current token [B,1,1] goes through the model against the
    caches (per layer a key and a value cache [B, H, seq, D], extended at position t), the greedy next token is written
    to out[:, t].  `weights` = (wte, wpe, [14 tensors per layer], lnf_g, lnf_b).
    Returns (next token [B,1,1], out, logits [B,1,V], new caches)."""
    wte, wpe, layers, lnf_g, lnf_b = weights
    B, S, d, H = c.batch, c.seq, c.d_model, c.heads
    D = d // H
    zero = _const_i32(g, 0)
    x = g.Gather(wte, tok, 2, [2], [0], [0], [1, d], False)                            # [B, 1, d]
    pos = g.DynamicSlice(wpe, [t, zero], [1, d])                                       # [1, d]
    x = g.Add(x, g.BroadcastInDim(pos, _Shape(dtype_code, (B, 1, d)), [1, 2]))
    # keys at positions <= t are visible: [1, 1, 1, S] broadcast over batch, heads and the one query
    visible = g.LessOrEqual(g.Iota(_Shape(C_I32, (1, 1, 1, S)), 3), g.BroadcastInDim(t, _Shape(C_I32, (1, 1, 1, S)), []))
    new_caches = []
    for li, (ln1_g, ln1_b, wqkv, bq, bk, bv, wo, bo, ln2_g, ln2_b, wfc, bfc, wproj, bproj) in enumerate(layers):
        h = g.FusedLayerNorm(x, [-1], c.eps, ln1_g, ln1_b)
        q, k, v = g.FusedAttentionQKVProjection(h, wqkv, bq, bk, bv, d, d)
        q, k, v = (g.Reshape(u, B, H, 1, D) for u in (q, k, v))
        kc = g.DynamicUpdateSlice(caches[2 * li], k, [zero, zero, t, zero])
        vc = g.DynamicUpdateSlice(caches[2 * li + 1], v, [zero, zero, t, zero])
        new_caches += [kc, vc]
        a = g.FusedScaledDotProductAttention(q, kc, vc, visible, H, H, LAYOUT_BHSD, 1.0 / math.sqrt(D), False)
        x = g.Add(x, g.FusedDense(g.Reshape(a, B, 1, d), wo, bo, ACT_NONE))
        h = g.FusedLayerNorm(x, [-1], c.eps, ln2_g, ln2_b)
        x = g.Add(x, g.FusedDense(g.FusedDense(h, wfc, bfc, ACT_GELU), wproj, bproj, ACT_NONE))
    x = g.FusedLayerNorm(x, [-1], c.eps, lnf_g, lnf_b)
    logits = g.DotGeneral(x, [2], None, wte, [1], None)                                # [B, 1, V]
    nxt = g.ArgMinMax(logits, 2, C_I32, False)                                         # [B, 1]
    out2 = g.DynamicUpdateSlice(out, nxt, [zero, t])
    return g.Reshape(nxt, B, 1, 1), out2, logits, new_caches


def gpt2_greedy_decode(f, c: GPT2Config, dtype_code, n_tokens: int, *params):
    """Greedy incremental decoding: n_tokens steps from one start token per batch entry, positions 0 .. n_tokens - 1, as ONE
    While loop.  State: step t, current token [B,1,1], the tokens produced so far [B, n_tokens], the last logits, and per
    layer a key and a value cache [B, H, seq, D] that each step extends by one position in place (heads before
    positions: the one query of a step then contracts with the cache where it lies, and [B,1,H,D] reshapes to
    [B,H,1,D] for free).  Every step attends over the whole cache under a mask `key position <= t`.
    Returns (tokens [B, n_tokens] int32, last step's logits [B, 1, V])."""
    it = iter(params)
    ids, wte, wpe = next(it), next(it), next(it)
    layers = [tuple(next(it) for _ in range(14)) for _ in range(c.layers)]
    lnf_g, lnf_b = next(it), next(it)
    weights = (wte, wpe, layers, lnf_g, lnf_b)
    B, S, d, H, V = c.batch, c.seq, c.d_model, c.heads, c.vocab
    D = d // H
    s_i, s_tok, s_out = _Shape(C_I32, ()), _Shape(C_I32, (B, 1, 1)), _Shape(C_I32, (B, n_tokens))
    s_cache, s_logits = _Shape(dtype_code, (B, H, S, D)), _Shape(dtype_code, (B, 1, V))
    state_shapes = [s_i, s_tok, s_out, s_logits] + [s_cache] * (2 * c.layers)

    def body(g, t, tok, out, _logits, *caches):
        nxt, out2, logits, new_caches = gpt2_decode_step(g, c, dtype_code, weights, t, tok, out, caches)
        return [g.Add(t, _const_i32(g, 1)), nxt, out2, logits] + new_caches

    cond = closure(f, state_shapes, lambda g, t, *rest: [g.LessThan(t, _const_i32(g, n_tokens))])
    loop = closure(f, state_shapes, body)
    float_np = {C_F32: np.float32}.get(dtype_code)
    if float_np is None:
        import ml_dtypes
        float_np = ml_dtypes.bfloat16
    # zero-filled initial values as broadcasts of a scalar: no large constants in the graph
    zeros = lambda shape, np_dt: f.BroadcastInDim(f.Constant(np.zeros(1, dtype=np_dt)), shape, [])
    init = [_const_i32(f, 0), ids, zeros(s_out, np.int32), zeros(s_logits, float_np)] + [zeros(s_cache, float_np) for _ in range(2 * c.layers)]
    res = f.While(cond, loop, *init)
    return res[2], res[3]


# ---------------------------------------------------------------------------------- Llama ---
@dataclass
class LlamaConfig:
    layers: int = 16
    d_model: int = 2048
    heads: int = 32
    kv_heads: int = 8
    d_ff: int = 8192
    seq: int = 2048
    vocab: int = 128256
    batch: int = 64
    eps: float = 1e-5
    rope_theta: float = 500000.0


def llama_param_shapes(c: LlamaConfig):
    d, D = c.d_model, c.d_model // c.heads
    kv = c.kv_heads * D
    out = [("ids", (c.batch, c.seq, 1)), ("embed", (c.vocab, d)), ("rope_cos", (c.seq, D)), ("rope_sin", (c.seq, D))]
    for i in range(c.layers):
        out += [(f"l{i}.norm1_g", (d,)), (f"l{i}.wqkv", (d, d + 2 * kv)), (f"l{i}.wo", (d, d)), (f"l{i}.norm2_g", (d,)),
                (f"l{i}.wgate", (d, c.d_ff)), (f"l{i}.wup", (d, c.d_ff)), (f"l{i}.wdown", (c.d_ff, d))]
    out += [("normf_g", (d,)), ("lm_head", (d, c.vocab))]
    return out


def rope_tables(c: LlamaConfig):
    """cos and SIGNED sin of position * theta^(-2i/D) over both halves of the head dim (rotate-half form):
    rope(x) = x * cos + swap_halves(x) * sin_signed, with sin_signed = concat(-sin, sin), which equals the usual
    x * cos + concat(-x2, x1) * sin exactly (the sign moves from the activations into the table)."""
    D = c.d_model // c.heads
    inv = c.rope_theta ** (-np.arange(0, D, 2, dtype=np.float64) / D)
    ang = np.arange(c.seq, dtype=np.float64)[:, None] * inv[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], axis=1)
    sin_signed = np.concatenate([-np.sin(ang), np.sin(ang)], axis=1)
    return cos.astype(np.float32), sin_signed.astype(np.float32)


def llama_init(c: LlamaConfig, seed=0, float_dtype=None):
    import ml_dtypes
    dt = float_dtype or ml_dtypes.bfloat16
    shapes = llama_param_shapes(c)
    arrays = _init_params(shapes, seed, dt, c.vocab)
    cos, sin = rope_tables(c)
    for i, (name, _) in enumerate(shapes):
        if name == "rope_cos":
            arrays[i] = cos.astype(dt)
        elif name == "rope_sin":
            arrays[i] = sin.astype(dt)
    return arrays


def _rope(f, x, cos_b, sin_b, dims, half):
    """x * cos + swap_halves(x) * sin_signed on the last axis (see rope_tables)."""
    r = len(dims)
    lo = f.Slice(x, [0] * r, dims[:-1] + [half], [1] * r)
    hi = f.Slice(x, [0] * (r - 1) + [half], dims, [1] * r)
    swapped = f.Concatenate(r - 1, hi, lo)
    return f.Add(f.Mul(x, cos_b), f.Mul(swapped, sin_b))


def llama_forward(f, c: LlamaConfig, dtype_code, *params):
    """Returns logits [B, S, V]."""
    it = iter(params)
    ids, embed, cos, sin = next(it), next(it), next(it), next(it)
    B, S, d, H, Hkv = c.batch, c.seq, c.d_model, c.heads, c.kv_heads
    D = d // H
    kv = Hkv * D
    x = f.Gather(embed, ids, 2, [2], [0], [0], [1, d], False)                     # [B, S, d]
    # tables spread over the heads once ([S, Hx, D], a few MB), then broadcast over the batch inside each fused chain
    def table(t, hx):
        per_head = f.BroadcastInDim(t, _Shape(dtype_code, (S, hx, D)), [0, 2])
        return f.BroadcastInDim(per_head, _Shape(dtype_code, (B, S, hx, D)), [1, 2, 3])
    cos_q, sin_q, cos_k, sin_k = table(cos, H), table(sin, H), table(cos, Hkv), table(sin, Hkv)
    for _ in range(c.layers):
        norm1_g, wqkv, wo, norm2_g, wgate, wup, wdown = (next(it) for _ in range(7))
        h = f.FusedRMSNorm(x, [-1], c.eps, norm1_g)
        q, k, v = f.FusedAttentionQKVProjection(h, wqkv, None, None, None, d, kv)
        q = _rope(f, f.Reshape(q, B, S, H, D), cos_q, sin_q, [B, S, H, D], D // 2)
        k = _rope(f, f.Reshape(k, B, S, Hkv, D), cos_k, sin_k, [B, S, Hkv, D], D // 2)
        v = f.Reshape(v, B, S, Hkv, D)
        a = f.FusedScaledDotProductAttention(q, k, v, None, H, Hkv, LAYOUT_BSHD, 1.0 / math.sqrt(D), True)
        x = f.Add(x, f.FusedDense(f.Reshape(a, B, S, d), wo, None, ACT_NONE))
        h = f.FusedRMSNorm(x, [-1], c.eps, norm2_g)
        gate = f.FusedDense(h, wgate, None, ACT_SILU)
        up = f.FusedDense(h, wup, None, ACT_NONE)
        x = f.Add(x, f.FusedDense(f.Mul(gate, up), wdown, None, ACT_NONE))
    normf_g, lm_head = next(it), next(it)
    x = f.FusedRMSNorm(x, [-1], c.eps, normf_g)
    return f.FusedDense(x, lm_head, None, ACT_NONE)


def llama_decode_param_shapes(c: LlamaConfig):
    """The forward's parameters with the token ids replaced by one start token per batch entry."""
    return [("ids", (c.batch, 1, 1))] + llama_param_shapes(c)[1:]


def llama_decode_step(g, c: LlamaConfig, dtype_code, weights, t, tok, out, caches):
    """One decoding step at position t (int32 scalar) of the Llama-shaped model: RMSNorm, fused QKV projection, rotary
    embedding of the one query and key at position t (the tables' row t, read with DynamicSlice), grouped-query attention
    of the query over the caches (per layer a key and a value cache [B, Hkv, seq, D], extended at position t) under a
    position mask, gated MLP.  `weights` = (embed, cos, sin, [7 tensors per layer], normf_g, lm_head).
    Returns (next token [B,1,1], out with the greedy token at [:, t], logits [B,1,V], new caches)."""
    embed, cos, sin, layers, normf_g, lm_head = weights
    B, S, d, H, Hkv = c.batch, c.seq, c.d_model, c.heads, c.kv_heads
    D = d // H
    kv = Hkv * D
    zero = _const_i32(g, 0)
    x = g.Gather(embed, tok, 2, [2], [0], [0], [1, d], False)                          # [B, 1, d]
    cos_t = g.DynamicSlice(cos, [t, zero], [1, D])                                     # [1, D]
    sin_t = g.DynamicSlice(sin, [t, zero], [1, D])
    table = lambda tb, hx: g.BroadcastInDim(tb, _Shape(dtype_code, (B, hx, 1, D)), [2, 3])
    cos_q, sin_q, cos_k, sin_k = table(cos_t, H), table(sin_t, H), table(cos_t, Hkv), table(sin_t, Hkv)
    visible = g.LessOrEqual(g.Iota(_Shape(C_I32, (1, 1, 1, S)), 3), g.BroadcastInDim(t, _Shape(C_I32, (1, 1, 1, S)), []))
    new_caches = []
    for li, (norm1_g, wqkv, wo, norm2_g, wgate, wup, wdown) in enumerate(layers):
        h = g.FusedRMSNorm(x, [-1], c.eps, norm1_g)
        q, k, v = g.FusedAttentionQKVProjection(h, wqkv, None, None, None, d, kv)
        q = _rope(g, g.Reshape(q, B, H, 1, D), cos_q, sin_q, [B, H, 1, D], D // 2)
        k = _rope(g, g.Reshape(k, B, Hkv, 1, D), cos_k, sin_k, [B, Hkv, 1, D], D // 2)
        kc = g.DynamicUpdateSlice(caches[2 * li], k, [zero, zero, t, zero])
        vc = g.DynamicUpdateSlice(caches[2 * li + 1], g.Reshape(v, B, Hkv, 1, D), [zero, zero, t, zero])
        new_caches += [kc, vc]
        a = g.FusedScaledDotProductAttention(q, kc, vc, visible, H, Hkv, LAYOUT_BHSD, 1.0 / math.sqrt(D), False)
        x = g.Add(x, g.FusedDense(g.Reshape(a, B, 1, d), wo, None, ACT_NONE))
        h = g.FusedRMSNorm(x, [-1], c.eps, norm2_g)
        gate = g.FusedDense(h, wgate, None, ACT_SILU)
        up = g.FusedDense(h, wup, None, ACT_NONE)
        x = g.Add(x, g.FusedDense(g.Mul(gate, up), wdown, None, ACT_NONE))
    x = g.FusedRMSNorm(x, [-1], c.eps, normf_g)
    logits = g.FusedDense(x, lm_head, None, ACT_NONE)                                  # [B, 1, V]
    nxt = g.ArgMinMax(logits, 2, C_I32, False)                                         # [B, 1]
    out2 = g.DynamicUpdateSlice(out, nxt, [zero, t])
    return g.Reshape(nxt, B, 1, 1), out2, logits, new_caches


def llama_greedy_decode(f, c: LlamaConfig, dtype_code, n_tokens: int, *params):
    """Greedy incremental decoding of the Llama-shaped model, n_tokens steps from one start token per batch entry, as ONE
    While loop (see gpt2_greedy_decode).  Returns (tokens [B, n_tokens] int32, last step's logits [B, 1, V])."""
    it = iter(params)
    ids, embed, cos, sin = next(it), next(it), next(it), next(it)
    layers = [tuple(next(it) for _ in range(7)) for _ in range(c.layers)]
    normf_g, lm_head = next(it), next(it)
    weights = (embed, cos, sin, layers, normf_g, lm_head)
    B, S, d, H, Hkv, V = c.batch, c.seq, c.d_model, c.heads, c.kv_heads, c.vocab
    D = d // H
    s_i, s_tok, s_out = _Shape(C_I32, ()), _Shape(C_I32, (B, 1, 1)), _Shape(C_I32, (B, n_tokens))
    s_cache, s_logits = _Shape(dtype_code, (B, Hkv, S, D)), _Shape(dtype_code, (B, 1, V))
    state_shapes = [s_i, s_tok, s_out, s_logits] + [s_cache] * (2 * c.layers)

    def body(g, t, tok, out, _logits, *caches):
        nxt, out2, logits, new_caches = llama_decode_step(g, c, dtype_code, weights, t, tok, out, caches)
        return [g.Add(t, _const_i32(g, 1)), nxt, out2, logits] + new_caches

    cond = closure(f, state_shapes, lambda g, t, *rest: [g.LessThan(t, _const_i32(g, n_tokens))])
    loop = closure(f, state_shapes, body)
    float_np = {C_F32: np.float32}.get(dtype_code)
    if float_np is None:
        import ml_dtypes
        float_np = ml_dtypes.bfloat16
    zeros = lambda shape, np_dt: f.BroadcastInDim(f.Constant(np.zeros(1, dtype=np_dt)), shape, [])
    init = [_const_i32(f, 0), ids, zeros(s_out, np.int32), zeros(s_logits, float_np)] + [zeros(s_cache, float_np) for _ in range(2 * c.layers)]
    res = f.While(cond, loop, *init)
    return res[2], res[3]


def llama_flops_per_token(c: LlamaConfig) -> float:
    d, S = c.d_model, c.seq
    kv = c.kv_heads * (d // c.heads)
    return c.layers * (2 * d * d * 2 + 2 * d * kv * 2 + 6 * d * c.d_ff + 4 * S * d) + 2 * d * c.vocab  # full S x S attention counted


def build_executable(pkg, backend, name, shapes_and_dtypes, forward):
    """Compiles `forward(f, *params)` with one Parameter per (shape, numpy dtype); returns (builder, executable)."""
    builder = backend.Builder(name)
    f = builder.Main()
    params = [f.Parameter(f"p{i}", pkg.Shape(pkg.dtypes.from_numpy(dt), shape)) for i, (shape, dt) in enumerate(shapes_and_dtypes)]
    out = forward(f, *params)
    f.Return(list(out) if isinstance(out, (list, tuple)) else [out], None)
    return builder, builder.Compile()


def make_device_params(pkg, torch, shapes, cfg, device: int, seed: int = 1234):
    """Seeded random parameters created directly in device memory (torch is only the random source and the owner
    of the allocations) and wrapped as backend buffers.  Returns (buffers, numpy dtypes, keep-alive list)."""
    import ctypes

    import ml_dtypes

    from . import _lib
    L = pkg.lib()
    dev = f"cuda:{device}"
    gen = torch.Generator(device=dev).manual_seed(seed + device)
    bufs, dts, keep = [], [], []
    for pname, shape in shapes:
        if pname == "ids":
            t = torch.randint(0, cfg.vocab, shape, generator=gen, device=dev, dtype=torch.int32)
            code, npdt = int(pkg.dtypes.Int32), np.dtype(np.int32)
        else:
            code, npdt = int(pkg.dtypes.BFloat16), np.dtype(ml_dtypes.bfloat16)
            if pname in ("rope_cos", "rope_sin"):
                cos, sin = rope_tables(cfg)
                t = torch.from_numpy(cos if pname == "rope_cos" else sin).to(dev).to(torch.bfloat16)
            elif pname.endswith("_g"):
                t = torch.ones(shape, device=dev, dtype=torch.bfloat16)
            elif pname.split(".")[-1].startswith("b") or pname.endswith("_b"):
                t = torch.zeros(shape, device=dev, dtype=torch.bfloat16)
            else:
                t = (0.02 * torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)).to(torch.bfloat16)
        keep.append(t)
        err = _lib.B200Error()
        h = L.b200_buffer_wrap(device, t.data_ptr(), code, (ctypes.c_int64 * max(len(shape), 1))(*shape), len(shape), ctypes.byref(err))
        if err.code:
            raise RuntimeError(L.take_string(err.message))
        bufs.append(pkg.Buffer(h))
        dts.append(npdt)
    torch.cuda.synchronize()
    return bufs, dts, keep
