"""Host-side checks of the model graph builders (no GPU): parameter lists, flop counts, oracle evaluation at toy size."""
import importlib.util
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _w():
    spec = importlib.util.spec_from_file_location("b200_workloads", os.path.join(ROOT, "go-darwinml_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["b200_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_flop_counts_match_the_stated_configs():
    w = _w()
    assert abs(w.gpt2_flops_per_token(w.GPT2Config()) / 1e6 - 284.8) < 0.5      # ~284.8 MFLOP per token
    assert abs(w.llama_flops_per_token(w.LlamaConfig()) / 1e9 - 2.74) < 0.02    # ~2.74 GFLOP per token


def test_toy_models_run_on_the_oracle():
    from oracle.oracle import OracleFunction
    w = _w()
    c = w.GPT2Config(layers=1, d_model=16, heads=2, d_ff=32, seq=8, vocab=19, batch=2)
    out = w.gpt2_forward(OracleFunction(), c, 7, *w.gpt2_init(c, 0, np.float32))
    assert out.shape == (2, 8, 19) and np.isfinite(out).all()
    lc = w.LlamaConfig(layers=1, d_model=16, heads=4, kv_heads=2, d_ff=32, seq=8, vocab=23, batch=2)
    out = w.llama_forward(OracleFunction(), lc, 7, *w.llama_init(lc, 0, np.float32))
    assert out.shape == (2, 8, 23) and np.isfinite(out).all()
    # causality: changing a later token must not change earlier logits
    params = w.llama_init(lc, 0, np.float32)
    ids2 = params[0].copy()
    ids2[:, -1, 0] = (ids2[:, -1, 0] + 1) % lc.vocab
    out2 = w.llama_forward(OracleFunction(), lc, 7, ids2, *params[1:])
    np.testing.assert_array_equal(out[:, :-1], out2[:, :-1])


def test_mlp_probabilities():
    from oracle.oracle import OracleFunction
    w = _w()
    out = w.mlp_forward(OracleFunction(), *w.mlp_init(0))
    assert out.shape == (64, 10)
    np.testing.assert_allclose(out.sum(-1), 1.0, rtol=1e-6)


def _scaled(w, shapes, arrays, scale):
    for i, (name, _) in enumerate(shapes):
        k = scale.get(name.split(".")[-1])
        if k:
            arrays[i] = (arrays[i] * k).astype(np.float32)
    return arrays


def test_incremental_decoding_equals_the_full_forward_on_the_prefix():
    """The decoding loops (KV caches extended in place, position mask, rotary embedding / position table at the
    loop-carried position) against the full-sequence causal forward of the same model on the tokens produced so far: the
    logits of step t must be the forward's logits at position t, so the greedy tokens agree.  CPU oracle, toy sizes."""
    import dataclasses

    from oracle.oracle import OracleFunction
    w = _w()
    n_tokens = 6
    # GPT-2 shape
    c = w.GPT2Config(layers=2, d_model=32, heads=2, d_ff=64, seq=8, vocab=29, batch=2)
    dshapes = w.gpt2_decode_param_shapes(c)
    arrays = _scaled(w, dshapes, w._init_params(dshapes, 3, np.float32, c.vocab), {"wte": 6.0, "wpe": 8.0, "wqkv": 40.0, "wo": 40.0, "wfc": 40.0, "wproj": 40.0})
    toks, last_logits = w.gpt2_greedy_decode(OracleFunction(), c, 7, n_tokens, *arrays)
    toks = np.asarray(toks)
    seq = np.concatenate([arrays[0].reshape(c.batch, 1), toks], axis=1)            # start token, then the greedy tokens
    for t in range(n_tokens):
        ct = dataclasses.replace(c, seq=t + 1)
        params = [seq[:, :t + 1].reshape(c.batch, t + 1, 1).astype(np.int32), arrays[1], arrays[2][:t + 1]] + list(arrays[3:])
        logits = np.asarray(w.gpt2_forward(OracleFunction(), ct, 7, *params))
        np.testing.assert_array_equal(logits[:, t].argmax(-1), toks[:, t])
        if t == n_tokens - 1:
            np.testing.assert_allclose(np.asarray(last_logits)[:, 0], logits[:, t], rtol=2e-4, atol=2e-4)
    # Llama shape (grouped-query attention, rotary embedding)
    lc = w.LlamaConfig(layers=2, d_model=32, heads=4, kv_heads=2, d_ff=64, seq=8, vocab=31, batch=2)
    lshapes = w.llama_decode_param_shapes(lc)
    larr = w._init_params(lshapes, 4, np.float32, lc.vocab)
    cos, sin = w.rope_tables(lc)
    for i, (name, _) in enumerate(lshapes):
        if name == "rope_cos":
            larr[i] = cos
        elif name == "rope_sin":
            larr[i] = sin
    larr = _scaled(w, lshapes, larr, {"embed": 20.0, "wqkv": 30.0, "wo": 30.0, "wgate": 30.0, "wup": 30.0, "wdown": 30.0, "lm_head": 30.0})
    toks, last_logits = w.llama_greedy_decode(OracleFunction(), lc, 7, n_tokens, *larr)
    toks = np.asarray(toks)
    seq = np.concatenate([larr[0].reshape(lc.batch, 1), toks], axis=1)
    for t in range(n_tokens):
        ct = dataclasses.replace(lc, seq=t + 1)
        params = [seq[:, :t + 1].reshape(lc.batch, t + 1, 1).astype(np.int32), larr[1], larr[2][:t + 1], larr[3][:t + 1]] + list(larr[4:])
        logits = np.asarray(w.llama_forward(OracleFunction(), ct, 7, *params))
        np.testing.assert_array_equal(logits[:, t].argmax(-1), toks[:, t])
        if t == n_tokens - 1:
            np.testing.assert_allclose(np.asarray(last_logits)[:, 0], logits[:, t], rtol=2e-4, atol=2e-4)
