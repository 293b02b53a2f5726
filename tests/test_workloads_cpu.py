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
