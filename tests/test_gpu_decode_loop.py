"""Incremental decoding: the GPT-2-shaped model generating tokens greedily inside ONE While loop, against the CPU oracle.

What this exercises beyond the full-sequence forward: a KV cache per layer extended in place by DynamicUpdateSlice
inside the loop body (one buffer per cache and for the token list, not two), attention of one query over the cache under a position mask,
ArgMinMax feeding Gather feeding the next step, DynamicSlice of the position table at a loop-carried index, and the
whole loop as a conditional node when the plan is replayed.  Tokens must match the oracle's exactly (fp32 model: the
argmax margins of a random model are far above rounding differences); the last logits at rel 1e-4.
"""
import numpy as np
import pytest

import go_darwinml_b200.workloads as w
from oracle.oracle import OracleFunction, compare

pytestmark = pytest.mark.gpu


def _decode_inputs(c, seed):
    shapes = w.gpt2_decode_param_shapes(c)
    arrays = w._init_params(shapes, seed, np.float32, c.vocab)
    # N(0, 0.02) weights give nearly flat logits and a model that repeats its input; scaled like this it produces varied
    # tokens whose argmax margins (0.2 and more on logits of magnitude 3) dwarf fp32 rounding differences
    scale = {"wte": 6.0, "wpe": 8.0, "wqkv": 40.0, "wo": 40.0, "wfc": 40.0, "wproj": 40.0}
    for i, (name, _) in enumerate(shapes):
        k = scale.get(name.split(".")[-1])
        if k:
            arrays[i] = (arrays[i] * k).astype(np.float32)
    return shapes, arrays


def test_greedy_decode_matches_the_oracle_token_for_token(b200, backend):
    c = w.GPT2Config(layers=2, d_model=64, heads=2, d_ff=128, seq=16, vocab=97, batch=3)
    n_tokens = 10
    shapes, arrays = _decode_inputs(c, 5)
    code = int(b200.dtypes.Float32)
    builder = backend.Builder("decode")
    f = builder.Main()
    params = [f.Parameter(name, b200.Shape(b200.dtypes.from_numpy(a.dtype), a.shape)) for (name, _), a in zip(shapes, arrays)]
    tokens, logits = w.gpt2_greedy_decode(f, c, code, n_tokens, *params)
    f.Return([tokens, logits], None)
    exe = builder.Compile()
    plan = exe.Describe()
    assert "while[" in plan and "(5 updated in place)" in plan and "on the device when replayed" in plan, plan
    want_tokens, want_logits = w.gpt2_greedy_decode(OracleFunction(), c, code, n_tokens, *arrays)
    assert len(np.unique(np.asarray(want_tokens))) > 3   # the model does produce different tokens
    bufs = [backend.FromNumpy(a) for a in arrays]
    for run in range(4):   # host-driven twice, then replayed with the loop on the device
        outs = exe.Execute(bufs, None, 0)
        got_tokens, got_logits = (backend.ToNumpy(o) for o in outs)
        for o in outs:
            backend.BufferFinalize(o)
        np.testing.assert_array_equal(got_tokens, np.asarray(want_tokens))
        ok, viol = compare(got_logits, np.asarray(want_logits), 1e-4, 1.0)
        assert ok, (run, viol)
    exe.Finalize()
    builder.Finalize()
