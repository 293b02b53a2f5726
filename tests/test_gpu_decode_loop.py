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
from tests.util import default_switches

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
    assert ("while[" in plan and "(5 updated in place)" in plan and "on the device when replayed" in plan) or not default_switches(), plan
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


def _llama_decode_inputs(c, seed, dtype):
    shapes = w.llama_decode_param_shapes(c)
    arrays = w._init_params(shapes, seed, np.float32, c.vocab)
    cos, sin = w.rope_tables(c)
    scale = {"embed": 20.0, "wqkv": 30.0, "wo": 30.0, "wgate": 30.0, "wup": 30.0, "wdown": 30.0, "lm_head": 30.0}
    for i, (name, _) in enumerate(shapes):
        if name == "rope_cos":
            arrays[i] = cos
        elif name == "rope_sin":
            arrays[i] = sin
        k = scale.get(name.split(".")[-1])
        if k:
            arrays[i] = arrays[i] * k
        if arrays[i].dtype != np.int32:
            arrays[i] = arrays[i].astype(dtype)
    return shapes, arrays


def _compile_llama_decode(b200, backend, c, code, n_tokens, shapes, arrays):
    builder = backend.Builder("llama_decode")
    f = builder.Main()
    params = [f.Parameter(name, b200.Shape(b200.dtypes.from_numpy(a.dtype), a.shape)) for (name, _), a in zip(shapes, arrays)]
    tokens, logits = w.llama_greedy_decode(f, c, code, n_tokens, *params)
    f.Return([tokens, logits], None)
    return builder, builder.Compile()


def test_llama_shaped_greedy_decode_matches_the_oracle_token_for_token(b200, backend):
    # rotary embedding at a loop-carried position, grouped-query attention over the caches (4 heads on 2 KV heads),
    # gated MLP; fp32, so tokens must agree exactly
    c = w.LlamaConfig(layers=2, d_model=256, heads=4, kv_heads=2, d_ff=512, seq=24, vocab=211, batch=3)
    n_tokens = 12
    shapes, arrays = _llama_decode_inputs(c, 7, np.float32)
    code = int(b200.dtypes.Float32)
    builder, exe = _compile_llama_decode(b200, backend, c, code, n_tokens, shapes, arrays)
    plan = exe.Describe()
    assert ("while[" in plan and "on the device when replayed" in plan) or not default_switches(), plan
    want_tokens, want_logits = w.llama_greedy_decode(OracleFunction(), c, code, n_tokens, *arrays)
    assert len(np.unique(np.asarray(want_tokens))) > 3
    bufs = [backend.FromNumpy(a) for a in arrays]
    for run in range(4):
        outs = exe.Execute(bufs, None, 0)
        got_tokens, got_logits = (backend.ToNumpy(o) for o in outs)
        for o in outs:
            backend.BufferFinalize(o)
        np.testing.assert_array_equal(got_tokens, np.asarray(want_tokens))
        ok, viol = compare(got_logits, np.asarray(want_logits), 1e-4, 1.0)
        assert ok, (run, viol)
    exe.Finalize()
    builder.Finalize()


def test_llama_shaped_decode_in_bf16_takes_the_decoding_kernels(b200, backend):
    # the same model in bf16: the step runs on the one-query tensor-core attention and the few-rows products; its first
    # step's logits agree with the oracle's bf16 evaluation to bf16 accuracy on the logits' scale
    import ml_dtypes
    bf16 = ml_dtypes.bfloat16
    c = w.LlamaConfig(layers=2, d_model=256, heads=4, kv_heads=2, d_ff=512, seq=32, vocab=256, batch=3)
    shapes, arrays = _llama_decode_inputs(c, 8, bf16)
    code = int(b200.dtypes.BFloat16)
    builder, exe = _compile_llama_decode(b200, backend, c, code, 1, shapes, arrays)
    plan = exe.Describe()
    assert ("attention_decode[" in plan and "Hkv=2" in plan and plan.count("few-rows") >= 2 * 4 + 1) or not default_switches(), plan
    _, want_logits = w.llama_greedy_decode(OracleFunction(), c, code, 1, *arrays)
    bufs = [backend.FromNumpy(a) for a in arrays]
    outs = exe.Execute(bufs, None, 0)
    got_logits = backend.ToNumpy(outs[1]).astype(np.float32)
    for o in outs:
        backend.BufferFinalize(o)
    want = np.asarray(want_logits).astype(np.float32)
    assert np.isfinite(got_logits).all()
    assert np.abs(got_logits - want).max() <= 0.04 * np.abs(want).max(), (np.abs(got_logits - want).max(), np.abs(want).max())
    exe.Finalize()
    builder.Finalize()


def test_an_update_of_an_updated_tensor_keeps_its_order(b200, backend):
    # two DynamicUpdateSlices with the same start and geometry, the second applied to the first's result: they must not
    # be joined into one side-by-side launch -- the second's block wins
    from tests.util import run_backend, run_oracle
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 6, 8)).astype(np.float32)
    a, b = rng.standard_normal((4, 1, 8)).astype(np.float32), rng.standard_normal((4, 1, 8)).astype(np.float32)
    t = np.array(3, dtype=np.int32)

    def build(f, xx, aa, bb, tt):
        zero = f.Constant(np.array([0], dtype=np.int32))
        first = f.DynamicUpdateSlice(xx, aa, [zero, tt, zero])
        return f.DynamicUpdateSlice(first, bb, [zero, tt, zero])
    (got,), plan = run_backend(b200, backend, build, [x, a, b, t], describe=True)
    (want,) = run_oracle(build, [x, a, b, t])
    assert ("a second one" not in plan) or not default_switches(), plan
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(got[:, 3, :], b[:, 0, :])
