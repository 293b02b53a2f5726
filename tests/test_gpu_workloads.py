"""The three model-shaped configurations at toy sizes: backend (through the C ABI) against the CPU oracle."""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import run_backend

pytestmark = pytest.mark.gpu


def _workloads():
    import go_darwinml_b200.workloads as w
    return w


def test_mlp_forward_config_matches_oracle(b200, backend):
    w = _workloads()
    inputs = w.mlp_init(seed=0)   # the full configuration: x[64,784], W1[784,512], W2[512,10]
    got = run_backend(b200, backend, lambda f, *p: w.mlp_forward(f, *p), inputs)[0]
    want = w.mlp_forward(OracleFunction(), *inputs)
    ok, viol = compare(got, want, 1e-5, 1.0)
    assert ok, viol
    np.testing.assert_allclose(got.sum(-1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("dtype,rtol", [(np.float32, 2e-4), (ml_dtypes.bfloat16, 5e-2)], ids=["f32", "bf16"])
def test_gpt2_toy_matches_oracle(b200, backend, dtype, rtol):
    w = _workloads()
    c = w.GPT2Config(layers=2, d_model=64, heads=4, d_ff=256, seq=32, vocab=101, batch=2)
    inputs = w.gpt2_init(c, seed=1, float_dtype=dtype)
    code = int(b200.dtypes.from_numpy(np.dtype(dtype)))
    got = run_backend(b200, backend, lambda f, *p: w.gpt2_forward(f, c, code, *p), inputs)[0]
    want = w.gpt2_forward(OracleFunction(), c, code, *inputs)
    assert got.shape == (2, 32, 101)
    ok, viol = compare(got, want, rtol, 1.0)
    assert ok, viol


@pytest.mark.parametrize("dtype,rtol", [(np.float32, 2e-4), (ml_dtypes.bfloat16, 5e-2)], ids=["f32", "bf16"])
def test_llama_toy_matches_oracle(b200, backend, dtype, rtol):
    w = _workloads()
    c = w.LlamaConfig(layers=2, d_model=64, heads=8, kv_heads=2, d_ff=128, seq=32, vocab=120, batch=2)
    inputs = w.llama_init(c, seed=2, float_dtype=dtype)
    code = int(b200.dtypes.from_numpy(np.dtype(dtype)))
    got = run_backend(b200, backend, lambda f, *p: w.llama_forward(f, c, code, *p), inputs)[0]
    want = w.llama_forward(OracleFunction(), c, code, *inputs)
    assert got.shape == (2, 32, 120)
    ok, viol = compare(got, want, rtol, 1.0)
    assert ok, viol


def test_argmax_of_logits_is_exact(b200, backend):
    # greedy next-token choice: bit-exact index result on tie-free inputs
    rng = np.random.default_rng(3)
    logits = rng.standard_normal((4, 16, 1000)).astype(np.float32)
    got = run_backend(b200, backend, lambda f, x: f.ArgMinMax(x, 2, b200.dtypes.Int32, False), [logits])[0]
    np.testing.assert_array_equal(got, logits.argmax(-1).astype(np.int32))
