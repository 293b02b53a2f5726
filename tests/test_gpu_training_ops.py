"""Training-side ops through the C ABI against the CPU oracle: ScatterSum / Max / Min, BatchNormForTraining,
BatchNormGradient, RNGBitGenerator (ref mpsgraph/gomlx/gather.go:441-641, function.go:1263-1527, 1627-1692).

Integer scatters, max / min scatters and the random bits are bit-exact.  A float ScatterSum combines with hardware
atomics in whatever order they arrive: compared at rel 1e-5 (fp32) with a norm-relative term.
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import assert_parity, rng_array, run_backend, run_oracle

pytestmark = pytest.mark.gpu

BF16 = ml_dtypes.bfloat16


# ------------------------------------------------------------------------------- scatter ---
@pytest.mark.parametrize("op", ["ScatterSum", "ScatterMax", "ScatterMin"])
@pytest.mark.parametrize("dtype", [np.float32, np.int32, np.int64, np.int8, np.uint16, np.float64, BF16, np.float16], ids=lambda d: np.dtype(d).name)
def test_scatter_rows_with_duplicates(b200, backend, op, dtype):
    # the embedding-gradient pattern: rows of `updates` combined into rows of the operand, many of them the same row
    rng = np.random.default_rng(120)
    V, D, N = 50, 24, 400
    operand = rng_array(rng, (V, D), dtype)
    ids = rng.integers(0, V, size=(N, 1)).astype(np.int32)
    if np.dtype(dtype) in (np.dtype(BF16), np.dtype(np.float16)) and op == "ScatterSum":
        # 16-bit sums round after every atomic add: keep the sums exactly representable (small integers)
        operand = rng.integers(-4, 5, size=(V, D)).astype(np.float32).astype(dtype)
        updates = rng.integers(-2, 3, size=(N, D)).astype(np.float32).astype(dtype)
    else:
        updates = rng_array(rng, (N, D), dtype)
    build = lambda f, o, i, u: getattr(f, op)(o, i, u, 1, [1], [0], [0], False, False)
    (got,) = run_backend(b200, backend, build, [operand, ids, updates])
    (want,) = run_oracle(build, [operand, ids, updates])
    exact = np.dtype(dtype).kind in "iu" or op != "ScatterSum" or np.dtype(dtype).itemsize == 2
    ok, viol = compare(got, want, 0.0 if exact else (1e-5 if np.dtype(dtype) == np.float32 else 1e-12), 0.0 if exact else 1.0)
    assert ok, viol


def test_scatter_general_forms(b200, backend):
    rng = np.random.default_rng(121)
    # (1) scalar updates into a rank-3 operand through 3-component index vectors, the index vector on axis 0
    operand = rng_array(rng, (5, 6, 7), np.float32)
    idx = np.stack([rng.integers(0, 5, 40), rng.integers(0, 6, 40), rng.integers(0, 7, 40)]).astype(np.int64)   # [3, 40]
    upd = rng_array(rng, (40,), np.float32)
    assert_parity(b200, backend, lambda f, o, i, u: f.ScatterSum(o, i, u, 0, [], [0, 1, 2], [0, 1, 2]), [operand, idx, upd], rtol=1e-5, atol_scale=1.0)
    # (2) windows of [2, 3] placed by 2-component indices mapped to axes (2, 0), windows walking axes 0 and 2; some fall off the edge
    operand = rng_array(rng, (8, 4, 9), np.float32)
    idx = np.stack([rng.integers(-1, 9, 12), rng.integers(-1, 8, 12)], axis=1).astype(np.int32)              # [12, 2] -> (axis 2, axis 0)
    upd = rng_array(rng, (12, 2, 3), np.float32)
    assert_parity(b200, backend, lambda f, o, i, u: f.ScatterMax(o, i, u, 1, [1, 2], [1], [2, 0]), [operand, idx, upd], rtol=0.0)
    # (3) implicit trailing index axis (indexVectorAxis == rank), batch of indices with two axes
    operand = np.zeros((30,), np.int32)
    idx = rng.integers(0, 30, size=(4, 5)).astype(np.uint8)
    upd = rng.integers(-9, 9, size=(4, 5)).astype(np.int32)
    assert_parity(b200, backend, lambda f, o, i, u: f.ScatterSum(o, i, u, 2, [], [0], [0]), [operand, idx, upd])
    # NaN propagates through max / min
    operand = np.zeros((4, 2), np.float32)
    upd = np.array([[1, np.nan], [3, 4], [5, 6]], np.float32)
    ids = np.array([[0], [2], [0]], np.int32)
    assert_parity(b200, backend, lambda f, o, i, u: f.ScatterMax(o, i, u, 1, [1], [0], [0]), [operand, ids, upd], rtol=0.0)


def test_scatter_sum_large_embedding_gradient(b200, backend):
    # GPT-2's embedding gradient shape at a reduced batch: 4096 token rows of 768 into a 50257-row table (fp32)
    rng = np.random.default_rng(122)
    V, D, N = 50257, 768, 4096
    operand = np.zeros((V, D), np.float32)
    ids = rng.integers(0, V, size=(N, 1)).astype(np.int32)
    ids[:64] = 7   # one hot row
    upd = rng_array(rng, (N, D), np.float32)
    build = lambda f, o, i, u: f.ScatterSum(o, i, u, 1, [1], [0], [0], False, False)
    (got,) = run_backend(b200, backend, build, [operand, ids, upd])
    (want,) = run_oracle(build, [operand, ids, upd])
    # The hot row is a sum of 64 + terms added by atomics in whatever order they arrive: its error bound is the sum's, a
    # few ulps of the largest partial sum per term, not 1e-5 of a result that may have cancelled to nearly nothing.
    hot = np.zeros(V, dtype=bool)
    hot[7] = True
    ok, viol = compare(got[~hot], want[~hot], 1e-5, 1.0)
    assert ok, viol
    terms = upd[(ids[:, 0] == 7)]
    bound = 2.0 * terms.shape[0] * np.finfo(np.float32).eps * np.abs(terms).sum(axis=0)
    assert (np.abs(got[7].astype(np.float64) - want[7].astype(np.float64)) <= bound).all()


def test_scatter_errors(b200, backend):
    builder = backend.Builder("scatter_errors")
    f = builder.Main()
    S = lambda dt, *d: b200.Shape(b200.dtypes.from_numpy(np.dtype(dt)), d)
    o, i, u = f.Parameter("o", S(np.float32, 4, 2)), f.Parameter("i", S(np.int32, 3, 1)), f.Parameter("u", S(np.float32, 3, 2))
    with pytest.raises(b200.BackendError, match="index vector size"):
        f.ScatterSum(o, i, u, 1, [1], [0], [0, 1])
    with pytest.raises(b200.BackendError, match="integers"):
        f.ScatterSum(o, u, u, 1, [1], [0], [0])
    with pytest.raises(b200.BackendError, match="batch dims"):
        f.ScatterSum(o, f.Parameter("i2", S(np.int32, 5, 1)), u, 1, [1], [0], [0])
    builder.Finalize()


# ---------------------------------------------------------------------------- batch norm ---
@pytest.mark.parametrize("dtype,rtol", [(np.float32, 1e-5), (BF16, 2e-2)], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape,axis", [((64, 32), 1), ((8, 16, 6, 6), 1), ((8, 6, 6, 16), 3), ((5, 7), 0), ((4, 12, 10), -2)])
def test_batch_norm_training_and_gradient(b200, backend, shape, axis, dtype, rtol):
    rng = np.random.default_rng(123)
    C = shape[axis]
    x = (rng_array(rng, shape, np.float32, 2.0) + 0.3).astype(dtype)
    scale = (1 + 0.2 * rng.standard_normal(C)).astype(np.float32).astype(dtype)
    offset = (0.1 * rng.standard_normal(C)).astype(np.float32).astype(dtype)
    dy = rng_array(rng, shape, dtype)

    def build(f, a, sc, of, g):
        y, m, v = f.BatchNormForTraining(a, sc, of, 1e-3, axis)
        ga, gs, go = f.BatchNormGradient(a, sc, m, v, g, 1e-3, axis)
        return y, m, v, ga, gs, go
    got = run_backend(b200, backend, build, [x, scale, offset, dy])
    want = run_oracle(build, [x, scale, offset, dy])
    for name, g, w in zip(("normalized", "mean", "variance", "gradOperand", "gradScale", "gradOffset"), got, want):
        assert g.shape == w.shape and g.dtype == w.dtype, name
        ok, viol = compare(g, w, rtol if dtype == np.float32 else 6e-2, 1.0)   # bf16: a dozen ops each rounded to 8 bits on the device side
        assert ok, (name, viol)
    if dtype == np.float32:   # size-independent property: the normalised value has per-feature mean `offset` and variance ~ scale^2
        red = tuple(i for i in range(len(shape)) if i != (axis % len(shape)))
        np.testing.assert_allclose(got[0].mean(axis=red), offset, atol=1e-4)


# ----------------------------------------------------------------------------------- RNG ---
@pytest.mark.parametrize("dtype", [np.uint32, np.uint64, np.int32, np.uint8, np.int16, np.float32, np.float64, BF16, np.float16],
                         ids=lambda d: np.dtype(d).name)
def test_rng_bits_match_the_restated_generator_exactly(b200, backend, dtype):
    state = np.array([0x0123456789abcdef, 0xffffffffffffff00, 5], dtype=np.uint64)   # the counter's low word wraps inside the run
    shape = b200.Shape(b200.dtypes.from_numpy(np.dtype(dtype)), (3, 1001))
    build = lambda f, s: f.RNGBitGenerator(s, shape)
    new_state, values = run_backend(b200, backend, build, [state])
    want_state, want_values = OracleFunction().RNGBitGenerator(state, shape)
    np.testing.assert_array_equal(new_state, want_state)
    assert values.dtype == np.dtype(dtype) and values.shape == (3, 1001)
    np.testing.assert_array_equal(values.view(np.uint8), np.asarray(want_values).view(np.uint8))


def test_rng_known_answers_statistics_and_state_advance(b200, backend):
    # published known-answer vectors of Philox4x32-10 (counter, key -> four words), through the whole stack
    S = lambda n: b200.Shape(b200.dtypes.Uint32, (n,))
    for ctr, key, want in (((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
                           ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
                           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0), (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))):
        state = np.array([key[0] | (key[1] << 32), ctr[0] | (ctr[1] << 32), ctr[2] | (ctr[3] << 32)], dtype=np.uint64)
        _, v = run_backend(b200, backend, lambda f, s: f.RNGBitGenerator(s, S(4)), [state])
        assert tuple(int(x) for x in v) == want
    # uniform floats: mean 1/2, variance 1/12, inside [0, 1); two draws chained through the returned state differ
    state = np.array([42, 0, 0], dtype=np.uint64)
    F = b200.Shape(b200.dtypes.Float32, (1 << 20,))

    def two_draws(f, s):
        s1, a = f.RNGBitGenerator(s, F)
        s2, b = f.RNGBitGenerator(s1, F)
        return a, b, s2
    a, b, s2 = run_backend(b200, backend, two_draws, [state])
    for v in (a, b):
        assert 0.0 <= v.min() and v.max() < 1.0
        assert abs(v.mean() - 0.5) < 2e-3 and abs(v.var() - 1 / 12) < 2e-3
    assert abs(np.corrcoef(a, b)[0, 1]) < 5e-3 and not np.array_equal(a, b)
    np.testing.assert_array_equal(s2, state + np.uint64(2))
    with pytest.raises(b200.BackendError, match=r"\[3\]"):
        run_backend(b200, backend, lambda f, s: f.RNGBitGenerator(s, F)[1], [np.zeros(4, np.uint64)])
