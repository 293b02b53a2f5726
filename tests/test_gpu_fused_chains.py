"""Fused elementwise chains and chain -> Reduce fusion through the run-time compiled kernels, against the CPU oracle.

A chain outside the two templated fast shapes is compiled at Compile() time into one straight-line kernel (the plan line
says "compiled"); a Reduce over one run of axes evaluates its elementwise operand inside the reduction kernel (the plan
line says "fused").  Checked here: one launch per chain, parity with the oracle (16-bit floats are rounded after every
op on both sides), bit-equality with the interpreter kernel the library falls back to without NVRTC, and the shapes
that switch code paths (broadcast / transposed / sliced leaves, misaligned operands, 64-bit types, every reduce type).
"""
import os

import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import compare
from tests.util import assert_parity, rng_array, run_backend, run_oracle

pytestmark = pytest.mark.gpu

BF16 = ml_dtypes.bfloat16


def _S(b200, dtype, *dims):
    return b200.Shape(b200.dtypes.from_numpy(np.dtype(dtype)), dims)


def _lines(plan):
    return [l for l in plan.strip().splitlines() if l.strip()]


def _chain4(b200, dt, R, C):
    """4 leaves, 6 ops: tanh((x * w + b) * y) - max(x, y) with a row vector w, a column vector b and a dense y."""
    full = _S(b200, dt, R, C)

    def build(f, x, w, b, y):
        t = f.Add(f.Mul(x, f.BroadcastInDim(w, full, [1])), f.BroadcastInDim(b, full, [0]))
        return f.Sub(f.Tanh(f.Mul(t, y)), f.Max(x, y))
    return build


@pytest.mark.parametrize("dt,rtol", [(np.float32, 2e-5), (BF16, 8e-3)], ids=["f32", "bf16"])
def test_general_chain_is_one_compiled_kernel(b200, backend, dt, rtol):
    rng = np.random.default_rng(100)
    R, C = 300, 1024
    x, y = rng_array(rng, (R, C), dt), rng_array(rng, (R, C), dt)
    w, b = rng_array(rng, (C,), dt), rng_array(rng, (R,), dt)
    build = _chain4(b200, dt, R, C)
    (got,), plan = run_backend(b200, backend, build, [x, w, b, y], describe=True)
    assert len(_lines(plan)) == 1 and "ewise[" in plan and "compiled" in plan, plan
    (want,) = run_oracle(build, [x, w, b, y])
    ok, viol = compare(got, want, rtol, 1.0)
    assert ok, viol
    # the interpreter kernel (what runs without NVRTC) computes the same ops with the same functions: equal bits,
    # up to the contraction of a multiply and an add INSIDE one op that the two compilers may choose differently (tanh)
    os.environ["B200MLX_JIT"] = "0"
    try:
        (interp,), plan0 = run_backend(b200, backend, build, [x, w, b, y], describe=True)
    finally:
        del os.environ["B200MLX_JIT"]
    assert "interpreted" in plan0, plan0
    ok, viol = compare(got, interp, 2e-6 if dt == np.float32 else 8e-3, 0.01)
    assert ok, viol


@pytest.mark.parametrize("dtype", [np.int8, np.int32, np.uint16, np.int64, np.float64, np.float16])
def test_chain_dtypes_compiled_equals_interpreted(b200, backend, dtype):
    rng = np.random.default_rng(101)
    a, b, c = (rng_array(rng, (37, 64), dtype) for _ in range(3))

    def build(f, x, y, z):
        t = f.Where(f.GreaterThan(x, y), f.Add(x, z), f.Sub(y, z))
        return f.Max(f.Mul(t, x), f.Min(y, z)), f.LessOrEqual(t, z)
    got = run_backend(b200, backend, build, [a, b, c])
    want = run_oracle(build, [a, b, c])
    for g, w in zip(got, want):
        ok, viol = compare(g, w, 1e-5 if np.dtype(dtype).kind == "f" else 0.0, 1.0)
        assert ok, viol
    os.environ["B200MLX_JIT"] = "0"
    try:
        interp = run_backend(b200, backend, build, [a, b, c])
    finally:
        del os.environ["B200MLX_JIT"]
    for g, i in zip(got, interp):
        np.testing.assert_array_equal(g, i)


def test_chain_with_transposed_sliced_reversed_and_iota_leaves(b200, backend):
    rng = np.random.default_rng(102)
    a = rng_array(rng, (48, 40), np.float32)       # read transposed
    b = rng_array(rng, (40, 100), np.float32)      # read through a slice with an odd start (misaligned vector loads)
    c = rng_array(rng, (40, 48), np.float32)       # read reversed along the last axis

    def build(f, x, y, z):
        xt = f.Transpose(x, 1, 0)
        ys = f.Slice(y, [0, 3], [40, 51], [1, 1])
        zr = f.Reverse(z, 1)
        io = f.ConvertDType(f.Iota(_S(b200, np.int32, 40, 48), 1), b200.dtypes.Float32)
        return f.Add(f.Mul(f.Add(xt, ys), zr), f.Exp(f.Neg(f.Abs(io))))
    assert_parity(b200, backend, build, [a, b, c], rtol=1e-5, atol_scale=0.01)


def test_chain_mixed_widths_and_a_scalar_leaf(b200, backend):
    # bf16 in, f32 out, Bool side result; a scalar leaf broadcast to every element
    rng = np.random.default_rng(103)
    x = rng_array(rng, (64, 520), BF16)
    s = np.array([0.5], dtype=np.float32)

    def build(f, a, sc):
        a32 = f.ConvertDType(a, b200.dtypes.Float32)
        scb = f.BroadcastInDim(f.Reshape(sc), _S(b200, np.float32, 64, 520), [])
        y = f.Mul(f.Logistic(a32), scb)
        return y, f.GreaterThan(y, scb)
    assert_parity(b200, backend, build, [x, s], rtol=2e-5, atol_scale=0.01)


# ------------------------------------------------------------------------------- reductions ---
def test_sum_of_squares_config_shape_is_one_fused_launch(b200, backend):
    rng = np.random.default_rng(104)
    x = rng_array(rng, (16384, 4096), BF16)
    build = lambda f, a: f.ReduceSum(f.Mul(a, a), 1)
    (got,), plan = run_backend(b200, backend, build, [x], describe=True)
    assert len(_lines(plan)) == 1 and "fused" in plan, plan
    (want,) = run_oracle(build, [x])
    ok, viol = compare(got, want, 8e-3, 0.0)   # products rounded to bf16 on both sides, fp32 / f64 sums, one final rounding
    assert ok, viol


@pytest.mark.parametrize("axes", [(2,), (0,), (1,), (1, 2), (0, 1), (0, 1, 2)], ids=str)
@pytest.mark.parametrize("op", ["ReduceSum", "ReduceMax", "ReduceMin", "ReduceProduct"])
def test_reduce_of_chain_over_any_run_of_axes(b200, backend, axes, op):
    rng = np.random.default_rng(105)
    x, y = rng_array(rng, (12, 40, 72), np.float32), rng_array(rng, (40, 72), np.float32)
    if op == "ReduceProduct":
        x, y = (1.0 + 0.01 * x).astype(np.float32), (0.02 * y).astype(np.float32)

    def build(f, a, b):
        return getattr(f, op)(f.Add(a, f.BroadcastInDim(b, _S(b200, np.float32, 12, 40, 72), [1, 2])), *axes)
    (got,), plan = run_backend(b200, backend, build, [x, y], describe=True)
    (want,) = run_oracle(build, [x, y])
    ok, viol = compare(got, want, 1e-5, 1.0)
    assert ok, (viol, plan)


@pytest.mark.parametrize("dtype", [np.int8, np.int32, np.uint8, np.int64, np.float64, BF16, np.float16, np.bool_], ids=lambda d: np.dtype(d).name)
def test_reduce_rows_and_cols_every_dtype(b200, backend, dtype):
    rng = np.random.default_rng(106)
    x = rng_array(rng, (300, 264), dtype) if np.dtype(dtype) != np.bool_ else (rng.integers(0, 8, size=(300, 264)) > 0)
    for axis in (0, 1):
        if np.dtype(dtype) == np.bool_:
            build = lambda f, a: (f.ReduceLogicalAnd(a, axis), f.ReduceLogicalOr(a, axis))
        else:
            build = lambda f, a: (f.ReduceSum(a, axis), f.ReduceMax(a, axis), f.ReduceMin(a, axis))
        got = run_backend(b200, backend, build, [x])
        want = run_oracle(build, [x])
        for g, w in zip(got, want):
            kind = np.dtype(dtype).kind
            ok, viol = compare(g, w, (1e-5 if np.dtype(dtype).itemsize >= 4 else 8e-3) if kind in "fV" else 0.0, 1.0)
            assert ok, (axis, viol)


def test_reduce_propagates_nan_and_handles_long_rows(b200, backend):
    rng = np.random.default_rng(107)
    x = rng_array(rng, (300, 40000), np.float32)     # long rows: one CTA per row
    x[5, 1234] = np.nan
    build = lambda f, a: (f.ReduceMax(a, 1), f.ReduceSum(f.Abs(a), 1))
    got = run_backend(b200, backend, build, [x])
    want = run_oracle(build, [x])
    for g, w in zip(got, want):
        ok, viol = compare(g, w, 1e-5, 1.0)
        assert ok, viol
    assert np.isnan(got[0][5]) and not np.isnan(got[0][6])


def test_reduce_that_needs_a_split_still_matches(b200, backend):
    # one row of 3 M elements: too little parallelism for the fused form, the split two-launch reduction runs instead
    rng = np.random.default_rng(108)
    x = rng_array(rng, (3_000_000,), np.float32)
    build = lambda f, a: f.ReduceSum(f.Mul(a, a))
    (got,), plan = run_backend(b200, backend, build, [x], describe=True)
    (want,) = run_oracle(build, [x])
    ok, viol = compare(got, want, 1e-5, 0.0)
    assert ok, (viol, plan)


# ------------------------------------------- LayerNorm and softmax spelled in primitives ---
def _scalar(b200, f, v, dt, dims):
    c = f.Constant(np.array([v], dtype=np.float32), 1)
    if np.dtype(dt) != np.float32:
        c = f.ConvertDType(c, b200.dtypes.from_numpy(np.dtype(dt)))
    return f.BroadcastInDim(f.Reshape(c), _S(b200, dt, *dims), [])


def _layer_norm_from_primitives(b200, spelling, dt, shape, eps, with_gamma, with_beta):
    """What a model emits when FusedLayerNorm is not offered: mean, centre, variance of the centred value, rsqrt, scale, shift
    (the chain of ref mpsgraph/gomlx/function.go:2430-2558), in the spellings GoMLX's helpers produce."""
    C, r = shape[-1], len(shape)
    keep = shape[:-1] + (1,)
    full = _S(b200, dt, *shape)
    lead = list(range(r - 1))

    def build(f, x, g, b):
        if spelling == "keepdims":          # ReduceAndKeep + implicit broadcast of the size-1 axis
            mean = f.Div(f.Reshape(f.ReduceSum(x, r - 1), *keep), _scalar(b200, f, float(C), dt, keep))
            d = f.Sub(x, mean)
            var = f.Div(f.Reshape(f.ReduceSum(f.Mul(d, d), r - 1), *keep), _scalar(b200, f, float(C), dt, keep))
            y = f.Mul(d, f.Rsqrt(f.Add(var, _scalar(b200, f, eps, dt, keep))))
        elif spelling == "broadcast":       # explicit BroadcastInDim back to the full shape, mean by Mul(1 / C)
            mean = f.BroadcastInDim(f.Mul(f.ReduceSum(x, r - 1), _scalar(b200, f, 1.0 / C, dt, shape[:-1])), full, lead)
            d = f.Sub(x, mean)
            var = f.Mul(f.ReduceSum(f.Mul(d, d), r - 1), _scalar(b200, f, 1.0 / C, dt, shape[:-1]))
            y = f.Mul(f.BroadcastInDim(f.Rsqrt(f.Add(var, _scalar(b200, f, eps, dt, shape[:-1]))), full, lead), d)
        else:                               # d / sqrt(var + eps)
            mean = f.Div(f.Reshape(f.ReduceSum(x, r - 1), *keep), _scalar(b200, f, float(C), dt, keep))
            d = f.Sub(x, mean)
            var = f.Div(f.ReduceSum(f.Mul(d, d), r - 1), _scalar(b200, f, float(C), dt, shape[:-1]))
            y = f.Div(d, f.BroadcastInDim(f.Sqrt(f.Add(var, _scalar(b200, f, eps, dt, shape[:-1]))), full, lead))
        if with_gamma:
            y = f.Mul(y, f.BroadcastInDim(g, full, [r - 1]))
        if with_beta:
            y = f.Add(y, f.BroadcastInDim(b, full, [r - 1]))
        return y
    return build


@pytest.mark.parametrize("spelling", ["keepdims", "broadcast", "div_sqrt"])
@pytest.mark.parametrize("dt", [np.float32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("with_gamma,with_beta", [(True, True), (True, False), (False, False)])
def test_layer_norm_from_primitives_is_one_kernel(b200, backend, spelling, dt, with_gamma, with_beta):
    rng = np.random.default_rng(110)
    shape = (3, 7, 256)
    x = (rng_array(rng, shape, np.float32) + 0.5).astype(dt)
    g = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32).astype(dt)
    b = (0.1 * rng.standard_normal(256)).astype(np.float32).astype(dt)
    build = _layer_norm_from_primitives(b200, spelling, dt, shape, 1e-5, with_gamma, with_beta)
    (got,), plan = run_backend(b200, backend, build, [x, g, b], describe=True)
    assert len(_lines(plan)) == 1 and "layer_norm[" in plan, plan
    assert f"gamma={int(with_gamma)} beta={int(with_beta)}" in plan, plan
    (want,) = run_oracle(build, [x, g, b])
    # 16-bit: the chain rounds the mean, the centred value and every later step to 8 bits, so its absolute error is a few
    # 2^-9 of the ROW's scale even where the result is near zero: norm-relative tolerance
    ok, viol = compare(got, want, 1e-5 if dt == np.float32 else 2e-2, 0.05 if dt == np.float32 else 1.0)
    assert ok, viol
    (fused,) = run_backend(b200, backend, lambda f, a, gg, bb: f.FusedLayerNorm(a, [-1], 1e-5, gg if with_gamma else None, bb if with_beta else None),
                           [x, g, b])
    np.testing.assert_array_equal(got, fused)


def test_layer_norm_lookalikes_are_left_alone(b200, backend):
    rng = np.random.default_rng(111)
    x = rng_array(rng, (6, 8, 16), np.float32)
    keep = (6, 8, 1)

    def wrong_mean_scale(f, a):     # subtracts sum / (C + 1), not the mean
        m = f.Div(f.Reshape(f.ReduceSum(a, 2), *keep), _scalar(b200, f, 17.0, np.float32, keep))
        d = f.Sub(a, m)
        v = f.Div(f.Reshape(f.ReduceSum(f.Mul(d, d), 2), *keep), _scalar(b200, f, 16.0, np.float32, keep))
        return f.Mul(d, f.Rsqrt(f.Add(v, _scalar(b200, f, 1e-5, np.float32, keep))))

    def mean_of_another_tensor(f, a):   # centres on the mean of 2a
        a2 = f.Add(a, a)
        m = f.Div(f.Reshape(f.ReduceSum(a2, 2), *keep), _scalar(b200, f, 16.0, np.float32, keep))
        d = f.Sub(a, m)
        v = f.Div(f.Reshape(f.ReduceSum(f.Mul(d, d), 2), *keep), _scalar(b200, f, 16.0, np.float32, keep))
        return f.Mul(d, f.Rsqrt(f.Add(v, _scalar(b200, f, 1e-5, np.float32, keep))))

    def stats_over_axis_1(f, a):    # the middle axis, not the last
        k1 = (6, 1, 16)
        m = f.Div(f.Reshape(f.ReduceSum(a, 1), *k1), _scalar(b200, f, 8.0, np.float32, k1))
        d = f.Sub(a, m)
        v = f.Div(f.Reshape(f.ReduceSum(f.Mul(d, d), 1), *k1), _scalar(b200, f, 8.0, np.float32, k1))
        return f.Mul(d, f.Rsqrt(f.Add(v, _scalar(b200, f, 1e-5, np.float32, k1))))

    for build in (wrong_mean_scale, mean_of_another_tensor, stats_over_axis_1):
        (got,), plan = run_backend(b200, backend, build, [x], describe=True)
        assert "layer_norm[" not in plan, (build.__name__, plan)
        (want,) = run_oracle(build, [x])
        ok, viol = compare(got, want, 1e-5, 0.05)
        assert ok, (build.__name__, viol)


def _softmax_from_primitives(b200, dt, shape, explicit_broadcast):
    r = len(shape)
    keep = shape[:-1] + (1,)
    full = _S(b200, dt, *shape)
    lead = list(range(r - 1))

    def build(f, x):
        if explicit_broadcast:
            m = f.BroadcastInDim(f.ReduceMax(x, r - 1), full, lead)
            e = f.Exp(f.Sub(x, m))
            return f.Div(e, f.BroadcastInDim(f.ReduceSum(e, r - 1), full, lead))
        m = f.Identity(f.Reshape(f.ReduceMax(x, r - 1), *keep))     # StopGradient reaches a backend as Identity
        e = f.Exp(f.Sub(x, m))
        return f.Div(e, f.Reshape(f.ReduceSum(e, r - 1), *keep))
    return build


@pytest.mark.parametrize("explicit_broadcast", [False, True], ids=["keepdims", "broadcast"])
@pytest.mark.parametrize("dt", [np.float32, BF16], ids=["f32", "bf16"])
def test_softmax_from_primitives_is_one_kernel(b200, backend, dt, explicit_broadcast):
    rng = np.random.default_rng(112)
    shape = (4, 9, 200)
    x = rng_array(rng, shape, dt, 2.0)
    build = _softmax_from_primitives(b200, dt, shape, explicit_broadcast)
    (got,), plan = run_backend(b200, backend, build, [x], describe=True)
    assert len(_lines(plan)) == 1 and "softmax" in plan, plan
    (want,) = run_oracle(build, [x])
    # 16-bit: the chain rounds x - max, the exponentials and their sum to 8 bits each; norm-relative tolerance
    ok, viol = compare(got, want, 1e-5 if dt == np.float32 else 2e-2, 0.01 if dt == np.float32 else 1.0)
    assert ok, viol
    (fused,) = run_backend(b200, backend, lambda f, a: f.FusedSoftmax(a, 2), [x])
    np.testing.assert_array_equal(got, fused)


def test_softmax_lookalikes_are_left_alone(b200, backend):
    rng = np.random.default_rng(113)
    x = rng_array(rng, (5, 6, 32), np.float32)
    keep = (5, 6, 1)

    def shifted_by_min(f, a):        # subtracts the row minimum
        e = f.Exp(f.Sub(a, f.Reshape(f.ReduceMin(a, 2), *keep)))
        return f.Div(e, f.Reshape(f.ReduceSum(e, 2), *keep))

    def normalised_by_another_sum(f, a):   # divides by the sum of exp(2 (x - max))
        d = f.Sub(a, f.Reshape(f.ReduceMax(a, 2), *keep))
        e, e2 = f.Exp(d), f.Exp(f.Add(d, d))
        return f.Div(e, f.Reshape(f.ReduceSum(e2, 2), *keep))

    def over_the_middle_axis(f, a):
        k1 = (5, 1, 32)
        e = f.Exp(f.Sub(a, f.Reshape(f.ReduceMax(a, 1), *k1)))
        return f.Div(e, f.Reshape(f.ReduceSum(e, 1), *k1))

    for build in (shifted_by_min, normalised_by_another_sum, over_the_middle_axis):
        (got,), plan = run_backend(b200, backend, build, [x], describe=True)
        assert "softmax" not in plan, (build.__name__, plan)
        (want,) = run_oracle(build, [x])
        ok, viol = compare(got, want, 1e-5, 0.01)
        assert ok, (build.__name__, viol)
