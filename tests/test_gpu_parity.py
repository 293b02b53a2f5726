"""Parity of the CUDA path against the CPU oracle on seeded inputs, through the C ABI.

Tolerances (stated by the target): bit-exact for integer, Bool and indexing results; rel 1e-5 for
fp32; rel 2e-2 for bf16 contractions.  Float comparisons add a norm-relative term (atol_scale * rtol
* rms(expected)) because the elementwise relative error of a zero-mean sum is unbounded.
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import compare
from tests.util import default_switches, assert_parity, rng_array, run_backend, run_oracle

pytestmark = pytest.mark.gpu

BF16 = ml_dtypes.bfloat16
F32_RTOL, BF16_RTOL = 1e-5, 2e-2


# --------------------------------------------------------------------------- elementwise ---
UNARY_F = ["Abs", "Neg", "Sqrt", "Rsqrt", "Exp", "Expm1", "Log", "Log1p", "Sin", "Cos", "Tanh", "Logistic", "Erf", "Floor", "Ceil",
           "Round", "Sign", "Identity"]


@pytest.mark.parametrize("op", UNARY_F)
@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
def test_unary_float(b200, backend, op, dtype):
    rng = np.random.default_rng(1)
    x = rng_array(rng, (37, 52), np.float32, 2.0)
    if op in ("Sqrt", "Rsqrt", "Log"):
        x = np.abs(x) + 0.1
    if op == "Log1p":
        x = np.abs(x)
    x = x.astype(dtype)
    rtol = 2e-5 if dtype == np.float32 else 8e-3   # bf16: half an ulp is 2^-9
    assert_parity(b200, backend, lambda f, a: getattr(f, op)(a), [x], rtol=rtol, atol_scale=1.0 if op in ("Expm1", "Log1p", "Sin", "Cos") else 0.01, what=op)


def test_round_ties_to_even(b200, backend):
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 3.5000002, 2.4999998], dtype=np.float32)
    got = run_backend(b200, backend, lambda f, a: f.Round(a), [x])[0]
    np.testing.assert_array_equal(got, np.rint(x))


BINARY_F = ["Add", "Sub", "Mul", "Div", "Max", "Min", "Pow", "Atan2", "Rem"]


@pytest.mark.parametrize("op", BINARY_F)
def test_binary_float_broadcast(b200, backend, op):
    rng = np.random.default_rng(2)
    a = rng_array(rng, (5, 1, 33), np.float32)
    b = rng_array(rng, (7, 33), np.float32)
    if op == "Pow":
        a = np.abs(a) + 0.5
    if op in ("Div", "Rem"):
        b = np.where(np.abs(b) < 0.1, 0.5, b).astype(np.float32)
    assert_parity(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, b], rtol=3e-5 if op == "Pow" else F32_RTOL,
                  atol_scale=1.0 if op == "Rem" else 0.0, what=op)


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32, np.int64, np.uint8, np.uint16, np.uint32, np.uint64])
@pytest.mark.parametrize("op", ["Add", "Sub", "Mul", "Div", "Rem", "Max", "Min", "BitwiseAnd", "BitwiseOr", "BitwiseXor"])
def test_binary_integer_exact(b200, backend, dtype, op):
    rng = np.random.default_rng(3)
    a = rng_array(rng, (64,), dtype)
    b = rng_array(rng, (64,), dtype)
    b[::7] = 0  # division by zero is defined: quotient all-ones, remainder the dividend
    assert_parity(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, b], what=f"{op}/{np.dtype(dtype).name}")


@pytest.mark.parametrize("dtype", [np.int32, np.uint8, np.int64])
@pytest.mark.parametrize("op", ["ShiftLeft", "ShiftRightArithmetic", "ShiftRightLogical"])
def test_shifts_exact(b200, backend, dtype, op):
    rng = np.random.default_rng(4)
    a = rng_array(rng, (40,), dtype)
    s = rng.integers(0, np.dtype(dtype).itemsize * 8 + 3, size=40).astype(dtype)
    assert_parity(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, s], what=op)


@pytest.mark.parametrize("op", ["Equal", "NotEqual", "LessThan", "LessOrEqual", "GreaterThan", "GreaterOrEqual"])
@pytest.mark.parametrize("dtype", [np.float32, np.int32, BF16], ids=["f32", "i32", "bf16"])
def test_compare_exact(b200, backend, op, dtype):
    rng = np.random.default_rng(5)
    a = rng.integers(-3, 4, size=(9, 31)).astype(np.float32).astype(dtype)
    b = rng.integers(-3, 4, size=(31,)).astype(np.float32).astype(dtype)
    assert_parity(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, b], what=op)


def test_logical_ops_exact(b200, backend):
    rng = np.random.default_rng(6)
    a, b = rng_array(rng, (50,), np.bool_), rng_array(rng, (50,), np.bool_)
    for op in ("LogicalAnd", "LogicalOr", "LogicalXor"):
        assert_parity(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, b], what=op)
    assert_parity(b200, backend, lambda f, x: f.LogicalNot(x), [a], what="LogicalNot")


def test_isfinite_isnan(b200, backend):
    x = np.array([0.0, np.inf, -np.inf, np.nan, 1.5, -2.0], dtype=np.float32)
    assert_parity(b200, backend, lambda f, a: (f.IsFinite(a), f.IsNaN(a)), [x])


def test_where_clamp(b200, backend):
    rng = np.random.default_rng(7)
    c = rng_array(rng, (6, 20), np.bool_)
    a, b = rng_array(rng, (6, 20), np.float32), rng_array(rng, (20,), np.float32)
    assert_parity(b200, backend, lambda f, cc, x, y: f.Where(cc, x, f.BroadcastInDim(y, _S(b200, np.float32, 6, 20), [1])), [c, a, b])
    lo, hi = np.array(-0.5, dtype=np.float32), np.array(0.25, dtype=np.float32)
    assert_parity(b200, backend, lambda f, l, x, h: f.Clamp(l, x, h), [lo, a, hi])


def _S(b200, dtype, *dims):
    return b200.Shape(b200.dtypes.from_numpy(np.dtype(dtype)), dims)


@pytest.mark.parametrize("src,dst", [(np.float32, np.int32), (np.float32, np.int8), (np.float32, np.uint8), (np.float32, np.int64),
                                     (np.int32, np.float32), (np.int64, np.float32), (np.float32, BF16), (BF16, np.float32),
                                     (np.int32, np.int8), (np.uint8, np.int32), (np.float32, np.bool_), (np.int32, np.bool_),
                                     (np.float32, np.float64), (np.float64, np.float32), (np.float32, np.float16)])
def test_convert_dtype(b200, backend, src, dst):
    rng = np.random.default_rng(8)
    x = rng_array(rng, (300,), src, 100.0)
    if np.dtype(src).kind == "f" or np.dtype(src) == np.dtype(BF16):
        x[:4] = np.array([1e10, -1e10, 0.0, -0.0], dtype=np.float32).astype(src)
    assert_parity(b200, backend, lambda f, a: f.ConvertDType(a, b200.dtypes.from_numpy(np.dtype(dst))), [x], rtol=0.0, what=f"{src}->{dst}")


def test_fused_chain_is_one_launch(b200, backend):
    rng = np.random.default_rng(9)
    x, w, b = rng_array(rng, (64, 128), np.float32), rng_array(rng, (128,), np.float32), rng_array(rng, (128,), np.float32)

    def build(f, xx, ww, bb):
        s = _S(b200, np.float32, 64, 128)
        return f.Tanh(f.Add(f.Mul(xx, f.BroadcastInDim(ww, s, [1])), f.BroadcastInDim(bb, s, [1])))

    (got,), plan = run_backend(b200, backend, build, [x, w, b], describe=True)
    assert plan.count("\n") == 1 and plan.startswith("ewise["), plan
    want = np.tanh((x.astype(np.float64) * w + b).astype(np.float32).astype(np.float64)).astype(np.float32)
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-6)


def test_bf16_chain_rounds_after_every_op(b200, backend):
    # a fused chain must equal the op-by-op result, so 16-bit intermediates are re-rounded
    rng = np.random.default_rng(10)
    a, b, c = (rng_array(rng, (1000,), BF16) for _ in range(3))
    assert_parity(b200, backend, lambda f, x, y, z: f.Mul(f.Add(x, y), z), [a, b, c], rtol=0.0, what="bf16 chain")


def test_iota_inside_chain_and_causal_mask_from_primitives(b200, backend):
    # the reference's SDPA builds its causal mask from two Int32 iotas and GreaterOrEqual (function.go:2777-2794)
    S = 19
    x = rng_array(np.random.default_rng(11), (3, S, S), np.float32)

    def build(f, s):
        shp = _S(b200, np.int32, S, S)
        keep = f.GreaterOrEqual(f.Iota(shp, 0), f.Iota(shp, 1))
        keep3 = f.BroadcastInDim(keep, _S(b200, np.bool_, 3, S, S), [1, 2])
        neg = f.BroadcastInDim(f.Constant(np.array([-np.inf], dtype=np.float32), 1), _S(b200, np.float32, 3, S, S), [2])
        return f.FusedSoftmax(f.Where(keep3, s, neg), 2)

    assert_parity(b200, backend, build, [x], rtol=F32_RTOL, atol_scale=0.01)


# ------------------------------------------------------------------------ data movement ---
@pytest.mark.parametrize("perm", [(1, 0), (0, 2, 1), (2, 0, 1), (0, 2, 1, 3), (3, 2, 1, 0)])
@pytest.mark.parametrize("dtype", [np.float32, BF16, np.int8, np.int64], ids=["f32", "bf16", "i8", "i64"])
def test_transpose_exact(b200, backend, perm, dtype):
    dims = (6, 10, 7, 16)[:len(perm)]
    x = rng_array(np.random.default_rng(12), dims, dtype)
    assert_parity(b200, backend, lambda f, a: f.Transpose(a, *perm), [x], what=f"Transpose{perm}")


def test_slice_reverse_concat_pad_broadcast_exact(b200, backend):
    rng = np.random.default_rng(13)
    x = rng_array(rng, (9, 12, 8), np.float32)
    y = rng_array(rng, (9, 5, 8), np.float32)
    assert_parity(b200, backend, lambda f, a: f.Slice(a, [1, 2, 0], [9, 11, 8], [2, 3, 1]), [x])
    assert_parity(b200, backend, lambda f, a: f.Reverse(a, 0, 2), [x])
    assert_parity(b200, backend, lambda f, a, b: f.Concatenate(1, a, b, a), [x, y])
    assert_parity(b200, backend, lambda f, a: f.Pad(a, f.Constant(np.array([7.0], dtype=np.float32)), (1, 2), (0, 0), (3, 0)), [x])
    assert_parity(b200, backend, lambda f, a: f.BroadcastInDim(a, _S(b200, np.float32, 4, 9, 5, 8), [1, 2, 3]), [y])
    # movement feeding arithmetic is folded into the consumer
    assert_parity(b200, backend, lambda f, a: f.Add(f.Transpose(a, 2, 1, 0), f.Transpose(a, 2, 1, 0)), [x], rtol=0.0)


def test_empty_and_scalar_shapes(b200, backend):
    s = np.array(3.5, dtype=np.float32)
    assert_parity(b200, backend, lambda f, a: f.Mul(a, a), [s], rtol=0.0)
    e = np.zeros((0, 4), dtype=np.float32)
    got = run_backend(b200, backend, lambda f, a: f.Exp(a), [e])[0]
    assert got.shape == (0, 4)
    got = run_backend(b200, backend, lambda f, a: f.ReduceSum(a, 0), [e])[0]
    np.testing.assert_array_equal(got, np.zeros(4, dtype=np.float32))


# --------------------------------------------------------------------------- reductions ---
@pytest.mark.parametrize("op", ["ReduceSum", "ReduceMax", "ReduceMin", "ReduceProduct"])
@pytest.mark.parametrize("axes", [(), (0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2)])
def test_reduce_float(b200, backend, op, axes):
    x = rng_array(np.random.default_rng(14), (7, 33, 20), np.float32, 0.9 if op == "ReduceProduct" else 1.0)
    if op == "ReduceProduct":
        x = (1.0 + 0.01 * x).astype(np.float32)
    assert_parity(b200, backend, lambda f, a: getattr(f, op)(a, *axes), [x], rtol=2e-5, atol_scale=1.0, what=f"{op}{axes}")


def test_reduce_large_uses_split_path(b200, backend):
    x = rng_array(np.random.default_rng(15), (3, 200_000), np.float32)
    (got,), plan = run_backend(b200, backend, lambda f, a: f.ReduceSum(a, 1), [x], describe=True)
    assert "split" in plan
    np.testing.assert_allclose(got, x.astype(np.float64).sum(axis=1), rtol=1e-5, atol=1e-2)
    x2 = rng_array(np.random.default_rng(16), (50_000, 6), np.float32)
    assert_parity(b200, backend, lambda f, a: f.ReduceMax(a, 0), [x2], rtol=0.0)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.uint8, np.int8])
def test_reduce_integer_exact(b200, backend, dtype):
    x = rng_array(np.random.default_rng(17), (11, 300), dtype)
    for op in ("ReduceSum", "ReduceMax", "ReduceMin"):
        assert_parity(b200, backend, lambda f, a: getattr(f, op)(a, 1), [x], what=op)


def test_reduce_logical(b200, backend):
    x = rng_array(np.random.default_rng(18), (9, 40), np.bool_)
    x[3] = True
    x[5] = False
    assert_parity(b200, backend, lambda f, a: (f.ReduceLogicalAnd(a, 1), f.ReduceLogicalOr(a, 1)), [x])


@pytest.mark.parametrize("axis", [0, 1, 2])
@pytest.mark.parametrize("is_min", [False, True])
@pytest.mark.parametrize("dtype", [np.float32, BF16, np.int32], ids=["f32", "bf16", "i32"])
def test_argminmax_exact(b200, backend, axis, is_min, dtype):
    x = rng_array(np.random.default_rng(19), (6, 301, 5), dtype)
    assert_parity(b200, backend, lambda f, a: f.ArgMinMax(a, axis, b200.dtypes.Int32, is_min), [x])


def test_argmax_ties_and_nan(b200, backend):
    x = np.array([[1, 7, 7, 3], [np.nan, 9, np.nan, 2], [5, 5, 5, 5]], dtype=np.float32)
    got = run_backend(b200, backend, lambda f, a: f.ArgMinMax(a, 1, b200.dtypes.Int64, False), [x])[0]
    np.testing.assert_array_equal(got, np.array([1, 0, 0], dtype=np.int64))  # lowest index on ties; first NaN wins


@pytest.mark.parametrize("rows,n", [(1, 8192), (3, 8191), (16, 50257), (2, 1000003), (147, 9000), (200, 9000)])
@pytest.mark.parametrize("dtype", [np.float32, BF16, np.int64, np.float64], ids=["f32", "bf16", "i64", "f64"])
def test_argminmax_long_rows_split_over_a_cluster(b200, backend, rows, n, dtype):
    # few, long rows: each row is scanned by several CTAs whose winners meet in one; ties across the CTAs' shares
    # must still go to the lowest index, and a NaN anywhere wins
    rng = np.random.default_rng(rows + n)
    x = rng_array(rng, (rows, n), dtype)
    if np.dtype(dtype).kind == "f":
        x = np.round(x.astype(np.float32) * 2).astype(dtype)   # few distinct values: many ties
        if rows > 2:
            x[1, n - 5] = np.nan
            x[2, 7] = np.nan
            x[2, n // 2] = np.nan
    for is_min in (False, True):
        assert_parity(b200, backend, lambda f, a: f.ArgMinMax(a, 1, b200.dtypes.Int32, is_min), [x])


def test_argmax_vocab_sized_rows(b200, backend):
    x = rng_array(np.random.default_rng(20), (4, 50257), np.float32)
    assert_parity(b200, backend, lambda f, a: f.ArgMinMax(a, -1 + 2, b200.dtypes.Int32, False), [x])


# ------------------------------------------------------------------------------- gather ---
def test_gather_embedding_rows_bf16(b200, backend):
    rng = np.random.default_rng(21)
    table = rng_array(rng, (1000, 768), BF16)
    ids = rng.integers(0, 1000, size=(4, 33, 1)).astype(np.int32)
    (got,), plan = run_backend(b200, backend, lambda f, t, i: f.Gather(t, i, 2, [2], [0], [0], [1, 768], False), [table, ids], describe=True)
    assert "gather_rows" in plan
    np.testing.assert_array_equal(got.view(np.uint16), table[ids[..., 0]].view(np.uint16))


def test_gather_clamps_out_of_range(b200, backend):
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    ids = np.array([[-5], [99], [2]], dtype=np.int32)
    assert_parity(b200, backend, lambda f, t, i: f.Gather(t, i, 1, [1], [0], [0], [1, 3], False), [table, ids])


def test_gather_general_windows(b200, backend):
    rng = np.random.default_rng(22)
    op = rng_array(rng, (6, 7, 8), np.float32)
    idx = rng.integers(0, 5, size=(5, 2)).astype(np.int32)
    # windows of [2, 7, 3] starting at (i, *, j)
    assert_parity(b200, backend, lambda f, t, i: f.Gather(t, i, 1, [1, 2, 3], [], [0, 2], [2, 7, 3], False), [op, idx])


# ----------------------------------------------------------------------------- softmax ---
@pytest.mark.parametrize("shape,axis", [((33, 1024), 1), ((5, 7, 96), 2), ((4, 50257), 1), ((6, 100, 12), 1), ((3, 4096), 1), ((2, 20000), 1),
                                        ((8, 17), 1)])
@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
def test_softmax(b200, backend, shape, axis, dtype):
    x = rng_array(np.random.default_rng(23), shape, dtype, 2.0)
    rtol = F32_RTOL if dtype == np.float32 else 8e-3
    assert_parity(b200, backend, lambda f, a: f.FusedSoftmax(a, axis), [x], rtol=rtol, atol_scale=0.01, what=f"softmax{shape}")


@pytest.mark.parametrize("sq,sk", [(64, 64), (128, 1024), (100, 100), (1024, 1024)])
def test_softmax_causal(b200, backend, sq, sk):
    x = rng_array(np.random.default_rng(24), (2, 3, sq, sk), np.float32, 2.0)
    got = assert_parity(b200, backend, lambda f, a: f.FusedSoftmaxMasked(a, 0.125, True, None), [x], rtol=F32_RTOL, atol_scale=0.01)[0]
    # masked positions are exactly zero, rows sum to one
    iu = np.triu_indices(sq, 1, sk)
    assert (got[..., iu[0], iu[1]] == 0).all()
    np.testing.assert_allclose(got.sum(-1), 1.0, rtol=1e-5)


def test_softmax_masks(b200, backend):
    rng = np.random.default_rng(25)
    x = rng_array(rng, (2, 3, 40, 48), np.float32)
    bm = rng.integers(0, 4, size=(2, 1, 40, 48)) > 0
    bm[..., 0] = True
    fm = rng_array(rng, (40, 48), np.float32)
    assert_parity(b200, backend, lambda f, a, m: f.FusedSoftmaxMasked(a, 1.0, False, m), [x, bm], rtol=F32_RTOL, atol_scale=0.01)
    assert_parity(b200, backend, lambda f, a, m: f.FusedSoftmaxMasked(a, 0.5, True, m), [x, fm], rtol=F32_RTOL, atol_scale=0.01)
    # a fully masked row is NaN (IEEE), as the oracle defines
    bm2 = bm.copy()
    bm2[0, 0, 5, :] = False
    assert_parity(b200, backend, lambda f, a, m: f.FusedSoftmaxMasked(a, 1.0, False, m), [x, bm2], rtol=F32_RTOL, atol_scale=0.01)


# ------------------------------------------------------------------------------- norms ---
@pytest.mark.parametrize("rows,cols", [(64, 4096), (33, 768), (17, 2048), (5, 100), (3, 16384), (2, 40000), (9, 8)])
@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("kind", ["layer", "rms"])
def test_norms(b200, backend, rows, cols, dtype, kind):
    rng = np.random.default_rng(26)
    x = rng_array(rng, (rows, cols), dtype)
    g = (1.0 + 0.02 * rng.standard_normal(cols)).astype(np.float32).astype(dtype)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32).astype(dtype)
    rtol = 2e-5 if dtype == np.float32 else 8e-3
    if kind == "layer":
        assert_parity(b200, backend, lambda f, a, gg, bb: f.FusedLayerNorm(a, [-1], 1e-6, gg, bb), [x, g, b], rtol=rtol, atol_scale=0.05)
    else:
        assert_parity(b200, backend, lambda f, a, gg: f.FusedRMSNorm(a, [-1], 1e-6, gg), [x, g], rtol=rtol, atol_scale=0.05)


def test_layer_norm_axes_and_param_shapes(b200, backend):
    rng = np.random.default_rng(27)
    x = rng_array(rng, (4, 6, 10), np.float32)
    g2 = rng_array(rng, (6, 10), np.float32)
    assert_parity(b200, backend, lambda f, a, g: f.FusedLayerNorm(a, [1, 2], 1e-5, g, None), [x, g2], rtol=2e-5, atol_scale=0.05)
    assert_parity(b200, backend, lambda f, a: f.FusedLayerNorm(a, [1], 1e-5, None, None), [x], rtol=2e-5, atol_scale=0.05)   # non-trailing axis
    g_full = rng_array(rng, (1, 1, 10), np.float32)
    assert_parity(b200, backend, lambda f, a, g: f.FusedLayerNorm(a, [-1], 1e-5, g, g), [x, g_full], rtol=2e-5, atol_scale=0.05)
    g_rows = rng_array(rng, (4, 1, 10), np.float32)  # varies off the normalised axis -> split into norm + mul
    assert_parity(b200, backend, lambda f, a, g: f.FusedLayerNorm(a, [-1], 1e-5, g, None), [x, g_rows], rtol=2e-5, atol_scale=0.05)


def test_gelu_both_forms(b200, backend):
    x = rng_array(np.random.default_rng(28), (1000,), np.float32, 2.0)
    assert_parity(b200, backend, lambda f, a: f.FusedGelu(a, True), [x], rtol=2e-5, atol_scale=0.01)
    assert_parity(b200, backend, lambda f, a: f.FusedGelu(a, False), [x], rtol=2e-5, atol_scale=0.01)


# -------------------------------------------------------------------------- DotGeneral ---
def _dot_tol(dtype):
    return (F32_RTOL, 1.0) if dtype == np.float32 else (BF16_RTOL, 1.0)


@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("form", ["BMK_BKN", "BKM_BKN", "BMK_BNK", "BKM_BNK"])
# the last two run on CTA pairs (256-row tiles; chosen for K >= 1024 and >= 32 tiles): a ragged last pair (its second CTA has
# no rows) with a ragged last column tile, and more tiles than resident pairs (both accumulators and every ring phase reused)
@pytest.mark.parametrize("B,M,N,K", [(1, 2, 2, 3), (2, 64, 48, 40), (3, 130, 70, 257), (2, 256, 256, 128), (1, 512, 384, 1024),
                                     (2, 392, 520, 192), (2, 1096, 1032, 1024), (4, 1280, 1024, 1024)])
def test_dot_general_forms(b200, backend, dtype, form, B, M, N, K):
    rng = np.random.default_rng(29)
    a = rng_array(rng, (B, M, K) if form.startswith("BMK") else (B, K, M), dtype)
    b = rng_array(rng, (B, K, N) if form.endswith("BKN") else (B, N, K), dtype)
    lc = [2] if form.startswith("BMK") else [1]
    rc = [1] if form.endswith("BKN") else [2]
    rtol, ascale = _dot_tol(dtype)
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, lc, [0], y, rc, [0]), [a, b], rtol=rtol, atol_scale=ascale, what=form)


def test_dot_general_needs_operand_copy(b200, backend):
    rng = np.random.default_rng(30)
    a = rng_array(rng, (5, 3, 7, 4), np.float32)   # [m1, b, k, m2]
    b = rng_array(rng, (7, 3, 6), np.float32)      # [k, b, n]
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, [2], [1], y, [0], [1]), [a, b], rtol=F32_RTOL, atol_scale=1.0)
    c = rng_array(rng, (4, 5, 6), np.float32)
    d = rng_array(rng, (6, 5, 3), np.float32)
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, [1, 2], [], y, [1, 0], []), [c, d], rtol=F32_RTOL, atol_scale=1.0)


@pytest.mark.parametrize("dtype", [np.int32, np.int64, np.float64])
def test_dot_general_other_dtypes(b200, backend, dtype):
    rng = np.random.default_rng(31)
    a, b = rng_array(rng, (9, 20), dtype), rng_array(rng, (20, 11), dtype)
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, [1], [], y, [0], []), [a, b], rtol=1e-12, atol_scale=1.0)


@pytest.mark.parametrize("act", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
def test_fused_dense(b200, backend, act, dtype):
    rng = np.random.default_rng(32)
    x, w, b = rng_array(rng, (4, 50, 96), dtype), rng_array(rng, (96, 160), dtype, 0.1), rng_array(rng, (160,), dtype)
    rtol, ascale = _dot_tol(dtype)
    assert_parity(b200, backend, lambda f, xx, ww, bb: f.FusedDense(xx, ww, bb, act), [x, w, b], rtol=rtol, atol_scale=ascale)


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("heads,kv_heads", [(4, 4), (8, 2)])
@pytest.mark.parametrize("causal", [False, True])
def test_sdpa(b200, backend, layout, heads, kv_heads, causal):
    rng = np.random.default_rng(33)
    B, S, D = 2, 48, 16
    shp = lambda h: (B, h, S, D) if layout == 0 else (B, S, h, D)
    q, k, v = rng_array(rng, shp(heads), np.float32), rng_array(rng, shp(kv_heads), np.float32), rng_array(rng, shp(kv_heads), np.float32)
    assert_parity(b200, backend,
                  lambda f, qq, kk, vv: f.FusedScaledDotProductAttention(qq, kk, vv, None, heads, kv_heads, layout, 0.25, causal),
                  [q, k, v], rtol=2e-5, atol_scale=1.0)


def test_qkv_projection(b200, backend):
    rng = np.random.default_rng(34)
    x, w = rng_array(rng, (3, 10, 32), np.float32), rng_array(rng, (32, 64 + 2 * 16), np.float32, 0.2)
    bq, bk, bv = rng_array(rng, (64,), np.float32), rng_array(rng, (16,), np.float32), rng_array(rng, (16,), np.float32)
    assert_parity(b200, backend, lambda f, xx, ww, a, b, c: f.FusedAttentionQKVProjection(xx, ww, a, b, c, 64, 16), [x, w, bq, bk, bv],
                  rtol=F32_RTOL, atol_scale=1.0)


# ----------------------------------------------------------------- boundary behaviour ---
def test_error_behaviour_matches_the_reference(b200, backend):
    builder = backend.Builder("errors")
    f = builder.Main()
    x = f.Parameter("x", b200.shapes.Make(b200.dtypes.Float32, 2, 3))
    w = f.Parameter("w", b200.shapes.Make(b200.dtypes.Float32, 4, 5))
    with pytest.raises(b200.BackendError, match="must match weight's first dim"):   # ref function.go:2582-2585
        f.FusedDense(x, w, None, 0)
    with pytest.raises(b200.BackendError, match="unsupported activation"):          # ref function.go:2662
        f.FusedDense(x, f.Constant(np.zeros(15, dtype=np.float32), 3, 5), None, 17)
    with pytest.raises(b200.BackendError, match="out of range"):                      # ref function.go:2423-2425
        f.FusedLayerNorm(x, [5], 1e-5, None, None)
    with pytest.raises(b200.BackendError, match="rank 4"):                            # ref function.go:2690-2692
        f.FusedScaledDotProductAttention(x, x, x, None, 1, 1, 0, 1.0, False)
    with pytest.raises(b200.BackendError, match="no outputs"):                        # ref builder.go:79-81
        builder.Compile()
    other = backend.Builder("other").Main()
    with pytest.raises(b200.BackendError, match="unrelated function scope"):          # ref function.go:194
        f.Add(x, other.Parameter("y", b200.shapes.Make(b200.dtypes.Float32, 2, 3)))
    f.Return([f.Add(x, x)], None)
    exe = builder.Compile()
    with pytest.raises(b200.BackendError, match="already been compiled"):             # ref builder.go:73-75
        builder.Compile()
    with pytest.raises(b200.BackendError, match="expected 2 inputs"):                 # ref executable.go:55-58
        exe.Execute([], None, 0)
    bad = backend.FromNumpy(np.zeros((3, 2), dtype=np.float32))
    good = backend.FromNumpy(np.zeros((4, 5), dtype=np.float32))
    with pytest.raises(b200.BackendError, match="shape mismatch"):                    # ref executable.go:66-72
        exe.Execute([bad, good], None, 0)
    backend.BufferFinalize(bad)
    with pytest.raises(b200.BackendError, match="finalized"):
        backend.BufferShape(bad)
    assert backend.HasSharedBuffers() is False
    with pytest.raises(b200.BackendError):
        backend.NewSharedBuffer(0, b200.shapes.Make(b200.dtypes.Float32, 2))


def test_execute_host_matches_device_path(b200, backend):
    rng = np.random.default_rng(35)
    x = rng_array(rng, (64, 256), np.float32)
    builder = backend.Builder("host")
    f = builder.Main()
    p = f.Parameter("x", b200.shapes.Make(b200.dtypes.Float32, 64, 256))
    f.Return([f.FusedSoftmax(p, 1), f.ReduceSum(p, 1)], None)
    exe = builder.Compile()
    host = exe.ExecuteHost([x])
    buf = backend.FromNumpy(x)
    dev = [backend.ToNumpy(b) for b in exe.Execute([buf], None, 0)]
    for h, d in zip(host, dev):
        np.testing.assert_array_equal(h, d)


@pytest.mark.parametrize("num_slices", [1, 2, 5])
def test_execute_host_sliced_equals_slice_by_slice(b200, backend, num_slices):
    # one executable compiled for a [4, 8, 256] slice; weights are shared by every slice
    rng = np.random.default_rng(36 + num_slices)
    D = b200.dtypes
    builder = backend.Builder("sliced")
    f = builder.Main()
    p = f.Parameter("x", b200.shapes.Make(D.Float32, 4, 8, 256))
    w = f.Parameter("w", b200.shapes.Make(D.Float32, 256, 32))
    g = f.Parameter("g", b200.shapes.Make(D.Float32, 256))
    sm = f.FusedSoftmaxMasked(p, 0.5, True, None)
    y = f.DotGeneral(f.FusedRMSNorm(p, [-1], 1e-6, g), [2], [], w, [0], [])
    f.Return([sm, y, f.ArgMinMax(p, 2, D.Int32, False)], None)
    exe = builder.Compile()
    x = rng_array(rng, (4 * num_slices, 8, 256), np.float32)
    wv, gv = rng_array(rng, (256, 32), np.float32), rng_array(rng, (256,), np.float32)
    got = exe.ExecuteHostSliced([x, wv, gv], [True, False, False], num_slices)
    assert got[0].shape == (4 * num_slices, 8, 256) and got[1].shape == (4 * num_slices, 8, 32) and got[2].shape == (4 * num_slices, 8)
    for s in range(num_slices):
        want = exe.ExecuteHost([x[4 * s:4 * s + 4], wv, gv])
        for o, wnt in zip(got, want):
            np.testing.assert_array_equal(o[4 * s:4 * s + 4], wnt)
    # repeated calls reuse the device blocks and streams
    again = exe.ExecuteHostSliced([x, wv, gv], [True, False, False], num_slices)
    for a, b_ in zip(got, again):
        np.testing.assert_array_equal(a, b_)


def test_execute_host_sliced_argument_checks(b200, backend):
    builder = backend.Builder("sliced_err")
    f = builder.Main()
    p = f.Parameter("x", b200.shapes.Make(b200.dtypes.Float32, 2, 8))
    f.Return([f.Neg(p)], None)
    exe = builder.Compile()
    assert exe.ExecuteHostSliced([np.zeros((0, 8), np.float32)], [True], 0)[0].shape == (0, 8)
    with pytest.raises(b200.BackendError, match="expected 1 inputs"):
        exe.ExecuteHostSliced([], [], 1)
    with pytest.raises(b200.BackendError, match="bytes"):
        exe.ExecuteHostSliced([np.zeros((3, 8), np.float32)], [True], 2)


def test_buffer_round_trip_and_scalar(b200, backend):
    for arr in (np.arange(24, dtype=np.int16).reshape(2, 3, 4), np.array(2.5, dtype=np.float64), np.zeros((0,), dtype=np.float32)):
        buf = backend.FromNumpy(arr)
        assert backend.BufferShape(buf).Dimensions == list(arr.shape)
        assert backend.BufferDeviceNum(buf) == 0
        np.testing.assert_array_equal(backend.ToNumpy(buf), arr)
        backend.BufferFinalize(buf)


def test_intermediates_share_arena_memory(b200, backend):
    # a chain of unfusable ops must not grow memory linearly: dead intermediates are reused
    builder = backend.Builder("arena")
    f = builder.Main()
    x = f.Parameter("x", b200.shapes.Make(b200.dtypes.Float32, 256, 256))
    v = x
    for _ in range(8):
        v = f.FusedSoftmax(v, 1)
    f.Return([v], None)
    exe = builder.Compile()
    one = 256 * 256 * 4
    assert b200.lib().b200_exec_arena_bytes(exe.handle) <= 2 * one + 1024
    assert exe.NumLaunches() == 8


def test_dot_general_unaligned_n_uses_tensor_cores(b200, backend):
    # N = 1003 is not a multiple of 8: rows of C are not 16-byte aligned; B is [N, K] so its rows still are
    rng = np.random.default_rng(36)
    a, b = rng_array(rng, (300, 128), BF16), rng_array(rng, (1003, 128), BF16)
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, [1], [], y, [1], []), [a, b], rtol=BF16_RTOL, atol_scale=1.0)
    a32, b32 = a.astype(np.float32), b.astype(np.float32)
    assert_parity(b200, backend, lambda f, x, y: f.DotGeneral(x, [1], [], y, [1], []), [a32, b32], rtol=F32_RTOL, atol_scale=1.0)


def test_batch_sharded_runner_matches_single_device(b200, backend):
    from go_darwinml_b200.sharding import BatchShardedRunner
    import ctypes
    from go_darwinml_b200 import _lib
    err = _lib.B200Error()
    ndev = b200.lib().b200_device_count(ctypes.byref(err))
    rng = np.random.default_rng(37)
    x, w = rng_array(rng, (6, 40, 64), np.float32), rng_array(rng, (64, 48), np.float32)
    build = lambda f, xx, ww: f.FusedSoftmax(f.FusedDense(xx, ww, None, 0), 2)
    single = run_backend(b200, backend, build, [x, w])[0]
    devices = [0, 1] if ndev >= 2 else [0, 0]   # two replicas; on a one-GPU box both live on device 0
    runner = BatchShardedRunner(b200, devices, build, [(x.shape, x.dtype), (w.shape, w.dtype)], [True, False])
    got = runner([x, w])[0]
    runner.close()
    np.testing.assert_array_equal(got, single)   # replicas run the same kernels: bit-identical


@pytest.mark.parametrize("layout", [0, 1], ids=["BHSD", "BSHD"])
@pytest.mark.parametrize("heads,kv_heads", [(2, 2), (8, 2)])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("sq,sk", [(64, 64), (128, 128), (200, 200), (300, 300), (1, 77), (130, 333)])
@pytest.mark.parametrize("dtype", [BF16, np.float16], ids=["bf16", "f16"])
def test_fused_attention_head_dim_64(b200, backend, layout, heads, kv_heads, causal, sq, sk, dtype):
    # the single-kernel path: 16-bit floats, head dim 64, no mask tensor
    if dtype == np.float16 and (heads, kv_heads, layout) != (8, 2, 1):
        pytest.skip("f16 covered on one head/layout combination")
    rng = np.random.default_rng(38)
    B, D = 2, 64
    shp = lambda h, s: (B, h, s, D) if layout == 0 else (B, s, h, D)
    q, k, v = rng_array(rng, shp(heads, sq), dtype), rng_array(rng, shp(kv_heads, sk), dtype), rng_array(rng, shp(kv_heads, sk), dtype)
    (got,), plan = run_backend(b200, backend,
                               lambda f, qq, kk, vv: f.FusedScaledDotProductAttention(qq, kk, vv, None, heads, kv_heads, layout, 0.125, causal),
                               [q, k, v], describe=True)
    # one query position without the causal flag takes the cache-reading kernel
    assert (plan.startswith("attention_decode[" if sq == 1 and not causal else "attention[") and plan.count("\n") == 1) or not default_switches(), plan
    # The fused kernel keeps the scores in fp32 (the unfused lowering rounds them to the storage type before the
    # softmax), so the yardstick is the oracle evaluated on the same inputs in fp32, rounded once at the end.
    from oracle.oracle import OracleFunction, compare
    want = OracleFunction().FusedScaledDotProductAttention(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), None, heads,
                                                           kv_heads, layout, 0.125, causal).astype(dtype)
    ok, viol = compare(got, want, BF16_RTOL, 1.0)
    assert ok, viol


# ---- RMSNorm spelled in primitives is recognised and runs as the one row kernel --------------------------------
def _rms_from_primitives(b200, spelling, dt, shape, eps=1e-6, with_gamma=True):
    """GoMLX has no fused RMSNorm: a model emits Mul, ReduceSum, Div/Mul, Add, Rsqrt, Mul(, Mul).  Several spellings."""
    C = shape[-1]
    full = _S(b200, dt, *shape)
    keep = shape[:-1] + (1,)
    lead = list(range(len(shape) - 1))

    def scalar(f, v, like_shape, axes_shape):
        c = f.Constant(np.array([v], dtype=np.float32), 1)
        c = f.ConvertDType(c, b200.dtypes.from_numpy(np.dtype(dt))) if np.dtype(dt) != np.float32 else c
        return f.BroadcastInDim(c, _S(b200, dt, *axes_shape), [len(axes_shape) - 1] if len(axes_shape) else [])

    def build(f, x, g):
        ss = f.ReduceSum(f.Mul(x, x), len(shape) - 1)                               # [lead]
        if spelling == "keepdims":      # reshape to [.., 1], mean by Div, broadcast last
            st = f.Reshape(ss, *keep)
            st = f.Div(st, scalar(f, float(C), keep, keep))
            st = f.Rsqrt(f.Add(st, scalar(f, eps, keep, keep)))
            y = f.Mul(x, f.BroadcastInDim(st, full, list(range(len(shape)))))
        elif spelling == "early_broadcast":  # statistic broadcast to the full shape first, mean by Mul(1/C)
            st = f.BroadcastInDim(ss, full, lead)
            st = f.Mul(scalar(f, 1.0 / C, shape, shape), st)
            y = f.Mul(f.Rsqrt(f.Add(scalar(f, eps, shape, shape), st)), x)
        else:                            # x / sqrt(mean + eps)
            st = f.Div(ss, scalar(f, float(C), shape[:-1], shape[:-1]))
            st = f.Sqrt(f.Add(st, scalar(f, eps, shape[:-1], shape[:-1])))
            y = f.Div(x, f.BroadcastInDim(st, full, lead))
        if with_gamma:
            y = f.Mul(y, f.BroadcastInDim(g, full, [len(shape) - 1]))
        return y
    return build


@pytest.mark.parametrize("spelling", ["keepdims", "early_broadcast", "div_sqrt"])
@pytest.mark.parametrize("dt", ["float32", "bfloat16"])
def test_rmsnorm_from_primitives_is_one_kernel(b200, backend, spelling, dt):
    import ml_dtypes
    npdt = np.dtype(np.float32) if dt == "float32" else np.dtype(ml_dtypes.bfloat16)
    rng = np.random.default_rng(91)
    shape = (3, 7, 256)
    x = rng_array(rng, shape, npdt)
    g = (1 + 0.1 * rng.standard_normal(256)).astype(np.float32).astype(npdt)
    build = _rms_from_primitives(b200, spelling, npdt, shape)
    (got,), plan = run_backend(b200, backend, build, [x, g], describe=True)
    assert "rms_norm[" in plan and "gamma=1" in plan, plan
    assert len([l for l in plan.strip().splitlines() if l.strip()]) == 1, plan
    (want,) = run_oracle(build, [x, g])
    # fp32: the fused kernel and the op-by-op chain agree to rounding; 16-bit: the chain rounds every step to 8 bits
    ok, viol = compare(got, want, 1e-5 if dt == "float32" else 2e-2, 0.0)
    assert ok, viol
    # and it equals the fused op the backend offers directly
    (fused,) = run_backend(b200, backend, lambda f, a, gg: f.FusedRMSNorm(a, [-1], 1e-6, gg), [x, g])
    np.testing.assert_array_equal(got, fused)


def test_rmsnorm_lookalikes_are_left_alone(b200, backend):
    rng = np.random.default_rng(92)
    x = rng_array(rng, (4, 4, 4), np.float32)
    full = _S(b200, np.float32, 4, 4, 4)

    def c(f, v, *dims):
        return f.BroadcastInDim(f.Constant(np.array([v], dtype=np.float32), 1), _S(b200, np.float32, *dims), [len(dims) - 1])

    def not_last_axis(f, a):       # statistic over axis 1, not the last
        ss = f.ReduceSum(f.Mul(a, a), 1)
        st = f.Rsqrt(f.Add(f.Div(ss, c(f, 4.0, 4, 4)), c(f, 1e-6, 4, 4)))
        return f.Mul(a, f.BroadcastInDim(st, full, [0, 2]))

    def wrong_rows(f, a):          # sum over the last axis, but broadcast back along axis 0: rows are permuted
        ss = f.ReduceSum(f.Mul(a, a), 2)
        st = f.Rsqrt(f.Add(f.Div(ss, c(f, 4.0, 4, 4)), c(f, 1e-6, 4, 4)))
        return f.Mul(a, f.BroadcastInDim(st, full, [1, 2]))

    def not_a_mean(f, a):          # divides by 3, not by the row length
        ss = f.ReduceSum(f.Mul(a, a), 2)
        st = f.Rsqrt(f.Add(f.Div(ss, c(f, 3.0, 4, 4)), c(f, 1e-6, 4, 4)))
        return f.Mul(a, f.BroadcastInDim(st, full, [0, 1]))

    def other_tensor(f, a):        # normalises a DIFFERENT tensor by x's statistic
        ss = f.ReduceSum(f.Mul(a, a), 2)
        st = f.Rsqrt(f.Add(f.Div(ss, c(f, 4.0, 4, 4)), c(f, 1e-6, 4, 4)))
        return f.Mul(f.Neg(a), f.BroadcastInDim(st, full, [0, 1]))

    for build in (not_last_axis, wrong_rows, not_a_mean, other_tensor):
        (got,), plan = run_backend(b200, backend, build, [x], describe=True)
        assert "rms_norm[" not in plan, (build.__name__, plan)
        (want,) = run_oracle(build, [x])
        ok, viol = compare(got, want, 1e-5, 0.0)
        assert ok, (build.__name__, viol)


def test_rmsnorm_rewrite_keeps_shared_intermediates(b200, backend):
    # the statistic is also an output, and the normalised value feeds two users: only the root is rewritten
    rng = np.random.default_rng(93)
    x = rng_array(rng, (5, 128), np.float32)
    g = rng_array(rng, (128,), np.float32)
    full = _S(b200, np.float32, 5, 128)

    def build(f, a, gg):
        ss = f.ReduceSum(f.Mul(a, a), 1)
        mean = f.Div(ss, f.BroadcastInDim(f.Constant(np.array([128.0], dtype=np.float32), 1), _S(b200, np.float32, 5), [0]))
        inv = f.Rsqrt(f.Add(mean, f.BroadcastInDim(f.Constant(np.array([1e-5], dtype=np.float32), 1), _S(b200, np.float32, 5), [0])))
        n = f.Mul(a, f.BroadcastInDim(inv, full, [0]))
        return [f.Mul(n, f.BroadcastInDim(gg, full, [1])), f.Neg(n), mean]

    got, plan = run_backend(b200, backend, build, [x, g], describe=True)
    assert "rms_norm[" in plan and "gamma=0" in plan, plan
    want = run_oracle(build, [x, g])
    for a, w in zip(got, want):
        ok, viol = compare(a, w, 1e-5, 0.0)
        assert ok, viol


# ---- Add(DotGeneral, r) runs in the GEMM epilogue and equals the two-op result bit for bit -----------------------
@pytest.mark.parametrize("dtype,shape", [(BF16, (2, 300, 256, 192)), (np.float32, (1, 130, 96, 64)), (BF16, (1, 9, 7, 5)),
                                         (BF16, (2, 520, 1030, 1024))], ids=["bf16", "f32", "bf16_tiny_simt", "bf16_pairs_ragged_n"])
def test_dense_plus_residual_is_one_gemm(b200, backend, dtype, shape):
    B, M, N, K = shape
    rng = np.random.default_rng(95)
    x, w = rng_array(rng, (B, M, K), dtype), rng_array(rng, (K, N), dtype, 0.1)
    bias, r = rng_array(rng, (N,), dtype), rng_array(rng, (B * M, N), dtype)

    def fused(f, xx, ww, bb, rr):
        y = f.FusedDense(xx, ww, bb, 1)                   # GELU in the epilogue too
        return f.Add(rr, f.Reshape(y, B * M, N))           # seen through the reshape; residual on the left

    def two_ops(f, xx, ww, bb, rr):
        y = f.FusedDense(xx, ww, bb, 1)
        return [f.Add(rr, f.Reshape(y, B * M, N)), y]      # y has a second user: the sum stays a separate kernel

    (got,), plan = run_backend(b200, backend, fused, [x, w, bias, r], describe=True)
    assert "+residual" in plan and len(plan.strip().splitlines()) == 1, plan
    (want, _), plan2 = run_backend(b200, backend, two_ops, [x, w, bias, r], describe=True)
    assert "+residual" not in plan2, plan2
    np.testing.assert_array_equal(got.view(np.uint16 if dtype is BF16 else np.uint32), want.view(np.uint16 if dtype is BF16 else np.uint32))
    rtol, ascale = _dot_tol(dtype)
    (oracle,) = run_oracle(fused, [x, w, bias, r])
    ok, viol = compare(got, oracle, rtol, ascale)
    assert ok, viol


def test_gated_mlp_product_is_fused_into_one_gemm(b200, backend):
    # act(x W1) * (x W2): the product runs in the epilogue of one of the two GEMMs; a scalar scale stays elementwise
    rng = np.random.default_rng(96)
    x, w1, w2 = rng_array(rng, (4, 70, 128), BF16), rng_array(rng, (128, 264), BF16, 0.1), rng_array(rng, (128, 264), BF16, 0.1)

    def gated(f, xx, a, b_):
        return f.Mul(f.FusedDense(xx, a, None, 3), f.FusedDense(xx, b_, None, 0))

    def unfused(f, xx, a, b_):
        g, u = f.FusedDense(xx, a, None, 3), f.FusedDense(xx, b_, None, 0)
        return [f.Mul(g, u), g, u]

    (got,), plan = run_backend(b200, backend, gated, [x, w1, w2], describe=True)
    assert plan.count("gemm[") == 2 and "*residual" in plan and "ewise" not in plan, plan
    (want, _, _), plan2 = run_backend(b200, backend, unfused, [x, w1, w2], describe=True)
    assert "*residual" not in plan2
    np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16))

    def scaled(f, xx, a, b_):
        c = f.BroadcastInDim(f.Constant(np.array([0.5], dtype=BF16), 1), _S(b200, BF16, 4, 70, 264), [2])
        return f.Mul(f.FusedDense(xx, a, None, 0), c)

    (_,), plan3 = run_backend(b200, backend, scaled, [x, w1, w2], describe=True)
    assert "residual" not in plan3, plan3


# ---- rotary embedding spelled with Slice / Concatenate / Mul / Add runs as one pass --------------------------------
def _rope_graph(b200, dt, B, S, H, D, hide=False):
    full = _S(b200, dt, B, S, H, D)

    def build(f, x, cos, sin):
        r = 4
        lo = f.Slice(x, [0, 0, 0, 0], [B, S, H, D // 2], [1] * r)
        hi = f.Slice(x, [0, 0, 0, D // 2], [B, S, H, D], [1] * r)
        swapped = f.Concatenate(3, hi, lo)
        c = f.BroadcastInDim(cos, full, [1, 2, 3])     # table [S, H, D] shared by every batch entry
        s = f.BroadcastInDim(sin, full, [1, 2, 3])
        xd = f.Identity(x) if hide else x              # a different node for the direct product: the matcher must not fire
        return f.Add(f.Mul(xd, c), f.Mul(swapped, s))
    return build


@pytest.mark.parametrize("dt", [BF16, np.float32], ids=["bf16", "f32"])
def test_rope_from_primitives_is_one_kernel(b200, backend, dt):
    B, S, H, D = 3, 17, 4, 64
    rng = np.random.default_rng(97)
    x = rng_array(rng, (B, S, H, D), dt)
    ang = rng.uniform(0, 6.28, size=(S, H, D))
    cos, sin = np.cos(ang).astype(np.float32).astype(dt), np.sin(ang).astype(np.float32).astype(dt)
    (got,), plan = run_backend(b200, backend, _rope_graph(b200, dt, B, S, H, D), [x, cos, sin], describe=True)
    assert plan.count("\n") == 1 and plan.startswith("rope["), plan
    assert f"table_period={S * H * D}" in plan, plan           # the batch broadcast is never materialised
    (plain,), plan2 = run_backend(b200, backend, _rope_graph(b200, dt, B, S, H, D, hide=True), [x, cos, sin], describe=True)
    assert "rope[" not in plan2, plan2
    word = np.uint16 if dt is BF16 else np.uint32
    np.testing.assert_array_equal(got.view(word), plain.view(word))     # the op-by-op value, bit for bit
    (want,) = run_oracle(_rope_graph(b200, dt, B, S, H, D), [x, cos, sin])
    ok, viol = compare(got, want, 8e-3 if dt is BF16 else 1e-6, 1.0)
    assert ok, viol


@pytest.mark.parametrize("dt", [BF16, np.float32], ids=["bf16", "f32"])
def test_rope_table_shared_by_the_heads_is_never_spread(b200, backend, dt):
    # tables [S, D] -> BroadcastInDim [S, H, D] -> BroadcastInDim [B, S, H, D]: the kernel indexes the [S, D] table itself
    B, S, H, D = 3, 19, 5, 64
    rng = np.random.default_rng(99)
    x = rng_array(rng, (B, S, H, D), dt)
    ang = rng.uniform(0, 6.28, size=(S, D))
    cos, sin = np.cos(ang).astype(np.float32).astype(dt), np.sin(ang).astype(np.float32).astype(dt)

    def build(f, xx, c_, s_):
        per_head = _S(b200, dt, S, H, D)
        c3, s3 = f.BroadcastInDim(c_, per_head, [0, 2]), f.BroadcastInDim(s_, per_head, [0, 2])
        return _rope_graph(b200, dt, B, S, H, D)(f, xx, c3, s3)

    (got,), plan = run_backend(b200, backend, build, [x, cos, sin], describe=True)
    assert plan.count("\n") == 1 and plan.startswith("rope[") and f"table_period={S * D} per-head" in plan, plan
    (want,) = run_oracle(build, [x, cos, sin])
    ok, viol = compare(got, want, 8e-3 if dt is BF16 else 1e-6, 1.0)
    assert ok, viol
    # the same tables spread by hand give the same bits
    cos3, sin3 = np.ascontiguousarray(np.broadcast_to(cos[:, None, :], (S, H, D))), np.ascontiguousarray(np.broadcast_to(sin[:, None, :], (S, H, D)))
    (spread,), _ = run_backend(b200, backend, _rope_graph(b200, dt, B, S, H, D), [x, cos3, sin3], describe=True)
    word = np.uint16 if dt is BF16 else np.uint32
    np.testing.assert_array_equal(got.view(word), spread.view(word))


def test_rope_reads_queries_inside_the_projection_buffer(b200, backend):
    # q = Reshape(Slice(QKV)) feeds the rotary kernel in place: no Slice copy in the plan
    B, S, H, D, W = 2, 24, 4, 64, 4 * 64 + 2 * 64
    rng = np.random.default_rng(98)
    qkv = rng_array(rng, (B, S, W), BF16)
    ang = rng.uniform(0, 6.28, size=(S, H, D))
    cos, sin = np.cos(ang).astype(np.float32).astype(BF16), np.sin(ang).astype(np.float32).astype(BF16)

    def build(f, t, c_, s_):
        q = f.Reshape(f.Slice(t, [0, 0, 64], [B, S, 64 + H * D], [1, 1, 1]), B, S, H, D)
        return [_rope_graph(b200, BF16, B, S, H, D)(f, q, c_, s_), f.Neg(t)]

    got, plan = run_backend(b200, backend, build, [qkv, cos, sin], describe=True)
    assert "rope[" in plan and f"pitch={W}" in plan and "move[" not in plan, plan
    want = run_oracle(build, [qkv, cos, sin])
    ok, viol = compare(got[0], want[0], 8e-3, 1.0)
    assert ok, viol


@pytest.mark.parametrize("dtype,M,N", [(BF16, 2050, 2051), (np.float32, 1040, 2050), (BF16, 4100, 1030)], ids=["bf16_odd", "f32_even", "bf16_even"])
def test_large_ragged_result_goes_through_a_padded_pitch(b200, backend, dtype, M, N):
    # rows that are not a whole number of 16-byte vectors, and no way to write them in row classes (M not a multiple of 8, or
    # fp32): GEMM into a padded pitch, then one packing pass
    rng = np.random.default_rng(99)
    a, w = rng_array(rng, (M, 64), dtype), rng_array(rng, (N, 64), dtype, 0.2)
    (got,), plan = run_backend(b200, backend, lambda f, x, y: f.DotGeneral(x, [1], [], y, [1], []), [a, w], describe=True)
    assert "move[pack" in plan and "ragged-rows" not in plan, plan
    (want,) = run_oracle(lambda f, x, y: f.DotGeneral(x, [1], [], y, [1], []), [a, w])
    rtol, ascale = _dot_tol(dtype)
    ok, viol = compare(got, want, rtol, ascale)
    assert ok, viol


def test_small_concatenation_is_one_launch(b200, backend):
    rng = np.random.default_rng(100)
    parts = [rng_array(rng, (n,), BF16) for n in (768, 768, 768, 5)]
    (got,), plan = run_backend(b200, backend, lambda f, *p: f.Concatenate(0, *p), parts, describe=True)
    assert plan.count("\n") == 1 and "flat" in plan, plan
    np.testing.assert_array_equal(got.view(np.uint16), np.concatenate(parts).view(np.uint16))
    ints = [rng_array(rng, (1, 3, 7), np.int64), rng_array(rng, (1, 2, 7), np.int64)]
    assert_parity(b200, backend, lambda f, a, b: f.Concatenate(1, a, b), ints)


# ---- DynamicSlice / DynamicUpdateSlice (ref function.go:1571-1621): start indices are values of the graph ----------
@pytest.mark.parametrize("dtype", [np.float32, BF16, np.int64, np.uint8], ids=["f32", "bf16", "i64", "u8"])
def test_dynamic_slice_and_update_exact(b200, backend, dtype):
    rng = np.random.default_rng(101)
    x = rng_array(rng, (5, 7, 33), dtype)
    u = rng_array(rng, (2, 7, 9), dtype)
    for starts in ([1, 0, 5], [3, 0, 24], [0, 0, 0]):
        s = [np.array(v, dtype=np.int32) for v in starts]
        assert_parity(b200, backend, lambda f, a, s0, s1, s2: f.DynamicSlice(a, [s0, s1, s2], [2, 7, 9]), [x] + s, rtol=0.0)
        assert_parity(b200, backend, lambda f, a, b, s0, s1, s2: f.DynamicUpdateSlice(a, b, [s0, s1, s2]), [x, u] + s, rtol=0.0)


def test_dynamic_slice_clamps_and_takes_computed_indices(b200, backend):
    # out-of-range starts are clamped so the block fits; an index may be any integer dtype and the result of other ops
    rng = np.random.default_rng(102)
    x = rng_array(rng, (6, 10), np.float32)
    u = rng_array(rng, (4, 3), np.float32)
    s0, s1 = np.array(-3, dtype=np.int64), np.array(200, dtype=np.uint8)

    def build(f, a, b, i, j):
        jj = f.Add(j, f.Constant(np.array([1], dtype=np.uint8)))           # 201: far past the end
        return [f.DynamicSlice(a, [i, jj], [4, 3]), f.DynamicUpdateSlice(a, b, [i, jj])]

    got = assert_parity(b200, backend, build, [x, u, s0, s1], rtol=0.0)
    np.testing.assert_array_equal(got[0], x[0:4, 7:10])
    want = x.copy()
    want[0:4, 7:10] = u
    np.testing.assert_array_equal(got[1], want)


def test_dynamic_slice_kv_cache_step(b200, backend):
    # the use the op exists for: write one position of a [B, S, H, D] cache and read a window back
    rng = np.random.default_rng(103)
    cache, new = rng_array(rng, (2, 64, 4, 16), BF16), rng_array(rng, (2, 1, 4, 16), BF16)
    pos, zero = np.array(37, dtype=np.int32), np.array(0, dtype=np.int32)

    def build(f, c, n, p, z):
        c2 = f.DynamicUpdateSlice(c, n, [z, p, z, z])
        return [c2, f.DynamicSlice(c2, [z, p, z, z], [2, 1, 4, 16])]

    got = assert_parity(b200, backend, build, [cache, new, pos, zero], rtol=0.0)
    np.testing.assert_array_equal(got[1].view(np.uint16), new.view(np.uint16))


def test_dynamic_slice_argument_checks(b200, backend):
    builder = backend.Builder("dyn_err")
    f = builder.Main()
    x = f.Parameter("x", b200.shapes.Make(b200.dtypes.Float32, 3, 4))
    i = f.Parameter("i", b200.shapes.Make(b200.dtypes.Int32))
    fl = f.Parameter("fl", b200.shapes.Make(b200.dtypes.Float32))
    with pytest.raises(b200.BackendError, match="start indices"):
        f.DynamicSlice(x, [i], [2, 2])
    with pytest.raises(b200.BackendError, match="integer"):
        f.DynamicSlice(x, [i, fl], [2, 2])
    with pytest.raises(b200.BackendError, match="exceeds"):
        f.DynamicSlice(x, [i, i], [2, 5])
    with pytest.raises(b200.BackendError, match="exceeds"):
        f.DynamicUpdateSlice(x, f.Parameter("u", b200.shapes.Make(b200.dtypes.Float32, 4, 4)), [i, i])


def test_repeated_execution_replays_a_cuda_graph(b200, backend):
    # a plan run again on the same addresses is recorded once and replayed; results must not change, and new input
    # CONTENT at the same address must be picked up
    rng = np.random.default_rng(104)
    x, w, g = rng_array(rng, (64, 256), BF16), rng_array(rng, (256, 128), BF16, 0.1), rng_array(rng, (256,), BF16)
    builder = backend.Builder("graph_replay")
    f = builder.Main()
    px = f.Parameter("x", _S(b200, BF16, 64, 256))
    pw = f.Parameter("w", _S(b200, BF16, 256, 128))
    pg = f.Parameter("g", _S(b200, BF16, 256))
    h = f.FusedRMSNorm(px, [-1], 1e-6, pg)
    y = f.FusedSoftmax(f.FusedDense(h, pw, None, 1), 1)
    z = f.ReduceSum(f.Tanh(y), 1)
    f.Return([y, z, f.ArgMinMax(y, 1, b200.dtypes.Int32, False)], None)
    exe = builder.Compile()
    assert exe.NumLaunches() >= 4
    bx, bw, bg = backend.FromNumpy(x), backend.FromNumpy(w), backend.FromNumpy(g)
    first = None
    for it in range(6):
        outs = exe.Execute([bx, bw, bg], None, 0)
        vals = [backend.ToNumpy(o) for o in outs]
        for o in outs:
            backend.BufferFinalize(o)           # the allocator hands the same blocks back: same addresses next time
        if first is None:
            first = vals
        for a, b_ in zip(vals, first):
            np.testing.assert_array_equal(a, b_)
    # same addresses, new content
    x2 = rng_array(rng, (64, 256), BF16)
    backend.BufferFinalize(bx)
    bx = backend.FromNumpy(x2)
    outs = exe.Execute([bx, bw, bg], None, 0)
    got = [backend.ToNumpy(o) for o in outs]
    want = run_oracle(lambda ff, a, b_, c: (lambda hh: (lambda yy: [yy, ff.ReduceSum(ff.Tanh(yy), 1), ff.ArgMinMax(yy, 1, b200.dtypes.Int32, False)])(
        ff.FusedSoftmax(ff.FusedDense(hh, b_, None, 1), 1)))(ff.FusedRMSNorm(a, [-1], 1e-6, c)), [x2, w, g])
    ok, viol = compare(got[0], want[0], BF16_RTOL, 1.0)
    assert ok, viol
    assert not np.array_equal(got[0], first[0])


def test_donated_cache_is_updated_in_place(b200, backend):
    # Execute's donate flag (ref executable.go:50-60): a donated input that an output is DynamicUpdateSlice of is updated
    # where it lies; without the flag the output is a fresh copy and the input stays valid and unchanged
    rng = np.random.default_rng(105)
    cache, new = rng_array(rng, (2, 64, 4, 16), BF16), rng_array(rng, (2, 1, 4, 16), BF16)
    L = b200.lib()
    builder = backend.Builder("donate")
    f = builder.Main()
    pc = f.Parameter("cache", _S(b200, BF16, 2, 64, 4, 16))
    pn = f.Parameter("new", _S(b200, BF16, 2, 1, 4, 16))
    pp = f.Parameter("pos", b200.shapes.Make(b200.dtypes.Int32))
    z = f.Constant(np.array([0], dtype=np.int32))
    z = f.Reshape(z)
    f.Return([f.DynamicUpdateSlice(pc, pn, [z, pp, z, z])], None)
    exe = builder.Compile()
    want = cache.copy()
    want[:, 37:38] = new
    bn, bp = backend.FromNumpy(new), backend.FromNumpy(np.array(37, dtype=np.int32))

    bc = backend.FromNumpy(cache)
    addr = L.b200_buffer_device_ptr(bc.handle)
    (out,) = exe.Execute([bc, bn, bp], [False, False, False], 0)
    assert L.b200_buffer_device_ptr(out.handle) != addr and bc.valid
    np.testing.assert_array_equal(backend.ToNumpy(out).view(np.uint16), want.view(np.uint16))
    np.testing.assert_array_equal(backend.ToNumpy(bc).view(np.uint16), cache.view(np.uint16))
    backend.BufferFinalize(out)

    for _ in range(3):   # repeated steps: each output becomes the next donated cache (and the plan may be replayed)
        (out,) = exe.Execute([bc, bn, bp], [True, False, False], 0)
        assert L.b200_buffer_device_ptr(out.handle) == addr and not bc.valid
        np.testing.assert_array_equal(backend.ToNumpy(out).view(np.uint16), want.view(np.uint16))
        bc = out
    with pytest.raises(b200.BackendError):
        exe.Execute([bc, bn, bp], [True, False], 0)


def test_concurrent_executes_do_not_leak_into_each_others_graph_recording(b200, backend):
    # two host threads drive two executables on the same device while each plan gets recorded into a CUDA graph: the
    # recording runs on a private stream, so the other thread's launches must neither be swallowed nor replayed
    import threading
    rng = np.random.default_rng(106)

    def make(tag, scale):
        builder = backend.Builder(tag)
        f = builder.Main()
        p = f.Parameter("x", _S(b200, np.float32, 256, 128))
        y = f.FusedSoftmax(p, 1)
        y = f.ReduceSum(f.Mul(y, f.BroadcastInDim(f.Constant(np.array([scale], dtype=np.float32), 1), _S(b200, np.float32, 256, 128), [1])), 1)
        z = f.FusedLayerNorm(f.Tanh(p), [-1], 1e-5, None, None)
        w = f.ArgMinMax(z, 1, b200.dtypes.Int32, True)
        f.Return([y, z, w], None)
        return builder.Compile()

    exes = [make("conc_a", 2.0), make("conc_b", 3.0)]
    xs = [rng_array(rng, (256, 128), np.float32) for _ in exes]
    bufs = [backend.FromNumpy(x) for x in xs]
    ref = []
    for exe, buf in zip(exes, bufs):
        outs = exe.Execute([buf], None, 0)
        ref.append([backend.ToNumpy(o) for o in outs])
        for o in outs:
            backend.BufferFinalize(o)
    errors = []

    def worker(i):
        try:
            for _ in range(25):
                outs = exes[i].Execute([bufs[i]], None, 0)
                vals = [backend.ToNumpy(o) for o in outs]
                for o in outs:
                    backend.BufferFinalize(o)
                for a, b_ in zip(vals, ref[i]):
                    np.testing.assert_array_equal(a, b_)
        except Exception as e:  # noqa: BLE001
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


# ------------------------------------------------ entry points that had no test of their own ---
def test_buffer_copy_to_device_same_device(b200, backend):
    # one visible GPU is enough: device 0 -> device 0 is a stream-ordered copy into a fresh buffer
    x = np.random.default_rng(70).standard_normal((33, 129)).astype(np.float32)
    src = backend.FromNumpy(x)
    dst = backend.BufferCopyToDevice(src, 0)
    assert backend.BufferDeviceNum(dst) == 0 and backend.BufferShape(dst) == backend.BufferShape(src)
    backend.BufferFinalize(src)                      # the copy must not depend on the source staying alive
    other = backend.FromNumpy(np.zeros_like(x))      # likely reuses the freed block
    np.testing.assert_array_equal(backend.ToNumpy(dst), x)
    for b in (dst, other):
        backend.BufferFinalize(b)
    with pytest.raises(b200.BackendError):
        backend.BufferCopyToDevice(backend.FromNumpy(x), 99)


@pytest.mark.parametrize("dtype", [np.float32, BF16], ids=["f32", "bf16"])
@pytest.mark.parametrize("axis", [1, 3, -1])
def test_batch_norm_for_inference(b200, backend, dtype, axis):
    # y = (x - mean) / sqrt(var + eps) * scale + offset along the feature axis (ref mpsgraph/gomlx/function.go:1244-1261)
    rng = np.random.default_rng(71)
    x = rng_array(rng, (3, 5, 4, 5), dtype)
    c = x.shape[axis]
    scale, offset, mean = (rng_array(rng, (c,), dtype) for _ in range(3))
    var = (np.abs(rng_array(rng, (c,), np.float32)) + 0.5).astype(dtype)

    def want_fn():
        shp = [1] * 4
        shp[axis] = c
        v64 = lambda t: t.astype(np.float64).reshape(shp)
        y = (x.astype(np.float64) - v64(mean)) / np.sqrt(v64(var) + float(np.float32(1e-3))) * v64(scale) + v64(offset)
        return y.astype(dtype)
    (got,) = run_backend(b200, backend, lambda f, a, s, o, m, v: f.BatchNormForInference(a, s, o, m, v, 1e-3, axis), [x, scale, offset, mean, var])
    ok, viol = compare(got, want_fn(), 1e-5 if dtype == np.float32 else 2e-2, 1.0)
    assert ok, viol


@pytest.mark.parametrize("op,plain", [("EqualTotalOrder", "Equal"), ("NotEqualTotalOrder", "NotEqual"), ("LessThanTotalOrder", "LessThan"),
                                      ("LessOrEqualTotalOrder", "LessOrEqual"), ("GreaterThanTotalOrder", "GreaterThan"),
                                      ("GreaterOrEqualTotalOrder", "GreaterOrEqual")])
def test_total_order_compares_delegate_to_plain_compares(b200, backend, op, plain):
    # the reference delegates every *TotalOrder compare to the plain one (ref mpsgraph/gomlx/function.go:2234-2256)
    rng = np.random.default_rng(72)
    a = rng.integers(-3, 4, size=(9, 31)).astype(np.float32)
    b = rng.integers(-3, 4, size=(31,)).astype(np.float32)
    if not hasattr(backend.Builder("probe").Main(), op):
        pytest.fail(f"Function has no {op}")
    (got,) = run_backend(b200, backend, lambda f, x, y: getattr(f, op)(x, y), [a, b])
    (want,) = run_backend(b200, backend, lambda f, x, y: getattr(f, plain)(x, y), [a, b])
    np.testing.assert_array_equal(got, want)
