"""Known-answer vectors transcribed from the reference's own test files.

Each case names the reference test it comes from (file:line inside
gomlx/go-darwinml), builds the same graph through a Function-like object `f`
(the backend's Function or the oracle's OracleFunction) and lists the expected
values and the ABSOLUTE tolerance that reference test uses (its assertClose
helper, mpsgraph/gomlx/mpsgraph_test.go:210-220).  tol == 0 means exact.

The reference is Go and links Apple frameworks, so it cannot run here; the
vectors were read from its test sources as text.  `python tests/golden/
reference_vectors.py` re-derives every expectation that the reference computes
with math.* calls instead of literals and prints the table, as a self-check.
"""
from __future__ import annotations

import math

import numpy as np

F32, I32, I64, U8, BOOL, BF16 = "float32", "int32", "int64", "uint8", "bool", "bfloat16"


def _a(values, dtype=F32, shape=None):
    if dtype == BF16:
        import ml_dtypes
        arr = np.asarray(values, dtype=np.float32).astype(ml_dtypes.bfloat16)
    else:
        arr = np.asarray(values, dtype=dtype)
    return arr.reshape(shape) if shape is not None else arr


class Case:
    def __init__(self, name, cite, inputs, build, expected, tol=1e-5, prefix=None):
        self.name, self.cite, self.inputs, self.build = name, cite, inputs, build
        self.expected = expected if isinstance(expected, (list, tuple)) and expected and isinstance(expected[0], np.ndarray) else [expected]
        self.tol = tol
        self.prefix = prefix  # compare only the first `prefix` flat elements (tests that check a slice of the output)


_e1, _e2, _e3 = math.exp(1), math.exp(2), math.exp(3)
_s = math.exp(1.0 / math.sqrt(3.0))
_w0, _w1 = _s / (_s + 1), 1 / (_s + 1)


def _sigmoid(x):
    return 1.0 / (1.0 + math.exp(-x))


def _eye_w(rows, cols):
    w = np.zeros((rows, cols), dtype=np.float32)
    for i in range(min(rows, cols)):
        w[i, i] = 1
    return w


# dtype codes of the C ABI (same numbers as the reference's bridge enum, mpsgraph bridge.h:23-37)
C_BOOL, C_I32, C_I64, C_BF16, C_F32 = 0, 3, 4, 6, 7
_CODE = {F32: C_F32, I32: C_I32, I64: C_I64, BF16: C_BF16, BOOL: C_BOOL}


class _Shape:
    """Duck-typed shapes.Shape: DType (code), Dimensions, Rank()."""

    def __init__(self, code, dims):
        self.DType, self.Dimensions = code, list(dims)

    def Rank(self):
        return len(self.Dimensions)


def _shape(f, dtype_name, *dims):
    return _Shape(_CODE[dtype_name], dims)


def closure(f, param_shapes, body):
    """body(c, *params) -> outputs, as a closure of function f (the cond / body of While, a branch of If, Sort's comparator):
    a Function.Closure() with its Parameters and Return on the backend, a callable on the oracle."""
    if hasattr(f, "MakeClosure"):
        return f.MakeClosure(param_shapes, body)
    c = f.Closure()
    params = [c.Parameter(f"p{i}", s) for i, s in enumerate(param_shapes)]
    c.Return(list(body(c, *params)), None)
    return c


def named_function(f, name, param_shapes, body):
    """The same for Builder.NewFunction(name), the target of Call."""
    if hasattr(f, "MakeClosure"):
        return f.MakeClosure(param_shapes, body)
    c = f.builder.NewFunction(name)
    params = [c.Parameter(f"p{i}", s) for i, s in enumerate(param_shapes)]
    c.Return(list(body(c, *params)), None)
    return c


def _const(f, value, dtype_name):
    return f.Constant(np.array([value], dtype=dtype_name))


def _while_sum(f, _dummy):
    s = _shape(f, I32)
    cond = closure(f, [s, s], lambda c, counter, total: [c.LessOrEqual(counter, _const(c, 10, I32))])
    body = closure(f, [s, s], lambda c, counter, total: [c.Add(counter, _const(c, 1, I32)), c.Add(total, counter)])
    return f.While(cond, body, _const(f, 1, I32), _const(f, 0, I32))[1]


def _while_factorial(f, _dummy):
    s = _shape(f, I32)
    cond = closure(f, [s, s], lambda c, n, result: [c.GreaterThan(n, _const(c, 1, I32))])
    body = closure(f, [s, s], lambda c, n, result: [c.Sub(n, _const(c, 1, I32)), c.Mul(result, n)])
    return f.While(cond, body, _const(f, 5, I32), _const(f, 1, I32))[1]


def _if_const(f, x):
    pred = f.GreaterThan(x, _const(f, 5, F32))
    return f.If(pred, closure(f, [], lambda c: [_const(c, 1, F32)]), closure(f, [], lambda c: [_const(c, -1, F32)]))[0]


def _if_captured(f, x):
    factor = _const(f, 10, F32)
    pred = f.GreaterThan(x, _const(f, 0, F32))
    return f.If(pred, closure(f, [], lambda c: [c.Mul(x, factor)]), closure(f, [], lambda c: [c.Neg(c.Mul(x, factor))]))[0]


def _sort(descending):
    def build(f, x):
        s = _shape(f, F32)
        comparator = closure(f, [s, s], lambda c, a, b: [c.GreaterThan(a, b) if descending else c.LessThan(a, b)])
        return f.Sort(comparator, 0, True, x)[0]
    return build


def _call_add(f, _dummy):
    s = _shape(f, F32)
    add = named_function(f, "add", [s, s], lambda c, a, b: [c.Add(a, b)])
    return f.Call(add, _const(f, 10, F32), _const(f, 32, F32))[0]


CASES = [
    Case("Add", "mpsgraph/gomlx/mpsgraph_test.go:223-238",
         [_a([1, 2, 3, 4, 5, 6], shape=(2, 3)), _a([10, 20, 30, 40, 50, 60], shape=(2, 3))],
         lambda f, x, y: f.Add(x, y), _a([11, 22, 33, 44, 55, 66], shape=(2, 3))),
    Case("Abs", "mpsgraph/gomlx/mpsgraph_test.go:256-257", [_a([-1, 2, -3, 4])], lambda f, x: f.Abs(x), _a([1, 2, 3, 4])),
    Case("Neg", "mpsgraph/gomlx/mpsgraph_test.go:258-259", [_a([-1, 2, -3, 4])], lambda f, x: f.Neg(x), _a([1, -2, 3, -4])),
    Case("Sqrt", "mpsgraph/gomlx/mpsgraph_test.go:260-261", [_a([1, 4, 9, 16])], lambda f, x: f.Sqrt(x), _a([1, 2, 3, 4])),
    Case("Exp", "mpsgraph/gomlx/mpsgraph_test.go:262-263", [_a([0, 1])], lambda f, x: f.Exp(x), _a([1, math.e])),
    Case("Log", "mpsgraph/gomlx/mpsgraph_test.go:264-265", [_a([1, math.e])], lambda f, x: f.Log(x), _a([0, 1]), tol=1e-4),
    Case("Tanh", "mpsgraph/gomlx/mpsgraph_test.go:266-267", [_a([0, 1])], lambda f, x: f.Tanh(x), _a([0, math.tanh(1)])),
    Case("Sub", "mpsgraph/gomlx/mpsgraph_test.go:289-294", [_a([10, 20, 30, 40]), _a([3, 5, 10, 8])], lambda f, x, y: f.Sub(x, y), _a([7, 15, 20, 32])),
    Case("Mul", "mpsgraph/gomlx/mpsgraph_test.go:296-301", [_a([10, 20, 30, 40]), _a([3, 5, 10, 8])], lambda f, x, y: f.Mul(x, y), _a([30, 100, 300, 320])),
    Case("Div", "mpsgraph/gomlx/mpsgraph_test.go:303-308", [_a([10, 20, 30, 40]), _a([3, 5, 10, 8])], lambda f, x, y: f.Div(x, y), _a([10.0 / 3, 4, 3, 5]), tol=1e-4),
    Case("Max", "mpsgraph/gomlx/mpsgraph_test.go:310-315", [_a([10, 20, 30, 40]), _a([3, 5, 10, 8])], lambda f, x, y: f.Max(x, y), _a([10, 20, 30, 40])),
    Case("Min", "mpsgraph/gomlx/mpsgraph_test.go:317-322", [_a([10, 20, 30, 40]), _a([3, 5, 10, 8])], lambda f, x, y: f.Min(x, y), _a([3, 5, 10, 8])),
    Case("ReduceSum axis 1", "mpsgraph/gomlx/mpsgraph_test.go:439-486", [_a([1, 2, 3, 4, 5, 6], shape=(2, 3))],
         lambda f, x: f.ReduceSum(x, 1), _a([6, 15])),
    Case("ReduceProduct axis 1", "mpsgraph/gomlx/mpsgraph_test.go:1318-1364", [_a([1, 2, 3, 4, 5, 6], shape=(2, 3))],
         lambda f, x: f.ReduceProduct(x, 1), _a([6, 120])),
    Case("DotGeneral simple matmul", "mpsgraph/gomlx/mpsgraph_test.go:496-544",
         [_a([1, 2, 3, 4, 5, 6], shape=(2, 3)), _a([1, 2, 3, 4, 5, 6], shape=(3, 2))],
         lambda f, a, b: f.DotGeneral(a, [1], None, b, [0], None), _a([22, 28, 49, 64], shape=(2, 2)), tol=1e-4),
    Case("DotGeneral batched", "mpsgraph/gomlx/mpsgraph_test.go:546-595",
         [_a(range(1, 13), shape=(2, 2, 3)), _a(range(1, 13), shape=(2, 3, 2))],
         lambda f, a, b: f.DotGeneral(a, [2], [0], b, [1], [0]), _a([22, 28, 49, 64, 220, 244, 301, 334], shape=(2, 2, 2)), tol=1e-3),
    Case("DotGeneral 2x3 . 3x4", "coreml/gomlx/integration_test.go:128-204",
         [_a([1, 2, 3, 4, 5, 6], shape=(2, 3)), _a(range(1, 13), shape=(3, 4))],
         lambda f, a, b: f.DotGeneral(a, [1], None, b, [0], None), _a([38, 44, 50, 56, 83, 98, 113, 128], shape=(2, 4)), tol=1e-4),
    Case("DotGeneral vector . vector", "coreml/gomlx/integration_test.go:291-370", [_a([1, 2, 3, 4]), _a([2, 3, 4, 5])],
         lambda f, a, b: f.DotGeneral(a, [0], None, b, [0], None), _a(40.0, shape=()), tol=0),
    Case("Gather embedding rows", "mpsgraph/gomlx/mpsgraph_test.go:599-674",
         [_a([10, 11, 12, 20, 21, 22, 30, 31, 32, 40, 41, 42], shape=(4, 3)), _a([1, 3], I32, (2, 1))],
         lambda f, t, i: f.Gather(t, i, 1, [1], [0], [0], [1, 3], False), _a([20, 21, 22, 40, 41, 42], shape=(2, 3)), tol=0),
    Case("Gather multi-dim indices", "coreml/gomlx/gather_test.go:215-325",
         [_a([0, 1, 2, 3, 10, 11, 12, 13, 20, 21, 22, 23, 30, 31, 32, 33, 40, 41, 42, 43], shape=(5, 4)), _a([0, 1, 2, 3, 4, 0], I32, (2, 3, 1))],
         lambda f, t, i: f.Gather(t, i, 2, [2], [0], [0], [1, 4], False),
         _a([0, 1, 2, 3, 10, 11, 12, 13, 20, 21, 22, 23, 30, 31, 32, 33, 40, 41, 42, 43, 0, 1, 2, 3], shape=(2, 3, 4)), tol=0),
    Case("Gather along a middle axis", "coreml/gomlx/gather_test.go:327-436",
         [_a([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 100, 101, 102, 103, 104, 105, 106, 107, 108, 109, 110, 111], shape=(2, 4, 3)), _a([1, 3], I32, (2, 1))],
         lambda f, t, i: f.Gather(t, i, 1, [0, 2], [1], [1], [2, 1, 3], False),
         _a([3, 4, 5, 9, 10, 11, 103, 104, 105, 109, 110, 111], shape=(2, 2, 3)), tol=0),
    Case("Gather N-d", "coreml/gomlx/gather_test.go:438-547",
         [_a([i * 100 + j * 10 + k for i in range(3) for j in range(4) for k in range(5)], shape=(3, 4, 5)), _a([1, 2, 2, 3], I32, (2, 2))],
         lambda f, t, i: f.Gather(t, i, 1, [1], [0, 1], [0, 1], [1, 1, 5], False),
         _a([120, 121, 122, 123, 124, 230, 231, 232, 233, 234], shape=(2, 5)), tol=0),
    Case("Gather int32 indices [3,1]", "mpsgraph/gomlx/mpsgraph_test.go:2775-2788",
         [_a([10, 20, 30], shape=(3, 1)), _a([2, 0, 1], I32, (3, 1))],
         lambda f, t, i: f.Gather(t, i, 1, [1], [0], [0], [1, 1], False), _a([30, 10, 20], shape=(3, 1)), tol=0),
    Case("Slice", "mpsgraph/gomlx/mpsgraph_test.go:677-727", [_a(range(1, 13), shape=(3, 4))],
         lambda f, x: f.Slice(x, [1, 1], [3, 3], [1, 1]), _a([6, 7, 10, 11], shape=(2, 2)), tol=0),
    Case("Concatenate axis 1", "mpsgraph/gomlx/mpsgraph_test.go:730-782", [_a([1, 2, 3, 4], shape=(2, 2)), _a([5, 6, 7, 8, 9, 10], shape=(2, 3))],
         lambda f, a, b: f.Concatenate(1, a, b), _a([1, 2, 5, 6, 7, 3, 4, 8, 9, 10], shape=(2, 5)), tol=0),
    Case("Iota axis 1 of [2,3]", "mpsgraph/gomlx/mpsgraph_test.go:785-822", [],
         lambda f: f.Iota(_shape(f, F32, 2, 3), 1), _a([0, 1, 2, 0, 1, 2], shape=(2, 3)), tol=0),
    Case("Iota Int32 [4]", "coreml/gomlx/iota_test.go:15-169", [],
         lambda f: f.Iota(_shape(f, I32, 4), 0), _a([0, 1, 2, 3], I32), tol=0),
    Case("Iota axis 0 of [3,2] Int32", "coreml/gomlx/iota_test.go:15-169", [],
         lambda f: f.Iota(_shape(f, I32, 3, 2), 0), _a([0, 0, 1, 1, 2, 2], I32, (3, 2)), tol=0),
    Case("BroadcastInDim", "mpsgraph/gomlx/mpsgraph_test.go:825-874", [_a([10, 20, 30])],
         lambda f, x: f.BroadcastInDim(x, _shape(f, F32, 2, 3), [1]), _a([10, 20, 30, 10, 20, 30], shape=(2, 3)), tol=0),
    Case("Pad", "mpsgraph/gomlx/mpsgraph_test.go:877-938", [_a([1, 2, 3, 4], shape=(2, 2))],
         lambda f, x: f.Pad(x, f.Reshape(f.Constant(np.array([0], dtype=np.float32), 1)), (1, 0), (0, 1)),
         _a([0, 0, 0, 1, 2, 0, 3, 4, 0], shape=(3, 3)), tol=0),
    Case("DynamicSlice [2,2] at (1,1)", "mpsgraph/gomlx/mpsgraph_test.go:993-1061",
         [_a(range(1, 13), shape=(3, 4)), _a([1], I32, ()), _a([1], I32, ())],
         lambda f, x, s0, s1: f.DynamicSlice(x, [s0, s1], [2, 2]), _a([6, 7, 10, 11], shape=(2, 2)), tol=0),
    Case("DynamicUpdateSlice [2,2] at (1,1)", "mpsgraph/gomlx/mpsgraph_test.go:1064-1130",
         [_a(range(1, 13), shape=(3, 4)), _a([100, 200, 300, 400], shape=(2, 2)), _a([1], I32, ()), _a([1], I32, ())],
         lambda f, x, u, s0, s1: f.DynamicUpdateSlice(x, u, [s0, s1]),
         _a([1, 2, 3, 4, 5, 100, 200, 8, 9, 300, 400, 12], shape=(3, 4)), tol=0),
    Case("ArgMax axis 1 Int32", "mpsgraph/gomlx/mpsgraph_test.go:941-991", [_a([1, 5, 3, 8, 2, 6], shape=(2, 3))],
         lambda f, x: f.ArgMinMax(x, 1, C_I32, False), _a([1, 0], I32), tol=0),
    Case("FusedSoftmax axis 1", "mpsgraph/gomlx/mpsgraph_test.go:1133-1190", [_a([1, 2, 3, 1, 1, 1], shape=(2, 3))],
         lambda f, x: f.FusedSoftmax(x, 1),
         _a([_e1 / (_e1 + _e2 + _e3), _e2 / (_e1 + _e2 + _e3), _e3 / (_e1 + _e2 + _e3), 1 / 3, 1 / 3, 1 / 3], shape=(2, 3)), tol=1e-4),
    Case("Reverse axis 1", "mpsgraph/gomlx/mpsgraph_test.go:1269-1315", [_a([1, 2, 3, 4, 5, 6], shape=(2, 3))],
         lambda f, x: f.Reverse(x, 1), _a([3, 2, 1, 6, 5, 4], shape=(2, 3)), tol=0),
    Case("Equal", "mpsgraph/gomlx/mpsgraph_test.go:1383-1384", [_a([1, 2, 3, 4]), _a([2, 2, 2, 2])], lambda f, x, y: f.Equal(x, y), _a([0, 1, 0, 0], BOOL), tol=0),
    Case("NotEqual", "mpsgraph/gomlx/mpsgraph_test.go:1385-1386", [_a([1, 2, 3, 4]), _a([2, 2, 2, 2])], lambda f, x, y: f.NotEqual(x, y), _a([1, 0, 1, 1], BOOL), tol=0),
    Case("GreaterThan", "mpsgraph/gomlx/mpsgraph_test.go:1387-1388", [_a([1, 2, 3, 4]), _a([2, 2, 2, 2])], lambda f, x, y: f.GreaterThan(x, y), _a([0, 0, 1, 1], BOOL), tol=0),
    Case("LessThan", "mpsgraph/gomlx/mpsgraph_test.go:1389-1390", [_a([1, 2, 3, 4]), _a([2, 2, 2, 2])], lambda f, x, y: f.LessThan(x, y), _a([1, 0, 0, 0], BOOL), tol=0),
    Case("Where", "mpsgraph/gomlx/mpsgraph_test.go:1436-1482", [_a([1, 0, 1, 0], BOOL), _a([10, 20, 30, 40]), _a([1, 2, 3, 4])],
         lambda f, c, t, e: f.Where(c, t, e), _a([10, 2, 30, 4]), tol=0),
    Case("ConvertDType f32 -> i32 truncates", "mpsgraph/gomlx/mpsgraph_test.go:1485-1532", [_a([1.7, 2.3, -0.9])],
         lambda f, x: f.ConvertDType(x, C_I32), _a([1, 2, 0], I32), tol=0),
    Case("ConvertDType f32 -> i64 truncates", "mpsgraph/gomlx/mpsgraph_test.go:2762-2773", [_a([1.5, 2.9, -3.1])],
         lambda f, x: f.ConvertDType(x, C_I64), _a([1, 2, -3], I64), tol=0),
    Case("Transpose [2,3]", "mpsgraph/gomlx/mpsgraph_test.go:1535-1581", [_a([1, 2, 3, 4, 5, 6], shape=(2, 3))],
         lambda f, x: f.Transpose(x, 1, 0), _a([1, 4, 2, 5, 3, 6], shape=(3, 2)), tol=0),
    Case("Multiple outputs", "mpsgraph/gomlx/mpsgraph_test.go:1584-1634", [_a([10, 20, 30]), _a([1, 2, 3])],
         lambda f, x, y: (f.Add(x, y), f.Sub(x, y)), [_a([11, 22, 33]), _a([9, 18, 27])]),
    Case("softmax(QK^T/sqrt d).V", "mpsgraph/gomlx/mpsgraph_test.go:1638-1724",
         [_a([1, 0, 0, 0, 1, 0], shape=(2, 3)), _a([1, 0, 0, 0, 1, 0], shape=(2, 3)), _a([10, 20, 30, 40, 50, 60], shape=(2, 3))],
         lambda f, q, k, v: f.DotGeneral(
             f.FusedSoftmax(f.Mul(f.DotGeneral(q, [1], None, k, [1], None),
                                  f.BroadcastInDim(f.Constant(np.array([1.0 / math.sqrt(3.0)], dtype=np.float32), 1), _shape(f, F32, 2, 2), [1])), 1),
             [1], None, v, [0], None),
         _a([_w0 * 10 + _w1 * 40, _w0 * 20 + _w1 * 50, _w0 * 30 + _w1 * 60, _w1 * 10 + _w0 * 40, _w1 * 20 + _w0 * 50, _w1 * 30 + _w0 * 60], shape=(2, 3)),
         tol=1e-3),
    Case("Chained sigmoid(x*w+b)", "mpsgraph/gomlx/mpsgraph_test.go:1727-1802", [_a([2.0, 3.0, -1.0, 0.5])],
         lambda f, x: f.Logistic(f.Add(f.Mul(x, f.Constant(np.array([0.5, -0.5, 1.0, -1.0], dtype=np.float32), 4)),
                                       f.Constant(np.array([0.1, 0.2, -0.1, 0.0], dtype=np.float32), 4))),
         _a([_sigmoid(1.1), _sigmoid(-1.3), _sigmoid(-1.1), _sigmoid(-0.5)])),
    Case("FusedLayerNorm basic", "mpsgraph/gomlx/mpsgraph_test.go:2598-2609", [_a(range(1, 9), shape=(2, 4))],
         lambda f, x: f.FusedLayerNorm(x, [-1], 1e-5, None, None),
         _a([-1.3416, -0.4472, 0.4472, 1.3416, -1.3416, -0.4472, 0.4472, 1.3416], shape=(2, 4)), tol=1e-3),
    Case("FusedLayerNorm gamma beta", "mpsgraph/gomlx/mpsgraph_test.go:2611-2625",
         [_a(range(1, 9), shape=(2, 4)), _a([2, 2, 2, 2], shape=(1, 4)), _a([1, 1, 1, 1], shape=(1, 4))],
         lambda f, x, g, b: f.FusedLayerNorm(x, [-1], 1e-5, g, b), _a([-1.6833, 0.1056, 1.8944, 3.6833], shape=(1, 4)), tol=1e-3, prefix=4),
    Case("FusedGelu exact", "mpsgraph/gomlx/mpsgraph_test.go:2646-2656", [_a([0.0, 1.0, -1.0, 3.0])],
         lambda f, x: f.FusedGelu(x, True), _a([0.0, 0.8413, -0.1587, 2.9960]), tol=1e-3),
    Case("Int64 add", "mpsgraph/gomlx/mpsgraph_test.go:2749-2760", [_a([1, 2, 3], I64), _a([10, 20, 30], I64)],
         lambda f, a, b: f.Add(a, b), _a([11, 22, 33], I64), tol=0),
    Case("Uint8 add", "mpsgraph/gomlx/mpsgraph_test.go:2790-2803", [_a([100, 200], U8), _a([10, 20], U8)],
         lambda f, a, b: f.Add(a, b), _a([110, 220], U8), tol=0),
    Case("FusedDense identity weight", "mpsgraph/gomlx/mpsgraph_test.go:2809-2825",
         [_a([1, 2, 3, 4, 5, 6], shape=(2, 3)), _a(_eye_w(3, 4))],
         lambda f, x, w: f.FusedDense(x, w, None, 0), _a([1, 2, 3, 0, 4, 5, 6, 0], shape=(2, 4)), tol=1e-4),
    Case("FusedDense with bias", "mpsgraph/gomlx/mpsgraph_test.go:2827-2840",
         [_a([1, 0, 0, 1], shape=(2, 2)), _a([2, 0, 0, 3], shape=(2, 2)), _a([10, 20])],
         lambda f, x, w, b: f.FusedDense(x, w, b, 0), _a([12, 20, 10, 23], shape=(2, 2)), tol=1e-4),
    Case("FusedDense relu", "mpsgraph/gomlx/mpsgraph_test.go:2842-2854",
         [_a([1, -1, -1, 1], shape=(2, 2)), _a([1, 0, 0, 1], shape=(2, 2))],
         lambda f, x, w: f.FusedDense(x, w, None, 2), _a([1, 0, 0, 1], shape=(2, 2)), tol=1e-4),
    Case("QKV projection identity weights", "mpsgraph/gomlx/mpsgraph_test.go:2900-2927",
         [_a(range(1, 13), shape=(2, 6)), _a(_eye_w(6, 6))],
         lambda f, x, w: f.FusedAttentionQKVProjection(x, w, None, None, None, 2, 2),
         [_a([1, 2, 7, 8], shape=(2, 2)), _a([3, 4, 9, 10], shape=(2, 2)), _a([5, 6, 11, 12], shape=(2, 2))], tol=1e-4),
    Case("QKV projection with biases", "mpsgraph/gomlx/mpsgraph_test.go:2929-2963",
         [_a([1, 2, 3, 4], shape=(1, 4)), _a(_eye_w(4, 6)), _a([10, 20]), _a([100, 200]), _a([1000, 2000])],
         lambda f, x, w, bq, bk, bv: f.FusedAttentionQKVProjection(x, w, bq, bk, bv, 2, 2),
         [_a([11, 22], shape=(1, 2)), _a([103, 204], shape=(1, 2)), _a([1000, 2000], shape=(1, 2))], tol=1e-4),
    Case("SDPA causal: row 0 = V[0]", "mpsgraph/gomlx/mpsgraph_test.go:2995-3014",
         [_a([1, 0, 0, 1, 1, 1], shape=(1, 1, 3, 2)), _a([1, 0, 0, 1, 1, 1], shape=(1, 1, 3, 2)), _a([1, 0, 0, 1, 0.5, 0.5], shape=(1, 1, 3, 2))],
         lambda f, q, k, v: f.FusedScaledDotProductAttention(q, k, v, None, 1, 1, 0, 1.0, True), _a([1, 0]), tol=1e-3, prefix=2),
    Case("SDPA bool mask: row 0 = V[0]", "mpsgraph/gomlx/mpsgraph_test.go:3033-3057",
         [_a([1, 0, 0, 1], shape=(1, 1, 2, 2)), _a([1, 0, 0, 1], shape=(1, 1, 2, 2)), _a([10, 20, 30, 40], shape=(1, 1, 2, 2)),
          _a([1, 0, 1, 1], BOOL, (1, 1, 2, 2))],
         lambda f, q, k, v, m: f.FusedScaledDotProductAttention(q, k, v, m, 1, 1, 0, 1.0, False), _a([10, 20]), tol=1e-3, prefix=2),
    Case("BFloat16 add", "mpsgraph/gomlx/mpsgraph_test.go:3131-3141", [_a([1.0, 2.0, 3.0, 4.0])],
         lambda f, x: f.ConvertDType((lambda b: f.Add(b, b))(f.ConvertDType(x, C_BF16)),
                                     C_F32),
         _a([2.0, 4.0, 6.0, 8.0]), tol=0.1),
    Case("BFloat16 matmul", "mpsgraph/gomlx/mpsgraph_test.go:3143-3156", [_a([1, 2, 3, 4], shape=(2, 2)), _a([5, 6, 7, 8], shape=(2, 2))],
         lambda f, a, b: f.ConvertDType(
             f.DotGeneral(f.ConvertDType(a, C_BF16), [1], None,
                          f.ConvertDType(b, C_BF16), [0], None),
             C_F32),
         _a([19, 22, 43, 50], shape=(2, 2)), tol=1.0),
    # training-side ops
    Case("ScatterSum embedding gradient", "mpsgraph/gomlx/mpsgraph_test.go:1192-1262",
         [_a([0] * 8, shape=(4, 2)), _a([0, 2, 0], I32, (3, 1)), _a([1, 2, 3, 4, 5, 6], shape=(3, 2))],
         lambda f, operand, indices, updates: f.ScatterSum(operand, indices, updates, 1, [1], [0], [0], False, False),
         _a([6, 8, 0, 0, 3, 4, 0, 0], shape=(4, 2)), tol=1e-5),
    Case("BatchNormForTraining basic (mean, variance)", "mpsgraph/gomlx/mpsgraph_test.go:3064-3101",
         [_a([1, 2, 3, 4, 5, 6, 7, 8], shape=(4, 2)), _a([1, 1]), _a([0, 0])],
         lambda f, op, sc, off: list(f.BatchNormForTraining(op, sc, off, 1e-5, 1)[1:]),
         [_a([4, 5]), _a([5, 5])], tol=1e-3),
    Case("BatchNormForTraining scale and offset", "mpsgraph/gomlx/mpsgraph_test.go:3103-3124",
         [_a([0, 10, 0, 10], shape=(2, 2)), _a([2, 3]), _a([1, -1])],
         lambda f, op, sc, off: list(f.BatchNormForTraining(op, sc, off, 1e-5, 1)[:2]),
         [_a([1, -1, 1, -1], shape=(2, 2)), _a([0, 10])], tol=1e-3),
    # control flow over closures
    Case("While sum 1..10", "mpsgraph/gomlx/mpsgraph_test.go:3379-3410", [_a(0, I32)], _while_sum, _a(55, I32), tol=0),
    Case("While factorial 5!", "mpsgraph/gomlx/mpsgraph_test.go:3412-3442", [_a(0, I32)], _while_factorial, _a(120, I32), tol=0),
    Case("If true branch (10 > 5)", "mpsgraph/gomlx/mpsgraph_test.go:3449-3472", [_a(10.0)], _if_const, _a(1.0), tol=0),
    Case("If false branch (3 > 5)", "mpsgraph/gomlx/mpsgraph_test.go:3474-3497", [_a(3.0)], _if_const, _a(-1.0), tol=0),
    Case("If with captured values (3 * 10)", "mpsgraph/gomlx/mpsgraph_test.go:3499-3523", [_a(3.0)], _if_captured, _a(30.0), tol=0),
    Case("Sort ascending", "mpsgraph/gomlx/mpsgraph_test.go:3529-3538", [_a([5, 2, 8, 1, 9, 3])], _sort(False), _a([1, 2, 3, 5, 8, 9]), tol=0),
    Case("Sort descending", "mpsgraph/gomlx/mpsgraph_test.go:3540-3549", [_a([5, 2, 8, 1, 9, 3])], _sort(True), _a([9, 8, 5, 3, 2, 1]), tol=0),
    Case("Call add(10, 32)", "mpsgraph/gomlx/mpsgraph_test.go:3556-3578", [_a(0.0)], _call_add, _a(42.0), tol=0),
]

# Shape-only expectations of the reference's tests (the test asserts a shape or finiteness, not values).
SHAPE_CASES = [
    ("SDPA BHSD basic", "mpsgraph/gomlx/mpsgraph_test.go:2969-2993", (1, 1, 2, 2), 0),
    ("SDPA BSHD layout", "mpsgraph/gomlx/mpsgraph_test.go:3016-3031", (1, 2, 1, 2), 1),
]


def check(outputs, case: Case):
    """Returns a list of mismatch descriptions (empty = pass)."""
    outs = outputs if isinstance(outputs, (list, tuple)) else [outputs]
    bad = []
    if len(outs) != len(case.expected):
        return [f"{case.name}: {len(outs)} outputs, expected {len(case.expected)}"]
    for i, (got, want) in enumerate(zip(outs, case.expected)):
        got = np.asarray(got)
        g = got.reshape(-1)
        w = want.reshape(-1)
        if case.prefix is not None:
            g = g[:case.prefix]
        elif got.shape != want.shape:
            bad.append(f"{case.name}[{i}]: shape {got.shape}, expected {want.shape}")
            continue
        if got.dtype != want.dtype:
            bad.append(f"{case.name}[{i}]: dtype {got.dtype}, expected {want.dtype}")
            continue
        if case.tol == 0 or want.dtype.kind in "biu":
            if not np.array_equal(g, w):
                bad.append(f"{case.name}[{i}]: got {g.tolist()}, expected exactly {w.tolist()}")
        else:
            diff = np.abs(g.astype(np.float64) - w.astype(np.float64))
            if not (diff <= case.tol).all():
                bad.append(f"{case.name}[{i}]: got {g.tolist()}, expected {w.tolist()} within {case.tol}")
    return bad


if __name__ == "__main__":
    for c in CASES:
        print(f"{c.name:40s} {c.cite:55s} tol={c.tol} expected={[e.reshape(-1).tolist() for e in c.expected]}")
