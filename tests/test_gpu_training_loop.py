"""A training run expressed in backend ops: linear regression by SGD, the 500 steps as ONE While loop.

The reference's TestTrainingLinearRegression (mpsgraph/gomlx/mpsgraph_test.go:2118-2194) trains y = 2 x1 + 3 x2 + 1 on
four examples with learning rate 0.1 for 500 steps through GoMLX's trainer (autodiff on the host, one Execute per step)
and asks for a loss below 5.0 and weights near [2, 3], bias near 1.  GoMLX's autodiff is not available here, so the
gradients of the mean squared error are written out by hand; what the test exercises is the same op mix per step
(DotGeneral in both operand orders, reductions, broadcasts, elementwise) and, beyond the reference, the whole loop
inside one executable: host-driven on the first runs, a conditional graph node on the device when replayed.
"""
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.golden.reference_vectors import closure
from tests.util import default_switches

pytestmark = pytest.mark.gpu

X = np.array([[1, 0], [0, 1], [1, 1], [2, 1]], dtype=np.float32)
Y = np.array([[3], [4], [6], [8]], dtype=np.float32)
STEPS, LR = 500, 0.1


def _sh(b200, dtype, *dims):
    return b200.Shape(b200.dtypes.from_numpy(np.dtype(dtype)), dims)


def _c(f, value, dtype):
    return f.Constant(np.array([value], dtype=dtype))


def _train(f, shape, x, y):
    """(steps done, weights [2,1], bias [1], loss) after STEPS steps of SGD on mean((x w + b - y)^2)."""
    si, sw, sb = shape(np.int32), shape(np.float32, 2, 1), shape(np.float32, 1)
    s41 = shape(np.float32, 4, 1)

    def predict(c, w, b):
        return c.Add(c.DotGeneral(x, [1], [], w, [0], []), c.BroadcastInDim(b, s41, [1]))

    def body(c, i, w, b):
        err = c.Sub(predict(c, w, b), y)                                   # [4, 1]
        scale = _c(c, 2.0 * LR / 4.0, np.float32)                          # lr * d(mean err^2)/d(pred) = lr * 2 err / 4
        gw = c.DotGeneral(x, [0], [], err, [0], [])                        # x^T err: [2, 1]
        gb = c.ReduceSum(err, 0)                                           # [1]
        w2 = c.Sub(w, c.Mul(gw, c.BroadcastInDim(scale, sw, [])))
        b2 = c.Sub(b, c.Mul(gb, c.BroadcastInDim(scale, sb, [])))
        return [c.Add(i, _c(c, 1, np.int32)), w2, b2]

    cond = closure(f, [si, sw, sb], lambda c, i, w, b: [c.LessThan(i, _c(c, STEPS, np.int32))])
    loop_body = closure(f, [si, sw, sb], body)
    w0 = f.Constant(np.zeros(2, dtype=np.float32), 2, 1)
    b0 = f.Constant(np.zeros(1, dtype=np.float32), 1)
    i_end, w, b = f.While(cond, loop_body, _c(f, 0, np.int32), w0, b0)
    err = f.Sub(predict(f, w, b), y)
    loss = f.Mul(f.ReduceSum(f.Mul(err, err)), _c(f, 0.25, np.float32))
    return [i_end, w, b, loss]


def test_linear_regression_sgd_as_one_loop(b200, backend):
    builder = backend.Builder("train")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 4, 2))
    y = f.Parameter("y", _sh(b200, np.float32, 4, 1))
    f.Return(_train(f, lambda dt, *d: _sh(b200, dt, *d), x, y), None)
    exe = builder.Compile()
    assert ("on the device when replayed" in exe.Describe()) or not default_switches(), exe.Describe()
    orc = OracleFunction()
    want = _train(orc, lambda dt, *d: _sh(b200, dt, *d), X, Y)
    bx, by = backend.FromNumpy(X), backend.FromNumpy(Y)
    for run in range(4):   # runs 3 and 4 replay the recorded plan: the 500 steps run without the host
        outs = exe.Execute([bx, by], None, 0)
        i_end, w, b, loss = (backend.ToNumpy(o) for o in outs)
        for o in outs:
            backend.BufferFinalize(o)
        assert int(i_end) == STEPS
        # the reference's own criteria (mpsgraph_test.go:2179-2181 and the comment at :2183)
        assert float(loss) < 5.0
        np.testing.assert_allclose(w.reshape(-1), [2.0, 3.0], atol=2e-2)
        np.testing.assert_allclose(b, [1.0], atol=3e-2)
        # and the same trajectory as the op-by-op oracle: 500 fp32 steps, each within rounding of it
        for got, ref, what in ((w, want[1], "weights"), (b, want[2], "bias")):
            ok, viol = compare(got, np.asarray(ref), 1e-4, 1.0)
            assert ok, (run, what, viol)
        assert abs(float(loss) - float(want[3])) <= 1e-5 + 1e-3 * abs(float(want[3]))
    exe.Finalize()
    builder.Finalize()
