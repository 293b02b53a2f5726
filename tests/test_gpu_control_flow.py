"""Control flow over closures -- Call, While, If, Sort -- through the C ABI, against the CPU oracle.

One graph-building routine drives both sides: `closure` / `named_function` (tests/golden/reference_vectors.py) build a
Function.Closure() / Builder.NewFunction() on the backend and a Python callable on the oracle, whose While / If / Sort
restate the reference's host-side executors (ref mpsgraph/gomlx/executable.go:219-480).  Integer and index work is
bit-exact; float loops compare at rel 1e-5.
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.golden.reference_vectors import closure, named_function
from tests.util import default_switches, assert_parity, run_backend, run_oracle

pytestmark = pytest.mark.gpu

BF16 = ml_dtypes.bfloat16


def _sh(b200, dtype, *dims):
    return b200.Shape(b200.dtypes.from_numpy(np.dtype(dtype)), dims)


def _c(f, value, dtype):
    return f.Constant(np.array([value], dtype=dtype))


# ------------------------------------------------------------------------------ While ---
def test_while_with_tensor_state_and_captured_values(b200, backend):
    # state: (counter i32, x f32[3, 257]); body captures y (an input) and a value computed from it in the parent
    rng = np.random.default_rng(0)
    x0 = rng.standard_normal((3, 257)).astype(np.float32)
    y = rng.standard_normal((3, 257)).astype(np.float32)
    limit = np.array(7, dtype=np.int32)

    def build(f, x, yy, lim):
        si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 3, 257)
        y2 = f.Mul(yy, yy)   # computed outside, captured by the body
        half = f.BroadcastInDim(_c(f, 0.5, np.float32), sx, [])
        cond = closure(f, [si, sx], lambda c, i, v: [c.LessThan(i, lim)])   # captures a parameter of main
        body = closure(f, [si, sx], lambda c, i, v: [c.Add(i, _c(c, 1, np.int32)), c.Add(c.Mul(v, half), c.Sub(y2, yy))])
        i_end, x_end = f.While(cond, body, _c(f, 0, np.int32), x)
        return i_end, f.Add(x_end, yy)   # the loop's result feeds further ops

    got = assert_parity(b200, backend, build, [x0, y, limit], rtol=1e-5, atol_scale=1.0, what="While")
    assert int(got[0]) == 7


def test_while_zero_trips_returns_the_initial_state(b200, backend):
    x0 = np.arange(12, dtype=np.int32).reshape(3, 4)

    def build(f, x):
        sx = _sh(b200, np.int32, 3, 4)
        cond = closure(f, [sx], lambda c, v: [c.LessThan(c.ReduceSum(v), _c(c, 0, np.int32))])   # sum = 66: false at once
        body = closure(f, [sx], lambda c, v: [c.Add(v, v)])
        return f.While(cond, body, x)[0]

    (got,) = assert_parity(b200, backend, build, [x0], what="While zero trips")
    np.testing.assert_array_equal(got, x0)


def test_two_loops_in_one_function_and_an_unused_state_value(b200, backend):
    # the reference allows one control-flow op per function (ref function.go:407-409); there is no such limit here
    def build(f, x):
        si = _sh(b200, np.int32)
        sv = _sh(b200, np.float32, 1000)
        cond = closure(f, [si, sv, sv], lambda c, i, a, b: [c.LessThan(i, _c(c, 5, np.int32))])
        body = closure(f, [si, sv, sv], lambda c, i, a, b: [c.Add(i, _c(c, 1, np.int32)), c.Add(a, b), c.Mul(b, c.BroadcastInDim(_c(c, 0.9, np.float32), sv, []))])
        _, a1, _ = f.While(cond, body, _c(f, 0, np.int32), x, x)   # counter and b are never read
        cond2 = closure(f, [sv], lambda c, a: [c.LessThan(c.ReduceMax(c.Abs(a)), _c(c, 1e4, np.float32))])
        body2 = closure(f, [sv], lambda c, a: [c.Add(a, a)])
        (a2,) = f.While(cond2, body2, a1)   # data-dependent trip count
        return a1, a2

    x = np.random.default_rng(1).standard_normal(1000).astype(np.float32)
    got = assert_parity(b200, backend, build, [x], rtol=1e-5, atol_scale=1.0, what="two loops")
    assert np.abs(got[1]).max() >= 1e4


def test_while_runs_the_same_on_every_execution(b200, backend):
    builder = backend.Builder("loop")
    f = builder.Main()
    n = f.Parameter("n", _sh(b200, np.int32))
    si = _sh(b200, np.int32)
    cond = closure(f, [si, si], lambda c, i, acc: [c.LessThan(i, n)])
    body = closure(f, [si, si], lambda c, i, acc: [c.Add(i, _c(c, 1, np.int32)), c.Add(acc, c.Mul(i, i))])
    f.Return([f.While(cond, body, _c(f, 0, np.int32), _c(f, 0, np.int32))[1]], None)
    exe = builder.Compile()
    assert "while[" in exe.Describe()
    for trips in (0, 1, 10, 10, 300, 3):   # the trip count is an input: one executable, any count
        buf = backend.FromNumpy(np.array(trips, dtype=np.int32))
        (out,) = exe.Execute([buf], None, 0)
        assert int(backend.ToNumpy(out)) == sum(i * i for i in range(trips))
        backend.BufferFinalize(out)
        backend.BufferFinalize(buf)
    exe.Finalize()
    builder.Finalize()


def test_while_on_the_device_when_the_plan_is_replayed(b200, backend):
    # the third run on the same buffers replays the plan as a CUDA graph in which the loop is a conditional node: cond,
    # body and the trip decision all run on the device.  Same results as the host-driven runs before it, for several
    # trip counts through ONE recorded graph (the count is data), including zero trips.
    rng = np.random.default_rng(7)
    x0 = rng.standard_normal((64, 96)).astype(np.float32)
    w = rng.standard_normal((64, 96)).astype(np.float32)
    builder = backend.Builder("device-loop")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 64, 96))
    ww = f.Parameter("w", _sh(b200, np.float32, 64, 96))
    n = f.Parameter("n", _sh(b200, np.int32))
    si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 64, 96)
    cond = closure(f, [si, sx], lambda c, i, v: [c.LessThan(i, n)])
    body = closure(f, [si, sx], lambda c, i, v: [c.Add(i, _c(c, 1, np.int32)), c.Tanh(c.Add(c.Mul(v, ww), c.Reverse(v, 1)))])
    i_end, x_end = f.While(cond, body, _c(f, 0, np.int32), x)
    f.Return([i_end, f.Neg(x_end)], None)
    exe = builder.Compile()
    assert ("on the device when replayed" in exe.Describe()) or not default_switches(), exe.Describe()
    bx, bw = backend.FromNumpy(x0), backend.FromNumpy(w)
    bn = backend.FromNumpy(np.array(0, dtype=np.int32))

    def want(trips):
        v = x0.astype(np.float64)
        for _ in range(trips):
            v = np.tanh(v * w.astype(np.float64) + v[:, ::-1])
        return -v

    for trips in (3, 3, 3, 0, 7, 1, 25, 0, 3):   # runs 1-2 are driven by the host, the rest replay the graph
        backend.BufferFinalize(bn)
        bn = backend.FromNumpy(np.array(trips, dtype=np.int32))   # the freed block comes back: same address, new count
        outs = exe.Execute([bx, bw, bn], None, 0)
        got_i, got_x = (backend.ToNumpy(o) for o in outs)
        for o in outs:
            backend.BufferFinalize(o)
        assert int(got_i) == trips
        ok, viol = compare(got_x, want(trips).astype(np.float32), 2e-5, 1.0)
        assert ok, (trips, viol)
    exe.Finalize()
    builder.Finalize()


def test_while_with_an_fp32_contraction_in_its_body_replays_on_the_device(b200, backend):
    # the fp32 DotGeneral's split planes live in the sub-plan's arena, so the loop is recordable
    rng = np.random.default_rng(8)
    x0 = rng.standard_normal((128, 128)).astype(np.float32)
    w = (0.1 * rng.standard_normal((128, 128))).astype(np.float32)
    builder = backend.Builder("device-loop-f32")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 128, 128))
    ww = f.Parameter("w", _sh(b200, np.float32, 128, 128))
    si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 128, 128)
    cond = closure(f, [si, sx], lambda c, i, v: [c.LessThan(i, _c(c, 4, np.int32))])
    body = closure(f, [si, sx], lambda c, i, v: [c.Add(i, _c(c, 1, np.int32)), c.Tanh(c.DotGeneral(v, [1], [], ww, [0], []))])
    f.Return([f.While(cond, body, _c(f, 0, np.int32), x)[1]], None)
    exe = builder.Compile()
    assert ("on the device when replayed" in exe.Describe()) or not default_switches(), exe.Describe()
    v = x0.astype(np.float64)
    for _ in range(4):
        v = np.tanh(v @ w.astype(np.float64))
    bx, bw = backend.FromNumpy(x0), backend.FromNumpy(w)
    for run in range(4):
        (out,) = exe.Execute([bx, bw], None, 0)
        got = backend.ToNumpy(out)
        backend.BufferFinalize(out)
        ok, viol = compare(got, v.astype(np.float32), 1e-5, 1.0)
        assert ok, (run, viol)
    exe.Finalize()
    builder.Finalize()


def test_nested_loops(b200, backend):
    # a loop inside a loop's body (the reference allows one control-flow op per function, ref function.go:407-409): the
    # inner loop's trip count depends on the outer counter, its body uses the outer body's parameters and a value of main
    rng = np.random.default_rng(9)
    x0 = rng.standard_normal((5, 40)).astype(np.float32)
    y = (0.1 * rng.standard_normal((5, 40))).astype(np.float32)

    def build(f, x, yy):
        si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 5, 40)

        def outer_body(c, i, v):
            # inner: j from 0 to i: w = w * 0.5 + v * y   (v: the outer body's parameter, yy: a value of main)
            icond = closure(c, [si, sx], lambda d, j, w: [d.LessThan(j, i)])
            ibody = closure(c, [si, sx], lambda d, j, w: [d.Add(j, _c(d, 1, np.int32)),
                                                          d.Add(d.Mul(w, d.BroadcastInDim(_c(d, 0.5, np.float32), sx, [])), d.Mul(v, yy))])
            _, w_end = c.While(icond, ibody, _c(c, 0, np.int32), v)
            return [c.Add(i, _c(c, 1, np.int32)), c.Tanh(w_end)]

        cond = closure(f, [si, sx], lambda c, i, v: [c.LessThan(i, _c(c, 4, np.int32))])
        body = closure(f, [si, sx], outer_body)
        i_end, v_end = f.While(cond, body, _c(f, 0, np.int32), x)
        return i_end, v_end

    got = assert_parity(b200, backend, build, [x0, y], rtol=1e-5, atol_scale=1.0, what="nested loops")
    assert int(got[0]) == 4
    # and replayed: the inner loop is a conditional node inside the outer loop's body graph
    builder = backend.Builder("nested")
    f = builder.Main()
    px, py = f.Parameter("x", _sh(b200, np.float32, 5, 40)), f.Parameter("y", _sh(b200, np.float32, 5, 40))
    f.Return(list(build(f, px, py)), None)
    exe = builder.Compile()
    bx, by = backend.FromNumpy(x0), backend.FromNumpy(y)
    for run in range(4):
        outs = exe.Execute([bx, by], None, 0)
        v = backend.ToNumpy(outs[1])
        for o in outs:
            backend.BufferFinalize(o)
        np.testing.assert_array_equal(v, got[1])   # every run, host-driven or replayed, gives the same bits
    exe.Finalize()
    builder.Finalize()


def test_a_loop_inside_a_function_that_is_called_twice(b200, backend):
    def build(f, x, n):
        si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 3, 50)

        def repeat(c, v, count):   # v <- tanh(v + 0.25) `count` times
            cond = closure(c, [si, sx], lambda d, j, w: [d.LessThan(j, count)])
            body = closure(c, [si, sx], lambda d, j, w: [d.Add(j, _c(d, 1, np.int32)),
                                                         d.Tanh(d.Add(w, d.BroadcastInDim(_c(d, 0.25, np.float32), sx, [])))])
            return [c.While(cond, body, _c(c, 0, np.int32), v)[1]]

        fn = named_function(f, "repeat", [sx, si], repeat)
        (a,) = f.Call(fn, x, n)
        (b,) = f.Call(fn, f.Neg(a), f.Add(n, n))   # the same function, other values, twice the trips
        return a, b

    x = np.random.default_rng(10).standard_normal((3, 50)).astype(np.float32)
    assert_parity(b200, backend, build, [x, np.array(3, dtype=np.int32)], rtol=1e-5, atol_scale=1.0, what="loop in a function")


def test_while_refusals(b200, backend):
    builder = backend.Builder("bad")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 4))
    sx, si = _sh(b200, np.float32, 4), _sh(b200, np.int32)
    ok_cond = closure(f, [sx], lambda c, v: [c.LessThan(c.ReduceSum(v), _c(c, 0, np.float32))])
    ok_body = closure(f, [sx], lambda c, v: [c.Add(v, v)])
    with pytest.raises(b200.BackendError, match="at least one initial state"):       # ref function.go:410-412
        f.While(ok_cond, ok_body)
    with pytest.raises(b200.BackendError, match="cond must return scalar bool"):      # ref function.go:443-445
        f.While(closure(f, [sx], lambda c, v: [c.ReduceSum(v)]), ok_body, x)
    with pytest.raises(b200.BackendError, match="cond must have 1 parameters"):       # ref function.go:429-432
        f.While(closure(f, [sx, sx], lambda c, v, w: [c.LessThan(c.ReduceSum(v), c.ReduceSum(w))]), ok_body, x)
    with pytest.raises(b200.BackendError, match="doesn't match state shape"):         # ref function.go:433-438
        f.While(closure(f, [si], lambda c, v: [c.LessThan(v, v)]), ok_body, x)
    with pytest.raises(b200.BackendError, match="body output 0 shape"):               # ref function.go:462-467
        f.While(ok_cond, closure(f, [sx], lambda c, v: [c.ReduceSum(v)]), x)
    other = builder.NewFunction("other")
    with pytest.raises(b200.BackendError, match="must be a closure of the current function"):   # ref function.go:239-241
        f.While(closure(other, [sx], lambda c, v: [c.LessThan(c.ReduceSum(v), c.ReduceSum(v))]), ok_body, x)
    unfinished = f.Closure()
    unfinished.Parameter("v", sx)
    with pytest.raises(b200.BackendError, match="must have Return\\(\\) called"):     # ref function.go:242-244
        f.While(unfinished, ok_body, x)
    with pytest.raises(b200.BackendError, match="unrelated function scope"):          # ref function.go:194
        inner = other.Closure()
        inner.Neg(x)   # x belongs to main, which is not an ancestor of `other`'s closure
    builder.Finalize()


# --------------------------------------------------------------------------------- If ---
@pytest.mark.parametrize("threshold", [-100.0, 100.0], ids=["true", "false"])
def test_if_with_tensor_outputs_and_captures(b200, backend, threshold):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((64, 130)).astype(np.float32)
    w = rng.standard_normal((130, 32)).astype(np.float32)

    def build(f, xx, ww):
        pred = f.GreaterThan(f.ReduceSum(xx), _c(f, threshold, np.float32))
        t = closure(f, [], lambda c: [c.DotGeneral(xx, [1], [], ww, [0], []), c.Exp(xx)])
        e = closure(f, [], lambda c: [c.Neg(c.DotGeneral(c.Abs(xx), [1], [], ww, [0], [])), c.Tanh(xx)])
        return f.If(pred, t, e)

    assert_parity(b200, backend, build, [x, w], rtol=1e-5, atol_scale=1.0, what="If")


def test_heavy_branches_run_one_at_a_time_and_on_the_device_when_replayed(b200, backend):
    # branches with contractions are not both evaluated: each is a sub-plan and one of them runs.  One executable, the
    # predicate flipping between runs; runs 3+ replay the recorded plan, where two conditional graph nodes pick the branch.
    rng = np.random.default_rng(11)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    w = rng.standard_normal((128, 32)).astype(np.float32)
    builder = backend.Builder("branch")
    f = builder.Main()
    px = f.Parameter("x", _sh(b200, np.float32, 64, 128))
    pw = f.Parameter("w", _sh(b200, np.float32, 128, 32))
    pt = f.Parameter("threshold", _sh(b200, np.float32))
    pred = f.GreaterThan(f.ReduceSum(px), pt)
    t = closure(f, [], lambda c: [c.DotGeneral(px, [1], [], pw, [0], []), c.Exp(px)])
    e = closure(f, [], lambda c: [c.Neg(c.DotGeneral(c.Abs(px), [1], [], pw, [0], [])), c.Tanh(px)])
    a, b = f.If(pred, t, e)
    f.Return([f.Add(a, a), b], None)   # the branch's results feed further ops
    exe = builder.Compile()
    assert ("if[" in exe.Describe() and "on the device when replayed" in exe.Describe()) or not default_switches(), exe.Describe()
    x64, w64 = x.astype(np.float64), w.astype(np.float64)
    want = {True: (2 * (x64 @ w64), np.exp(x64)), False: (-2 * (np.abs(x64) @ w64), np.tanh(x64))}
    bx, bw = backend.FromNumpy(x), backend.FromNumpy(w)
    bt = backend.FromNumpy(np.array(0, dtype=np.float32))
    for thr in (-1e6, -1e6, -1e6, 1e6, -1e6, 1e6, 1e6):
        backend.BufferFinalize(bt)
        bt = backend.FromNumpy(np.array(thr, dtype=np.float32))   # the freed block comes back: same address, new threshold
        outs = exe.Execute([bx, bw, bt], None, 0)
        got = [backend.ToNumpy(o) for o in outs]
        for o in outs:
            backend.BufferFinalize(o)
        taken = bool(x.sum() > thr)
        for g, wnt in zip(got, want[taken]):
            ok, viol = compare(g, wnt.astype(np.float32), 1e-5, 1.0)
            assert ok, (thr, viol)
    exe.Finalize()
    builder.Finalize()


def test_a_branch_inside_a_loop(b200, backend):
    # Collatz steps on a vector's first element decide, per trip, which heavy branch transforms the vector
    def build(f, x, n):
        si, sx = _sh(b200, np.int32), _sh(b200, np.float32, 8, 8)

        def body(c, i, v):
            even = c.Equal(c.Rem(i, _c(c, 2, np.int32)), _c(c, 0, np.int32))
            t = closure(c, [], lambda d: [d.Tanh(d.DotGeneral(v, [1], [], v, [0], []))])
            e = closure(c, [], lambda d: [d.Neg(d.DotGeneral(v, [0], [], v, [0], []))])
            (nv,) = c.If(even, t, e)
            return [c.Add(i, _c(c, 1, np.int32)), c.Mul(nv, c.BroadcastInDim(_c(c, 0.3, np.float32), sx, []))]

        cond = closure(f, [si, sx], lambda c, i, v: [c.LessThan(i, n)])
        return f.While(cond, closure(f, [si, sx], body), _c(f, 0, np.int32), x)[1]

    x = (0.5 * np.random.default_rng(12).standard_normal((8, 8))).astype(np.float32)
    assert_parity(b200, backend, build, [x, np.array(5, dtype=np.int32)], rtol=1e-5, atol_scale=1.0, what="branch in a loop")


def test_if_refusals(b200, backend):
    builder = backend.Builder("bad-if")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 4))
    pred = f.GreaterThan(f.ReduceSum(x), _c(f, 0, np.float32))
    t = closure(f, [], lambda c: [c.Neg(x)])
    with pytest.raises(b200.BackendError, match="pred must be scalar bool"):          # ref function.go:502-504
        f.If(f.ReduceSum(x), t, t)
    with pytest.raises(b200.BackendError, match="trueBranch must have no parameters"):   # ref function.go:516-518
        f.If(pred, closure(f, [_sh(b200, np.float32, 4)], lambda c, v: [v]), t)
    with pytest.raises(b200.BackendError, match="same number of outputs"):            # ref function.go:524-527
        f.If(pred, t, closure(f, [], lambda c: [c.Neg(x), c.Abs(x)]))
    with pytest.raises(b200.BackendError, match="output 0 shapes must match"):        # ref function.go:528-533
        f.If(pred, t, closure(f, [], lambda c: [c.ReduceSum(x)]))
    builder.Finalize()


# ------------------------------------------------------------------------------- Call ---
def test_call_twice_and_nested(b200, backend):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((8, 16)).astype(np.float32)
    b = rng.standard_normal((8, 16)).astype(np.float32)

    def build(f, aa, bb):
        s = _sh(b200, np.float32, 8, 16)
        fma = named_function(f, "fma", [s, s], lambda c, u, v: [c.Add(c.Mul(u, v), u), c.Sub(u, v)])
        twice = named_function(f, "twice", [s], lambda c, u: [c.Call(fma, u, u)[0]])   # a function that calls a function
        p, q = f.Call(fma, aa, bb)
        r, _ = f.Call(fma, q, p)   # the same function again, on other values
        (t,) = f.Call(twice, r)
        return p, q, r, t

    assert_parity(b200, backend, build, [a, b], rtol=1e-5, atol_scale=1.0, what="Call")


def test_call_refusals(b200, backend):
    builder = backend.Builder("bad-call")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 4))
    s = _sh(b200, np.float32, 4)
    g = named_function(f, "g", [s, s], lambda c, u, v: [c.Add(u, v)])
    with pytest.raises(b200.BackendError, match="expects 2 parameters, got 1"):       # ref function.go:373-376
        f.Call(g, x)
    with pytest.raises(b200.BackendError, match="parameter 1 shape mismatch"):        # ref function.go:377-382
        f.Call(g, x, f.ReduceSum(x))
    h = builder.NewFunction("h")
    h.Parameter("u", s)
    with pytest.raises(b200.BackendError, match="must have Return\\(\\) called"):     # ref function.go:368-370
        f.Call(h, x)
    other = backend.Builder("elsewhere")
    with pytest.raises(b200.BackendError, match="same builder"):                     # ref function.go:365-367
        f.Call(named_function(other.Main(), "k", [s], lambda c, u: [c.Neg(u)]), x)
    other.Finalize()
    builder.Finalize()


# ------------------------------------------------------------------------------- Sort ---
def _sort_build(b200, dtype, axis, descending, n_inputs=1):
    def build(f, *xs):
        s = _sh(b200, dtype)
        shapes = [s, s] + [_sh(b200, np.int32)] * (2 * (n_inputs - 1))
        comparator = closure(f, shapes, lambda c, a, b, *rest: [c.GreaterThan(a, b) if descending else c.LessThan(a, b)])
        return f.Sort(comparator, axis, True, *xs)
    return build


@pytest.mark.parametrize("dtype", [np.float32, BF16, np.float16, np.int32, np.int16, np.int8, np.uint8, np.uint32],
                         ids=["f32", "bf16", "f16", "i32", "i16", "i8", "u8", "u32"])
@pytest.mark.parametrize("descending", [False, True], ids=["asc", "desc"])
def test_sort_dtypes_on_each_axis(b200, backend, dtype, descending):
    rng = np.random.default_rng(4)
    if np.dtype(dtype).kind in "iu":
        info = np.iinfo(dtype)
        x = rng.integers(info.min, int(info.max) + 1, size=(5, 37, 6), dtype=np.int64).astype(dtype)
        x[0, 0, 0], x[0, 1, 0] = info.min, info.max
    else:
        x = rng.standard_normal((5, 37, 6)).astype(np.float32).astype(dtype)
        x[1, 3, 2], x[1, 4, 2] = np.inf, -np.inf
    for axis in (0, 1, -1):
        (got,) = run_backend(b200, backend, _sort_build(b200, dtype, axis, descending), [x])
        want = np.sort(x, axis=axis, kind="stable")
        if descending:
            want = np.flip(want, axis=axis)
        np.testing.assert_array_equal(got.view(np.uint8), np.ascontiguousarray(want).view(np.uint8))


@pytest.mark.parametrize("n", [1, 2, 7, 1000, 4096, 4097, 70001])
def test_sort_row_lengths_against_the_comparator_oracle_and_numpy(b200, backend, n):
    # rows up to 4096 keys sort in shared memory, longer ones in device scratch; keys repeat, so stability shows in the payload
    rng = np.random.default_rng(n)
    keys = rng.integers(0, max(2, n // 3), size=(3, n)).astype(np.float32)
    payload = np.broadcast_to(np.arange(n, dtype=np.int32), (3, n)).copy()
    for descending in (False, True):
        got = run_backend(b200, backend, _sort_build(b200, np.float32, 1, descending, 2), [keys, payload])
        order = np.argsort(-keys if descending else keys, axis=1, kind="stable")
        np.testing.assert_array_equal(got[0], np.take_along_axis(keys, order, 1))
        np.testing.assert_array_equal(got[1], order.astype(np.int32))   # equal keys keep their input order
        if n <= 1000:   # the comparison-sort restatement of the reference's executor (pure Python: small cases)
            want = run_oracle(_sort_build(b200, np.float32, 1, descending, 2), [keys, payload])
            np.testing.assert_array_equal(got[0], want[0])
            np.testing.assert_array_equal(got[1], want[1])


def test_sort_many_rows_properties(b200, backend):
    # size-independent properties at a size the Python oracle cannot reach: sortedness, and the output is a permutation
    rng = np.random.default_rng(5)
    x = rng.standard_normal((4096, 2048)).astype(np.float32)
    idx = np.broadcast_to(np.arange(2048, dtype=np.int32), x.shape).copy()
    got, perm = run_backend(b200, backend, _sort_build(b200, np.float32, -1, False, 2), [x, idx])
    assert (np.diff(got, axis=1) >= 0).all()
    np.testing.assert_array_equal(np.sort(perm, axis=1), idx)
    np.testing.assert_array_equal(np.take_along_axis(x, perm.astype(np.int64), 1), got)


def test_sort_nan_last_and_signed_zeros_tie(b200, backend):
    x = np.array([3.0, np.nan, -0.0, 0.0, -1.0, np.nan, 0.0, -0.0, np.inf, -np.inf], dtype=np.float32)
    tag = np.arange(10, dtype=np.int32)
    asc = run_backend(b200, backend, _sort_build(b200, np.float32, 0, False, 2), [x, tag])
    np.testing.assert_array_equal(asc[1], [9, 4, 2, 3, 6, 7, 0, 8, 1, 5])    # zeros of either sign tie; NaNs last, in input order
    desc = run_backend(b200, backend, _sort_build(b200, np.float32, 0, True, 2), [x, tag])
    np.testing.assert_array_equal(desc[1], [8, 0, 2, 3, 6, 7, 4, 9, 1, 5])


def test_sort_refusals(b200, backend):
    builder = backend.Builder("bad-sort")
    f = builder.Main()
    x = f.Parameter("x", _sh(b200, np.float32, 6))
    y = f.Parameter("y", _sh(b200, np.float32, 6))
    s = _sh(b200, np.float32)
    lt = closure(f, [s, s], lambda c, a, b: [c.LessThan(a, b)])
    with pytest.raises(b200.BackendError, match="at least one input"):                # ref function.go:567-569
        f.Sort(lt, 0, True)
    with pytest.raises(b200.BackendError, match="axis 1 out of range for rank 1"):    # ref function.go:599-601
        f.Sort(lt, 1, True, x)
    with pytest.raises(b200.BackendError, match="comparator must have 4 parameters, got 2"):   # ref function.go:605-608
        f.Sort(lt, 0, True, x, y)
    with pytest.raises(b200.BackendError, match="dtype"):                              # ref function.go:617-620
        f.Sort(closure(f, [_sh(b200, np.int32)] * 2, lambda c, a, b: [c.LessThan(a, b)]), 0, True, x)
    with pytest.raises(b200.BackendError, match="must be scalar"):                    # ref function.go:613-616
        f.Sort(closure(f, [_sh(b200, np.float32, 1)] * 2, lambda c, a, b: [c.Reshape(c.LessThan(a, b))]), 0, True, x)
    with pytest.raises(b200.BackendError, match="order by the first input"):          # this backend's stated limit
        f.Sort(closure(f, [s] * 4, lambda c, a, b, p, q: [c.LessThan(p, q)]), 0, True, x, y)
    builder.Finalize()


def test_capabilities_list_the_control_flow_ops(b200, backend):
    caps = backend.Capabilities()
    assert caps.Functions
    for op in ("Call", "While", "If", "Sort"):
        assert caps.Operations.get(op), op
