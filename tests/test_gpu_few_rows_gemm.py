"""16-bit matrix products with at most 64 rows (a decoding step's projections): the K-split kernel against the oracle.

K is cut into slices that different CTAs multiply; the slices' fp32 partial sums are added in slice order by the last
CTA to arrive (or met through a cluster's shared memory), then bias, activation and residual are applied.  Checked: every row count 1..16 and the edges of the 32- and 64-row forms, K that does not
divide evenly among the slices, one slice only, epilogue combinations, that the counters are left ready for the next
run (the same executable run many times), and that two runs give identical bits.
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import default_switches, rng_array, run_backend

pytestmark = pytest.mark.gpu
BF16 = ml_dtypes.bfloat16
RTOL = 2e-2


def _dense(f, x, w, b, act, res):
    y = f.FusedDense(x, w, b, act)
    return f.Add(y, res) if res is not None else y


def _check(b200, backend, M, N, K, dtype, bias, act, residual, seed=0, lead=None):
    rng = np.random.default_rng(seed)
    xs = (M, K) if lead is None else lead + (K,)
    x = rng_array(rng, xs, dtype, 1.0)
    w = rng_array(rng, (K, N), dtype, 1.0 / np.sqrt(K))
    inputs = [x, w]
    bi = ri = None
    if bias:
        bi = len(inputs); inputs.append(rng_array(rng, (N,), dtype))
    if residual:
        ri = len(inputs); inputs.append(rng_array(rng, xs[:-1] + (N,), dtype))
    build = lambda f, *p: _dense(f, p[0], p[1], p[bi] if bias else None, act, p[ri] if residual else None)
    (got,), plan = run_backend(b200, backend, build, inputs, describe=True)
    assert ("few-rows" in plan and plan.count("\n") == 1) or not default_switches(), plan
    # the yardstick: exact product rounded once (twice with a residual), as the fused epilogue does
    o = OracleFunction()
    want = o.FusedDense(x.astype(np.float32), w.astype(np.float32), inputs[bi].astype(np.float32) if bias else None, act).astype(dtype)
    if residual:
        want = (want.astype(np.float32) + inputs[ri].astype(np.float32)).astype(dtype)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol
    return got


@pytest.mark.parametrize("M", list(range(1, 17)) + [17, 24, 32, 33, 47, 64])
def test_every_row_count(b200, backend, M):
    _check(b200, backend, M, 768, 768, BF16, True, 0, False, seed=M)


@pytest.mark.parametrize("N,K", [(64, 16), (64, 48), (128, 8192), (768, 3072), (2304, 768), (3072, 768), (4096, 11008), (1024, 1040), (320, 80),
                                 (32000 // 64 * 64, 512)])
def test_shapes(b200, backend, N, K):
    _check(b200, backend, 16, N, K, BF16, False, 0, False, seed=N + K)


@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("act", [0, 1, 2, 3, 4], ids=["none", "gelu", "relu", "silu", "tanh"])
@pytest.mark.parametrize("residual", [False, True])
def test_epilogues(b200, backend, bias, act, residual):
    _check(b200, backend, 7, 512, 1024, BF16, bias, act, residual, seed=17)


@pytest.mark.parametrize("M", [32, 64])
@pytest.mark.parametrize("N,K", [(768, 3072), (3072, 768), (4096, 6144), (4096, 6400), (1024, 11008), (64, 16)])
def test_more_rows(b200, backend, M, N, K):
    # 6144 is the longest K whose slices fit one cluster at 64 rows; 6400 and 11008 go through global memory
    _check(b200, backend, M, N, K, BF16, True, 1, True, seed=M + N + K)


def test_f16_and_leading_dims(b200, backend):
    _check(b200, backend, 12, 768, 3072, np.float16, True, 1, True, seed=3)
    _check(b200, backend, 16, 768, 768, BF16, True, 0, True, seed=4, lead=(16, 1))
    _check(b200, backend, 6, 256, 256, np.float16, False, 0, False, seed=5, lead=(2, 3))


def test_repeated_runs_are_identical_and_leave_the_counters_ready(b200, backend):
    rng = np.random.default_rng(8)
    x, w, b = rng_array(rng, (16, 3072), BF16), rng_array(rng, (3072, 768), BF16, 0.02), rng_array(rng, (768,), BF16)
    builder = backend.Builder("few_rows")
    f = builder.Main()
    params = [f.Parameter(f"p{i}", b200.Shape(b200.dtypes.from_numpy(a.dtype), a.shape)) for i, a in enumerate((x, w, b))]
    f.Return([f.FusedDense(params[0], params[1], params[2], 1)], None)
    exe = builder.Compile()
    bufs = [backend.FromNumpy(a) for a in (x, w, b)]
    first = None
    for run in range(12):   # direct launches first, then the recorded plan
        (r,) = exe.Execute(bufs, None, 0)
        got = backend.ToNumpy(r)
        backend.BufferFinalize(r)
        if first is None:
            first = got
        else:
            np.testing.assert_array_equal(got.view(np.uint16), first.view(np.uint16))
    want = OracleFunction().FusedDense(x.astype(np.float32), w.astype(np.float32), b.astype(np.float32), 1).astype(BF16)
    ok, viol = compare(first, want, RTOL, 1.0)
    assert ok, viol
    exe.Finalize()
    builder.Finalize()


def test_two_products_in_one_plan_have_counters_of_their_own(b200, backend):
    rng = np.random.default_rng(9)
    x, w1, w2 = rng_array(rng, (4, 256), BF16), rng_array(rng, (256, 1024), BF16, 0.06), rng_array(rng, (1024, 256), BF16, 0.03)
    build = lambda f, xx, a, b: f.FusedDense(f.FusedDense(xx, a, None, 2), b, None, 0)
    (got,), plan = run_backend(b200, backend, build, [x, w1, w2], describe=True)
    assert (plan.count("few-rows") == 2) or not default_switches(), plan
    o = OracleFunction()
    h = o.FusedDense(x.astype(np.float32), w1.astype(np.float32), None, 2).astype(BF16)
    want = o.FusedDense(h.astype(np.float32), w2.astype(np.float32), None, 0).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_other_shapes_keep_their_kernels(b200, backend):
    rng = np.random.default_rng(10)
    for M, N, K in [(65, 768, 768), (16, 100, 64), (16, 64, 24)]:
        x, w = rng_array(rng, (M, K), BF16), rng_array(rng, (K, N), BF16, 0.1)
        (got,), plan = run_backend(b200, backend, lambda f, a, b: f.FusedDense(a, b, None, 0), [x, w], describe=True)
        assert ("few-rows" not in plan) or not default_switches(), plan
        want = OracleFunction().FusedDense(x.astype(np.float32), w.astype(np.float32), None, 0).astype(BF16)
        ok, viol = compare(got, want, RTOL, 1.0)
        assert ok, viol


@pytest.mark.parametrize("M", [1, 16, 40])
@pytest.mark.parametrize("N,K", [(64, 64), (100, 64), (777, 768), (4096, 2048), (50257, 768), (32768, 256), (1000, 16), (130, 8192)])
def test_weights_stored_n_major_and_a_ragged_n(b200, backend, M, N, K):
    # an LM head tied to the embedding table: W is [N, K] and N is whatever the vocabulary is
    rng = np.random.default_rng(M + N + K)
    x = rng_array(rng, (M, K), BF16)
    w = rng_array(rng, (N, K), BF16, 1.0 / np.sqrt(K))
    (got,), plan = run_backend(b200, backend, lambda f, a, b: f.DotGeneral(a, [1], [], b, [1], []), [x, w], describe=True)
    # (beyond 32768 columns the tensor-core tile fills the GPU and keeps the product)
    assert (("few-rows" in plan) == (N <= 32768) and "b:NK" in plan and plan.count("\n") == 1) or not default_switches(), plan
    want = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_n_major_weights_in_f16(b200, backend):
    rng = np.random.default_rng(77)
    x, w = rng_array(rng, (9, 512), np.float16), rng_array(rng, (333, 512), np.float16, 0.05)
    (got,), plan = run_backend(b200, backend, lambda f, a, b: f.DotGeneral(a, [1], [], b, [1], []), [x, w], describe=True)
    assert ("few-rows" in plan) or not default_switches(), plan
    want = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


@pytest.mark.parametrize("M", [1, 16, 17, 32])
@pytest.mark.parametrize("N,K,act", [(512, 256, 3), (8192, 2048, 3), (1024, 4096, 1), (64, 16, 0)])
def test_gated_pair_of_products_in_one_launch(b200, backend, M, N, K, act):
    # act(x W1) * (x W2): one launch with two weights, bit for bit the two-launch result (both products rounded, multiplied,
    # rounded again)
    rng = np.random.default_rng(M + N + K)
    x = rng_array(rng, (M, K), BF16)
    w1, w2 = rng_array(rng, (K, N), BF16, 1.0 / np.sqrt(K)), rng_array(rng, (K, N), BF16, 1.0 / np.sqrt(K))
    build = lambda f, a, b, c: f.Mul(f.FusedDense(a, b, None, act), f.FusedDense(a, c, None, 0))
    (got,), plan = run_backend(b200, backend, build, [x, w1, w2], describe=True)
    assert ("*second-product" in plan and "few-rows" in plan and plan.count("\n") == 1) or not default_switches(), plan
    o = OracleFunction()
    g = o.FusedDense(x.astype(np.float32), w1.astype(np.float32), None, act).astype(BF16)
    u = o.FusedDense(x.astype(np.float32), w2.astype(np.float32), None, 0).astype(BF16)
    want = (g.astype(np.float32) * u.astype(np.float32)).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_gated_pair_is_left_alone_when_the_second_product_is_used_elsewhere(b200, backend):
    rng = np.random.default_rng(31)
    x, w1, w2 = rng_array(rng, (8, 256), BF16), rng_array(rng, (256, 512), BF16, 0.06), rng_array(rng, (256, 512), BF16, 0.06)

    def build(f, a, b, c):
        up = f.FusedDense(a, c, None, 0)
        return [f.Mul(f.FusedDense(a, b, None, 3), up), up]
    got, plan = run_backend(b200, backend, build, [x, w1, w2], describe=True)
    assert ("*second-product" not in plan) or not default_switches(), plan
    o = OracleFunction()
    g = o.FusedDense(x.astype(np.float32), w1.astype(np.float32), None, 3).astype(BF16)
    u = o.FusedDense(x.astype(np.float32), w2.astype(np.float32), None, 0).astype(BF16)
    ok, viol = compare(got[0], (g.astype(np.float32) * u.astype(np.float32)).astype(BF16), RTOL, 1.0)
    assert ok, viol
    ok, viol = compare(got[1], u, RTOL, 1.0)
    assert ok, viol


def _rms(x, gamma, eps):
    v = x.astype(np.float64)
    return (v / np.sqrt((v * v).mean(axis=-1, keepdims=True) + eps) * gamma.astype(np.float64))


@pytest.mark.parametrize("M", [1, 7, 16, 32])
@pytest.mark.parametrize("N,K", [(512, 256), (3072, 2048), (64, 16), (768, 1040)])
def test_rms_norm_applied_inside_the_product(b200, backend, M, N, K):
    # RMSNorm(x) W as one launch: gamma on X's fragments, the rows' sums of squares from the same fragments, rstd on the sums
    rng = np.random.default_rng(M * 7 + N + K)
    x = (rng_array(rng, (M, K), BF16).astype(np.float32) * 3 + 0.5).astype(BF16)
    gamma = (1.0 + 0.3 * rng.standard_normal(K)).astype(np.float32).astype(BF16)
    w, bias = rng_array(rng, (K, N), BF16, 1.0 / np.sqrt(K)), rng_array(rng, (N,), BF16)
    build = lambda f, a, gm, b, c: f.FusedDense(f.FusedRMSNorm(a, [-1], 1e-5, gm), b, c, 1)
    (got,), plan = run_backend(b200, backend, build, [x, gamma, w, bias], describe=True)
    assert ("of-rms-norm" in plan and "few-rows" in plan and "rms_norm[" not in plan and plan.count("\n") == 1) or not default_switches(), plan
    h = _rms(x, gamma, 1e-5)
    want = OracleFunction().FusedDense(h.astype(np.float32), w.astype(np.float32), bias.astype(np.float32), 1).astype(BF16)
    ok, viol = compare(got, want, RTOL, 1.0)
    assert ok, viol


def test_rms_norm_inside_a_gated_pair_and_f16(b200, backend):
    rng = np.random.default_rng(91)
    for dt in (BF16, np.float16):
        x = rng_array(rng, (5, 512), dt)
        gamma = (1.0 + 0.2 * rng.standard_normal(512)).astype(np.float32).astype(dt)
        w1, w2 = rng_array(rng, (512, 1024), dt, 0.05), rng_array(rng, (512, 1024), dt, 0.05)

        def build(f, a, gm, b, c):
            h = f.FusedRMSNorm(a, [-1], 1e-6, gm)
            return f.Mul(f.FusedDense(h, b, None, 3), f.FusedDense(h, c, None, 0))
        (got,), plan = run_backend(b200, backend, build, [x, gamma, w1, w2], describe=True)
        assert ("of-rms-norm" in plan and "*second-product" in plan and plan.count("\n") == 1) or not default_switches(), plan
        h = _rms(x, gamma, 1e-6).astype(np.float32)
        o = OracleFunction()
        g = o.FusedDense(h, w1.astype(np.float32), None, 3).astype(dt)
        u = o.FusedDense(h, w2.astype(np.float32), None, 0).astype(dt)
        want = (g.astype(np.float32) * u.astype(np.float32)).astype(dt)
        ok, viol = compare(got, want, RTOL, 1.0)
        assert ok, viol


def test_rms_norm_with_another_user_keeps_its_own_launch(b200, backend):
    rng = np.random.default_rng(92)
    x, gamma, w = rng_array(rng, (8, 256), BF16), np.ones(256, np.float32).astype(BF16), rng_array(rng, (256, 512), BF16, 0.06)

    def build(f, a, gm, b):
        h = f.FusedRMSNorm(a, [-1], 1e-5, gm)
        return [f.FusedDense(h, b, None, 0), h]
    got, plan = run_backend(b200, backend, build, [x, gamma, w], describe=True)
    assert ("of-rms-norm" not in plan and "rms_norm[" in plan) or not default_switches(), plan
    h = _rms(x, gamma, 1e-5).astype(np.float32).astype(BF16)
    ok, viol = compare(got[1], h, RTOL, 1.0)
    assert ok, viol
    want = OracleFunction().FusedDense(h.astype(np.float32), w.astype(np.float32), None, 0).astype(BF16)
    ok, viol = compare(got[0], want, RTOL, 1.0)
    assert ok, viol
