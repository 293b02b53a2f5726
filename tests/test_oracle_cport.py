"""Pins the C restatement (the timed CPU baseline) against the NumPy oracle."""
import ml_dtypes
import numpy as np

from oracle import cport
from oracle.oracle import OracleFunction, compare

BF16 = ml_dtypes.bfloat16


def test_softmax_causal_matches_numpy_oracle():
    rng = np.random.default_rng(0)
    x = (2.0 * rng.standard_normal((2, 3, 64, 64))).astype(np.float32)
    want = OracleFunction().FusedSoftmaxMasked(x, 1.0, True, None)
    ok, viol = compare(cport.softmax_f32(x, 1.0, True), want, 1e-5, 0.01)
    assert ok, viol
    want = OracleFunction().FusedSoftmax(x, 3)
    ok, viol = compare(cport.softmax_f32(x), want, 1e-5, 0.01)
    assert ok, viol


def test_norms_match_numpy_oracle():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((32, 512)).astype(np.float32).astype(BF16)
    g = (1 + 0.02 * rng.standard_normal(512)).astype(np.float32).astype(BF16)
    b = (0.1 * rng.standard_normal(512)).astype(np.float32).astype(BF16)
    f = OracleFunction()
    ok, viol = compare(cport.norm(x, g, b, 1e-6, False), f.FusedLayerNorm(x, [-1], 1e-6, g, b), 8e-3, 0.05)
    assert ok, viol
    ok, viol = compare(cport.norm(x, g, None, 1e-6, True), f.FusedRMSNorm(x, [-1], 1e-6, g), 8e-3, 0.05)
    assert ok, viol
    x32 = x.astype(np.float32)
    ok, viol = compare(cport.norm(x32, None, None, 1e-5, False), f.FusedLayerNorm(x32, [-1], 1e-5, None, None), 1e-5, 0.05)
    assert ok, viol


def test_gemm_forms_match_numpy_oracle():
    rng = np.random.default_rng(2)
    f = OracleFunction()
    for dt, rtol in ((np.float32, 1e-5), (BF16, 2e-2)):
        a = rng.standard_normal((2, 24, 40)).astype(np.float32).astype(dt)
        bt = rng.standard_normal((2, 40, 16)).astype(np.float32).astype(dt)
        ok, viol = compare(cport.gemm(a, bt, True, False), f.DotGeneral(a, [2], [0], bt, [1], [0]), rtol, 1.0)
        assert ok, viol
        at = np.ascontiguousarray(np.swapaxes(a, 1, 2))
        ok, viol = compare(cport.gemm(at, bt, False, False), f.DotGeneral(at, [1], [0], bt, [1], [0]), rtol, 1.0)
        assert ok, viol
