"""Parity at the benchmarked sizes: the code paths bench.py times, compared with the CPU oracle through the C ABI.

The small-shape parity tests never reach the persistent row loop of the norm kernel (rows >> 2 * SMs * row groups),
the hundreds of ring wrap-arounds of a K = 8192 contraction, the fp32 three-plane split at K = 8192, or attention
over 2048 keys.  These do.  Whole outputs are compared where the float64 oracle finishes in seconds (evaluated in
row chunks to bound host memory); otherwise a seeded sample of rows.

Tolerances: rel 1e-5 fp32, rel 2e-2 for 16-bit contractions, half-ulp-scale 8e-3 for 16-bit row norms; every
comparison adds the norm-relative term of oracle.compare (atol_scale * rtol * rms(expected)).
"""
import ml_dtypes
import numpy as np
import pytest

from oracle.oracle import OracleFunction, compare
from tests.util import run_backend

pytestmark = pytest.mark.gpu

BF16 = ml_dtypes.bfloat16
EPS = 1e-6


def _normal(rng, shape, dtype, scale=1.0):
    """N(0, scale^2) generated in float32 chunks (bounded temporaries), rounded to dtype."""
    n = int(np.prod(shape))
    out = np.empty(n, dtype=dtype)
    step = 1 << 24
    for lo in range(0, n, step):
        v = rng.standard_normal(min(step, n - lo), dtype=np.float32)
        if scale != 1.0:
            v *= scale
        out[lo:lo + v.size] = v.astype(dtype)
    return out.reshape(shape)


def _check_rows(got, want_fn, row_chunks, rtol, atol_scale, what):
    """Compares got[rows] with want_fn(rows) chunk by chunk; want_fn gets a slice or an index array."""
    for rows in row_chunks:
        ok, viol = compare(got[rows], want_fn(rows), rtol, atol_scale)
        assert ok, f"{what}: rows {rows if isinstance(rows, slice) else rows[:4]} differ from the oracle (worst violation {viol:.3e})"


# ------------------------------------------------------------------------------ norms ---
@pytest.mark.parametrize("rows,cols,dtype,rtol", [(16384, 4096, BF16, 8e-3), (5000, 4096, np.float32, 1e-5), (16384, 768, BF16, 8e-3),
                                                  (131072 // 8, 2048, BF16, 8e-3)],
                         ids=["config-bf16-16384x4096", "f32-5000x4096", "gpt2-bf16-16384x768", "llama-bf16-16384x2048"])
def test_norms_through_the_persistent_row_loop(b200, backend, rows, cols, dtype, rtol):
    rng = np.random.default_rng(0)
    x = _normal(rng, (rows, cols), dtype)
    g = (1.0 + 0.02 * rng.standard_normal(cols)).astype(np.float32).astype(dtype)
    b = (0.1 * rng.standard_normal(cols)).astype(np.float32).astype(dtype)
    rms, ln = run_backend(b200, backend, lambda f, a, gg, bb: (f.FusedRMSNorm(a, [-1], EPS, gg), f.FusedLayerNorm(a, [-1], EPS, gg, bb)),
                          [x, g, b])
    orc = OracleFunction()
    chunks = [slice(lo, min(rows, lo + 2048)) for lo in range(0, rows, 2048)]
    _check_rows(rms, lambda r: orc.FusedRMSNorm(x[r], [-1], EPS, g), chunks, rtol, 0.05, "RMSNorm")
    _check_rows(ln, lambda r: orc.FusedLayerNorm(x[r], [-1], EPS, g, b), chunks, rtol, 0.05, "LayerNorm")


def test_layer_norm_fp32_row_with_an_outlier_first_element(b200, backend):
    # a shifted one-pass variance that centres on the first element cancels catastrophically here; the reference is
    # two-pass (ref mpsgraph/gomlx/function.go:2430-2558)
    rng = np.random.default_rng(1)
    x = (0.1 * rng.standard_normal((300, 4096))).astype(np.float32)
    x[:, 0] = 1e4
    x[7, 0] = -1e4
    x[11] += 500.0   # large common offset, small spread
    g = (1.0 + 0.02 * rng.standard_normal(4096)).astype(np.float32)
    b = (0.1 * rng.standard_normal(4096)).astype(np.float32)
    (got,) = run_backend(b200, backend, lambda f, a, gg, bb: f.FusedLayerNorm(a, [-1], 1e-5, gg, bb), [x, g, b])
    want = OracleFunction().FusedLayerNorm(x, [-1], 1e-5, g, b)
    ok, viol = compare(got, want, 1e-5, 0.05)
    assert ok, viol
    for cols in (768, 100, 20000):   # the other row-group widths
        xs = (0.1 * rng.standard_normal((40, cols))).astype(np.float32)
        xs[:, 0] = 1e4
        (got,) = run_backend(b200, backend, lambda f, a: f.FusedLayerNorm(a, [-1], 1e-5, None, None), [xs])
        ok, viol = compare(got, OracleFunction().FusedLayerNorm(xs, [-1], 1e-5, None, None), 1e-5, 0.05)
        assert ok, (cols, viol)


# ---------------------------------------------------------------------------- softmax ---
def test_causal_softmax_fp32_quarter_config_whole_output(b200, backend):
    rng = np.random.default_rng(0)
    x = _normal(rng, (4, 16, 1024, 1024), np.float32, 2.0)
    (got,) = run_backend(b200, backend, lambda f, a: f.FusedSoftmaxMasked(a, 1.0, True, None), [x])
    orc = OracleFunction()
    for bi in range(4):
        for h0 in range(0, 16, 4):
            ok, viol = compare(got[bi, h0:h0 + 4], orc.FusedSoftmaxMasked(x[bi, h0:h0 + 4], 1.0, True, None), 1e-5, 0.01)
            assert ok, (bi, h0, viol)
    # size-independent properties: rows sum to 1, nothing right of the diagonal
    np.testing.assert_allclose(got.sum(-1, dtype=np.float64), 1.0, rtol=1e-5)
    assert not np.triu(got[3, 15], 1).any()


@pytest.mark.parametrize("causal", [True, False], ids=["causal", "plain"])
def test_softmax_fp32_full_config_sampled_rows(b200, backend, causal):
    rng = np.random.default_rng(0)
    shape = (32, 16, 1024, 1024)
    x = _normal(rng, shape, np.float32, 2.0)
    (got,) = run_backend(b200, backend, lambda f, a: f.FusedSoftmaxMasked(a, 1.0, causal, None), [x])
    orc = OracleFunction()
    pick = np.random.default_rng(5)
    planes = sorted({(int(pick.integers(32)), int(pick.integers(16))) for _ in range(12)} | {(0, 0), (31, 15)})
    for (bi, h) in planes:   # whole [1024, 1024] planes: the mask needs the row's position inside its plane
        ok, viol = compare(got[bi, h], orc.FusedSoftmaxMasked(x[bi, h], 1.0, causal, None), 1e-5, 0.01)
        assert ok, (bi, h, viol)
    sums = got.reshape(-1, 1024).sum(-1, dtype=np.float64)
    np.testing.assert_allclose(sums, 1.0, rtol=1e-5)


# ------------------------------------------------------------------------- DotGeneral ---
@pytest.mark.parametrize("dtype,rtol", [(BF16, 2e-2), (np.float32, 1e-5)], ids=["bf16", "f32"])
@pytest.mark.parametrize("form", ["BMK_BKN", "BKM_BKN"])
@pytest.mark.parametrize("n", [4096, 8192])
def test_dot_general_config_sizes_sampled_rows(b200, backend, n, form, dtype, rtol):
    rng = np.random.default_rng(n)
    a = _normal(rng, (8, n, n), dtype)
    b = _normal(rng, (8, n, n), dtype)
    lc = [2] if form == "BMK_BKN" else [1]
    (got,) = run_backend(b200, backend, lambda f, x, y: f.DotGeneral(x, lc, [0], y, [1], [0]), [a, b])
    assert got.shape == (8, n, n) and got.dtype == np.dtype(dtype)
    pick = np.random.default_rng(9)
    for bi in range(8):
        rows = np.sort(pick.choice(n, size=64, replace=False))
        rows[0], rows[-1] = 0, n - 1
        lhs = a[bi, rows, :] if form == "BMK_BKN" else a[bi][:, rows].T
        want = (lhs.astype(np.float64) @ b[bi].astype(np.float64)).astype(dtype)
        ok, viol = compare(got[bi, rows], want, rtol, 1.0)
        assert ok, (bi, viol)


@pytest.mark.parametrize("m,n,k,batch", [(1024, 1001, 768, 1), (1024, 50257, 64, 1), (2048, 1003, 1024, 2), (1024, 254, 256, 3), (3072, 777, 128, 1),
                                          (1032, 1006, 512, 1), (1024, 2044, 2048, 2)],
                         ids=["single-q1", "vocab-q1", "pair-q3-batched", "q6-narrower-than-a-tile", "q1-three-tiles-per-class", "m-ragged-q6",
                              "pair-q4"])
@pytest.mark.parametrize("dtype", [BF16, np.float16], ids=["bf16", "f16"])
def test_dot_general_rows_not_a_multiple_of_the_vector_width(b200, backend, m, n, k, batch, dtype):
    # a dense 16-bit result with N % 8 != 0: the tensor-core kernel cuts the rows into 8 classes (row mod 8) and shifts each
    # class's column window so that every store is an aligned vector; the first and last vector of a row go out by element
    rng = np.random.default_rng(m + n)
    a = _normal(rng, (batch, m, k), dtype)
    w = _normal(rng, (batch, n, k), dtype)   # [B, N, K]: what x @ table^T contracts
    (got,), plan = run_backend(b200, backend, lambda f, x, y: f.DotGeneral(x, [2], [0], y, [2], [0]), [a, w], describe=True)
    assert "ragged-rows" in plan and "pack" not in plan, plan
    assert got.shape == (batch, m, n)
    for bi in range(batch):
        want = (a[bi].astype(np.float64) @ w[bi].astype(np.float64).T).astype(dtype)
        ok, viol = compare(got[bi], want, 2e-2, 1.0)
        assert ok, (bi, viol)


# -------------------------------------------------------------------------- attention ---
@pytest.mark.parametrize("causal", [True, False], ids=["causal", "full"])
def test_fused_attention_llama_shape_sampled_heads(b200, backend, causal):
    rng = np.random.default_rng(2)
    B, S, H, HKV, D = 1, 2048, 32, 8, 64
    q, k, v = (_normal(rng, (B, S, h, D), BF16) for h in (H, HKV, HKV))
    (got,), plan = run_backend(b200, backend, lambda f, qq, kk, vv: f.FusedScaledDotProductAttention(qq, kk, vv, None, H, HKV, 1, 0.125, causal),
                               [q, k, v], describe=True)
    assert plan.startswith("attention["), plan
    orc = OracleFunction()
    for h in (0, 5, 18, 31):
        kv = h // (H // HKV)   # each KV head serves H/HKV consecutive query heads (ref function.go:2910-2955)
        qh, kh, vh = q[:, :, h:h + 1], k[:, :, kv:kv + 1], v[:, :, kv:kv + 1]
        # (1) the kernel's own arithmetic: fp32 scores, one rounding at the end
        want32 = orc.FusedScaledDotProductAttention(qh.astype(np.float32), kh.astype(np.float32), vh.astype(np.float32), None, 1, 1, 1, 0.125,
                                                    causal).astype(BF16)
        ok, viol = compare(got[:, :, h:h + 1], want32, 2e-2, 1.0)
        assert ok, (h, "fp32-score oracle", viol)
        # (2) the reference's decomposition unchanged (ref function.go:2669-2907): scores, probabilities and output each
        # rounded to bf16.  Rounding a score of magnitude 16..32 to bf16 moves it by up to 0.06, i.e. the weight of a
        # dominant key by up to 0.8 %, which the fused kernel (fp32 scores) does not reproduce element by element.  So:
        # the two agree to 2e-2 in norm, and the fused result is at least as close to the exact (float64) attention as
        # the decomposition is.
        want16 = orc.FusedScaledDotProductAttention(qh, kh, vh, None, 1, 1, 1, 0.125, causal).astype(np.float64)
        exact = orc.FusedScaledDotProductAttention(qh.astype(np.float64), kh.astype(np.float64), vh.astype(np.float64), None, 1, 1, 1, 0.125, causal)
        g64 = got[:, :, h:h + 1].astype(np.float64)
        rms = lambda t: float(np.sqrt(np.mean(t * t)))
        assert rms(g64 - want16) <= 2e-2 * rms(want16), (h, "bf16 decomposition oracle, norm", rms(g64 - want16) / rms(want16))
        assert rms(g64 - exact) <= rms(want16 - exact) * 1.05 + 1e-6, (h, rms(g64 - exact), rms(want16 - exact))


# ----------------------------------------------------------------- transformer forwards ---
def test_gpt2_forward_real_width_two_layers(b200, backend):
    # GPT-2 small's real widths (d 768, 12 heads, MLP 3072, S 1024, V 50257 -- the ragged LM head) at 2 layers, batch 1
    import go_darwinml_b200.workloads as w
    c = w.GPT2Config(layers=2, batch=1)
    inputs = w.gpt2_init(c, seed=3, float_dtype=BF16)
    code = int(b200.dtypes.BFloat16)
    (got,) = run_backend(b200, backend, lambda f, *p: w.gpt2_forward(f, c, code, *p), inputs)
    want = w.gpt2_forward(OracleFunction(), c, code, *inputs)
    assert got.shape == (1, 1024, 50257)
    ok, viol = compare(got, want, 5e-2, 1.0)   # bf16 end to end through 2 blocks: every op rounds to 8 bits on both sides
    assert ok, viol
