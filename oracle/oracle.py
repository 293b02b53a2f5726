"""CPU oracle: a NumPy restatement of the reference's op semantics.

TEST INFRASTRUCTURE ONLY.  Nothing in the product imports this module; only
tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference
legs may, and only as the checker or the timed CPU baseline.

The reference (gomlx/go-darwinml) contains no arithmetic of its own: every op
is one call into Apple's closed MPSGraph framework (mpsgraph/gomlx/internal/
bridge/bridge.m), and its shape rules come from the third-party module
github.com/gomlx/gomlx v0.26.1-0.20260223064152-358aaf0bc270 (package
backends/shapeinference, pinned in mpsgraph/gomlx/go.mod:6), which is not in
the reference tree.  Neither can be built or run outside macOS.  This file
therefore restates, op by op, what the reference's Go lowering asks the
framework to compute, citing the call site it follows, and is pinned against
every known-answer vector in the reference's own tests (tests/golden/).

Behaviour that no reference test pins is DEFINED here (and marked "unpinned"):
RMSNorm (absent from the reference), fp32 accumulation with one final rounding
for bf16/f16 contractions and norms, IEEE NaN for a fully masked softmax row,
lowest-index ties and NaN-as-extreme for ArgMin/ArgMax, clamped out-of-range
Gather indices, C-style truncated Rem, saturating float->int conversion.

Precision policy: float ops are evaluated in float64 from the exact input bits
and rounded ONCE to the op's dtype; a fused op (softmax, LayerNorm, GELU,
Dense, SDPA) rounds once at its end.  Integer ops wrap like two's complement.

`OracleFunction` has the method names of the reference's Function type
(mpsgraph/gomlx/function.go) so one graph-building routine can drive both the
backend under test and this oracle.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np

try:
    import ml_dtypes

    bfloat16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    bfloat16 = None

# dtype codes shared with the C ABI (ref bridge.h:23-37)
BOOL, I8, I16, I32, I64, F16, BF16, F32, F64, U8, U16, U32, U64 = range(13)
NP = {BOOL: np.dtype(np.bool_), I8: np.dtype(np.int8), I16: np.dtype(np.int16), I32: np.dtype(np.int32),
      I64: np.dtype(np.int64), F16: np.dtype(np.float16), BF16: bfloat16, F32: np.dtype(np.float32),
      F64: np.dtype(np.float64), U8: np.dtype(np.uint8), U16: np.dtype(np.uint16), U32: np.dtype(np.uint32),
      U64: np.dtype(np.uint64)}

ACT_NONE, ACT_GELU, ACT_RELU, ACT_SILU, ACT_TANH = range(5)
LAYOUT_BHSD, LAYOUT_BSHD = 0, 1


def is_float(dt) -> bool:
    dt = np.dtype(dt)
    return dt.kind == "f" or dt == bfloat16


def _f64(x):
    return np.asarray(x).astype(np.float64)


def _round(x64, dt):
    """One rounding from float64 to the storage dtype."""
    with np.errstate(over="ignore", invalid="ignore"):
        return np.asarray(x64).astype(dt)


def _erf(x):
    return np.vectorize(math.erf, otypes=[np.float64])(x)


def _dtype_of(shape_or_dtype):
    dt = getattr(shape_or_dtype, "DType", shape_or_dtype)
    if isinstance(dt, (int, np.integer)) and not isinstance(dt, np.dtype):
        return NP[int(dt)]
    return np.dtype(dt)


def _dims_of(shape):
    return list(getattr(shape, "Dimensions", shape))


class OracleError(ValueError):
    pass


class OracleFunction:
    """Eager evaluation: every method takes and returns numpy arrays."""

    # ---- leaves -------------------------------------------------------------
    def Constant(self, flat, *dims):
        return np.asarray(flat).reshape(dims)

    def Iota(self, shape, iota_axis: int):
        # value = coordinate along the axis, any dtype (ref function.go:1127-1135; bridge.m:237-259)
        dt, dims = _dtype_of(shape), _dims_of(shape)
        ax = iota_axis + len(dims) if iota_axis < 0 else iota_axis
        view = [1] * len(dims)
        view[ax] = dims[ax]
        ramp = np.arange(dims[ax], dtype=np.int64).reshape(view)
        return np.broadcast_to(ramp, dims).astype(dt)

    # ---- unary (ref function.go:658-790; bridge.m:265-354) --------------------
    def _funary(self, x, fn):
        if not is_float(x.dtype):
            raise OracleError("float operand required")
        with np.errstate(all="ignore"):
            return _round(fn(_f64(x)), x.dtype)

    def Abs(self, x):
        return np.abs(x) if is_float(x.dtype) else np.abs(x.astype(np.int64)).astype(x.dtype) if x.dtype.kind == "i" else x.copy()

    def Neg(self, x):
        with np.errstate(over="ignore"):
            return (-x.astype(np.float64)).astype(x.dtype) if is_float(x.dtype) else (0 - x).astype(x.dtype)

    def Sqrt(self, x): return self._funary(x, np.sqrt)
    def Rsqrt(self, x): return self._funary(x, lambda v: 1.0 / np.sqrt(v))
    def Exp(self, x): return self._funary(x, np.exp)
    def Expm1(self, x): return self._funary(x, np.expm1)   # the reference builds exp(x)-1 (bridge.m:315-333); tests use tolerances
    def Log(self, x): return self._funary(x, np.log)
    def Log1p(self, x): return self._funary(x, np.log1p)
    def Sin(self, x): return self._funary(x, np.sin)
    def Cos(self, x): return self._funary(x, np.cos)
    def Tanh(self, x): return self._funary(x, np.tanh)
    def Logistic(self, x): return self._funary(x, lambda v: 1.0 / (1.0 + np.exp(-v)))
    def Erf(self, x): return self._funary(x, _erf)
    def Floor(self, x): return self._funary(x, np.floor)
    def Ceil(self, x): return self._funary(x, np.ceil)
    def Round(self, x): return self._funary(x, np.rint)   # ties to even (ref bridge.m:293)

    def Sign(self, x):
        if is_float(x.dtype):
            v = _f64(x)
            return _round(np.where(v > 0, 1.0, np.where(v < 0, -1.0, v)), x.dtype)
        return np.sign(x).astype(x.dtype)

    def LogicalNot(self, x): return np.logical_not(x)
    def BitwiseNot(self, x): return np.logical_not(x) if x.dtype == np.bool_ else np.invert(x)
    def IsFinite(self, x): return np.isfinite(_f64(x)) if is_float(x.dtype) else np.ones(x.shape, np.bool_)
    def IsNaN(self, x): return np.isnan(_f64(x)) if is_float(x.dtype) else np.zeros(x.shape, np.bool_)
    def Identity(self, x): return x.copy()

    # ---- binary (ref function.go:792-905; bridge.m:360-401) -------------------
    def _check2(self, a, b):
        if a.dtype != b.dtype:
            raise OracleError(f"operand dtypes differ ({a.dtype} vs {b.dtype})")
        np.broadcast_shapes(a.shape, b.shape)

    def _fbinary(self, a, b, fn):
        with np.errstate(all="ignore"):
            return _round(fn(_f64(a), _f64(b)), a.dtype)

    def _arith(self, a, b, ffn, ifn):
        self._check2(a, b)
        if is_float(a.dtype):
            return self._fbinary(a, b, ffn)
        with np.errstate(all="ignore"):
            return ifn(a, b).astype(a.dtype)

    def Add(self, a, b): return self._arith(a, b, np.add, np.add)
    def Sub(self, a, b): return self._arith(a, b, np.subtract, np.subtract)
    def Mul(self, a, b): return self._arith(a, b, np.multiply, np.multiply)

    @staticmethod
    def _int_div(a, b):
        big_a, big_b = a.astype(object), b.astype(object)
        out = np.empty(np.broadcast_shapes(a.shape, b.shape), dtype=object)
        for idx in np.ndindex(out.shape):
            x, y = int(np.broadcast_to(big_a, out.shape)[idx]), int(np.broadcast_to(big_b, out.shape)[idx])
            out[idx] = -1 if y == 0 else int(math.copysign(abs(x) // abs(y), x * y)) if x * y != 0 else 0
        bits = a.dtype.itemsize * 8
        return (np.vectorize(lambda v: v & ((1 << bits) - 1), otypes=[object])(out)).astype(np.uint64).astype(a.dtype)

    @staticmethod
    def _int_rem(a, b):
        out = np.empty(np.broadcast_shapes(a.shape, b.shape), dtype=object)
        A, B = np.broadcast_to(a, out.shape), np.broadcast_to(b, out.shape)
        for idx in np.ndindex(out.shape):
            x, y = int(A[idx]), int(B[idx])
            out[idx] = x if y == 0 else int(math.fmod(x, y)) if abs(x) < 2**52 and abs(y) < 2**52 else x - y * int(math.copysign(abs(x) // abs(y), x * y))
        bits = a.dtype.itemsize * 8
        return (np.vectorize(lambda v: v & ((1 << bits) - 1), otypes=[object])(out)).astype(np.uint64).astype(a.dtype)

    def Div(self, a, b):
        self._check2(a, b)
        return self._fbinary(a, b, np.divide) if is_float(a.dtype) else self._int_div(a, b)

    def Rem(self, a, b):
        # unpinned: the reference's two backends disagree for negative operands; defined as C fmod / truncated remainder
        self._check2(a, b)
        return self._fbinary(a, b, np.fmod) if is_float(a.dtype) else self._int_rem(a, b)

    def Pow(self, a, b): return self._arith(a, b, np.power, lambda x, y: np.power(x.astype(np.int64), np.maximum(y.astype(np.int64), 0)))

    def Max(self, a, b): return self._arith(a, b, np.maximum, np.maximum)   # NaN-propagating
    def Min(self, a, b): return self._arith(a, b, np.minimum, np.minimum)
    def Atan2(self, a, b): return self._arith(a, b, np.arctan2, None)
    def LogicalAnd(self, a, b): return np.logical_and(a, b)
    def LogicalOr(self, a, b): return np.logical_or(a, b)
    def LogicalXor(self, a, b): return np.logical_xor(a, b)
    def BitwiseAnd(self, a, b): return np.bitwise_and(a, b)
    def BitwiseOr(self, a, b): return np.bitwise_or(a, b)
    def BitwiseXor(self, a, b): return np.bitwise_xor(a, b)

    def _shift(self, a, b, fn):
        self._check2(a, b)
        bits = a.dtype.itemsize * 8
        out = np.empty(np.broadcast_shapes(a.shape, b.shape), dtype=a.dtype)
        A, B = np.broadcast_to(a, out.shape), np.broadcast_to(b, out.shape)
        for idx in np.ndindex(out.shape):
            x, s = int(A[idx]), int(B[idx]) & ((1 << bits) - 1)
            out[idx] = np.array(fn(x, s, bits) & ((1 << bits) - 1)).astype(np.uint64).astype(a.dtype)
        return out

    def ShiftLeft(self, a, b):
        return self._shift(a, b, lambda x, s, bits: 0 if s >= bits else (x << s))

    def ShiftRightArithmetic(self, a, b):
        return self._shift(a, b, lambda x, s, bits: (-1 if x < 0 else 0) if s >= bits else (x >> s))

    def ShiftRightLogical(self, a, b):
        return self._shift(a, b, lambda x, s, bits: 0 if s >= bits else ((x & ((1 << bits) - 1)) >> s))

    # ---- comparisons -> Bool (ref function.go:907-963) ------------------------
    def _cmp(self, a, b, fn):
        self._check2(a, b)
        if is_float(a.dtype):
            return fn(_f64(a), _f64(b))
        return fn(a, b)

    def Equal(self, a, b): return self._cmp(a, b, np.equal)
    def NotEqual(self, a, b): return self._cmp(a, b, np.not_equal)
    def LessThan(self, a, b): return self._cmp(a, b, np.less)
    def LessOrEqual(self, a, b): return self._cmp(a, b, np.less_equal)
    def GreaterThan(self, a, b): return self._cmp(a, b, np.greater)
    def GreaterOrEqual(self, a, b): return self._cmp(a, b, np.greater_equal)

    # ---- shape ops (ref function.go:969-1125, 1533-1565) -----------------------
    def Reshape(self, x, *dims): return x.reshape(dims)
    def Transpose(self, x, *perm): return np.ascontiguousarray(np.transpose(x, perm))

    def ConvertDType(self, x, dtype):
        dt = _dtype_of(dtype)
        if dt == x.dtype:
            return x.copy()
        if dt == np.bool_:
            return (_f64(x) != 0) if is_float(x.dtype) else (x != 0)
        if is_float(x.dtype) and not is_float(dt):
            # truncation toward zero pinned by ref mpsgraph_test.go:1485-1532; saturation / NaN->0 unpinned
            v = np.trunc(_f64(x))
            info = np.iinfo(dt)
            v = np.where(np.isnan(v), 0.0, v)
            v = np.clip(v, float(info.min), float(info.max))
            out = np.empty(v.shape, dtype=dt)
            flat = out.reshape(-1)
            for i, e in enumerate(v.reshape(-1)):
                flat[i] = min(max(int(e), info.min), info.max)
            return out
        if is_float(dt):
            return _round(_f64(x), dt) if is_float(x.dtype) else x.astype(np.float64).astype(dt) if x.dtype.itemsize < 8 else x.astype(dt)
        with np.errstate(over="ignore"):
            return x.astype(dt)  # integer -> integer wraps

    def BroadcastInDim(self, x, output_shape, broadcast_axes):
        dims = _dims_of(output_shape)
        view = [1] * len(dims)
        for i, ax in enumerate(broadcast_axes):
            view[ax] = x.shape[i]
        return np.ascontiguousarray(np.broadcast_to(x.reshape(view), dims))

    def Slice(self, x, starts, limits, strides):
        return np.ascontiguousarray(x[tuple(slice(s, l, st) for s, l, st in zip(starts, limits, strides))])

    def Concatenate(self, axis, *operands): return np.concatenate(operands, axis=axis)
    def Reverse(self, x, *axes): return np.ascontiguousarray(np.flip(x, axis=tuple(axes)))

    def Pad(self, x, fill_value, *axes_config):
        pads = [(c[0], c[1]) for c in axes_config]
        return np.pad(x, pads, mode="constant", constant_values=np.asarray(fill_value).reshape(-1)[0])

    @staticmethod
    def _clamped_starts(what, operand, starts, sizes):
        if len(starts) != operand.ndim:
            raise OracleError(f"{what}: one start index per axis")
        out = []
        for d, (s, n) in enumerate(zip(starts, sizes)):
            s = np.asarray(s)
            if s.size != 1 or s.dtype.kind not in "iu":
                raise OracleError(f"{what}: start index {d} must be one integer value")
            out.append(int(min(max(int(s.reshape(-1)[0]), 0), operand.shape[d] - n)))
        return out

    def DynamicSlice(self, operand, start_indices, slice_sizes):
        # ref function.go:1571-1594; starts clamped so the slice fits (GoMLX's documented DynamicSlice)
        if len(slice_sizes) != operand.ndim or any(n < 0 or n > d for n, d in zip(slice_sizes, operand.shape)):
            raise OracleError("DynamicSlice: slice sizes")
        st = self._clamped_starts("DynamicSlice", operand, start_indices, slice_sizes)
        return np.ascontiguousarray(operand[tuple(slice(s, s + n) for s, n in zip(st, slice_sizes))])

    def DynamicUpdateSlice(self, operand, update, start_indices):
        # ref function.go:1596-1621
        if update.dtype != operand.dtype or update.ndim != operand.ndim or any(u > d for u, d in zip(update.shape, operand.shape)):
            raise OracleError("DynamicUpdateSlice: update shape or dtype")
        st = self._clamped_starts("DynamicUpdateSlice", operand, start_indices, update.shape)
        out = operand.copy()
        out[tuple(slice(s, s + n) for s, n in zip(st, update.shape))] = update
        return out

    def Where(self, cond, on_true, on_false):
        if cond.dtype != np.bool_ or on_true.dtype != on_false.dtype:
            raise OracleError("Where: dtypes")
        return np.where(cond, on_true, on_false)

    def Clamp(self, lo, x, hi):
        if is_float(x.dtype):
            return _round(np.minimum(np.maximum(_f64(x), _f64(lo)), _f64(hi)), x.dtype)
        return np.minimum(np.maximum(x, lo), hi)

    # ---- DotGeneral (ref dotgeneral.go:15-53, 65-164, 186-227) -----------------
    def DotGeneral(self, lhs, lc, lb, rhs, rc, rb, config=None):
        lc, lb, rc, rb = list(lc or []), list(lb or []), list(rc or []), list(rb or [])
        if lhs.dtype != rhs.dtype:
            raise OracleError("DotGeneral: operand dtypes differ")
        lfree = [i for i in range(lhs.ndim) if i not in lc and i not in lb]
        rfree = [i for i in range(rhs.ndim) if i not in rc and i not in rb]
        # perm = batch ++ free ++ contracting (classifyAxes, ref dotgeneral.go:186-227)
        a = np.transpose(lhs, lb + lfree + lc)
        b = np.transpose(rhs, rb + rfree + rc)
        bd = [lhs.shape[i] for i in lb]
        md = [lhs.shape[i] for i in lfree]
        nd = [rhs.shape[i] for i in rfree]
        kd = [lhs.shape[i] for i in lc]
        if kd != [rhs.shape[i] for i in rc] or bd != [rhs.shape[i] for i in rb]:
            raise OracleError("DotGeneral: dims differ")
        B, M, N, K = (int(np.prod(d, dtype=np.int64)) for d in (bd, md, nd, kd))
        if is_float(lhs.dtype):
            a3 = _f64(a).reshape(B, M, K)
            b3 = _f64(b).reshape(B, N, K)
            out = np.einsum("bmk,bnk->bmn", a3, b3, optimize=True)
            return _round(out, lhs.dtype).reshape(bd + md + nd)  # output dtype = lhs dtype (ref dotgeneral.go:52)
        a3 = a.reshape(B, M, K).astype(np.int64)
        b3 = b.reshape(B, N, K).astype(np.int64)
        with np.errstate(over="ignore"):
            out = np.einsum("bmk,bnk->bmn", a3, b3)
        return out.astype(lhs.dtype).reshape(bd + md + nd)

    # ---- reductions (ref function.go:1147-1198, 2262-2270) ---------------------
    def _reduce(self, x, axes, ffn, ifn):
        axes = tuple(range(x.ndim)) if len(axes) == 0 else tuple(a + x.ndim if a < 0 else a for a in axes)  # empty = all
        if is_float(x.dtype):
            with np.errstate(all="ignore"):
                return _round(ffn(_f64(x), axis=axes), x.dtype)
        if x.dtype == np.bool_:
            return ifn(x, axis=axes).astype(np.bool_)
        with np.errstate(over="ignore"):
            wide = np.int64 if x.dtype.kind == "i" else np.uint64
            return ifn(x.astype(wide), axis=axes).astype(x.dtype)

    def ReduceSum(self, x, *axes): return self._reduce(x, axes, np.sum, np.sum)
    def ReduceProduct(self, x, *axes): return self._reduce(x, axes, np.prod, np.prod)
    def ReduceMax(self, x, *axes): return self._reduce(x, axes, np.max, np.max)
    def ReduceMin(self, x, *axes): return self._reduce(x, axes, np.min, np.min)
    def ReduceLogicalAnd(self, x, *axes): return self.ReduceMin(x, *axes)
    def ReduceLogicalOr(self, x, *axes): return self.ReduceMax(x, *axes)

    def ArgMinMax(self, x, axis, output_dtype, is_min):
        # axis removed, result cast to output dtype (ref function.go:1204-1242).
        # unpinned: lowest index wins ties; NaN counts as the extreme (NumPy rule).
        v = _f64(x) if is_float(x.dtype) else x
        r = np.argmin(v, axis=axis) if is_min else np.argmax(v, axis=axis)
        return r.astype(_dtype_of(output_dtype))

    # ---- Gather (XLA semantics; ref gather.go:24-434) --------------------------
    def Gather(self, operand, start_indices, index_vector_axis, offset_output_axes, collapsed_slice_axes, start_index_map, slice_sizes,
               indices_are_sorted=False):
        idx = start_indices
        if index_vector_axis == idx.ndim:
            idx = idx.reshape(idx.shape + (1,))
        idx = np.moveaxis(idx, index_vector_axis, -1)
        batch_shape = idx.shape[:-1]
        offset_dims = [slice_sizes[i] for i in range(operand.ndim) if i not in collapsed_slice_axes]
        out_rank = len(batch_shape) + len(offset_dims)
        out_shape = [0] * out_rank
        bi = oi = 0
        for d in range(out_rank):
            if d in offset_output_axes:
                out_shape[d] = offset_dims[oi]; oi += 1
            else:
                out_shape[d] = batch_shape[bi]; bi += 1
        out = np.empty(out_shape, dtype=operand.dtype)
        offset_operand_axes = [i for i in range(operand.ndim) if i not in collapsed_slice_axes]
        for o in np.ndindex(*out_shape):
            batch = tuple(o[d] for d in range(out_rank) if d not in offset_output_axes)
            offs = [o[d] for d in offset_output_axes]
            start = [0] * operand.ndim
            for c, ax in enumerate(start_index_map):
                s = int(idx[batch + (c,)])
                start[ax] = min(max(s, 0), operand.shape[ax] - slice_sizes[ax])  # unpinned: XLA clamp
            src = list(start)
            for j, ax in enumerate(offset_operand_axes):
                src[ax] += offs[j]
            out[o] = operand[tuple(src)]
        return out

    # ---- fused ops --------------------------------------------------------------
    def FusedSoftmax(self, x, axis):
        # standard max-subtracted form; agrees with ref mpsgraph_test.go:1182-1189
        v = _f64(x)
        with np.errstate(all="ignore"):
            e = np.exp(v - np.max(v, axis=axis, keepdims=True))
            return _round(e / np.sum(e, axis=axis, keepdims=True), x.dtype)

    def FusedSoftmaxMasked(self, x, scale=1.0, causal=False, mask=None):
        # the scale / causal / mask / softmax segment of SDPA (ref function.go:2756-2894)
        v = _f64(x) * float(np.float32(scale))  # scale constants pass through float32 (ref function.go:212-231)
        sq, sk = x.shape[-2], x.shape[-1]
        if mask is not None:
            m = np.asarray(mask)
            if m.dtype == np.bool_:
                v = np.where(np.broadcast_to(m, x.shape), v, -np.inf)
            else:
                v = v + _f64(m)
        if causal:
            keep = np.arange(sq)[:, None] >= np.arange(sk)[None, :]   # row >= col (ref function.go:2777-2794)
            v = np.where(keep, v, -np.inf)
        with np.errstate(all="ignore"):
            e = np.exp(v - np.max(v, axis=-1, keepdims=True))   # fully masked row -> NaN (unpinned, IEEE)
            return _round(e / np.sum(e, axis=-1, keepdims=True), x.dtype)

    def FusedGelu(self, x, exact):
        # constants from ref function.go:2299-2407
        v = _f64(x)
        if exact:
            y = 0.5 * v * (1.0 + _erf(v * 0.7071067811865475))
        else:
            c = float(np.float32(0.7978845608))
            k = float(np.float32(0.044715))
            y = 0.5 * v * (1.0 + np.tanh(c * (v + k * v * v * v)))
        return _round(y, x.dtype)

    def FusedLayerNorm(self, x, axes, epsilon, gamma=None, beta=None):
        # two-pass biased variance, rsqrt(var+eps), *gamma, +beta (ref function.go:2410-2565)
        ax = tuple(sorted(a + x.ndim if a < 0 else a for a in axes))
        v = _f64(x)
        mean = v.mean(axis=ax, keepdims=True)
        d = v - mean
        var = (d * d).mean(axis=ax, keepdims=True)
        y = d / np.sqrt(var + float(np.float32(epsilon)))
        y = self._scale_shift(x, y, ax, gamma, beta)
        return _round(y, x.dtype)

    def FusedRMSNorm(self, x, axes, epsilon, gamma=None):
        # unpinned (absent from the reference): y = x * rsqrt(mean(x^2) + eps) * gamma
        ax = tuple(sorted(a + x.ndim if a < 0 else a for a in axes))
        v = _f64(x)
        y = v / np.sqrt((v * v).mean(axis=ax, keepdims=True) + float(np.float32(epsilon)))
        y = self._scale_shift(x, y, ax, gamma, None)
        return _round(y, x.dtype)

    @staticmethod
    def _scale_shift(x, y, ax, gamma, beta):
        def lay(p):
            p = _f64(p)
            if p.ndim >= x.ndim:
                return p
            view = [1] * x.ndim   # lower rank: laid onto the normalised axes in order (ref function.go:2499-2530)
            for i, a in enumerate(ax[:p.ndim]):
                view[a] = p.shape[i]
            return p.reshape(view)
        if gamma is not None:
            y = y * lay(gamma)
        if beta is not None:
            y = y + lay(beta)
        return y

    def FusedDense(self, x, weight, bias, activation):
        # ref function.go:2567-2667
        if x.ndim < 1 or weight.ndim < 2 or x.shape[-1] != weight.shape[0]:
            raise OracleError("FusedDense: shapes")
        y = np.tensordot(_f64(x), _f64(weight), axes=([x.ndim - 1], [0]))
        if bias is not None:
            y = y + _f64(bias)
        if activation == ACT_GELU:
            c, k = float(np.float32(0.7978845608)), float(np.float32(0.044715))
            y = 0.5 * y * (1.0 + np.tanh(c * (y + k * y ** 3)))
        elif activation == ACT_RELU:
            y = np.maximum(y, 0.0)
        elif activation == ACT_SILU:
            y = y / (1.0 + np.exp(-y))
        elif activation == ACT_TANH:
            y = np.tanh(y)
        elif activation != ACT_NONE:
            raise OracleError("FusedDense: unsupported activation type")
        return _round(y, x.dtype)

    def FusedAttentionQKVProjection(self, x, w_qkv, bias_q, bias_k, bias_v, query_dim, key_value_dim):
        # ref function.go:2976-3075
        combined = _round(np.tensordot(_f64(x), _f64(w_qkv), axes=([x.ndim - 1], [0])), x.dtype)
        parts = []
        lo = 0
        for size, b in ((query_dim, bias_q), (key_value_dim, bias_k), (key_value_dim, bias_v)):
            p = combined[..., lo:lo + size]
            if b is not None:
                p = _round(_f64(p) + _f64(b), x.dtype)
            parts.append(np.ascontiguousarray(p))
            lo += size
        return tuple(parts)

    def FusedScaledDotProductAttention(self, query, key, value, mask, num_heads, num_kv_heads, axes_layout, scale, causal, options=None):
        # ref function.go:2669-2907
        if query.ndim != 4:
            raise OracleError("SDPA: query must have rank 4")
        if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads != 0:
            raise OracleError("SDPA: heads")
        q, k, v, m = query, key, value, mask
        if axes_layout == LAYOUT_BSHD:
            q, k, v = (np.transpose(t, (0, 2, 1, 3)) for t in (q, k, v))
            if m is not None and m.ndim == 4:
                m = np.transpose(m, (0, 2, 1, 3))
        rep = num_heads // num_kv_heads
        if rep > 1:  # each KV head repeated `rep` times consecutively (ref function.go:2910-2955)
            k = np.repeat(k, rep, axis=1)
            v = np.repeat(v, rep, axis=1)
        scores = _round(np.einsum("bhqd,bhkd->bhqk", _f64(q), _f64(k)), query.dtype)
        probs = self.FusedSoftmaxMasked(scores, scale, causal, m)
        out = _round(np.einsum("bhqk,bhkd->bhqd", _f64(probs), _f64(v)), query.dtype)
        if axes_layout == LAYOUT_BSHD:
            out = np.ascontiguousarray(np.transpose(out, (0, 2, 1, 3)))
        return out

    # ---- training-side ops ------------------------------------------------------
    def BatchNormForInference(self, operand, scale, offset, mean, variance, epsilon, feature_axis):
        # (x - mean) * rsqrt(var + eps) * scale + offset along the feature axis (ref function.go:1248-1261)
        ax = feature_axis + operand.ndim if feature_axis < 0 else feature_axis
        view = [1] * operand.ndim
        view[ax] = operand.shape[ax]
        lay = lambda p: _f64(p).reshape(view)
        y = (_f64(operand) - lay(mean)) / np.sqrt(lay(variance) + float(np.float32(epsilon))) * lay(scale) + lay(offset)
        return _round(y, operand.dtype)

    def BatchNormForTraining(self, operand, scale, offset, epsilon, feature_axis):
        # batch mean, biased variance of the centred value, normalise, scale, offset (ref function.go:1263-1375)
        ax = feature_axis + operand.ndim if feature_axis < 0 else feature_axis
        batch = tuple(i for i in range(operand.ndim) if i != ax)
        view = [1] * operand.ndim
        view[ax] = operand.shape[ax]
        v = _f64(operand)
        mean = v.mean(axis=batch, keepdims=True) if batch else v
        d = v - mean
        var = (d * d).mean(axis=batch, keepdims=True) if batch else d * d
        y = d / np.sqrt(var + float(np.float32(epsilon))) * _f64(scale).reshape(view) + _f64(offset).reshape(view)
        return _round(y, operand.dtype), _round(mean.reshape(-1), operand.dtype), _round(var.reshape(-1), operand.dtype)

    def BatchNormGradient(self, operand, scale, mean, variance, grad_output, epsilon, feature_axis):
        # ref function.go:1377-1527
        ax = feature_axis + operand.ndim if feature_axis < 0 else feature_axis
        batch = tuple(i for i in range(operand.ndim) if i != ax)
        view = [1] * operand.ndim
        view[ax] = operand.shape[ax]
        n = 1
        for i in batch:
            n *= operand.shape[i]
        lay = lambda p: _f64(p).reshape(view)
        inv = 1.0 / np.sqrt(lay(variance) + float(np.float32(epsilon)))
        xhat = (_f64(operand) - lay(mean)) * inv
        dy = _f64(grad_output)
        g_off = dy.sum(axis=batch, keepdims=True) if batch else dy
        g_sc = (dy * xhat).sum(axis=batch, keepdims=True) if batch else dy * xhat
        g_op = (1.0 / n) * lay(scale) * inv * (n * dy - g_off - xhat * g_sc)
        return _round(g_op, operand.dtype), _round(g_sc.reshape(-1), operand.dtype), _round(g_off.reshape(-1), operand.dtype)

    def _scatter(self, mode, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                 scatter_axes_to_operand_axes):
        # XLA scatter with a combiner (ref gather.go:441-641); elements that land outside the operand are dropped (unpinned)
        idx = np.asarray(scatter_indices).astype(np.int64)
        if index_vector_axis == idx.ndim:
            idx = idx[..., None]
        idx = np.moveaxis(idx, index_vector_axis, -1)                 # [batch..., components]
        upd = np.asarray(updates)
        uw = list(update_window_axes)
        scatter_axes = [d for d in range(upd.ndim) if d not in uw]
        window_operand_axes = [d for d in range(operand.ndim) if d not in list(inserted_window_axes)]
        grids = np.meshgrid(*[np.arange(n) for n in upd.shape], indexing="ij") if upd.ndim else []
        coord = [np.zeros(upd.shape, dtype=np.int64) for _ in range(operand.ndim)]
        batch_index = tuple(grids[d] for d in scatter_axes)
        for c, ax in enumerate(scatter_axes_to_operand_axes):
            coord[ax] = coord[ax] + (idx[batch_index + (c,)] if batch_index else idx[c])
        for j, ax in enumerate(window_operand_axes):
            coord[ax] = coord[ax] + grids[uw[j]]
        inside = np.ones(upd.shape, dtype=bool)
        for d in range(operand.ndim):
            inside &= (coord[d] >= 0) & (coord[d] < operand.shape[d])
        flat = np.zeros(upd.shape, dtype=np.int64)
        for d in range(operand.ndim):
            flat = flat * operand.shape[d] + np.where(inside, coord[d], 0)
        isf = is_float(operand.dtype)
        out = (_f64(operand) if isf else np.asarray(operand).astype(np.int64 if np.dtype(operand.dtype).kind == "i" else np.uint64)).reshape(-1).copy()
        vals = (_f64(upd) if isf else upd.astype(out.dtype))[inside]
        dst = flat[inside]
        if mode == 0:
            np.add.at(out, dst, vals)
        elif mode == 1:
            np.maximum.at(out, dst, vals)    # NaN-propagating, like the kernels
        else:
            np.minimum.at(out, dst, vals)
        out = out.reshape(operand.shape)
        return _round(out, operand.dtype) if isf else out.astype(operand.dtype)

    def ScatterSum(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False):
        return self._scatter(0, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes, scatter_axes_to_operand_axes)

    def ScatterMax(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False):
        return self._scatter(1, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes, scatter_axes_to_operand_axes)

    def ScatterMin(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False):
        return self._scatter(2, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes, scatter_axes_to_operand_axes)

    def RNGBitGenerator(self, state, shape):
        # unpinned: the reference takes its values from Apple's generator (ref function.go:1627-1692) and only adds 1 to every
        # state word.  Defined here as Philox4x32-10 (Salmon et al., SC'11): key = state[0], counter = (state[2] : state[1]) +
        # block number, four 32-bit words per block; integers take the raw bits, floats a uniform [0, 1) from the top bits.
        st = np.asarray(state, dtype=np.uint64)
        dt = np.dtype(_dtype_of(shape))
        dims = _dims_of(shape)
        n = int(np.prod(dims)) if len(dims) else 1
        wide = dt.itemsize == 8
        per = 2 if wide else 4
        blocks = (n + per - 1) // per
        b = np.arange(blocks, dtype=np.uint64)
        with np.errstate(over="ignore"):
            c_lo = st[1] + b
            c_hi = st[2] + (c_lo < st[1]).astype(np.uint64)
        M32 = np.uint64(0xffffffff)
        c0, c1, c2, c3 = c_lo & M32, c_lo >> np.uint64(32), c_hi & M32, c_hi >> np.uint64(32)
        k0, k1 = np.uint64(int(st[0]) & 0xffffffff), np.uint64(int(st[0]) >> 32)
        for _ in range(10):
            p0, p1 = np.uint64(0xD2511F53) * c0, np.uint64(0xCD9E8D57) * c2   # 32 x 32 -> 64 bits, exact in uint64
            c0, c1, c2, c3 = (p1 >> np.uint64(32)) ^ c1 ^ k0, p1 & M32, (p0 >> np.uint64(32)) ^ c3 ^ k1, p0 & M32
            k0, k1 = (k0 + np.uint64(0x9E3779B9)) & M32, (k1 + np.uint64(0xBB67AE85)) & M32
        words = np.stack([c0, c1, c2, c3], axis=1).reshape(-1)
        if wide:
            v = (words[0::2] | (words[1::2] << np.uint64(32)))[:n]
            vals = (v >> np.uint64(11)).astype(np.float64) * 2.0 ** -53 if dt == np.float64 else v.astype(dt)
        else:
            w = words[:n]
            if dt == np.float32:
                vals = ((w >> np.uint64(8)).astype(np.float64) * 2.0 ** -24).astype(np.float32)
            elif dt == np.float16:
                vals = ((w >> np.uint64(21)).astype(np.float64) * 2.0 ** -11).astype(np.float16)
            elif is_float(dt):   # bfloat16
                vals = ((w >> np.uint64(24)).astype(np.float64) * 2.0 ** -8).astype(np.float32).astype(dt)
            else:
                vals = (w & np.uint64((1 << (8 * dt.itemsize)) - 1)).astype(dt)
        with np.errstate(over="ignore"):
            new_state = st + np.uint64(1)
        return new_state, vals.reshape(dims)

    # ---- control flow over closures (ref function.go:354-652; executable.go:219-480) ----
    # The oracle evaluates eagerly, so a closure here is a Python callable over arrays: MakeClosure(param_shapes, body) wraps
    # body(f, *params) -> list of outputs and checks the arguments against the declared parameter shapes on every call.
    def MakeClosure(self, param_shapes, body):
        shapes = [(np.dtype(_dtype_of(s)), tuple(_dims_of(s))) for s in param_shapes]

        def call(*args):
            if len(args) != len(shapes):
                raise OracleError(f"closure expects {len(shapes)} parameters, got {len(args)}")
            for i, (a, (dt, dims)) in enumerate(zip(args, shapes)):
                a = np.asarray(a)
                if a.dtype != dt or tuple(a.shape) != dims:
                    raise OracleError(f"closure parameter {i}: expected {dt}{list(dims)}, got {a.dtype}{list(a.shape)}")
            return [np.asarray(o) for o in body(self, *[np.asarray(a) for a in args])]

        call.num_params = len(shapes)
        return call

    def Call(self, fn, *inputs):
        # ref function.go:354-403; executable.go:449-480: run the target on the inputs
        return fn(*inputs)

    def While(self, cond, body, *initial_state):
        # ref function.go:406-489; executable.go:219-283: cond(state) -> scalar bool, body(state) -> state, at most 1e6 trips
        if len(initial_state) == 0:
            raise OracleError("While: requires at least one initial state value")
        state = [np.asarray(v) for v in initial_state]
        for _ in range(1000000):
            (go,) = cond(*state)
            if go.dtype != np.bool_ or go.ndim != 0:
                raise OracleError("While: cond must return scalar bool")
            if not bool(go):
                return state
            new = body(*state)
            if len(new) != len(state) or any(n.dtype != o.dtype or n.shape != o.shape for n, o in zip(new, state)):
                raise OracleError("While: body output must match state shape")
            state = new
        raise OracleError("While: exceeded maximum iterations (1000000)")

    def If(self, pred, true_branch, false_branch):
        # ref function.go:492-560; executable.go:286-318: the chosen branch alone runs; branches take no parameters
        pred = np.asarray(pred)
        if pred.dtype != np.bool_ or pred.ndim != 0:
            raise OracleError("If: pred must be scalar bool")
        return true_branch() if bool(pred) else false_branch()

    def Sort(self, comparator, axis, is_stable, *inputs):
        # ref function.go:563-652; executable.go:321-446: every row along `axis` is sorted on the host by a comparison sort
        # that asks the comparator (lhs_0, rhs_0, lhs_1, rhs_1, ...) -> "lhs before rhs"; all inputs are permuted alike.
        # Always stable here (a stable order is one of the orders an unstable sort may return).
        import functools
        if len(inputs) == 0:
            raise OracleError("Sort: requires at least one input tensor")
        ins = [np.asarray(v) for v in inputs]
        if any(v.shape != ins[0].shape for v in ins):
            raise OracleError("Sort: all inputs must have same dimensions")
        rank = ins[0].ndim
        ax = axis + rank if axis < 0 else axis
        if ax < 0 or ax >= rank:
            raise OracleError(f"Sort: axis {axis} out of range for rank {rank}")
        moved = [np.moveaxis(v, ax, -1) for v in ins]
        outs = [np.empty_like(m) for m in moved]
        n = ins[0].shape[ax]
        for row in np.ndindex(*moved[0].shape[:-1]):
            def before(a, b):
                args = []
                for m in moved:
                    args += [m[row][a], m[row][b]]
                (r,) = comparator(*args)
                return bool(r)
            order = sorted(range(n), key=functools.cmp_to_key(lambda a, b: -1 if before(a, b) else (1 if before(b, a) else 0)))
            for m, o in zip(moved, outs):
                o[row] = m[row][order]
        return [np.ascontiguousarray(np.moveaxis(o, -1, ax)) for o in outs]


def compare(got: np.ndarray, want: np.ndarray, rtol: float, atol_scale: float = 0.0):
    """Returns (ok, max_violation).  Float rule: |got-want| <= rtol*|want| + atol, atol = atol_scale * rtol * rms(want)
    (norm-relative term: the elementwise relative error of a zero-mean dot product is unbounded).
    Non-float arrays must be bit-identical.  NaNs must coincide."""
    got, want = np.asarray(got), np.asarray(want)
    if got.shape != want.shape or got.dtype != want.dtype:
        return False, float("inf")
    if not is_float(want.dtype):
        return bool(np.array_equal(got, want)), 0.0
    g, w = _f64(got), _f64(want)
    nan_g, nan_w = np.isnan(g), np.isnan(w)
    if not np.array_equal(nan_g, nan_w):
        return False, float("inf")
    inf_mask = np.isinf(w)
    if not np.array_equal(g[inf_mask], w[inf_mask]):
        return False, float("inf")
    fin = ~(nan_w | inf_mask)
    if not fin.any():
        return True, 0.0
    rms = float(np.sqrt(np.mean(w[fin] ** 2))) if fin.any() else 0.0
    tol = rtol * np.abs(w[fin]) + atol_scale * rtol * rms
    err = np.abs(g[fin] - w[fin])
    viol = err - tol
    return bool((viol <= 0).all()), float(viol.max())
