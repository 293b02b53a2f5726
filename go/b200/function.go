//go:build cgo && linux

package b200

import (
	"reflect"

	"github.com/gomlx/go-darwinml/b200/internal/bridge"
	"github.com/gomlx/gomlx/backends"
	"github.com/gomlx/gomlx/backends/notimplemented"
	"github.com/gomlx/gomlx/pkg/core/shapes"
	"github.com/gomlx/gopjrt/dtypes"
	"github.com/pkg/errors"
)

// node is this backend's backends.Value: a native graph node and its shape (the reference's graphNode,
// mpsgraph/gomlx/function.go:32-37).
type node struct {
	value bridge.Value
	shape shapes.Shape
	owner *Function
}

type param struct {
	value bridge.Value
	name  string
	shape shapes.Shape
}

// Function implements backends.Function over one native graph.  Ops the C ABI does not lower fall through to the
// embedded notimplemented.Function, which returns notimplemented.NotImplementedError (as in the reference, function.go:41).
// Shapes come back from the native graph after every call, so shape inference and validation have one implementation
// (the C++ one); errors carry the op's name like the reference's (function.go:661, 799).
type Function struct {
	notimplemented.Function

	builder  *Builder
	name     string
	parent   *Function // set for closures
	sub      bool      // a closure or a named sub-function: its parameters are closure parameters, not executable inputs
	params   []param
	outputs  []*node
	returned bool
}

var _ backends.Function = (*Function)(nil)

func (f *Function) Name() string { return f.name }

func (f *Function) Parent() backends.Function {
	if f.parent == nil {
		return nil
	}
	return f.parent
}

// Closure creates a closure of this function: the cond / body of While, a branch of If, Sort's comparator
// (mpsgraph/gomlx/function.go:120-131).  It shares the builder's native context and captures the values of its
// ancestors by using them; the reference gives every closure a context of its own and feeds captures through placeholders.
func (f *Function) Closure() (backends.Function, error) {
	return &Function{builder: f.builder, parent: f, sub: true}, nil
}

func (f *Function) ctx() bridge.Context { return f.builder.ctx }

// resolve checks that v is a live value of this function or, for a closure, of one of its ancestors; other foreign
// values are errors (resolveNode, mpsgraph/gomlx/function.go:179-195).
func (f *Function) resolve(op string, v backends.Value) (*node, error) {
	n, ok := v.(*node)
	if !ok || n == nil {
		return nil, errors.Errorf("%s: value of type %T does not belong to the b200 backend", op, v)
	}
	for p := f; p != nil; p = p.parent {
		if n.owner == p {
			return n, nil
		}
	}
	return nil, errors.Errorf("%s: node from unrelated function scope", op)
}

func (f *Function) resolveAll(op string, vs []backends.Value) ([]*node, []bridge.Value, error) {
	ns := make([]*node, len(vs))
	hs := make([]bridge.Value, len(vs))
	for i, v := range vs {
		n, err := f.resolve(op, v)
		if err != nil {
			return nil, nil, err
		}
		ns[i], hs[i] = n, n.value
	}
	return ns, hs, nil
}

// optional resolves a value that may be nil (a bias, a mask).
func (f *Function) optional(op string, v backends.Value) (bridge.Value, error) {
	if v == nil {
		return nil, nil
	}
	n, err := f.resolve(op, v)
	if err != nil {
		return nil, err
	}
	return n.value, nil
}

// wrap reads the result's dtype and dims back from the native graph.
func (f *Function) wrap(op string, v bridge.Value, err error) (backends.Value, error) {
	if err != nil {
		return nil, errors.Wrap(err, op)
	}
	dt, dims := bridge.ValueShape(v)
	goDT, derr := dtypeFromBridge(dt)
	if derr != nil {
		return nil, errors.Wrap(derr, op)
	}
	return &node{value: v, shape: shapes.Make(goDT, dims...), owner: f}, nil
}

func dtypeFromBridge(code int) (dtypes.DType, error) {
	table := []dtypes.DType{dtypes.Bool, dtypes.Int8, dtypes.Int16, dtypes.Int32, dtypes.Int64, dtypes.Float16, dtypes.BFloat16,
		dtypes.Float32, dtypes.Float64, dtypes.Uint8, dtypes.Uint16, dtypes.Uint32, dtypes.Uint64}
	if code < 0 || code >= len(table) {
		return dtypes.InvalidDType, errors.Errorf("b200: native dtype code %d", code)
	}
	return table[code], nil
}

// ---- leaves (mpsgraph/gomlx/function.go:288-351) ----

func (f *Function) Parameter(name string, shape shapes.Shape, sharding *backends.ShardingSpec) (backends.Value, error) {
	dt, err := dtypeToBridge(shape.DType)
	if err != nil {
		return nil, errors.Wrap(err, "Parameter")
	}
	newParam := f.ctx().Placeholder
	if f.sub {
		newParam = f.ctx().ClosureParameter
	}
	v, err := newParam(dt, dims64(shape.Dimensions))
	if err != nil {
		return nil, errors.Wrapf(err, "Parameter(%q)", name)
	}
	f.params = append(f.params, param{value: v, name: name, shape: shape})
	return &node{value: v, shape: shape, owner: f}, nil
}

func (f *Function) Constant(flat any, dims ...int) (backends.Value, error) {
	dt := dtypes.FromGoType(reflect.TypeOf(flat).Elem())
	code, err := dtypeToBridge(dt)
	if err != nil {
		return nil, errors.Wrap(err, "Constant")
	}
	ptr, nbytes, err := flatBytes(flat)
	if err != nil {
		return nil, errors.Wrap(err, "Constant")
	}
	v, err := f.ctx().Constant(ptr, nbytes, code, dims64(dims))
	return f.wrap("Constant", v, err)
}

func (f *Function) Return(outputs []backends.Value, shardings []*backends.ShardingSpec) error {
	if f.returned {
		return errors.New("Return: already called")
	}
	if len(outputs) == 0 {
		return errors.New("Return: no outputs")
	}
	for i, o := range outputs {
		n, err := f.resolve("Return", o)
		if err != nil {
			return errors.Wrapf(err, "output #%d", i)
		}
		f.outputs = append(f.outputs, n)
	}
	f.returned = true
	return nil
}

func (f *Function) Iota(shape shapes.Shape, iotaAxis int) (backends.Value, error) {
	dt, err := dtypeToBridge(shape.DType)
	if err != nil {
		return nil, errors.Wrap(err, "Iota")
	}
	v, err := f.ctx().Iota(dt, dims64(shape.Dimensions), iotaAxis)
	return f.wrap("Iota", v, err)
}

// ---- elementwise families (mpsgraph/gomlx/function.go:658-963, 2234-2256) ----

func (f *Function) unary(op string, code int, x backends.Value) (backends.Value, error) {
	n, err := f.resolve(op, x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Unary(code, n.value)
	return f.wrap(op, v, err)
}

func (f *Function) binary(op string, code int, lhs, rhs backends.Value) (backends.Value, error) {
	a, err := f.resolve(op, lhs)
	if err != nil {
		return nil, err
	}
	b, err := f.resolve(op, rhs)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Binary(code, a.value, b.value)
	return f.wrap(op, v, err)
}

func (f *Function) Abs(x backends.Value) (backends.Value, error)   { return f.unary("Abs", bridge.OpAbs, x) }
func (f *Function) Neg(x backends.Value) (backends.Value, error)   { return f.unary("Neg", bridge.OpNeg, x) }
func (f *Function) Sqrt(x backends.Value) (backends.Value, error)  { return f.unary("Sqrt", bridge.OpSqrt, x) }
func (f *Function) Rsqrt(x backends.Value) (backends.Value, error) { return f.unary("Rsqrt", bridge.OpRsqrt, x) }
func (f *Function) Exp(x backends.Value) (backends.Value, error)   { return f.unary("Exp", bridge.OpExp, x) }
func (f *Function) Expm1(x backends.Value) (backends.Value, error) { return f.unary("Expm1", bridge.OpExpm1, x) }
func (f *Function) Log(x backends.Value) (backends.Value, error)   { return f.unary("Log", bridge.OpLog, x) }
func (f *Function) Log1p(x backends.Value) (backends.Value, error) { return f.unary("Log1p", bridge.OpLog1p, x) }
func (f *Function) Sin(x backends.Value) (backends.Value, error)   { return f.unary("Sin", bridge.OpSin, x) }
func (f *Function) Cos(x backends.Value) (backends.Value, error)   { return f.unary("Cos", bridge.OpCos, x) }
func (f *Function) Tanh(x backends.Value) (backends.Value, error)  { return f.unary("Tanh", bridge.OpTanh, x) }
func (f *Function) Logistic(x backends.Value) (backends.Value, error) {
	return f.unary("Logistic", bridge.OpLogistic, x)
}
func (f *Function) Erf(x backends.Value) (backends.Value, error)   { return f.unary("Erf", bridge.OpErf, x) }
func (f *Function) Floor(x backends.Value) (backends.Value, error) { return f.unary("Floor", bridge.OpFloor, x) }
func (f *Function) Ceil(x backends.Value) (backends.Value, error)  { return f.unary("Ceil", bridge.OpCeil, x) }
func (f *Function) Round(x backends.Value) (backends.Value, error) { return f.unary("Round", bridge.OpRound, x) }
func (f *Function) Sign(x backends.Value) (backends.Value, error)  { return f.unary("Sign", bridge.OpSign, x) }
func (f *Function) LogicalNot(x backends.Value) (backends.Value, error) {
	return f.unary("LogicalNot", bridge.OpLogicalNot, x)
}
func (f *Function) BitwiseNot(x backends.Value) (backends.Value, error) {
	return f.unary("BitwiseNot", bridge.OpBitwiseNot, x)
}
func (f *Function) IsFinite(x backends.Value) (backends.Value, error) { return f.unary("IsFinite", bridge.OpIsFinite, x) }
func (f *Function) IsNaN(x backends.Value) (backends.Value, error)    { return f.unary("IsNaN", bridge.OpIsNaN, x) }
func (f *Function) Identity(x backends.Value) (backends.Value, error) { return f.unary("Identity", bridge.OpIdentity, x) }

func (f *Function) Add(a, b backends.Value) (backends.Value, error) { return f.binary("Add", bridge.OpAdd, a, b) }
func (f *Function) Sub(a, b backends.Value) (backends.Value, error) { return f.binary("Sub", bridge.OpSub, a, b) }
func (f *Function) Mul(a, b backends.Value) (backends.Value, error) { return f.binary("Mul", bridge.OpMul, a, b) }
func (f *Function) Div(a, b backends.Value) (backends.Value, error) { return f.binary("Div", bridge.OpDiv, a, b) }
func (f *Function) Rem(a, b backends.Value) (backends.Value, error) { return f.binary("Rem", bridge.OpRem, a, b) }
func (f *Function) Pow(a, b backends.Value) (backends.Value, error) { return f.binary("Pow", bridge.OpPow, a, b) }
func (f *Function) Max(a, b backends.Value) (backends.Value, error) { return f.binary("Max", bridge.OpMax, a, b) }
func (f *Function) Min(a, b backends.Value) (backends.Value, error) { return f.binary("Min", bridge.OpMin, a, b) }
func (f *Function) Atan2(a, b backends.Value) (backends.Value, error) {
	return f.binary("Atan2", bridge.OpAtan2, a, b)
}
func (f *Function) LogicalAnd(a, b backends.Value) (backends.Value, error) {
	return f.binary("LogicalAnd", bridge.OpLogicalAnd, a, b)
}
func (f *Function) LogicalOr(a, b backends.Value) (backends.Value, error) {
	return f.binary("LogicalOr", bridge.OpLogicalOr, a, b)
}
func (f *Function) LogicalXor(a, b backends.Value) (backends.Value, error) {
	return f.binary("LogicalXor", bridge.OpLogicalXor, a, b)
}
func (f *Function) BitwiseAnd(a, b backends.Value) (backends.Value, error) {
	return f.binary("BitwiseAnd", bridge.OpBitwiseAnd, a, b)
}
func (f *Function) BitwiseOr(a, b backends.Value) (backends.Value, error) {
	return f.binary("BitwiseOr", bridge.OpBitwiseOr, a, b)
}
func (f *Function) BitwiseXor(a, b backends.Value) (backends.Value, error) {
	return f.binary("BitwiseXor", bridge.OpBitwiseXor, a, b)
}
func (f *Function) ShiftLeft(a, b backends.Value) (backends.Value, error) {
	return f.binary("ShiftLeft", bridge.OpShiftLeft, a, b)
}
func (f *Function) ShiftRightArithmetic(a, b backends.Value) (backends.Value, error) {
	return f.binary("ShiftRightArithmetic", bridge.OpShiftRightArithmetic, a, b)
}
func (f *Function) ShiftRightLogical(a, b backends.Value) (backends.Value, error) {
	return f.binary("ShiftRightLogical", bridge.OpShiftRightLogical, a, b)
}

func (f *Function) Equal(a, b backends.Value) (backends.Value, error) { return f.binary("Equal", bridge.OpEqual, a, b) }
func (f *Function) NotEqual(a, b backends.Value) (backends.Value, error) {
	return f.binary("NotEqual", bridge.OpNotEqual, a, b)
}
func (f *Function) LessThan(a, b backends.Value) (backends.Value, error) {
	return f.binary("LessThan", bridge.OpLessThan, a, b)
}
func (f *Function) LessOrEqual(a, b backends.Value) (backends.Value, error) {
	return f.binary("LessOrEqual", bridge.OpLessOrEqual, a, b)
}
func (f *Function) GreaterThan(a, b backends.Value) (backends.Value, error) {
	return f.binary("GreaterThan", bridge.OpGreaterThan, a, b)
}
func (f *Function) GreaterOrEqual(a, b backends.Value) (backends.Value, error) {
	return f.binary("GreaterOrEqual", bridge.OpGreaterOrEqual, a, b)
}

// The total-order compares delegate to the plain ones, as the reference's do (function.go:2234-2256).
func (f *Function) EqualTotalOrder(a, b backends.Value) (backends.Value, error)    { return f.Equal(a, b) }
func (f *Function) NotEqualTotalOrder(a, b backends.Value) (backends.Value, error) { return f.NotEqual(a, b) }
func (f *Function) LessThanTotalOrder(a, b backends.Value) (backends.Value, error) { return f.LessThan(a, b) }
func (f *Function) LessOrEqualTotalOrder(a, b backends.Value) (backends.Value, error) {
	return f.LessOrEqual(a, b)
}
func (f *Function) GreaterThanTotalOrder(a, b backends.Value) (backends.Value, error) {
	return f.GreaterThan(a, b)
}
func (f *Function) GreaterOrEqualTotalOrder(a, b backends.Value) (backends.Value, error) {
	return f.GreaterOrEqual(a, b)
}

// ---- shape ops (mpsgraph/gomlx/function.go:969-1135, 1533-1621) ----

func (f *Function) Reshape(x backends.Value, dimensions ...int) (backends.Value, error) {
	n, err := f.resolve("Reshape", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Reshape(n.value, dims64(dimensions))
	return f.wrap("Reshape", v, err)
}

func (f *Function) Transpose(x backends.Value, permutation ...int) (backends.Value, error) {
	n, err := f.resolve("Transpose", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Transpose(n.value, permutation)
	return f.wrap("Transpose", v, err)
}

func (f *Function) ConvertDType(x backends.Value, dtype dtypes.DType) (backends.Value, error) {
	n, err := f.resolve("ConvertDType", x)
	if err != nil {
		return nil, err
	}
	code, err := dtypeToBridge(dtype)
	if err != nil {
		return nil, errors.Wrap(err, "ConvertDType")
	}
	v, err := f.ctx().Cast(n.value, code)
	return f.wrap("ConvertDType", v, err)
}

func (f *Function) BroadcastInDim(x backends.Value, outputShape shapes.Shape, broadcastAxes []int) (backends.Value, error) {
	n, err := f.resolve("BroadcastInDim", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().BroadcastInDim(n.value, dims64(outputShape.Dimensions), broadcastAxes)
	return f.wrap("BroadcastInDim", v, err)
}

func (f *Function) Where(condition, onTrue, onFalse backends.Value) (backends.Value, error) {
	c, err := f.resolve("Where", condition)
	if err != nil {
		return nil, err
	}
	a, err := f.resolve("Where", onTrue)
	if err != nil {
		return nil, err
	}
	b, err := f.resolve("Where", onFalse)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Where(c.value, a.value, b.value)
	return f.wrap("Where", v, err)
}

func (f *Function) Clamp(min, x, max backends.Value) (backends.Value, error) {
	lo, err := f.resolve("Clamp", min)
	if err != nil {
		return nil, err
	}
	n, err := f.resolve("Clamp", x)
	if err != nil {
		return nil, err
	}
	hi, err := f.resolve("Clamp", max)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Clamp(lo.value, n.value, hi.value)
	return f.wrap("Clamp", v, err)
}

func (f *Function) Slice(operand backends.Value, starts, limits, strides []int) (backends.Value, error) {
	n, err := f.resolve("Slice", operand)
	if err != nil {
		return nil, err
	}
	st := strides
	if len(st) == 0 { // GoMLX passes nil for unit strides
		st = make([]int, len(starts))
		for i := range st {
			st[i] = 1
		}
	}
	v, err := f.ctx().Slice(n.value, dims64(starts), dims64(limits), dims64(st))
	return f.wrap("Slice", v, err)
}

func (f *Function) Concatenate(axis int, operands ...backends.Value) (backends.Value, error) {
	vals := make([]bridge.Value, len(operands))
	for i, o := range operands {
		n, err := f.resolve("Concatenate", o)
		if err != nil {
			return nil, errors.Wrapf(err, "operand #%d", i)
		}
		vals[i] = n.value
	}
	v, err := f.ctx().Concatenate(vals, axis)
	return f.wrap("Concatenate", v, err)
}

func (f *Function) Reverse(x backends.Value, axes ...int) (backends.Value, error) {
	n, err := f.resolve("Reverse", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Reverse(n.value, axes)
	return f.wrap("Reverse", v, err)
}

// Pad supports edge padding only, like the reference (interior padding is an error: function.go:1533-1565).
func (f *Function) Pad(operand, fillValue backends.Value, axesConfig ...backends.PadAxis) (backends.Value, error) {
	n, err := f.resolve("Pad", operand)
	if err != nil {
		return nil, err
	}
	fill, err := f.resolve("Pad", fillValue)
	if err != nil {
		return nil, err
	}
	before := make([]int64, n.shape.Rank())
	after := make([]int64, n.shape.Rank())
	for i, c := range axesConfig {
		if i >= n.shape.Rank() {
			return nil, errors.Errorf("Pad: %d axis configurations for a rank-%d operand", len(axesConfig), n.shape.Rank())
		}
		if c.Interior != 0 {
			return nil, errors.New("Pad: interior padding is not supported")
		}
		before[i], after[i] = int64(c.Start), int64(c.End)
	}
	v, err := f.ctx().Pad(n.value, fill.value, before, after)
	return f.wrap("Pad", v, err)
}

func (f *Function) startValues(op string, starts []backends.Value) ([]bridge.Value, error) {
	vals := make([]bridge.Value, len(starts))
	for i, s := range starts {
		n, err := f.resolve(op, s)
		if err != nil {
			return nil, errors.Wrapf(err, "start index #%d", i)
		}
		vals[i] = n.value
	}
	return vals, nil
}

func (f *Function) DynamicSlice(operand backends.Value, startIndices []backends.Value, sliceSizes []int) (backends.Value, error) {
	n, err := f.resolve("DynamicSlice", operand)
	if err != nil {
		return nil, err
	}
	starts, err := f.startValues("DynamicSlice", startIndices)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().DynamicSlice(n.value, starts, dims64(sliceSizes))
	return f.wrap("DynamicSlice", v, err)
}

func (f *Function) DynamicUpdateSlice(operand, update backends.Value, startIndices []backends.Value) (backends.Value, error) {
	n, err := f.resolve("DynamicUpdateSlice", operand)
	if err != nil {
		return nil, err
	}
	u, err := f.resolve("DynamicUpdateSlice", update)
	if err != nil {
		return nil, err
	}
	starts, err := f.startValues("DynamicUpdateSlice", startIndices)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().DynamicUpdateSlice(n.value, u.value, starts)
	return f.wrap("DynamicUpdateSlice", v, err)
}

// ---- contraction, reductions, indexing (dotgeneral.go:65-237, function.go:1147-1242, gather.go:24-641) ----

func (f *Function) DotGeneral(lhs backends.Value, lhsContractingAxes, lhsBatchAxes []int, rhs backends.Value,
	rhsContractingAxes, rhsBatchAxes []int, config backends.DotGeneralConfig) (backends.Value, error) {
	a, err := f.resolve("DotGeneral", lhs)
	if err != nil {
		return nil, err
	}
	b, err := f.resolve("DotGeneral", rhs)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().DotGeneral(a.value, lhsContractingAxes, lhsBatchAxes, b.value, rhsContractingAxes, rhsBatchAxes)
	return f.wrap("DotGeneral", v, err)
}

func (f *Function) reduce(op string, reduceType int, x backends.Value, axes []int) (backends.Value, error) {
	n, err := f.resolve(op, x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Reduce(n.value, reduceType, axes) // no axes = all axes (function.go:1153-1158)
	return f.wrap(op, v, err)
}

func (f *Function) ReduceSum(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceSum", bridge.ReduceSum, x, axes)
}
func (f *Function) ReduceProduct(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceProduct", bridge.ReduceProduct, x, axes)
}
func (f *Function) ReduceMax(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceMax", bridge.ReduceMax, x, axes)
}
func (f *Function) ReduceMin(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceMin", bridge.ReduceMin, x, axes)
}

// Logical reductions are min / max over Bool (function.go:2262-2270).
func (f *Function) ReduceLogicalAnd(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceLogicalAnd", bridge.ReduceMin, x, axes)
}
func (f *Function) ReduceLogicalOr(x backends.Value, axes ...int) (backends.Value, error) {
	return f.reduce("ReduceLogicalOr", bridge.ReduceMax, x, axes)
}

func (f *Function) ArgMinMax(x backends.Value, axis int, outputDType dtypes.DType, isMin bool) (backends.Value, error) {
	n, err := f.resolve("ArgMinMax", x)
	if err != nil {
		return nil, err
	}
	code, err := dtypeToBridge(outputDType)
	if err != nil {
		return nil, errors.Wrap(err, "ArgMinMax")
	}
	v, err := f.ctx().ArgMinMax(n.value, axis, code, isMin)
	return f.wrap("ArgMinMax", v, err)
}

func (f *Function) Gather(operand, startIndices backends.Value, indexVectorAxis int, offsetOutputAxes, collapsedSliceAxes,
	startIndexMap, sliceSizes []int, indicesAreSorted bool) (backends.Value, error) {
	o, err := f.resolve("Gather", operand)
	if err != nil {
		return nil, err
	}
	i, err := f.resolve("Gather", startIndices)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Gather(o.value, i.value, indexVectorAxis, offsetOutputAxes, collapsedSliceAxes, startIndexMap, dims64(sliceSizes),
		indicesAreSorted)
	return f.wrap("Gather", v, err)
}

func (f *Function) scatter(op string, mode int, operand, scatterIndices, updates backends.Value, indexVectorAxis int,
	updateWindowAxes, insertedWindowAxes, scatterAxesToOperandAxes []int, indicesAreSorted, uniqueIndices bool) (backends.Value, error) {
	o, err := f.resolve(op, operand)
	if err != nil {
		return nil, err
	}
	i, err := f.resolve(op, scatterIndices)
	if err != nil {
		return nil, err
	}
	u, err := f.resolve(op, updates)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Scatter(mode, o.value, i.value, u.value, indexVectorAxis, updateWindowAxes, insertedWindowAxes,
		scatterAxesToOperandAxes, indicesAreSorted, uniqueIndices)
	return f.wrap(op, v, err)
}

func (f *Function) ScatterSum(operand, scatterIndices, updates backends.Value, indexVectorAxis int,
	updateWindowAxes, insertedWindowAxes, scatterAxesToOperandAxes []int, indicesAreSorted, uniqueIndices bool) (backends.Value, error) {
	return f.scatter("ScatterSum", bridge.ScatterModeAdd, operand, scatterIndices, updates, indexVectorAxis, updateWindowAxes,
		insertedWindowAxes, scatterAxesToOperandAxes, indicesAreSorted, uniqueIndices)
}
func (f *Function) ScatterMax(operand, scatterIndices, updates backends.Value, indexVectorAxis int,
	updateWindowAxes, insertedWindowAxes, scatterAxesToOperandAxes []int, indicesAreSorted, uniqueIndices bool) (backends.Value, error) {
	return f.scatter("ScatterMax", bridge.ScatterModeMax, operand, scatterIndices, updates, indexVectorAxis, updateWindowAxes,
		insertedWindowAxes, scatterAxesToOperandAxes, indicesAreSorted, uniqueIndices)
}
func (f *Function) ScatterMin(operand, scatterIndices, updates backends.Value, indexVectorAxis int,
	updateWindowAxes, insertedWindowAxes, scatterAxesToOperandAxes []int, indicesAreSorted, uniqueIndices bool) (backends.Value, error) {
	return f.scatter("ScatterMin", bridge.ScatterModeMin, operand, scatterIndices, updates, indexVectorAxis, updateWindowAxes,
		insertedWindowAxes, scatterAxesToOperandAxes, indicesAreSorted, uniqueIndices)
}

// ---- fused ops: one native call each (the reference composes them from primitives, function.go:2276-3075) ----

func (f *Function) FusedSoftmax(x backends.Value, axis int) (backends.Value, error) {
	n, err := f.resolve("FusedSoftmax", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Softmax(n.value, axis)
	return f.wrap("FusedSoftmax", v, err)
}

func (f *Function) FusedGelu(x backends.Value, exact bool) (backends.Value, error) {
	n, err := f.resolve("FusedGelu", x)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().Gelu(n.value, exact)
	return f.wrap("FusedGelu", v, err)
}

func (f *Function) FusedLayerNorm(x backends.Value, axes []int, epsilon float64, gamma, beta backends.Value) (backends.Value, error) {
	n, err := f.resolve("FusedLayerNorm", x)
	if err != nil {
		return nil, err
	}
	g, err := f.optional("FusedLayerNorm", gamma)
	if err != nil {
		return nil, err
	}
	b, err := f.optional("FusedLayerNorm", beta)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().LayerNorm(n.value, axes, epsilon, g, b)
	return f.wrap("FusedLayerNorm", v, err)
}

// FusedRMSNorm is not part of GoMLX's interface today (models spell RMSNorm in primitives, which Compile recognises
// and turns into this op); it is exported for callers that want to name it.
func (f *Function) FusedRMSNorm(x backends.Value, axes []int, epsilon float64, gamma backends.Value) (backends.Value, error) {
	n, err := f.resolve("FusedRMSNorm", x)
	if err != nil {
		return nil, err
	}
	g, err := f.optional("FusedRMSNorm", gamma)
	if err != nil {
		return nil, err
	}
	v, err := f.ctx().RMSNorm(n.value, axes, epsilon, g)
	return f.wrap("FusedRMSNorm", v, err)
}

func (f *Function) FusedDense(x, weight, bias backends.Value, activation backends.ActivationType) (backends.Value, error) {
	n, err := f.resolve("FusedDense", x)
	if err != nil {
		return nil, err
	}
	w, err := f.resolve("FusedDense", weight)
	if err != nil {
		return nil, err
	}
	b, err := f.optional("FusedDense", bias)
	if err != nil {
		return nil, err
	}
	// backends.ActivationNone / Gelu / Relu / Silu / Tanh are 0..4, the C ABI's B200Activation (function.go:2624-2664)
	v, err := f.ctx().Dense(n.value, w.value, b, int(activation))
	return f.wrap("FusedDense", v, err)
}

func (f *Function) FusedAttentionQKVProjection(x, wQKV, biasQ, biasK, biasV backends.Value, queryDim, keyValueDim int) (
	query, key, value backends.Value, err error) {
	n, err := f.resolve("FusedAttentionQKVProjection", x)
	if err != nil {
		return nil, nil, nil, err
	}
	w, err := f.resolve("FusedAttentionQKVProjection", wQKV)
	if err != nil {
		return nil, nil, nil, err
	}
	var biases [3]bridge.Value
	for i, b := range []backends.Value{biasQ, biasK, biasV} {
		if biases[i], err = f.optional("FusedAttentionQKVProjection", b); err != nil {
			return nil, nil, nil, err
		}
	}
	q, k, v, err := f.ctx().AttentionQKVProjection(n.value, w.value, biases[0], biases[1], biases[2], queryDim, keyValueDim)
	if err != nil {
		return nil, nil, nil, errors.Wrap(err, "FusedAttentionQKVProjection")
	}
	if query, err = f.wrap("FusedAttentionQKVProjection", q, nil); err != nil {
		return nil, nil, nil, err
	}
	if key, err = f.wrap("FusedAttentionQKVProjection", k, nil); err != nil {
		return nil, nil, nil, err
	}
	value, err = f.wrap("FusedAttentionQKVProjection", v, nil)
	return query, key, value, err
}

func (f *Function) FusedScaledDotProductAttention(query, key, value, mask backends.Value, numHeads, numKVHeads int,
	axesLayout backends.AxesLayout, scale float64, causal bool, options *backends.ScaledDotProductAttentionConfig) (backends.Value, error) {
	q, err := f.resolve("FusedScaledDotProductAttention", query)
	if err != nil {
		return nil, err
	}
	k, err := f.resolve("FusedScaledDotProductAttention", key)
	if err != nil {
		return nil, err
	}
	v, err := f.resolve("FusedScaledDotProductAttention", value)
	if err != nil {
		return nil, err
	}
	m, err := f.optional("FusedScaledDotProductAttention", mask)
	if err != nil {
		return nil, err
	}
	// backends.AxesLayoutBHSD / BSHD map to B200_LAYOUT_BHSD (0) / B200_LAYOUT_BSHD (1)
	layout := 0
	if axesLayout == backends.AxesLayoutBSHD {
		layout = 1
	}
	out, err := f.ctx().ScaledDotProductAttention(q.value, k.value, v.value, m, numHeads, numKVHeads, layout, scale, causal)
	return f.wrap("FusedScaledDotProductAttention", out, err)
}

// ---- batch norm, random bits (function.go:1248-1527, 1627-1692) ----

func (f *Function) BatchNormForInference(operand, scale, offset, mean, variance backends.Value, epsilon float32, featureAxis int) (backends.Value, error) {
	ns := make([]*node, 5)
	for i, v := range []backends.Value{operand, scale, offset, mean, variance} {
		n, err := f.resolve("BatchNormForInference", v)
		if err != nil {
			return nil, err
		}
		ns[i] = n
	}
	v, err := f.ctx().BatchNormInference(ns[0].value, ns[3].value, ns[4].value, ns[1].value, ns[2].value, epsilon, featureAxis)
	return f.wrap("BatchNormForInference", v, err)
}

func (f *Function) BatchNormForTraining(operand, scale, offset backends.Value, epsilon float32, featureAxis int) (
	normalized, batchMean, batchVariance backends.Value, err error) {
	ns := make([]*node, 3)
	for i, v := range []backends.Value{operand, scale, offset} {
		if ns[i], err = f.resolve("BatchNormForTraining", v); err != nil {
			return nil, nil, nil, err
		}
	}
	y, m, v, err := f.ctx().BatchNormTraining(ns[0].value, ns[1].value, ns[2].value, epsilon, featureAxis)
	if err != nil {
		return nil, nil, nil, errors.Wrap(err, "BatchNormForTraining")
	}
	if normalized, err = f.wrap("BatchNormForTraining", y, nil); err != nil {
		return nil, nil, nil, err
	}
	if batchMean, err = f.wrap("BatchNormForTraining", m, nil); err != nil {
		return nil, nil, nil, err
	}
	batchVariance, err = f.wrap("BatchNormForTraining", v, nil)
	return normalized, batchMean, batchVariance, err
}

func (f *Function) BatchNormGradient(operand, scale, mean, variance, gradOutput backends.Value, epsilon float32, featureAxis int) (
	gradOperand, gradScale, gradOffset backends.Value, err error) {
	ns := make([]*node, 5)
	for i, v := range []backends.Value{operand, scale, mean, variance, gradOutput} {
		if ns[i], err = f.resolve("BatchNormGradient", v); err != nil {
			return nil, nil, nil, err
		}
	}
	gx, gs, gb, err := f.ctx().BatchNormGradient(ns[0].value, ns[1].value, ns[2].value, ns[3].value, ns[4].value, epsilon, featureAxis)
	if err != nil {
		return nil, nil, nil, errors.Wrap(err, "BatchNormGradient")
	}
	if gradOperand, err = f.wrap("BatchNormGradient", gx, nil); err != nil {
		return nil, nil, nil, err
	}
	if gradScale, err = f.wrap("BatchNormGradient", gs, nil); err != nil {
		return nil, nil, nil, err
	}
	gradOffset, err = f.wrap("BatchNormGradient", gb, nil)
	return gradOperand, gradScale, gradOffset, err
}

func (f *Function) RNGBitGenerator(state backends.Value, shape shapes.Shape) (newState, values backends.Value, err error) {
	s, err := f.resolve("RNGBitGenerator", state)
	if err != nil {
		return nil, nil, err
	}
	code, err := dtypeToBridge(shape.DType)
	if err != nil {
		return nil, nil, errors.Wrap(err, "RNGBitGenerator")
	}
	ns, v, err := f.ctx().RNGBitGenerator(s.value, code, dims64(shape.Dimensions))
	if err != nil {
		return nil, nil, errors.Wrap(err, "RNGBitGenerator")
	}
	if newState, err = f.wrap("RNGBitGenerator", ns, nil); err != nil {
		return nil, nil, err
	}
	values, err = f.wrap("RNGBitGenerator", v, nil)
	return newState, values, err
}

// ---- control flow over closures (mpsgraph/gomlx/function.go:354-652) ----
// Validation and messages follow the reference; unlike it there is no limit of one control-flow op per function.

func (f *Function) validateClosure(op, role string, fn backends.Function) (*Function, error) {
	c, ok := fn.(*Function)
	if !ok || c == nil {
		return nil, errors.Errorf("%s: %s must be a *b200.Function, got %T", op, role, fn)
	}
	if c.parent != f {
		return nil, errors.Errorf("%s: %s must be a closure of the current function", op, role)
	}
	if !c.returned {
		return nil, errors.Errorf("%s: %s must have Return() called", op, role)
	}
	return c, nil
}

func paramValues(c *Function) []bridge.Value {
	hs := make([]bridge.Value, len(c.params))
	for i, p := range c.params {
		hs[i] = p.value
	}
	return hs
}

func outputValues(c *Function) []bridge.Value {
	hs := make([]bridge.Value, len(c.outputs))
	for i, o := range c.outputs {
		hs[i] = o.value
	}
	return hs
}

func (f *Function) wrapAll(op string, vs []bridge.Value, err error) ([]backends.Value, error) {
	if err != nil {
		return nil, errors.Wrap(err, op)
	}
	out := make([]backends.Value, len(vs))
	for i, v := range vs {
		if out[i], err = f.wrap(op, v, nil); err != nil {
			return nil, err
		}
	}
	return out, nil
}

func (f *Function) Call(fn backends.Function, inputs ...backends.Value) ([]backends.Value, error) {
	ins, hs, err := f.resolveAll("Call", inputs)
	if err != nil {
		return nil, err
	}
	target, ok := fn.(*Function)
	if !ok || target == nil {
		return nil, errors.Errorf("Call: target must be *b200.Function, got %T", fn)
	}
	if target.builder != f.builder {
		return nil, errors.New("Call: target function must be from the same builder")
	}
	if !target.returned {
		return nil, errors.Errorf("Call: target function %q must have Return() called", target.name)
	}
	if len(ins) != len(target.params) {
		return nil, errors.Errorf("Call: function %q expects %d parameters, got %d inputs", target.name, len(target.params), len(ins))
	}
	for i, p := range target.params {
		if !p.shape.Equal(ins[i].shape) {
			return nil, errors.Errorf("Call: parameter %d shape mismatch: expected %s, got %s", i, p.shape, ins[i].shape)
		}
	}
	res, err := f.ctx().Call(paramValues(target), outputValues(target), hs)
	return f.wrapAll("Call", res, err)
}

func (f *Function) While(cond, body backends.Function, initialState ...backends.Value) ([]backends.Value, error) {
	if len(initialState) == 0 {
		return nil, errors.New("While: requires at least one initial state value")
	}
	state, hs, err := f.resolveAll("While", initialState)
	if err != nil {
		return nil, err
	}
	c, err := f.validateClosure("While", "cond", cond)
	if err != nil {
		return nil, err
	}
	b, err := f.validateClosure("While", "body", body)
	if err != nil {
		return nil, err
	}
	for _, role := range []struct {
		name string
		fn   *Function
	}{{"cond", c}, {"body", b}} {
		if len(role.fn.params) != len(state) {
			return nil, errors.Errorf("While: %s must have %d parameters, got %d", role.name, len(state), len(role.fn.params))
		}
		for i, p := range role.fn.params {
			if !p.shape.Equal(state[i].shape) {
				return nil, errors.Errorf("While: %s parameter %d shape %s doesn't match state shape %s", role.name, i, p.shape, state[i].shape)
			}
		}
	}
	if len(c.outputs) != 1 {
		return nil, errors.Errorf("While: cond must return exactly one value, got %d", len(c.outputs))
	}
	if c.outputs[0].shape.Rank() != 0 || c.outputs[0].shape.DType != dtypes.Bool {
		return nil, errors.Errorf("While: cond must return scalar bool, got %s", c.outputs[0].shape)
	}
	if len(b.outputs) != len(state) {
		return nil, errors.Errorf("While: body must return %d values, got %d", len(state), len(b.outputs))
	}
	for i, o := range b.outputs {
		if !o.shape.Equal(state[i].shape) {
			return nil, errors.Errorf("While: body output %d shape %s must match state shape %s", i, o.shape, state[i].shape)
		}
	}
	res, err := f.ctx().While(paramValues(c), c.outputs[0].value, paramValues(b), outputValues(b), hs)
	return f.wrapAll("While", res, err)
}

func (f *Function) If(pred backends.Value, trueBranch, falseBranch backends.Function) ([]backends.Value, error) {
	p, err := f.resolve("If: pred", pred)
	if err != nil {
		return nil, err
	}
	if p.shape.Rank() != 0 || p.shape.DType != dtypes.Bool {
		return nil, errors.Errorf("If: pred must be scalar bool, got %s", p.shape)
	}
	t, err := f.validateClosure("If", "trueBranch", trueBranch)
	if err != nil {
		return nil, err
	}
	e, err := f.validateClosure("If", "falseBranch", falseBranch)
	if err != nil {
		return nil, err
	}
	if len(t.params) != 0 {
		return nil, errors.Errorf("If: trueBranch must have no parameters, got %d", len(t.params))
	}
	if len(e.params) != 0 {
		return nil, errors.Errorf("If: falseBranch must have no parameters, got %d", len(e.params))
	}
	if len(t.outputs) != len(e.outputs) {
		return nil, errors.Errorf("If: branches must return same number of outputs (true=%d, false=%d)", len(t.outputs), len(e.outputs))
	}
	for i := range t.outputs {
		if !t.outputs[i].shape.Equal(e.outputs[i].shape) {
			return nil, errors.Errorf("If: output %d shapes must match (true=%s, false=%s)", i, t.outputs[i].shape, e.outputs[i].shape)
		}
	}
	res, err := f.ctx().If(p.value, outputValues(t), outputValues(e))
	return f.wrapAll("If", res, err)
}

func (f *Function) Sort(comparator backends.Function, axis int, isStable bool, inputs ...backends.Value) ([]backends.Value, error) {
	if len(inputs) == 0 {
		return nil, errors.New("Sort: requires at least one input tensor")
	}
	ins, hs, err := f.resolveAll("Sort", inputs)
	if err != nil {
		return nil, err
	}
	c, err := f.validateClosure("Sort", "comparator", comparator)
	if err != nil {
		return nil, err
	}
	first := ins[0].shape
	for i, n := range ins[1:] {
		if first.Rank() != n.shape.Rank() {
			return nil, errors.Errorf("Sort: all inputs must have same rank, input 0 rank=%d, input %d rank=%d", first.Rank(), i+1, n.shape.Rank())
		}
		for j := range first.Dimensions {
			if first.Dimensions[j] != n.shape.Dimensions[j] {
				return nil, errors.Errorf("Sort: all inputs must have same dimensions")
			}
		}
	}
	rank := first.Rank()
	if axis < 0 {
		axis += rank
	}
	if axis < 0 || axis >= rank {
		return nil, errors.Errorf("Sort: axis %d out of range for rank %d", axis, rank)
	}
	if len(c.params) != 2*len(ins) {
		return nil, errors.Errorf("Sort: comparator must have %d parameters, got %d", 2*len(ins), len(c.params))
	}
	for i, n := range ins {
		for j := 0; j < 2; j++ {
			p := c.params[2*i+j]
			if p.shape.Rank() != 0 {
				return nil, errors.Errorf("Sort: comparator parameter %d must be scalar, got %s", 2*i+j, p.shape)
			}
			if p.shape.DType != n.shape.DType {
				return nil, errors.Errorf("Sort: comparator parameter %d dtype %s must match input dtype %s", 2*i+j, p.shape.DType, n.shape.DType)
			}
		}
	}
	if len(c.outputs) != 1 {
		return nil, errors.Errorf("Sort: comparator must return exactly one value, got %d", len(c.outputs))
	}
	if c.outputs[0].shape.Rank() != 0 || c.outputs[0].shape.DType != dtypes.Bool {
		return nil, errors.Errorf("Sort: comparator must return scalar bool, got %s", c.outputs[0].shape)
	}
	res, err := f.ctx().Sort(paramValues(c), c.outputs[0].value, axis, isStable, hs)
	return f.wrapAll("Sort", res, err)
}
