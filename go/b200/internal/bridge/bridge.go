//go:build cgo && linux

// Package bridge is the cgo layer over the C ABI of libb200mlx.so (include/b200mlx.h): one Go function per C entry
// point, Go errors from the {code, message} struct, no Go pointer kept by C after a call returns.  It replaces the
// reference's Objective-C bridge binding (mpsgraph/gomlx/internal/bridge/bridge.go:62-974).
//
// STATUS: written, not compiled (no Go toolchain where this library was built).
package bridge

/*
#cgo LDFLAGS: -lb200mlx
#include <stdlib.h>
#include "b200mlx.h"

// One dispatcher per op family keeps the Go side to one function per family.
typedef B200Value (*b200go_unary_fn)(B200Context, B200Value, B200Error*);
typedef B200Value (*b200go_binary_fn)(B200Context, B200Value, B200Value, B200Error*);
static const b200go_unary_fn b200go_unary_table[] = {
  b200_abs, b200_neg, b200_sqrt, b200_rsqrt, b200_exp, b200_expm1, b200_log, b200_log1p, b200_sin, b200_cos, b200_tanh,
  b200_sigmoid, b200_erf, b200_floor, b200_ceil, b200_round, b200_sign, b200_logical_not, b200_bitwise_not, b200_is_finite,
  b200_is_nan, b200_identity};
static const b200go_binary_fn b200go_binary_table[] = {
  b200_add, b200_sub, b200_mul, b200_div, b200_rem, b200_pow, b200_max, b200_min, b200_atan2, b200_logical_and,
  b200_logical_or, b200_logical_xor, b200_bitwise_and, b200_bitwise_or, b200_bitwise_xor, b200_shift_left, b200_shift_right,
  b200_shift_right_logical, b200_equal, b200_not_equal, b200_less_than, b200_less_or_equal, b200_greater_than,
  b200_greater_or_equal};
static B200Value b200go_unary(int op, B200Context c, B200Value x, B200Error* e) { return b200go_unary_table[op](c, x, e); }
static B200Value b200go_binary(int op, B200Context c, B200Value a, B200Value b, B200Error* e) { return b200go_binary_table[op](c, a, b, e); }
*/
import "C"

import (
	"fmt"
	"runtime"
	"unsafe"
)

// DType numbers of the C ABI (the reference bridge's: internal/bridge/bridge.h:23-37).
const (
	DTypeBool = iota
	DTypeInt8
	DTypeInt16
	DTypeInt32
	DTypeInt64
	DTypeFloat16
	DTypeBFloat16
	DTypeFloat32
	DTypeFloat64
	DTypeUint8
	DTypeUint16
	DTypeUint32
	DTypeUint64
)

// Unary and binary op codes: indexes into the dispatch tables of the cgo preamble.
const (
	OpAbs = iota
	OpNeg
	OpSqrt
	OpRsqrt
	OpExp
	OpExpm1
	OpLog
	OpLog1p
	OpSin
	OpCos
	OpTanh
	OpLogistic
	OpErf
	OpFloor
	OpCeil
	OpRound
	OpSign
	OpLogicalNot
	OpBitwiseNot
	OpIsFinite
	OpIsNaN
	OpIdentity
)
const (
	OpAdd = iota
	OpSub
	OpMul
	OpDiv
	OpRem
	OpPow
	OpMax
	OpMin
	OpAtan2
	OpLogicalAnd
	OpLogicalOr
	OpLogicalXor
	OpBitwiseAnd
	OpBitwiseOr
	OpBitwiseXor
	OpShiftLeft
	OpShiftRightArithmetic
	OpShiftRightLogical
	OpEqual
	OpNotEqual
	OpLessThan
	OpLessOrEqual
	OpGreaterThan
	OpGreaterOrEqual
)

const (
	ReduceSum = iota
	ReduceProduct
	ReduceMax
	ReduceMin
)

const (
	ScatterModeAdd = iota
	ScatterModeMax
	ScatterModeMin
)

// Error carries the C ABI's error code (B200ErrCode) and message.
type Error struct {
	Code    int
	Message string
}

func (e *Error) Error() string { return fmt.Sprintf("b200mlx error %d: %s", e.Code, e.Message) }

// takeError converts and frees a C error (the message is malloc'd: include/b200mlx.h, "caller frees").
func takeError(e *C.B200Error) error {
	if e.code == 0 {
		return nil
	}
	err := &Error{Code: int(e.code)}
	if e.message != nil {
		err.Message = C.GoString(e.message)
		C.free(unsafe.Pointer(e.message))
		e.message = nil
	}
	return err
}

// Value is a non-owning handle to a graph node, valid while its Context lives.  Buffer and Exec own native objects.
type (
	Value  = C.B200Value
	Buffer = C.B200Buffer
)

func i64ptr(s []int64) *C.int64_t {
	if len(s) == 0 {
		return nil
	}
	return (*C.int64_t)(unsafe.Pointer(&s[0]))
}
func intsToC(s []int) []C.int {
	out := make([]C.int, len(s))
	for i, v := range s {
		out[i] = C.int(v)
	}
	return out
}
func cintptr(s []C.int) *C.int {
	if len(s) == 0 {
		return nil
	}
	return &s[0]
}
func valptr(s []Value) *C.B200Value {
	if len(s) == 0 {
		return nil
	}
	return &s[0]
}

// ---- library / devices ----

func DeviceCount() (int, error) {
	var e C.B200Error
	n := C.b200_device_count(&e)
	if err := takeError(&e); err != nil {
		return 0, err
	}
	return int(n), nil
}

func DeviceName(device int) (string, error) {
	ctx, err := NewContext(device)
	if err != nil {
		return "", err
	}
	defer ctx.Destroy()
	p := C.b200_device_name(ctx.h)
	if p == nil {
		return "", nil
	}
	defer C.free(unsafe.Pointer(p))
	return C.GoString(p), nil
}

func DeviceSynchronize(device int) error {
	var e C.B200Error
	C.b200_device_synchronize(C.int(device), &e)
	return takeError(&e)
}

// ---- context: one graph under construction ----

type contextImpl struct{ h C.B200Context }

// Context is the graph-building handle; every op method returns a Value that belongs to it.
type Context = *contextImpl

func NewContext(device int) (Context, error) {
	var e C.B200Error
	h := C.b200_create_context(C.int(device), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return &contextImpl{h: h}, nil
}

func (c *contextImpl) Destroy() {
	if c.h != nil {
		C.b200_destroy_context(c.h)
		c.h = nil
	}
}

func (c *contextImpl) wrap(v C.B200Value, e *C.B200Error) (Value, error) {
	if err := takeError(e); err != nil {
		return nil, err
	}
	return v, nil
}

func (c *contextImpl) Placeholder(dtype int, dims []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_placeholder(c.h, C.int(dtype), i64ptr(dims), C.int(len(dims)), &e), &e)
}

// Constant copies nbytes at data into the graph (the callee copies: include/b200mlx.h).
func (c *contextImpl) Constant(data unsafe.Pointer, nbytes int64, dtype int, dims []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_constant(c.h, data, C.int64_t(nbytes), C.int(dtype), i64ptr(dims), C.int(len(dims)), &e), &e)
}

func (c *contextImpl) Iota(dtype int, dims []int64, axis int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_iota(c.h, C.int(dtype), i64ptr(dims), C.int(len(dims)), C.int(axis), &e), &e)
}

func (c *contextImpl) Unary(op int, x Value) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200go_unary(C.int(op), c.h, x, &e), &e)
}

func (c *contextImpl) Binary(op int, a, b Value) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200go_binary(C.int(op), c.h, a, b, &e), &e)
}

func (c *contextImpl) Reshape(x Value, dims []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_reshape(c.h, x, i64ptr(dims), C.int(len(dims)), &e), &e)
}

func (c *contextImpl) Transpose(x Value, perm []int) (Value, error) {
	var e C.B200Error
	p := intsToC(perm)
	return c.wrap(C.b200_transpose(c.h, x, cintptr(p), C.int(len(p)), &e), &e)
}

func (c *contextImpl) Cast(x Value, dtype int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_cast(c.h, x, C.int(dtype), &e), &e)
}

func (c *contextImpl) BroadcastInDim(x Value, dims []int64, axes []int) (Value, error) {
	var e C.B200Error
	a := intsToC(axes)
	return c.wrap(C.b200_broadcast_in_dim(c.h, x, i64ptr(dims), C.int(len(dims)), cintptr(a), C.int(len(a)), &e), &e)
}

func (c *contextImpl) Slice(x Value, starts, limits, strides []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_slice(c.h, x, i64ptr(starts), i64ptr(limits), i64ptr(strides), C.int(len(starts)), &e), &e)
}

func (c *contextImpl) Concatenate(xs []Value, axis int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_concatenate(c.h, valptr(xs), C.int(len(xs)), C.int(axis), &e), &e)
}

func (c *contextImpl) Reverse(x Value, axes []int) (Value, error) {
	var e C.B200Error
	a := intsToC(axes)
	return c.wrap(C.b200_reverse(c.h, x, cintptr(a), C.int(len(a)), &e), &e)
}

func (c *contextImpl) Pad(x, fill Value, before, after []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_pad(c.h, x, fill, i64ptr(before), i64ptr(after), C.int(len(before)), &e), &e)
}

func (c *contextImpl) DynamicSlice(x Value, starts []Value, sizes []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_dynamic_slice(c.h, x, valptr(starts), C.int(len(starts)), i64ptr(sizes), C.int(len(sizes)), &e), &e)
}

func (c *contextImpl) DynamicUpdateSlice(x, update Value, starts []Value) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_dynamic_update_slice(c.h, x, update, valptr(starts), C.int(len(starts)), &e), &e)
}

func (c *contextImpl) Where(cond, onTrue, onFalse Value) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_where(c.h, cond, onTrue, onFalse, &e), &e)
}

func (c *contextImpl) Clamp(lo, x, hi Value) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_clamp(c.h, lo, x, hi, &e), &e)
}

func (c *contextImpl) DotGeneral(lhs Value, lhsContracting, lhsBatch []int, rhs Value, rhsContracting, rhsBatch []int) (Value, error) {
	var e C.B200Error
	lc, lb, rc, rb := intsToC(lhsContracting), intsToC(lhsBatch), intsToC(rhsContracting), intsToC(rhsBatch)
	return c.wrap(C.b200_dot_general(c.h, lhs, cintptr(lc), C.int(len(lc)), cintptr(lb), C.int(len(lb)), rhs, cintptr(rc),
		C.int(len(rc)), cintptr(rb), C.int(len(rb)), &e), &e)
}

func (c *contextImpl) Reduce(x Value, reduceType int, axes []int) (Value, error) {
	var e C.B200Error
	a := intsToC(axes)
	return c.wrap(C.b200_reduce(c.h, x, C.int(reduceType), cintptr(a), C.int(len(a)), &e), &e)
}

func (c *contextImpl) ArgMinMax(x Value, axis, outDType int, isMin bool) (Value, error) {
	var e C.B200Error
	if isMin {
		return c.wrap(C.b200_argmin(c.h, x, C.int(axis), C.int(outDType), &e), &e)
	}
	return c.wrap(C.b200_argmax(c.h, x, C.int(axis), C.int(outDType), &e), &e)
}

func (c *contextImpl) Gather(operand, indices Value, indexVectorAxis int, offsetOutputAxes, collapsedSliceAxes, startIndexMap []int,
	sliceSizes []int64, sorted bool) (Value, error) {
	var e C.B200Error
	oo, cs, sm := intsToC(offsetOutputAxes), intsToC(collapsedSliceAxes), intsToC(startIndexMap)
	return c.wrap(C.b200_gather(c.h, operand, indices, C.int(indexVectorAxis), cintptr(oo), C.int(len(oo)), cintptr(cs), C.int(len(cs)),
		cintptr(sm), C.int(len(sm)), i64ptr(sliceSizes), C.int(len(sliceSizes)), C.bool(sorted), &e), &e)
}

func (c *contextImpl) Scatter(mode int, operand, indices, updates Value, indexVectorAxis int, updateWindowAxes, insertedWindowAxes,
	scatterAxesToOperandAxes []int, sorted, unique bool) (Value, error) {
	var e C.B200Error
	uw, iw, sa := intsToC(updateWindowAxes), intsToC(insertedWindowAxes), intsToC(scatterAxesToOperandAxes)
	return c.wrap(C.b200_scatter(c.h, C.int(mode), operand, indices, updates, C.int(indexVectorAxis), cintptr(uw), C.int(len(uw)),
		cintptr(iw), C.int(len(iw)), cintptr(sa), C.int(len(sa)), C.bool(sorted), C.bool(unique), &e), &e)
}

func (c *contextImpl) Softmax(x Value, axis int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_softmax(c.h, x, C.int(axis), &e), &e)
}

func (c *contextImpl) Gelu(x Value, exact bool) (Value, error) {
	var e C.B200Error
	ex := 0
	if exact {
		ex = 1
	}
	return c.wrap(C.b200_gelu(c.h, x, C.int(ex), &e), &e)
}

func (c *contextImpl) LayerNorm(x Value, axes []int, epsilon float64, gamma, beta Value) (Value, error) {
	var e C.B200Error
	a := intsToC(axes)
	return c.wrap(C.b200_layer_norm(c.h, x, cintptr(a), C.int(len(a)), C.double(epsilon), gamma, beta, &e), &e)
}

func (c *contextImpl) RMSNorm(x Value, axes []int, epsilon float64, gamma Value) (Value, error) {
	var e C.B200Error
	a := intsToC(axes)
	return c.wrap(C.b200_rms_norm(c.h, x, cintptr(a), C.int(len(a)), C.double(epsilon), gamma, &e), &e)
}

func (c *contextImpl) Dense(x, weight, bias Value, activation int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_dense(c.h, x, weight, bias, C.int(activation), &e), &e)
}

func (c *contextImpl) AttentionQKVProjection(x, wQKV, biasQ, biasK, biasV Value, queryDim, keyValueDim int) (q, k, v Value, err error) {
	var e C.B200Error
	C.b200_attention_qkv_projection(c.h, x, wQKV, biasQ, biasK, biasV, C.int(queryDim), C.int(keyValueDim), &q, &k, &v, &e)
	return q, k, v, takeError(&e)
}

func (c *contextImpl) ScaledDotProductAttention(q, k, v, mask Value, numHeads, numKVHeads, layout int, scale float64, causal bool) (Value, error) {
	var e C.B200Error
	ca := 0
	if causal {
		ca = 1
	}
	return c.wrap(C.b200_scaled_dot_product_attention(c.h, q, k, v, mask, C.int(numHeads), C.int(numKVHeads), C.int(layout), C.double(scale),
		C.int(ca), &e), &e)
}

func (c *contextImpl) BatchNormInference(x, mean, variance, scale, offset Value, epsilon float32, featureAxis int) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_batch_norm_inference(c.h, x, mean, variance, scale, offset, C.float(epsilon), C.int(featureAxis), &e), &e)
}

func (c *contextImpl) BatchNormTraining(x, scale, offset Value, epsilon float32, featureAxis int) (y, mean, variance Value, err error) {
	var e C.B200Error
	C.b200_batch_norm_training(c.h, x, scale, offset, C.float(epsilon), C.int(featureAxis), &y, &mean, &variance, &e)
	return y, mean, variance, takeError(&e)
}

func (c *contextImpl) BatchNormGradient(x, scale, mean, variance, gradOutput Value, epsilon float32, featureAxis int) (gx, gs, go_ Value, err error) {
	var e C.B200Error
	C.b200_batch_norm_gradient(c.h, x, scale, mean, variance, gradOutput, C.float(epsilon), C.int(featureAxis), &gx, &gs, &go_, &e)
	return gx, gs, go_, takeError(&e)
}

func (c *contextImpl) RNGBitGenerator(state Value, dtype int, dims []int64) (newState, values Value, err error) {
	var e C.B200Error
	C.b200_rng_bit_generator(c.h, state, C.int(dtype), i64ptr(dims), C.int(len(dims)), &newState, &values, &e)
	return newState, values, takeError(&e)
}

// ---- control flow over closures ----

// ClosureParameter is a parameter of a closure or of a named sub-function (built in the same context as its parent).
func (c *contextImpl) ClosureParameter(dtype int, dims []int64) (Value, error) {
	var e C.B200Error
	return c.wrap(C.b200_closure_parameter(c.h, C.int(dtype), i64ptr(dims), C.int(len(dims)), &e), &e)
}

func (c *contextImpl) Call(params, outputs, inputs []Value) ([]Value, error) {
	var e C.B200Error
	results := make([]Value, len(outputs))
	C.b200_call(c.h, valptr(params), C.int(len(params)), valptr(outputs), C.int(len(outputs)), valptr(inputs), valptr(results), &e)
	return results, takeError(&e)
}

func (c *contextImpl) If(pred Value, trueOutputs, falseOutputs []Value) ([]Value, error) {
	var e C.B200Error
	results := make([]Value, len(trueOutputs))
	C.b200_if(c.h, pred, valptr(trueOutputs), valptr(falseOutputs), C.int(len(trueOutputs)), valptr(results), &e)
	return results, takeError(&e)
}

func (c *contextImpl) While(condParams []Value, condOutput Value, bodyParams, bodyOutputs, initialState []Value) ([]Value, error) {
	var e C.B200Error
	results := make([]Value, len(initialState))
	C.b200_while(c.h, valptr(condParams), condOutput, valptr(bodyParams), valptr(bodyOutputs), C.int(len(initialState)),
		valptr(initialState), valptr(results), &e)
	return results, takeError(&e)
}

func (c *contextImpl) Sort(comparatorParams []Value, comparatorOutput Value, axis int, isStable bool, inputs []Value) ([]Value, error) {
	var e C.B200Error
	results := make([]Value, len(inputs))
	C.b200_sort(c.h, valptr(comparatorParams), C.int(len(comparatorParams)), comparatorOutput, C.int(axis), C.bool(isStable),
		valptr(inputs), C.int(len(inputs)), valptr(results), &e)
	return results, takeError(&e)
}

// ---- compile / execute ----

type execImpl struct{ h C.B200Exec }

// Exec is a compiled launch plan.
type Exec = *execImpl

func (c *contextImpl) Compile(feeds, targets []Value) (Exec, error) {
	var e C.B200Error
	h := C.b200_compile(c.h, valptr(feeds), C.int(len(feeds)), valptr(targets), C.int(len(targets)), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return &execImpl{h: h}, nil
}

func (x *execImpl) Destroy() {
	if x.h != nil {
		C.b200_destroy_exec(x.h)
		x.h = nil
	}
}

func bufptr(s []Buffer) *C.B200Buffer {
	if len(s) == 0 {
		return nil
	}
	return &s[0]
}

// Execute enqueues the plan and returns device buffers the caller owns; it does not wait.  The goroutine stays on its OS
// thread for the call, as the reference's bridge does (bridge.go:844-845): the CUDA runtime's current device is per thread.
func (x *execImpl) Execute(inputs []Buffer, numOutputs int) ([]Buffer, error) {
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	outs := make([]Buffer, numOutputs)
	var e C.B200Error
	C.b200_execute(x.h, bufptr(inputs), C.int(len(inputs)), bufptr(outs), C.int(numOutputs), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return outs, nil
}

func (x *execImpl) ExecuteDonating(inputs []Buffer, donate []bool, numOutputs int) ([]Buffer, error) {
	runtime.LockOSThread()
	defer runtime.UnlockOSThread()
	flags := make([]C.uchar, len(inputs))
	for i := range inputs {
		if i < len(donate) && donate[i] {
			flags[i] = 1
		}
	}
	var fp *C.uchar
	if len(flags) > 0 {
		fp = &flags[0]
	}
	outs := make([]Buffer, numOutputs)
	var e C.B200Error
	C.b200_execute_donating(x.h, bufptr(inputs), fp, C.int(len(inputs)), bufptr(outs), C.int(numOutputs), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return outs, nil
}

// ---- buffers ----

func BufferFromHost(device int, data unsafe.Pointer, nbytes int64, dtype int, dims []int64) (Buffer, error) {
	var e C.B200Error
	h := C.b200_buffer_from_host(C.int(device), data, C.int64_t(nbytes), C.int(dtype), i64ptr(dims), C.int(len(dims)), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return h, nil
}

func BufferToHost(b Buffer, data unsafe.Pointer, nbytes int64) error {
	var e C.B200Error
	C.b200_buffer_to_host(b, data, C.int64_t(nbytes), &e)
	return takeError(&e)
}

func BufferCopyToDevice(b Buffer, device int) (Buffer, error) {
	var e C.B200Error
	h := C.b200_buffer_copy_to_device(b, C.int(device), &e)
	if err := takeError(&e); err != nil {
		return nil, err
	}
	return h, nil
}

func BufferFree(b Buffer)         { C.b200_buffer_free(b) }
func BufferBytes(b Buffer) int64  { return int64(C.b200_buffer_nbytes(b)) }
func BufferDevice(b Buffer) int   { return int(C.b200_buffer_device(b)) }

// ValueShape reads a graph node's dtype code and dims back from the native graph.
func ValueShape(v Value) (dtype int, dims []int) {
	var buf [16]C.int64_t
	r := int(C.b200_value_shape(v, &buf[0], 16))
	dims = make([]int, r)
	for i := 0; i < r; i++ {
		dims[i] = int(buf[i])
	}
	return int(C.b200_value_dtype(v)), dims
}
