"""Host-side mirror of the reference's GoMLX plugin surface, over the C ABI.

The reference implements GoMLX's ``backends.Backend``, ``Builder``,
``Function`` and ``Executable`` in Go (mpsgraph/gomlx/backend.go, builder.go,
function.go, executable.go).  No Go toolchain exists where this library is
built, so this module restates that surface in Python with the SAME method
names, argument order, argument meaning and error behaviour, each method one
call into libb200mlx.so.  A Go plugin binds the identical C functions through
cgo; nothing below does any arithmetic itself.

Errors: every method raises ``BackendError`` carrying the C ABI's code and
message, where the Go methods return ``error``.  ``Backend.Builder`` never
fails softly, like the reference (backend.go:70-77 panics).
"""
from __future__ import annotations

import ctypes
import threading
from typing import List, Optional, Sequence

import numpy as np

from . import _lib

try:
    import ml_dtypes

    _BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover - ml_dtypes is present in the build image
    _BF16 = None

BackendName = "b200"  # ref backend.go:19 BackendName = "mpsgraph"


class BackendError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


class DType(int):
    """GoMLX dtypes with the numeric values of the bridge enum (ref bridge.h:23-37)."""

    _names = ["Bool", "Int8", "Int16", "Int32", "Int64", "Float16", "BFloat16", "Float32", "Float64", "Uint8", "Uint16",
              "Uint32", "Uint64"]

    def __repr__(self):
        return self._names[int(self)]

    @property
    def np(self) -> np.dtype:
        return _NP_OF[int(self)]

    @property
    def size(self) -> int:
        return self.np.itemsize


class dtypes:  # namespace, mirrors github.com/gomlx/gopjrt/dtypes names used by the reference
    Bool, Int8, Int16, Int32, Int64 = DType(0), DType(1), DType(2), DType(3), DType(4)
    Float16, BFloat16, Float32, Float64 = DType(5), DType(6), DType(7), DType(8)
    Uint8, Uint16, Uint32, Uint64 = DType(9), DType(10), DType(11), DType(12)

    @staticmethod
    def from_numpy(dt) -> DType:
        dt = np.dtype(dt)
        for k, v in _NP_OF.items():
            if v == dt:
                return DType(k)
        raise BackendError(1, f"unsupported numpy dtype {dt}")


_NP_OF = {
    0: np.dtype(np.bool_), 1: np.dtype(np.int8), 2: np.dtype(np.int16), 3: np.dtype(np.int32), 4: np.dtype(np.int64),
    5: np.dtype(np.float16), 6: _BF16, 7: np.dtype(np.float32), 8: np.dtype(np.float64), 9: np.dtype(np.uint8),
    10: np.dtype(np.uint16), 11: np.dtype(np.uint32), 12: np.dtype(np.uint64),
}


class Shape:
    """shapes.Shape: dtype + dimensions."""

    def __init__(self, dtype: DType, dims: Sequence[int]):
        self.DType = DType(dtype)
        self.Dimensions = [int(d) for d in dims]

    def Rank(self) -> int:
        return len(self.Dimensions)

    def Size(self) -> int:
        n = 1
        for d in self.Dimensions:
            n *= d
        return n

    def __eq__(self, other):
        return isinstance(other, Shape) and self.DType == other.DType and self.Dimensions == other.Dimensions

    def __repr__(self):
        return f"({self.DType!r}){self.Dimensions}"


class shapes:  # namespace
    @staticmethod
    def Make(dtype: DType, *dims: int) -> Shape:
        return Shape(dtype, dims)


# backends.ActivationType / AxesLayout / reduce types (ref function.go:2624-2664, 2699; bridge.h:40-45)
ActivationNone, ActivationGelu, ActivationRelu, ActivationSilu, ActivationTanh = 0, 1, 2, 3, 4
AxesLayoutBHSD, AxesLayoutBSHD = 0, 1
ReduceSum, ReduceProduct, ReduceMax, ReduceMin = 0, 1, 2, 3


def _i64(values) -> "ctypes.Array":
    vals = [int(v) for v in values]
    return (ctypes.c_int64 * max(len(vals), 1))(*vals)


def _i32(values) -> "ctypes.Array":
    vals = [int(v) for v in values]
    return (ctypes.c_int * max(len(vals), 1))(*vals)


def _check(err: "_lib.B200Error", what: str = ""):
    if err.code != 0:
        msg = _lib.lib().take_string(err.message)
        err.message = None
        raise BackendError(err.code, f"{what}: {msg}" if what else msg)


class Value:
    """backends.Value: an opaque graph node (ref function.go:32-37 graphNode)."""

    def __init__(self, handle, owner: "Function"):
        self.handle = handle
        self.owner = owner

    @property
    def shape(self) -> Shape:
        L = _lib.lib()
        dims = (ctypes.c_int64 * 16)()
        r = L.b200_value_shape(self.handle, dims, 16)
        return Shape(DType(L.b200_value_dtype(self.handle)), list(dims[:r]))


class Buffer:
    """backends.Buffer: a device allocation (ref buffer.go:20-31 gpuBuffer is a Go slice instead)."""

    def __init__(self, handle):
        self.handle = handle
        self.valid = True

    def _h(self):
        if not self.valid or not self.handle:
            raise BackendError(1, "buffer is nil or has been finalized")
        return self.handle


class Backend:
    """backends.Backend + backends.DataInterface (ref backend.go:22-167)."""

    def __init__(self, config: str = ""):
        self._L = _lib.lib()
        self._mu = threading.Lock()
        self._finalized = False
        self._device = 0
        # "k=v,k=v"; unknown keys are errors (the convention of the reference's second backend, coreml/gomlx/backend.go:61-71)
        for item in [c for c in config.split(",") if c.strip()]:
            k, _, v = item.partition("=")
            k = k.strip()
            if k == "device":
                self._device = int(v)
            else:
                raise BackendError(1, f"unknown backend option {k!r}")
        err = _lib.B200Error()
        n = self._L.b200_device_count(ctypes.byref(err))
        _check(err, "New")
        if self._device >= n:
            raise BackendError(1, f"device {self._device} requested but only {n} visible")
        self._num_devices = n

    # --- identity (ref backend.go:46-67) ---
    def Name(self) -> str:
        return BackendName

    def String(self) -> str:
        return BackendName

    def Description(self) -> str:
        return "B200 (sm_100a) native backend"

    def NumDevices(self) -> int:
        return self._num_devices

    def DeviceDescription(self, device_num: int) -> str:
        err = _lib.B200Error()
        ctx = self._L.b200_create_context(int(device_num), ctypes.byref(err))
        _check(err, "DeviceDescription")
        try:
            return self._L.take_string(self._L.b200_device_name(ctx))
        finally:
            self._L.b200_destroy_context(ctx)

    def Capabilities(self):
        from .capabilities import backend_capabilities

        return backend_capabilities()

    def Builder(self, name: str) -> "Builder":
        if self._finalized:
            raise BackendError(1, "backend has been finalized")
        return Builder(self, name, self._device)

    def Finalize(self):
        with self._mu:
            self._finalized = True  # idempotent (ref backend.go:80-92)

    def IsFinalized(self) -> bool:
        return self._finalized

    # --- DataInterface (ref backend.go:103-167) ---
    def BufferFinalize(self, buffer: Buffer):
        if buffer is None or not isinstance(buffer, Buffer):
            raise BackendError(1, "BufferFinalize: not a buffer of this backend")
        if buffer.valid:
            self._L.b200_buffer_free(buffer.handle)
            buffer.valid = False
            buffer.handle = None

    def BufferShape(self, buffer: Buffer) -> Shape:
        h = buffer._h()
        dims = (ctypes.c_int64 * 16)()
        r = self._L.b200_buffer_shape(h, dims, 16)
        return Shape(DType(self._L.b200_buffer_dtype(h)), list(dims[:r]))

    def BufferDeviceNum(self, buffer: Buffer) -> int:
        return self._L.b200_buffer_device(buffer._h())

    def BufferToFlatData(self, buffer: Buffer, flat: np.ndarray):
        h = buffer._h()
        shape = self.BufferShape(buffer)
        if not isinstance(flat, np.ndarray) or not flat.flags["C_CONTIGUOUS"]:
            raise BackendError(1, "BufferToFlatData: flat must be a contiguous numpy array")
        if flat.dtype != shape.DType.np or flat.size != max(shape.Size(), 1 if shape.Rank() == 0 else 0):
            raise BackendError(1, f"BufferToFlatData: flat is {flat.dtype}[{flat.size}], buffer is {shape}")
        err = _lib.B200Error()
        self._L.b200_buffer_to_host(h, flat.ctypes.data_as(ctypes.c_void_p), flat.nbytes, ctypes.byref(err))
        _check(err, "BufferToFlatData")

    def BufferFromFlatData(self, device_num: int, flat: np.ndarray, shape: Shape) -> Buffer:
        flat = np.ascontiguousarray(flat)
        if flat.dtype != shape.DType.np:
            raise BackendError(1, f"BufferFromFlatData: flat dtype {flat.dtype} does not match shape {shape}")
        if flat.size != shape.Size():
            raise BackendError(1, f"BufferFromFlatData: flat has {flat.size} elements, shape {shape} needs {shape.Size()}")
        err = _lib.B200Error()
        h = self._L.b200_buffer_from_host(int(device_num), flat.ctypes.data_as(ctypes.c_void_p), flat.nbytes, int(shape.DType),
                                          _i64(shape.Dimensions), shape.Rank(), ctypes.byref(err))
        _check(err, "BufferFromFlatData")
        return Buffer(h)

    def HasSharedBuffers(self) -> bool:
        return False  # buffers are device memory (the reference answers true: its buffers are Go slices, backend.go:144-153)

    def NewSharedBuffer(self, device_num: int, shape: Shape):
        raise BackendError(3, "NewSharedBuffer: this backend has no shared buffers (HasSharedBuffers() is false)")

    def BufferData(self, buffer: Buffer):
        raise BackendError(3, "BufferData: this backend has no shared buffers (HasSharedBuffers() is false)")

    def BufferCopyToDevice(self, source: Buffer, device_num: int) -> Buffer:
        err = _lib.B200Error()
        h = self._L.b200_buffer_copy_to_device(source._h(), int(device_num), ctypes.byref(err))
        _check(err, "BufferCopyToDevice")
        return Buffer(h)

    # --- not in the Go interface: conveniences the tests and benchmarks use ---
    def Synchronize(self, device_num: Optional[int] = None):
        err = _lib.B200Error()
        self._L.b200_device_synchronize(self._device if device_num is None else int(device_num), ctypes.byref(err))
        _check(err, "Synchronize")

    def FromNumpy(self, array: np.ndarray, device_num: Optional[int] = None) -> Buffer:
        array = np.asarray(array)  # (ascontiguousarray would turn a 0-d array into shape (1,))
        if not array.flags["C_CONTIGUOUS"]:
            array = array.copy()
        return self.BufferFromFlatData(self._device if device_num is None else device_num, array.reshape(-1),
                                       Shape(dtypes.from_numpy(array.dtype), array.shape))

    def ToNumpy(self, buffer: Buffer) -> np.ndarray:
        shape = self.BufferShape(buffer)
        out = np.empty(shape.Size(), dtype=shape.DType.np)
        self.BufferToFlatData(buffer, out)
        return out.reshape(shape.Dimensions)


def New(config: str = "") -> Backend:
    """ref backend.go:33-43.  Fails when no CUDA device is usable: there is no CPU fallback."""
    return Backend(config)


class Builder:
    """backends.Builder (ref builder.go:15-109)."""

    def __init__(self, backend: Backend, name: str, device: int):
        self.backend = backend
        self.name = name
        self._L = backend._L
        err = _lib.B200Error()
        self.ctx = self._L.b200_create_context(device, ctypes.byref(err))
        _check(err, f"Builder({name!r})")
        self._main: Optional[Function] = None
        self._compiled = False

    def Name(self) -> str:
        return self.name

    def Main(self) -> "Function":
        if self._main is None:
            self._main = Function(self, "main")
        return self._main

    def NewFunction(self, name: str) -> "Function":
        """A named sub-function, the target of Call (ref builder.go:57-60).  It is built in the builder's own context."""
        return Function(self, name, parent=None, is_main=False)

    def OpShape(self, value: Value) -> Shape:
        if not isinstance(value, Value) or value.owner.builder is not self:
            raise BackendError(1, "OpShape: value does not belong to this builder")
        return value.shape

    def Compile(self) -> "Executable":
        # same three refusals as ref builder.go:73-81
        if self._compiled:
            raise BackendError(1, "builder has already been compiled")
        if self._main is None:
            raise BackendError(1, "no main function defined")
        if self._main.outputs is None:
            raise BackendError(1, "main function has no outputs; call Return()")
        fn = self._main
        feeds = (ctypes.c_void_p * max(len(fn.params), 1))(*[p.handle for p in fn.params])
        targets = (ctypes.c_void_p * max(len(fn.outputs), 1))(*[o.handle for o in fn.outputs])
        err = _lib.B200Error()
        h = self._L.b200_compile(self.ctx, feeds, len(fn.params), targets, len(fn.outputs), ctypes.byref(err))
        _check(err, "Compile")
        self._compiled = True
        return Executable(self, h, list(fn.param_names), [p.shape for p in fn.params], [o.shape for o in fn.outputs])

    def Finalize(self):
        if self.ctx:
            self._L.b200_destroy_context(self.ctx)
            self.ctx = None


class Function:
    """backends.Function: one method per op (ref function.go, dotgeneral.go, gather.go)."""

    def __init__(self, builder: Builder, name: str, parent: Optional["Function"] = None, is_main: bool = True):
        self.builder = builder
        self.name = name
        self.parent = parent
        self.is_main = is_main
        self._L = builder._L
        self.params: List[Value] = []
        self.param_names: List[str] = []
        self.outputs: Optional[List[Value]] = None

    def Name(self) -> str:
        return self.name

    def Parent(self):
        return self.parent

    def Closure(self) -> "Function":
        """A closure of this function: the cond / body of While, a branch of If, the comparator of Sort (ref
        function.go:120-131).  It is built in the same context as its parent and captures the parent's values by using
        them; the reference gives each closure a context of its own and feeds captures through placeholders."""
        return Function(self.builder, "", parent=self, is_main=False)

    # -- helpers --
    def _h(self, v, what: str):
        # a closure may use its ancestors' values; other foreign values are refused, like resolveNode (ref function.go:179-195)
        if not isinstance(v, Value):
            raise BackendError(1, f"{what}: expected a Value of this backend, got {type(v).__name__}")
        if v.owner is self:
            return v.handle
        p = self.parent
        while p is not None:
            if v.owner is p:
                return v.handle
            p = p.parent
        raise BackendError(1, f"{what}: node from unrelated function scope")

    def _wrap(self, handle, err, what: str) -> Value:
        _check(err, what)
        return Value(handle, self)

    def _unary(self, cname: str, what: str, x) -> Value:
        err = _lib.B200Error()
        return self._wrap(getattr(self._L, cname)(self.builder.ctx, self._h(x, what), ctypes.byref(err)), err, what)

    def _binary(self, cname: str, what: str, lhs, rhs) -> Value:
        err = _lib.B200Error()
        return self._wrap(getattr(self._L, cname)(self.builder.ctx, self._h(lhs, what), self._h(rhs, what), ctypes.byref(err)), err, what)

    # -- leaves (ref function.go:288-351) --
    def Parameter(self, name: str, shape: Shape, sharding=None) -> Value:
        err = _lib.B200Error()
        make = self._L.b200_placeholder if self.is_main else self._L.b200_closure_parameter
        v = self._wrap(make(self.builder.ctx, int(shape.DType), _i64(shape.Dimensions), shape.Rank(), ctypes.byref(err)), err, "Parameter")
        self.params.append(v)
        self.param_names.append(name)
        return v

    def Constant(self, flat, *dims: int) -> Value:
        flat = np.ascontiguousarray(flat)
        dt = dtypes.from_numpy(flat.dtype)
        n = 1
        for d in dims:
            n *= d
        if flat.size != n:
            raise BackendError(1, f"Constant: flat has {flat.size} elements, dims {list(dims)} need {n}")
        err = _lib.B200Error()
        return self._wrap(self._L.b200_constant(self.builder.ctx, flat.ctypes.data_as(ctypes.c_void_p), flat.nbytes, int(dt), _i64(dims),
                                                len(dims), ctypes.byref(err)), err, "Constant")

    def Return(self, outputs: Sequence[Value], shardings=None):
        if len(outputs) == 0:
            raise BackendError(1, "Return: no outputs")
        for o in outputs:
            self._h(o, "Return")
        self.outputs = list(outputs)

    # -- control flow over closures (ref function.go:354-652) --
    def _closure(self, op: str, role: str, fn) -> "Function":
        # ref validateClosure, function.go:234-246
        if not isinstance(fn, Function):
            raise BackendError(1, f"{op}: {role} must be a Function of this backend, got {type(fn).__name__}")
        if fn.parent is not self:
            raise BackendError(1, f"{op}: {role} must be a closure of the current function")
        if fn.outputs is None:
            raise BackendError(1, f"{op}: {role} must have Return() called")
        return fn

    @staticmethod
    def _handles(values) -> "ctypes.Array":
        return (ctypes.c_void_p * max(len(values), 1))(*[v if isinstance(v, int) or v is None else v.handle for v in values])

    def Call(self, fn, *inputs) -> List[Value]:
        """ref function.go:354-403.  The callee is inlined where it is called."""
        hs = [self._h(v, "Call") for v in inputs]
        if not isinstance(fn, Function):
            raise BackendError(1, f"Call: target must be a Function of this backend, got {type(fn).__name__}")
        if fn.builder is not self.builder:
            raise BackendError(1, "Call: target function must be from the same builder")
        if fn.outputs is None:
            raise BackendError(1, f"Call: target function {fn.name!r} must have Return() called")
        if len(hs) != len(fn.params):
            raise BackendError(1, f"Call: function {fn.name!r} expects {len(fn.params)} parameters, got {len(hs)} inputs")
        for i, (p, v) in enumerate(zip(fn.params, inputs)):
            if p.shape != v.shape:
                raise BackendError(1, f"Call: parameter {i} shape mismatch: expected {p.shape}, got {v.shape}")
        n = len(fn.outputs)
        res = (ctypes.c_void_p * n)()
        err = _lib.B200Error()
        self._L.b200_call(self.builder.ctx, self._handles(fn.params), len(fn.params), self._handles(fn.outputs), n,
                          (ctypes.c_void_p * max(len(hs), 1))(*hs), res, ctypes.byref(err))
        _check(err, "Call")
        return [Value(res[i], self) for i in range(n)]

    def While(self, cond, body, *initial_state) -> List[Value]:
        """ref function.go:406-489: state -> cond(state) scalar bool, state -> body(state); returns the final state."""
        if len(initial_state) == 0:
            raise BackendError(1, "While: requires at least one initial state value")
        hs = [self._h(v, "While") for v in initial_state]
        c = self._closure("While", "cond", cond)
        b = self._closure("While", "body", body)
        n = len(hs)
        for role, fn in (("cond", c), ("body", b)):
            if len(fn.params) != n:
                raise BackendError(1, f"While: {role} must have {n} parameters, got {len(fn.params)}")
            for i, (p, v) in enumerate(zip(fn.params, initial_state)):
                if p.shape != v.shape:
                    raise BackendError(1, f"While: {role} parameter {i} shape {p.shape} doesn't match state shape {v.shape}")
        if len(c.outputs) != 1:
            raise BackendError(1, f"While: cond must return exactly one value, got {len(c.outputs)}")
        if c.outputs[0].shape.Rank() != 0 or c.outputs[0].shape.DType != dtypes.Bool:
            raise BackendError(1, f"While: cond must return scalar bool, got {c.outputs[0].shape}")
        if len(b.outputs) != n:
            raise BackendError(1, f"While: body must return {n} values, got {len(b.outputs)}")
        for i, (o, v) in enumerate(zip(b.outputs, initial_state)):
            if o.shape != v.shape:
                raise BackendError(1, f"While: body output {i} shape {o.shape} must match state shape {v.shape}")
        res = (ctypes.c_void_p * n)()
        err = _lib.B200Error()
        self._L.b200_while(self.builder.ctx, self._handles(c.params), c.outputs[0].handle, self._handles(b.params), self._handles(b.outputs), n,
                           (ctypes.c_void_p * n)(*hs), res, ctypes.byref(err))
        _check(err, "While")
        return [Value(res[i], self) for i in range(n)]

    def If(self, pred, true_branch, false_branch) -> List[Value]:
        """ref function.go:492-560.  Light branches are both evaluated (they are pure) and the outputs selected by pred; heavy
        ones (contractions, reductions, loops ...) become two sub-plans of which one runs."""
        ph = self._h(pred, "If: pred")
        if pred.shape.Rank() != 0 or pred.shape.DType != dtypes.Bool:
            raise BackendError(1, f"If: pred must be scalar bool, got {pred.shape}")
        t = self._closure("If", "trueBranch", true_branch)
        f = self._closure("If", "falseBranch", false_branch)
        if len(t.params) != 0:
            raise BackendError(1, f"If: trueBranch must have no parameters, got {len(t.params)}")
        if len(f.params) != 0:
            raise BackendError(1, f"If: falseBranch must have no parameters, got {len(f.params)}")
        if len(t.outputs) != len(f.outputs):
            raise BackendError(1, f"If: branches must return same number of outputs (true={len(t.outputs)}, false={len(f.outputs)})")
        for i, (a, b) in enumerate(zip(t.outputs, f.outputs)):
            if a.shape != b.shape:
                raise BackendError(1, f"If: output {i} shapes must match (true={a.shape}, false={b.shape})")
        n = len(t.outputs)
        res = (ctypes.c_void_p * n)()
        err = _lib.B200Error()
        self._L.b200_if(self.builder.ctx, ph, self._handles(t.outputs), self._handles(f.outputs), n, res, ctypes.byref(err))
        _check(err, "If")
        return [Value(res[i], self) for i in range(n)]

    def Sort(self, comparator, axis: int, is_stable: bool, *inputs) -> List[Value]:
        """ref function.go:563-652.  The comparator must order by the first input alone (LessThan / GreaterThan of its first
        two parameters, what GoMLX's Sort builds); every input is permuted alike.  Always stable; NaN keys sort last."""
        if len(inputs) == 0:
            raise BackendError(1, "Sort: requires at least one input tensor")
        hs = [self._h(v, "Sort") for v in inputs]
        c = self._closure("Sort", "comparator", comparator)
        first = inputs[0].shape
        for i, v in enumerate(inputs[1:]):
            if v.shape.Rank() != first.Rank():
                raise BackendError(1, f"Sort: all inputs must have same rank, input 0 rank={first.Rank()}, input {i + 1} rank={v.shape.Rank()}")
            if tuple(v.shape.Dimensions) != tuple(first.Dimensions):
                raise BackendError(1, "Sort: all inputs must have same dimensions")
        rank = first.Rank()
        a = axis + rank if axis < 0 else axis
        if a < 0 or a >= rank:
            raise BackendError(1, f"Sort: axis {axis} out of range for rank {rank}")
        if len(c.params) != 2 * len(inputs):
            raise BackendError(1, f"Sort: comparator must have {2 * len(inputs)} parameters, got {len(c.params)}")
        for i, v in enumerate(inputs):
            for j in range(2):
                p = c.params[2 * i + j]
                if p.shape.Rank() != 0:
                    raise BackendError(1, f"Sort: comparator parameter {2 * i + j} must be scalar, got {p.shape}")
                if p.shape.DType != v.shape.DType:
                    raise BackendError(1, f"Sort: comparator parameter {2 * i + j} dtype {p.shape.DType!r} must match input dtype {v.shape.DType!r}")
        if len(c.outputs) != 1:
            raise BackendError(1, f"Sort: comparator must return exactly one value, got {len(c.outputs)}")
        if c.outputs[0].shape.Rank() != 0 or c.outputs[0].shape.DType != dtypes.Bool:
            raise BackendError(1, f"Sort: comparator must return scalar bool, got {c.outputs[0].shape}")
        n = len(inputs)
        res = (ctypes.c_void_p * n)()
        err = _lib.B200Error()
        self._L.b200_sort(self.builder.ctx, self._handles(c.params), len(c.params), c.outputs[0].handle, a, bool(is_stable),
                          (ctypes.c_void_p * n)(*hs), n, res, ctypes.byref(err))
        _check(err, "Sort")
        return [Value(res[i], self) for i in range(n)]

    def Iota(self, shape: Shape, iota_axis: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_iota(self.builder.ctx, int(shape.DType), _i64(shape.Dimensions), shape.Rank(), int(iota_axis),
                                            ctypes.byref(err)), err, "Iota")

    # -- unary (ref function.go:658-790) --
    def Abs(self, x): return self._unary("b200_abs", "Abs", x)
    def Neg(self, x): return self._unary("b200_neg", "Neg", x)
    def Sqrt(self, x): return self._unary("b200_sqrt", "Sqrt", x)
    def Rsqrt(self, x): return self._unary("b200_rsqrt", "Rsqrt", x)
    def Exp(self, x): return self._unary("b200_exp", "Exp", x)
    def Expm1(self, x): return self._unary("b200_expm1", "Expm1", x)
    def Log(self, x): return self._unary("b200_log", "Log", x)
    def Log1p(self, x): return self._unary("b200_log1p", "Log1p", x)
    def Sin(self, x): return self._unary("b200_sin", "Sin", x)
    def Cos(self, x): return self._unary("b200_cos", "Cos", x)
    def Tanh(self, x): return self._unary("b200_tanh", "Tanh", x)
    def Logistic(self, x): return self._unary("b200_sigmoid", "Logistic", x)
    def Erf(self, x): return self._unary("b200_erf", "Erf", x)
    def Floor(self, x): return self._unary("b200_floor", "Floor", x)
    def Ceil(self, x): return self._unary("b200_ceil", "Ceil", x)
    def Round(self, x): return self._unary("b200_round", "Round", x)
    def Sign(self, x): return self._unary("b200_sign", "Sign", x)
    def LogicalNot(self, x): return self._unary("b200_logical_not", "LogicalNot", x)
    def BitwiseNot(self, x): return self._unary("b200_bitwise_not", "BitwiseNot", x)
    def IsFinite(self, x): return self._unary("b200_is_finite", "IsFinite", x)
    def IsNaN(self, x): return self._unary("b200_is_nan", "IsNaN", x)
    def Identity(self, x): return self._unary("b200_identity", "Identity", x)

    # -- binary (ref function.go:792-905) --
    def Add(self, a, b): return self._binary("b200_add", "Add", a, b)
    def Sub(self, a, b): return self._binary("b200_sub", "Sub", a, b)
    def Mul(self, a, b): return self._binary("b200_mul", "Mul", a, b)
    def Div(self, a, b): return self._binary("b200_div", "Div", a, b)
    def Rem(self, a, b): return self._binary("b200_rem", "Rem", a, b)
    def Pow(self, a, b): return self._binary("b200_pow", "Pow", a, b)
    def Max(self, a, b): return self._binary("b200_max", "Max", a, b)
    def Min(self, a, b): return self._binary("b200_min", "Min", a, b)
    def Atan2(self, a, b): return self._binary("b200_atan2", "Atan2", a, b)
    def LogicalAnd(self, a, b): return self._binary("b200_logical_and", "LogicalAnd", a, b)
    def LogicalOr(self, a, b): return self._binary("b200_logical_or", "LogicalOr", a, b)
    def LogicalXor(self, a, b): return self._binary("b200_logical_xor", "LogicalXor", a, b)
    def BitwiseAnd(self, a, b): return self._binary("b200_bitwise_and", "BitwiseAnd", a, b)
    def BitwiseOr(self, a, b): return self._binary("b200_bitwise_or", "BitwiseOr", a, b)
    def BitwiseXor(self, a, b): return self._binary("b200_bitwise_xor", "BitwiseXor", a, b)
    def ShiftLeft(self, a, b): return self._binary("b200_shift_left", "ShiftLeft", a, b)
    def ShiftRightArithmetic(self, a, b): return self._binary("b200_shift_right", "ShiftRightArithmetic", a, b)
    def ShiftRightLogical(self, a, b): return self._binary("b200_shift_right_logical", "ShiftRightLogical", a, b)

    # -- comparisons (ref function.go:907-963, 2234-2256: the TotalOrder forms delegate to the plain ones) --
    def Equal(self, a, b): return self._binary("b200_equal", "Equal", a, b)
    def NotEqual(self, a, b): return self._binary("b200_not_equal", "NotEqual", a, b)
    def LessThan(self, a, b): return self._binary("b200_less_than", "LessThan", a, b)
    def LessOrEqual(self, a, b): return self._binary("b200_less_or_equal", "LessOrEqual", a, b)
    def GreaterThan(self, a, b): return self._binary("b200_greater_than", "GreaterThan", a, b)
    def GreaterOrEqual(self, a, b): return self._binary("b200_greater_or_equal", "GreaterOrEqual", a, b)
    EqualTotalOrder, NotEqualTotalOrder = Equal, NotEqual
    LessThanTotalOrder, LessOrEqualTotalOrder = LessThan, LessOrEqual
    GreaterThanTotalOrder, GreaterOrEqualTotalOrder = GreaterThan, GreaterOrEqual

    # -- shape ops (ref function.go:969-1125) --
    def Reshape(self, x, *dims: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_reshape(self.builder.ctx, self._h(x, "Reshape"), _i64(dims), len(dims), ctypes.byref(err)), err, "Reshape")

    def Transpose(self, x, *permutation: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_transpose(self.builder.ctx, self._h(x, "Transpose"), _i32(permutation), len(permutation),
                                                 ctypes.byref(err)), err, "Transpose")

    def ConvertDType(self, x, dtype: DType) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_cast(self.builder.ctx, self._h(x, "ConvertDType"), int(dtype), ctypes.byref(err)), err, "ConvertDType")

    def BroadcastInDim(self, x, output_shape: Shape, broadcast_axes: Sequence[int]) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_broadcast_in_dim(self.builder.ctx, self._h(x, "BroadcastInDim"), _i64(output_shape.Dimensions),
                                                        output_shape.Rank(), _i32(broadcast_axes), len(broadcast_axes), ctypes.byref(err)),
                          err, "BroadcastInDim")

    def Slice(self, x, starts: Sequence[int], limits: Sequence[int], strides: Sequence[int]) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_slice(self.builder.ctx, self._h(x, "Slice"), _i64(starts), _i64(limits), _i64(strides), len(starts),
                                             ctypes.byref(err)), err, "Slice")

    def Concatenate(self, axis: int, *operands) -> Value:
        hs = (ctypes.c_void_p * max(len(operands), 1))(*[self._h(o, "Concatenate") for o in operands])
        err = _lib.B200Error()
        return self._wrap(self._L.b200_concatenate(self.builder.ctx, hs, len(operands), int(axis), ctypes.byref(err)), err, "Concatenate")

    def Reverse(self, x, *axes: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_reverse(self.builder.ctx, self._h(x, "Reverse"), _i32(axes), len(axes), ctypes.byref(err)), err, "Reverse")

    def Pad(self, x, fill_value, *axes_config: Sequence[int]) -> Value:
        """axes_config: per axis (Start, End, Interior) like backends.PadAxis (ref function.go:1533-1565); Interior must be 0."""
        for cfg in axes_config:
            if len(cfg) > 2 and cfg[2] != 0:
                raise BackendError(3, "Pad: interior padding is not supported")
        before = [c[0] for c in axes_config]
        after = [c[1] for c in axes_config]
        err = _lib.B200Error()
        return self._wrap(self._L.b200_pad(self.builder.ctx, self._h(x, "Pad"), self._h(fill_value, "Pad"), _i64(before), _i64(after),
                                           len(axes_config), ctypes.byref(err)), err, "Pad")

    def DynamicSlice(self, operand, start_indices: Sequence[Value], slice_sizes: Sequence[int]) -> Value:
        """Slice at start indices given as scalar integer Values, one per axis (ref function.go:1571-1594)."""
        err = _lib.B200Error()
        hs = [self._h(v, "DynamicSlice: start index") for v in start_indices]
        arr = (ctypes.c_void_p * max(len(hs), 1))(*hs)
        return self._wrap(self._L.b200_dynamic_slice(self.builder.ctx, self._h(operand, "DynamicSlice"), arr, len(hs), _i64(slice_sizes),
                                                     len(slice_sizes), ctypes.byref(err)), err, "DynamicSlice")

    def DynamicUpdateSlice(self, operand, update, start_indices: Sequence[Value]) -> Value:
        """operand with `update` written at the start indices (ref function.go:1596-1621)."""
        err = _lib.B200Error()
        hs = [self._h(v, "DynamicUpdateSlice: start index") for v in start_indices]
        arr = (ctypes.c_void_p * max(len(hs), 1))(*hs)
        return self._wrap(self._L.b200_dynamic_update_slice(self.builder.ctx, self._h(operand, "DynamicUpdateSlice"),
                                                            self._h(update, "DynamicUpdateSlice"), arr, len(hs), ctypes.byref(err)),
                          err, "DynamicUpdateSlice")

    def Where(self, condition, on_true, on_false) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_where(self.builder.ctx, self._h(condition, "Where"), self._h(on_true, "Where"), self._h(on_false, "Where"),
                                             ctypes.byref(err)), err, "Where")

    def Clamp(self, min_value, x, max_value) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_clamp(self.builder.ctx, self._h(min_value, "Clamp"), self._h(x, "Clamp"), self._h(max_value, "Clamp"),
                                             ctypes.byref(err)), err, "Clamp")

    # -- contraction (ref dotgeneral.go:65-69) --
    def DotGeneral(self, lhs, lhs_contracting_axes, lhs_batch_axes, rhs, rhs_contracting_axes, rhs_batch_axes, config=None) -> Value:
        lc, lb = list(lhs_contracting_axes or []), list(lhs_batch_axes or [])
        rc, rb = list(rhs_contracting_axes or []), list(rhs_batch_axes or [])
        err = _lib.B200Error()
        return self._wrap(self._L.b200_dot_general(self.builder.ctx, self._h(lhs, "DotGeneral: lhs"), _i32(lc), len(lc), _i32(lb), len(lb),
                                                   self._h(rhs, "DotGeneral: rhs"), _i32(rc), len(rc), _i32(rb), len(rb), ctypes.byref(err)),
                          err, "DotGeneral")

    # -- reductions (ref function.go:1147-1242, 2262-2270) --
    def _reduce(self, what: str, rt: int, x, axes) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_reduce(self.builder.ctx, self._h(x, what), rt, _i32(axes), len(axes), ctypes.byref(err)), err, what)

    def ReduceSum(self, x, *axes): return self._reduce("ReduceSum", ReduceSum, x, axes)
    def ReduceProduct(self, x, *axes): return self._reduce("ReduceProduct", ReduceProduct, x, axes)
    def ReduceMax(self, x, *axes): return self._reduce("ReduceMax", ReduceMax, x, axes)
    def ReduceMin(self, x, *axes): return self._reduce("ReduceMin", ReduceMin, x, axes)
    def ReduceLogicalAnd(self, x, *axes): return self._reduce("ReduceLogicalAnd", ReduceMin, x, axes)
    def ReduceLogicalOr(self, x, *axes): return self._reduce("ReduceLogicalOr", ReduceMax, x, axes)

    def ArgMinMax(self, x, axis: int, output_dtype: DType, is_min: bool) -> Value:
        err = _lib.B200Error()
        fn = self._L.b200_argmin if is_min else self._L.b200_argmax
        return self._wrap(fn(self.builder.ctx, self._h(x, "ArgMinMax"), int(axis), int(output_dtype), ctypes.byref(err)), err, "ArgMinMax")

    # -- gather (ref gather.go:24-29) --
    def Gather(self, operand, start_indices, index_vector_axis, offset_output_axes, collapsed_slice_axes, start_index_map, slice_sizes,
               indices_are_sorted=False) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_gather(self.builder.ctx, self._h(operand, "Gather: operand"), self._h(start_indices, "Gather: startIndices"),
                                              int(index_vector_axis), _i32(offset_output_axes), len(offset_output_axes),
                                              _i32(collapsed_slice_axes), len(collapsed_slice_axes), _i32(start_index_map),
                                              len(start_index_map), _i64(slice_sizes), len(slice_sizes), bool(indices_are_sorted),
                                              ctypes.byref(err)), err, "Gather")

    # -- fused ops (ref function.go:2276-3075) --
    def FusedSoftmax(self, x, axis: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_softmax(self.builder.ctx, self._h(x, "FusedSoftmax"), int(axis), ctypes.byref(err)), err, "FusedSoftmax")

    def FusedSoftmaxMasked(self, x, scale: float = 1.0, causal: bool = False, mask=None) -> Value:
        err = _lib.B200Error()
        mh = self._h(mask, "FusedSoftmaxMasked: mask") if mask is not None else None
        return self._wrap(self._L.b200_softmax_masked(self.builder.ctx, self._h(x, "FusedSoftmaxMasked"), float(scale), int(bool(causal)), mh,
                                                      ctypes.byref(err)), err, "FusedSoftmaxMasked")

    def FusedGelu(self, x, exact: bool) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_gelu(self.builder.ctx, self._h(x, "FusedGelu"), int(bool(exact)), ctypes.byref(err)), err, "FusedGelu")

    def FusedLayerNorm(self, x, axes: Sequence[int], epsilon: float, gamma=None, beta=None) -> Value:
        err = _lib.B200Error()
        gh = self._h(gamma, "FusedLayerNorm: gamma") if gamma is not None else None
        bh = self._h(beta, "FusedLayerNorm: beta") if beta is not None else None
        return self._wrap(self._L.b200_layer_norm(self.builder.ctx, self._h(x, "FusedLayerNorm"), _i32(axes), len(axes), float(epsilon), gh, bh,
                                                  ctypes.byref(err)), err, "FusedLayerNorm")

    def FusedRMSNorm(self, x, axes: Sequence[int], epsilon: float, gamma=None) -> Value:
        err = _lib.B200Error()
        gh = self._h(gamma, "FusedRMSNorm: gamma") if gamma is not None else None
        return self._wrap(self._L.b200_rms_norm(self.builder.ctx, self._h(x, "FusedRMSNorm"), _i32(axes), len(axes), float(epsilon), gh,
                                                ctypes.byref(err)), err, "FusedRMSNorm")

    def FusedDense(self, x, weight, bias, activation: int) -> Value:
        err = _lib.B200Error()
        bh = self._h(bias, "FusedDense: bias") if bias is not None else None
        return self._wrap(self._L.b200_dense(self.builder.ctx, self._h(x, "FusedDense: x"), self._h(weight, "FusedDense: weight"), bh,
                                             int(activation), ctypes.byref(err)), err, "FusedDense")

    def FusedAttentionQKVProjection(self, x, w_qkv, bias_q, bias_k, bias_v, query_dim: int, key_value_dim: int):
        err = _lib.B200Error()
        q, k, v = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        hb = [self._h(b, "FusedAttentionQKVProjection: bias") if b is not None else None for b in (bias_q, bias_k, bias_v)]
        self._L.b200_attention_qkv_projection(self.builder.ctx, self._h(x, "FusedAttentionQKVProjection: x"),
                                              self._h(w_qkv, "FusedAttentionQKVProjection: wQKV"), hb[0], hb[1], hb[2], int(query_dim),
                                              int(key_value_dim), ctypes.byref(q), ctypes.byref(k), ctypes.byref(v), ctypes.byref(err))
        _check(err, "FusedAttentionQKVProjection")
        return Value(q.value, self), Value(k.value, self), Value(v.value, self)

    def FusedScaledDotProductAttention(self, query, key, value, mask, num_heads: int, num_kv_heads: int, axes_layout: int, scale: float,
                                       causal: bool, options=None) -> Value:
        err = _lib.B200Error()
        mh = self._h(mask, "SDPA: mask") if mask is not None else None
        return self._wrap(self._L.b200_scaled_dot_product_attention(self.builder.ctx, self._h(query, "SDPA: query"), self._h(key, "SDPA: key"),
                                                                    self._h(value, "SDPA: value"), mh, int(num_heads), int(num_kv_heads),
                                                                    int(axes_layout), float(scale), int(bool(causal)), ctypes.byref(err)),
                          err, "SDPA")

    def BatchNormForInference(self, operand, scale, offset, mean, variance, epsilon: float, feature_axis: int) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_batch_norm_inference(self.builder.ctx, self._h(operand, "BatchNormForInference"),
                                                            self._h(mean, "BatchNormForInference"), self._h(variance, "BatchNormForInference"),
                                                            self._h(scale, "BatchNormForInference"), self._h(offset, "BatchNormForInference"),
                                                            float(epsilon), int(feature_axis), ctypes.byref(err)), err, "BatchNormForInference")

    # -- training-side ops (ref function.go:1263-1527, 1627-1692; gather.go:441-641) --
    def BatchNormForTraining(self, operand, scale, offset, epsilon: float, feature_axis: int):
        """Returns (normalized, batchMean, batchVariance) (ref function.go:1263-1375)."""
        err = _lib.B200Error()
        y, m, v = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        self._L.b200_batch_norm_training(self.builder.ctx, self._h(operand, "BatchNormForTraining: operand"),
                                         self._h(scale, "BatchNormForTraining: scale"), self._h(offset, "BatchNormForTraining: offset"),
                                         float(epsilon), int(feature_axis), ctypes.byref(y), ctypes.byref(m), ctypes.byref(v), ctypes.byref(err))
        _check(err, "BatchNormForTraining")
        return Value(y.value, self), Value(m.value, self), Value(v.value, self)

    def BatchNormGradient(self, operand, scale, mean, variance, grad_output, epsilon: float, feature_axis: int):
        """Returns (gradOperand, gradScale, gradOffset) (ref function.go:1377-1527)."""
        err = _lib.B200Error()
        a, b, c = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        self._L.b200_batch_norm_gradient(self.builder.ctx, self._h(operand, "BatchNormGradient: operand"), self._h(scale, "BatchNormGradient: scale"),
                                         self._h(mean, "BatchNormGradient: mean"), self._h(variance, "BatchNormGradient: variance"),
                                         self._h(grad_output, "BatchNormGradient: gradOutput"), float(epsilon), int(feature_axis),
                                         ctypes.byref(a), ctypes.byref(b), ctypes.byref(c), ctypes.byref(err))
        _check(err, "BatchNormGradient")
        return Value(a.value, self), Value(b.value, self), Value(c.value, self)

    def _scatter(self, what: str, mode: int, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                 scatter_axes_to_operand_axes, indices_are_sorted, unique_indices) -> Value:
        err = _lib.B200Error()
        return self._wrap(self._L.b200_scatter(self.builder.ctx, mode, self._h(operand, what + ": operand"), self._h(scatter_indices, what + ": indices"),
                                               self._h(updates, what + ": updates"), int(index_vector_axis), _i32(update_window_axes),
                                               len(update_window_axes), _i32(inserted_window_axes), len(inserted_window_axes),
                                               _i32(scatter_axes_to_operand_axes), len(scatter_axes_to_operand_axes), bool(indices_are_sorted),
                                               bool(unique_indices), ctypes.byref(err)), err, what)

    def ScatterSum(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False) -> Value:
        return self._scatter("ScatterSum", 0, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                             scatter_axes_to_operand_axes, indices_are_sorted, unique_indices)

    def ScatterMax(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False) -> Value:
        return self._scatter("ScatterMax", 1, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                             scatter_axes_to_operand_axes, indices_are_sorted, unique_indices)

    def ScatterMin(self, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                   scatter_axes_to_operand_axes, indices_are_sorted=False, unique_indices=False) -> Value:
        return self._scatter("ScatterMin", 2, operand, scatter_indices, updates, index_vector_axis, update_window_axes, inserted_window_axes,
                             scatter_axes_to_operand_axes, indices_are_sorted, unique_indices)

    def RNGBitGenerator(self, state, shape: Shape):
        """Returns (newState, values) (ref function.go:1627-1692); state is (Uint64)[3]."""
        err = _lib.B200Error()
        ns, v = ctypes.c_void_p(), ctypes.c_void_p()
        self._L.b200_rng_bit_generator(self.builder.ctx, self._h(state, "RNGBitGenerator: state"), int(shape.DType), _i64(shape.Dimensions),
                                       shape.Rank(), ctypes.byref(ns), ctypes.byref(v), ctypes.byref(err))
        _check(err, "RNGBitGenerator")
        return Value(ns.value, self), Value(v.value, self)


class Executable:
    """backends.Executable (ref executable.go:18-112)."""

    def __init__(self, builder: Builder, handle, input_names, input_shapes, output_shapes):
        self.builder = builder
        self._L = builder._L
        self.handle = handle
        self.input_names = input_names
        self.input_shapes = input_shapes
        self.output_shapes = output_shapes
        self._mu = threading.Lock()

    def Finalize(self):
        if self.handle:
            self._L.b200_destroy_exec(self.handle)
            self.handle = None

    def Inputs(self):
        return self.input_names, self.input_shapes

    def Outputs(self):
        return self.output_shapes

    def NumLaunches(self) -> int:
        return self._L.b200_exec_num_launches(self.handle)

    def Describe(self) -> str:
        n = self._L.b200_exec_describe(self.handle, None, 0)
        buf = ctypes.create_string_buffer(n + 1)
        self._L.b200_exec_describe(self.handle, ctypes.cast(buf, ctypes.c_void_p), n + 1)
        return buf.value.decode()

    def Execute(self, inputs: Sequence[Buffer], donate=None, default_device: int = 0) -> List[Buffer]:
        """Device buffers in, fresh device buffers out; enqueues and returns (no wait).  donate[i] hands input i to the
        call: it is finalized, and an output that is DynamicUpdateSlice of it is updated in place."""
        if self.handle is None:
            raise BackendError(1, "Execute: executable has been finalized")
        if len(inputs) != len(self.input_shapes):
            raise BackendError(1, f"Execute: expected {len(self.input_shapes)} inputs, got {len(inputs)}")
        hs = []
        for i, b in enumerate(inputs):
            if not isinstance(b, Buffer):
                raise BackendError(1, f"Execute: input #{i} is not a buffer of this backend")
            hs.append(b._h())
        ins = (ctypes.c_void_p * max(len(hs), 1))(*hs)
        outs = (ctypes.c_void_p * max(len(self.output_shapes), 1))()
        err = _lib.B200Error()
        flags = None
        if donate is not None and any(donate):
            if len(donate) != len(inputs):
                raise BackendError(1, f"Execute: {len(donate)} donate flags for {len(inputs)} inputs")
            flags = (ctypes.c_ubyte * max(len(hs), 1))(*[1 if d else 0 for d in donate])
        with self._mu:
            if flags is None:
                self._L.b200_execute(self.handle, ins, len(hs), outs, len(self.output_shapes), ctypes.byref(err))
            else:
                self._L.b200_execute_donating(self.handle, ins, flags, len(hs), outs, len(self.output_shapes), ctypes.byref(err))
        _check(err, "Execute")
        if flags is not None:
            for b, d in zip(inputs, donate):   # donated buffers were finalized by the call (ref backends.Executable.Execute's contract)
                if d and b.valid:
                    b.valid = False
                    b.handle = None
        return [Buffer(outs[i]) for i in range(len(self.output_shapes))]

    def ExecuteProfiled(self, inputs: Sequence[Buffer]):
        """Execute with every step of the launch plan timed by CUDA events; returns (outputs, report text)."""
        hs = [b._h() for b in inputs]
        ins = (ctypes.c_void_p * max(len(hs), 1))(*hs)
        outs = (ctypes.c_void_p * max(len(self.output_shapes), 1))()
        cap = 1 << 20
        buf = ctypes.create_string_buffer(cap)
        err = _lib.B200Error()
        with self._mu:
            self._L.b200_execute_profiled(self.handle, ins, len(hs), outs, len(self.output_shapes), ctypes.cast(buf, ctypes.c_void_p), cap,
                                          ctypes.byref(err))
        _check(err, "ExecuteProfiled")
        return [Buffer(outs[i]) for i in range(len(self.output_shapes))], buf.value.decode()

    def ExecuteHost(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        """Host arrays in, host arrays out, through b200_execute_host: the calling shape of the
        reference's native execute (ref bridge.h:167-172), copies and wait included."""
        n_in, n_out = len(self.input_shapes), len(self.output_shapes)
        if len(inputs) != n_in:
            raise BackendError(1, f"Execute: expected {n_in} inputs, got {len(inputs)}")
        arrs = [np.ascontiguousarray(a) for a in inputs]
        outs = [np.empty(max(s.Size(), 1) if s.Rank() == 0 else s.Size(), dtype=s.DType.np) for s in self.output_shapes]
        in_ptrs = (ctypes.c_void_p * max(n_in, 1))(*[a.ctypes.data for a in arrs])
        in_sizes = _i64([a.nbytes for a in arrs])
        in_dtypes = _i32([int(s.DType) for s in self.input_shapes])
        shape_arrays = [_i64(s.Dimensions) for s in self.input_shapes]
        in_shapes = (ctypes.POINTER(ctypes.c_int64) * max(n_in, 1))(*[ctypes.cast(a, ctypes.POINTER(ctypes.c_int64)) for a in shape_arrays])
        in_ranks = _i32([s.Rank() for s in self.input_shapes])
        out_ptrs = (ctypes.c_void_p * max(n_out, 1))(*[a.ctypes.data for a in outs])
        out_sizes = _i64([a.nbytes for a in outs])
        out_dtypes = _i32([int(s.DType) for s in self.output_shapes])
        oshape_arrays = [_i64(s.Dimensions) for s in self.output_shapes]
        out_shapes = (ctypes.POINTER(ctypes.c_int64) * max(n_out, 1))(*[ctypes.cast(a, ctypes.POINTER(ctypes.c_int64)) for a in oshape_arrays])
        out_ranks = _i32([s.Rank() for s in self.output_shapes])
        err = _lib.B200Error()
        with self._mu:
            self._L.b200_execute_host(self.handle, in_ptrs, in_sizes, in_dtypes, in_shapes, in_ranks, n_in, out_ptrs, out_sizes, out_dtypes,
                                      out_shapes, out_ranks, n_out, ctypes.byref(err))
        _check(err, "Execute")
        return [o.reshape(s.Dimensions) for o, s in zip(outs, self.output_shapes)]

    def ExecuteHostSliced(self, inputs: Sequence[np.ndarray], sliced: Sequence[bool], num_slices: int,
                          outputs: Optional[Sequence[np.ndarray]] = None) -> List[np.ndarray]:
        """Runs this executable (compiled for ONE slice) over `num_slices` leading-axis slices of host arrays through
        b200_execute_host_sliced: uploads, kernels and downloads of neighbouring slices overlap.  inputs[i] with
        sliced[i] has shape [num_slices * d0, d1, ...] for an executable input [d0, d1, ...]; the others are passed
        whole to every slice.  Returns (or fills `outputs` with) arrays of shape [num_slices * o0, o1, ...]."""
        n_in, n_out = len(self.input_shapes), len(self.output_shapes)
        if len(inputs) != n_in or len(sliced) != n_in:
            raise BackendError(1, f"ExecuteSliced: expected {n_in} inputs and flags, got {len(inputs)} and {len(sliced)}")
        if num_slices < 0:
            raise BackendError(1, "ExecuteSliced: negative slice count")
        arrs = [np.ascontiguousarray(a) for a in inputs]
        for i, (a, s, fl) in enumerate(zip(arrs, self.input_shapes, sliced)):
            want = s.Size() * s.DType.np.itemsize * (num_slices if fl else 1)
            if a.nbytes != want or a.dtype != s.DType.np:
                raise BackendError(1, f"ExecuteSliced: input {i} has {a.nbytes} bytes of {a.dtype}, expected {want} of {s.DType.np}")
            if fl and s.Rank() == 0:
                raise BackendError(1, f"ExecuteSliced: input {i} is a scalar and cannot be sliced")
        if outputs is None:
            outs = [np.empty((num_slices * s.Dimensions[0],) + tuple(s.Dimensions[1:]) if s.Rank() > 0 else (num_slices,), dtype=s.DType.np)
                    for s in self.output_shapes]
        else:
            outs = list(outputs)
            for j, (o, s) in enumerate(zip(outs, self.output_shapes)):
                if o.nbytes != num_slices * s.Size() * s.DType.np.itemsize or not o.flags.c_contiguous:
                    raise BackendError(1, f"ExecuteSliced: output {j} must be a contiguous array of {num_slices} slices")
        in_ptrs = (ctypes.c_void_p * max(n_in, 1))(*[a.ctypes.data for a in arrs])
        flags = _i32([1 if f else 0 for f in sliced])
        out_ptrs = (ctypes.c_void_p * max(n_out, 1))(*[a.ctypes.data for a in outs])
        err = _lib.B200Error()
        with self._mu:
            self._L.b200_execute_host_sliced(self.handle, in_ptrs, flags, n_in, out_ptrs, n_out, num_slices, ctypes.byref(err))
        _check(err, "ExecuteSliced")
        return outs
