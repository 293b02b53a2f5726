//go:build cgo && linux

package b200

import (
	"reflect"
	"unsafe"

	"github.com/gomlx/go-darwinml/b200/internal/bridge"
	"github.com/gomlx/gomlx/backends"
	"github.com/gomlx/gomlx/pkg/core/shapes"
	"github.com/gomlx/gopjrt/dtypes"
	"github.com/pkg/errors"
)

// Buffer is a device allocation owned by the caller until BufferFinalize (the reference's gpuBuffer is a Go slice:
// mpsgraph/gomlx/buffer.go:20-34).
type Buffer struct {
	handle bridge.Buffer
	shape  shapes.Shape
	valid  bool
}

var _ backends.Buffer = (*Buffer)(nil)

// dtypeToBridge maps a GoMLX dtype to the C ABI's enum; the numbers are the reference bridge's
// (mpsgraph/gomlx/buffer.go:90-119, internal/bridge/bridge.h:23-37).
func dtypeToBridge(dt dtypes.DType) (int, error) {
	switch dt {
	case dtypes.Bool:
		return bridge.DTypeBool, nil
	case dtypes.Int8:
		return bridge.DTypeInt8, nil
	case dtypes.Int16:
		return bridge.DTypeInt16, nil
	case dtypes.Int32:
		return bridge.DTypeInt32, nil
	case dtypes.Int64:
		return bridge.DTypeInt64, nil
	case dtypes.Float16:
		return bridge.DTypeFloat16, nil
	case dtypes.BFloat16:
		return bridge.DTypeBFloat16, nil
	case dtypes.Float32:
		return bridge.DTypeFloat32, nil
	case dtypes.Float64:
		return bridge.DTypeFloat64, nil
	case dtypes.Uint8:
		return bridge.DTypeUint8, nil
	case dtypes.Uint16:
		return bridge.DTypeUint16, nil
	case dtypes.Uint32:
		return bridge.DTypeUint32, nil
	case dtypes.Uint64:
		return bridge.DTypeUint64, nil
	}
	return 0, errors.Errorf("b200: unsupported dtype %s", dt)
}

func dims64(dims []int) []int64 {
	out := make([]int64, len(dims))
	for i, d := range dims {
		out[i] = int64(d)
	}
	return out
}

// flatBytes returns the address and byte length of a flat Go slice of a supported element type.
func flatBytes(flat any) (unsafe.Pointer, int64, error) {
	v := reflect.ValueOf(flat)
	if v.Kind() != reflect.Slice {
		return nil, 0, errors.Errorf("b200: flat data must be a slice, got %T", flat)
	}
	n := int64(v.Len()) * int64(v.Type().Elem().Size())
	if v.Len() == 0 {
		return nil, 0, nil
	}
	return v.UnsafePointer(), n, nil
}

func (b *Backend) buffer(buf backends.Buffer, what string) (*Buffer, error) {
	g, ok := buf.(*Buffer)
	if !ok || g == nil {
		return nil, errors.Errorf("%s: buffer of type %T does not belong to the b200 backend", what, buf)
	}
	if !g.valid {
		return nil, errors.Errorf("%s: buffer has been finalized", what)
	}
	return g, nil
}
