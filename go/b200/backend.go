//go:build cgo && linux

package b200

import (
	"fmt"
	"strconv"
	"strings"
	"sync"

	"github.com/gomlx/go-darwinml/b200/internal/bridge"
	"github.com/gomlx/gomlx/backends"
	"github.com/gomlx/gomlx/pkg/core/shapes"
	"github.com/pkg/errors"
)

// Backend implements backends.Backend and backends.DataInterface (the reference: mpsgraph/gomlx/backend.go:22-167).
type Backend struct {
	mu         sync.Mutex
	device     int
	numDevices int
	finalized  bool
}

var _ backends.Backend = (*Backend)(nil)

// New parses "k=v,k=v"; the only key is device=<ordinal>.  Unknown keys are errors (the convention of the reference's
// second backend, coreml/gomlx/backend.go:61-71).  Fails when no CUDA device is usable: there is no CPU fallback.
func New(config string) (backends.Backend, error) {
	b := &Backend{}
	for _, item := range strings.Split(config, ",") {
		item = strings.TrimSpace(item)
		if item == "" {
			continue
		}
		k, v, _ := strings.Cut(item, "=")
		switch strings.TrimSpace(k) {
		case "device":
			n, err := strconv.Atoi(strings.TrimSpace(v))
			if err != nil {
				return nil, errors.Wrapf(err, "b200: bad device ordinal %q", v)
			}
			b.device = n
		default:
			return nil, errors.Errorf("b200: unknown backend option %q", k)
		}
	}
	n, err := bridge.DeviceCount()
	if err != nil {
		return nil, errors.Wrap(err, "b200: New")
	}
	if b.device >= n {
		return nil, errors.Errorf("b200: device %d requested but only %d visible", b.device, n)
	}
	b.numDevices = n
	return b, nil
}

func (b *Backend) Name() string        { return BackendName }
func (b *Backend) String() string      { return BackendName }
func (b *Backend) Description() string { return "B200 (sm_100a) native backend" }
func (b *Backend) NumDevices() int     { return b.numDevices }

func (b *Backend) DeviceDescription(deviceNum backends.DeviceNum) string {
	name, err := bridge.DeviceName(int(deviceNum))
	if err != nil {
		return fmt.Sprintf("cuda:%d", int(deviceNum))
	}
	return name
}

func (b *Backend) Capabilities() backends.Capabilities { return backendCapabilities }

// Builder panics on a finalized backend: graph building panics by GoMLX convention (mpsgraph/gomlx/backend.go:70-78).
func (b *Backend) Builder(name string) backends.Builder {
	b.mu.Lock()
	defer b.mu.Unlock()
	if b.finalized {
		panic(errors.New("b200: backend has been finalized"))
	}
	ctx, err := bridge.NewContext(b.device)
	if err != nil {
		panic(errors.Wrap(err, "b200: Builder"))
	}
	bld := &Builder{backend: b, name: name, ctx: ctx}
	bld.main = &Function{builder: bld, name: backends.MainName}
	return bld
}

// Finalize is idempotent (mpsgraph/gomlx/backend.go:80-92).  Device memory still held by live buffers and executables
// is released by their own Finalize calls.
func (b *Backend) Finalize() {
	b.mu.Lock()
	b.finalized = true
	b.mu.Unlock()
}

func (b *Backend) IsFinalized() bool {
	b.mu.Lock()
	defer b.mu.Unlock()
	return b.finalized
}

// ---- backends.DataInterface (mpsgraph/gomlx/backend.go:103-167) ----

func (b *Backend) BufferFinalize(buffer backends.Buffer) error {
	g, ok := buffer.(*Buffer)
	if !ok || g == nil {
		return errors.Errorf("BufferFinalize: buffer of type %T does not belong to the b200 backend", buffer)
	}
	if g.valid {
		bridge.BufferFree(g.handle)
		g.valid = false
	}
	return nil
}

func (b *Backend) BufferShape(buffer backends.Buffer) (shapes.Shape, error) {
	g, err := b.buffer(buffer, "BufferShape")
	if err != nil {
		return shapes.Shape{}, err
	}
	return g.shape, nil
}

func (b *Backend) BufferDeviceNum(buffer backends.Buffer) (backends.DeviceNum, error) {
	g, err := b.buffer(buffer, "BufferDeviceNum")
	if err != nil {
		return 0, err
	}
	return backends.DeviceNum(bridge.BufferDevice(g.handle)), nil
}

// BufferToFlatData waits for everything enqueued on the buffer's device and copies it into flat.
func (b *Backend) BufferToFlatData(buffer backends.Buffer, flat any) error {
	g, err := b.buffer(buffer, "BufferToFlatData")
	if err != nil {
		return err
	}
	ptr, nbytes, err := flatBytes(flat)
	if err != nil {
		return errors.Wrap(err, "BufferToFlatData")
	}
	if want := bridge.BufferBytes(g.handle); nbytes != want {
		return errors.Errorf("BufferToFlatData: flat holds %d bytes, buffer %s holds %d", nbytes, g.shape, want)
	}
	return errors.Wrap(bridge.BufferToHost(g.handle, ptr, nbytes), "BufferToFlatData")
}

func (b *Backend) BufferFromFlatData(deviceNum backends.DeviceNum, flat any, shape shapes.Shape) (backends.Buffer, error) {
	dt, err := dtypeToBridge(shape.DType)
	if err != nil {
		return nil, errors.Wrap(err, "BufferFromFlatData")
	}
	ptr, nbytes, err := flatBytes(flat)
	if err != nil {
		return nil, errors.Wrap(err, "BufferFromFlatData")
	}
	if want := int64(shape.Size()) * int64(shape.DType.Size()); nbytes != want {
		return nil, errors.Errorf("BufferFromFlatData: flat holds %d bytes, shape %s needs %d", nbytes, shape, want)
	}
	h, err := bridge.BufferFromHost(int(deviceNum), ptr, nbytes, dt, dims64(shape.Dimensions))
	if err != nil {
		return nil, errors.Wrap(err, "BufferFromFlatData")
	}
	return &Buffer{handle: h, shape: shape, valid: true}, nil
}

// HasSharedBuffers is false: buffers are device memory (the reference answers true because its buffers are Go slices,
// mpsgraph/gomlx/backend.go:144-153).  Callers must check it before using the two methods below.
func (b *Backend) HasSharedBuffers() bool { return false }

func (b *Backend) NewSharedBuffer(deviceNum backends.DeviceNum, shape shapes.Shape) (backends.Buffer, any, error) {
	return nil, nil, errors.New("NewSharedBuffer: the b200 backend has no shared buffers (HasSharedBuffers() is false)")
}

func (b *Backend) BufferData(buffer backends.Buffer) (any, error) {
	return nil, errors.New("BufferData: the b200 backend has no shared buffers (HasSharedBuffers() is false)")
}

// BufferCopyToDevice is a stream-ordered peer copy; the source may be finalized right after it returns.
func (b *Backend) BufferCopyToDevice(source backends.Buffer, deviceNum backends.DeviceNum) (backends.Buffer, error) {
	g, err := b.buffer(source, "BufferCopyToDevice")
	if err != nil {
		return nil, err
	}
	h, err := bridge.BufferCopyToDevice(g.handle, int(deviceNum))
	if err != nil {
		return nil, errors.Wrap(err, "BufferCopyToDevice")
	}
	return &Buffer{handle: h, shape: g.shape, valid: true}, nil
}
