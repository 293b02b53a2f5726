//go:build cgo && linux

package b200

import (
	"sync"

	"github.com/gomlx/go-darwinml/b200/internal/bridge"
	"github.com/gomlx/gomlx/backends"
	"github.com/gomlx/gomlx/pkg/core/shapes"
	"github.com/pkg/errors"
)

// Executable is a compiled launch plan (the reference's: mpsgraph/gomlx/executable.go:18-112).
type Executable struct {
	builder      *Builder
	exec         bridge.Exec
	mu           sync.Mutex // Execute on one executable is serialised, as in the reference (executable.go:25, 51)
	inputNames   []string
	inputShapes  []shapes.Shape
	outputShapes []shapes.Shape
}

var _ backends.Executable = (*Executable)(nil)

func (e *Executable) Finalize() {
	e.mu.Lock()
	defer e.mu.Unlock()
	if e.exec != nil {
		e.exec.Destroy()
		e.exec = nil
	}
}

func (e *Executable) Inputs() ([]string, []shapes.Shape) { return e.inputNames, e.inputShapes }
func (e *Executable) Outputs() []shapes.Shape            { return e.outputShapes }

// Execute enqueues the plan on the device's stream and returns device buffers without waiting; the caller owns the
// outputs.  Inputs are validated by count, buffer type and shape (executable.go:55-75).  A donated input is consumed:
// when an output is DynamicUpdateSlice of it, the update happens in place (the reference accepts and ignores donate).
func (e *Executable) Execute(inputs []backends.Buffer, donate []bool, defaultDevice backends.DeviceNum) ([]backends.Buffer, error) {
	e.mu.Lock()
	defer e.mu.Unlock()
	if e.exec == nil {
		return nil, errors.New("b200: Execute on a finalized executable")
	}
	if len(inputs) != len(e.inputShapes) {
		return nil, errors.Errorf("b200: Execute expects %d inputs, got %d", len(e.inputShapes), len(inputs))
	}
	handles := make([]bridge.Buffer, len(inputs))
	for i, in := range inputs {
		g, err := e.builder.backend.buffer(in, "Execute")
		if err != nil {
			return nil, errors.Wrapf(err, "input #%d (%q)", i, e.inputNames[i])
		}
		if !g.shape.Equal(e.inputShapes[i]) {
			return nil, errors.Errorf("b200: Execute input #%d (%q) has shape %s, the executable was compiled for %s", i, e.inputNames[i], g.shape, e.inputShapes[i])
		}
		handles[i] = g.handle
	}
	anyDonated := false
	for _, d := range donate {
		anyDonated = anyDonated || d
	}
	var outs []bridge.Buffer
	var err error
	if anyDonated {
		outs, err = e.exec.ExecuteDonating(handles, donate, len(e.outputShapes))
	} else {
		outs, err = e.exec.Execute(handles, len(e.outputShapes))
	}
	if err != nil {
		return nil, errors.Wrap(err, "b200: Execute")
	}
	if anyDonated {
		for i, d := range donate {
			if d && i < len(inputs) {
				inputs[i].(*Buffer).valid = false // the native call finalized it
			}
		}
	}
	result := make([]backends.Buffer, len(outs))
	for i, h := range outs {
		result[i] = &Buffer{handle: h, shape: e.outputShapes[i], valid: true}
	}
	return result, nil
}
