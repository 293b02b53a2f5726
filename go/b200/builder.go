//go:build cgo && linux

package b200

import (
	"github.com/gomlx/go-darwinml/b200/internal/bridge"
	"github.com/gomlx/gomlx/backends"
	"github.com/gomlx/gomlx/backends/notimplemented"
	"github.com/gomlx/gomlx/pkg/core/shapes"
	"github.com/pkg/errors"
)

// Builder owns one graph under construction (one native context), like the reference's (mpsgraph/gomlx/builder.go:15-109).
type Builder struct {
	notimplemented.Builder

	backend  *Backend
	name     string
	ctx      bridge.Context
	main     *Function
	compiled bool
}

var _ backends.Builder = (*Builder)(nil)

func (b *Builder) Name() string            { return b.name }
func (b *Builder) Main() backends.Function { return b.main }

// NewFunction creates a named sub-function, the target of Call (mpsgraph/gomlx/builder.go:57-60).  It is built in the
// builder's own native context; Call inlines it.
func (b *Builder) NewFunction(name string) (backends.Function, error) {
	return &Function{builder: b, name: name, sub: true}, nil
}

func (b *Builder) OpShape(op backends.Value) (shapes.Shape, error) {
	n, ok := op.(*node)
	if !ok || n == nil {
		return shapes.Shape{}, errors.Errorf("OpShape: value of type %T does not belong to the b200 backend", op)
	}
	return n.shape, nil
}

// Compile errors if called twice, without a Return, or with no outputs (mpsgraph/gomlx/builder.go:72-81).
func (b *Builder) Compile() (backends.Executable, error) {
	if b.compiled {
		return nil, errors.New("b200: builder has already been compiled")
	}
	if !b.main.returned {
		return nil, errors.New("b200: Main function has no Return")
	}
	feeds := make([]bridge.Value, len(b.main.params))
	names := make([]string, len(b.main.params))
	inShapes := make([]shapes.Shape, len(b.main.params))
	for i, p := range b.main.params {
		feeds[i], names[i], inShapes[i] = p.value, p.name, p.shape
	}
	targets := make([]bridge.Value, len(b.main.outputs))
	outShapes := make([]shapes.Shape, len(b.main.outputs))
	for i, o := range b.main.outputs {
		targets[i], outShapes[i] = o.value, o.shape
	}
	exec, err := b.ctx.Compile(feeds, targets)
	if err != nil {
		return nil, errors.Wrap(err, "b200: Compile")
	}
	b.compiled = true
	return &Executable{builder: b, exec: exec, inputNames: names, inputShapes: inShapes, outputShapes: outShapes}, nil
}

// Finalize releases the native graph; executables compiled from it stay valid.
func (b *Builder) Finalize() {
	if b.ctx != nil {
		b.ctx.Destroy()
		b.ctx = nil
	}
}
