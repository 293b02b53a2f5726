//go:build !(cgo && linux)

package b200

import (
	"github.com/gomlx/gomlx/backends"
	"github.com/pkg/errors"
)

// BackendName is the name the backend registers under where it can be built.
const BackendName = "b200"

// New fails on platforms without cgo or off Linux: the library is CUDA-only and has no CPU fallback (the reference's
// stub for non-darwin builds does the same: mpsgraph/gomlx/stub_other.go:17-20).
func New(config string) (backends.Backend, error) {
	return nil, errors.New("b200: this backend needs cgo on Linux with a CUDA device (there is no CPU fallback)")
}
