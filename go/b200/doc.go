// Package b200 is the GoMLX backend plugin over libb200mlx.so: it registers under the name "b200" through a blank
// import and implements GoMLX's backends.Backend, backends.DataInterface, backends.Builder, backends.Function and
// backends.Executable on top of the C ABI declared in include/b200mlx.h.
//
// It plays the part mpsgraph/gomlx plays in gomlx/go-darwinml (register_darwin.go, backend.go, buffer.go,
// capabilities.go, builder.go, function.go, dotgeneral.go, gather.go, executable.go over internal/bridge), with two
// differences that follow from the C ABI: buffers are device allocations (HasSharedBuffers is false), and the fused
// ops are single calls instead of compositions of primitives.
//
// STATUS: written, not compiled.  The image this library was built in has no Go toolchain and no copy of
// github.com/gomlx/gomlx (the reference pins v0.26.1-0.20260223064152-358aaf0bc270), so these files have never been
// through `go build` or `go vet`: interface signatures are taken from the reference's implementing methods, which its
// compiler checked with `var _ backends.X = ...` assertions.  Everything with behaviour (shape inference, validation,
// lowering, memory planning, execution) lives behind the C ABI, where it is tested; the Python mirror
// go-darwinml_b200/backend.py drives exactly the calls made here, method for method.
//
// Use:
//
//	import _ "github.com/gomlx/go-darwinml/b200"   // or wherever this directory is vendored
//	backend, err := backends.NewWithConfig("b200:device=0")
//
// Build: CGO_CFLAGS=-I<repo>/include CGO_LDFLAGS="-L<repo>/go-darwinml_b200 -lb200mlx" go build ./...
package b200
