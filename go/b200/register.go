//go:build cgo && linux

package b200

import "github.com/gomlx/gomlx/backends"

// BackendName is the name this backend registers under (the reference registers "mpsgraph": register_darwin.go:9-11).
const BackendName = "b200"

func init() {
	backends.Register(BackendName, New)
}
