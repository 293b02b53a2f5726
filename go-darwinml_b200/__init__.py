"""b200mlx: a B200-native GoMLX backend behind the reference's plugin surface.

The directory name carries a hyphen, so import it through the `go_darwinml_b200`
module at the repository root (a three-line loader), e.g.::

    import go_darwinml_b200 as b200
    backend = b200.New("")

Everything computes on the GPU through libb200mlx.so (csrc/); importing this
package without that library raises ImportError, and creating a backend without
a usable CUDA device raises BackendError.  There is no CPU path.
"""
from .backend import (ActivationGelu, ActivationNone, ActivationRelu, ActivationSilu, ActivationTanh, AxesLayoutBHSD,  # noqa: F401
                      AxesLayoutBSHD, Backend, BackendError, BackendName, Buffer, Builder, DType, Executable, Function, New,
                      Shape, Value, dtypes, shapes)
from ._lib import lib  # noqa: F401

lib()  # fail at import time when the CUDA library is missing
