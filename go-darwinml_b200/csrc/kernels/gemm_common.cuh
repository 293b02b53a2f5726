// Epilogue pieces shared by the GEMM kernels.
#pragma once

#include <cuda_runtime.h>

#include "../../../include/b200mlx.h"

namespace b200 {
namespace k {

// Activations of FusedDense (ref function.go:2624-2664).  GELU is the tanh
// approximation with the reference's constants (function.go:2356-2407).
__device__ __forceinline__ float apply_activation(int act, float v) {
  switch (act) {
    case B200_ACT_GELU: return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    case B200_ACT_RELU: return fmaxf(v, 0.0f);
    case B200_ACT_SILU: return v / (1.0f + expf(-v));
    case B200_ACT_TANH: return tanhf(v);
    default: return v;
  }
}

}  // namespace k
}  // namespace b200
