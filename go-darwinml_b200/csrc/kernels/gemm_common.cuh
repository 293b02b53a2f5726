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

// The same over a register array, with the switch hoisted out of the loop.  FAST selects the hardware tanh / exp
// approximations (relative error about 2^-11): enough when the result is rounded to a 16-bit float (2^-9), and it keeps
// the GEMM epilogue of a GELU layer shorter than its main loop.
template <int N, bool FAST>
__device__ __forceinline__ void apply_activation_n(int act, float* v) {
  auto fast_tanh = [](float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
  };
  switch (act) {
    case B200_ACT_GELU:
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float u = 0.7978845608028654f * (v[j] + 0.044715f * v[j] * v[j] * v[j]);
        v[j] = 0.5f * v[j] * (1.0f + (FAST ? fast_tanh(u) : tanhf(u)));
      }
      break;
    case B200_ACT_RELU:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = fmaxf(v[j], 0.0f);
      break;
    case B200_ACT_SILU:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = FAST ? __fdividef(v[j], 1.0f + __expf(-v[j])) : v[j] / (1.0f + expf(-v[j]));
      break;
    case B200_ACT_TANH:
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = FAST ? fast_tanh(v[j]) : tanhf(v[j]);
      break;
    default:
      break;
  }
}

}  // namespace k
}  // namespace b200
