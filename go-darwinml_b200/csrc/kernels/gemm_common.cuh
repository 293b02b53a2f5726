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
      if constexpr (FAST && N % 2 == 0) {
        // Two elements per instruction with the packed fp32 forms of sm_100 (mul / fma .f32x2): the GELU epilogue of a
        // short-K layer is bound by instruction issue, and this takes the arithmetic from ~8 to 2.5 instructions per
        // element beside the one tanh.approx.  u = x (c0 + c1 x^2), y = h + h tanh(u) with h = x / 2.
        const float2 c0 = make_float2(0.7978845608028654f, 0.7978845608028654f);
        const float2 c1 = make_float2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f);
        const float2 half2 = make_float2(0.5f, 0.5f);
#pragma unroll
        for (int j = 0; j < N; j += 2) {
          const float2 x = make_float2(v[j], v[j + 1]);
          const float2 u = __fmul2_rn(__ffma2_rn(__fmul2_rn(x, x), c1, c0), x);
          const float2 t = make_float2(fast_tanh(u.x), fast_tanh(u.y));
          const float2 h = __fmul2_rn(x, half2);
          const float2 y = __ffma2_rn(h, t, h);
          v[j] = y.x;
          v[j + 1] = y.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float u = 0.7978845608028654f * (v[j] + 0.044715f * v[j] * v[j] * v[j]);
          v[j] = 0.5f * v[j] * (1.0f + (FAST ? fast_tanh(u) : tanhf(u)));
        }
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
