// Helpers shared by the row kernels (softmax, LayerNorm, RMSNorm, arg-reduce):
// 128-bit vectorised streaming loads/stores, element conversion, and warp /
// row-group reductions by shuffle.
//
// A "row group" is the set of TPR threads (a power of two, 32..1024) that
// cooperate on one row.  TPR == 32 is one warp per row and needs no shared
// memory; larger groups reduce across their warps through shared memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace b200 {
namespace k {

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

// 16-byte payload, element-accessible after conversion to float.
struct alignas(16) Raw16 { uint32_t w[4]; };

__device__ __forceinline__ Raw16 ld_stream16(const void* p) {
  Raw16 r;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream16(void* p, const Raw16& r) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.w[0]), "r"(r.w[1]), "r"(r.w[2]), "r"(r.w[3]) : "memory");
}
__device__ __forceinline__ Raw16 ld_cached16(const void* p) {
  Raw16 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]) : "l"(p));
  return r;
}

// Unpack a 16-byte vector of T into VecOf<T>::N floats and back.
template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static constexpr int N = 4;
  __device__ __forceinline__ static void unpack(const Raw16& r, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(r.w[i]);
  }
  __device__ __forceinline__ static void pack(const float* f, Raw16& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r.w[i] = __float_as_uint(f[i]);
  }
  __device__ __forceinline__ static float load1(const float* p) { return *p; }
  __device__ __forceinline__ static void store1(float* p, float v) { *p = v; }
};
template <> struct Cvt<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(const Raw16& r, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(r.w[i] << 16);
      f[2 * i + 1] = __uint_as_float(r.w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ static void pack(const float* f, Raw16& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      r.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  __device__ __forceinline__ static float load1(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ __forceinline__ static void store1(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Cvt<__half> {
  static constexpr int N = 8;
  __device__ __forceinline__ static void unpack(const Raw16& r, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = *reinterpret_cast<const __half2*>(&r.w[i]);
      float2 v = __half22float2(h);
      f[2 * i] = v.x;
      f[2 * i + 1] = v.y;
    }
  }
  __device__ __forceinline__ static void pack(const float* f, Raw16& r) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      r.w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  __device__ __forceinline__ static float load1(const __half* p) { return __half2float(*p); }
  __device__ __forceinline__ static void store1(__half* p, float v) { *p = __float2half_rn(v); }
};

struct SumOp { __device__ __forceinline__ float operator()(float a, float b) const { return a + b; } };
struct MaxOp { __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); } };

template <typename F> __device__ __forceinline__ float warp_reduce(float v, F f) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Reduce over the TPR threads of a row group; every thread of the group gets
// the result.  `smem` must hold blockDim.x/32 floats and is reused between
// calls (two barriers per call when TPR > 32).
template <int TPR, typename F>
__device__ __forceinline__ float group_reduce(float v, F f, float identity, float* smem) {
  v = warp_reduce(v, f);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group_first_warp = (warp / WPR) * WPR;
    __syncthreads();  // previous use of smem is over
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = (lane < WPR) ? smem[group_first_warp + lane] : identity;
    v = warp_reduce(t, f);
  }
  return v;
}

}  // namespace k
}  // namespace b200
