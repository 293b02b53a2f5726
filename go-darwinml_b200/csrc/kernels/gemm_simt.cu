// SIMT GEMM for the shapes and types the tcgen05 kernel does not take: tiny or
// ragged problems (the reference's 2x3 . 3x2 style tests), F64 and integer
// contractions.  C[b, m, n] = sum_k A(b, m, k) * B(b, k, n) with arbitrary
// element strides, so all four operand-major combinations of DotGeneral
// (ref dotgeneral.go:100-148 materialises transposes instead) read in place.
// Floats accumulate in fp32 (F64 in f64), integers in their own width.
// 64x64 output tile per CTA, 4x4 outputs per thread, K stepped by 16 through
// shared memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../kernels.h"
#include "gemm_common.cuh"

namespace b200 {
namespace k {

namespace {

template <typename T> struct GAcc { using type = T; };
template <> struct GAcc<__nv_bfloat16> { using type = float; };
template <> struct GAcc<__half> { using type = float; };
template <> struct GAcc<int8_t> { using type = int32_t; };
template <> struct GAcc<int16_t> { using type = int32_t; };
template <> struct GAcc<uint8_t> { using type = uint32_t; };
template <> struct GAcc<uint16_t> { using type = uint32_t; };

template <typename T, typename A> __device__ __forceinline__ A g_load(const T* p) { return (A)(*p); }
template <> __device__ __forceinline__ float g_load<__nv_bfloat16, float>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float g_load<__half, float>(const __half* p) { return __half2float(*p); }
template <typename A, typename T> __device__ __forceinline__ void g_store(T* p, A v) { *p = (T)v; }
template <> __device__ __forceinline__ void g_store<float, __nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void g_store<float, __half>(__half* p, float v) { *p = __float2half_rn(v); }

struct SimtArgs {
  const void* a;
  const void* b;
  void* c;
  const void* bias;
  const void* residual;
  int residual_op;
  int64_t m, n, k, ldc;
  int64_t a_sm, a_sk, a_sb;  // element strides of A along m, k, batch
  int64_t b_sk, b_sn, b_sb;
  int activation;
};

template <typename T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtArgs g) {
  using A = typename GAcc<T>::type;
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ A sa[BK][BM + 1];
  __shared__ A sb[BK][BN + 1];
  const int64_t batch = blockIdx.z;
  const T* a = reinterpret_cast<const T*>(g.a) + batch * g.a_sb;
  const T* b = reinterpret_cast<const T*>(g.b) + batch * g.b_sb;
  T* c = reinterpret_cast<T*>(g.c) + batch * g.m * g.ldc;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  A acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (A)0;
  for (int64_t k0 = 0; k0 < g.k; k0 += BK) {
    // Each thread loads 4 elements of each tile.  Pick the thread->element map
    // so that the fastest-varying thread index follows the unit-stride axis.
#pragma unroll
    for (int l = 0; l < 4; ++l) {
      const int e = threadIdx.x + l * 256;  // 0..1023
      int mm, kk;
      if (g.a_sk == 1) { kk = e % BK; mm = e / BK; } else { mm = e % BM; kk = e / BM; }
      const int64_t gm = m0 + mm, gk = k0 + kk;
      sa[kk][mm] = (gm < g.m && gk < g.k) ? g_load<T, A>(a + gm * g.a_sm + gk * g.a_sk) : (A)0;
      int nn, kb;
      if (g.b_sk == 1) { kb = e % BK; nn = e / BK; } else { nn = e % BN; kb = e / BN; }
      const int64_t gn = n0 + nn, gkb = k0 + kb;
      sb[kb][nn] = (gn < g.n && gkb < g.k) ? g_load<T, A>(b + gkb * g.b_sk + gn * g.b_sn) : (A)0;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      A av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= g.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t gn = n0 + tx * 4 + j;
      if (gn >= g.n) continue;
      A v = acc[i][j];
      if constexpr (std::is_same<A, float>::value) {
        if (g.bias) v += g_load<T, A>(reinterpret_cast<const T*>(g.bias) + gn);
        v = apply_activation(g.activation, v);
      } else {
        if (g.bias) v += g_load<T, A>(reinterpret_cast<const T*>(g.bias) + gn);
      }
      if (g.residual) {
        // the sum is rounded to the storage type first, as a separate DotGeneral would have left it
        T t;
        g_store<A, T>(&t, v);
        const A rv = g_load<T, A>(reinterpret_cast<const T*>(g.residual) + (c - reinterpret_cast<T*>(g.c)) + gm * g.ldc + gn);
        v = g.residual_op ? g_load<T, A>(&t) * rv : g_load<T, A>(&t) + rv;
      }
      g_store<A, T>(c + gm * g.ldc + gn, v);
    }
  }
}

}  // namespace

Status gemm_simt(Device* dev, const GemmParams& p) {
  if (p.batch * p.m * p.n == 0) return Status::OK();
  SimtArgs g;
  g.a = p.a; g.b = p.b; g.c = p.c; g.bias = p.bias; g.residual = p.residual; g.residual_op = p.residual_op;
  g.m = p.m; g.n = p.n; g.k = p.k; g.ldc = p.ldc > 0 ? p.ldc : p.n;
  g.a_sm = p.a_k_major ? p.k : 1;
  g.a_sk = p.a_k_major ? 1 : p.m;
  g.b_sk = p.b_k_major ? 1 : p.n;
  g.b_sn = p.b_k_major ? p.k : 1;
  g.a_sb = p.a_batch_stride >= 0 ? p.a_batch_stride : p.m * p.k;
  g.b_sb = p.b_batch_stride >= 0 ? p.b_batch_stride : p.k * p.n;
  g.activation = p.activation;
  if (p.batch > 65535 || (p.m + 63) / 64 > 65535) return Status::Unsupported("gemm_simt: grid too large");
  if (p.activation != B200_ACT_NONE && !(p.dtype == B200_FLOAT32 || p.dtype == B200_BFLOAT16 || p.dtype == B200_FLOAT16))
    return Status::Unsupported("gemm: activation needs a 16/32-bit float type");
  B200_TRY(dev->MakeCurrent());
  dim3 grid((unsigned)((p.n + 63) / 64), (unsigned)((p.m + 63) / 64), (unsigned)p.batch);
  cudaStream_t s = dev->stream();
#define GCASE(DT, T) case DT: gemm_simt_kernel<T><<<grid, 256, 0, s>>>(g); break;
  switch (p.dtype) {
    GCASE(B200_FLOAT32, float) GCASE(B200_FLOAT64, double) GCASE(B200_BFLOAT16, __nv_bfloat16) GCASE(B200_FLOAT16, __half)
    GCASE(B200_INT8, int8_t) GCASE(B200_INT16, int16_t) GCASE(B200_INT32, int32_t) GCASE(B200_INT64, int64_t)
    GCASE(B200_UINT8, uint8_t) GCASE(B200_UINT16, uint16_t) GCASE(B200_UINT32, uint32_t) GCASE(B200_UINT64, uint64_t)
    default: return Status::Unsupported(strfmt("gemm: dtype %s", dtype_name(p.dtype)));
  }
#undef GCASE
  return dev->CheckLaunch("gemm_simt");
}

}  // namespace k
}  // namespace b200
