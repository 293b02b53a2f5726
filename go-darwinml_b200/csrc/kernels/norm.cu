// LayerNorm and RMSNorm row kernels.
//
//   LayerNorm: mu = sum(x)/n; d = x - mu; var = sum(d*d)/n (biased, two-pass);
//              y = d * rsqrt(var + eps) [* gamma] [+ beta]
//              (the formula of the reference's FusedLayerNorm lowering,
//              mpsgraph function.go:2430-2558, which spends ~12 graph ops on it)
//   RMSNorm:   y = x * rsqrt(sum(x*x)/n + eps) [* gamma]   (no reference counterpart)
//
// Statistics are accumulated in fp32 whatever the storage type; the result is
// rounded once.  One row group (32, 256 or 1024 threads) owns a row: the row is
// loaded once with 128-bit streaming loads, stays in registers as packed 16-byte
// vectors for all passes, reductions are warp shuffles, and it is stored once.
// HBM-bound: algorithmic bytes = 2 * rows * cols * sizeof(T) (+ gamma, beta once).
#include "../kernels.h"
#include "rowwise.cuh"

namespace b200 {
namespace k {

namespace {

struct NArgs {
  const void* x;
  const void* gamma;
  const void* beta;
  void* y;
  int64_t rows, cols;
  float eps;
};

template <typename T, int ITERS, int TPR, bool RMS>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256) norm_rows_kernel(const NArgs a) {
  constexpr int V = Cvt<T>::N;
  __shared__ float red[32];
  const int rows_per_cta = blockDim.x / TPR;
  int64_t row = (int64_t)blockIdx.x * rows_per_cta + threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const bool active = row < a.rows;
  if (!active) row = a.rows - 1;
  const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
  T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
  const float inv_n = 1.0f / (float)a.cols;

  Raw16 raw[ITERS];
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < a.cols) raw[it] = ld_stream16(xr + c0);
  }
  float mean = 0.f;
  if constexpr (!RMS) {
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int64_t c0 = (int64_t)(it * TPR + t) * V;
      if (c0 < a.cols) {
        float f[V];
        Cvt<T>::unpack(raw[it], f);
#pragma unroll
        for (int e = 0; e < V; ++e) s += f[e];
      }
    }
    mean = group_reduce<TPR>(s, SumOp(), 0.f, red) * inv_n;
  }
  float sq = 0.f;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < a.cols) {
      float f[V];
      Cvt<T>::unpack(raw[it], f);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float d = f[e] - mean;
        sq += d * d;
      }
    }
  }
  sq = group_reduce<TPR>(sq, SumOp(), 0.f, red);
  const float rstd = rsqrtf(sq * inv_n + a.eps);
  if (!active) return;
#pragma unroll
  for (int it = 0; it < ITERS; ++it) {
    const int64_t c0 = (int64_t)(it * TPR + t) * V;
    if (c0 < a.cols) {
      float f[V];
      Cvt<T>::unpack(raw[it], f);
#pragma unroll
      for (int e = 0; e < V; ++e) f[e] = (f[e] - mean) * rstd;
      if (a.gamma) {
        float g[V];
        Cvt<T>::unpack(ld_cached16(reinterpret_cast<const T*>(a.gamma) + c0), g);
#pragma unroll
        for (int e = 0; e < V; ++e) f[e] *= g[e];
      }
      if (!RMS && a.beta) {
        float b[V];
        Cvt<T>::unpack(ld_cached16(reinterpret_cast<const T*>(a.beta) + c0), b);
#pragma unroll
        for (int e = 0; e < V; ++e) f[e] += b[e];
      }
      Raw16 o;
      Cvt<T>::pack(f, o);
      st_stream16(yr + c0, o);
    }
  }
}

// Any cols / alignment: one CTA per row, three passes with scalar accesses.
template <typename T, bool RMS>
__global__ void __launch_bounds__(256) norm_generic_kernel(const NArgs a) {
  __shared__ float red[32];
  const int64_t row = blockIdx.x;
  const T* xr = reinterpret_cast<const T*>(a.x) + row * a.cols;
  T* yr = reinterpret_cast<T*>(a.y) + row * a.cols;
  const float inv_n = 1.0f / (float)a.cols;
  float mean = 0.f;
  if (!RMS) {
    float s = 0.f;
    for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) s += Cvt<T>::load1(xr + j);
    mean = group_reduce<256>(s, SumOp(), 0.f, red) * inv_n;
  }
  float sq = 0.f;
  for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) {
    const float d = Cvt<T>::load1(xr + j) - mean;
    sq += d * d;
  }
  sq = group_reduce<256>(sq, SumOp(), 0.f, red);
  const float rstd = rsqrtf(sq * inv_n + a.eps);
  for (int64_t j = threadIdx.x; j < a.cols; j += blockDim.x) {
    float v = (Cvt<T>::load1(xr + j) - mean) * rstd;
    if (a.gamma) v *= Cvt<T>::load1(reinterpret_cast<const T*>(a.gamma) + j);
    if (!RMS && a.beta) v += Cvt<T>::load1(reinterpret_cast<const T*>(a.beta) + j);
    Cvt<T>::store1(yr + j, v);
  }
}

template <typename T, int TPR, bool RMS>
void launch_tpr(const NArgs& a, int iters, cudaStream_t s) {
  const int block = TPR > 256 ? TPR : 256;
  const int rows_per_cta = block / TPR;
  const unsigned grid = (unsigned)((a.rows + rows_per_cta - 1) / rows_per_cta);
  switch (iters) {
    case 1: norm_rows_kernel<T, 1, TPR, RMS><<<grid, block, 0, s>>>(a); break;
    case 2: norm_rows_kernel<T, 2, TPR, RMS><<<grid, block, 0, s>>>(a); break;
    case 4: norm_rows_kernel<T, 4, TPR, RMS><<<grid, block, 0, s>>>(a); break;
    case 8: norm_rows_kernel<T, 8, TPR, RMS><<<grid, block, 0, s>>>(a); break;
    default: norm_rows_kernel<T, 16, TPR, RMS><<<grid, block, 0, s>>>(a); break;
  }
}

template <typename T, bool RMS>
void launch_typed(const NArgs& a, cudaStream_t s) {
  constexpr int V = Cvt<T>::N;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec_ok = (a.cols % V == 0) && al16(a.x) && al16(a.y) && al16(a.gamma) && al16(a.beta) &&
                      a.cols <= (int64_t)1024 * V * 16;
  if (!vec_ok) {
    norm_generic_kernel<T, RMS><<<(unsigned)a.rows, 256, 0, s>>>(a);
    return;
  }
  const int64_t vecs = a.cols / V;
  int tpr = 32;
  if (vecs > 32 * 16) tpr = 256;
  if (vecs > 256 * 16) tpr = 1024;
  int iters = 1;
  while ((int64_t)iters * tpr < vecs) iters *= 2;
  if (tpr == 32) launch_tpr<T, 32, RMS>(a, iters, s);
  else if (tpr == 256) launch_tpr<T, 256, RMS>(a, iters, s);
  else launch_tpr<T, 1024, RMS>(a, iters, s);
}

}  // namespace

Status norm_rows(Device* dev, const NormParams& p) {
  if (p.rows == 0 || p.cols == 0) return Status::OK();
  if (p.rows > 0x7fffffffLL) return Status::Unsupported("norm: more than 2^31-1 rows");
  NArgs a{p.x, p.gamma, p.rms ? nullptr : p.beta, p.y, p.rows, p.cols, (float)p.epsilon};
  B200_TRY(dev->MakeCurrent());
  cudaStream_t s = dev->stream();
  switch (p.dtype) {
    case B200_FLOAT32: p.rms ? launch_typed<float, true>(a, s) : launch_typed<float, false>(a, s); break;
    case B200_BFLOAT16: p.rms ? launch_typed<__nv_bfloat16, true>(a, s) : launch_typed<__nv_bfloat16, false>(a, s); break;
    case B200_FLOAT16: p.rms ? launch_typed<__half, true>(a, s) : launch_typed<__half, false>(a, s); break;
    default: return Status::Unsupported(strfmt("norm: dtype %s", dtype_name(p.dtype)));
  }
  return dev->CheckLaunch(p.rms ? "rms_norm" : "layer_norm");
}

}  // namespace k
}  // namespace b200
